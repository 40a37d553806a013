/*
 * llmb200_train_kernels.h -- kernel-level C ABI of the LoRA-SFT step (sm_100a).
 *
 * One entry point per fused device operation of the training engine. Each
 * names the reference dispatches (src/nn/fast_metal.h) and shader kernels
 * (shaders/q8_kernels.metal) whose arithmetic it carries out. All tensors are
 * fp32 in device memory and row-major; "rows" are tokens: a batch of S
 * sequences of N tokens is one [S*N, .] matrix, sequence s owning rows
 * s*N .. s*N+N-1 (the reference trains one sequence, S = 1).
 *
 * Every function enqueues on `stream` (a cudaStream_t) and returns 0, a
 * positive cudaError_t, or a negative B200_E_* code. Nothing allocates.
 */
#ifndef LLMB200_TRAIN_KERNELS_H
#define LLMB200_TRAIN_KERNELS_H

#include <stddef.h>
#include <stdint.h>
#include "llmb200_kernels.h"   /* B200_E_* */

#ifdef __cplusplus
extern "C" {
#endif

/* C[M,N] = alpha * sum_k A(m,k) * B(k,n) + (R ? R[m,n] : 0), fp32.
 * A(m,k) = A[m*a_row + k*a_col], B(k,n) = B[k*b_row + n*b_col]; one of the two
 * strides of each operand must be 1. Covers the reference's f16_matmul
 * (:383-407, B = weight [N,K]: b_row = 1, b_col = K), f16_matmul_nt (:411-435),
 * float_matmul (:1043-1067), float_matmul_tn (:1070-1094) and float_matmul_nt
 * (:1128-1152); the frozen weights are held as fp32 copies of their binary16
 * values, so every product equals the reference's float(half) product. */
typedef struct {
    const float *A; long long a_row, a_col;
    const float *B; long long b_row, b_col;
    float *C; long long ldc;
    const float *R; long long ldr;
    int M, N, K;
    float alpha;
    unsigned *d_err;     /* optional device word; the tensor-core kernel stores a non-zero code there when a
                            bounded wait runs out (the product is then incomplete) */
} b200_gemm_args;

/* CUDA-core version: any shape, any of the stride combinations above. */
int b200_gemm_f32(const b200_gemm_args *a, void *stream);
/* Tensor-core version (tcgen05.mma kind::tf32, fp32 accumulate in tensor
 * memory, operands staged by TMA). Requires a_col == 1 and b_row == 1 (both
 * operands contiguous along k), K a multiple of 4, A, B 16-byte aligned with
 * row strides that are multiples of 4 elements. Operands are rounded to TF32
 * by the tensor core (weights holding binary16 values stay exact).
 * Returns B200_E_UNSUPPORTED when a condition does not hold. */
int b200_gemm_tf32(const b200_gemm_args *a, void *stream);
/* The same kernel on binary16 operands (tcgen05.mma kind::f16): A and B point
 * to binary16 data (strides in elements, K and the row strides multiples of
 * 8), C and R stay fp32, accumulation is fp32. Half the operand bytes of the
 * TF32 form, which is what bounds the kernel. */
int b200_gemm_f16(const b200_gemm_args *a, void *stream);
/* dst[i] = binary16(src[i] * scale), round to nearest even: the operand copies
 * b200_gemm_f16 reads (gradients are scaled by a power of two into binary16's
 * range and the product scaled back through alpha). */
int b200_f32_to_f16(const float *src, size_t n, float scale, void *dst, void *stream);
int b200_transpose_f16(const void *src, int rows, int cols, void *dst, void *stream);

/* x[m,:] = scale * emb[tokens[m],:]  (src/nn/fast_sft.c:1118-1126). */
int b200_embed_rows(const float *emb, const uint32_t *tokens, int rows, int dim, int vocab, float scale,
                    float *x, void *stream);

/* w[i] = float(half(w[i])) in place: the value the reference's F16 weight
 * container holds (src/nn/wmat.c wmat_create_f16), kept in fp32 storage. */
int b200_round_f16(float *w, size_t n, void *stream);
/* dst[cols, rows] = transpose of src[rows, cols]. */
int b200_transpose_f32(const float *src, int rows, int cols, float *dst, void *stream);

/* out = x * rsqrt(mean(x^2) + eps) * gamma per row (rms_norm :133-158); rows
 * are contiguous, dim apart. */
int b200_rms_norm_rows(const float *x, const float *gamma, float *out, int rows, int dim, float eps, void *stream);

/* dx (+)= rms_norm backward of dy through x (rms_norm_train_backward :584-624);
 * accumulate != 0 adds into dx (the reference's residual_add that follows);
 * clamp > 0 clips the result to +-clamp afterwards (clamp_tensor :1155-1161). */
int b200_rms_norm_bwd_rows(const float *x, const float *dy, long long dy_ld, const float *gamma, float *dx, int rows,
                           int dim, float eps, int accumulate, float clamp, void *stream);

/* Per-head RMSNorm then rotary embedding of the q and k column blocks of the
 * fused projection output qkv [rows, ld] (q heads first, then kv heads of k,
 * then v), written token-major to q_out [rows, n_q*hd] and k_out [rows, n_kv*hd].
 * Position = row % seq_len. inv_freq[hd/2] = 1/pow(theta, 2d/hd).
 * (rms_norm over H*N rows + rope_train :495-538; the transposes :438-473 are
 * not materialised.) */
int b200_qk_norm_rope(const float *qkv, long long ld, const float *q_gamma, const float *k_gamma,
                      const float *inv_freq, int rows, int seq_len, int n_q, int n_kv, int hd, float eps,
                      float *q_out, float *k_out, void *stream);
/* Backward of the above, in place on the q and k blocks of dqkv [rows, dld]:
 * inverse rotation (rope_train_bwd :997-1040) then RMSNorm backward through
 * the saved pre-norm values in qkv [rows, ld]. */
int b200_qk_norm_rope_bwd(float *dqkv, const float *qkv, long long ld, long long dld, const float *q_gamma, const float *k_gamma,
                          const float *inv_freq, int rows, int seq_len, int n_q, int n_kv, int hd, float eps,
                          void *stream);

/* Causal attention over each sequence (attn_train_fwd :769-851 with repeat_kv
 * :476-492 folded into the indexing). q [rows, n_q*hd], k [rows, n_kv*hd],
 * v = columns v_off.. of a matrix with row stride v_ld. probs [S, n_q, N, N]
 * keeps the softmax (zeros above the diagonal); out [rows, n_q*hd]. */
int b200_attn_train_fwd(const float *q, const float *k, const float *v, long long v_ld, int n_seq, int seq_len,
                        int n_q, int n_kv, int hd, float scale, float *probs, float *out, void *stream);
/* attn_bwd_dq (:857-925), attn_bwd_dkv (:931-968) and repeat_kv_bwd (:973-992):
 * d_out [rows, n_q*hd] -> dq, dk, dv written into the q, k, v column blocks of
 * dqkv [rows, ld]. d_score is scratch of S*n_q*N*max(N, 2*hd) floats (the
 * score gradients, or per-head dK/dV partial sums for short sequences). */
int b200_attn_train_bwd(const float *d_out, const float *probs, const float *q, const float *k, const float *v,
                        long long v_ld, int n_seq, int seq_len, int n_q, int n_kv, int hd, float scale,
                        float *d_score, float *dqkv, long long ld, void *stream);

/* act[m,i] = silu(gu[m,i]) * gu[m,inter+i] (silu_mul :337-348) for the fused
 * gate/up output gu [rows, 2*inter]. */
int b200_silu_mul_rows(const float *gu, int rows, int inter, float *act, void *stream);
/* silu_mul_backward (:540-556): d_act [rows, inter] -> d_gu [rows, 2*inter]. */
int b200_silu_mul_bwd_rows(const float *d_act, const float *gu, int rows, int inter, float *d_gu, void *stream);

/* y[m, col0+c] += sc * sum_r mid[m*mid_ld + r] * B[c,r] for c < n_cols
 * (float_matmul with K = rank + add_scaled, src/nn/fast_sft.c:639-643). rank <= 64. */
int b200_lora_add(float *y, long long ld, int col0, int n_cols, const float *mid, long long mid_ld, const float *B,
                  int rank, float sc, int rows, void *stream);
/* Refreshes the LoRA rows appended to the fused q/k/v weight and to its
 * transposed copy, so that the two big products of a layer also deliver the
 * rank-R intermediates of fast_sft.c:639-641 (ln1 A^T) and :948-949, :963-964
 * (sc dq B_q, sc dv B_v):
 *   w_ext  [q_cols + 2 kv_cols + xr, d]: extra rows 0..R-1 = A_q, R..2R-1 = A_v, rest 0
 *   wt_ext [d + xr, q_cols + 2 kv_cols]: extra row r = sc B_q[:, r] over the q columns,
 *                                        extra row R+r = sc B_v[:, r] over the v columns, rest 0 */
int b200_lora_pack(float *w_ext, float *wt_ext, const float *A_q, const float *B_q, const float *A_v,
                   const float *B_v, int d, int q_cols, int kv_cols, int rank, int xr, float sc, void *stream);
/* The same with binary16 destinations. */
int b200_lora_pack_f16(void *w_ext, void *wt_ext, const float *A_q, const float *B_q, const float *A_v,
                       const float *B_v, int d, int q_cols, int kv_cols, int rank, int xr, float sc, void *stream);

/* C(p, r) = alpha * sum_m X[m*ld_x + p] * Y[m*ld_y + r] for p < P, r < R <= 16
 * (B200_E_UNSUPPORTED for wider ranks: use b200_gemm_f32),
 * stored at C[p*c_p + r*c_r]: float_matmul_tn (:1070-1094) for the rank-R LoRA
 * gradients dB = sc dY^T mid (c_p = R, c_r = 1) and dA = tmp^T ln1 (c_p = 1,
 * c_r = P), src/nn/fast_sft.c:946-950, 961-965. Row order of the sum is fixed. */
int b200_xty_skinny(const float *X, long long ld_x, const float *Y, long long ld_y, int rows, int P, int R,
                    float alpha, float *C, long long c_p, long long c_r, void *stream);

/* softmax_ce_train (:646-690) followed by scale_tensor(grad_scale):
 * losses[m] = logsumexp - logit[target]; dlogits = (softmax - onehot) * grad_scale. */
int b200_softmax_ce_rows(const float *logits, const uint32_t *targets, int rows, int vocab, float grad_scale,
                         float *losses, float *dlogits, void *stream);

/* GeGLU on the fused gate|up layout gu [rows, 2 * inter] (gelu_mul :351-363, gelu_mul_backward :561-580; tanh form,
 * argument clamped to +-15): act[rows, inter] = gelu(gate) * up; d_gu[rows, 2 * inter] = (d gate | d up). */
int b200_gelu_mul_rows(const float *gu, int rows, int inter, float *act, void *stream);
int b200_gelu_mul_bwd_rows(const float *d_act, const float *gu, int rows, int inter, float *d_gu, void *stream);
/* out[i] = a[i] + b[i] (residual_add :369-375); out may be a or b. */
int b200_add(const float *a, const float *b, float *out, size_t n, void *stream);

/* grpo_policy_grad (shaders/q8_kernels.metal:698-761; dispatch fast_metal.m:963-981), one row per position:
 * new_logprobs[m] = logit[action] - logsumexp; ratio = exp(new - old); the PPO clip keeps the position
 * (weight = -advantage) or drops it (0); dlogits = weight * ratio * (softmax - onehot(action)). */
int b200_grpo_policy_grad(const float *logits, const uint32_t *actions, const float *old_logprobs, const float *advantages,
                          float *new_logprobs, float *dlogits, int rows, int vocab, float clip_eps, void *stream);

/* f16_sgd_apply (shaders/q8_kernels.metal:1195-1206) for weights and accumulated gradients kept as fp32
 * holders of binary16 values: w[i] = half(w[i] - lr * g[i]); g[i] = 0. */
int b200_sgd_apply_f16(float *w, float *g, size_t n, float lr, void *stream);

/* scale_tensor (fast_metal.m:722-731): x[i] *= alpha for i < n. */
int b200_scale(float *x, float alpha, size_t n, void *stream);

/* Global-norm clip + AdamW over one flat parameter vector
 * (src/nn/fast_sft.c:1045-1107). Step 1 writes per-block double partial sums
 * of g^2 into partials[n_partials]; step 2 adds them in index order (double),
 * takes the fp32 square root, scales g by max_norm/norm when norm > max_norm
 * (writing the scaled gradient back, as the reference does) and applies
 * p -= lr*((m/bc1)/(sqrt(v/bc2)+eps) + wd*p). bc1 = 1-powf(beta1,step) and bc2
 * are computed by the caller. norm_out[0] receives the norm. */
int b200_sumsq_partials(const float *g, size_t n, double *partials, int n_partials, void *stream);
int b200_clip_adamw(float *p, float *g, float *m, float *v, size_t n, const double *partials, int n_partials,
                    float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                    int apply_update, float *norm_out, void *stream);

/* Variants that also (or only) write a binary16 copy of their result, the
 * operand the next tensor-core product reads, so that no separate conversion
 * pass is needed. *_h pointers may be NULL; where noted the fp32 output may be
 * NULL instead. h_scale multiplies the value before it is rounded (gradients
 * are moved into binary16's range by a power of two). */
int b200_rms_norm_rows_h(const float *x, const float *gamma, float *out, void *out_h, int rows, int dim, float eps,
                         void *stream);
int b200_rms_norm_bwd_rows_h(const float *x, const float *dy, long long dy_ld, const float *gamma, float *dx, int rows,
                             int dim, float eps, int accumulate, float clamp, void *dx_h, float h_scale, void *stream);
/* out may be NULL when out_h is given */
int b200_attn_train_fwd_h(const float *q, const float *k, const float *v, long long v_ld, int n_seq, int seq_len,
                          int n_q, int n_kv, int hd, float scale, float *probs, float *out, void *out_h, void *stream);
/* act may be NULL when act_h is given; likewise d_gu / d_gu_h */
int b200_silu_mul_rows_h(const float *gu, int rows, int inter, float *act, void *act_h, void *stream);
int b200_silu_mul_bwd_rows_h(const float *d_act, const float *gu, int rows, int inter, float *d_gu, void *d_gu_h,
                             float h_scale, void *stream);
int b200_softmax_ce_rows_h(const float *logits, const uint32_t *targets, int rows, int vocab, float grad_scale,
                           float *losses, float *dlogits, void *dlogits_h, float h_scale, void *stream);

#define B200_E_UNSUPPORTED (-4)

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_TRAIN_KERNELS_H */
