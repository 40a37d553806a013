/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * A CPU stand-in for the reference's Metal dispatch layer (src/nn/fast_metal.h,
 * implementation src/nn/fast_metal.m) so that the reference's own fast engines
 * -- src/nn/fast_sft.c and src/nn/fast_inference.c, compiled unmodified from
 * where they lie -- run on host cores and pin the restatements under oracle/.
 *
 * Every metal_enqueue_* below executes at once what the dispatch of the same
 * name would run on the GPU: the command buffer of fast_metal.m is in-order
 * with a buffer-scope barrier after every dispatch (fast_metal.m:231-233) and
 * the buffers are shared-storage, so immediate execution yields the same
 * values. Argument-to-buffer-slot binding follows each wrapper in fast_metal.m
 * (cited per function); the arithmetic follows the kernel of
 * shaders/q8_kernels.metal bound to that pipeline (cited per function),
 * including the order of summation wherever the shader fixes it: per-thread
 * strided partial sums, then the halving tree over the threadgroup
 * (e.g. q8_kernels.metal:146-154). Where the hardware's order is unspecified
 * (simd_sum, dot of a float4) a halving tree / left-to-right sum is used.
 * Metal's fast-math exp/cos/sin/pow/tanh/rsqrt become the libm float functions.
 *
 * metal_buf_create / _from_data / _free / _ptr live in ref_stubs.c.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct MetalBuf MetalBuf;
void *metal_buf_ptr(MetalBuf *b);

typedef _Float16 half_t;

#define F(b) ((float *)metal_buf_ptr(b))
#define FO(b, off) ((float *)((char *)metal_buf_ptr(b) + (off)))
#define MINI(a, b) ((a) < (b) ? (a) : (b))

int  fast_metal_init(void) { return 0; }       /* fast_metal.m:75-168 */
void fast_metal_shutdown(void) {}              /* fast_metal.m:170-190 */
void metal_flush(void) {}                      /* fast_metal.m:235-247: everything has already run */

/* threadgroup halving tree, e.g. q8_kernels.metal:150-153 */
static float tg_tree_sum(float *sh, int tg)
{
    for (int s = tg / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) sh[t] += sh[t + s];
    return sh[0];
}
static float tg_tree_max(float *sh, int tg)
{
    for (int s = tg / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) sh[t] = sh[t] > sh[t + s] ? sh[t] : sh[t + s];
    return sh[0];
}
/* simd_sum over 32 lanes */
static float simd_tree_sum(float *v)
{
    for (int s = 16; s > 0; s >>= 1)
        for (int t = 0; t < s; ++t) v[t] += v[t + s];
    return v[0];
}

/* ---------------------------------------------------------------- decode kernels */

/* fast_metal.m:253-270 -> q8_matvec, q8_kernels.metal:9-38 */
void metal_enqueue_q8_matvec(MetalBuf *W_buf, MetalBuf *x_buf, MetalBuf *y_buf, int rows, int nb)
{
    const unsigned char *W = metal_buf_ptr(W_buf);
    const float *x = F(x_buf);
    float *y = F(y_buf);
    for (int r = 0; r < rows; ++r) {
        const unsigned char *rp = W + (size_t)r * nb * 34u;
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const unsigned char *blk = rp + (size_t)b * 34u;
            half_t h;
            memcpy(&h, blk, 2);
            float scale = (float)h, prod[32];
            const signed char *q = (const signed char *)(blk + 2);
            for (int lane = 0; lane < 32; ++lane) prod[lane] = (float)q[lane] * x[b * 32 + lane];
            sum += scale * simd_tree_sum(prod);
        }
        y[r] = sum;
    }
}

/* one row of f16_matvec / f16_batch_matvec: q8_kernels.metal:103-118 (and :63-78) */
static float f16_row_dot(const half_t *w, const float *x, int cols)
{
    float lane_sum[32];
    int aligned = cols & ~127;
    for (int lane = 0; lane < 32; ++lane) {
        float s = 0.0f;
        for (int base = lane * 4; base < aligned; base += 128) {
            float d = 0.0f;
            for (int e = 0; e < 4; ++e) d += (float)w[base + e] * x[base + e];
            s += d;
        }
        for (int i = aligned + lane; i < cols; i += 32) s += (float)w[i] * x[i];
        lane_sum[lane] = s;
    }
    return simd_tree_sum(lane_sum);
}

/* fast_metal.m:272-289 -> f16_matvec, q8_kernels.metal:88-120 */
void metal_enqueue_f16_matvec(MetalBuf *W_buf, MetalBuf *x_buf, MetalBuf *y_buf, int rows, int cols)
{
    const half_t *W = metal_buf_ptr(W_buf);
    for (int r = 0; r < rows; ++r) F(y_buf)[r] = f16_row_dot(W + (size_t)r * cols, F(x_buf), cols);
}

/* fast_metal.m:291-307 -> f16_batch_matvec, q8_kernels.metal:44-82 */
void metal_enqueue_f16_batch_matvec(MetalBuf *W_buf, MetalBuf *X_buf, MetalBuf *Y_buf, int rows, int cols, int B)
{
    const half_t *W = metal_buf_ptr(W_buf);
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < B; ++b)
            F(Y_buf)[(size_t)b * rows + r] = f16_row_dot(W + (size_t)r * cols, F(X_buf) + (size_t)b * cols, cols);
}

/* rms_norm, q8_kernels.metal:125-158; one threadgroup of tg threads per row */
static void rms_norm_rows(const float *x, const float *gamma, float *out, int dim, float eps, int rows, int tg)
{
    float sh[256];
    for (int b = 0; b < rows; ++b) {
        const float *xr = x + (size_t)b * dim;
        float *o = out + (size_t)b * dim;
        for (int t = 0; t < tg; ++t) {
            float p = 0.0f;
            for (int i = t; i < dim; i += tg) p += xr[i] * xr[i];
            sh[t] = p;
        }
        float inv_rms = 1.0f / sqrtf(tg_tree_sum(sh, tg) / (float)dim + eps);
        for (int i = 0; i < dim; ++i) o[i] = xr[i] * inv_rms * gamma[i];
    }
}

/* fast_metal.m:309-324 */
void metal_enqueue_rms_norm(MetalBuf *x_buf, MetalBuf *gamma_buf, MetalBuf *out_buf, int dim, float eps)
{
    rms_norm_rows(F(x_buf), F(gamma_buf), F(out_buf), dim, eps, 1, MINI(256, dim));
}
/* fast_metal.m:326-341 */
void metal_enqueue_rms_norm_batched(MetalBuf *x_buf, MetalBuf *gamma_buf, MetalBuf *out_buf, int dim, float eps, int B)
{
    rms_norm_rows(F(x_buf), F(gamma_buf), F(out_buf), dim, eps, B, MINI(256, dim));
}
/* fast_metal.m:343-357 and :468-483 -> per_head_rms_norm, q8_kernels.metal:165-190 (the same arithmetic per head) */
void metal_enqueue_per_head_rms_norm_off(MetalBuf *vec_buf, size_t vec_off, MetalBuf *gamma_buf, int n_heads, int head_dim, float eps)
{
    rms_norm_rows(FO(vec_buf, vec_off), F(gamma_buf), FO(vec_buf, vec_off), head_dim, eps, n_heads, MINI(256, head_dim));
}
void metal_enqueue_per_head_rms_norm(MetalBuf *vec_buf, MetalBuf *gamma_buf, int n_heads, int head_dim, float eps)
{
    metal_enqueue_per_head_rms_norm_off(vec_buf, 0, gamma_buf, n_heads, head_dim, eps);
}

/* the rotation of rope / rope_train / rope_train_bwd: q8_kernels.metal:219-227, :531-539, :1012-1021 */
static void rotate_pair(float *vec, int d, int hd, int pos, float theta, int inverse)
{
    int half = hd / 2;
    float freq = 1.0f / powf(theta, (float)(2 * d) / (float)hd);
    float angle = (float)pos * freq;
    float c = cosf(angle), s = sinf(angle);
    float x0 = vec[d], x1 = vec[d + half];
    if (!inverse) {
        vec[d] = x0 * c - x1 * s;
        vec[d + half] = x0 * s + x1 * c;
    } else {
        vec[d] = x0 * c + x1 * s;
        vec[d + half] = -x0 * s + x1 * c;
    }
}

/* fast_metal.m:359-379 and :485-506 -> rope, q8_kernels.metal:195-228 */
void metal_enqueue_rope_off(MetalBuf *q_buf, size_t q_off, MetalBuf *k_buf, size_t k_off, int Hq, int Hkv, int hd, int pos, float theta)
{
    float *q = FO(q_buf, q_off), *k = FO(k_buf, k_off);
    for (int h = 0; h < Hq; ++h)
        for (int d = 0; d < hd / 2; ++d) rotate_pair(q + (size_t)h * hd, d, hd, pos, theta, 0);
    for (int h = 0; h < Hkv; ++h)
        for (int d = 0; d < hd / 2; ++d) rotate_pair(k + (size_t)h * hd, d, hd, pos, theta, 0);
}
void metal_enqueue_rope(MetalBuf *q_buf, MetalBuf *k_buf, int Hq, int Hkv, int hd, int pos, float theta)
{
    metal_enqueue_rope_off(q_buf, 0, k_buf, 0, Hq, Hkv, hd, pos, theta);
}

/* fast_metal.m:381-402 and :508-530 -> kv_cache_store, q8_kernels.metal:233-252 */
void metal_enqueue_kv_cache_store_off(MetalBuf *k_buf, size_t k_off, MetalBuf *v_buf, size_t v_off, MetalBuf *k_cache,
                                      MetalBuf *v_cache, int Hkv, int max_seq, int hd, int pos)
{
    const float *k = FO(k_buf, k_off), *v = FO(v_buf, v_off);
    for (int h = 0; h < Hkv; ++h)
        for (int d = 0; d < hd; ++d) {
            size_t ci = ((size_t)h * max_seq + pos) * hd + d;
            F(k_cache)[ci] = k[h * hd + d];
            F(v_cache)[ci] = v[h * hd + d];
        }
}
void metal_enqueue_kv_cache_store(MetalBuf *k_buf, MetalBuf *v_buf, MetalBuf *k_cache, MetalBuf *v_cache, int Hkv, int max_seq, int hd, int pos)
{
    metal_enqueue_kv_cache_store_off(k_buf, 0, v_buf, 0, k_cache, v_cache, Hkv, max_seq, hd, pos);
}

/* fast_metal.m:404-426 and :532-556 -> attention, q8_kernels.metal:258-326; 256 threads per query head */
void metal_enqueue_attention_off(MetalBuf *Q_buf, size_t q_off, MetalBuf *Kc_buf, MetalBuf *Vc_buf, MetalBuf *attn_out_buf, size_t out_off,
                                 int n_attend, int hd, int max_seq, int Hq, int group_ratio)
{
    const int tg = 256;
    float inv_sqrt_hd = 1.0f / sqrtf((float)hd);
    float *scores = malloc(sizeof(float) * (size_t)(n_attend > 0 ? n_attend : 1)), sh[256];
    for (int hq = 0; hq < Hq; ++hq) {
        int hkv = hq / group_ratio;
        const float *qp = FO(Q_buf, q_off) + (size_t)hq * hd;
        const float *kp = F(Kc_buf) + (size_t)hkv * max_seq * hd;
        const float *vp = F(Vc_buf) + (size_t)hkv * max_seq * hd;
        float *out = FO(attn_out_buf, out_off) + (size_t)hq * hd;
        for (int j = 0; j < n_attend; ++j) {
            float dot = 0;
            for (int d = 0; d < hd; ++d) dot += qp[d] * kp[(size_t)j * hd + d];
            scores[j] = dot * inv_sqrt_hd;
        }
        for (int t = 0; t < tg; ++t) {
            float m = -1e30f;
            for (int j = t; j < n_attend; j += tg) m = m > scores[j] ? m : scores[j];
            sh[t] = m;
        }
        float max_val = tg_tree_max(sh, tg);
        for (int t = 0; t < tg; ++t) {
            float s = 0;
            for (int j = t; j < n_attend; j += tg) {
                scores[j] = expf(scores[j] - max_val);
                s += scores[j];
            }
            sh[t] = s;
        }
        float inv_sum = 1.0f / tg_tree_sum(sh, tg);
        for (int j = 0; j < n_attend; ++j) scores[j] *= inv_sum;
        for (int d = 0; d < hd; ++d) {
            float val = 0;
            for (int j = 0; j < n_attend; ++j) val += scores[j] * vp[(size_t)j * hd + d];
            out[d] = val;
        }
    }
    free(scores);
}
void metal_enqueue_attention(MetalBuf *Q_buf, MetalBuf *Kc_buf, MetalBuf *Vc_buf, MetalBuf *attn_out_buf, int n_attend, int hd,
                             int max_seq, int Hq, int group_ratio)
{
    metal_enqueue_attention_off(Q_buf, 0, Kc_buf, Vc_buf, attn_out_buf, 0, n_attend, hd, max_seq, Hq, group_ratio);
}

/* fast_metal.m:428-438 -> silu_mul, q8_kernels.metal:331-338 */
void metal_enqueue_silu_mul(MetalBuf *gate_buf, MetalBuf *up_buf, int n)
{
    float *g = F(gate_buf);
    const float *u = F(up_buf);
    for (int i = 0; i < n; ++i) g[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}

static float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* fast_metal.m:440-450 -> gelu_mul, q8_kernels.metal:344-356 */
void metal_enqueue_gelu_mul(MetalBuf *gate_buf, MetalBuf *up_buf, int n)
{
    float *gp = F(gate_buf);
    const float *u = F(up_buf);
    for (int i = 0; i < n; ++i) {
        float g = gp[i], g3 = g * g * g;
        float inner = clampf(0.7978845608f * (g + 0.044715f * g3), -15.0f, 15.0f);
        gp[i] = 0.5f * g * (1.0f + tanhf(inner)) * u[i];
    }
}

/* fast_metal.m:452-462 -> residual_add, q8_kernels.metal:361-367 */
void metal_enqueue_residual_add(MetalBuf *x_buf, MetalBuf *y_buf, int n)
{
    for (int i = 0; i < n; ++i) F(x_buf)[i] += F(y_buf)[i];
}

/* ---------------------------------------------------------------- training kernels */

/* fast_metal.m:562-577: the first argument lands in slot 0 (the float activations A), the second in slot 1
 * (the binary16 weights W) -> f16_matmul, q8_kernels.metal:383-407: C[M,N] = A[M,K] W[N,K]^T, k ascending */
void metal_enqueue_f16_matmul(MetalBuf *A_buf, MetalBuf *W_buf, MetalBuf *C_buf, int M, int N, int K)
{
    const float *A = F(A_buf);
    const half_t *W = metal_buf_ptr(W_buf);
    float *Cm = F(C_buf);
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            float sum = 0;
            for (int k = 0; k < K; ++k) sum += A[(size_t)r * K + k] * (float)W[(size_t)c * K + k];
            Cm[(size_t)r * N + c] = sum;
        }
}

/* fast_metal.m:579-594 -> f16_matmul_nt, q8_kernels.metal:411-435: C[M,K] = A[M,N] W[N,K] */
void metal_enqueue_f16_matmul_nt(MetalBuf *A_buf, MetalBuf *W_buf, MetalBuf *C_buf, int M, int N, int K)
{
    const float *A = F(A_buf);
    const half_t *W = metal_buf_ptr(W_buf);
    float *Cm = F(C_buf);
    float *acc = malloc(sizeof(float) * (size_t)K);
    for (int r = 0; r < M; ++r) {
        for (int c = 0; c < K; ++c) acc[c] = 0;
        for (int n = 0; n < N; ++n) {                       /* n ascending per output, as in the shader */
            float a = A[(size_t)r * N + n];
            const half_t *w = W + (size_t)n * K;
            for (int c = 0; c < K; ++c) acc[c] += a * (float)w[c];
        }
        memcpy(Cm + (size_t)r * K, acc, sizeof(float) * (size_t)K);
    }
    free(acc);
}

/* fast_metal.m:596-612 -> transpose_heads_fwd, q8_kernels.metal:438-454: [N, H*D] -> [H, N, D] */
void metal_enqueue_transpose_heads_fwd(MetalBuf *src, MetalBuf *dst, int seq_len, int n_heads, int head_dim)
{
    for (int n = 0; n < seq_len; ++n)
        for (int h = 0; h < n_heads; ++h)
            memcpy(F(dst) + ((size_t)h * seq_len + n) * head_dim, F(src) + ((size_t)n * n_heads + h) * head_dim, sizeof(float) * (size_t)head_dim);
}
/* fast_metal.m:614-630 -> transpose_heads_rev, q8_kernels.metal:457-473: [H, N, D] -> [N, H*D] */
void metal_enqueue_transpose_heads_rev(MetalBuf *src, MetalBuf *dst, int seq_len, int n_heads, int head_dim)
{
    for (int h = 0; h < n_heads; ++h)
        for (int n = 0; n < seq_len; ++n)
            memcpy(F(dst) + ((size_t)n * n_heads + h) * head_dim, F(src) + ((size_t)h * seq_len + n) * head_dim, sizeof(float) * (size_t)head_dim);
}
/* fast_metal.m:632-650 -> repeat_kv, q8_kernels.metal:476-492: [Hkv, N, D] -> [Hq, N, D] */
void metal_enqueue_repeat_kv(MetalBuf *src, MetalBuf *dst, int n_kv, int seq_len, int head_dim, int group_ratio)
{
    size_t ND = (size_t)seq_len * head_dim;
    for (int hq = 0; hq < n_kv * group_ratio; ++hq)
        memcpy(F(dst) + hq * ND, F(src) + (size_t)(hq / group_ratio) * ND, sizeof(float) * ND);
}
/* fast_metal.m:830-848 -> repeat_kv_bwd, q8_kernels.metal:972-990 */
void metal_enqueue_repeat_kv_bwd(MetalBuf *d_expanded, MetalBuf *d_kv, int n_kv, int seq_len, int head_dim, int group_ratio)
{
    size_t ND = (size_t)seq_len * head_dim;
    for (int hkv = 0; hkv < n_kv; ++hkv)
        for (size_t rem = 0; rem < ND; ++rem) {
            float sum = 0;
            for (int g = 0; g < group_ratio; ++g) sum += F(d_expanded)[((size_t)hkv * group_ratio + g) * ND + rem];
            F(d_kv)[hkv * ND + rem] = sum;
        }
}

static void rope_rows(float *q, float *k, int Hq, int Hkv, int hd, int seq_len, float theta, int inverse)
{
    for (int h = 0; h < Hq; ++h)
        for (int pos = 0; pos < seq_len; ++pos)
            for (int d = 0; d < hd / 2; ++d) rotate_pair(q + ((size_t)h * seq_len + pos) * hd, d, hd, pos, theta, inverse);
    for (int h = 0; h < Hkv; ++h)
        for (int pos = 0; pos < seq_len; ++pos)
            for (int d = 0; d < hd / 2; ++d) rotate_pair(k + ((size_t)h * seq_len + pos) * hd, d, hd, pos, theta, inverse);
}
/* fast_metal.m:652-672 -> rope_train, q8_kernels.metal:495-540 */
void metal_enqueue_rope_train(MetalBuf *q_buf, MetalBuf *k_buf, int Hq, int Hkv, int hd, int seq_len, float theta)
{
    rope_rows(F(q_buf), F(k_buf), Hq, Hkv, hd, seq_len, theta, 0);
}
/* fast_metal.m:850-870 -> rope_train_bwd, q8_kernels.metal:993-1037 */
void metal_enqueue_rope_train_bwd(MetalBuf *q_buf, MetalBuf *k_buf, int Hq, int Hkv, int hd, int seq_len, float theta)
{
    rope_rows(F(q_buf), F(k_buf), Hq, Hkv, hd, seq_len, theta, 1);
}

/* fast_metal.m:674-687 -> silu_mul_backward, q8_kernels.metal:545-561 */
void metal_enqueue_silu_mul_backward(MetalBuf *dout, MetalBuf *gate, MetalBuf *up, MetalBuf *dgate, MetalBuf *dup, int n)
{
    for (int i = 0; i < n; ++i) {
        float g = F(gate)[i], u = F(up)[i], dy = F(dout)[i];
        float sig = 1.0f / (1.0f + expf(-g));
        float silu_g = g * sig;
        float silu_grad = sig * (1.0f + g * (1.0f - sig));
        F(dgate)[i] = dy * u * silu_grad;
        F(dup)[i] = dy * silu_g;
    }
}
/* fast_metal.m:689-702 -> gelu_mul_backward, q8_kernels.metal:566-585 */
void metal_enqueue_gelu_mul_backward(MetalBuf *dout, MetalBuf *gate, MetalBuf *up, MetalBuf *dgate, MetalBuf *dup, int n)
{
    for (int i = 0; i < n; ++i) {
        float g = F(gate)[i], u = F(up)[i], dy = F(dout)[i];
        float g3 = g * g * g;
        float inner = clampf(0.7978845608f * (g + 0.044715f * g3), -15.0f, 15.0f);
        float th = tanhf(inner);
        float gelu_g = 0.5f * g * (1.0f + th);
        float sech2 = 1.0f - th * th;
        float gelu_grad = 0.5f * (1.0f + th) + 0.5f * g * sech2 * 0.7978845608f * (1.0f + 3.0f * 0.044715f * g * g);
        F(dgate)[i] = dy * u * gelu_grad;
        F(dup)[i] = dy * gelu_g;
    }
}

/* fast_metal.m:704-720 -> rms_norm_train_backward, q8_kernels.metal:589-629 */
void metal_enqueue_rms_norm_backward(MetalBuf *x_buf, MetalBuf *dy_buf, MetalBuf *gamma_buf, MetalBuf *dx_buf, int batch, int dim, float eps)
{
    int tg = MINI(256, dim);
    const float *gamma = F(gamma_buf);
    float sh[256];
    for (int b = 0; b < batch; ++b) {
        const float *x = F(x_buf) + (size_t)b * dim, *dy = F(dy_buf) + (size_t)b * dim;
        float *dx = F(dx_buf) + (size_t)b * dim;
        for (int t = 0; t < tg; ++t) {
            float p = 0;
            for (int i = t; i < dim; i += tg) p += x[i] * x[i];
            sh[t] = p;
        }
        float inv_rms = 1.0f / sqrtf(tg_tree_sum(sh, tg) / (float)dim + eps);
        for (int t = 0; t < tg; ++t) {
            float p = 0;
            for (int i = t; i < dim; i += tg) p += dy[i] * gamma[i] * x[i];
            sh[t] = p;
        }
        float coeff = tg_tree_sum(sh, tg) * inv_rms * inv_rms / (float)dim;
        for (int i = 0; i < dim; ++i) dx[i] = (gamma[i] * dy[i] - coeff * x[i]) * inv_rms;
    }
}

/* fast_metal.m:722-731 -> scale_tensor, q8_kernels.metal:632-638 */
void metal_enqueue_scale(MetalBuf *x, float alpha, int n)
{
    for (int i = 0; i < n; ++i) F(x)[i] *= alpha;
}
/* fast_metal.m:733-743 -> add_scaled, q8_kernels.metal:641-648 */
void metal_enqueue_add_scaled(MetalBuf *y, MetalBuf *x, float alpha, int n)
{
    for (int i = 0; i < n; ++i) F(y)[i] += alpha * F(x)[i];
}

/* fast_metal.m:745-760 -> softmax_ce_train, q8_kernels.metal:651-699 */
void metal_enqueue_softmax_ce(MetalBuf *logits_buf, MetalBuf *targets, MetalBuf *losses, MetalBuf *dlogits_buf, int batch, int vocab_size)
{
    int tg = MINI(256, vocab_size);
    float sh[256];
    const uint32_t *tgts = metal_buf_ptr(targets);
    for (int b = 0; b < batch; ++b) {
        const float *lg = F(logits_buf) + (size_t)b * vocab_size;
        float *dl = F(dlogits_buf) + (size_t)b * vocab_size;
        uint32_t tgt = tgts[b];
        for (int t = 0; t < tg; ++t) {
            float m = -1e30f;
            for (int i = t; i < vocab_size; i += tg) m = m > lg[i] ? m : lg[i];
            sh[t] = m;
        }
        float max_val = tg_tree_max(sh, tg);
        for (int t = 0; t < tg; ++t) {
            float s = 0;
            for (int i = t; i < vocab_size; i += tg) s += expf(lg[i] - max_val);
            sh[t] = s;
        }
        float log_sum = logf(tg_tree_sum(sh, tg)) + max_val;
        F(losses)[b] = log_sum - lg[tgt];
        for (int i = 0; i < vocab_size; ++i) dl[i] = expf(lg[i] - log_sum) - ((uint32_t)i == tgt ? 1.0f : 0.0f);
    }
}

/* fast_metal.m:766-785 -> attn_train_fwd, q8_kernels.metal:770-846; threadgroup (h, i) of min(256, N) threads */
void metal_enqueue_attn_train_fwd(MetalBuf *Qb, MetalBuf *Kb, MetalBuf *Vb, MetalBuf *outb, MetalBuf *probsb, int H, int N, int D, float scale)
{
    int tg = MINI(256, N);
    size_t ND = (size_t)N * D, NN = (size_t)N * N;
    float *scores = malloc(sizeof(float) * (size_t)N), sh[256];
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < N; ++i) {
            const float *q_row = F(Qb) + h * ND + (size_t)i * D, *K_h = F(Kb) + h * ND, *V_h = F(Vb) + h * ND;
            float *out_row = F(outb) + h * ND + (size_t)i * D, *prob_row = F(probsb) + h * NN + (size_t)i * N;
            for (int j = 0; j <= i; ++j) {
                float dot = 0;
                for (int d = 0; d < D; ++d) dot += q_row[d] * K_h[(size_t)j * D + d];
                scores[j] = dot * scale;
            }
            for (int j = i + 1; j < N; ++j) scores[j] = -1e30f;
            for (int t = 0; t < tg; ++t) {
                float m = -1e30f;
                for (int j = t; j < N; j += tg) m = m > scores[j] ? m : scores[j];
                sh[t] = m;
            }
            float max_val = tg_tree_max(sh, tg);
            for (int t = 0; t < tg; ++t) {
                float s = 0;
                for (int j = t; j <= i; j += tg) {
                    scores[j] = expf(scores[j] - max_val);
                    s += scores[j];
                }
                sh[t] = s;
            }
            for (int j = i + 1; j < N; ++j) scores[j] = 0;
            float inv_sum = 1.0f / tg_tree_sum(sh, tg);
            for (int j = 0; j < N; ++j) {
                scores[j] *= inv_sum;
                prob_row[j] = scores[j];
            }
            for (int d = 0; d < D; ++d) {
                float val = 0;
                for (int j = 0; j <= i; ++j) val += scores[j] * V_h[(size_t)j * D + d];
                out_row[d] = val;
            }
        }
    free(scores);
}

/* fast_metal.m:787-807 -> attn_bwd_dq, q8_kernels.metal:850-916 */
void metal_enqueue_attn_bwd_dq(MetalBuf *d_outb, MetalBuf *probsb, MetalBuf *Vb, MetalBuf *Kb, MetalBuf *d_scoreb, MetalBuf *dQb,
                               int H, int N, int D, float scale)
{
    int tg = MINI(256, N);
    size_t ND = (size_t)N * D, NN = (size_t)N * N;
    float *d_raw = malloc(sizeof(float) * (size_t)N), sh[256];
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < N; ++i) {
            const float *dout_row = F(d_outb) + h * ND + (size_t)i * D, *prob_row = F(probsb) + h * NN + (size_t)i * N;
            const float *V_h = F(Vb) + h * ND, *K_h = F(Kb) + h * ND;
            float *ds_row = F(d_scoreb) + h * NN + (size_t)i * N, *dQ_row = F(dQb) + h * ND + (size_t)i * D;
            for (int j = 0; j <= i; ++j) {
                float dot = 0;
                for (int d = 0; d < D; ++d) dot += dout_row[d] * V_h[(size_t)j * D + d];
                d_raw[j] = dot;
            }
            for (int j = i + 1; j < N; ++j) d_raw[j] = 0;
            for (int t = 0; t < tg; ++t) {
                float s = 0;
                for (int j = t; j <= i; j += tg) s += prob_row[j] * d_raw[j];
                sh[t] = s;
            }
            float dp_sum = tg_tree_sum(sh, tg);
            for (int j = 0; j < N; ++j) {
                float ds = j <= i ? prob_row[j] * (d_raw[j] - dp_sum) * scale : 0;
                d_raw[j] = ds;
                ds_row[j] = ds;
            }
            for (int d = 0; d < D; ++d) {
                float val = 0;
                for (int j = 0; j <= i; ++j) val += d_raw[j] * K_h[(size_t)j * D + d];
                dQ_row[d] = val;
            }
        }
    free(d_raw);
}

/* fast_metal.m:809-828 -> attn_bwd_dkv, q8_kernels.metal:920-957 */
void metal_enqueue_attn_bwd_dkv(MetalBuf *d_scoreb, MetalBuf *Qb, MetalBuf *probsb, MetalBuf *d_outb, MetalBuf *dKb, MetalBuf *dVb,
                                int H, int N, int D)
{
    size_t ND = (size_t)N * D, NN = (size_t)N * N;
    for (int h = 0; h < H; ++h)
        for (int j = 0; j < N; ++j) {
            const float *Q_h = F(Qb) + h * ND, *dout_h = F(d_outb) + h * ND;
            float *dK_row = F(dKb) + h * ND + (size_t)j * D, *dV_row = F(dVb) + h * ND + (size_t)j * D;
            for (int d = 0; d < D; ++d) {
                float dk = 0, dv = 0;
                for (int i = j; i < N; ++i) {
                    float ds = F(d_scoreb)[h * NN + (size_t)i * N + j], pr = F(probsb)[h * NN + (size_t)i * N + j];
                    dk += ds * Q_h[(size_t)i * D + d];
                    dv += pr * dout_h[(size_t)i * D + d];
                }
                dK_row[d] = dk;
                dV_row[d] = dv;
            }
        }
}

/* fast_metal.m:872-887 -> float_matmul, q8_kernels.metal:1040-1064: C[M,N] = A[M,K] W[N,K]^T */
void metal_enqueue_float_matmul(MetalBuf *Ab, MetalBuf *Wb, MetalBuf *Cb, int M, int N, int K)
{
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            float sum = 0;
            for (int k = 0; k < K; ++k) sum += F(Ab)[(size_t)r * K + k] * F(Wb)[(size_t)c * K + k];
            F(Cb)[(size_t)r * N + c] = sum;
        }
}
/* fast_metal.m:889-904 -> float_matmul_tn, q8_kernels.metal:1067-1091: C[M,N] = A[K,M]^T B[K,N] */
void metal_enqueue_float_matmul_tn(MetalBuf *Ab, MetalBuf *Bb, MetalBuf *Cb, int M, int N, int K)
{
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            float sum = 0;
            for (int k = 0; k < K; ++k) sum += F(Ab)[(size_t)k * M + r] * F(Bb)[(size_t)k * N + c];
            F(Cb)[(size_t)r * N + c] = sum;
        }
}
/* fast_metal.m:906-921 -> float_matmul_nt, q8_kernels.metal:1124-1148: C[M,K] = A[M,N] W[N,K] */
void metal_enqueue_float_matmul_nt(MetalBuf *Ab, MetalBuf *Wb, MetalBuf *Cb, int M, int N, int K)
{
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < K; ++c) {
            float sum = 0;
            for (int n = 0; n < N; ++n) sum += F(Ab)[(size_t)r * N + n] * F(Wb)[(size_t)n * K + c];
            F(Cb)[(size_t)r * K + c] = sum;
        }
}

/* fast_metal.m:923-932 -> buf_copy, q8_kernels.metal:1208-1214 */
void metal_enqueue_copy(MetalBuf *src, MetalBuf *dst, int n)
{
    memmove(F(dst), F(src), sizeof(float) * (size_t)n);
}
/* fast_metal.m:934-943 -> clamp_tensor, q8_kernels.metal:1151-1157 */
void metal_enqueue_clamp(MetalBuf *x, float max_val, int n)
{
    for (int i = 0; i < n; ++i) F(x)[i] = clampf(F(x)[i], -max_val, max_val);
}

/* dW[M,N] = dY[K,M]^T X[K,N], the product inside f16_sgd_fused / f16_grad_accum: q8_kernels.metal:1094-1121, :1160-1188 */
static float dw_entry(const float *dY, const float *X, int M, int K, int N, int row, int col)
{
    float sum = 0;
    for (int k = 0; k < K; ++k) sum += dY[(size_t)k * M + row] * X[(size_t)k * N + col];
    return sum;
}
/* fast_metal.m:945-961 */
void metal_enqueue_f16_sgd_fused(MetalBuf *Wb, MetalBuf *dYb, MetalBuf *Xb, int M, int K, int N, float lr)
{
    half_t *W = metal_buf_ptr(Wb);
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            size_t idx = (size_t)r * N + c;
            W[idx] = (half_t)((float)W[idx] - lr * dw_entry(F(dYb), F(Xb), M, K, N, r, c));
        }
}
/* fast_metal.m:983-998 */
void metal_enqueue_f16_grad_accum(MetalBuf *Gb, MetalBuf *dYb, MetalBuf *Xb, int M, int K, int N)
{
    half_t *G = metal_buf_ptr(Gb);
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            size_t idx = (size_t)r * N + c;
            G[idx] = (half_t)((float)G[idx] + dw_entry(F(dYb), F(Xb), M, K, N, r, c));
        }
}
/* fast_metal.m:1000-1011 -> f16_sgd_apply, q8_kernels.metal:1192-1205 */
void metal_enqueue_f16_sgd_apply(MetalBuf *Wb, MetalBuf *Gb, int n, float lr)
{
    half_t *W = metal_buf_ptr(Wb), *G = metal_buf_ptr(Gb);
    for (int i = 0; i < n; ++i) {
        W[i] = (half_t)((float)W[i] - lr * (float)G[i]);
        G[i] = (half_t)0.0f;
    }
}

/* fast_metal.m:963-981 -> grpo_policy_grad, q8_kernels.metal:705-764 */
void metal_enqueue_grpo_policy_grad(MetalBuf *logits_buf, MetalBuf *actions, MetalBuf *old_lp, MetalBuf *advs, MetalBuf *new_lp,
                                    MetalBuf *dlogits_buf, int N, int V, float clip_eps)
{
    int tg = 256;
    float sh[256];
    const uint32_t *act = metal_buf_ptr(actions);
    for (int b = 0; b < N; ++b) {
        const float *lg = F(logits_buf) + (size_t)b * V;
        float *dl = F(dlogits_buf) + (size_t)b * V;
        uint32_t action = act[b];
        float old = F(old_lp)[b], adv = F(advs)[b];
        for (int t = 0; t < tg; ++t) {
            float m = -1e30f;
            for (int i = t; i < V; i += tg) m = m > lg[i] ? m : lg[i];
            sh[t] = m;
        }
        float max_val = tg_tree_max(sh, tg);
        for (int t = 0; t < tg; ++t) {
            float s = 0;
            for (int i = t; i < V; i += tg) s += expf(lg[i] - max_val);
            sh[t] = s;
        }
        float lse = logf(tg_tree_sum(sh, tg)) + max_val;
        float nlp = lg[action] - lse;
        F(new_lp)[b] = nlp;
        float ratio = expf(nlp - old);
        float clipped = clampf(ratio, 1.0f - clip_eps, 1.0f + clip_eps);
        float weight = adv >= 0 ? (ratio <= clipped ? -adv : 0.0f) : (ratio >= clipped ? -adv : 0.0f);
        for (int i = 0; i < V; ++i) dl[i] = weight * ratio * (expf(lg[i] - lse) - ((uint32_t)i == action ? 1.0f : 0.0f));
    }
}
