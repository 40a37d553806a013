/*
 * llmb200_sft.h -- the LoRA-SFT engine at the drop-in boundary.
 *
 * Part 1 declares, under the reference's names and with the same argument
 * meaning, the LoRA subset of llm.metal's fast SFT engine
 * (src/nn/fast_sft.h:14-111; implementation src/nn/fast_sft.c): LoRA and
 * full-parameter training of Qwen3 and of Gemma3.
 *
 * Part 2 is additive: layer-by-layer construction, several sequences per
 * step (their LoRA gradients are averaged, then one clip + AdamW as in the
 * reference), the flat gradient vector a data-parallel caller all-reduces,
 * and parity / measurement hooks.
 *
 * Buffers the reference exposes as shared CPU/GPU memory (x, losses, LoRA
 * gradients, logits) are device memory here with pinned host mirrors: a host
 * pointer returned by an accessor is refreshed from the device by that call,
 * and host data is pushed to the device by the call that consumes it
 * (forward_to_logits reads the x mirror, sft_set_lora_grad writes through).
 */
#ifndef LLMB200_SFT_H
#define LLMB200_SFT_H

#include <stdint.h>
#include "llmb200_model_abi.h"
#include "llmb200_wmat.h"
#include "llmb200_inference.h"   /* llmb200_config */

#ifdef __cplusplus
extern "C" {
#endif

/* ========================= Part 1: reference interface ==================== */

typedef struct SFTState SFTState;

/* Uploads every matrix rounded to binary16 values, initialises LoRA on the Q
 * and V projections (from model->q_loras / v_loras when attached, else
 * A ~ uniform(+-1/sqrt(d_model)) from rand(), B = 0) and allocates the saved
 * activations for one sequence of seq_len tokens. NULL with a message on
 * stderr on failure. Replaces sft_state_create (src/nn/fast_sft.c:171-278). */
SFTState *sft_state_create(llmb200_qwen3_model *model, int seq_len, int lora_rank, float lora_alpha);
void sft_state_free(SFTState *state);                              /* :1360-1422 */

/* Embedding gather, forward, cross-entropy against target_tokens, backward,
 * then step_count++, global-norm clip at 1.0 and AdamW (beta 0.9/0.999,
 * eps 1e-8, weight decay 0.01) on the LoRA matrices. Returns the mean loss.
 * Replaces sft_train_step (:1113-1157). */
float sft_train_step(SFTState *state, const uint32_t *input_tokens, const uint32_t *target_tokens, float lr);

/* Forward from the embeddings the caller placed in sft_get_x_cpu() to the
 * logits (:616-752), and backward from the gradient in sft_get_dlogits() to
 * the LoRA gradients (:766-982 LoRA branch, sft_backward :984). */
void forward_to_logits(SFTState *state);
void sft_backward(SFTState *state);

MetalBuf *sft_get_logits(SFTState *state);                         /* [N, V] fp32; :1210 */
MetalBuf *sft_get_dlogits(SFTState *state);                        /* :1211 */
float *sft_get_x_cpu(SFTState *state);                             /* [N, D] host, read by forward_to_logits */
float *sft_get_losses_cpu(SFTState *state);                        /* [N] host, refreshed by this call */
int sft_get_seq_len(SFTState *state);
int sft_get_vocab_size(SFTState *state);
int sft_get_d_model(SFTState *state);
int sft_get_lora_rank(SFTState *state);
int sft_get_n_layers(SFTState *state);
float sft_get_emb_scale(SFTState *state);
const float *sft_get_token_emb(SFTState *state);                   /* host copy; NULL for a streamed state */
int sft_get_step_count(SFTState *state);
void sft_set_step_count(SFTState *state, int step);

/* 4 gradient buffers per layer in the order dA_q, dB_q, dA_v, dB_v (:1225-1246).
 * The pointer addresses a host mirror refreshed by the call. */
int sft_get_n_lora_grad_bufs(SFTState *state);
float *sft_get_lora_grad_ptr(SFTState *state, int idx, int *out_size);
void sft_set_lora_grad(SFTState *state, int idx, const float *data, int size);
/* Clip + AdamW with the current step_count (does not increment it; :1248-1251). */
void sft_lora_update(SFTState *state, float lr);
/* "LORA" adapter file: u32 0x4C4F5241, i32 n_layers, i32 rank, then per layer
 * A_q[R,D] B_q[Hq*hd,R] A_v[R,D] B_v[Hkv*hd,R] fp32 (:1255-1285). */
void sft_save_lora(SFTState *state, const char *path);
/* sub: 0 = A_q, 1 = B_q, 2 = A_v, 3 = B_v; device buffers (:1253-1263). */
MetalBuf *sft_get_lora_weight_buf(SFTState *state, int layer, int sub);
float sft_get_lora_scaling(SFTState *state);
/* Copies the LoRA matrices into model->q_loras / v_loras, which must be
 * attached (the reference attaches them itself through qwen3_attach_lora,
 * which lives outside this library; :1163-1181). Returns silently otherwise. */
void sft_sync_lora_to_model(SFTState *state, llmb200_qwen3_model *model);

/* Weight-sharing accessors, used by inference_state_create_from_sft
 * (src/nn/fast_sft.h:101-111; src/nn/fast_sft.c:1346-1354). The containers are
 * views of this state's device memory: every WMat is one projection as
 * row-major binary16 [rows, cols] (metal_buf_ptr on its buffer gives the
 * reference's canonical bytes), every norm vector an fp32 buffer. They stay
 * valid until sft_state_free and must not be freed by the caller. */
LayerW *sft_get_layers(SFTState *state);
WMat *sft_get_lm_head(SFTState *state);
MetalBuf *sft_get_final_norm_g(SFTState *state);
ModelType sft_get_model_type(SFTState *state);
int sft_get_n_q_heads(SFTState *state);
int sft_get_n_kv_heads(SFTState *state);
int sft_get_head_dim(SFTState *state);
int sft_get_intermediate_size(SFTState *state);
const float *sft_get_rope_thetas(SFTState *state);

/* ---- full-parameter mode (src/nn/fast_sft.h:21-41) ----
 * sft_state_create_full: no adapter; q, k, v, o, gate, up, down of every layer and the LM head are trained by
 * plain SGD on their binary16 values (src/nn/fast_sft.c:402-501). Held as fp32 copies of binary16 values; every
 * product of such a state runs in fp32 on the CUDA cores. On such a state
 *   sft_train_step        forward, loss, and a backward pass that steps each weight as its gradient is formed:
 *                         W <- half(W - lr dY^T X) (f16_sgd_fused, q8_kernels.metal:1097-1125); q, k, v step
 *                         before the gradient goes on through them, the others after (:766-982). No optimizer
 *                         state, the step count stays.
 *   sft_backward_sgd      that backward pass alone, from the gradient in sft_get_dlogits().
 *   sft_alloc_grad_accum  binary16 accumulators for every matrix, zeroed (:996-1019). From then on every
 *                         backward pass of the state (sft_train_step and sft_backward_sgd included, as in the
 *                         reference) adds G <- half(G + dY^T X) (f16_grad_accum, :1164-1191) and moves no weight.
 *   sft_backward_accum    the accumulating backward pass (:986).
 *   sft_apply_grad_sgd    W <- half(W - lr G), G <- 0 (f16_sgd_apply, :1195-1206; :1021-1039).
 *   sft_save_full_checkpoint   "FULL" header of nine words, then every matrix as binary16 (:1287-1343).
 * A decode state made from the state (inference_state_create_from_sft) follows the stepped weights. */
SFTState *sft_state_create_full(llmb200_qwen3_model *model, int seq_len);
int  sft_is_full_param(SFTState *state);
void sft_backward_sgd(SFTState *state, float lr);
void sft_alloc_grad_accum(SFTState *state);
void sft_backward_accum(SFTState *state);
void sft_apply_grad_sgd(SFTState *state, float lr);
void sft_save_full_checkpoint(SFTState *state, const char *path);

/* ---- Gemma3 (src/nn/fast_sft.h:17-19, 23, 55; src/nn/fast_sft.c:284-396, 507-610) ----
 * The same calls on a Gemma3 model: four norms per layer (the post-attention and post-feedforward norms act on
 * the projection outputs before the residual add), GeGLU, embeddings scaled by sqrt(d_model), the LM head a
 * binary16 copy of the embedding table, the RoPE base per layer by position in the stack (every sixth layer
 * global). Such a state computes every product in fp32 on the CUDA cores. */
SFTState *sft_state_create_gemma3(llmb200_gemma3_model *model, int seq_len, int lora_rank, float lora_alpha);
SFTState *sft_state_create_gemma3_full(llmb200_gemma3_model *model, int seq_len);
void sft_sync_lora_to_gemma3(SFTState *state, llmb200_gemma3_model *model);

/* ========================= Part 2: additions ============================== */

/* cfg->max_seq_len and use_fp16 are ignored. n_seq sequences of seq_len tokens
 * form one step. */
SFTState *llmb200_sft_begin(const llmb200_config *cfg, int seq_len, int n_seq, int lora_rank, float lora_alpha);
/* refs holds the layer's fp32 matrices and norm gammas. lora = {A_q, B_q, A_v,
 * B_v} host pointers; NULL entries (or lora == NULL) take the default init. */
int llmb200_sft_load_layer(SFTState *state, int layer, const LayerWeightRef *refs, float rope_theta,
                           const float *const lora[4]);
/* keep_host_emb != 0 keeps a host copy of the table for sft_get_token_emb. */
int llmb200_sft_finish(SFTState *state, const float *lm_head, const float *final_norm_gamma,
                       const float *token_emb, int keep_host_emb);

/* inputs/targets [n_seq * seq_len]. Forward + loss + backward for all
 * sequences in one pass; the LoRA gradients are the mean over sequences of the
 * reference's per-sequence gradients. Returns the mean loss; no update. */
float llmb200_sft_forward_backward(SFTState *state, const uint32_t *inputs, const uint32_t *targets);
/* step_count++, clip, AdamW (the tail of sft_train_step). */
void llmb200_sft_apply_update(SFTState *state, float lr);
/* forward_backward + apply_update. */
float llmb200_sft_train_batch(SFTState *state, const uint32_t *inputs, const uint32_t *targets, float lr);

/* The flat device vector of all LoRA gradients (layer-major, dA_q dB_q dA_v
 * dB_v within a layer): what data-parallel ranks all-reduce (mean) between
 * llmb200_sft_forward_backward and llmb200_sft_apply_update. Returns the
 * element count. */
size_t llmb200_sft_grad_vector(SFTState *state, void **device_ptr);
size_t llmb200_sft_param_vector(SFTState *state, void **device_ptr);
/* Gradient norm seen by the last clip. */
float llmb200_sft_last_grad_norm(SFTState *state);
/* Device milliseconds (CUDA events) of the last forward+loss+backward and of
 * the last clip+AdamW. */
float llmb200_sft_last_step_ms(SFTState *state, float *update_ms);
/* Returns 1 when the state runs the frozen projections on the tensor cores
 * (binary16 operands, fp32 accumulate; the default when the dimensions allow
 * it), 0 when every product runs on the CUDA cores in fp32 (LLMB200_SFT_TC=0
 * at creation). The mode is fixed when the state is created -- the weights are
 * stored for it -- so `on` is ignored. */
int llmb200_sft_use_tensor_cores(SFTState *state, int on);
/* Non-zero once a launch or copy has failed. */
int llmb200_sft_error(SFTState *state);

/* Parity hook: copies a saved activation or intermediate of `layer` to dst
 * (fp32, cap floats); returns the element count or 0. */
enum { LLMB200_SFT_X_IN = 0, LLMB200_SFT_LN1, LLMB200_SFT_QKV, LLMB200_SFT_Q_FINAL, LLMB200_SFT_K_FINAL,
       LLMB200_SFT_PROBS, LLMB200_SFT_X_MID, LLMB200_SFT_LN2, LLMB200_SFT_GATE_UP, LLMB200_SFT_MID_Q,
       LLMB200_SFT_MID_V, LLMB200_SFT_LOGITS = 100, LLMB200_SFT_DLOGITS, LLMB200_SFT_LOSSES, LLMB200_SFT_X_FINAL,
       LLMB200_SFT_LORA_GRADS = 200, LLMB200_SFT_LORA_PARAMS /* the flat vectors; layer is ignored */ };
size_t llmb200_sft_export(SFTState *state, int what, int layer, float *dst, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_SFT_H */
