/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement of llm.metal's decode path, used only as the checker in
 * tests/, in __graft_entry__.smoke() and in bench.py's cpu_baseline leg.
 * Nothing under llm.metal_b200/ links, loads or calls it.
 *
 * Parity pin: oracle/_ref (the reference's own C sources compiled in place,
 * see oracle/Makefile) is run against this restatement by
 * tests/test_oracle_vs_ref.py and produced the vectors under tests/golden/.
 * The reference's own tests hold no golden vector for this path.
 */
#ifndef LLMB200_ORACLE_H
#define LLMB200_ORACLE_H

#include <stddef.h>
#include <stdint.h>
#include "../include/llmb200_model_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* fp32 [rows, cols] -> rows*cols/32 canonical 34-byte blocks {u16 d; i8 qs[32]}.  src/nn/wmat.c:12-61 */
void oracle_q8_quantize(const float *src, int rows, int cols, uint8_t *blocks);
/* blocks -> fp32, w = (float)q * f16_to_f32(d).  src/data/gguf.c:225-253 */
void oracle_q8_dequantize(const uint8_t *blocks, size_t n_blocks, float *dst);
/* fp32 -> binary16 bits, round to nearest even.  src/nn/wmat.c:63-75 */
void oracle_f16_bits(const float *src, size_t n, uint16_t *dst);
float oracle_f16_to_f32(uint16_t h);

/* y[r] = sum_b f16(d_rb) * (sum_l q_rbl * x[32b+l]), fp32.  shaders/q8_kernels.metal:10-42 */
void oracle_q8_matvec(const uint8_t *blocks, const float *x, float *y, int rows, int nb);
/* y[r] = sum_c float(W[r,c]) * x[c].  shaders/q8_kernels.metal:97-127 */
void oracle_f16_matvec(const uint16_t *w, const float *x, float *y, int rows, int cols);
/* y = W x with fp32 W, sequential fp32 accumulation.  src/nn/layers.c:136-150 */
void oracle_linear(const float *w, const float *x, float *y, int rows, int cols);
/* y = gamma * x * (1/sqrtf(mean(x^2)+eps)).  src/nn/layers.c:362-377 */
void oracle_rms_norm(const float *x, const float *gamma, float *y, int dim, float eps);

typedef struct oracle_model oracle_model;
/* Copies the model, replacing every matrix by the values the fast path
 * multiplies with (Q8_0 or F16 rounding; use_fp16 as in inference_state_create). */
oracle_model *oracle_model_qwen3(const llmb200_qwen3_model *m, int use_fp16, int max_seq);
oracle_model *oracle_model_gemma3(const llmb200_gemma3_model *m, int use_fp16, int max_seq);
void oracle_model_free(oracle_model *m);
/* 0 (default): fp32 KV cache as in the reference; 1: K (after norm + RoPE) and
 * V are rounded to binary16 when stored, as the B200 build keeps them. */
void oracle_model_set_kv_f16(oracle_model *m, int on);
/* One token at position pos; logits may be NULL.  src/nn/fast_inference.c:376-467
 * with CPU arithmetic of src/nn/layers.c and src/nn/attention.c:660-856. */
void oracle_forward_token(oracle_model *m, int token, int pos, float *logits);
/* Greedy loop.  src/nn/fast_inference.c:614-675. logits_out (optional) gets one
 * row per logits-producing forward; seconds[0] prefill, seconds[1] decode. */
int oracle_generate(oracle_model *m, const uint32_t *prompt, int P, uint32_t *out, int max_gen,
                    const int *eos, int n_eos, float *logits_out, double *seconds);

#ifdef __cplusplus
}
#endif
#endif
