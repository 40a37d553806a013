/*
 * llmb200_synth.h -- seeded synthetic weights and models (libllmb200_synth.so).
 *
 * Benchmarks and parity tests have no checkpoints to load; they build models of
 * the named architectures with reproducible random weights instead. The
 * reference initialises with Box-Muller on libc rand() (src/core/tensor.c:107-123),
 * which differs between C libraries; this generator is counter based and
 * bit-reproducible everywhere. Pure host code, no CUDA.
 */
#ifndef LLMB200_SYNTH_H
#define LLMB200_SYNTH_H

#include <stddef.h>
#include <stdint.h>
#include "llmb200_model_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    uint64_t seed;
    int   n_layers, d_model, n_q_heads, n_kv_heads, head_dim, intermediate_size, vocab_size;
    float rope_theta;          /* Qwen3 base; Gemma3 global-layer base */
    float local_rope_theta;    /* Gemma3 local-layer base */
    int   sliding_window;      /* Gemma3 field, carried but never applied (as in the reference) */
    float weight_std;          /* every matrix and the embedding: N(0, weight_std) */
    float gamma_jitter;        /* 0: all RMSNorm gammas 1.0 (reference default); >0: N(1, jitter) */
} llmb200_synth_spec;

/* which-values for llmb200_synth_tensor_id */
enum { LLMB200_T_Q = 0, LLMB200_T_K, LLMB200_T_V, LLMB200_T_O, LLMB200_T_GATE, LLMB200_T_UP, LLMB200_T_DOWN,
       LLMB200_T_QNORM, LLMB200_T_KNORM, LLMB200_T_INPUT_NORM, LLMB200_T_POST_ATTN_NORM,
       LLMB200_T_PRE_FF_NORM, LLMB200_T_POST_FF_NORM,
       LLMB200_T_EMB = 100, LLMB200_T_LM_HEAD, LLMB200_T_FINAL_NORM };
uint64_t llmb200_synth_tensor_id(int layer, int which);

/* dst[i] = mean + std * z_i for elements first..first+n of tensor `tensor_id`. */
void llmb200_synth_normal_range(float *dst, size_t first, size_t n, uint64_t seed, uint64_t tensor_id,
                                float mean, float std, int n_threads);
void llmb200_synth_normal(float *dst, size_t n, uint64_t seed, uint64_t tensor_id, float mean, float std, int n_threads);
/* Uniform token ids in [0, vocab). */
void llmb200_synth_tokens(uint32_t *dst, size_t n, uint64_t seed, uint32_t vocab);

llmb200_qwen3_model  *llmb200_synth_qwen3(const llmb200_synth_spec *spec, int n_threads);
void                  llmb200_synth_free_qwen3(llmb200_qwen3_model *m);
llmb200_gemma3_model *llmb200_synth_gemma3(const llmb200_synth_spec *spec, int n_threads);
void                  llmb200_synth_free_gemma3(llmb200_gemma3_model *m);

/* sizeof/offsetof table of the boundary structures (model ABI + weight
 * containers) as these headers declare them; returns the entry count. */
int llmb200_abi_layout(size_t *out, int cap);

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_SYNTH_H */
