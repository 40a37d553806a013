/*
 * llmb200_model_abi.h -- host-side model structures read at the drop-in boundary.
 *
 * The decode and SFT engines of llm.metal never own the model: they receive a
 * Qwen3Model* / Gemma3Model* built by the caller (loader or random init) and
 * read only fp32 data pointers and integer dimensions out of it
 * (src/nn/fast_inference.c:113-168, 285-313; src/nn/fast_sft.c:212-239).
 * For a shared library to be callable with those very pointers the structure
 * layouts below have to agree, field for field, with the caller's:
 *
 *   Tensor                 src/core/tensor.h:15-29
 *   Linear/Embedding/RMSNorm  src/nn/layers.h:11-16, 38-42, 52-56
 *   GroupedQueryAttention  src/nn/attention.h:42-55
 *   LoRALinear             src/nn/lora.h:14-24
 *   Qwen3Block/Qwen3Model  src/nn/qwen3.h:15-45
 *   Gemma3Block/Gemma3Model src/nn/gemma3.h:14-53
 *
 * Only layout matters here; none of the reference's functions on these types
 * is re-implemented. tests/test_abi_layout.py checks sizeof/offsetof of every
 * structure against the reference headers when the reference tree is present.
 */
#ifndef LLMB200_MODEL_ABI_H
#define LLMB200_MODEL_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLMB200_TENSOR_RANK_MAX 4

typedef enum { LLMB200_F32 = 0, LLMB200_F16 = 1, LLMB200_U32 = 2 } llmb200_dtype;

/* Dense host tensor. Exactly one of the three data pointers is live, chosen by
 * dtype; the engines only ever dereference `data` (fp32). */
typedef struct llmb200_tensor {
    float    *data;
    uint16_t *data_f16;          /* binary16 payload (the caller sees _Float16*) */
    uint32_t *data_u32;
    int       ndim;
    int       shape[LLMB200_TENSOR_RANK_MAX];
    int       stride[LLMB200_TENSOR_RANK_MAX];
    size_t    size;              /* elements */
    size_t    bytes;
    int       dtype;             /* llmb200_dtype */
    void     *device_buf;        /* caller's accelerator handle; unused here */
    struct llmb200_tensor *grad;
    int       requires_grad;
    int       owns_data;
} llmb200_tensor;

typedef struct { llmb200_tensor *weight; llmb200_tensor *bias; int in_features; int out_features; } llmb200_linear;
typedef struct { llmb200_tensor *weight; int vocab_size; int dim; } llmb200_embedding;
typedef struct { llmb200_tensor *gamma; int dim; float eps; } llmb200_rmsnorm;

typedef struct {
    int   d_model, n_q_heads, n_kv_heads, head_dim;
    float scale, rope_theta;
    llmb200_linear  *q_proj, *k_proj, *v_proj, *o_proj;   /* [out, in] row-major */
    llmb200_rmsnorm *q_norm, *k_norm;                     /* gamma[head_dim] */
} llmb200_gqa;

typedef struct {
    llmb200_linear *base;
    llmb200_tensor *lora_A;      /* [rank, in]  */
    llmb200_tensor *lora_B;      /* [out, rank] */
    int   in_features, out_features, rank;
    float alpha, scaling;
    int   enabled;
} llmb200_lora_linear;

typedef struct {
    llmb200_rmsnorm *input_norm;
    llmb200_gqa     *attn;
    llmb200_rmsnorm *post_attn_norm;
    llmb200_linear  *gate_proj, *up_proj, *down_proj;
    int d_model;
} llmb200_qwen3_block;

typedef struct {
    llmb200_embedding    *token_emb;
    llmb200_qwen3_block **blocks;
    llmb200_rmsnorm      *final_norm;
    llmb200_linear       *lm_head;
    int   n_layers, d_model, vocab_size, n_q_heads, n_kv_heads, head_dim, intermediate_size;
    float rope_theta;
    llmb200_lora_linear **q_loras, **v_loras;   /* [n_layers] or NULL */
} llmb200_qwen3_model;

typedef struct {
    llmb200_rmsnorm *input_norm;
    llmb200_gqa     *attn;
    llmb200_rmsnorm *post_attn_norm;   /* applied to the attention output before the residual add */
    llmb200_rmsnorm *pre_ff_norm;
    llmb200_linear  *gate_proj, *up_proj, *down_proj;
    llmb200_rmsnorm *post_ff_norm;     /* applied to the FFN output before the residual add */
    int d_model;
    int is_sliding;                    /* 1: local layer (local RoPE base), 0: global */
} llmb200_gemma3_block;

typedef struct {
    llmb200_embedding     *token_emb;  /* also the (tied) LM head */
    llmb200_gemma3_block **blocks;
    llmb200_rmsnorm       *final_norm;
    int   n_layers, d_model, vocab_size, n_q_heads, n_kv_heads, head_dim, intermediate_size;
    int   sliding_window;
    float local_rope_theta, global_rope_theta;
    llmb200_lora_linear **q_loras, **v_loras;
} llmb200_gemma3_model;

/* The reference spells these types without a prefix. Translation units that do
 * not also include the reference's own headers can ask for those spellings. */
#ifdef LLMB200_REFERENCE_TYPE_NAMES
typedef llmb200_tensor        Tensor;
typedef llmb200_linear        Linear;
typedef llmb200_embedding     Embedding;
typedef llmb200_rmsnorm       RMSNorm;
typedef llmb200_gqa           GroupedQueryAttention;
typedef llmb200_lora_linear   LoRALinear;
typedef llmb200_qwen3_block   Qwen3Block;
typedef llmb200_qwen3_model   Qwen3Model;
typedef llmb200_gemma3_block  Gemma3Block;
typedef llmb200_gemma3_model  Gemma3Model;
#endif

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_MODEL_ABI_H */
