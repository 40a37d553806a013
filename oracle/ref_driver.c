/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Drives the reference's own CPU code (compiled from its sources where they
 * lie, see oracle/Makefile) through the decode path so that its results can
 * pin oracle/oracle.c and serve as the timed CPU baseline:
 *
 *   quantiser        wmat_create_q8 / wmat_create_f16   (src/nn/wmat.c:47-75)
 *   per-token block  the call sequence of qwen3_block_forward_cached
 *                    (src/nn/qwen3.c:81-125) built from rms_norm_forward,
 *                    gqa_forward_cached, linear_forward, silu_forward,
 *                    elementwise_mul -- with cache->cur_len set to the token
 *                    position before every layer. qwen3_forward_cached itself
 *                    is not usable: gqa_forward_cached advances cur_len once
 *                    per layer (src/nn/attention.c:675, 794), so layer l of
 *                    token t would be placed at position t*L+l.
 *   Gemma3           the reference has no CPU Gemma3 forward; the block order
 *                    of src/nn/fast_inference.c:386-466 is assembled from the
 *                    same CPU primitives (gelu_forward for the GeGLU gate).
 *   full recompute   qwen3_forward (src/nn/qwen3.c:376-396), used to cross-check
 *                    the cached driver.
 *
 * The weights the fast path multiplies with are Q8_0 or F16 roundings of the
 * fp32 model, so ref_requant_* first replaces every matrix W by
 * dequant(quant(W)) -- quantised by the reference's wmat.c, expanded as
 * (float)q * (float)d like dequantize_q8_0 (src/data/gguf.c:225-253).
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "nn/gemma3.h"
#include "nn/qwen3.h"
#include "nn/wmat.h"

size_t ref_q8_blocks(const float *src, int rows, int cols, void *out)
{
    WMat *w = wmat_create_q8(src, rows, cols);
    size_t bytes = (size_t)rows * w->nb * 34;
    if (out) memcpy(out, metal_buf_ptr(w->mbuf), bytes);
    wmat_free(w);
    return bytes;
}

size_t ref_f16_bits(const float *src, int rows, int cols, void *out)
{
    WMat *w = wmat_create_f16(src, rows, cols);
    size_t bytes = (size_t)rows * cols * 2;
    if (out) memcpy(out, metal_buf_ptr(w->mbuf), bytes);
    wmat_free(w);
    return bytes;
}

/* dst <- the values the fast path multiplies with */
static void requant_into(const float *src, float *dst, int rows, int cols, int use_fp16)
{
    /* row chunks keep the temporary small for the LM head */
    const int chunk = 4096;
    for (int r0 = 0; r0 < rows; r0 += chunk) {
        int nr = rows - r0 < chunk ? rows - r0 : chunk;
        const float *s = src + (size_t)r0 * cols;
        float *d = dst + (size_t)r0 * cols;
        if (use_fp16) {
            WMat *w = wmat_create_f16(s, nr, cols);
            const _Float16 *h = metal_buf_ptr(w->mbuf);
            for (size_t i = 0; i < (size_t)nr * cols; ++i) d[i] = (float)h[i];
            wmat_free(w);
        } else {
            WMat *w = wmat_create_q8(s, nr, cols);
            const unsigned char *b = metal_buf_ptr(w->mbuf);
            size_t nblk = (size_t)nr * w->nb;
            for (size_t k = 0; k < nblk; ++k) {
                _Float16 h;
                memcpy(&h, b + k * 34, 2);
                const signed char *q = (const signed char *)(b + k * 34 + 2);
                for (int j = 0; j < 32; ++j) d[k * 32 + j] = (float)q[j] * (float)h;
            }
            wmat_free(w);
        }
    }
}

static void requant_linear(Linear *l, int use_fp16)
{
    requant_into(l->weight->data, l->weight->data, l->out_features, l->in_features, use_fp16);
}

static void requant_gqa(GroupedQueryAttention *a, int f)
{
    requant_linear(a->q_proj, f); requant_linear(a->k_proj, f);
    requant_linear(a->v_proj, f); requant_linear(a->o_proj, f);
}

void ref_requant_qwen3(Qwen3Model *m, int use_fp16)
{
    for (int i = 0; i < m->n_layers; ++i) {
        Qwen3Block *b = m->blocks[i];
        requant_gqa(b->attn, use_fp16);
        requant_linear(b->gate_proj, use_fp16); requant_linear(b->up_proj, use_fp16); requant_linear(b->down_proj, use_fp16);
    }
    requant_linear(m->lm_head, use_fp16);       /* token_emb stays fp32: src/nn/fast_inference.c:248 */
}

void ref_requant_gemma3(Gemma3Model *m, int use_fp16)
{
    for (int i = 0; i < m->n_layers; ++i) {
        Gemma3Block *b = m->blocks[i];
        requant_gqa(b->attn, use_fp16);
        requant_linear(b->gate_proj, use_fp16); requant_linear(b->up_proj, use_fp16); requant_linear(b->down_proj, use_fp16);
    }
    /* the tied LM head is converted separately in ref_gemma3_generate; the table itself stays fp32 */
}

static int argmax_first(const float *v, int n)
{
    int best = 0;
    float bv = v[0];
    for (int i = 1; i < n; ++i) if (v[i] > bv) { bv = v[i]; best = i; }
    return best;
}

static Tensor *add_rows(Tensor *a, Tensor *b, int n)
{
    int sh[] = {1, n};
    Tensor *o = tensor_create(sh, 2, DTYPE_FP32, 0);
    for (int i = 0; i < n; ++i) o->data[i] = a->data[i] + b->data[i];
    return o;
}

static Tensor *embed_one(Embedding *e, int token)
{
    int sh[] = {1};
    Tensor *t = tensor_create(sh, 1, DTYPE_UINT32, 0);
    t->data_u32[0] = (uint32_t)token;
    Tensor *x = embedding_forward(e, t, NULL);
    tensor_free(t);
    return x;
}

static void qwen3_token(Qwen3Model *m, KVCache *cache, int token, int pos, float *logits)
{
    Tensor *x = embed_one(m->token_emb, token);
    for (int i = 0; i < m->n_layers; ++i) {
        Qwen3Block *b = m->blocks[i];
        Tensor *ln1 = rms_norm_forward(b->input_norm, x, NULL);
        cache->cur_len = pos;
        Tensor *at = gqa_forward_cached(b->attn, ln1, 1, 1, i, cache);
        Tensor *x2 = add_rows(x, at, m->d_model);
        Tensor *ln2 = rms_norm_forward(b->post_attn_norm, x2, NULL);
        Tensor *gate = linear_forward(b->gate_proj, ln2, NULL);
        Tensor *ga = silu_forward(gate, NULL);
        Tensor *up = linear_forward(b->up_proj, ln2, NULL);
        Tensor *pr = elementwise_mul(ga, up, NULL);
        Tensor *ff = linear_forward(b->down_proj, pr, NULL);
        Tensor *x3 = add_rows(x2, ff, m->d_model);
        tensor_free(ln1); tensor_free(at); tensor_free(x2); tensor_free(ln2); tensor_free(gate);
        tensor_free(ga); tensor_free(up); tensor_free(pr); tensor_free(ff); tensor_free(x);
        x = x3;
    }
    if (logits) {
        Tensor *nm = rms_norm_forward(m->final_norm, x, NULL);
        Tensor *lg = linear_forward(m->lm_head, nm, NULL);
        memcpy(logits, lg->data, (size_t)m->vocab_size * sizeof(float));
        tensor_free(nm); tensor_free(lg);
    }
    tensor_free(x);
}

static void gemma3_token(Gemma3Model *m, Linear *lm_head, KVCache *cache, int token, int pos, float *logits)
{
    Tensor *x = embed_one(m->token_emb, token);
    const float sc = sqrtf((float)m->d_model);
    for (int i = 0; i < m->d_model; ++i) x->data[i] *= sc;
    for (int i = 0; i < m->n_layers; ++i) {
        Gemma3Block *b = m->blocks[i];
        Tensor *ln1 = rms_norm_forward(b->input_norm, x, NULL);
        cache->cur_len = pos;
        Tensor *at = gqa_forward_cached(b->attn, ln1, 1, 1, i, cache);
        Tensor *atn = rms_norm_forward(b->post_attn_norm, at, NULL);
        Tensor *x2 = add_rows(x, atn, m->d_model);
        Tensor *ln2 = rms_norm_forward(b->pre_ff_norm, x2, NULL);
        Tensor *gate = linear_forward(b->gate_proj, ln2, NULL);
        Tensor *ga = gelu_forward(gate, NULL);
        Tensor *up = linear_forward(b->up_proj, ln2, NULL);
        Tensor *pr = elementwise_mul(ga, up, NULL);
        Tensor *ff = linear_forward(b->down_proj, pr, NULL);
        Tensor *ffn = rms_norm_forward(b->post_ff_norm, ff, NULL);
        Tensor *x3 = add_rows(x2, ffn, m->d_model);
        tensor_free(ln1); tensor_free(at); tensor_free(atn); tensor_free(x2); tensor_free(ln2); tensor_free(gate);
        tensor_free(ga); tensor_free(up); tensor_free(pr); tensor_free(ff); tensor_free(ffn); tensor_free(x);
        x = x3;
    }
    if (logits) {
        Tensor *nm = rms_norm_forward(m->final_norm, x, NULL);
        Tensor *lg = linear_forward(lm_head, nm, NULL);
        memcpy(logits, lg->data, (size_t)m->vocab_size * sizeof(float));
        tensor_free(nm); tensor_free(lg);
    }
    tensor_free(x);
}

static int is_eos(int t, const int *eos, int n) { for (int i = 0; i < n; ++i) if (t == eos[i]) return 1; return 0; }

static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + t.tv_nsec * 1e-9; }

/* Greedy loop of inference_generate (src/nn/fast_inference.c:614-675).
 * logits_out, when given, receives one row of V floats per forward that
 * produces logits the loop uses: row 0 = last prompt position, row g = g-th
 * decode forward. seconds[0] = prefill, seconds[1] = decode loop. */
int ref_qwen3_generate(Qwen3Model *m, const uint32_t *prompt, int P, uint32_t *out, int max_gen, int max_seq,
                       const int *eos, int n_eos, float *logits_out, double *seconds)
{
    KVCache *cache = kv_cache_create(m->n_layers, m->n_kv_heads, m->head_dim, max_seq);
    const int V = m->vocab_size;
    float *lg = malloc((size_t)V * sizeof(float));
    double t0 = now_s();
    for (int i = 0; i < P; ++i) qwen3_token(m, cache, (int)prompt[i], i, i == P - 1 ? lg : NULL);
    double t1 = now_s();
    int cur = P, next = argmax_first(lg, V), n = 1;
    if (logits_out) memcpy(logits_out, lg, (size_t)V * sizeof(float));
    out[0] = (uint32_t)next;
    for (int g = 1; g < max_gen && cur < max_seq; ++g) {
        if (is_eos(next, eos, n_eos)) break;
        qwen3_token(m, cache, next, cur, lg);
        cur++;
        if (logits_out) memcpy(logits_out + (size_t)n * V, lg, (size_t)V * sizeof(float));
        next = argmax_first(lg, V);
        out[n++] = (uint32_t)next;
    }
    double t2 = now_s();
    if (seconds) { seconds[0] = t1 - t0; seconds[1] = t2 - t1; }
    free(lg);
    kv_cache_free(cache);
    return n;
}

int ref_gemma3_generate(Gemma3Model *m, int use_fp16, const uint32_t *prompt, int P, uint32_t *out, int max_gen, int max_seq,
                        const int *eos, int n_eos, float *logits_out, double *seconds)
{
    KVCache *cache = kv_cache_create(m->n_layers, m->n_kv_heads, m->head_dim, max_seq);
    const int V = m->vocab_size;
    /* tied LM head: a converted copy of the embedding table (src/nn/fast_inference.c:307-313, 246) */
    Linear lm = {0};
    int sh[] = {V, m->d_model};
    lm.weight = tensor_create(sh, 2, DTYPE_FP32, 0);
    lm.in_features = m->d_model; lm.out_features = V;
    requant_into(m->token_emb->weight->data, lm.weight->data, V, m->d_model, use_fp16);
    float *lg = malloc((size_t)V * sizeof(float));
    double t0 = now_s();
    for (int i = 0; i < P; ++i) gemma3_token(m, &lm, cache, (int)prompt[i], i, i == P - 1 ? lg : NULL);
    double t1 = now_s();
    int cur = P, next = argmax_first(lg, V), n = 1;
    if (logits_out) memcpy(logits_out, lg, (size_t)V * sizeof(float));
    out[0] = (uint32_t)next;
    for (int g = 1; g < max_gen && cur < max_seq; ++g) {
        if (is_eos(next, eos, n_eos)) break;
        gemma3_token(m, &lm, cache, next, cur, lg);
        cur++;
        if (logits_out) memcpy(logits_out + (size_t)n * V, lg, (size_t)V * sizeof(float));
        next = argmax_first(lg, V);
        out[n++] = (uint32_t)next;
    }
    double t2 = now_s();
    if (seconds) { seconds[0] = t1 - t0; seconds[1] = t2 - t1; }
    free(lg);
    tensor_free(lm.weight);
    kv_cache_free(cache);
    return n;
}

/* Full causal recompute over tokens[0..n): logits of the last position. */
void ref_qwen3_forward_full(Qwen3Model *m, const uint32_t *tokens, int n, float *logits_last)
{
    int sh[] = {n};
    Tensor *t = tensor_create(sh, 1, DTYPE_UINT32, 0);
    memcpy(t->data_u32, tokens, (size_t)n * sizeof(uint32_t));
    Tensor *lg = qwen3_forward(m, t, 1, n, NULL);
    memcpy(logits_last, lg->data + (size_t)(n - 1) * m->vocab_size, (size_t)m->vocab_size * sizeof(float));
    tensor_free(t);
    /* intermediates of qwen3_forward are owned by nobody without a graph; the process is short-lived */
    tensor_free(lg);
}

/* One plain CPU linear layer y = W x (src/nn/layers.c:136-150), for the matvec sweep. */
void ref_linear(const float *w, const float *x, float *y, int rows, int cols)
{
    Linear l = {0};
    Tensor wt = {0}, xt = {0};
    wt.data = (float *)w; wt.ndim = 2; wt.shape[0] = rows; wt.shape[1] = cols; wt.size = (size_t)rows * cols;
    xt.data = (float *)x; xt.ndim = 2; xt.shape[0] = 1; xt.shape[1] = cols; xt.size = (size_t)cols;
    l.weight = &wt; l.in_features = cols; l.out_features = rows;
    Tensor *o = linear_forward(&l, &xt, NULL);
    memcpy(y, o->data, (size_t)rows * sizeof(float));
    tensor_free(o);
}

/* sizeof/offsetof table of the caller-side structures, for the layout test. */
#include <stddef.h>
int ref_abi_layout(size_t *out, int cap)
{
    size_t v[] = {
        sizeof(Tensor), offsetof(Tensor, data), offsetof(Tensor, ndim), offsetof(Tensor, shape), offsetof(Tensor, stride),
        offsetof(Tensor, size), offsetof(Tensor, bytes), offsetof(Tensor, dtype), offsetof(Tensor, metal_buf),
        offsetof(Tensor, grad), offsetof(Tensor, requires_grad), offsetof(Tensor, owns_data),
        sizeof(Linear), offsetof(Linear, weight), offsetof(Linear, in_features), offsetof(Linear, out_features),
        sizeof(Embedding), offsetof(Embedding, weight), offsetof(Embedding, dim),
        sizeof(RMSNorm), offsetof(RMSNorm, gamma), offsetof(RMSNorm, dim), offsetof(RMSNorm, eps),
        sizeof(GroupedQueryAttention), offsetof(GroupedQueryAttention, rope_theta), offsetof(GroupedQueryAttention, q_proj),
        offsetof(GroupedQueryAttention, o_proj), offsetof(GroupedQueryAttention, q_norm), offsetof(GroupedQueryAttention, k_norm),
        sizeof(LoRALinear), offsetof(LoRALinear, lora_A), offsetof(LoRALinear, lora_B), offsetof(LoRALinear, rank),
        offsetof(LoRALinear, scaling), offsetof(LoRALinear, enabled),
        sizeof(Qwen3Block), offsetof(Qwen3Block, attn), offsetof(Qwen3Block, post_attn_norm), offsetof(Qwen3Block, down_proj),
        sizeof(Qwen3Model), offsetof(Qwen3Model, blocks), offsetof(Qwen3Model, lm_head), offsetof(Qwen3Model, n_layers),
        offsetof(Qwen3Model, intermediate_size), offsetof(Qwen3Model, rope_theta), offsetof(Qwen3Model, q_loras),
        offsetof(Qwen3Model, v_loras),
        sizeof(Gemma3Block), offsetof(Gemma3Block, pre_ff_norm), offsetof(Gemma3Block, post_ff_norm), offsetof(Gemma3Block, is_sliding),
        sizeof(Gemma3Model), offsetof(Gemma3Model, final_norm), offsetof(Gemma3Model, n_layers), offsetof(Gemma3Model, sliding_window),
        offsetof(Gemma3Model, local_rope_theta), offsetof(Gemma3Model, global_rope_theta), offsetof(Gemma3Model, q_loras),
        sizeof(WMat), offsetof(WMat, rows), offsetof(WMat, nb),
        sizeof(LayerW), offsetof(LayerW, down_proj), offsetof(LayerW, input_norm_g), offsetof(LayerW, k_norm_g),
        sizeof(WeightRef), sizeof(LayerWeightRef), offsetof(LayerWeightRef, input_norm_g), offsetof(LayerWeightRef, d_model),
        offsetof(LayerWeightRef, head_dim),
    };
    int n = (int)(sizeof(v) / sizeof(v[0]));
    for (int i = 0; i < n && i < cap; ++i) out[i] = v[i];
    return n;
}
