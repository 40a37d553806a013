/*
 * Batched F16 decode of libllmb200 (host side, C): B sequences advance one position per step and share
 * one read of the weights.
 *
 * Stands in for BatchState / forward_token_batch / qwen3_generate_fast_batch
 * (src/nn/fast_inference.c:696-985). The reference keeps the matvec shape and loops the batch inside
 * the kernel (f16_batch_matvec, shaders/q8_kernels.metal:49-90); with B rows the projections are small
 * matrix products, so here they run on the tensor cores (b200_gemm_f16: binary16 weights, a binary16
 * copy of the B activation rows, fp32 accumulate), the row-wise steps use the training kernels over
 * B rows, and attention is the decode kernel with the batch as a third grid dimension over per-sequence
 * F16 KV caches. The arg-max, the token feedback and the position live on the device: one step is one
 * CUDA graph.
 */
#include "internal.h"
#include "../../include/llmb200_inference.h"
#include "../../include/llmb200_train_kernels.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct {
    void *qkv, *o, *gu, *down;            /* binary16 [rows, cols] */
    float *g_in, *g_post, *g_q, *g_k, *inv_freq;
    void *k_cache, *v_cache;              /* binary16 [B][n_kv][max_seq][hd] */
    int loaded;
} BLayer;

struct llmb200_batch_state {
    int D, Hq, Hkv, hd, IS, V, L, B, max_seq, QKV, n_split;
    BLayer *layers;
    void *lm_head;
    float *g_final, *emb;
    float *x[2], *ln, *qkv, *att, *gu, *logits, *scratch;
    void *xh;
    unsigned *tickets, *d_tok, *d_hist, *d_done;
    int *d_ctl;
    unsigned *h_tok;                      /* pinned [max(B, max_hist)] */
    int *h_ctl;
    int hist_cap;
    int eos[4], n_eos;
    cudaGraphExec_t graph;
    int finished, err;
    double last_decode_ms;
    int last_steps;
    int kernels_per_step;
};
typedef struct llmb200_batch_state BState;

#define B_TRY(s, call)                                                                       \
    do {                                                                                     \
        int e__ = (call);                                                                    \
        if (e__ != 0 && !(s)->err) {                                                         \
            (s)->err = e__;                                                                  \
            fprintf(stderr, "[llmb200] batch: %s failed: code %d (%s:%d)\n", #call, e__, __FILE__, __LINE__); \
        }                                                                                    \
    } while (0)

static void *dmalloc(BState *s, size_t bytes)
{
    void *p = NULL;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        fprintf(stderr, "[BatchGen] allocating %zu bytes failed: %s\n", bytes, cudaGetErrorString(e));
        if (!s->err) s->err = (int)e;
        return NULL;
    }
    return p;
}

void llmb200_batch_free(BState *s)
{
    if (!s) return;
    if (g_rt.refs > 0) cudaStreamSynchronize(g_rt.stream);
    if (s->graph) cudaGraphExecDestroy(s->graph);
    for (int l = 0; l < s->L && s->layers; ++l) {
        BLayer *y = &s->layers[l];
        void *b[] = { y->qkv, y->o, y->gu, y->down, y->g_in, y->g_post, y->g_q, y->g_k, y->inv_freq, y->k_cache, y->v_cache };
        for (size_t i = 0; i < sizeof(b) / sizeof(b[0]); ++i) cudaFree(b[i]);
    }
    void *b[] = { s->lm_head, s->g_final, s->emb, s->x[0], s->x[1], s->ln, s->qkv, s->att, s->gu, s->logits, s->scratch,
                  s->xh, s->tickets, s->d_tok, s->d_hist, s->d_done, s->d_ctl };
    for (size_t i = 0; i < sizeof(b) / sizeof(b[0]); ++i) cudaFree(b[i]);
    if (s->h_tok) cudaFreeHost(s->h_tok);
    if (s->h_ctl) cudaFreeHost(s->h_ctl);
    free(s->layers);
    free(s);
    fast_metal_shutdown();
}

BState *llmb200_batch_begin(const llmb200_config *c, int batch_size, int max_gen_len)
{
    if (!c || batch_size < 1 || batch_size > 32 || max_gen_len < 1 || c->model_type != MODEL_QWEN3 ||
        (c->head_dim != 64 && c->head_dim != 128 && c->head_dim != 256) || c->n_kv_heads <= 0 ||
        c->n_q_heads % c->n_kv_heads || (c->d_model % 8) || (c->intermediate_size % 8) || c->vocab_size < 64) {
        fprintf(stderr, "[BatchGen] unsupported configuration (Qwen3 only, batch 1..32, dimensions in multiples of 8)\n");
        return NULL;
    }
    if (fast_metal_init() != 0) {
        fprintf(stderr, "[BatchGen] device init failed\n");
        return NULL;
    }
    BState *s = calloc(1, sizeof(BState));
    if (!s) { fast_metal_shutdown(); return NULL; }
    s->D = c->d_model; s->Hq = c->n_q_heads; s->Hkv = c->n_kv_heads; s->hd = c->head_dim; s->IS = c->intermediate_size;
    s->V = c->vocab_size; s->L = c->n_layers; s->B = batch_size;
    s->max_seq = c->max_seq_len > 4096 ? 4096 : c->max_seq_len;          /* as the reference clamps (:720) */
    if (s->max_seq < 1) s->max_seq = 1;
    s->QKV = (s->Hq + 2 * s->Hkv) * s->hd;
    {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g_rt.device) != cudaSuccess || sms <= 0) sms = 1;
        s->n_split = sms / (s->Hkv * s->B);
    }
    if (s->n_split < 1) s->n_split = 1;
    if (s->n_split > (s->max_seq + 63) / 64) s->n_split = (s->max_seq + 63) / 64;
    s->hist_cap = max_gen_len;
    s->eos[0] = 151645; s->eos[1] = 151643; s->eos[2] = 0; s->n_eos = 3;  /* the reference's list, id 0 included (:944-946) */
    s->layers = calloc(s->L, sizeof(BLayer));
    const size_t B = s->B, D = s->D, Hq_hd = (size_t)s->Hq * s->hd, Hkv_hd = (size_t)s->Hkv * s->hd;
    for (int l = 0; l < s->L && !s->err; ++l) {
        BLayer *y = &s->layers[l];
        y->qkv = dmalloc(s, (size_t)s->QKV * D * 2); y->o = dmalloc(s, D * Hq_hd * 2);
        y->gu = dmalloc(s, (size_t)2 * s->IS * D * 2); y->down = dmalloc(s, D * s->IS * 2);
        y->g_in = dmalloc(s, D * 4); y->g_post = dmalloc(s, D * 4);
        y->g_q = dmalloc(s, s->hd * 4); y->g_k = dmalloc(s, s->hd * 4); y->inv_freq = dmalloc(s, s->hd * 2);
        y->k_cache = dmalloc(s, B * Hkv_hd * s->max_seq * 2); y->v_cache = dmalloc(s, B * Hkv_hd * s->max_seq * 2);
    }
    s->lm_head = dmalloc(s, (size_t)s->V * D * 2);
    s->g_final = dmalloc(s, D * 4); s->emb = dmalloc(s, (size_t)s->V * D * 4);
    s->x[0] = dmalloc(s, B * D * 4); s->x[1] = dmalloc(s, B * D * 4); s->ln = dmalloc(s, B * D * 4);
    s->qkv = dmalloc(s, B * s->QKV * 4); s->att = dmalloc(s, B * Hq_hd * 4); s->gu = dmalloc(s, B * 2 * s->IS * 4);
    s->logits = dmalloc(s, B * (size_t)s->V * 4);
    size_t widest = (size_t)(2 * s->IS > s->QKV ? 2 * s->IS : s->QKV);
    if (D > widest) widest = D;
    s->xh = dmalloc(s, B * widest * 2);
    s->scratch = dmalloc(s, B * b200_attn_scratch_floats(s->Hq, s->hd, s->n_split) * 4);
    s->tickets = dmalloc(s, B * s->Hkv * 4);
    s->d_tok = dmalloc(s, B * 4); s->d_hist = dmalloc(s, (size_t)s->hist_cap * B * 4);
    s->d_done = dmalloc(s, 4); s->d_ctl = dmalloc(s, 16);
    if (!s->err) {
        cudaMemsetAsync(s->tickets, 0, B * s->Hkv * 4, g_rt.stream);
        cudaMemsetAsync(s->d_done, 0, 4, g_rt.stream);
        cudaMemsetAsync(s->d_ctl, 0, 16, g_rt.stream);
        size_t ht = (size_t)s->hist_cap * B;
        if (cudaMallocHost((void **)&s->h_tok, (ht > B ? ht : B) * 4) != cudaSuccess ||
            cudaMallocHost((void **)&s->h_ctl, 16) != cudaSuccess)
            s->err = -11;
    }
    if (s->err) { llmb200_batch_free(s); return NULL; }
    return s;
}

static int put_half(void *dst, size_t row0, int cols, const float *src, int rows)
{
    if (!src) return B200_E_BADARG;
    return llmb200_upload_f16_into((char *)dst + row0 * cols * 2, src, (size_t)rows * cols);
}

int llmb200_batch_load_layer(BState *s, int l, const LayerWeightRef *r, float rope_theta)
{
    if (!s || !r || l < 0 || l >= s->L) return B200_E_BADARG;
    BLayer *y = &s->layers[l];
    const int D = s->D, Hq_hd = s->Hq * s->hd, Hkv_hd = s->Hkv * s->hd;
    if (r->q_proj.rows != Hq_hd || r->q_proj.cols != D || r->k_proj.rows != Hkv_hd || r->v_proj.rows != Hkv_hd ||
        r->o_proj.rows != D || r->o_proj.cols != Hq_hd || r->gate_proj.rows != s->IS || r->up_proj.rows != s->IS ||
        r->down_proj.rows != D || r->down_proj.cols != s->IS)
        return B200_E_BADARG;
    int rc = put_half(y->qkv, 0, D, r->q_proj.data, Hq_hd);
    if (!rc) rc = put_half(y->qkv, Hq_hd, D, r->k_proj.data, Hkv_hd);
    if (!rc) rc = put_half(y->qkv, Hq_hd + Hkv_hd, D, r->v_proj.data, Hkv_hd);
    if (!rc) rc = put_half(y->o, 0, Hq_hd, r->o_proj.data, D);
    if (!rc) rc = put_half(y->gu, 0, D, r->gate_proj.data, s->IS);
    if (!rc) rc = put_half(y->gu, s->IS, D, r->up_proj.data, s->IS);
    if (!rc) rc = put_half(y->down, 0, s->IS, r->down_proj.data, D);
    if (!rc) rc = r->input_norm_g ? llmb200_upload_f32_into(y->g_in, r->input_norm_g, D) : B200_E_BADARG;
    if (!rc) rc = r->post_attn_norm_g ? llmb200_upload_f32_into(y->g_post, r->post_attn_norm_g, D) : B200_E_BADARG;
    if (!rc) rc = r->q_norm_g ? llmb200_upload_f32_into(y->g_q, r->q_norm_g, s->hd) : B200_E_BADARG;
    if (!rc) rc = r->k_norm_g ? llmb200_upload_f32_into(y->g_k, r->k_norm_g, s->hd) : B200_E_BADARG;
    if (rc) return rc;
    const int half = s->hd / 2;
    float *f = malloc(half * sizeof(float));
    for (int d = 0; d < half; ++d) f[d] = 1.0f / powf(rope_theta, (float)(2 * d) / (float)s->hd);   /* attention.c:757-758 */
    rc = llmb200_upload_f32_into(y->inv_freq, f, half);
    free(f);
    y->loaded = rc == 0;
    return rc;
}

int llmb200_batch_finish(BState *s, const float *lm_head, const float *final_norm_gamma, const float *token_emb)
{
    if (!s || !lm_head || !final_norm_gamma || !token_emb) return B200_E_BADARG;
    for (int l = 0; l < s->L; ++l)
        if (!s->layers[l].loaded) return B200_E_STATE;
    int rc = put_half(s->lm_head, 0, s->D, lm_head, s->V);
    if (!rc) rc = llmb200_upload_f32_into(s->g_final, final_norm_gamma, s->D);
    if (!rc) rc = llmb200_upload_f32_into(s->emb, token_emb, (size_t)s->V * s->D);
    if (!rc) rc = (int)cudaStreamSynchronize(g_rt.stream);
    s->finished = rc == 0;
    return rc;
}

/* C[B, N] = half(A)[B, K] * Wh[N, K]^T (+ R); A == NULL: the operand is already in xh */
static void proj(BState *s, const float *A, const void *Wh, int N, int K, float *C, const float *R)
{
    if (A) B_TRY(s, b200_f32_to_f16(A, (size_t)s->B * K, 1.0f, s->xh, g_rt.stream));
    b200_gemm_args g;
    memset(&g, 0, sizeof(g));
    g.A = (const float *)s->xh; g.a_row = K; g.a_col = 1;
    g.B = (const float *)Wh; g.b_row = 1; g.b_col = K;
    g.C = C; g.ldc = N; g.R = R; g.ldr = N;
    g.M = s->B; g.N = N; g.K = K; g.alpha = 1.0f;
    B_TRY(s, b200_gemm_f16(&g, g_rt.stream));
}

/* one step for all sequences: tokens from d_tok at position d_ctl[0] */
static void enqueue_step(BState *s)
{
    void *st = g_rt.stream;
    const int B = s->B, D = s->D, Hq_hd = s->Hq * s->hd, Hkv_hd = s->Hkv * s->hd;
    float *x = s->x[0], *x2 = s->x[1];
    B_TRY(s, b200_embed_rows(s->emb, s->d_tok, B, D, s->V, 1.0f, x, st));
    for (int l = 0; l < s->L; ++l) {
        BLayer *y = &s->layers[l];
        B_TRY(s, b200_rms_norm_rows_h(x, y->g_in, s->ln, s->xh, B, D, 1e-6f, st));
        proj(s, NULL, y->qkv, s->QKV, D, s->qkv, NULL);
        b200_attn_args at;
        memset(&at, 0, sizeof(at));
        at.d_qkv = s->qkv; at.d_q_gamma = y->g_q; at.d_k_gamma = y->g_k; at.d_inv_freq = y->inv_freq;
        at.d_k_cache = y->k_cache; at.d_v_cache = y->v_cache;
        at.d_out = s->att; at.d_scratch = s->scratch; at.d_tickets = s->tickets; at.d_pos = s->d_ctl;
        at.n_q = s->Hq; at.n_kv = s->Hkv; at.hd = s->hd; at.max_seq = s->max_seq; at.n_split = s->n_split;
        at.eps = 1e-6f; at.use_pdl = 0;
        at.n_items = B; at.qkv_item_stride = s->QKV; at.out_item_stride = Hq_hd;
        at.cache_item_stride = (long long)Hkv_hd * s->max_seq;
        B_TRY(s, b200_attn_decode(&at, st));
        proj(s, s->att, y->o, D, Hq_hd, x2, x);                               /* + residual */
        B_TRY(s, b200_rms_norm_rows_h(x2, y->g_post, s->ln, s->xh, B, D, 1e-6f, st));
        proj(s, NULL, y->gu, 2 * s->IS, D, s->gu, NULL);
        B_TRY(s, b200_silu_mul_rows_h(s->gu, B, s->IS, NULL, s->xh, st));
        proj(s, NULL, y->down, D, s->IS, x, x2);                              /* + residual */
    }
    B_TRY(s, b200_rms_norm_rows_h(x, s->g_final, s->ln, s->xh, B, D, 1e-6f, st));
    proj(s, NULL, s->lm_head, s->V, D, s->logits, NULL);
    B_TRY(s, b200_argmax_rows(s->logits, B, s->V, s->d_tok, s->d_hist, s->hist_cap, s->d_ctl, s->d_done, st));
}

static int ensure_graph(BState *s)
{
    if (s->graph) return 0;
    /* One eager pass first: kernels set their attributes and look up their symbols on first use, which must
     * not happen inside a capture. Its side effects (position, tokens, cache row 0) are reset by the caller. */
    cudaMemsetAsync(s->d_tok, 0, (size_t)s->B * 4, g_rt.stream);
    enqueue_step(s);
    if (s->err || cudaStreamSynchronize(g_rt.stream) != cudaSuccess) {
        fprintf(stderr, "[BatchGen] the first decode step failed\n");
        return -1;
    }
    cudaGraph_t g = NULL;
    CU_TRY(cudaStreamBeginCapture(g_rt.stream, cudaStreamCaptureModeThreadLocal), return -1);
    const unsigned long long before = b200_launch_count(0);
    enqueue_step(s);
    s->kernels_per_step = (int)(b200_launch_count(0) - before);
    cudaError_t e = cudaStreamEndCapture(g_rt.stream, &g);
    if (s->err || e != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        fprintf(stderr, "[BatchGen] CUDA graph capture failed\n");
        return -1;
    }
    e = cudaGraphInstantiate(&s->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { s->graph = NULL; cudaGetLastError(); return -1; }
    return 0;
}

static int is_eos(const BState *s, unsigned t)
{
    for (int i = 0; i < s->n_eos; ++i)
        if ((int)t == s->eos[i]) return 1;
    return 0;
}

void llmb200_batch_set_eos(BState *s, const int *eos, int n)
{
    if (!s) return;
    s->n_eos = n < 0 ? 0 : n > 4 ? 4 : n;
    for (int i = 0; i < s->n_eos; ++i) s->eos[i] = eos[i];
}

/* prompts [B][prompt_len] (every sequence its own prompt of the same length), output [B][max_gen_len].
 * Returns the number of steps generated (every sequence gets that many tokens), 0 on error. */
int llmb200_batch_generate(BState *s, const uint32_t *prompts, int prompt_len, uint32_t *output_tokens, int max_gen_len)
{
    if (!s || !s->finished || !prompts || !output_tokens || prompt_len < 1 || max_gen_len < 1) return 0;
    if (max_gen_len > s->hist_cap) max_gen_len = s->hist_cap;
    if (prompt_len > s->max_seq) {               /* as inference_generate: refused, not truncated (the row stride is prompt_len) */
        fprintf(stderr, "[BatchGen] prompt of %d tokens exceeds the KV cache (%d)\n", prompt_len, s->max_seq);
        return 0;
    }
    if (ensure_graph(s) != 0) return 0;
    const int B = s->B;
    cudaStream_t st = g_rt.stream;
    struct timespec t0, t1;
    fprintf(stderr, "[BatchGen] Prefilling %d tokens...\n", prompt_len);
    clock_gettime(CLOCK_MONOTONIC, &t0);
    s->h_ctl[0] = 0; s->h_ctl[1] = 0; s->h_ctl[2] = 0; s->h_ctl[3] = 0;
    CU_TRY(cudaMemcpyAsync(s->d_ctl, s->h_ctl, 16, cudaMemcpyHostToDevice, st), return 0);
    CU_TRY(cudaStreamSynchronize(st), return 0);
    for (int i = 0; i < prompt_len; ++i) {
        for (int b = 0; b < B; ++b) s->h_tok[b] = prompts[(size_t)b * prompt_len + i];
        CU_TRY(cudaMemcpyAsync(s->d_tok, s->h_tok, (size_t)B * 4, cudaMemcpyHostToDevice, st), return 0);
        if (i == prompt_len - 1) {               /* the last prompt position yields the first generated token */
            s->h_ctl[3] = 1;
            CU_TRY(cudaMemcpyAsync(s->d_ctl + 2, s->h_ctl + 3, 4, cudaMemcpyHostToDevice, st), return 0);
        }
        CU_TRY(cudaGraphLaunch(s->graph, st), return 0);
        CU_TRY(cudaStreamSynchronize(st), return 0);     /* h_tok is reused by the next position */
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    double ms = (t1.tv_sec - t0.tv_sec) * 1000.0 + (t1.tv_nsec - t0.tv_nsec) / 1e6;
    fprintf(stderr, "[BatchGen] Prefill: %.0f ms (%.1f tok/s)\n", ms, prompt_len * 1000.0 / ms);
    fprintf(stderr, "[BatchGen] Decoding (batch=%d)...\n", B);
    clock_gettime(CLOCK_MONOTONIC, &t0);
    int n_gen = 1, cur = prompt_len;
    unsigned *active = calloc(B, sizeof(unsigned));
    for (int b = 0; b < B; ++b) active[b] = 1;
    /* tokens of the previous step decide whether another step runs (as the reference's loop, :940-950) */
    CU_TRY(cudaMemcpy(s->h_tok, s->d_hist, (size_t)B * 4, cudaMemcpyDeviceToHost), { free(active); return 0; });
    while (n_gen < max_gen_len && cur < s->max_seq) {
        int any = 0;
        for (int b = 0; b < B; ++b) {
            if (active[b] && is_eos(s, s->h_tok[(size_t)(n_gen - 1) * B + b])) active[b] = 0;
            any |= (int)active[b];
        }
        if (!any) break;
        CU_TRY(cudaGraphLaunch(s->graph, st), { free(active); return 0; });
        CU_TRY(cudaMemcpyAsync(s->h_tok + (size_t)n_gen * B, s->d_hist + (size_t)n_gen * B, (size_t)B * 4,
                               cudaMemcpyDeviceToHost, st), { free(active); return 0; });
        CU_TRY(cudaStreamSynchronize(st), { free(active); return 0; });
        ++n_gen;
        ++cur;
    }
    free(active);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    ms = (t1.tv_sec - t0.tv_sec) * 1000.0 + (t1.tv_nsec - t0.tv_nsec) / 1e6;
    s->last_decode_ms = ms;
    s->last_steps = n_gen - 1;
    if (n_gen > 1) {
        fprintf(stderr, "[BatchGen] Decode: %d steps x %d batch = %d tokens in %.0f ms\n", n_gen - 1, B, (n_gen - 1) * B, ms);
        fprintf(stderr, "[BatchGen]   Throughput: %.1f tok/s\n", (n_gen - 1) * B * 1000.0 / ms);
        fprintf(stderr, "[BatchGen]   Latency: %.2f ms/step\n", ms / (n_gen - 1));
    }
    for (int b = 0; b < B; ++b)
        for (int g = 0; g < n_gen; ++g) output_tokens[(size_t)b * max_gen_len + g] = s->h_tok[(size_t)g * B + b];
    return s->err ? 0 : n_gen;
}

double llmb200_batch_last_decode_ms(BState *s, int *n_steps)
{
    if (!s) return -1.0;
    if (n_steps) *n_steps = s->last_steps;
    return s->last_decode_ms;
}

int llmb200_batch_graph_kernels(BState *s) { return s ? s->kernels_per_step : 0; }

const float *llmb200_batch_logits(BState *s, float *dst, size_t cap)
{
    if (!s || !dst || cap < (size_t)s->B * s->V) return NULL;
    if (g_rt.refs > 0) cudaStreamSynchronize(g_rt.stream);
    if (cudaMemcpy(dst, s->logits, (size_t)s->B * s->V * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return NULL;
    return dst;
}

/* Replaces qwen3_generate_fast_batch (src/nn/fast_inference.c:895-985): every sequence starts from the same
 * prompt; output_tokens is [batch_size][max_gen_len]; returns the number of tokens generated per sequence. */
int qwen3_generate_fast_batch(llmb200_qwen3_model *m, const uint32_t *prompt_tokens, int prompt_len,
                              uint32_t *output_tokens, int max_gen_len, int max_seq_len, int batch_size)
{
    if (!m || !prompt_tokens || !output_tokens || prompt_len < 1 || max_gen_len < 1) return 0;
    llmb200_config cfg = { MODEL_QWEN3, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                           m->vocab_size, m->n_layers, max_seq_len, 1 };
    BState *s = llmb200_batch_begin(&cfg, batch_size, max_gen_len);
    if (!s) { fprintf(stderr, "[BatchGen] state creation failed\n"); return 0; }
    const int Hq_hd = s->Hq * s->hd, Hkv_hd = s->Hkv * s->hd;
    for (int i = 0; i < s->L; ++i) {
        llmb200_qwen3_block *b = m->blocks[i];
        LayerWeightRef r;
        memset(&r, 0, sizeof(r));
        r.q_proj = (WeightRef){ b->attn->q_proj->weight->data, Hq_hd, s->D };
        r.k_proj = (WeightRef){ b->attn->k_proj->weight->data, Hkv_hd, s->D };
        r.v_proj = (WeightRef){ b->attn->v_proj->weight->data, Hkv_hd, s->D };
        r.o_proj = (WeightRef){ b->attn->o_proj->weight->data, s->D, Hq_hd };
        r.gate_proj = (WeightRef){ b->gate_proj->weight->data, s->IS, s->D };
        r.up_proj = (WeightRef){ b->up_proj->weight->data, s->IS, s->D };
        r.down_proj = (WeightRef){ b->down_proj->weight->data, s->D, s->IS };
        r.input_norm_g = b->input_norm->gamma->data;
        r.post_attn_norm_g = b->post_attn_norm->gamma->data;
        r.q_norm_g = b->attn->q_norm->gamma->data;
        r.k_norm_g = b->attn->k_norm->gamma->data;
        r.d_model = s->D; r.head_dim = s->hd;
        if (llmb200_batch_load_layer(s, i, &r, m->rope_theta) != 0) { llmb200_batch_free(s); return 0; }
    }
    if (llmb200_batch_finish(s, m->lm_head->weight->data, m->final_norm->gamma->data, m->token_emb->weight->data) != 0) {
        llmb200_batch_free(s);
        return 0;
    }
    uint32_t *rep = malloc((size_t)batch_size * prompt_len * sizeof(uint32_t));
    for (int b = 0; b < batch_size; ++b) memcpy(rep + (size_t)b * prompt_len, prompt_tokens, (size_t)prompt_len * 4);
    const int n = llmb200_batch_generate(s, rep, prompt_len, output_tokens, max_gen_len);
    free(rep);
    llmb200_batch_free(s);
    return n;
}
