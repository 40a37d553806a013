/*
 * Seeded synthetic models for benchmarks and parity tests.
 *
 * No checkpoint is available offline, so benchmarks and tests run on random
 * weights of the named architectures. Values come from a counter-based
 * generator keyed by (seed, tensor id, element index): any sub-range of any
 * tensor can be produced independently (threads, tensor-parallel ranks, the
 * CPU oracle and the GPU harness all see the same numbers). The normal
 * deviates use Box-Muller with log/sin/cos written out in IEEE double
 * arithmetic (no libm, built with -ffp-contract=off), so the bits do not
 * depend on the C library or on the CPU the generator runs on.
 *
 * The structures built here use the layouts of llmb200_model_abi.h, i.e. the
 * reference's Qwen3Model / Gemma3Model, so the same object can be handed to
 * libllmb200 and to the reference's own CPU code.
 */
#include "../../include/llmb200_synth.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

static inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* natural log of x in (0, 1], basic double operations only */
static double det_log(double x)
{
    int e;
    double m = frexp(x, &e);                 /* exact: x = m * 2^e, m in [0.5, 1) */
    if (m < 0.70710678118654752440) { m *= 2.0; e -= 1; }
    const double t = (m - 1.0) / (m + 1.0), t2 = t * t;
    double s = 0.0;
    for (int k = 25; k >= 1; k -= 2) s = s * t2 + 1.0 / (double)k;   /* 2*atanh(t) series, |t| < 0.1716 */
    return 2.0 * t * s + (double)e * 0.69314718055994530942;
}

/* sin and cos of 2*pi*u for u = j / 2^24, basic double operations only */
static void det_sincos_2pi(uint32_t j24, double *sn, double *cs)
{
    const uint32_t oct = j24 >> 21;                       /* eighth of the circle */
    const double r = (double)(j24 & 0x1FFFFFu) * (1.0 / 2097152.0);   /* position inside it, [0,1) */
    const double x = r * 0.78539816339744830962, x2 = x * x;
    double s = 0.0, c = 0.0;
    for (int k = 19; k >= 3; k -= 2) s = (s + 1.0) * (-x2 / (double)(k * (k - 1)));
    s = (s + 1.0) * x;
    for (int k = 18; k >= 2; k -= 2) c = (c + 1.0) * (-x2 / (double)(k * (k - 1)));
    c = c + 1.0;
    const double h = 0.70710678118654752440;
    double so, co;
    switch (oct) {                                        /* angle = oct*pi/4 + x */
    case 0: so = s; co = c; break;
    case 1: so = h * (s + c); co = h * (c - s); break;
    case 2: so = c; co = -s; break;
    case 3: so = h * (c - s); co = -h * (c + s); break;
    case 4: so = -s; co = -c; break;
    case 5: so = -h * (s + c); co = h * (s - c); break;
    case 6: so = -c; co = s; break;
    default: so = h * (s - c); co = h * (c + s); break;
    }
    *sn = so; *cs = co;
}

static inline void normal_pair(uint64_t key, uint64_t pair, float std, float *z0, float *z1)
{
    const uint64_t h = mix64(key + pair * 0xD1342543DE82EF95ull);
    const double u1 = (double)((h >> 40) + 1) * (1.0 / 16777216.0);     /* (0, 1] */
    const uint32_t j = (uint32_t)(h >> 8) & 0xFFFFFFu;
    const double r = sqrt(-2.0 * det_log(u1));
    double sn, cs;
    det_sincos_2pi(j, &sn, &cs);
    *z0 = (float)(r * cs) * std;
    *z1 = (float)(r * sn) * std;
}

static uint64_t tensor_key(uint64_t seed, uint64_t tensor_id) { return mix64(seed ^ mix64(tensor_id + 0x51ull)); }

typedef struct { float *dst; size_t first, n; uint64_t key; float std, mean; } fill_job;

static void fill_range(const fill_job *j)
{
    size_t i = j->first, end = j->first + j->n;
    float *dst = j->dst - j->first;                       /* dst[i] addresses element i of the tensor */
    if (i < end && (i & 1)) {
        float a, b;
        normal_pair(j->key, i >> 1, j->std, &a, &b);
        dst[i] = b + j->mean;
        ++i;
    }
    for (; i + 1 < end; i += 2) {
        float a, b;
        normal_pair(j->key, i >> 1, j->std, &a, &b);
        dst[i] = a + j->mean; dst[i + 1] = b + j->mean;
    }
    if (i < end) {
        float a, b;
        normal_pair(j->key, i >> 1, j->std, &a, &b);
        dst[i] = a + j->mean;
    }
}

static void *fill_thread(void *arg) { fill_range((const fill_job *)arg); return NULL; }

void llmb200_synth_normal_range(float *dst, size_t first, size_t n, uint64_t seed, uint64_t tensor_id,
                                float mean, float std, int n_threads)
{
    if (!dst || n == 0) return;
    const uint64_t key = tensor_key(seed, tensor_id);
    if (n_threads < 1) n_threads = 1;
    if (n_threads > 64) n_threads = 64;
    if (n < 65536 || n_threads == 1) {
        fill_job j = {dst, first, n, key, std, mean};
        fill_range(&j);
        return;
    }
    pthread_t th[64];
    fill_job jobs[64];
    const size_t per = ((n / (size_t)n_threads) + 1) & ~(size_t)1;    /* even, so pairs are not split */
    int started = 0;
    for (int t = 0; t < n_threads; ++t) {
        size_t lo = (size_t)t * per;
        if (lo >= n) break;
        size_t len = (lo + per > n) ? n - lo : per;
        /* keep `first + lo` on the parity of `first` so that pair boundaries line up */
        jobs[t] = (fill_job){dst + lo, first + lo, len, key, std, mean};
        if (pthread_create(&th[t], NULL, fill_thread, &jobs[t]) != 0) { fill_range(&jobs[t]); th[t] = 0; }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t) if (th[t]) pthread_join(th[t], NULL);
}

void llmb200_synth_normal(float *dst, size_t n, uint64_t seed, uint64_t tensor_id, float mean, float std, int n_threads)
{
    llmb200_synth_normal_range(dst, 0, n, seed, tensor_id, mean, std, n_threads);
}

void llmb200_synth_tokens(uint32_t *dst, size_t n, uint64_t seed, uint32_t vocab)
{
    const uint64_t key = tensor_key(seed, 0x70CE45ull);
    for (size_t i = 0; i < n; ++i) dst[i] = (uint32_t)(mix64(key + i * 0xD1342543DE82EF95ull) % vocab);
}

/* ---------------------------------------------------------------- structs */

static llmb200_tensor *tensor_new(int d0, int d1)
{
    llmb200_tensor *t = calloc(1, sizeof(*t));
    if (!t) return NULL;
    t->ndim = d1 > 0 ? 2 : 1;
    t->shape[0] = d0; t->shape[1] = d1 > 0 ? d1 : 0;
    t->stride[0] = d1 > 0 ? d1 : 1; t->stride[1] = d1 > 0 ? 1 : 0;
    t->size = (size_t)d0 * (size_t)(d1 > 0 ? d1 : 1);
    t->bytes = t->size * sizeof(float);
    t->dtype = LLMB200_F32;
    t->owns_data = 1;
    t->data = malloc(t->bytes ? t->bytes : 4);
    if (!t->data) { free(t); return NULL; }
    return t;
}

static void tensor_del(llmb200_tensor *t) { if (t) { free(t->data); free(t); } }

static llmb200_linear *linear_new(int in_f, int out_f, uint64_t seed, uint64_t id, float std, int nt)
{
    llmb200_linear *l = calloc(1, sizeof(*l));
    if (!l) return NULL;
    l->in_features = in_f; l->out_features = out_f;
    l->weight = tensor_new(out_f, in_f);
    if (!l->weight) { free(l); return NULL; }
    llmb200_synth_normal(l->weight->data, l->weight->size, seed, id, 0.0f, std, nt);
    return l;
}

static void linear_del(llmb200_linear *l) { if (l) { tensor_del(l->weight); free(l); } }

static llmb200_rmsnorm *norm_new(int dim, uint64_t seed, uint64_t id, float jitter)
{
    llmb200_rmsnorm *n = calloc(1, sizeof(*n));
    if (!n) return NULL;
    n->dim = dim; n->eps = 1e-6f;
    n->gamma = tensor_new(dim, 0);
    if (!n->gamma) { free(n); return NULL; }
    if (jitter > 0.0f) llmb200_synth_normal(n->gamma->data, (size_t)dim, seed, id, 1.0f, jitter, 1);
    else for (int i = 0; i < dim; ++i) n->gamma->data[i] = 1.0f;
    return n;
}

static void norm_del(llmb200_rmsnorm *n) { if (n) { tensor_del(n->gamma); free(n); } }

static llmb200_gqa *gqa_new(const llmb200_synth_spec *sp, int layer, float theta, int nt)
{
    llmb200_gqa *a = calloc(1, sizeof(*a));
    if (!a) return NULL;
    const uint64_t b = (uint64_t)layer * 16;
    a->d_model = sp->d_model; a->n_q_heads = sp->n_q_heads; a->n_kv_heads = sp->n_kv_heads; a->head_dim = sp->head_dim;
    a->scale = 1.0f / sqrtf((float)sp->head_dim);
    a->rope_theta = theta;
    a->q_proj = linear_new(sp->d_model, sp->n_q_heads * sp->head_dim, sp->seed, b + 0, sp->weight_std, nt);
    a->k_proj = linear_new(sp->d_model, sp->n_kv_heads * sp->head_dim, sp->seed, b + 1, sp->weight_std, nt);
    a->v_proj = linear_new(sp->d_model, sp->n_kv_heads * sp->head_dim, sp->seed, b + 2, sp->weight_std, nt);
    a->o_proj = linear_new(sp->n_q_heads * sp->head_dim, sp->d_model, sp->seed, b + 3, sp->weight_std, nt);
    a->q_norm = norm_new(sp->head_dim, sp->seed, b + 7, sp->gamma_jitter);
    a->k_norm = norm_new(sp->head_dim, sp->seed, b + 8, sp->gamma_jitter);
    return a;
}

static void gqa_del(llmb200_gqa *a)
{
    if (!a) return;
    linear_del(a->q_proj); linear_del(a->k_proj); linear_del(a->v_proj); linear_del(a->o_proj);
    norm_del(a->q_norm); norm_del(a->k_norm);
    free(a);
}

#define ID_EMB   (1ull << 20)
#define ID_LM    ((1ull << 20) + 1)
#define ID_FINAL ((1ull << 20) + 2)

llmb200_qwen3_model *llmb200_synth_qwen3(const llmb200_synth_spec *sp, int nt)
{
    if (!sp) return NULL;
    llmb200_qwen3_model *m = calloc(1, sizeof(*m));
    if (!m) return NULL;
    m->n_layers = sp->n_layers; m->d_model = sp->d_model; m->vocab_size = sp->vocab_size;
    m->n_q_heads = sp->n_q_heads; m->n_kv_heads = sp->n_kv_heads; m->head_dim = sp->head_dim;
    m->intermediate_size = sp->intermediate_size; m->rope_theta = sp->rope_theta;
    m->token_emb = calloc(1, sizeof(llmb200_embedding));
    m->token_emb->vocab_size = sp->vocab_size; m->token_emb->dim = sp->d_model;
    m->token_emb->weight = tensor_new(sp->vocab_size, sp->d_model);
    llmb200_synth_normal(m->token_emb->weight->data, m->token_emb->weight->size, sp->seed, ID_EMB, 0.0f, sp->weight_std, nt);
    m->blocks = calloc((size_t)sp->n_layers, sizeof(*m->blocks));
    for (int i = 0; i < sp->n_layers; ++i) {
        llmb200_qwen3_block *b = calloc(1, sizeof(*b));
        const uint64_t id = (uint64_t)i * 16;
        b->d_model = sp->d_model;
        b->input_norm = norm_new(sp->d_model, sp->seed, id + 9, sp->gamma_jitter);
        b->attn = gqa_new(sp, i, sp->rope_theta, nt);
        b->post_attn_norm = norm_new(sp->d_model, sp->seed, id + 10, sp->gamma_jitter);
        b->gate_proj = linear_new(sp->d_model, sp->intermediate_size, sp->seed, id + 4, sp->weight_std, nt);
        b->up_proj = linear_new(sp->d_model, sp->intermediate_size, sp->seed, id + 5, sp->weight_std, nt);
        b->down_proj = linear_new(sp->intermediate_size, sp->d_model, sp->seed, id + 6, sp->weight_std, nt);
        m->blocks[i] = b;
    }
    m->final_norm = norm_new(sp->d_model, sp->seed, ID_FINAL, sp->gamma_jitter);
    m->lm_head = linear_new(sp->d_model, sp->vocab_size, sp->seed, ID_LM, sp->weight_std, nt);
    return m;
}

void llmb200_synth_free_qwen3(llmb200_qwen3_model *m)
{
    if (!m) return;
    if (m->token_emb) { tensor_del(m->token_emb->weight); free(m->token_emb); }
    for (int i = 0; m->blocks && i < m->n_layers; ++i) {
        llmb200_qwen3_block *b = m->blocks[i];
        if (!b) continue;
        norm_del(b->input_norm); gqa_del(b->attn); norm_del(b->post_attn_norm);
        linear_del(b->gate_proj); linear_del(b->up_proj); linear_del(b->down_proj);
        free(b);
    }
    free(m->blocks);
    norm_del(m->final_norm); linear_del(m->lm_head);
    free(m);
}

llmb200_gemma3_model *llmb200_synth_gemma3(const llmb200_synth_spec *sp, int nt)
{
    if (!sp) return NULL;
    llmb200_gemma3_model *m = calloc(1, sizeof(*m));
    if (!m) return NULL;
    m->n_layers = sp->n_layers; m->d_model = sp->d_model; m->vocab_size = sp->vocab_size;
    m->n_q_heads = sp->n_q_heads; m->n_kv_heads = sp->n_kv_heads; m->head_dim = sp->head_dim;
    m->intermediate_size = sp->intermediate_size; m->sliding_window = sp->sliding_window;
    m->local_rope_theta = sp->local_rope_theta; m->global_rope_theta = sp->rope_theta;
    m->token_emb = calloc(1, sizeof(llmb200_embedding));
    m->token_emb->vocab_size = sp->vocab_size; m->token_emb->dim = sp->d_model;
    m->token_emb->weight = tensor_new(sp->vocab_size, sp->d_model);
    llmb200_synth_normal(m->token_emb->weight->data, m->token_emb->weight->size, sp->seed, ID_EMB, 0.0f, sp->weight_std, nt);
    m->blocks = calloc((size_t)sp->n_layers, sizeof(*m->blocks));
    for (int i = 0; i < sp->n_layers; ++i) {
        llmb200_gemma3_block *b = calloc(1, sizeof(*b));
        const uint64_t id = (uint64_t)i * 16;
        b->d_model = sp->d_model;
        b->is_sliding = (i % 6) != 0;                      /* src/nn/gemma3.c:50-52 */
        b->input_norm = norm_new(sp->d_model, sp->seed, id + 9, sp->gamma_jitter);
        b->attn = gqa_new(sp, i, b->is_sliding ? sp->local_rope_theta : sp->rope_theta, nt);
        b->post_attn_norm = norm_new(sp->d_model, sp->seed, id + 10, sp->gamma_jitter);
        b->pre_ff_norm = norm_new(sp->d_model, sp->seed, id + 11, sp->gamma_jitter);
        b->gate_proj = linear_new(sp->d_model, sp->intermediate_size, sp->seed, id + 4, sp->weight_std, nt);
        b->up_proj = linear_new(sp->d_model, sp->intermediate_size, sp->seed, id + 5, sp->weight_std, nt);
        b->down_proj = linear_new(sp->intermediate_size, sp->d_model, sp->seed, id + 6, sp->weight_std, nt);
        b->post_ff_norm = norm_new(sp->d_model, sp->seed, id + 12, sp->gamma_jitter);
        m->blocks[i] = b;
    }
    m->final_norm = norm_new(sp->d_model, sp->seed, ID_FINAL, sp->gamma_jitter);
    return m;
}

void llmb200_synth_free_gemma3(llmb200_gemma3_model *m)
{
    if (!m) return;
    if (m->token_emb) { tensor_del(m->token_emb->weight); free(m->token_emb); }
    for (int i = 0; m->blocks && i < m->n_layers; ++i) {
        llmb200_gemma3_block *b = m->blocks[i];
        if (!b) continue;
        norm_del(b->input_norm); gqa_del(b->attn); norm_del(b->post_attn_norm); norm_del(b->pre_ff_norm);
        linear_del(b->gate_proj); linear_del(b->up_proj); linear_del(b->down_proj); norm_del(b->post_ff_norm);
        free(b);
    }
    free(m->blocks);
    norm_del(m->final_norm);
    free(m);
}

/* Tensor ids, for callers that generate single tensors (streaming construction). */
uint64_t llmb200_synth_tensor_id(int layer, int which)
{
    if (which == LLMB200_T_EMB) return ID_EMB;
    if (which == LLMB200_T_LM_HEAD) return ID_LM;
    if (which == LLMB200_T_FINAL_NORM) return ID_FINAL;
    return (uint64_t)layer * 16 + (uint64_t)which;
}

/* sizeof/offsetof table of the boundary structures as this library declares
 * them; tests compare it with the same table computed from the caller's own
 * headers. */
#include <stddef.h>
#include "../../include/llmb200_wmat.h"
int llmb200_abi_layout(size_t *out, int cap)
{
    typedef llmb200_tensor T; typedef llmb200_linear Li; typedef llmb200_embedding Em; typedef llmb200_rmsnorm Rn;
    typedef llmb200_gqa Gq; typedef llmb200_lora_linear Lo; typedef llmb200_qwen3_block Qb; typedef llmb200_qwen3_model Qm;
    typedef llmb200_gemma3_block Gb; typedef llmb200_gemma3_model Gm;
    size_t v[] = {
        sizeof(T), offsetof(T, data), offsetof(T, ndim), offsetof(T, shape), offsetof(T, stride),
        offsetof(T, size), offsetof(T, bytes), offsetof(T, dtype), offsetof(T, device_buf),
        offsetof(T, grad), offsetof(T, requires_grad), offsetof(T, owns_data),
        sizeof(Li), offsetof(Li, weight), offsetof(Li, in_features), offsetof(Li, out_features),
        sizeof(Em), offsetof(Em, weight), offsetof(Em, dim),
        sizeof(Rn), offsetof(Rn, gamma), offsetof(Rn, dim), offsetof(Rn, eps),
        sizeof(Gq), offsetof(Gq, rope_theta), offsetof(Gq, q_proj), offsetof(Gq, o_proj), offsetof(Gq, q_norm), offsetof(Gq, k_norm),
        sizeof(Lo), offsetof(Lo, lora_A), offsetof(Lo, lora_B), offsetof(Lo, rank), offsetof(Lo, scaling), offsetof(Lo, enabled),
        sizeof(Qb), offsetof(Qb, attn), offsetof(Qb, post_attn_norm), offsetof(Qb, down_proj),
        sizeof(Qm), offsetof(Qm, blocks), offsetof(Qm, lm_head), offsetof(Qm, n_layers),
        offsetof(Qm, intermediate_size), offsetof(Qm, rope_theta), offsetof(Qm, q_loras), offsetof(Qm, v_loras),
        sizeof(Gb), offsetof(Gb, pre_ff_norm), offsetof(Gb, post_ff_norm), offsetof(Gb, is_sliding),
        sizeof(Gm), offsetof(Gm, final_norm), offsetof(Gm, n_layers), offsetof(Gm, sliding_window),
        offsetof(Gm, local_rope_theta), offsetof(Gm, global_rope_theta), offsetof(Gm, q_loras),
        sizeof(WMat), offsetof(WMat, rows), offsetof(WMat, nb),
        sizeof(LayerW), offsetof(LayerW, down_proj), offsetof(LayerW, input_norm_g), offsetof(LayerW, k_norm_g),
        sizeof(WeightRef), sizeof(LayerWeightRef), offsetof(LayerWeightRef, input_norm_g), offsetof(LayerWeightRef, d_model),
        offsetof(LayerWeightRef, head_dim),
    };
    int n = (int)(sizeof(v) / sizeof(v[0]));
    for (int i = 0; i < n && i < cap; ++i) out[i] = v[i];
    return n;
}
