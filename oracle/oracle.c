/*
 * TEST INFRASTRUCTURE -- not part of the product (see oracle.h).
 *
 * CPU restatement of the decode path of llm.metal in plain C. Every function
 * names the reference lines it follows. Arithmetic is the reference CPU
 * path's: fp32, sequential accumulation, libm sinf/cosf/powf/expf/tanhf.
 */
#include "oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* ---- binary16 ---------------------------------------------------------- */

/* src/nn/wmat.c:29,69-71 rely on the compiler's (__fp16) cast = IEEE RNE. */
static uint16_t f32_to_f16_bits(float f)
{
    _Float16 h = (_Float16)f;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

/* src/data/gguf.c:232-244 */
float oracle_f16_to_f32(uint16_t h)
{
    const uint32_t sign = (h >> 15) & 1, ex = (h >> 10) & 0x1F, mant = h & 0x3FF;
    float v;
    if (ex == 0) v = ldexpf((float)mant, -24);
    else if (ex == 31) v = mant == 0 ? INFINITY : NAN;
    else v = ldexpf((float)(mant + 1024), (int)ex - 25);
    return sign ? -v : v;
}

void oracle_f16_bits(const float *src, size_t n, uint16_t *dst)
{
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_f16_bits(src[i]);
}

/* ---- Q8_0 ---------------------------------------------------------------- */

/* src/nn/wmat.c:19-41 */
void oracle_q8_quantize(const float *src, int rows, int cols, uint8_t *blocks)
{
    const int nb = cols / 32;
    for (int r = 0; r < rows; ++r) {
        for (int b = 0; b < nb; ++b) {
            const float *sp = src + (size_t)r * cols + (size_t)b * 32;
            uint8_t *blk = blocks + ((size_t)r * nb + b) * 34;
            float amax = 0.0f;
            for (int j = 0; j < 32; ++j) { float a = fabsf(sp[j]); if (a > amax) amax = a; }
            const float scale = amax / 127.0f;
            const uint16_t d = f32_to_f16_bits(scale);
            memcpy(blk, &d, 2);
            int8_t *qs = (int8_t *)(blk + 2);
            if (scale != 0.0f) {
                const float inv = 1.0f / scale;
                for (int j = 0; j < 32; ++j) {
                    int v = (int)roundf(sp[j] * inv);
                    qs[j] = (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
                }
            } else {
                memset(qs, 0, 32);
            }
        }
    }
}

/* src/data/gguf.c:225-253 */
void oracle_q8_dequantize(const uint8_t *blocks, size_t n_blocks, float *dst)
{
    for (size_t b = 0; b < n_blocks; ++b) {
        uint16_t d;
        memcpy(&d, blocks + b * 34, 2);
        const float scale = oracle_f16_to_f32(d);
        const int8_t *q = (const int8_t *)(blocks + b * 34 + 2);
        for (int i = 0; i < 32; ++i) dst[b * 32 + i] = (float)q[i] * scale;
    }
}

/* shaders/q8_kernels.metal:10-42: per block, 32 lane products are summed and
 * the block sum is scaled; block results accumulate in fp32. */
void oracle_q8_matvec(const uint8_t *blocks, const float *x, float *y, int rows, int nb)
{
    for (int r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const uint8_t *blk = blocks + ((size_t)r * nb + b) * 34;
            uint16_t d;
            memcpy(&d, blk, 2);
            const int8_t *q = (const int8_t *)(blk + 2);
            float bs = 0.0f;
            for (int l = 0; l < 32; ++l) bs += (float)q[l] * x[b * 32 + l];
            sum += oracle_f16_to_f32(d) * bs;
        }
        y[r] = sum;
    }
}

/* shaders/q8_kernels.metal:97-127 */
void oracle_f16_matvec(const uint16_t *w, const float *x, float *y, int rows, int cols)
{
    for (int r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (int c = 0; c < cols; ++c) sum += oracle_f16_to_f32(w[(size_t)r * cols + c]) * x[c];
        y[r] = sum;
    }
}

/* src/nn/layers.c:136-150. Rows are independent, so splitting them over
 * threads (ORACLE_THREADS, default 1) changes no sum. */
typedef struct { const float *w, *x; float *y; int r0, r1, cols; } lin_job;

static void *lin_rows(void *arg)
{
    const lin_job *j = arg;
    for (int r = j->r0; r < j->r1; ++r) {
        const float *wr = j->w + (size_t)r * j->cols;
        float sum = 0.0f;
        for (int k = 0; k < j->cols; ++k) sum += j->x[k] * wr[k];
        j->y[r] = sum;
    }
    return NULL;
}

static int oracle_threads(void)
{
    static int n = 0;
    if (!n) {
        const char *e = getenv("ORACLE_THREADS");
        n = e ? atoi(e) : 1;
        if (n < 1) n = 1;
        if (n > 64) n = 64;
    }
    return n;
}

void oracle_linear(const float *w, const float *x, float *y, int rows, int cols)
{
    int nt = oracle_threads();
    if ((size_t)rows * cols < 262144 || nt == 1 || rows < nt) {
        lin_job j = {w, x, y, 0, rows, cols};
        lin_rows(&j);
        return;
    }
    pthread_t th[64];
    lin_job jobs[64];
    for (int t = 0; t < nt; ++t) {
        jobs[t] = (lin_job){w, x, y, (int)((long long)rows * t / nt), (int)((long long)rows * (t + 1) / nt), cols};
        if (pthread_create(&th[t], NULL, lin_rows, &jobs[t]) != 0) { lin_rows(&jobs[t]); th[t] = 0; }
    }
    for (int t = 0; t < nt; ++t) if (th[t]) pthread_join(th[t], NULL);
}

/* src/nn/layers.c:362-377 */
void oracle_rms_norm(const float *x, const float *gamma, float *y, int dim, float eps)
{
    float ss = 0.0f;
    for (int i = 0; i < dim; ++i) ss += x[i] * x[i];
    const float inv_rms = 1.0f / sqrtf(ss / dim + eps);
    for (int i = 0; i < dim; ++i) y[i] = gamma[i] * x[i] * inv_rms;
}

/* ---- model ------------------------------------------------------------- */

typedef struct {
    float *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    float *g_input, *g_post_attn, *g_pre_ff, *g_post_ff, *g_qn, *g_kn;
    float theta;
    float *kc, *vc;              /* [Hkv][max_seq][hd] */
} olayer;

struct oracle_model {
    int gemma, D, Hq, Hkv, hd, IS, V, L, max_seq, kv_f16;
    olayer *layers;
    float *lm, *g_final;
    const float *emb;            /* borrowed from the source model, like the reference */
    float *x, *x2, *ln, *q, *k, *v, *att, *gate, *up, *ff, *tmp, *scores;
};

static float *convert(const float *src, int rows, int cols, int use_fp16)
{
    const size_t n = (size_t)rows * cols;
    float *dst = malloc(n * sizeof(float));
    if (use_fp16) {
        for (size_t i = 0; i < n; ++i) dst[i] = oracle_f16_to_f32(f32_to_f16_bits(src[i]));
    } else {
        uint8_t *blk = malloc(n / 32 * 34);
        oracle_q8_quantize(src, rows, cols, blk);
        oracle_q8_dequantize(blk, n / 32, dst);
        free(blk);
    }
    return dst;
}

static float *dup(const float *src, size_t n)
{
    float *d = malloc(n * sizeof(float));
    memcpy(d, src, n * sizeof(float));
    return d;
}

static oracle_model *model_alloc(int gemma, int D, int Hq, int Hkv, int hd, int IS, int V, int L, int max_seq)
{
    oracle_model *o = calloc(1, sizeof(*o));
    o->gemma = gemma; o->D = D; o->Hq = Hq; o->Hkv = Hkv; o->hd = hd; o->IS = IS; o->V = V; o->L = L; o->max_seq = max_seq;
    o->layers = calloc((size_t)L, sizeof(olayer));
    o->x = malloc(D * sizeof(float)); o->x2 = malloc(D * sizeof(float)); o->ln = malloc(D * sizeof(float));
    o->tmp = malloc(D * sizeof(float));
    o->q = malloc((size_t)Hq * hd * sizeof(float)); o->k = malloc((size_t)Hkv * hd * sizeof(float));
    o->v = malloc((size_t)Hkv * hd * sizeof(float)); o->att = malloc((size_t)Hq * hd * sizeof(float));
    o->gate = malloc(IS * sizeof(float)); o->up = malloc(IS * sizeof(float)); o->ff = malloc(D * sizeof(float));
    o->scores = malloc((size_t)max_seq * sizeof(float));
    return o;
}

static void layer_common(oracle_model *o, olayer *ly, const llmb200_gqa *a, const llmb200_linear *g, const llmb200_linear *u,
                         const llmb200_linear *d, int f16)
{
    const int D = o->D, hd = o->hd;
    ly->wq = convert(a->q_proj->weight->data, o->Hq * hd, D, f16);
    ly->wk = convert(a->k_proj->weight->data, o->Hkv * hd, D, f16);
    ly->wv = convert(a->v_proj->weight->data, o->Hkv * hd, D, f16);
    ly->wo = convert(a->o_proj->weight->data, D, o->Hq * hd, f16);
    ly->wg = convert(g->weight->data, o->IS, D, f16);
    ly->wu = convert(u->weight->data, o->IS, D, f16);
    ly->wd = convert(d->weight->data, D, o->IS, f16);
    ly->g_qn = a->q_norm ? dup(a->q_norm->gamma->data, hd) : NULL;
    ly->g_kn = a->k_norm ? dup(a->k_norm->gamma->data, hd) : NULL;
    ly->theta = a->rope_theta;
    ly->kc = calloc((size_t)o->Hkv * o->max_seq * hd, sizeof(float));
    ly->vc = calloc((size_t)o->Hkv * o->max_seq * hd, sizeof(float));
}

oracle_model *oracle_model_qwen3(const llmb200_qwen3_model *m, int use_fp16, int max_seq)
{
    oracle_model *o = model_alloc(0, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                                  m->vocab_size, m->n_layers, max_seq);
    for (int i = 0; i < o->L; ++i) {
        const llmb200_qwen3_block *b = m->blocks[i];
        olayer *ly = &o->layers[i];
        layer_common(o, ly, b->attn, b->gate_proj, b->up_proj, b->down_proj, use_fp16);
        ly->g_input = dup(b->input_norm->gamma->data, o->D);
        ly->g_post_attn = dup(b->post_attn_norm->gamma->data, o->D);
    }
    o->lm = convert(m->lm_head->weight->data, o->V, o->D, use_fp16);
    o->g_final = dup(m->final_norm->gamma->data, o->D);
    o->emb = m->token_emb->weight->data;          /* fp32, unconverted: src/nn/fast_inference.c:248 */
    return o;
}

oracle_model *oracle_model_gemma3(const llmb200_gemma3_model *m, int use_fp16, int max_seq)
{
    oracle_model *o = model_alloc(1, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                                  m->vocab_size, m->n_layers, max_seq);
    for (int i = 0; i < o->L; ++i) {
        const llmb200_gemma3_block *b = m->blocks[i];
        olayer *ly = &o->layers[i];
        layer_common(o, ly, b->attn, b->gate_proj, b->up_proj, b->down_proj, use_fp16);
        ly->g_input = dup(b->input_norm->gamma->data, o->D);
        ly->g_post_attn = dup(b->post_attn_norm->gamma->data, o->D);
        ly->g_pre_ff = dup(b->pre_ff_norm->gamma->data, o->D);
        ly->g_post_ff = dup(b->post_ff_norm->gamma->data, o->D);
        /* per-layer base: src/nn/fast_inference.c:301-303 */
        ly->theta = b->is_sliding ? m->local_rope_theta : m->global_rope_theta;
    }
    o->lm = convert(m->token_emb->weight->data, o->V, o->D, use_fp16);   /* tied: src/nn/fast_inference.c:307-313 */
    o->g_final = dup(m->final_norm->gamma->data, o->D);
    o->emb = m->token_emb->weight->data;
    return o;
}

void oracle_model_free(oracle_model *o)
{
    if (!o) return;
    for (int i = 0; i < o->L; ++i) {
        olayer *l = &o->layers[i];
        free(l->wq); free(l->wk); free(l->wv); free(l->wo); free(l->wg); free(l->wu); free(l->wd);
        free(l->g_input); free(l->g_post_attn); free(l->g_pre_ff); free(l->g_post_ff); free(l->g_qn); free(l->g_kn);
        free(l->kc); free(l->vc);
    }
    free(o->layers); free(o->lm); free(o->g_final);
    free(o->x); free(o->x2); free(o->ln); free(o->tmp); free(o->q); free(o->k); free(o->v); free(o->att);
    free(o->gate); free(o->up); free(o->ff); free(o->scores);
    free(o);
}

void oracle_model_set_kv_f16(oracle_model *m, int on) { m->kv_f16 = on ? 1 : 0; }

/* half-split rotation of one head: src/nn/attention.c:752-768 (= shaders/q8_kernels.metal:219-230) */
static void rope_head(float *h, int hd, int pos, float theta)
{
    const int half = hd / 2;
    for (int d = 0; d < half; ++d) {
        const float freq = 1.0f / powf(theta, (float)(2 * d) / (float)hd);
        const float angle = (float)pos * freq;
        const float c = cosf(angle), s = sinf(angle);
        const float x0 = h[d], x1 = h[d + half];
        h[d] = x0 * c - x1 * s;
        h[d + half] = x0 * s + x1 * c;
    }
}

/* src/nn/attention.c:660-856 for one new token (batch 1, n_new 1), without the output projection */
static void attention_cached(oracle_model *o, olayer *ly, int pos)
{
    const int Hq = o->Hq, Hkv = o->Hkv, hd = o->hd, ms = o->max_seq, group = Hq / Hkv;
    const float eps = 1e-6f, scale = 1.0f / sqrtf((float)hd);
    for (int h = 0; h < Hkv; ++h) {           /* store raw K/V, then norm and rotate K in the cache */
        float *kr = ly->kc + ((size_t)h * ms + pos) * hd, *vr = ly->vc + ((size_t)h * ms + pos) * hd;
        memcpy(kr, o->k + (size_t)h * hd, hd * sizeof(float));
        memcpy(vr, o->v + (size_t)h * hd, hd * sizeof(float));
        if (ly->g_kn) { oracle_rms_norm(kr, ly->g_kn, o->tmp, hd, eps); memcpy(kr, o->tmp, hd * sizeof(float)); }
        rope_head(kr, hd, pos, ly->theta);
        if (o->kv_f16)
            for (int d = 0; d < hd; ++d) {
                kr[d] = oracle_f16_to_f32(f32_to_f16_bits(kr[d]));
                vr[d] = oracle_f16_to_f32(f32_to_f16_bits(vr[d]));
            }
    }
    for (int h = 0; h < Hq; ++h) {
        float *qh = o->q + (size_t)h * hd;
        if (ly->g_qn) { oracle_rms_norm(qh, ly->g_qn, o->tmp, hd, eps); memcpy(qh, o->tmp, hd * sizeof(float)); }
        rope_head(qh, hd, pos, ly->theta);
    }
    const int n = pos + 1;
    for (int hq = 0; hq < Hq; ++hq) {
        const int hkv = hq / group;
        const float *qp = o->q + (size_t)hq * hd;
        const float *kp = ly->kc + (size_t)hkv * ms * hd, *vp = ly->vc + (size_t)hkv * ms * hd;
        float mx = -1e30f;
        for (int j = 0; j < n; ++j) {
            float sc = 0.0f;
            for (int d = 0; d < hd; ++d) sc += qp[d] * kp[(size_t)j * hd + d];
            sc *= scale;
            o->scores[j] = sc;
            if (sc > mx) mx = sc;
        }
        float sum = 0.0f;
        for (int j = 0; j < n; ++j) { o->scores[j] = expf(o->scores[j] - mx); sum += o->scores[j]; }
        const float inv = sum > 0 ? 1.0f / sum : 0.0f;
        float *out = o->att + (size_t)hq * hd;
        for (int d = 0; d < hd; ++d) {
            float val = 0.0f;
            for (int j = 0; j < n; ++j) val += o->scores[j] * inv * vp[(size_t)j * hd + d];
            out[d] = val;
        }
    }
}

/* src/nn/layers.c:558-580 (SiLU), :507-530 (tanh GELU), :615-633 (multiply) */
static void glu(oracle_model *o)
{
    for (int i = 0; i < o->IS; ++i) {
        const float g = o->gate[i];
        float a;
        if (o->gemma) {
            const float inner = 0.7978845608f * (g + 0.044715f * g * g * g);
            a = 0.5f * g * (1.0f + tanhf(inner));
        } else {
            const float sig = 1.0f / (1.0f + expf(-g));
            a = g * sig;
        }
        o->gate[i] = a * o->up[i];
    }
}

/* Op order of src/nn/fast_inference.c:376-467 */
void oracle_forward_token(oracle_model *o, int token, int pos, float *logits)
{
    const int D = o->D, hd = o->hd;
    const float eps = 1e-6f;
    memcpy(o->x, o->emb + (size_t)token * D, D * sizeof(float));
    if (o->gemma) { const float sc = sqrtf((float)D); for (int i = 0; i < D; ++i) o->x[i] *= sc; }
    for (int l = 0; l < o->L; ++l) {
        olayer *ly = &o->layers[l];
        oracle_rms_norm(o->x, ly->g_input, o->ln, D, eps);
        oracle_linear(ly->wq, o->ln, o->q, o->Hq * hd, D);
        oracle_linear(ly->wk, o->ln, o->k, o->Hkv * hd, D);
        oracle_linear(ly->wv, o->ln, o->v, o->Hkv * hd, D);
        attention_cached(o, ly, pos);
        oracle_linear(ly->wo, o->att, o->x2, D, o->Hq * hd);
        if (o->gemma) {
            oracle_rms_norm(o->x2, ly->g_post_attn, o->ln, D, eps);
            for (int i = 0; i < D; ++i) o->x[i] += o->ln[i];
        } else {
            for (int i = 0; i < D; ++i) o->x[i] += o->x2[i];
        }
        oracle_rms_norm(o->x, o->gemma ? ly->g_pre_ff : ly->g_post_attn, o->ln, D, eps);
        oracle_linear(ly->wg, o->ln, o->gate, o->IS, D);
        oracle_linear(ly->wu, o->ln, o->up, o->IS, D);
        glu(o);
        oracle_linear(ly->wd, o->gate, o->ff, D, o->IS);
        if (o->gemma) {
            oracle_rms_norm(o->ff, ly->g_post_ff, o->x2, D, eps);
            for (int i = 0; i < D; ++i) o->x[i] += o->x2[i];
        } else {
            for (int i = 0; i < D; ++i) o->x[i] += o->ff[i];
        }
    }
    if (logits) {
        oracle_rms_norm(o->x, o->g_final, o->ln, D, eps);
        oracle_linear(o->lm, o->ln, logits, o->V, D);
    }
}

/* src/nn/fast_inference.c:469-476 */
static int argmax_first(const float *v, int n)
{
    int best = 0;
    float bv = v[0];
    for (int i = 1; i < n; ++i) if (v[i] > bv) { bv = v[i]; best = i; }
    return best;
}

static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + t.tv_nsec * 1e-9; }

/* src/nn/fast_inference.c:614-675 */
int oracle_generate(oracle_model *o, const uint32_t *prompt, int P, uint32_t *out, int max_gen,
                    const int *eos, int n_eos, float *logits_out, double *seconds)
{
    const int V = o->V;
    float *lg = malloc((size_t)V * sizeof(float));
    double t0 = now_s();
    for (int i = 0; i < P; ++i) oracle_forward_token(o, (int)prompt[i], i, i == P - 1 ? lg : NULL);
    double t1 = now_s();
    int cur = P, next = argmax_first(lg, V), n = 1;
    if (logits_out) memcpy(logits_out, lg, (size_t)V * sizeof(float));
    out[0] = (uint32_t)next;
    for (int g = 1; g < max_gen && cur < o->max_seq; ++g) {
        int stop = 0;
        for (int e = 0; e < n_eos; ++e) if (next == eos[e]) { stop = 1; break; }
        if (stop) break;
        oracle_forward_token(o, next, cur, lg);
        cur++;
        if (logits_out) memcpy(logits_out + (size_t)n * V, lg, (size_t)V * sizeof(float));
        next = argmax_first(lg, V);
        out[n++] = (uint32_t)next;
    }
    double t2 = now_s();
    if (seconds) { seconds[0] = t1 - t0; seconds[1] = t2 - t1; }
    free(lg);
    return n;
}
