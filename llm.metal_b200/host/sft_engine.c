/*
 * LoRA-SFT engine of libllmb200 (host side, C).
 *
 * Stands in for src/nn/fast_sft.c (LoRA branch, Qwen3 block order): state
 * creation :171-278, forward_to_logits :616-752, sft_apply_ce_loss :754-760,
 * sft_backward_ex :766-982, clip_grad_norm / adamw_update / lora_update
 * :1045-1107, sft_train_step :1113-1157, accessors :1206-1285.
 *
 * Differences in structure, not in arithmetic:
 *  - S sequences of N tokens are one [S*N, .] activation matrix, so every
 *    frozen projection is ONE matrix product per layer and pass (the reference
 *    runs one sequence per step). Q/K/V and gate/up are fused row-wise.
 *  - No transposed, repeated or copied activations: kernels index heads and
 *    KV groups in place; residual adds ride on the product's epilogue; saved
 *    activations are the buffers the forward wrote, not copies.
 *  - The frozen weights keep their binary16 values. With tensor cores on (the
 *    default) they are stored as binary16, once as [out, in] and once
 *    transposed, so that the forward and the backward product both read
 *    operands contiguous along the contraction; the activation operand of each
 *    product is a binary16 copy made just before it (gradients scaled by a power
 *    of two into binary16's range, scaled back in the product's epilogue) and
 *    accumulation is fp32. With tensor cores off (LLMB200_SFT_TC=0) the weights
 *    are fp32 copies of the binary16 values and every product runs on the CUDA
 *    cores in fp32: exactly the reference's float(half) * float.
 *  - Clip + AdamW run on the device over one flat parameter vector.
 */
#include "internal.h"
#include "../../include/llmb200_sft.h"
#include "../../include/llmb200_train_kernels.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct {
    float *w;        /* fp32 [rows, cols]          (CUDA-core mode; q/k/v also fp32 wt) */
    float *wt;       /* fp32 [cols, rows] or NULL */
    void *wh;        /* binary16 [rows, cols]      (tensor-core mode) */
    void *wth;       /* binary16 [cols, rows] */
    int rows, cols;
} SftMat;

typedef struct {
    SftMat qkv, o, gu, down;
    float *g_in, *g_post, *g_q, *g_k;   /* norm gammas */
    float *g_pre_ff, *g_post_ff;        /* Gemma3: the two norms around the FFN */
    float *o_out, *ff_raw;              /* Gemma3: saved o-projection and down-projection outputs (inputs of its post norms) */
    float *inv_freq;                    /* [hd/2] */
    /* saved activations */
    float *x_in, *ln1, *qkv_out, *q_f, *k_f, *probs, *x_mid, *ln2, *gu_out;
    float *mid_q, *mid_v;               /* columns QKV.. of qkv_out (row stride QKVX), not separate buffers */
    size_t lora_off;                    /* offset of this layer in the flat LoRA vectors */
    float *acc[4];                      /* full-parameter mode: gradient accumulators of qkv, o, gu, down (binary16 values) */
    MetalBuf *lora_buf[4];              /* handles made on demand by sft_get_lora_weight_buf */
    int loaded;
} SftLayer;

struct SFTState {
    int D, Hq, Hkv, hd, IS, V, NL, N, S, M, QKV;
    int XR, QKVX;               /* LoRA columns appended to the fused q/k/v product (2R rounded up to 4) */
    int Hq_hd, Hkv_hd;
    float eps, lora_scaling, emb_scale;
    int lora_rank, step_count, model_type;
    int use_tc, err, finished;
    /* Full-parameter mode (sft_state_create_full): no LoRA (rank 0); every projection and the LM head are
     * trained by plain SGD inside the backward pass. wmode says what a backward pass does with a weight
     * gradient dW = dY^T X: 0 nothing, 1 W <- half(W - lr dW) at once, 2 G <- half(G + dW) into accumulators. */
    int gemma;                  /* Gemma3 block order: four norms per layer, GeGLU, embeddings scaled and tied to the LM head */
    int full_param, wmode;
    float sgd_lr;
    float *acc_lm;
    unsigned long long weights_version;   /* counts changes of the base matrices: a decode state made from this one re-reads them */
    float *rope_thetas;

    SftLayer *layers;
    SftMat lm_head;
    float *final_g, *d_emb;
    float *token_emb_host;

    /* flat LoRA vectors (device) + pinned mirror of the gradients */
    size_t n_lora, per_layer, sizes[4], sub_off[4];
    float *lora_p, *lora_g, *lora_m, *lora_v;
    float *h_grad;

    /* scratch */
    float *x_final, *ln_final, *att, *act, *logits, *dlogits, *losses;
    float *dx, *d_ln, *d_lnx, *d_act, *d_gu, *d_att, *dqkv, *d_score;
    void *xh;                   /* binary16 operand copy of the activation / gradient a product reads */
    float gscale;               /* power of two applied to gradient operands before rounding to binary16 */
    int xh_has_dlogits;         /* the loss kernel has left half(dlogits * gscale) in xh */
    uint32_t *tokens, *targets;
    double *partials;
    float *d_norm;
    float *x_shared;            /* managed [M, D]: sft_get_x_cpu */
    float *losses_shared;       /* managed [M]:    sft_get_losses_cpu */
    uint32_t *h_tok;            /* pinned [2*M] */
    float *h_loss;              /* pinned [M + 1] */
    MetalBuf *mb_logits, *mb_dlogits;

    /* views handed out by the weight-sharing accessors, made on first use */
    LayerW *share_layers;
    WMat *share_lm;
    MetalBuf *share_final_g;

    /* forward + loss + backward of a step as one CUDA graph: captured on the second step (the first one runs
     * eagerly and finishes every lazy initialisation), replayed from then on */
    cudaGraphExec_t step_graph;
    int step_graph_state;       /* 0 first step pending, 1 capture pending, 2 ready, -1 not available */
    unsigned long long step_graph_kernels;

    cudaEvent_t ev[4];
    /* The four LoRA-gradient products of a layer feed nothing before the optimizer: they run on a second stream
     * beside the rest of the backward pass and are joined before the buffers they read are written again. */
    cudaStream_t side;
    cudaEvent_t ev_fork, ev_join;
    int side_pending;
    float last_step_ms, last_update_ms, last_norm;
};

#define N_PARTIALS 1024

#define S_TRY(s, call)                                                                     \
    do {                                                                                   \
        int e__ = (call);                                                                  \
        if (e__ != 0 && !(s)->err) {                                                       \
            (s)->err = e__;                                                                \
            fprintf(stderr, "[llmb200] sft: %s failed: code %d%s%s (%s:%d)\n", #call, e__, \
                    e__ > 0 ? " " : "", e__ > 0 ? cudaGetErrorString((cudaError_t)e__) : "", \
                    __FILE__, __LINE__);                                                   \
        }                                                                                  \
    } while (0)

static float *dalloc(SFTState *s, size_t n_floats)
{
    float *p = NULL;
    cudaError_t e = cudaMalloc((void **)&p, (n_floats ? n_floats : 1) * sizeof(float));
    if (e != cudaSuccess) {
        fprintf(stderr, "[llmb200] sft: allocating %zu floats failed: %s\n", n_floats, cudaGetErrorString(e));
        if (!s->err) s->err = (int)e;
        return NULL;
    }
    return p;
}

/* ---------------------------------------------------------------- weights */

static void *halloc(SFTState *s, size_t n_halves)
{
    void *p = NULL;
    cudaError_t e = cudaMalloc(&p, (n_halves ? n_halves : 1) * 2);
    if (e != cudaSuccess) {
        fprintf(stderr, "[llmb200] sft: allocating %zu halves failed: %s\n", n_halves, cudaGetErrorString(e));
        if (!s->err) s->err = (int)e;
        return NULL;
    }
    return p;
}

/* rows of `src` ([rows, cols] fp32, host) into rows row0.. of the device matrix, as binary16 values */
static int mat_put(SFTState *s, SftMat *m, int row0, const float *src, int rows)
{
    if (!src) return B200_E_BADARG;
    const size_t off = (size_t)row0 * m->cols, n = (size_t)rows * m->cols;
    if (s->use_tc) return llmb200_upload_f16_into((char *)m->wh + off * 2, src, n);
    int rc = llmb200_upload_f32_into(m->w + off, src, n);
    if (rc) return rc;
    return b200_round_f16(m->w + off, n, g_rt.stream);
}

static int mat_alloc(SFTState *s, SftMat *m, int rows, int cols)
{
    m->rows = rows;
    m->cols = cols;
    if (s->use_tc) {
        m->wh = halloc(s, (size_t)rows * cols);
        m->wth = halloc(s, (size_t)rows * cols);
        return (m->wh && m->wth) ? 0 : -1;
    }
    m->w = dalloc(s, (size_t)rows * cols);
    return m->w ? 0 : -1;
}

/* The fused q/k/v matrix carries XR extra rows (the LoRA A matrices) and always has a transposed copy
 * [D + XR, QKV] whose extra rows hold sc * B (see b200_lora_pack). */
static int qkv_alloc(SFTState *s, SftMat *m)
{
    const size_t n = (size_t)s->QKVX * s->D, nt = (size_t)(s->D + s->XR) * s->QKV;
    m->rows = s->QKVX;
    m->cols = s->D;
    if (s->use_tc) {
        m->wh = halloc(s, n);
        m->wth = halloc(s, nt);
        if (m->wh) cudaMemsetAsync(m->wh, 0, n * 2, g_rt.stream);
        if (m->wth) cudaMemsetAsync(m->wth, 0, nt * 2, g_rt.stream);
        return (m->wh && m->wth) ? 0 : -1;
    }
    m->w = dalloc(s, n);
    m->wt = dalloc(s, nt);
    if (m->w) cudaMemsetAsync(m->w, 0, n * 4, g_rt.stream);
    if (m->wt) cudaMemsetAsync(m->wt, 0, nt * 4, g_rt.stream);
    return (m->w && m->wt) ? 0 : -1;
}

/* the transposed copy of the first `rows` rows (all of them unless the matrix carries extra rows) */
static int mat_finish_rows(SFTState *s, SftMat *m, int rows)
{
    if (s->use_tc) return b200_transpose_f16(m->wh, rows, m->cols, m->wth, g_rt.stream);
    if (!m->wt) return 0;
    return b200_transpose_f32(m->w, rows, m->cols, m->wt, g_rt.stream);
}
static int mat_finish(SFTState *s, SftMat *m) { return mat_finish_rows(s, m, m->rows); }

static void mat_free(SftMat *m)
{
    cudaFree(m->w);
    cudaFree(m->wt);
    cudaFree(m->wh);
    cudaFree(m->wth);
    m->w = m->wt = NULL;
    m->wh = m->wth = NULL;
}

/* One product on the tensor cores: C[M, N] = alpha * half(A * a_scale)[M, K] * Bh[N, K]^T (+ R). */
static void gemm_tc(SFTState *s, const float *A, float a_scale, const void *Bh, float *C, long long ldc, const float *R,
                    int N, int K)
{
    /* A == NULL: the producing kernel has already left the binary16 operand (times a_scale) in xh */
    if (A) S_TRY(s, b200_f32_to_f16(A, (size_t)s->M * K, a_scale, s->xh, g_rt.stream));
    b200_gemm_args g = {0};
    g.A = (const float *)s->xh; g.a_row = K; g.a_col = 1;
    g.B = (const float *)Bh; g.b_row = 1; g.b_col = K;
    g.C = C; g.ldc = ldc;
    g.R = R; g.ldr = ldc;
    g.M = s->M; g.N = N; g.K = K;
    g.alpha = 1.0f / a_scale;
    g.d_err = (unsigned *)s->d_norm + 1;
    S_TRY(s, b200_gemm_f16(&g, g_rt.stream));
}

/* C[M, W.rows] = A[M, W.cols] * W^T (+ R): the reference's f16_matmul. */
static void gemm_fwd(SFTState *s, const float *A, const SftMat *W, float *C, const float *R)
{
    if (s->use_tc) { gemm_tc(s, A, 1.0f, W->wh, C, W->rows, R, W->rows, W->cols); return; }
    b200_gemm_args g = {0};
    g.A = A; g.a_row = W->cols; g.a_col = 1;
    g.B = W->w; g.b_row = 1; g.b_col = W->cols;
    g.C = C; g.ldc = W->rows;
    g.R = R; g.ldr = W->rows;
    g.M = s->M; g.N = W->rows; g.K = W->cols;
    g.alpha = 1.0f;
    S_TRY(s, b200_gemm_f32(&g, g_rt.stream));
}

/* C[M, W.cols] = A[M, W.rows] * W: the reference's f16_matmul_nt. A is a gradient. */
static void gemm_bwd(SFTState *s, const float *A, const SftMat *W, float *C)
{
    if (s->use_tc) { gemm_tc(s, A, s->gscale, W->wth, C, W->cols, NULL, W->cols, W->rows); return; }
    b200_gemm_args g = {0};
    g.A = A; g.a_row = W->rows; g.a_col = 1;
    g.B = W->w; g.b_row = W->cols; g.b_col = 1;
    g.C = C; g.ldc = W->cols;
    g.M = s->M; g.N = W->cols; g.K = W->rows;
    g.alpha = 1.0f;
    S_TRY(s, b200_gemm_f32(&g, g_rt.stream));
}

/* generic small product on the CUDA cores */
static void gemm_small(SFTState *s, const float *A, long long a_row, long long a_col, const float *B, long long b_row,
                       long long b_col, float *C, long long ldc, const float *R, int M, int N, int K, float alpha)
{
    b200_gemm_args g = {0};
    g.A = A; g.a_row = a_row; g.a_col = a_col;
    g.B = B; g.b_row = b_row; g.b_col = b_col;
    g.C = C; g.ldc = ldc; g.R = R; g.ldr = ldc;
    g.M = M; g.N = N; g.K = K; g.alpha = alpha;
    S_TRY(s, b200_gemm_f32(&g, g_rt.stream));
}

/* ---------------------------------------------------------------- create */

static SFTState *sft_begin(const llmb200_config *cfg, int seq_len, int n_seq, int lora_rank, float lora_alpha, int full_param)
{
    if (!cfg || seq_len <= 0 || n_seq <= 0 || lora_rank < (full_param ? 0 : 1) || lora_rank > 64 || (full_param && lora_rank)) {
        fprintf(stderr, "[FastSFT] bad arguments (seq_len %d, sequences %d, rank %d; rank must be 1..64)\n", seq_len,
                n_seq, lora_rank);
        return NULL;
    }
    if (cfg->model_type != MODEL_QWEN3 && cfg->model_type != MODEL_GEMMA3) {
        fprintf(stderr, "[FastSFT] unknown model type %d\n", (int)cfg->model_type);
        return NULL;
    }
    if (cfg->n_kv_heads <= 0 || cfg->n_q_heads % cfg->n_kv_heads ||
        (cfg->head_dim != 64 && cfg->head_dim != 128 && cfg->head_dim != 256)) {
        fprintf(stderr, "[FastSFT] unsupported head layout (%d q, %d kv, head_dim %d)\n", cfg->n_q_heads,
                cfg->n_kv_heads, cfg->head_dim);
        return NULL;
    }
    if (fast_metal_init() != 0) {
        fprintf(stderr, "[FastSFT] device init failed\n");
        return NULL;
    }
    SFTState *s = calloc(1, sizeof(SFTState));
    if (!s) { fast_metal_shutdown(); return NULL; }
    s->model_type = cfg->model_type;
    s->gemma = cfg->model_type == MODEL_GEMMA3;
    s->D = cfg->d_model; s->Hq = cfg->n_q_heads; s->Hkv = cfg->n_kv_heads; s->hd = cfg->head_dim;
    s->IS = cfg->intermediate_size; s->V = cfg->vocab_size; s->NL = cfg->n_layers;
    s->N = seq_len; s->S = n_seq; s->M = seq_len * n_seq;
    s->Hq_hd = s->Hq * s->hd; s->Hkv_hd = s->Hkv * s->hd; s->QKV = s->Hq_hd + 2 * s->Hkv_hd;
    s->XR = (2 * lora_rank + 3) & ~3;
    s->QKVX = s->QKV + s->XR;
    s->emb_scale = s->gemma ? sqrtf((float)s->D) : 1.0f;       /* src/nn/fast_sft.c:302 */
    s->eps = 1e-6f;
    s->lora_rank = lora_rank;
    s->lora_scaling = lora_rank ? lora_alpha / (float)lora_rank : 0.0f;
    s->full_param = full_param;
    /* Tensor cores need 16-byte operand rows (dimensions in multiples of 8 halves) and at least 16 x 64
     * outputs; otherwise, or with LLMB200_SFT_TC=0, every product runs on the CUDA cores in fp32. */
    const char *tc = getenv("LLMB200_SFT_TC");
    s->use_tc = !(tc && tc[0] == '0') && s->M >= 16 && s->D >= 64 && s->V >= 64 && !(s->D % 8) && !(s->Hq_hd % 8) &&
                !(s->Hkv_hd % 8) && !(s->IS % 8);
    /* the weight gradients and their SGD steps are fp32 products over fp32 activations: CUDA-core mode */
    if (full_param) s->use_tc = 0;
    /* the Gemma3 block order is implemented on the fp32 path only */
    if (s->gemma) s->use_tc = 0;
    /* gradients reach at most 1/M (the loss scale) at the logits: 8 * M rounded up to a power of two maps
     * them to ~8 in binary16 and leaves four decades below before the subnormals start */
    s->gscale = 8.0f;
    while (s->gscale < 8.0f * (float)s->M) s->gscale *= 2.0f;
    s->rope_thetas = calloc(s->NL, sizeof(float));
    s->layers = calloc(s->NL, sizeof(SftLayer));

    const int R = lora_rank, M = s->M;
    s->sizes[0] = (size_t)R * s->D; s->sizes[1] = (size_t)s->Hq_hd * R;
    s->sizes[2] = (size_t)R * s->D; s->sizes[3] = (size_t)s->Hkv_hd * R;
    s->sub_off[0] = 0;
    for (int i = 1; i < 4; ++i) s->sub_off[i] = s->sub_off[i - 1] + s->sizes[i - 1];
    s->per_layer = s->sub_off[3] + s->sizes[3];
    s->n_lora = s->per_layer * s->NL;
    s->lora_p = dalloc(s, s->n_lora); s->lora_g = dalloc(s, s->n_lora);
    s->lora_m = dalloc(s, s->n_lora); s->lora_v = dalloc(s, s->n_lora);
    if (!s->err) {
        cudaMemsetAsync(s->lora_p, 0, s->n_lora * 4, g_rt.stream);
        cudaMemsetAsync(s->lora_g, 0, s->n_lora * 4, g_rt.stream);
        cudaMemsetAsync(s->lora_m, 0, s->n_lora * 4, g_rt.stream);
        cudaMemsetAsync(s->lora_v, 0, s->n_lora * 4, g_rt.stream);
    }
    if (cudaMallocHost((void **)&s->h_grad, (s->n_lora ? s->n_lora : 1) * 4) != cudaSuccess) s->err = -10;

    for (int L = 0; L < s->NL && !s->err; ++L) {
        SftLayer *l = &s->layers[L];
        l->lora_off = s->per_layer * L;
        qkv_alloc(s, &l->qkv);
        mat_alloc(s, &l->o, s->D, s->Hq_hd);
        mat_alloc(s, &l->gu, 2 * s->IS, s->D);
        mat_alloc(s, &l->down, s->D, s->IS);
        l->g_in = dalloc(s, s->D); l->g_post = dalloc(s, s->D);
        l->g_q = dalloc(s, s->hd); l->g_k = dalloc(s, s->hd);
        l->inv_freq = dalloc(s, s->hd / 2);
        l->x_in = dalloc(s, (size_t)M * s->D); l->ln1 = dalloc(s, (size_t)M * s->D);
        l->qkv_out = dalloc(s, (size_t)M * s->QKVX);
        if (l->qkv_out) { l->mid_q = l->qkv_out + s->QKV; l->mid_v = l->mid_q + R; }
        l->q_f = dalloc(s, (size_t)M * s->Hq_hd); l->k_f = dalloc(s, (size_t)M * s->Hkv_hd);
        l->probs = dalloc(s, (size_t)s->S * s->Hq * s->N * s->N);
        l->x_mid = dalloc(s, (size_t)M * s->D); l->ln2 = dalloc(s, (size_t)M * s->D);
        l->gu_out = dalloc(s, (size_t)M * 2 * s->IS);
        if (s->gemma) {
            l->g_pre_ff = dalloc(s, s->D); l->g_post_ff = dalloc(s, s->D);
            l->o_out = dalloc(s, (size_t)M * s->D); l->ff_raw = dalloc(s, (size_t)M * s->D);
        }
    }
    mat_alloc(s, &s->lm_head, s->V, s->D);
    s->final_g = dalloc(s, s->D);
    s->d_emb = dalloc(s, (size_t)s->V * s->D);

    s->x_final = dalloc(s, (size_t)M * s->D); s->ln_final = dalloc(s, (size_t)M * s->D);
    s->att = dalloc(s, (size_t)M * s->Hq_hd); s->act = dalloc(s, (size_t)M * s->IS);
    s->logits = dalloc(s, (size_t)M * s->V); s->dlogits = dalloc(s, (size_t)M * s->V);
    s->losses = dalloc(s, M);
    s->dx = dalloc(s, (size_t)M * s->D); s->d_ln = dalloc(s, (size_t)M * s->D);
    s->d_lnx = dalloc(s, (size_t)M * (s->D + s->XR));
    s->d_act = dalloc(s, (size_t)M * s->IS); s->d_gu = dalloc(s, (size_t)M * 2 * s->IS);
    s->d_att = dalloc(s, (size_t)M * s->Hq_hd); s->dqkv = dalloc(s, (size_t)M * s->QKV);
    s->d_score = dalloc(s, (size_t)s->S * s->Hq * s->N * (s->N > 2 * s->hd ? s->N : 2 * s->hd));
    if (s->use_tc) {
        size_t widest = (size_t)s->V;
        if ((size_t)2 * s->IS > widest) widest = (size_t)2 * s->IS;
        if ((size_t)s->QKV > widest) widest = (size_t)s->QKV;
        if ((size_t)s->D > widest) widest = (size_t)s->D;
        s->xh = halloc(s, (size_t)M * widest);
    }
    s->tokens = (uint32_t *)dalloc(s, M); s->targets = (uint32_t *)dalloc(s, M);
    s->partials = (double *)dalloc(s, 2 * N_PARTIALS);
    s->d_norm = dalloc(s, 2);                 /* [0] gradient norm, [1] error word of the tensor-core products */
    if (s->d_norm) cudaMemsetAsync(s->d_norm, 0, 8, g_rt.stream);
    if (!s->err) {
        if (cudaMallocManaged((void **)&s->x_shared, (size_t)M * s->D * 4, cudaMemAttachGlobal) != cudaSuccess ||
            cudaMallocManaged((void **)&s->losses_shared, (size_t)M * 4, cudaMemAttachGlobal) != cudaSuccess ||
            cudaMallocHost((void **)&s->h_tok, (size_t)2 * M * 4) != cudaSuccess ||
            cudaMallocHost((void **)&s->h_loss, (size_t)(M + 1) * 4) != cudaSuccess)
            s->err = -11;
    }
    if (!s->err) {
        memset(s->x_shared, 0, (size_t)M * s->D * 4);
        memset(s->losses_shared, 0, (size_t)M * 4);
        s->mb_logits = llmb200_buf_wrap(s->logits, (size_t)M * s->V * 4);
        s->mb_dlogits = llmb200_buf_wrap(s->dlogits, (size_t)M * s->V * 4);
        for (int i = 0; i < 4; ++i)
            if (cudaEventCreate(&s->ev[i]) != cudaSuccess) s->err = -12;
        if (!getenv("LLMB200_SFT_NO_OVERLAP") && lora_rank > 0) {
            if (cudaStreamCreateWithFlags(&s->side, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&s->ev_join, cudaEventDisableTiming) != cudaSuccess)
                s->err = -13;
        }
    }
    if (s->err) {
        fprintf(stderr, "[FastSFT] state allocation failed\n");
        sft_state_free(s);
        return NULL;
    }
    return s;
}

SFTState *llmb200_sft_begin(const llmb200_config *cfg, int seq_len, int n_seq, int lora_rank, float lora_alpha)
{
    return sft_begin(cfg, seq_len, n_seq, lora_rank, lora_alpha, 0);
}

static int upload_small(float *d, const float *src, size_t n)
{
    return src ? llmb200_upload_f32_into(d, src, n) : B200_E_BADARG;
}

int llmb200_sft_load_layer(SFTState *s, int L, const LayerWeightRef *r, float rope_theta, const float *const lora[4])
{
    if (!s || !r || L < 0 || L >= s->NL) return B200_E_BADARG;
    SftLayer *l = &s->layers[L];
    if (r->q_proj.rows != s->Hq_hd || r->q_proj.cols != s->D || r->k_proj.rows != s->Hkv_hd ||
        r->v_proj.rows != s->Hkv_hd || r->o_proj.rows != s->D || r->o_proj.cols != s->Hq_hd ||
        r->gate_proj.rows != s->IS || r->up_proj.rows != s->IS || r->down_proj.rows != s->D ||
        r->down_proj.cols != s->IS) {
        fprintf(stderr, "[FastSFT] layer %d: matrix shapes do not match the configuration\n", L);
        return B200_E_BADARG;
    }
    int rc = 0;
    if (!rc) rc = mat_put(s, &l->qkv, 0, r->q_proj.data, s->Hq_hd);
    if (!rc) rc = mat_put(s, &l->qkv, s->Hq_hd, r->k_proj.data, s->Hkv_hd);
    if (!rc) rc = mat_put(s, &l->qkv, s->Hq_hd + s->Hkv_hd, r->v_proj.data, s->Hkv_hd);
    if (!rc) rc = mat_put(s, &l->o, 0, r->o_proj.data, s->D);
    if (!rc) rc = mat_put(s, &l->gu, 0, r->gate_proj.data, s->IS);
    if (!rc) rc = mat_put(s, &l->gu, s->IS, r->up_proj.data, s->IS);
    if (!rc) rc = mat_put(s, &l->down, 0, r->down_proj.data, s->D);
    if (!rc) rc = mat_finish_rows(s, &l->qkv, s->QKV);          /* rows 0..D-1 of the transposed copy */
    if (!rc) rc = mat_finish(s, &l->o);
    if (!rc) rc = mat_finish(s, &l->gu);
    if (!rc) rc = mat_finish(s, &l->down);
    if (!rc) rc = upload_small(l->g_in, r->input_norm_g, s->D);
    if (!rc) rc = upload_small(l->g_post, r->post_attn_norm_g, s->D);
    if (!rc) rc = upload_small(l->g_q, r->q_norm_g, s->hd);
    if (!rc) rc = upload_small(l->g_k, r->k_norm_g, s->hd);
    if (!rc && s->gemma) rc = upload_small(l->g_pre_ff, r->pre_ff_norm_g, s->D);
    if (!rc && s->gemma) rc = upload_small(l->g_post_ff, r->post_ff_norm_g, s->D);
    if (rc) return rc;

    /* 1 / pow(theta, 2d/hd) as the shader computes it per element (q8_kernels.metal:531) */
    const int half = s->hd / 2;
    float *f = malloc(half * sizeof(float));
    for (int d = 0; d < half; ++d) f[d] = 1.0f / powf(rope_theta, (float)(2 * d) / (float)s->hd);
    rc = llmb200_upload_f32_into(l->inv_freq, f, half);
    free(f);
    s->rope_thetas[L] = rope_theta;
    if (rc) return rc;

    /* LoRA init (src/nn/fast_sft.c:96-122): supplied matrices, else A uniform(+-1/sqrt(D)) from rand(), B = 0 */
    for (int sub = 0; sub < 4 && !rc; ++sub) {
        float *dst = s->lora_p + l->lora_off + s->sub_off[sub];
        const size_t n = s->sizes[sub];
        if (n == 0) continue;                                    /* full-parameter mode: no LoRA, no rand() drawn */
        if (lora && lora[sub]) {
            rc = llmb200_upload_f32_into(dst, lora[sub], n);
        } else if (sub == 0 || sub == 2) {
            float *tmp = malloc(n * sizeof(float));
            const float std_a = 1.0f / sqrtf((float)s->D);
            for (size_t j = 0; j < n; ++j) tmp[j] = ((float)rand() / (float)RAND_MAX - 0.5f) * 2.0f * std_a;
            rc = llmb200_upload_f32_into(dst, tmp, n);
            free(tmp);
        } else {
            rc = (int)cudaMemsetAsync(dst, 0, n * 4, g_rt.stream);
        }
    }
    l->loaded = 1;
    return rc;
}

int llmb200_sft_finish(SFTState *s, const float *lm_head, const float *final_norm_gamma, const float *token_emb,
                       int keep_host_emb)
{
    if (!s || !lm_head || !final_norm_gamma || !token_emb) return B200_E_BADARG;
    for (int L = 0; L < s->NL; ++L)
        if (!s->layers[L].loaded) {
            fprintf(stderr, "[FastSFT] layer %d was never loaded\n", L);
            return B200_E_STATE;
        }
    int rc = mat_put(s, &s->lm_head, 0, lm_head, s->V);
    if (!rc) rc = mat_finish(s, &s->lm_head);
    if (!rc) rc = llmb200_upload_f32_into(s->final_g, final_norm_gamma, s->D);
    if (!rc) rc = llmb200_upload_f32_into(s->d_emb, token_emb, (size_t)s->V * s->D);
    if (!rc && keep_host_emb) {
        s->token_emb_host = malloc((size_t)s->V * s->D * sizeof(float));
        if (s->token_emb_host) memcpy(s->token_emb_host, token_emb, (size_t)s->V * s->D * sizeof(float));
    }
    if (!rc) rc = (int)cudaStreamSynchronize(g_rt.stream);
    s->finished = rc == 0;
    return rc;
}

static SFTState *create_from_qwen3(llmb200_qwen3_model *m, int seq_len, int lora_rank, float lora_alpha, int full_param)
{
    if (!m) return NULL;
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    printf(full_param ? "[FastSFT] Converting Qwen3 weights to F16 (full-param)...\n" : "[FastSFT] Converting weights to F16...\n");
    llmb200_config cfg = { MODEL_QWEN3, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                           m->vocab_size, m->n_layers, seq_len, 1 };
    SFTState *s = sft_begin(&cfg, seq_len, 1, lora_rank, lora_alpha, full_param);
    if (!s) return NULL;
    if (full_param) s->step_graph_state = -1;      /* the learning rate is an argument of every step's kernels: no replay */
    const int Hq_hd = s->Hq_hd, Hkv_hd = s->Hkv_hd;
    for (int i = 0; i < s->NL; ++i) {
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
        r.d_model = s->D;
        r.head_dim = s->hd;
        const float *lora[4] = { NULL, NULL, NULL, NULL };
        if (!full_param && m->q_loras && m->q_loras[i]) { lora[0] = m->q_loras[i]->lora_A->data; lora[1] = m->q_loras[i]->lora_B->data; }
        if (!full_param && m->v_loras && m->v_loras[i]) { lora[2] = m->v_loras[i]->lora_A->data; lora[3] = m->v_loras[i]->lora_B->data; }
        if (llmb200_sft_load_layer(s, i, &r, m->rope_theta, lora) != 0) { sft_state_free(s); return NULL; }
    }
    if (llmb200_sft_finish(s, m->lm_head->weight->data, m->final_norm->gamma->data, m->token_emb->weight->data, 1) != 0) {
        sft_state_free(s);
        return NULL;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (t1.tv_sec - t0.tv_sec) * 1000.0 + (t1.tv_nsec - t0.tv_nsec) / 1e6;
    if (full_param) printf("[FastSFT] Qwen3 Full-param Init: %.0f ms, seq=%d\n", ms, seq_len);
    else printf("[FastSFT] Init: %.0f ms, seq=%d, lora_rank=%d\n", ms, seq_len, lora_rank);
    return s;
}

SFTState *sft_state_create(llmb200_qwen3_model *m, int seq_len, int lora_rank, float lora_alpha)
{
    return create_from_qwen3(m, seq_len, lora_rank, lora_alpha, 0);
}

/* Every projection and the LM head trainable by SGD, no adapter (src/nn/fast_sft.c:402-501). The matrices are
 * kept as fp32 holders of binary16 values and every product runs in fp32 on the CUDA cores. */
SFTState *sft_state_create_full(llmb200_qwen3_model *m, int seq_len)
{
    return create_from_qwen3(m, seq_len, 0, 0.0f, 1);
}

/* ---------------------------------------------------------------- weight sharing (src/nn/fast_sft.h:101-111) */

/* A WMat over `rows` rows of binary16 [., cols] device memory. The tensor-core mode keeps its frozen
 * matrices in exactly that form, so the view borrows them; the CUDA-core mode keeps fp32 copies of the
 * binary16 values, which are narrowed (losslessly) into memory the view owns. */
static WMat *share_view(SFTState *s, const SftMat *m, int row0, int rows)
{
    WMat *w = calloc(1, sizeof(WMat));
    MetalBuf *b = calloc(1, sizeof(MetalBuf));
    if (!w || !b) { free(w); free(b); return NULL; }
    const size_t n = (size_t)rows * m->cols;
    b->kind = MB_F16; b->rows = rows; b->cols = m->cols; b->row_stride = (long long)m->cols * 2; b->size = n * 2;
    if (m->wh) {
        b->dev = (char *)m->wh + (size_t)row0 * m->cols * 2;
        b->borrowed = 1;
    } else {
        if (cudaMalloc(&b->dev, n * 2) != cudaSuccess ||
            b200_f32_to_f16(m->w + (size_t)row0 * m->cols, n, 1.0f, b->dev, g_rt.stream) != 0) {
            if (b->dev) cudaFree(b->dev);
            free(w); free(b);
            return NULL;
        }
    }
    w->mbuf = b; w->rows = rows; w->cols = m->cols; w->nb = 0;
    return w;
}

static void share_free(SFTState *s)
{
    if (s->share_layers) {
        for (int L = 0; L < s->NL; ++L) {
            LayerW *lw = &s->share_layers[L];
            WMat *ws[] = { lw->q_proj, lw->k_proj, lw->v_proj, lw->o_proj, lw->gate_proj, lw->up_proj, lw->down_proj };
            for (int i = 0; i < 7; ++i) if (ws[i]) { metal_buf_free(ws[i]->mbuf); free(ws[i]); }
            MetalBuf *gs[] = { lw->input_norm_g, lw->post_attn_norm_g, lw->q_norm_g, lw->k_norm_g, lw->pre_ff_norm_g, lw->post_ff_norm_g };
            for (int i = 0; i < 6; ++i) metal_buf_free(gs[i]);
        }
        free(s->share_layers);
        s->share_layers = NULL;
    }
    if (s->share_lm) { metal_buf_free(s->share_lm->mbuf); free(s->share_lm); s->share_lm = NULL; }
    metal_buf_free(s->share_final_g);
    s->share_final_g = NULL;
}

/* Views that own narrowed copies (CUDA-core mode) go stale when full-parameter training changes a matrix:
 * narrow them again and drop any host mirror made from the old bytes. */
static void share_refresh_one(SFTState *s, WMat *w, const SftMat *m, int row0)
{
    if (!w || !w->mbuf || w->mbuf->borrowed || !m->w) return;
    S_TRY(s, b200_f32_to_f16(m->w + (size_t)row0 * m->cols, (size_t)w->rows * m->cols, 1.0f, w->mbuf->dev, g_rt.stream));
    free(w->mbuf->host_mirror);
    w->mbuf->host_mirror = NULL;
}

static void share_refresh(SFTState *s)
{
    for (int L = 0; L < s->NL && s->share_layers; ++L) {
        SftLayer *l = &s->layers[L];
        LayerW *lw = &s->share_layers[L];
        share_refresh_one(s, lw->q_proj, &l->qkv, 0);
        share_refresh_one(s, lw->k_proj, &l->qkv, s->Hq_hd);
        share_refresh_one(s, lw->v_proj, &l->qkv, s->Hq_hd + s->Hkv_hd);
        share_refresh_one(s, lw->o_proj, &l->o, 0);
        share_refresh_one(s, lw->gate_proj, &l->gu, 0);
        share_refresh_one(s, lw->up_proj, &l->gu, s->IS);
        share_refresh_one(s, lw->down_proj, &l->down, 0);
    }
    if (s->share_lm) share_refresh_one(s, s->share_lm, &s->lm_head, 0);
}

/* For a decode state made from this one: how often the base matrices have changed, and the views brought
 * up to date (on the library's stream) before it copies them again. */
unsigned long long llmb200_sft_weights_version(SFTState *s) { return s ? s->weights_version : 0; }
void llmb200_sft_refresh_views(SFTState *s) { if (s && s->finished) share_refresh(s); }

/* The frozen base as the reference's containers: one WMat per projection (binary16 [rows, cols], row-major)
 * and one buffer per norm vector, all views of this state's device memory; valid until sft_state_free.
 * Replaces sft_get_layers (src/nn/fast_sft.c:1346; declared in fast_sft.h:103). */
LayerW *sft_get_layers(SFTState *s)
{
    if (!s || !s->finished) return NULL;
    if (s->share_layers) return s->share_layers;
    LayerW *out = calloc((size_t)s->NL, sizeof(LayerW));
    if (!out) return NULL;
    s->share_layers = out;
    for (int L = 0; L < s->NL; ++L) {
        SftLayer *l = &s->layers[L];
        LayerW *lw = &out[L];
        lw->q_proj = share_view(s, &l->qkv, 0, s->Hq_hd);
        lw->k_proj = share_view(s, &l->qkv, s->Hq_hd, s->Hkv_hd);
        lw->v_proj = share_view(s, &l->qkv, s->Hq_hd + s->Hkv_hd, s->Hkv_hd);
        lw->o_proj = share_view(s, &l->o, 0, s->D);
        lw->gate_proj = share_view(s, &l->gu, 0, s->IS);
        lw->up_proj = share_view(s, &l->gu, s->IS, s->IS);
        lw->down_proj = share_view(s, &l->down, 0, s->D);
        lw->input_norm_g = llmb200_buf_wrap(l->g_in, (size_t)s->D * 4);
        lw->post_attn_norm_g = llmb200_buf_wrap(l->g_post, (size_t)s->D * 4);
        lw->q_norm_g = llmb200_buf_wrap(l->g_q, (size_t)s->hd * 4);
        lw->k_norm_g = llmb200_buf_wrap(l->g_k, (size_t)s->hd * 4);
        if (s->gemma) {
            lw->pre_ff_norm_g = llmb200_buf_wrap(l->g_pre_ff, (size_t)s->D * 4);
            lw->post_ff_norm_g = llmb200_buf_wrap(l->g_post_ff, (size_t)s->D * 4);
        }
        if (!lw->q_proj || !lw->k_proj || !lw->v_proj || !lw->o_proj || !lw->gate_proj || !lw->up_proj || !lw->down_proj ||
            !lw->input_norm_g || !lw->post_attn_norm_g || !lw->q_norm_g || !lw->k_norm_g) {
            share_free(s);
            return NULL;
        }
    }
    metal_flush();
    return out;
}

WMat *sft_get_lm_head(SFTState *s)                                  /* src/nn/fast_sft.c:1347 */
{
    if (!s || !s->finished) return NULL;
    if (!s->share_lm) { s->share_lm = share_view(s, &s->lm_head, 0, s->V); metal_flush(); }
    return s->share_lm;
}

MetalBuf *sft_get_final_norm_g(SFTState *s)                         /* :1348 */
{
    if (!s || !s->finished) return NULL;
    if (!s->share_final_g) s->share_final_g = llmb200_buf_wrap(s->final_g, (size_t)s->D * 4);
    return s->share_final_g;
}

ModelType sft_get_model_type(SFTState *s) { return s ? (ModelType)s->model_type : MODEL_QWEN3; }   /* :1349 */
int sft_get_n_q_heads(SFTState *s) { return s ? s->Hq : 0; }                                      /* :1350 */
int sft_get_n_kv_heads(SFTState *s) { return s ? s->Hkv : 0; }
int sft_get_head_dim(SFTState *s) { return s ? s->hd : 0; }
int sft_get_intermediate_size(SFTState *s) { return s ? s->IS : 0; }
const float *sft_get_rope_thetas(SFTState *s) { return s ? s->rope_thetas : NULL; }               /* :1354 */
/* The embedding table on the device (the reference hands out its host copy through sft_get_token_emb). */
const float *llmb200_sft_device_emb(SFTState *s) { return s ? s->d_emb : NULL; }

void sft_state_free(SFTState *s)
{
    if (!s) return;
    if (g_rt.refs > 0) cudaStreamSynchronize(g_rt.stream);
    for (int L = 0; L < s->NL && s->layers; ++L) {
        SftLayer *l = &s->layers[L];
        mat_free(&l->qkv); mat_free(&l->o); mat_free(&l->gu); mat_free(&l->down);
        float *bufs[] = { l->g_in, l->g_post, l->g_q, l->g_k, l->inv_freq, l->x_in, l->ln1, l->qkv_out, l->q_f, l->k_f,
                          l->probs, l->x_mid, l->ln2, l->gu_out, l->g_pre_ff, l->g_post_ff, l->o_out, l->ff_raw };
        for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); ++i) cudaFree(bufs[i]);
        for (int i = 0; i < 4; ++i) metal_buf_free(l->lora_buf[i]);
        for (int i = 0; i < 4; ++i) cudaFree(l->acc[i]);
    }
    cudaFree(s->acc_lm);
    mat_free(&s->lm_head);
    void *bufs[] = { s->final_g, s->d_emb, s->lora_p, s->lora_g, s->lora_m, s->lora_v, s->x_final, s->ln_final, s->att,
                     s->act, s->logits, s->dlogits, s->losses, s->dx, s->d_ln, s->d_act, s->d_gu, s->d_att, s->dqkv,
                     s->d_score, s->d_lnx, s->xh, s->tokens, s->targets, s->partials, s->d_norm, s->x_shared,
                     s->losses_shared };
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); ++i) cudaFree(bufs[i]);
    cudaFreeHost(s->h_grad); cudaFreeHost(s->h_tok); cudaFreeHost(s->h_loss);
    metal_buf_free(s->mb_logits); metal_buf_free(s->mb_dlogits);
    if (s->step_graph) cudaGraphExecDestroy(s->step_graph);
    share_free(s);
    for (int i = 0; i < 4; ++i) if (s->ev[i]) cudaEventDestroy(s->ev[i]);
    if (s->ev_fork) cudaEventDestroy(s->ev_fork);
    if (s->ev_join) cudaEventDestroy(s->ev_join);
    if (s->side) cudaStreamDestroy(s->side);
    free(s->token_emb_host);
    free(s->rope_thetas);
    free(s->layers);
    free(s);
    fast_metal_shutdown();
}

/* ---------------------------------------------------------------- forward */

static float *layer_out(SFTState *s, int L) { return L + 1 < s->NL ? s->layers[L + 1].x_in : s->x_final; }

/* x of layer 0 must be in layers[0].x_in */
static void forward_device(SFTState *s)
{
    cudaStream_t st = g_rt.stream;
    const int M = s->M, R = s->lora_rank;
    const float sc = s->lora_scaling, attn_scale = 1.0f / sqrtf((float)s->hd);
    s->xh_has_dlogits = 0;
    for (int L = 0; L < s->NL; ++L) {
        SftLayer *l = &s->layers[L];
        float *pA_q = s->lora_p + l->lora_off + s->sub_off[0], *pB_q = s->lora_p + l->lora_off + s->sub_off[1];
        float *pA_v = s->lora_p + l->lora_off + s->sub_off[2], *pB_v = s->lora_p + l->lora_off + s->sub_off[3];
        S_TRY(s, b200_rms_norm_rows_h(l->x_in, l->g_in, l->ln1, s->xh, M, s->D, s->eps, st));
        /* the LoRA matrices ride along with the frozen q/k/v weight: the product below also yields
         * mid_q = ln1 A_q^T and mid_v = ln1 A_v^T in the last columns of qkv_out (:639, :652) */
        if (R > 0) {
            if (s->use_tc)
                S_TRY(s, b200_lora_pack_f16(l->qkv.wh, l->qkv.wth, pA_q, pB_q, pA_v, pB_v, s->D, s->Hq_hd, s->Hkv_hd, R, s->XR,
                                            sc, st));
            else
                S_TRY(s, b200_lora_pack(l->qkv.w, l->qkv.wt, pA_q, pB_q, pA_v, pB_v, s->D, s->Hq_hd, s->Hkv_hd, R, s->XR, sc,
                                        st));
        }
        gemm_fwd(s, s->use_tc ? NULL : l->ln1, &l->qkv, l->qkv_out, NULL);
        if (R > 0) {
            /* q += sc * mid_q B_q^T, v += sc * mid_v B_v^T (:641-643, :654-656) */
            S_TRY(s, b200_lora_add(l->qkv_out, s->QKVX, 0, s->Hq_hd, l->mid_q, s->QKVX, pB_q, R, sc, M, st));
            S_TRY(s, b200_lora_add(l->qkv_out, s->QKVX, s->Hq_hd + s->Hkv_hd, s->Hkv_hd, l->mid_v, s->QKVX, pB_v, R, sc, M, st));
        }
        S_TRY(s, b200_qk_norm_rope(l->qkv_out, s->QKVX, l->g_q, l->g_k, l->inv_freq, M, s->N, s->Hq, s->Hkv, s->hd,
                                   s->eps, l->q_f, l->k_f, st));
        /* with tensor cores on, the operand of the next product is written as binary16 straight into xh and
         * the fp32 copy of a tensor nothing else reads (attention output, activation) is not written at all */
        S_TRY(s, b200_attn_train_fwd_h(l->q_f, l->k_f, l->qkv_out + s->Hq_hd + s->Hkv_hd, s->QKVX, s->S, s->N, s->Hq,
                                       s->Hkv, s->hd, attn_scale, l->probs, s->use_tc ? NULL : s->att, s->xh, st));
        if (s->gemma) {
            /* Gemma3 (:697-704, :725-738): o -> post-attention norm -> + residual -> pre-FFN norm -> GeGLU FFN ->
             * post-FFN norm -> + residual; the raw projection outputs are saved for the backward pass. dx is free here. */
            const size_t md = (size_t)M * s->D;
            gemm_fwd(s, s->att, &l->o, l->o_out, NULL);
            S_TRY(s, b200_rms_norm_rows(l->o_out, l->g_post, s->dx, M, s->D, s->eps, st));
            S_TRY(s, b200_add(l->x_in, s->dx, l->x_mid, md, st));
            S_TRY(s, b200_rms_norm_rows(l->x_mid, l->g_pre_ff, l->ln2, M, s->D, s->eps, st));
            gemm_fwd(s, l->ln2, &l->gu, l->gu_out, NULL);
            S_TRY(s, b200_gelu_mul_rows(l->gu_out, M, s->IS, s->act, st));
            gemm_fwd(s, s->act, &l->down, l->ff_raw, NULL);
            S_TRY(s, b200_rms_norm_rows(l->ff_raw, l->g_post_ff, s->dx, M, s->D, s->eps, st));
            S_TRY(s, b200_add(l->x_mid, s->dx, layer_out(s, L), md, st));
            continue;
        }
        gemm_fwd(s, s->use_tc ? NULL : s->att, &l->o, l->x_mid, l->x_in);    /* + residual (:686) */
        S_TRY(s, b200_rms_norm_rows_h(l->x_mid, l->g_post, l->ln2, s->xh, M, s->D, s->eps, st));
        gemm_fwd(s, s->use_tc ? NULL : l->ln2, &l->gu, l->gu_out, NULL);
        S_TRY(s, b200_silu_mul_rows_h(l->gu_out, M, s->IS, s->use_tc ? NULL : s->act, s->xh, st));
        gemm_fwd(s, s->use_tc ? NULL : s->act, &l->down, layer_out(s, L), l->x_mid);   /* + residual (:738) */
    }
    S_TRY(s, b200_rms_norm_rows_h(s->x_final, s->final_g, s->ln_final, s->xh, M, s->D, s->eps, st));
    gemm_fwd(s, s->use_tc ? NULL : s->ln_final, &s->lm_head, s->logits, NULL);
}

static void loss_device(SFTState *s)
{
    /* 1/N per sequence (:759), and the mean over the S sequences of a step */
    const float gs = 1.0f / ((float)s->N * (float)s->S);
    S_TRY(s, b200_softmax_ce_rows_h(s->logits, s->targets, s->M, s->V, gs, s->losses, s->dlogits, s->xh, s->gscale,
                                    g_rt.stream));
    s->xh_has_dlogits = s->use_tc;
}

/* ---------------------------------------------------------------- backward */

/* Full-parameter mode: the weight gradient dW = dY^T X over the M token rows (dY [M, ldy], X [M, ldx]) goes
 * into rows 0..rows-1 of the matrix the way wmode says: W <- half(W - lr dW) (f16_sgd_fused,
 * shaders/q8_kernels.metal:1097-1125) or G <- half(G + dW) (f16_grad_accum, :1164-1191). One fp32 sum over
 * the tokens in ascending order per element, one rounding to binary16, as there. The matrices are fp32
 * holders of binary16 values in this mode, so the product adds into them in place and a rounding pass follows. */
static void weight_step(SFTState *s, SftMat *W, float *acc, int rows, const float *dY, long long ldy, const float *X,
                        long long ldx)
{
    if (!s->full_param || !s->wmode) return;
    float *dst = s->wmode == 2 ? acc : W->w;
    if (!dst) {
        if (!s->err) { s->err = B200_E_STATE; fprintf(stderr, "[FastSFT] gradient accumulation without sft_alloc_grad_accum\n"); }
        return;
    }
    b200_gemm_args g = {0};
    g.A = dY; g.a_row = 1; g.a_col = ldy;          /* A[m, k] = dY[k, m] */
    g.B = X; g.b_row = ldx; g.b_col = 1;           /* B[k, n] = X[k, n] */
    g.C = dst; g.ldc = W->cols;
    g.R = dst; g.ldr = W->cols;                    /* in place: every element is read and written by one thread */
    g.M = rows; g.N = W->cols; g.K = s->M;
    g.alpha = s->wmode == 2 ? 1.0f : -s->sgd_lr;
    S_TRY(s, b200_gemm_f32(&g, g_rt.stream));
    S_TRY(s, b200_round_f16(dst, (size_t)rows * W->cols, g_rt.stream));
    if (s->wmode == 1) s->weights_version++;
}

static void backward_device(SFTState *s)
{
    cudaStream_t st = g_rt.stream;
    const int M = s->M, R = s->lora_rank, QKV = s->QKV;
    const float sc = s->lora_scaling, attn_scale = 1.0f / sqrtf((float)s->hd);
    /* the loss kernel leaves the binary16 copy of dlogits in xh; a caller that wrote dlogits itself
     * (sft_get_dlogits + sft_backward) gets it converted here */
    gemm_bwd(s, s->xh_has_dlogits ? NULL : s->dlogits, &s->lm_head, s->d_ln);                /* :777 */
    weight_step(s, &s->lm_head, s->acc_lm, s->V, s->dlogits, s->V, s->ln_final, s->D);       /* :778-785 */
    s->xh_has_dlogits = 0;
    const float hs = s->gscale;
    S_TRY(s, b200_rms_norm_bwd_rows_h(s->x_final, s->d_ln, s->D, s->final_g, s->dx, M, s->D, s->eps, 0, 0.f, s->xh, hs, st));
    for (int L = s->NL - 1; L >= 0; --L) {
        SftLayer *l = &s->layers[L];
        float *pA_q = s->lora_p + l->lora_off + s->sub_off[0], *pB_q = s->lora_p + l->lora_off + s->sub_off[1];
        float *pA_v = s->lora_p + l->lora_off + s->sub_off[2], *pB_v = s->lora_p + l->lora_off + s->sub_off[3];
        float *gA_q = s->lora_g + l->lora_off + s->sub_off[0], *gB_q = s->lora_g + l->lora_off + s->sub_off[1];
        float *gA_v = s->lora_g + l->lora_off + s->sub_off[2], *gB_v = s->lora_g + l->lora_off + s->sub_off[3];
        const float *d_o = s->dx;          /* the gradient that enters the o projection: dx, or (Gemma3) dx through the post-attention norm */
        if (s->gemma) {
            /* FFN, Gemma3 (:797-838): post-FFN norm, down, GeGLU, gate/up, pre-FFN norm; dx gains the result */
            S_TRY(s, b200_rms_norm_bwd_rows(l->ff_raw, s->dx, s->D, l->g_post_ff, s->d_ln, M, s->D, s->eps, 0, 0.f, st));
            gemm_bwd(s, s->d_ln, &l->down, s->d_act);
            if (s->full_param && s->wmode) {
                S_TRY(s, b200_gelu_mul_rows(l->gu_out, M, s->IS, s->act, st));
                weight_step(s, &l->down, l->acc[3], s->D, s->d_ln, s->D, s->act, s->IS);
            }
            S_TRY(s, b200_gelu_mul_bwd_rows(s->d_act, l->gu_out, M, s->IS, s->d_gu, st));
            gemm_bwd(s, s->d_gu, &l->gu, s->d_ln);
            weight_step(s, &l->gu, l->acc[2], 2 * s->IS, s->d_gu, 2 * s->IS, l->ln2, s->D);
            S_TRY(s, b200_rms_norm_bwd_rows(l->x_mid, s->d_ln, s->D, l->g_pre_ff, s->dx, M, s->D, s->eps, 1, 0.f, st));
            /* attention, Gemma3 (:875-888): through the post-attention norm first */
            S_TRY(s, b200_rms_norm_bwd_rows(l->o_out, s->dx, s->D, l->g_post, s->d_ln, M, s->D, s->eps, 0, 0.f, st));
            d_o = s->d_ln;
            goto attention;
        }
        /* FFN (:841-872) */
        gemm_bwd(s, s->use_tc ? NULL : s->dx, &l->down, s->d_act);           /* dx is in xh already */
        if (s->full_param && s->wmode) {
            /* the activation of this layer is not kept by the forward pass: made again from the saved gate/up (:842-849) */
            S_TRY(s, b200_silu_mul_rows_h(l->gu_out, M, s->IS, s->act, NULL, st));
            weight_step(s, &l->down, l->acc[3], s->D, s->dx, s->D, s->act, s->IS);
        }
        S_TRY(s, b200_silu_mul_bwd_rows_h(s->d_act, l->gu_out, M, s->IS, s->use_tc ? NULL : s->d_gu, s->xh, hs, st));
        gemm_bwd(s, s->use_tc ? NULL : s->d_gu, &l->gu, s->d_ln);
        weight_step(s, &l->gu, l->acc[2], 2 * s->IS, s->d_gu, 2 * s->IS, l->ln2, s->D);      /* gate and up rows (:853-868) */
        S_TRY(s, b200_rms_norm_bwd_rows_h(l->x_mid, s->d_ln, s->D, l->g_post, s->dx, M, s->D, s->eps, 1, 0.f, s->xh, hs, st));
        /* attention (:889-918) */
    attention:;
        gemm_bwd(s, s->use_tc ? NULL : d_o, &l->o, s->d_att);
        const float *v = l->qkv_out + s->Hq_hd + s->Hkv_hd;
        if (s->full_param && s->wmode) {
            /* likewise the attention output, from the saved q, k, v (probs is rewritten with the same values) (:892-899) */
            S_TRY(s, b200_attn_train_fwd_h(l->q_f, l->k_f, v, s->QKVX, s->S, s->N, s->Hq, s->Hkv, s->hd, attn_scale, l->probs,
                                           s->att, NULL, st));
            weight_step(s, &l->o, l->acc[1], s->D, d_o, s->D, s->att, s->Hq_hd);
        }
        /* dqkv is about to be rewritten: the LoRA-gradient products of the layer above must have read it */
        if (s->side_pending) { S_TRY(s, (int)cudaStreamWaitEvent(st, s->ev_join, 0)); s->side_pending = 0; }
        S_TRY(s, b200_attn_train_bwd(s->d_att, l->probs, l->q_f, l->k_f, v, s->QKVX, s->S, s->N, s->Hq, s->Hkv, s->hd,
                                     attn_scale, s->d_score, s->dqkv, QKV, st));
        S_TRY(s, b200_qk_norm_rope_bwd(s->dqkv, l->qkv_out, s->QKVX, QKV, l->g_q, l->g_k, l->inv_freq, M, s->N, s->Hq,
                                       s->Hkv, s->hd, s->eps, st));
        const float *dq = s->dqkv, *dv = s->dqkv + s->Hq_hd + s->Hkv_hd;
        /* Through the frozen q, k, v projections (:955-958, :968-970). The transposed weight carries sc*B_q and
         * sc*B_v as extra rows, so the same product leaves tmp_q = sc dq B_q and tmp_v = sc dv B_v (:948-949,
         * :963-964) in columns D.. of d_lnx. */
        const int DX = s->D + s->XR;
        if (s->full_param && s->wmode) {
            /* q, k, v take their step BEFORE the gradient goes on through them (:922-945): the product below
             * reads the updated matrices when the step is immediate */
            weight_step(s, &l->qkv, l->acc[0], QKV, s->dqkv, QKV, l->ln1, s->D);
            if (s->wmode == 1) S_TRY(s, mat_finish_rows(s, &l->qkv, QKV));
        }
        if (s->use_tc) {
            gemm_tc(s, s->dqkv, s->gscale, l->qkv.wth, s->d_lnx, DX, NULL, DX, QKV);
        } else {
            b200_gemm_args g = {0};
            g.A = s->dqkv; g.a_row = QKV; g.a_col = 1;
            g.B = l->qkv.wt; g.b_row = 1; g.b_col = QKV;
            g.C = s->d_lnx; g.ldc = DX;
            g.M = M; g.N = DX; g.K = QKV; g.alpha = 1.0f;
            S_TRY(s, b200_gemm_f32(&g, st));
        }
        const float *tmp_q = s->d_lnx + s->D, *tmp_v = tmp_q + R;
        /* dB = sc dq^T mid (:946-947, :961-962); dA = tmp^T ln1 (:950, :965) */
        if (R == 0) {
            /* full-parameter mode: no adapter */
        } else if (R <= 16) {
            /* They read dqkv, the saved mid and ln1 of this layer and the tmp columns of d_lnx, none of which
             * changes before the next layer's attention backward (dqkv) and q/k/v product (d_lnx) -- both after the join. */
            cudaStream_t xs = st;
            if (s->side) {
                S_TRY(s, (int)cudaEventRecord(s->ev_fork, st));
                S_TRY(s, (int)cudaStreamWaitEvent(s->side, s->ev_fork, 0));
                xs = s->side;
            }
            S_TRY(s, b200_xty_skinny(dq, QKV, l->mid_q, s->QKVX, M, s->Hq_hd, R, sc, gB_q, R, 1, xs));
            S_TRY(s, b200_xty_skinny(l->ln1, s->D, tmp_q, DX, M, s->D, R, 1.0f, gA_q, 1, s->D, xs));
            S_TRY(s, b200_xty_skinny(dv, QKV, l->mid_v, s->QKVX, M, s->Hkv_hd, R, sc, gB_v, R, 1, xs));
            S_TRY(s, b200_xty_skinny(l->ln1, s->D, tmp_v, DX, M, s->D, R, 1.0f, gA_v, 1, s->D, xs));
            if (s->side) { S_TRY(s, (int)cudaEventRecord(s->ev_join, s->side)); s->side_pending = 1; }
        } else {
            gemm_small(s, dq, 1, QKV, l->mid_q, s->QKVX, 1, gB_q, R, NULL, s->Hq_hd, R, M, sc);
            gemm_small(s, tmp_q, 1, DX, l->ln1, s->D, 1, gA_q, s->D, NULL, R, s->D, M, 1.0f);
            gemm_small(s, dv, 1, QKV, l->mid_v, s->QKVX, 1, gB_v, R, NULL, s->Hkv_hd, R, M, sc);
            gemm_small(s, tmp_v, 1, DX, l->ln1, s->D, 1, gA_v, s->D, NULL, R, s->D, M, 1.0f);
        }
        /* d_ln += tmp_q A_q + tmp_v A_v (:951-953, :966, :970): one product over the 2R packed rows of the weight */
        if (R == 0) {
        } else if (s->use_tc) {                       /* the packed rows are binary16 there: take A_q, A_v from the LoRA vector */
            gemm_small(s, tmp_q, DX, 1, pA_q, s->D, 1, s->d_lnx, DX, s->d_lnx, M, s->D, R, 1.0f);
            gemm_small(s, tmp_v, DX, 1, pA_v, s->D, 1, s->d_lnx, DX, s->d_lnx, M, s->D, R, 1.0f);
        } else {
            gemm_small(s, tmp_q, DX, 1, l->qkv.w + (size_t)QKV * s->D, s->D, 1, s->d_lnx, DX, s->d_lnx, M, s->D, 2 * R, 1.0f);
        }
        /* input norm + residual + clamp (:974-979) */
        S_TRY(s, b200_rms_norm_bwd_rows_h(l->x_in, s->d_lnx, DX, l->g_in, s->dx, M, s->D, s->eps, 1, 1e6f, s->xh, hs, st));
    }
    /* the gradients of the first layer: whatever follows on the main stream (the optimizer, a read-back) waits for them */
    if (s->side_pending) { S_TRY(s, (int)cudaStreamWaitEvent(st, s->ev_join, 0)); s->side_pending = 0; }
}

/* ---------------------------------------------------------------- update */

static void update_device(SFTState *s, float lr, int step)
{
    if (s->n_lora == 0) return;                  /* a full-parameter state has no adapter to update */
    const float beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, wd = 0.01f;
    const float bc1 = 1.0f - powf(beta1, (float)step), bc2 = 1.0f - powf(beta2, (float)step);
    cudaStream_t st = g_rt.stream;
    cudaEventRecord(s->ev[2], st);
    S_TRY(s, b200_sumsq_partials(s->lora_g, s->n_lora, s->partials, N_PARTIALS, st));
    S_TRY(s, b200_clip_adamw(s->lora_p, s->lora_g, s->lora_m, s->lora_v, s->n_lora, s->partials, N_PARTIALS, 1.0f, lr,
                             beta1, beta2, eps, wd, bc1, bc2, 1, s->d_norm, st));
    cudaEventRecord(s->ev[3], st);
    S_TRY(s, (int)cudaMemcpyAsync(&s->h_loss[s->M], s->d_norm, 4, cudaMemcpyDeviceToHost, st));
    S_TRY(s, (int)cudaStreamSynchronize(st));
    s->last_norm = s->h_loss[s->M];
    cudaEventElapsedTime(&s->last_update_ms, s->ev[2], s->ev[3]);
}

static float mean_loss_host(SFTState *s)
{
    /* summed on the host in position order like the reference (:1142-1144) */
    S_TRY(s, (int)cudaMemcpyAsync(s->h_loss, s->losses, (size_t)s->M * 4, cudaMemcpyDeviceToHost, g_rt.stream));
    S_TRY(s, (int)cudaMemcpyAsync(&s->h_loss[s->M], s->d_norm + 1, 4, cudaMemcpyDeviceToHost, g_rt.stream));
    S_TRY(s, (int)cudaStreamSynchronize(g_rt.stream));
    unsigned gemm_err;
    memcpy(&gemm_err, &s->h_loss[s->M], 4);
    if (gemm_err && !s->err) {
        s->err = (int)gemm_err;
        fprintf(stderr, "[llmb200] sft: a tensor-core product gave up waiting (code 0x%x)\n", gemm_err);
    }
    float total = 0.f;
    for (int i = 0; i < s->M; ++i) total += s->h_loss[i];
    return total / (float)s->M;
}

float llmb200_sft_forward_backward(SFTState *s, const uint32_t *inputs, const uint32_t *targets)
{
    if (!s || !s->finished || !inputs || !targets) return NAN;
    if (s->err) return NAN;      /* after a failed pass (e.g. an aborted split product leaves its turn counters set) the state is dead */
    cudaStream_t st = g_rt.stream;
    memcpy(s->h_tok, inputs, (size_t)s->M * 4);
    memcpy(s->h_tok + s->M, targets, (size_t)s->M * 4);
    S_TRY(s, (int)cudaMemcpyAsync(s->tokens, s->h_tok, (size_t)s->M * 4, cudaMemcpyHostToDevice, st));
    S_TRY(s, (int)cudaMemcpyAsync(s->targets, s->h_tok + s->M, (size_t)s->M * 4, cudaMemcpyHostToDevice, st));
    cudaEventRecord(s->ev[0], st);
    if (s->step_graph_state == 1 && !s->err) {
        /* capture: nothing runs here, the launches only become nodes */
        s->step_graph_state = -1;
        const unsigned long long before = b200_launch_count(0);
        if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
            S_TRY(s, b200_embed_rows(s->d_emb, s->tokens, s->M, s->D, s->V, s->emb_scale, s->layers[0].x_in, st));
            forward_device(s);
            loss_device(s);
            backward_device(s);
            cudaGraph_t g = NULL;
            const cudaError_t ce = cudaStreamEndCapture(st, &g);
            if (ce == cudaSuccess && g && !s->err && cudaGraphInstantiate(&s->step_graph, g, 0) == cudaSuccess) {
                s->step_graph_kernels = b200_launch_count(0) - before;
                s->step_graph_state = 2;
            } else {
                (void)cudaGetLastError();
                s->err = 0;                      /* a launch refused under capture is not a failed step */
                fprintf(stderr, "[FastSFT] the step could not be captured as a CUDA graph; launching kernel by kernel\n");
            }
            if (g) cudaGraphDestroy(g);
        } else (void)cudaGetLastError();
        /* the capture advanced the count without launching anything */
        b200_launch_count_add(0ull - (b200_launch_count(0) - before));
    }
    if (s->step_graph_state == 2) {
        S_TRY(s, (int)cudaGraphLaunch(s->step_graph, st));
        b200_launch_count_add(s->step_graph_kernels);
        s->xh_has_dlogits = 0;
    } else {
        S_TRY(s, b200_embed_rows(s->d_emb, s->tokens, s->M, s->D, s->V, s->emb_scale, s->layers[0].x_in, st));
        forward_device(s);
        loss_device(s);
        backward_device(s);
        if (s->step_graph_state == 0) s->step_graph_state = getenv("LLMB200_SFT_NO_GRAPH") ? -1 : 1;
    }
    cudaEventRecord(s->ev[1], st);
    const float loss = mean_loss_host(s);
    cudaEventElapsedTime(&s->last_step_ms, s->ev[0], s->ev[1]);
    return s->err ? NAN : loss;
}

void llmb200_sft_apply_update(SFTState *s, float lr)
{
    if (!s || !s->finished) return;
    s->step_count++;
    update_device(s, lr, s->step_count);
}

float llmb200_sft_train_batch(SFTState *s, const uint32_t *inputs, const uint32_t *targets, float lr)
{
    if (s && s->full_param) {
        /* full-parameter step (:1136-1137): the weights move inside the backward pass; no optimizer state, no step count */
        s->wmode = s->acc_lm ? 2 : 1;             /* with accumulators allocated the reference's step accumulates (:778-785) */
        s->sgd_lr = lr;
        const float l = llmb200_sft_forward_backward(s, inputs, targets);
        s->wmode = 0;
        return l;
    }
    const float loss = llmb200_sft_forward_backward(s, inputs, targets);
    /* A failed pass (a device wait gave up, a launch failed) or a loss that is not finite leaves partial
     * gradients: the parameters, the Adam moments and the step count stay as they were. */
    if (!s || s->err || !isfinite(loss)) {
        if (s) fprintf(stderr, "[llmb200] sft: step skipped (error %d, loss %g); LoRA parameters unchanged\n", s->err, loss);
        return loss;
    }
    llmb200_sft_apply_update(s, lr);
    return loss;
}

float sft_train_step(SFTState *s, const uint32_t *input_tokens, const uint32_t *target_tokens, float lr)
{
    return llmb200_sft_train_batch(s, input_tokens, target_tokens, lr);
}

void forward_to_logits(SFTState *s)
{
    if (!s || !s->finished) return;
    /* the caller wrote the embeddings into the shared x buffer */
    S_TRY(s, (int)cudaMemcpyAsync(s->layers[0].x_in, s->x_shared, (size_t)s->M * s->D * 4, cudaMemcpyDefault,
                                  g_rt.stream));
    forward_device(s);
}

void sft_backward(SFTState *s)
{
    if (!s || !s->finished) return;
    s->wmode = 0;                 /* a full-parameter state: the reference steps with lr = 0 here, which changes nothing */
    backward_device(s);
}

void sft_lora_update(SFTState *s, float lr)
{
    /* The reference clips here and once more inside lora_update (:1248-1251, :1094); the second
     * clip sees a norm of 1 and changes nothing beyond rounding, so one clip is applied. */
    if (!s || !s->finished) return;
    update_device(s, lr, s->step_count);
}

/* ---------------------------------------------------------------- Gemma3 and full-parameter modes */

/* Gemma3 (src/nn/fast_sft.c:284-396 LoRA, :507-610 full-parameter): four norms per layer, GeGLU, embeddings scaled by
 * sqrt(d_model), the LM head a binary16 copy of the embedding table, the RoPE base per layer by position in the
 * stack (every sixth layer global, the others local: :310-313). fp32 path. */
static SFTState *create_from_gemma3(llmb200_gemma3_model *m, int seq_len, int lora_rank, float lora_alpha, int full_param)
{
    if (!m) return NULL;
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    printf(full_param ? "[FastSFT] Converting Gemma3 weights to F16 (full-param)...\n" : "[FastSFT] Converting Gemma3 weights to F16...\n");
    llmb200_config cfg = { MODEL_GEMMA3, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                           m->vocab_size, m->n_layers, seq_len, 1 };
    SFTState *s = sft_begin(&cfg, seq_len, 1, lora_rank, lora_alpha, full_param);
    if (!s) return NULL;
    s->step_graph_state = -1;                    /* the fp32 path is launched kernel by kernel */
    const int Hq_hd = s->Hq_hd, Hkv_hd = s->Hkv_hd;
    for (int i = 0; i < s->NL; ++i) {
        llmb200_gemma3_block *b = m->blocks[i];
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
        r.pre_ff_norm_g = b->pre_ff_norm->gamma->data;
        r.post_ff_norm_g = b->post_ff_norm->gamma->data;
        r.q_norm_g = b->attn->q_norm->gamma->data;
        r.k_norm_g = b->attn->k_norm->gamma->data;
        r.d_model = s->D;
        r.head_dim = s->hd;
        const float *lora[4] = { NULL, NULL, NULL, NULL };
        if (!full_param && m->q_loras && m->q_loras[i]) { lora[0] = m->q_loras[i]->lora_A->data; lora[1] = m->q_loras[i]->lora_B->data; }
        if (!full_param && m->v_loras && m->v_loras[i]) { lora[2] = m->v_loras[i]->lora_A->data; lora[3] = m->v_loras[i]->lora_B->data; }
        const float theta = (i % 6) != 0 ? m->local_rope_theta : m->global_rope_theta;
        if (llmb200_sft_load_layer(s, i, &r, theta, lora) != 0) { sft_state_free(s); return NULL; }
    }
    if (llmb200_sft_finish(s, m->token_emb->weight->data, m->final_norm->gamma->data, m->token_emb->weight->data, 1) != 0) {
        sft_state_free(s);
        return NULL;
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (t1.tv_sec - t0.tv_sec) * 1000.0 + (t1.tv_nsec - t0.tv_nsec) / 1e6;
    if (full_param) printf("[FastSFT] Gemma3 Full-param Init: %.0f ms, seq=%d\n", ms, seq_len);
    else printf("[FastSFT] Gemma3 Init: %.0f ms, seq=%d, lora_rank=%d\n", ms, seq_len, lora_rank);
    return s;
}

SFTState *sft_state_create_gemma3(llmb200_gemma3_model *model, int seq_len, int lora_rank, float lora_alpha)
{
    return create_from_gemma3(model, seq_len, lora_rank, lora_alpha, 0);
}

SFTState *sft_state_create_gemma3_full(llmb200_gemma3_model *model, int seq_len)
{
    return create_from_gemma3(model, seq_len, 0, 0.0f, 1);
}

int sft_is_full_param(SFTState *s) { return s ? s->full_param : 0; }                       /* src/nn/fast_sft.c:987 */

static int full_only(SFTState *s, const char *what)
{
    if (s && s->finished && s->full_param) return 1;
    fprintf(stderr, "[FastSFT] %s: not a full-parameter state\n", what);
    return 0;
}

/* Backward from the gradient in sft_get_dlogits() with every weight stepped as its gradient is formed
 * (sft_backward_ex with a learning rate, :766-982). */
void sft_backward_sgd(SFTState *s, float lr)
{
    if (!full_only(s, "sft_backward_sgd")) return;
    s->wmode = s->acc_lm ? 2 : 1;                 /* as above: accumulators, once allocated, take every gradient */
    s->sgd_lr = lr;
    backward_device(s);
    s->wmode = 0;
}

/* Accumulators for every matrix, zeroed (:996-1019); binary16 values, like the reference's F16 buffers. */
void sft_alloc_grad_accum(SFTState *s)
{
    if (!full_only(s, "sft_alloc_grad_accum") || s->acc_lm) return;
    size_t total = 0;
    for (int L = 0; L < s->NL; ++L) {
        SftLayer *l = &s->layers[L];
        const SftMat *ms[4] = { &l->qkv, &l->o, &l->gu, &l->down };
        for (int i = 0; i < 4; ++i) {
            const size_t n = (size_t)(i == 0 ? s->QKV : ms[i]->rows) * ms[i]->cols;
            l->acc[i] = dalloc(s, n);
            if (l->acc[i]) cudaMemsetAsync(l->acc[i], 0, n * 4, g_rt.stream);
            total += n;
        }
    }
    s->acc_lm = dalloc(s, (size_t)s->V * s->D);
    if (s->acc_lm) cudaMemsetAsync(s->acc_lm, 0, (size_t)s->V * s->D * 4, g_rt.stream);
    total += (size_t)s->V * s->D;
    printf("[FastSFT] Grad accum buffers allocated: %.2f MB\n", (float)(total * 2) / (1024.0f * 1024.0f));
}

/* Backward that adds every weight gradient into its accumulator and leaves the weights alone (:986). */
void sft_backward_accum(SFTState *s)
{
    if (!full_only(s, "sft_backward_accum")) return;
    s->wmode = s->acc_lm ? 2 : 1;                 /* without accumulators the reference steps with lr = 0: nothing changes */
    s->sgd_lr = 0.0f;
    backward_device(s);
    s->wmode = 0;
}

/* W <- half(W - lr G), G <- 0 for every matrix (:1021-1039). */
void sft_apply_grad_sgd(SFTState *s, float lr)
{
    if (!full_only(s, "sft_apply_grad_sgd") || !s->acc_lm) return;
    cudaStream_t st = g_rt.stream;
    for (int L = 0; L < s->NL; ++L) {
        SftLayer *l = &s->layers[L];
        SftMat *ms[4] = { &l->qkv, &l->o, &l->gu, &l->down };
        for (int i = 0; i < 4; ++i)
            S_TRY(s, b200_sgd_apply_f16(ms[i]->w, l->acc[i], (size_t)(i == 0 ? s->QKV : ms[i]->rows) * ms[i]->cols, lr, st));
        S_TRY(s, mat_finish_rows(s, &l->qkv, s->QKV));
    }
    S_TRY(s, b200_sgd_apply_f16(s->lm_head.w, s->acc_lm, (size_t)s->V * s->D, lr, st));
    s->weights_version++;
}

/* Header of nine 32-bit words, then per layer q, k, v, o, gate, up, down and at the end the LM head, each as
 * row-major binary16 (:1287-1343). */
void sft_save_full_checkpoint(SFTState *s, const char *path)
{
    if (!s || !s->finished || !path) return;
    FILE *fp = fopen(path, "wb");
    if (!fp) {
        fprintf(stderr, "[FastSFT] Failed to open %s for writing\n", path);
        return;
    }
    LayerW *lw = sft_get_layers(s);
    WMat *lm = sft_get_lm_head(s);
    if (!lw || !lm) { fclose(fp); fprintf(stderr, "[FastSFT] reading the weights back failed\n"); return; }
    share_refresh(s);
    const uint32_t head[9] = { 0x46554C4Cu, (uint32_t)s->model_type, (uint32_t)s->NL, (uint32_t)s->D, (uint32_t)s->Hq,
                               (uint32_t)s->Hkv, (uint32_t)s->hd, (uint32_t)s->IS, (uint32_t)s->V };
    fwrite(head, 4, 9, fp);
    size_t total = 0;
    for (int L = 0; L < s->NL; ++L) {
        WMat *ws[7] = { lw[L].q_proj, lw[L].k_proj, lw[L].v_proj, lw[L].o_proj, lw[L].gate_proj, lw[L].up_proj, lw[L].down_proj };
        for (int i = 0; i < 7; ++i) {
            const size_t bytes = (size_t)ws[i]->rows * ws[i]->cols * 2;
            const void *h = metal_buf_ptr(ws[i]->mbuf);
            if (h) fwrite(h, 1, bytes, fp);
            total += bytes;
        }
    }
    const size_t lm_bytes = (size_t)s->V * s->D * 2;
    const void *h = metal_buf_ptr(lm->mbuf);
    if (h) fwrite(h, 1, lm_bytes, fp);
    total += lm_bytes;
    fclose(fp);
    printf("[FastSFT] Full checkpoint saved to %s (%.2f MB)\n", path, (float)total / (1024.0f * 1024.0f));
}
/* ---------------------------------------------------------------- accessors */

MetalBuf *sft_get_logits(SFTState *s) { return s ? s->mb_logits : NULL; }
MetalBuf *sft_get_dlogits(SFTState *s) { return s ? s->mb_dlogits : NULL; }
float *sft_get_x_cpu(SFTState *s) { if (!s) return NULL; metal_flush(); return s->x_shared; }
float *sft_get_losses_cpu(SFTState *s)
{
    if (!s) return NULL;
    cudaMemcpyAsync(s->losses_shared, s->losses, (size_t)s->M * 4, cudaMemcpyDefault, g_rt.stream);
    metal_flush();
    return s->losses_shared;
}
int sft_get_seq_len(SFTState *s) { return s->N; }
int sft_get_vocab_size(SFTState *s) { return s->V; }
int sft_get_d_model(SFTState *s) { return s->D; }
int sft_get_lora_rank(SFTState *s) { return s->lora_rank; }
int sft_get_n_layers(SFTState *s) { return s->NL; }
float sft_get_emb_scale(SFTState *s) { return s->emb_scale; }
const float *sft_get_token_emb(SFTState *s) { return s->token_emb_host; }
int sft_get_step_count(SFTState *s) { return s->step_count; }
void sft_set_step_count(SFTState *s, int step) { s->step_count = step; }
int sft_get_n_lora_grad_bufs(SFTState *s) { return s->NL * 4; }
float sft_get_lora_scaling(SFTState *s) { return s->lora_scaling; }

float *sft_get_lora_grad_ptr(SFTState *s, int idx, int *out_size)
{
    if (!s || idx < 0 || idx >= s->NL * 4) return NULL;
    const int L = idx / 4, sub = idx % 4;
    const size_t off = s->layers[L].lora_off + s->sub_off[sub];
    if (out_size) *out_size = (int)s->sizes[sub];
    cudaMemcpyAsync(s->h_grad + off, s->lora_g + off, s->sizes[sub] * 4, cudaMemcpyDeviceToHost, g_rt.stream);
    metal_flush();
    return s->h_grad + off;
}

void sft_set_lora_grad(SFTState *s, int idx, const float *data, int size)
{
    if (!s || !data || idx < 0 || idx >= s->NL * 4) return;
    const int L = idx / 4, sub = idx % 4;
    if (size < 0 || (size_t)size > s->sizes[sub]) return;
    const size_t off = s->layers[L].lora_off + s->sub_off[sub];
    if (data != s->h_grad + off) memcpy(s->h_grad + off, data, (size_t)size * 4);
    cudaMemcpyAsync(s->lora_g + off, s->h_grad + off, (size_t)size * 4, cudaMemcpyHostToDevice, g_rt.stream);
    metal_flush();
}

MetalBuf *sft_get_lora_weight_buf(SFTState *s, int layer, int sub)
{
    if (!s || layer < 0 || layer >= s->NL || sub < 0 || sub > 3) return NULL;
    SftLayer *l = &s->layers[layer];
    if (!l->lora_buf[sub])
        l->lora_buf[sub] = llmb200_buf_wrap(s->lora_p + l->lora_off + s->sub_off[sub], s->sizes[sub] * 4);
    return l->lora_buf[sub];
}

static float *lora_params_host(SFTState *s)
{
    float *h = malloc(s->n_lora * sizeof(float));
    if (!h) return NULL;
    metal_flush();
    if (cudaMemcpy(h, s->lora_p, s->n_lora * 4, cudaMemcpyDeviceToHost) != cudaSuccess) { free(h); return NULL; }
    return h;
}

void sft_save_lora(SFTState *s, const char *path)
{
    if (!s || !path) return;
    FILE *fp = fopen(path, "wb");
    if (!fp) {
        fprintf(stderr, "[FastSFT] Failed to open %s for writing\n", path);
        return;
    }
    float *h = lora_params_host(s);
    if (!h) { fclose(fp); fprintf(stderr, "[FastSFT] reading the LoRA weights back failed\n"); return; }
    const uint32_t magic = 0x4C4F5241u;
    const int32_t n_layers = s->NL, rank = s->lora_rank;
    fwrite(&magic, 4, 1, fp);
    fwrite(&n_layers, 4, 1, fp);
    fwrite(&rank, 4, 1, fp);
    fwrite(h, sizeof(float), s->n_lora, fp);        /* the flat vector is already in file order */
    fclose(fp);
    free(h);
    printf("[FastSFT] LoRA saved to %s (rank=%d, %.2f MB)\n", path, rank,
           (float)(s->n_lora * sizeof(float)) / (1024.0f * 1024.0f));
}

void sft_sync_lora_to_model(SFTState *s, llmb200_qwen3_model *m)
{
    if (!s || !m || !m->q_loras || !m->v_loras) return;
    float *h = lora_params_host(s);
    if (!h) return;
    for (int L = 0; L < s->NL; ++L) {
        const float *base = h + s->layers[L].lora_off;
        if (m->q_loras[L]) {
            memcpy(m->q_loras[L]->lora_A->data, base + s->sub_off[0], s->sizes[0] * 4);
            memcpy(m->q_loras[L]->lora_B->data, base + s->sub_off[1], s->sizes[1] * 4);
        }
        if (m->v_loras[L]) {
            memcpy(m->v_loras[L]->lora_A->data, base + s->sub_off[2], s->sizes[2] * 4);
            memcpy(m->v_loras[L]->lora_B->data, base + s->sub_off[3], s->sizes[3] * 4);
        }
    }
    free(h);
}

void sft_sync_lora_to_gemma3(SFTState *s, llmb200_gemma3_model *m)                          /* src/nn/fast_sft.c:1184-1206 */
{
    if (!s || !m || !m->q_loras || !m->v_loras || !s->n_lora) return;
    float *h = lora_params_host(s);
    if (!h) return;
    for (int L = 0; L < s->NL; ++L) {
        const float *base = h + s->layers[L].lora_off;
        if (m->q_loras[L]) {
            memcpy(m->q_loras[L]->lora_A->data, base + s->sub_off[0], s->sizes[0] * 4);
            memcpy(m->q_loras[L]->lora_B->data, base + s->sub_off[1], s->sizes[1] * 4);
        }
        if (m->v_loras[L]) {
            memcpy(m->v_loras[L]->lora_A->data, base + s->sub_off[2], s->sizes[2] * 4);
            memcpy(m->v_loras[L]->lora_B->data, base + s->sub_off[3], s->sizes[3] * 4);
        }
    }
    free(h);
}

size_t llmb200_sft_grad_vector(SFTState *s, void **p) { if (!s) return 0; if (p) *p = s->lora_g; return s->n_lora; }
size_t llmb200_sft_param_vector(SFTState *s, void **p) { if (!s) return 0; if (p) *p = s->lora_p; return s->n_lora; }
float llmb200_sft_last_grad_norm(SFTState *s) { return s ? s->last_norm : NAN; }
float llmb200_sft_last_step_ms(SFTState *s, float *update_ms)
{
    if (!s) return -1.f;
    if (update_ms) *update_ms = s->last_update_ms;
    return s->last_step_ms;
}
int llmb200_sft_use_tensor_cores(SFTState *s, int on)
{
    if (!s) return 0;
    /* the weights are stored for one mode or the other when the state is created */
    (void)on;
    return s->use_tc;
}
int llmb200_sft_error(SFTState *s) { return s ? s->err : -1; }

size_t llmb200_sft_export(SFTState *s, int what, int layer, float *dst, size_t cap)
{
    if (!s || !dst) return 0;
    const float *src = NULL;
    size_t n = 0;
    const size_t M = s->M;
    if (what < 100) {
        if (layer < 0 || layer >= s->NL) return 0;
        SftLayer *l = &s->layers[layer];
        switch (what) {
        case LLMB200_SFT_X_IN: src = l->x_in; n = M * s->D; break;
        case LLMB200_SFT_LN1: src = l->ln1; n = M * s->D; break;
        case LLMB200_SFT_QKV: src = l->qkv_out; n = M * s->QKVX; break;
        case LLMB200_SFT_Q_FINAL: src = l->q_f; n = M * s->Hq_hd; break;
        case LLMB200_SFT_K_FINAL: src = l->k_f; n = M * s->Hkv_hd; break;
        case LLMB200_SFT_PROBS: src = l->probs; n = (size_t)s->S * s->Hq * s->N * s->N; break;
        case LLMB200_SFT_X_MID: src = l->x_mid; n = M * s->D; break;
        case LLMB200_SFT_LN2: src = l->ln2; n = M * s->D; break;
        case LLMB200_SFT_GATE_UP: src = l->gu_out; n = M * 2 * s->IS; break;
        case LLMB200_SFT_MID_Q:
        case LLMB200_SFT_MID_V:
            n = M * s->lora_rank;
            if (n > cap) return 0;
            metal_flush();
            if (cudaMemcpy2D(dst, (size_t)s->lora_rank * 4, what == LLMB200_SFT_MID_Q ? l->mid_q : l->mid_v,
                             (size_t)s->QKVX * 4, (size_t)s->lora_rank * 4, M, cudaMemcpyDeviceToHost) != cudaSuccess)
                return 0;
            return n;
        default: return 0;
        }
    } else {
        switch (what) {
        case LLMB200_SFT_LOGITS: src = s->logits; n = M * s->V; break;
        case LLMB200_SFT_DLOGITS: src = s->dlogits; n = M * s->V; break;
        case LLMB200_SFT_LOSSES: src = s->losses; n = M; break;
        case LLMB200_SFT_X_FINAL: src = s->x_final; n = M * s->D; break;
        case LLMB200_SFT_LORA_GRADS: src = s->lora_g; n = s->n_lora; break;
        case LLMB200_SFT_LORA_PARAMS: src = s->lora_p; n = s->n_lora; break;
        default: return 0;
        }
    }
    if (n > cap) return 0;
    metal_flush();
    if (cudaMemcpy(dst, src, n * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    return n;
}
