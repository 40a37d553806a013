/*
 * Decode engine of libllmb200 (host side, C): persistent state, the per-token
 * CUDA graph and the greedy generate loop.
 *
 * Stands in for src/nn/fast_inference.c of llm.metal: InferenceState (:58-95),
 * inference_state_init_common (:171-275), forward_token (:376-467) and
 * inference_generate (:614-675). What the reference enqueues as 17 (Qwen3) or
 * 19 (Gemma3) barrier-separated dispatches per layer becomes five launches:
 *
 *   qkv     embedding / residual assembly + RMSNorm + fused Q|K|V matvec
 *   attn    QK-norm + RoPE + KV store + split-sequence attention (F16 cache)
 *   o       O matvec into this rank's all-reduce slot on every peer
 *   gateup  slot sum + residual + RMSNorm + interleaved gate/up matvec + SiLU/GELU*up
 *   down    down matvec into the second all-reduce slot
 *
 * and the LM head launch does final norm + matvec + greedy argmax, so the next
 * token id never leaves the device. The whole token is one CUDA graph whose
 * nodes are chained by programmatic dependent launch; position, token ids and
 * the tensor-parallel epoch live in device memory, so the same graph is
 * replayed for every position.
 *
 * Tensor parallelism (one process per GPU): matrices are sliced at upload
 * (rows of Q/K/V, gate, up, LM head; input columns of O and down; every cut a
 * multiple of 32, so Q8_0 blocks are those of the unsharded quantisation), the
 * O and down kernels store their partial vectors straight into every peer's
 * slot over NVLink and raise a flag, and the consumer kernel sums the slots in
 * rank order -- the all-reduce is the epilogue of one kernel and the prologue
 * of the next.
 */
#include "internal.h"
#include "../../include/llmb200_inference.h"
#include "../../include/llmb200_sft.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>

typedef struct { void *w; long long stride; int rows, cols; } PackedMat;

typedef struct {
    PackedMat qkv, o, gateup, down;
    float *g_input, *g_post_attn, *g_pre_ff, *g_post_ff, *g_qn, *g_kn;
    float *inv_freq;
    float rope_theta;
    const float *rope;       /* this layer's table in InferenceState.rope_tab (whole-token kernel) */
    void *k_cache, *v_cache;
    int loaded;
} Layer;

enum { K_QKV = 0, K_ATTN, K_O, K_GATEUP, K_DOWN, K_LM, K_KINDS };

struct InferenceState {
    int D, Hq, Hkv, hd, IS, V, L, max_seq, use_fp16, wtype;
    ModelType mt;
    int tp_rank, tp_size, Hq_l, Hkv_l, IS_l, V_l;
    float emb_scale;
    int eos[4], n_eos;

    Layer *layers;
    PackedMat lm;
    float *g_final, *emb;
    int finished;
    unsigned long long weight_bytes;

    /* activations and scratch (device) */
    float *resid[2], *qkv, *attn_out, *act, *attn_scratch, *am_scratch;
    unsigned *attn_tickets, *mv_ticket;
    int n_split;

    /* control words (device): pos, prompt_len, err, epoch, tokens[max_seq+2] */
    int *d_pos, *d_prompt_len, *d_err, *d_tokens;
    unsigned *d_epoch;

    /* all-reduce region, shared with the peers */
    char *comm;
    size_t comm_bytes, off_slots_o, off_slots_dn, off_flags, off_am_val, off_am_idx, off_logits;
    char *peer[B200_MAX_PEERS];
    int connected, loopback;
    /* single-process tensor parallelism (LLMB200_TP=k): the handle a caller holds is rank 0's state */
    int group_n, group_dev[B200_MAX_PEERS], local_peers;
    struct InferenceState *group[B200_MAX_PEERS];

    /* host side */
    float *h_logits;
    int *h_tok;              /* pinned ring for generated ids */
    int *h_ctl;              /* pinned staging for control writes */
    cudaEvent_t tok_ev[4];
    cudaEvent_t ev_a, ev_b;
    cudaGraphExec_t g_full, g_nolm;
    int kernels_full, kernels_nolm;   /* kernel nodes per graph */
    int use_pdl;
    /* LoRA adapter attached with inference_state_set_lora: device pointers into the SFT state's vectors */
    struct { const float *A_q, *B_q, *A_v, *B_v; } *lora;
    int lora_rank;
    float lora_scaling;
    SFTState *sft_src;                    /* the SFT state whose matrices this state copied, or NULL */
    unsigned long long sft_version;       /* its weights_version at the time of the copy */
    float *xnorm;            /* [D]: the normalised layer input, kept by the q/k/v matvec for the LoRA kernel */
    int cur_len;
    double last_decode_ms, last_prefill_ms;
    int last_n_decoded;

    /* instrumentation */
    cudaEvent_t *prof_ev;
    int prof_n, prof_cap, prof_on;
    /* whole-token kernel: layer table on the device, flagged hand-over vectors, launch arguments */
    b200_token_layer *d_tk_layers;
    float *rope_tab[8];      /* rotation tables, one per distinct RoPE base */
    int n_rope_tab;
    b200_flagged *fl_qkv, *fl_part, *fl_attn, *fl_act, *fl_am;
    size_t off_fl_slots_o, off_fl_slots_dn, off_fl_am, off_counters;
    b200_token_args tk;              /* planned arguments; with_lm is set per launch */
    int fused, tk_planned, n_sm;
    unsigned long long *d_step_ns;   /* stage trace of the whole-token kernel (LLMB200_TRACE=1) */
    int only_kind;           /* >= 0: enqueue_token launches only this kind of kernel (timing loops) */
    int *prof_kind;
};

/* per host thread: the ranks of a single-process group are threads */
static __thread int g_tp_rank = -1, g_tp_size = -1;

int llmb200_set_tp(int rank, int world)
{
    if (world < 1 || world > B200_MAX_PEERS || rank < 0 || rank >= world) return B200_E_BADARG;
    g_tp_rank = rank; g_tp_size = world;
    return 0;
}

static void tp_from_env(int *rank, int *world)
{
    *rank = 0; *world = 1;
    if (g_tp_size > 0) { *rank = g_tp_rank; *world = g_tp_size; return; }
    const char *w = getenv("LLMB200_TP_SIZE"), *r = getenv("LLMB200_TP_RANK");
    if (w && r && atoi(w) >= 1 && atoi(w) <= B200_MAX_PEERS && atoi(r) >= 0 && atoi(r) < atoi(w)) {
        *world = atoi(w); *rank = atoi(r);
    }
}

static double now_ms(void)
{
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return t.tv_sec * 1000.0 + t.tv_nsec / 1e6;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

/* ------------------------------------------------------------ allocation */

static int alloc_mat(PackedMat *m, int wtype, int rows, int cols)
{
    m->rows = rows; m->cols = cols;
    m->stride = (long long)b200_packed_row_stride(wtype, cols);
    CU_TRY(cudaMalloc(&m->w, (size_t)m->stride * (size_t)rows), return -1);
    return 0;
}

static float *dev_zero(size_t bytes)
{
    void *p = NULL;
    CU_TRY(cudaMalloc(&p, bytes ? bytes : 4), return NULL);
    CU_TRY(cudaMemsetAsync(p, 0, bytes ? bytes : 4, g_rt.stream), { cudaFree(p); return NULL; });
    return (float *)p;
}

InferenceState *llmb200_state_begin(const llmb200_config *c)
{
    if (!c || c->d_model <= 0 || c->n_layers <= 0 || c->n_q_heads <= 0 || c->n_kv_heads <= 0 ||
        c->head_dim <= 0 || c->intermediate_size <= 0 || c->vocab_size <= 0 || c->max_seq_len <= 0) {
        fprintf(stderr, "[FastGen] invalid model configuration\n");
        return NULL;
    }
    if (fast_metal_init() != 0) {
        fprintf(stderr, "[FastGen] CUDA init failed\n");
        return NULL;
    }
    int max_seq = c->max_seq_len;
    if (max_seq > 4096) {
        fprintf(stderr, "[FastGen] Warning: clamping max_seq_len to 4096 (kernel limit)\n");
        max_seq = 4096;
    }
    InferenceState *s = calloc(1, sizeof(*s));
    if (!s) { fast_metal_shutdown(); return NULL; }
    s->D = c->d_model; s->Hq = c->n_q_heads; s->Hkv = c->n_kv_heads; s->hd = c->head_dim;
    s->IS = c->intermediate_size; s->V = c->vocab_size; s->L = c->n_layers; s->max_seq = max_seq;
    s->use_fp16 = c->use_fp16 ? 1 : 0;
    s->wtype = s->use_fp16 ? B200_WT_F16 : B200_WT_Q8;
    s->mt = c->model_type == MODEL_GEMMA3 ? MODEL_GEMMA3 : MODEL_QWEN3;
    s->emb_scale = s->mt == MODEL_GEMMA3 ? sqrtf((float)s->D) : 1.0f;
    if (s->mt == MODEL_GEMMA3) { s->eos[0] = 1; s->eos[1] = 106; s->n_eos = 2; }
    else { s->eos[0] = 151645; s->eos[1] = 151643; s->n_eos = 2; }
    tp_from_env(&s->tp_rank, &s->tp_size);
    const int k = s->tp_size;
    const int align = s->wtype == B200_WT_Q8 ? 32 : 8;
    if (s->Hkv % k || s->Hq % k || s->IS % k || s->V % k || (s->IS / k) % align || (s->Hq / k * s->hd) % align ||
        s->D % align || (s->hd != 64 && s->hd != 128 && s->hd != 256) ||
        (s->Hq / s->Hkv != 1 && s->Hq / s->Hkv != 2 && s->Hq / s->Hkv != 4 && s->Hq / s->Hkv != 8) || s->Hq % s->Hkv) {
        fprintf(stderr, "[FastGen] unsupported shape for %d-way tensor parallelism (heads %d/%d, head_dim %d, ffn %d, vocab %d)\n",
                k, s->Hq, s->Hkv, s->hd, s->IS, s->V);
        free(s); fast_metal_shutdown();
        return NULL;
    }
    s->Hq_l = s->Hq / k; s->Hkv_l = s->Hkv / k; s->IS_l = s->IS / k; s->V_l = s->V / k;

    s->layers = calloc((size_t)s->L, sizeof(Layer));
    if (!s->layers) goto fail;
    const int qkv_rows = (s->Hq_l + 2 * s->Hkv_l) * s->hd;
    const size_t cache_bytes = (size_t)s->Hkv_l * max_seq * s->hd * 2;
    for (int i = 0; i < s->L; ++i) {
        Layer *ly = &s->layers[i];
        if (alloc_mat(&ly->qkv, s->wtype, qkv_rows, s->D) || alloc_mat(&ly->o, s->wtype, s->D, s->Hq_l * s->hd) ||
            alloc_mat(&ly->gateup, s->wtype, 2 * s->IS_l, s->D) || alloc_mat(&ly->down, s->wtype, s->D, s->IS_l))
            goto fail;
        ly->k_cache = dev_zero(cache_bytes);
        ly->v_cache = dev_zero(cache_bytes);
        if (!ly->k_cache || !ly->v_cache) goto fail;
        s->weight_bytes += (unsigned long long)ly->qkv.stride * ly->qkv.rows + (unsigned long long)ly->o.stride * ly->o.rows +
                           (unsigned long long)ly->gateup.stride * ly->gateup.rows + (unsigned long long)ly->down.stride * ly->down.rows;
    }
    if (alloc_mat(&s->lm, s->wtype, s->V_l, s->D)) goto fail;
    s->weight_bytes += (unsigned long long)s->lm.stride * s->lm.rows;

    if (cudaDeviceGetAttribute(&s->n_sm, cudaDevAttrMultiProcessorCount, g_rt.device) != cudaSuccess || s->n_sm <= 0) {
        fprintf(stderr, "[FastGen] cannot read the multiprocessor count\n");
        goto fail;
    }
    /* sequence splits: enough blocks to cover the GPU, at least 32 cache rows each at full length */
    s->n_split = s->n_sm / s->Hkv_l;
    {   /* the merge folds one batch of splits without predicates: 18, or 9 where a thread owns two outputs */
        const int batch = (s->Hq_l / s->Hkv_l) * s->hd > 512 ? 9 : 18;
        if (s->n_split > batch) s->n_split = batch;
    }
    const char *sp = getenv("LLMB200_ATT_SPLITS");                /* experiments */
    if (sp && atoi(sp) > 0 && atoi(sp) <= 64) s->n_split = atoi(sp);
    if (s->n_split > (max_seq + 31) / 32) s->n_split = (max_seq + 31) / 32;    /* at least 32 cache rows per split */
    if (s->n_split < 1) s->n_split = 1;

    s->resid[0] = dev_zero((size_t)s->D * 4);
    s->resid[1] = dev_zero((size_t)s->D * 4);
    s->qkv = dev_zero((size_t)qkv_rows * 4);
    s->attn_out = dev_zero((size_t)s->Hq_l * s->hd * 4);
    s->act = dev_zero((size_t)s->IS_l * 4);
    s->attn_scratch = dev_zero(b200_attn_scratch_floats(s->Hq_l, s->hd, s->n_split) * 4);
    s->am_scratch = dev_zero((size_t)2 * s->n_sm * 32 * 4);
    s->attn_tickets = (unsigned *)dev_zero((size_t)s->Hkv_l * 4);
    s->mv_ticket = (unsigned *)dev_zero(4);
    int *ctl = (int *)dev_zero((size_t)(8 + max_seq + 2) * 4);
    if (!s->resid[0] || !s->resid[1] || !s->qkv || !s->attn_out || !s->act || !s->attn_scratch || !s->am_scratch ||
        !s->attn_tickets || !s->mv_ticket || !ctl)
        goto fail;
    s->d_pos = ctl; s->d_prompt_len = ctl + 1; s->d_err = ctl + 2; s->d_epoch = (unsigned *)(ctl + 3);
    s->d_tokens = ctl + 8;

    /* all-reduce region: [slots_o 8xD][slots_dn 8xD][flags 3x8][am_val 8][am_idx 8][logits V] */
    size_t off = 0;
    s->off_slots_o = off;  off += align_up((size_t)B200_MAX_PEERS * s->D * 4, 256);
    s->off_slots_dn = off; off += align_up((size_t)B200_MAX_PEERS * s->D * 4, 256);
    s->off_flags = off;    off += 256;
    s->off_am_val = off;   off += 128;
    s->off_am_idx = off;   off += 128;
    s->off_logits = off;   off += align_up((size_t)s->V * 4, 256);
    /* flagged vectors of the whole-token kernel: [k][D] per exchange, (value, row) pair per rank */
    s->off_fl_slots_o = off;  off += align_up((size_t)B200_MAX_PEERS * s->D * 8, 256);
    s->off_fl_slots_dn = off; off += align_up((size_t)B200_MAX_PEERS * s->D * 8, 256);
    s->off_fl_am = off;       off += 256;
    s->off_counters = off;    off += (size_t)72 * B200_CNT_STRIDE * 4;   /* arrival counters, one 128-byte line each */
    s->comm_bytes = off;
    s->comm = (char *)dev_zero(off);
    if (!s->comm) goto fail;
    s->peer[s->tp_rank] = s->comm;
    s->connected = (k == 1);

    CU_TRY(cudaMallocHost((void **)&s->h_logits, (size_t)s->V * 4), goto fail);
    CU_TRY(cudaMallocHost((void **)&s->h_tok, 256), goto fail);    /* [0]: the first id; [8 ..]: four groups of ids read back */
    CU_TRY(cudaMallocHost((void **)&s->h_ctl, (size_t)(8 + max_seq + 2) * 4), goto fail);
    for (int i = 0; i < 4; ++i) CU_TRY(cudaEventCreateWithFlags(&s->tok_ev[i], cudaEventDisableTiming), goto fail);
    CU_TRY(cudaEventCreate(&s->ev_a), goto fail);
    CU_TRY(cudaEventCreate(&s->ev_b), goto fail);
    s->use_pdl = getenv("LLMB200_NO_PDL") ? 0 : 1;
    s->only_kind = -1;
    return s;
fail:
    inference_state_free(s);
    return NULL;
}

/* ------------------------------------------------------------ weights */

static float *upload_gamma(const float *g, int n) { return g ? llmb200_upload_f32(g, (size_t)n) : NULL; }

int llmb200_state_load_layer(InferenceState *s, int li, const LayerWeightRef *r, float rope_theta)
{
    if (!s || !r || li < 0 || li >= s->L) return B200_E_BADARG;
    const int D = s->D, hd = s->hd, k = s->tp_rank;
    const int Hq_hd = s->Hq * hd, Hkv_hd = s->Hkv * hd;
    if (r->q_proj.rows != Hq_hd || r->q_proj.cols != D || r->k_proj.rows != Hkv_hd || r->k_proj.cols != D ||
        r->v_proj.rows != Hkv_hd || r->v_proj.cols != D || r->o_proj.rows != D || r->o_proj.cols != Hq_hd ||
        r->gate_proj.rows != s->IS || r->gate_proj.cols != D || r->up_proj.rows != s->IS || r->up_proj.cols != D ||
        r->down_proj.rows != D || r->down_proj.cols != s->IS || !r->input_norm_g || !r->post_attn_norm_g) {
        fprintf(stderr, "[FastGen] layer %d: weight shapes do not match the configuration\n", li);
        return B200_E_BADARG;
    }
    Layer *ly = &s->layers[li];
    const int wt = s->wtype;
    const int ql = s->Hq_l * hd, kl = s->Hkv_l * hd, il = s->IS_l;
    int rc = 0;
    /* fused Q|K|V: this rank's query heads, then its key heads, then its value heads */
    rc |= llmb200_upload_packed(wt, r->q_proj.data + (size_t)k * ql * D, D, ql, 0, D, ly->qkv.w, ly->qkv.stride, 0, 1);
    rc |= llmb200_upload_packed(wt, r->k_proj.data + (size_t)k * kl * D, D, kl, 0, D, ly->qkv.w, ly->qkv.stride, ql, 1);
    rc |= llmb200_upload_packed(wt, r->v_proj.data + (size_t)k * kl * D, D, kl, 0, D, ly->qkv.w, ly->qkv.stride, ql + kl, 1);
    /* O: input columns of this rank's heads */
    rc |= llmb200_upload_packed(wt, r->o_proj.data, Hq_hd, D, k * ql, ql, ly->o.w, ly->o.stride, 0, 1);
    /* gate/up rows interleaved g0,u0,g1,u1,... so one warp finishes a (gate, up) pair */
    rc |= llmb200_upload_packed(wt, r->gate_proj.data + (size_t)k * il * D, D, il, 0, D, ly->gateup.w, ly->gateup.stride, 0, 2);
    rc |= llmb200_upload_packed(wt, r->up_proj.data + (size_t)k * il * D, D, il, 0, D, ly->gateup.w, ly->gateup.stride, 1, 2);
    /* down: input columns of this rank's slice of the FFN */
    rc |= llmb200_upload_packed(wt, r->down_proj.data, s->IS, D, k * il, il, ly->down.w, ly->down.stride, 0, 1);
    if (rc) return rc;

    ly->g_input = upload_gamma(r->input_norm_g, D);
    ly->g_post_attn = upload_gamma(r->post_attn_norm_g, D);
    ly->g_pre_ff = upload_gamma(r->pre_ff_norm_g, D);
    ly->g_post_ff = upload_gamma(r->post_ff_norm_g, D);
    ly->g_qn = upload_gamma(r->q_norm_g, hd);
    ly->g_kn = upload_gamma(r->k_norm_g, hd);
    if (!ly->g_input || !ly->g_post_attn) return -1;
    if (s->mt == MODEL_GEMMA3 && (!ly->g_pre_ff || !ly->g_post_ff)) {
        fprintf(stderr, "[FastGen] layer %d: a Gemma3 layer needs its pre- and post-feedforward norm weights\n", li);
        return B200_E_BADARG;
    }

    /* RoPE frequencies exactly as the reference's CPU path forms them:
     * 1.0f / powf(theta, (float)(2*d) / (float)hd)  (src/nn/attention.c:757-758) */
    float *f = malloc((size_t)(hd / 2) * sizeof(float));
    if (!f) return -1;
    for (int d = 0; d < hd / 2; ++d) f[d] = 1.0f / powf(rope_theta, (float)(2 * d) / (float)hd);
    ly->inv_freq = llmb200_upload_f32(f, (size_t)(hd / 2));
    free(f);
    if (!ly->inv_freq) return -1;
    ly->rope_theta = rope_theta;
    ly->loaded = 1;
    return 0;
}

static void free_graphs(InferenceState *s)
{
    if (s->g_full) { cudaGraphExecDestroy(s->g_full); s->g_full = NULL; }
    if (s->g_nolm) { cudaGraphExecDestroy(s->g_nolm); s->g_nolm = NULL; }
}

int llmb200_state_finish(InferenceState *s, const float *lm_head, const float *final_norm_gamma, const float *token_emb)
{
    if (!s || !lm_head || !final_norm_gamma || !token_emb) return B200_E_BADARG;
    for (int i = 0; i < s->L; ++i)
        if (!s->layers[i].loaded) { fprintf(stderr, "[FastGen] layer %d was never loaded\n", i); return B200_E_STATE; }
    int rc = llmb200_upload_packed(s->wtype, lm_head + (size_t)s->tp_rank * s->V_l * s->D, s->D, s->V_l, 0, s->D,
                                   s->lm.w, s->lm.stride, 0, 1);
    if (rc) return rc;
    s->g_final = llmb200_upload_f32(final_norm_gamma, (size_t)s->D);
    s->emb = llmb200_upload_f32(token_emb, (size_t)s->V * s->D);
    if (!s->g_final || !s->emb) return -1;
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1);
    s->finished = 1;
    return 0;
}

/* ------------------------------------------------------------ one token */

static void prof_mark(InferenceState *s, int kind)
{
    if (!s->prof_on || s->prof_n >= s->prof_cap) return;
    if (kind >= 0) {
        s->prof_kind[s->prof_n / 2] = kind;
        cudaEventRecord(s->prof_ev[s->prof_n++], g_rt.stream);
    } else {
        cudaEventRecord(s->prof_ev[s->prof_n++], g_rt.stream);
    }
}

static unsigned *flags_of(InferenceState *s, int peer, int which) /* which: 0 o, 1 down, 2 argmax */
{
    return (unsigned *)(s->peer[peer] + s->off_flags) + which * B200_MAX_PEERS;
}

static void base_args(InferenceState *s, b200_matvec_args *a, const PackedMat *m, int pdl)
{
    memset(a, 0, sizeof(*a));
    a->d_w = m->w; a->row_stride = m->stride; a->rows = m->rows; a->cols = m->cols; a->wtype = s->wtype;
    a->eps = 1e-6f;                               /* hard-wired in the reference: src/nn/fast_inference.c:383 */
    a->d_pos = s->d_pos; a->d_pos_rw = s->d_pos;
    a->d_epoch = s->d_epoch; a->d_epoch_rw = s->d_epoch; a->d_err = s->d_err;
    a->epoch_mul = s->L + 1;
    a->use_pdl = pdl;
}

/* Timing loops launch one kind of kernel only; such launches must not touch the token state. */
static int want(InferenceState *s, int kind, b200_matvec_args *a)
{
    if (s->only_kind < 0) return 1;
    if (s->only_kind != kind) return 0;
    if (a) {
        a->n_wait = 0; a->n_signal = 0; a->advance_pos = 0; a->advance_epoch = 0; a->d_next_token = NULL;
        if (!a->d_argmax_scratch) a->d_ticket = NULL;
    }
    return 1;
}

/* Enqueue every kernel of one token on the library stream. */
static int enqueue_token(InferenceState *s, int with_lm, int pdl)
{
    const int k = s->tp_size, me = s->tp_rank, D = s->D, L = s->L;
    const int gemma = s->mt == MODEL_GEMMA3;
    float *slots_o = (float *)(s->comm + s->off_slots_o), *slots_dn = (float *)(s->comm + s->off_slots_dn);
    b200_matvec_args a;
    void *st = g_rt.stream;
    for (int l = 0; l < L; ++l) {
        Layer *ly = &s->layers[l];
        /* --- qkv --- */
        base_args(s, &a, &ly->qkv, pdl);
        if (l == 0) {
            a.in_mode = B200_IN_EMBED; a.d_emb = s->emb; a.d_tokens = s->d_tokens; a.emb_scale = s->emb_scale;
            a.emb_rows = s->V;
            a.epoch_add = -1;                     /* previous token's last down signal */
        } else {
            a.in_mode = B200_IN_RESID; a.d_resid_in = s->resid[0];
            a.d_slots = slots_dn; a.n_slots = k; a.slot_stride = D;
            a.d_slot_norm_gamma = gemma ? s->layers[l - 1].g_post_ff : NULL;
            a.epoch_add = l;                      /* down signal of layer l-1 */
        }
        if (k > 1) { a.d_wait_flags = flags_of(s, me, 1); a.n_wait = k; }
        a.d_resid_out = s->resid[1];
        a.d_norm_gamma = ly->g_input;
        a.out_mode = B200_OUT_STORE; a.d_out[0] = s->qkv; a.n_out = 1;
        if (s->lora) a.d_in_copy = s->xnorm;
        prof_mark(s, K_QKV);
        if (want(s, K_QKV, &a)) K_TRY(b200_matvec(&a, st), return -1);
        /* q += s B_q (A_q ln), v += s B_v (A_v ln)  (src/nn/fast_inference.c:406-421) */
        if (s->lora && (s->only_kind < 0 || s->only_kind == K_QKV))
            K_TRY(b200_lora_decode(s->xnorm, s->lora[l].A_q, s->lora[l].B_q, s->lora[l].A_v, s->lora[l].B_v, s->qkv, D,
                                   s->Hq_l * s->hd, s->Hkv_l * s->hd, s->lora_rank, s->lora_scaling, st), return -1);
        prof_mark(s, -1);
        /* --- attention --- */
        b200_attn_args at;
        memset(&at, 0, sizeof(at));
        at.d_qkv = s->qkv; at.d_q_gamma = ly->g_qn; at.d_k_gamma = ly->g_kn; at.d_inv_freq = ly->inv_freq;
        at.d_k_cache = ly->k_cache; at.d_v_cache = ly->v_cache;
        at.d_out = s->attn_out; at.d_scratch = s->attn_scratch; at.d_tickets = s->attn_tickets; at.d_pos = s->d_pos;
        at.n_q = s->Hq_l; at.n_kv = s->Hkv_l; at.hd = s->hd; at.max_seq = s->max_seq; at.n_split = s->n_split;
        at.eps = 1e-6f; at.use_pdl = pdl;
        prof_mark(s, K_ATTN);
        if (want(s, K_ATTN, NULL)) K_TRY(b200_attn_decode(&at, st), return -1);
        prof_mark(s, -1);
        /* --- o: partial sums into slot `me` of every rank --- */
        base_args(s, &a, &ly->o, pdl);
        a.in_mode = B200_IN_VEC; a.d_in_vec = s->attn_out;
        a.out_mode = B200_OUT_STORE; a.n_out = k;
        for (int p = 0; p < k; ++p) a.d_out[p] = (float *)(s->peer[p] + s->off_slots_o) + (size_t)me * D;
        if (k > 1) {
            a.d_ticket = s->mv_ticket; a.n_signal = k; a.signal_index = me; a.epoch_add = l + 1;
            for (int p = 0; p < k; ++p) a.d_signal_flags[p] = flags_of(s, p, 0);
        }
        prof_mark(s, K_O);
        if (want(s, K_O, &a)) K_TRY(b200_matvec(&a, st), return -1);
        prof_mark(s, -1);
        /* --- gate/up --- */
        base_args(s, &a, &ly->gateup, pdl);
        a.in_mode = B200_IN_RESID; a.d_resid_in = s->resid[1]; a.d_resid_out = s->resid[0];
        a.d_slots = slots_o; a.n_slots = k; a.slot_stride = D;
        a.d_slot_norm_gamma = gemma ? ly->g_post_attn : NULL;
        a.d_norm_gamma = gemma ? ly->g_pre_ff : ly->g_post_attn;
        if (k > 1) { a.d_wait_flags = flags_of(s, me, 0); a.n_wait = k; a.epoch_add = l + 1; }
        a.out_mode = B200_OUT_GLU; a.act = gemma ? 1 : 0; a.d_out[0] = s->act; a.n_out = 1;
        prof_mark(s, K_GATEUP);
        if (want(s, K_GATEUP, &a)) K_TRY(b200_matvec(&a, st), return -1);
        prof_mark(s, -1);
        /* --- down --- */
        base_args(s, &a, &ly->down, pdl);
        a.in_mode = B200_IN_VEC; a.d_in_vec = s->act;
        a.out_mode = B200_OUT_STORE; a.n_out = k;
        for (int p = 0; p < k; ++p) a.d_out[p] = (float *)(s->peer[p] + s->off_slots_dn) + (size_t)me * D;
        if (k > 1) {
            a.d_ticket = s->mv_ticket; a.n_signal = k; a.signal_index = me; a.epoch_add = l + 1;
            for (int p = 0; p < k; ++p) a.d_signal_flags[p] = flags_of(s, p, 1);
        }
        if (!with_lm && l == L - 1) { a.d_ticket = s->mv_ticket; a.advance_pos = 1; a.advance_epoch = 1; }
        prof_mark(s, K_DOWN);
        if (want(s, K_DOWN, &a)) K_TRY(b200_matvec(&a, st), return -1);
        prof_mark(s, -1);
    }
    if (!with_lm) return 0;
    /* --- final norm + LM head + greedy pick --- */
    base_args(s, &a, &s->lm, pdl);
    a.in_mode = B200_IN_RESID; a.d_resid_in = s->resid[0];
    a.d_slots = slots_dn; a.n_slots = k; a.slot_stride = D;
    a.d_slot_norm_gamma = gemma ? s->layers[L - 1].g_post_ff : NULL;
    a.d_norm_gamma = s->g_final;
    if (k > 1) { a.d_wait_flags = flags_of(s, me, 1); a.n_wait = k; a.epoch_add = L; }
    a.out_mode = B200_OUT_STORE; a.n_out = k; a.out_offset = (long long)me * s->V_l;
    for (int p = 0; p < k; ++p) a.d_out[p] = (float *)(s->peer[p] + s->off_logits);
    a.d_ticket = s->mv_ticket; a.d_argmax_scratch = s->am_scratch;
    a.n_argmax_out = k;
    for (int p = 0; p < k; ++p) {
        a.d_argmax_val[p] = (float *)(s->peer[p] + s->off_am_val) + me;
        a.d_argmax_idx[p] = (int *)(s->peer[p] + s->off_am_idx) + me;
    }
    if (k == 1) {
        a.d_next_token = s->d_tokens; a.d_prompt_len = s->d_prompt_len; a.advance_pos = 1; a.advance_epoch = 1;
    } else {
        a.n_signal = k; a.signal_index = me;
        for (int p = 0; p < k; ++p) a.d_signal_flags[p] = flags_of(s, p, 2);
        /* the wait above used epoch_add = L; the argmax flags carry L + 1 */
    }
    if (k > 1) {
        /* one kernel cannot wait with one value and signal with another: the LM head
         * waits on the down flags (value L) and signals the argmax flags with the
         * same value L; the finalize kernel waits for that value. */
        a.epoch_add = L;
    }
    prof_mark(s, K_LM);
    if (want(s, K_LM, &a)) K_TRY(b200_matvec(&a, st), return -1);
    prof_mark(s, -1);
    if (k > 1 && s->only_kind < 0) {
        K_TRY(b200_tp_argmax_finalize((const float *)(s->comm + s->off_am_val), (const int *)(s->comm + s->off_am_idx), k,
                                      flags_of(s, me, 2), s->d_epoch, L + 1, L, s->d_tokens, s->d_pos, s->d_prompt_len,
                                      s->d_epoch, s->d_err, pdl, st), return -1);
    }
    return 0;
}

/* ------------------------------------------------------------ whole-token kernel */

/* Plans the whole-token kernel for this model: geometry of the five matvec stages, the layer table and
 * the flagged hand-over vectors. Returns 0 when the kernel can run this model, 1 when it cannot (shape
 * or shared-memory budget outside its limits), -1 on a CUDA error. */
static int build_plan(InferenceState *s)
{
    if (s->tk_planned) return 0;
    const int k = s->tp_size, me = s->tp_rank, D = s->D, L = s->L;
    b200_token_args *a = &s->tk;
    memset(a, 0, sizeof(*a));
    a->n_layers = L; a->wtype = s->wtype; a->gemma = s->mt == MODEL_GEMMA3;
    const Layer *l0 = &s->layers[0];
    const PackedMat *m[B200_ST_KINDS] = {&l0->qkv, &l0->o, &l0->gateup, &l0->down, &s->lm};
    for (int i = 0; i < B200_ST_KINDS; ++i) {
        a->g[i].rows = m[i]->rows; a->g[i].cols = m[i]->cols; a->g[i].row_stride = m[i]->stride;
        a->g[i].glu = i == B200_ST_GATEUP;
    }
    a->w_lm = s->lm.w; a->g_final = s->g_final;
    a->d_emb = s->emb; a->emb_rows = s->V; a->emb_scale = s->emb_scale;
    a->eps = 1e-6f;                               /* hard-wired in the reference: src/nn/fast_inference.c:383 */
    a->d_model = D; a->n_q = s->Hq_l; a->n_kv = s->Hkv_l; a->hd = s->hd; a->max_seq = s->max_seq;
    a->n_split = 0;
    {   /* few enough splits that a merging block reads little: 18 at head_dim <= 128, 9 above */
        int cap = s->hd > 128 ? 9 : 18;
        const char *sp = getenv("LLMB200_ATT_SPLITS");
        if (sp && atoi(sp) > 0 && atoi(sp) <= 32) cap = atoi(sp);
        a->n_split = s->n_sm / s->Hkv_l < cap ? s->n_sm / s->Hkv_l : cap;
    }
    a->n_ranks = k; a->rank = me;
    {
        const char *la = getenv("LLMB200_L2_AHEAD_KB");         /* experiments: L2 prefetch of the following stage */
        if (la && atoi(la) > 0) a->l2_ahead_bytes = atoi(la) * 1024;
    }
    int rc = b200_token_plan(a, s->n_sm);
    if (rc != 0) return 1;

    /* Rotation tables: cos / sin of pos * inv_freq[d] for every position, one table per distinct base, from
     * the C library's cosf / sinf on the angle formed as the reference's CPU path forms it
     * (src/nn/attention.c:757-766): no trigonometry on the device's critical path. */
    for (int l = 0; l < L; ++l) {
        Layer *ly = &s->layers[l];
        if (ly->rope) continue;
        for (int m = 0; m < l && !ly->rope; ++m)
            if (s->layers[m].rope_theta == ly->rope_theta) ly->rope = s->layers[m].rope;
        if (ly->rope) continue;
        if (s->n_rope_tab >= 8) { fprintf(stderr, "[FastGen] more than 8 distinct RoPE bases\n"); return 1; }
        const int half = s->hd / 2;
        const size_t n = (size_t)s->max_seq * half * 2;
        float *h = malloc(n * sizeof(float));
        if (!h) return -1;
        for (int d = 0; d < half; ++d) {
            const float freq = 1.0f / powf(ly->rope_theta, (float)(2 * d) / (float)s->hd);
            for (int pos = 0; pos < s->max_seq; ++pos) {
                const float angle = (float)pos * freq;
                h[((size_t)pos * half + d) * 2] = cosf(angle);
                h[((size_t)pos * half + d) * 2 + 1] = sinf(angle);
            }
        }
        float *dt = llmb200_upload_f32(h, n);
        free(h);
        if (!dt) return -1;
        s->rope_tab[s->n_rope_tab++] = dt;
        ly->rope = dt;
    }
    b200_token_layer *tl = calloc((size_t)L, sizeof(*tl));
    if (!tl) return -1;
    for (int l = 0; l < L; ++l) {
        const Layer *ly = &s->layers[l];
        tl[l].w_qkv = ly->qkv.w; tl[l].w_o = ly->o.w; tl[l].w_gateup = ly->gateup.w; tl[l].w_down = ly->down.w;
        tl[l].g_input = ly->g_input; tl[l].g_post_attn = ly->g_post_attn; tl[l].g_pre_ff = ly->g_pre_ff;
        tl[l].g_post_ff = ly->g_post_ff; tl[l].g_qn = ly->g_qn; tl[l].g_kn = ly->g_kn; tl[l].rope = ly->rope;
        tl[l].k_cache = ly->k_cache; tl[l].v_cache = ly->v_cache;
    }
    if (!s->d_tk_layers) CU_TRY(cudaMalloc((void **)&s->d_tk_layers, (size_t)L * sizeof(*tl)), { free(tl); return -1; });
    CU_TRY(cudaMemcpy(s->d_tk_layers, tl, (size_t)L * sizeof(*tl), cudaMemcpyHostToDevice), { free(tl); return -1; });
    free(tl);
    const int qkv_rows = (s->Hq_l + 2 * s->Hkv_l) * s->hd;
    if (!s->fl_qkv) s->fl_qkv = (b200_flagged *)dev_zero((size_t)qkv_rows * 8);
    if (!s->fl_part) s->fl_part = (b200_flagged *)dev_zero((size_t)s->Hq_l * a->n_split * (s->hd + 2) * 8);
    if (!s->fl_attn) s->fl_attn = (b200_flagged *)dev_zero((size_t)s->Hq_l * s->hd * 8);
    if (!s->fl_act) s->fl_act = (b200_flagged *)dev_zero((size_t)s->IS_l * 8);
    if (!s->fl_am) s->fl_am = (b200_flagged *)dev_zero((size_t)2 * s->n_sm * 8);
    if (!s->fl_qkv || !s->fl_part || !s->fl_attn || !s->fl_act || !s->fl_am) return -1;
    if (getenv("LLMB200_TRACE") && !s->d_step_ns)
        s->d_step_ns = (unsigned long long *)dev_zero((size_t)s->n_sm * (6 * L + 1) * 16 * 8);
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1);

    a->d_layers = s->d_tk_layers;
    a->d_pos = s->d_pos; a->d_tokens = s->d_tokens; a->d_prompt_len = s->d_prompt_len; a->d_epoch = s->d_epoch; a->d_err = s->d_err;
    a->d_qkv = s->fl_qkv; a->d_attn_part = s->fl_part; a->d_attn_out = s->fl_attn; a->d_act = s->fl_act; a->d_am = s->fl_am;
    a->d_logits = (float *)(s->comm + s->off_logits); a->logits_offset = (long long)me * s->V_l;
    a->d_trace = s->d_step_ns;
    {
        const char *sl = getenv("LLMB200_SPIN_LIMIT");
        a->spin_limit = sl && atoi(sl) > 0 ? atoi(sl) : 0;
        /* Readers poll the flagged words straight away (measured on Qwen3-4B: 675 tok/s against 639 with one
         * thread per block watching the arrival counter first); LLMB200_DIRECT_POLL=0 brings the counters back. */
        const char *dp = getenv("LLMB200_DIRECT_POLL");
        const int direct = dp ? atoi(dp) > 0 : 1;
        a->counter_spin_limit = direct ? 0 : (a->spin_limit > 0 ? a->spin_limit : 1 << 20);
    }
    s->tk_planned = 1;
    return 0;
}

/* Pointers into the peers' exchange regions: valid only once the peers are connected. */
static void bind_peers(InferenceState *s)
{
    const int k = s->tp_size, me = s->tp_rank, D = s->D;
    b200_token_args *a = &s->tk;
    a->d_slots_o = (const b200_flagged *)(s->comm + s->off_fl_slots_o);
    a->d_slots_dn = (const b200_flagged *)(s->comm + s->off_fl_slots_dn);
    a->d_am_rank = (const b200_flagged *)(s->comm + s->off_fl_am);
    a->d_counters = (unsigned *)(s->comm + s->off_counters);
    for (int p = 0; p < k; ++p) {
        a->d_peer_slots_o[p] = (b200_flagged *)(s->peer[p] + s->off_fl_slots_o) + (size_t)me * D;
        a->d_peer_slots_dn[p] = (b200_flagged *)(s->peer[p] + s->off_fl_slots_dn) + (size_t)me * D;
        a->d_peer_am[p] = (b200_flagged *)(s->peer[p] + s->off_fl_am) + 2 * me;
        a->d_peer_counters[p] = (unsigned *)(s->peer[p] + s->off_counters);
    }
}

static int enqueue_token_fused(InferenceState *s, int with_lm)
{
    b200_token_args a = s->tk;
    a.with_lm = with_lm;
    K_TRY(b200_decode_token(&a, g_rt.stream), return -1);
    return 0;
}

static int capture(InferenceState *s, int with_lm, int pdl, cudaGraphExec_t *out)
{
    cudaGraph_t g = NULL;
    CU_TRY(cudaStreamBeginCapture(g_rt.stream, cudaStreamCaptureModeThreadLocal), return -1);
    const unsigned long long before = b200_launch_count(0);
    int rc = s->fused ? enqueue_token_fused(s, with_lm) : enqueue_token(s, with_lm, pdl);
    if (with_lm) s->kernels_full = (int)(b200_launch_count(0) - before);
    else s->kernels_nolm = (int)(b200_launch_count(0) - before);
    cudaError_t e = cudaStreamEndCapture(g_rt.stream, &g);
    if (rc != 0 || e != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();
        return -1;
    }
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { cudaGetLastError(); *out = NULL; return -1; }
    return 0;
}

static int ensure_graphs(InferenceState *s)
{
    if (s->g_full && s->g_nolm) return 0;
    if (!s->finished) { fprintf(stderr, "[FastGen] state is not fully loaded\n"); return -1; }
    if (!s->connected) { fprintf(stderr, "[FastGen] tensor-parallel peers are not connected (llmb200_state_connect)\n"); return -1; }
    free_graphs(s);
    /* The whole-token persistent kernel (one launch per token) is the default; LLMB200_TOKEN_KERNEL=0
     * selects one kernel per stage, which is also what runs when the model is outside the persistent
     * kernel's limits or a LoRA adapter is attached (it has no LoRA side path). */
    s->fused = 0;
    const char *tk = getenv("LLMB200_TOKEN_KERNEL");
    if (!(tk && tk[0] == '0') && !s->lora) {
        int pr = build_plan(s);
        if (pr < 0) return -1;
        if (pr == 0) {
            bind_peers(s);
            s->fused = 1;
            if (capture(s, 1, 0, &s->g_full) == 0 && capture(s, 0, 0, &s->g_nolm) == 0) return 0;
            fprintf(stderr, "[FastGen] whole-token kernel could not be captured; using one kernel per stage\n");
            free_graphs(s);
            s->fused = 0;
        }
    }
    if (capture(s, 1, s->use_pdl, &s->g_full) != 0 || capture(s, 0, s->use_pdl, &s->g_nolm) != 0) {
        if (s->use_pdl) {
            fprintf(stderr, "[FastGen] graph capture with programmatic dependent launch failed; retrying without\n");
            free_graphs(s);
            s->use_pdl = 0;
            if (capture(s, 1, 0, &s->g_full) == 0 && capture(s, 0, 0, &s->g_nolm) == 0) return 0;
        }
        fprintf(stderr, "[FastGen] CUDA graph capture failed\n");
        free_graphs(s);
        return -1;
    }
    return 0;
}

/* ------------------------------------------------------------ TP plumbing */

int llmb200_state_comm_handle(InferenceState *s, void *out)
{
    if (!s || !out) return B200_E_BADARG;
    cudaIpcMemHandle_t h;
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1);
    CU_TRY(cudaIpcGetMemHandle(&h, s->comm), return -1);
    memset(out, 0, LLMB200_HANDLE_BYTES);
    memcpy(out, &h, sizeof(h) < LLMB200_HANDLE_BYTES ? sizeof(h) : LLMB200_HANDLE_BYTES);
    return 0;
}

int llmb200_state_connect(InferenceState *s, const void *handles, int world)
{
    if (!s || !handles || world != s->tp_size) return B200_E_BADARG;
    for (int p = 0; p < world; ++p) {
        if (p == s->tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)p * LLMB200_HANDLE_BYTES, sizeof(h));
        void *ptr = NULL;
        CU_TRY(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), return -1);
        s->peer[p] = (char *)ptr;
    }
    s->connected = 1;
    free_graphs(s);
    return 0;
}

/* ------------------------------------------------------------ reference API */

static void fill_refs_common(LayerWeightRef *r, llmb200_gqa *at, llmb200_linear *gate, llmb200_linear *up,
                             llmb200_linear *down, int D, int Hq_hd, int Hkv_hd, int IS, int hd)
{
    r->q_proj = (WeightRef){at->q_proj->weight->data, Hq_hd, D};
    r->k_proj = (WeightRef){at->k_proj->weight->data, Hkv_hd, D};
    r->v_proj = (WeightRef){at->v_proj->weight->data, Hkv_hd, D};
    r->o_proj = (WeightRef){at->o_proj->weight->data, D, Hq_hd};
    r->gate_proj = (WeightRef){gate->weight->data, IS, D};
    r->up_proj = (WeightRef){up->weight->data, IS, D};
    r->down_proj = (WeightRef){down->weight->data, D, IS};
    r->q_norm_g = at->q_norm ? at->q_norm->gamma->data : NULL;
    r->k_norm_g = at->k_norm ? at->k_norm->gamma->data : NULL;
    r->d_model = D; r->head_dim = hd;
}

static InferenceState *create_qwen3_one(llmb200_qwen3_model *m, int max_seq_len, int use_fp16)
{
    if (!m) return NULL;
    llmb200_config c = {MODEL_QWEN3, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                        m->vocab_size, m->n_layers, max_seq_len, use_fp16};
    InferenceState *s = llmb200_state_begin(&c);
    if (!s) return NULL;
    const char *mode = use_fp16 ? "F16" : "Q8_0";
    fprintf(stderr, "[FastGen] Converting weights to %s + uploading to GPU...\n", mode);
    const double t0 = now_ms();
    for (int i = 0; i < m->n_layers; ++i) {
        llmb200_qwen3_block *b = m->blocks[i];
        LayerWeightRef r;
        memset(&r, 0, sizeof(r));
        fill_refs_common(&r, b->attn, b->gate_proj, b->up_proj, b->down_proj, m->d_model, m->n_q_heads * m->head_dim,
                         m->n_kv_heads * m->head_dim, m->intermediate_size, m->head_dim);
        r.input_norm_g = b->input_norm->gamma->data;
        r.post_attn_norm_g = b->post_attn_norm->gamma->data;
        if (llmb200_state_load_layer(s, i, &r, m->rope_theta) != 0) { inference_state_free(s); return NULL; }
    }
    if (llmb200_state_finish(s, m->lm_head->weight->data, m->final_norm->gamma->data, m->token_emb->weight->data) != 0) {
        inference_state_free(s);
        return NULL;
    }
    fprintf(stderr, "[FastGen] %s + GPU upload: %.0f ms\n", mode, now_ms() - t0);
    return s;
}

static InferenceState *create_gemma3_one(llmb200_gemma3_model *m, int max_seq_len, int use_fp16)
{
    if (!m) return NULL;
    llmb200_config c = {MODEL_GEMMA3, m->d_model, m->n_q_heads, m->n_kv_heads, m->head_dim, m->intermediate_size,
                        m->vocab_size, m->n_layers, max_seq_len, use_fp16};
    InferenceState *s = llmb200_state_begin(&c);
    if (!s) return NULL;
    const char *mode = use_fp16 ? "F16" : "Q8_0";
    fprintf(stderr, "[FastGen] Converting weights to %s + uploading to GPU...\n", mode);
    const double t0 = now_ms();
    for (int i = 0; i < m->n_layers; ++i) {
        llmb200_gemma3_block *b = m->blocks[i];
        LayerWeightRef r;
        memset(&r, 0, sizeof(r));
        fill_refs_common(&r, b->attn, b->gate_proj, b->up_proj, b->down_proj, m->d_model, m->n_q_heads * m->head_dim,
                         m->n_kv_heads * m->head_dim, m->intermediate_size, m->head_dim);
        r.input_norm_g = b->input_norm->gamma->data;
        r.post_attn_norm_g = b->post_attn_norm->gamma->data;
        r.pre_ff_norm_g = b->pre_ff_norm->gamma->data;
        r.post_ff_norm_g = b->post_ff_norm->gamma->data;
        const float theta = b->is_sliding ? m->local_rope_theta : m->global_rope_theta;
        if (llmb200_state_load_layer(s, i, &r, theta) != 0) { inference_state_free(s); return NULL; }
    }
    /* tied embeddings: the LM head is the embedding table (src/nn/fast_inference.c:307-313) */
    if (llmb200_state_finish(s, m->token_emb->weight->data, m->final_norm->gamma->data, m->token_emb->weight->data) != 0) {
        inference_state_free(s);
        return NULL;
    }
    fprintf(stderr, "[FastGen] %s + GPU upload: %.0f ms\n", mode, now_ms() - t0);
    return s;
}

/* Attaches the SFT state's LoRA matrices (Q and V projections) to the decode step; the adapter is read in
 * place, so later training steps are seen by later tokens. Replaces inference_state_set_lora
 * (src/nn/fast_inference.c:496-520). One GPU only: with tensor parallelism the call is refused. */
/* One F16 projection of the SFT state (binary16 [rows, ld] row-major on the device, as sft_get_layers hands it
 * out) into packed rows dst_row0 + r*dst_row_step: the packed F16 layout is row-major binary16 with a padded
 * stride, so this is a strided device-to-device copy. */
static int share_rows(const WMat *w, int col0, int cols, PackedMat *dst, int dst_row0, int dst_row_step)
{
    if (!w || !w->mbuf || !w->mbuf->dev) return B200_E_BADARG;
    CU_TRY(cudaMemcpy2DAsync((char *)dst->w + (size_t)dst_row0 * dst->stride, (size_t)dst->stride * dst_row_step,
                             (const char *)w->mbuf->dev + (size_t)col0 * 2, (size_t)w->cols * 2, (size_t)cols * 2,
                             (size_t)w->rows, cudaMemcpyDeviceToDevice, g_rt.stream), return -1);
    return 0;
}

static float *clone_f32(const void *d_src, size_t n)
{
    float *p = NULL;
    CU_TRY(cudaMalloc((void **)&p, n * 4), return NULL);
    CU_TRY(cudaMemcpyAsync(p, d_src, n * 4, cudaMemcpyDeviceToDevice, g_rt.stream), { cudaFree(p); return NULL; });
    return p;
}

/* The seven projections of every layer and the LM head, re-laid for the decode kernels by device-to-device
 * copies from the SFT state's views. Also run again whenever full-parameter training has changed them. */
static int take_sft_matrices(InferenceState *s, SFTState *sft)
{
    LayerW *lw = sft_get_layers(sft);
    WMat *lm = sft_get_lm_head(sft);
    if (!lw || !lm) return -1;
    llmb200_sft_refresh_views(sft);
    const int D = s->D, ql = s->Hq * s->hd, kl = s->Hkv * s->hd;
    int rc = 0;
    for (int i = 0; i < s->L && !rc; ++i) {
        Layer *ly = &s->layers[i];
        const LayerW *r = &lw[i];
        rc |= share_rows(r->q_proj, 0, D, &ly->qkv, 0, 1);
        rc |= share_rows(r->k_proj, 0, D, &ly->qkv, ql, 1);
        rc |= share_rows(r->v_proj, 0, D, &ly->qkv, ql + kl, 1);
        rc |= share_rows(r->o_proj, 0, ql, &ly->o, 0, 1);
        rc |= share_rows(r->gate_proj, 0, D, &ly->gateup, 0, 2);
        rc |= share_rows(r->up_proj, 0, D, &ly->gateup, 1, 2);
        rc |= share_rows(r->down_proj, 0, s->IS, &ly->down, 0, 1);
    }
    if (!rc) rc = share_rows(lm, 0, D, &s->lm, 0, 1);
    s->sft_src = sft;
    s->sft_version = llmb200_sft_weights_version(sft);
    return rc;
}

/* The reference's decode state aliases the SFT state's buffers, so a full-parameter step shows in the next
 * token; here the matrices are copies in the decode layout, taken again when the SFT state says they changed.
 * The SFT state must outlive the decode state made from it (as in the reference). */
static void follow_sft(InferenceState *s)
{
    if (!s || !s->sft_src || llmb200_sft_weights_version(s->sft_src) == s->sft_version) return;
    if (take_sft_matrices(s, s->sft_src) != 0) {
        fprintf(stderr, "[FastGen] re-reading the SFT state's weights failed\n");
    }
}

/* A decode state over the weights an SFT state already holds on the device, with that state's LoRA attached
 * (read in place, so decoding follows training). The frozen matrices are re-laid for the decode kernels by
 * device-to-device copies -- no host round trip, no second conversion; they never change in LoRA training, so
 * a copy and the reference's aliasing behave the same. F16 weights, one GPU. max_seq_len above 4096 is
 * clamped. Replaces inference_state_create_from_sft (src/nn/fast_inference.c:526-608; fast_inference.h:50). */
InferenceState *inference_state_create_from_sft(SFTState *sft, int max_seq_len)
{
    if (!sft) return NULL;
    LayerW *lw = sft_get_layers(sft);
    WMat *lm = sft_get_lm_head(sft);
    MetalBuf *fg = sft_get_final_norm_g(sft);
    const float *thetas = sft_get_rope_thetas(sft);
    const float *d_emb = llmb200_sft_device_emb(sft);
    if (!lw || !lm || !fg || !thetas || !d_emb) {
        fprintf(stderr, "[FastGen] the SFT state is not complete\n");
        return NULL;
    }
    llmb200_config c = { sft_get_model_type(sft), sft_get_d_model(sft), sft_get_n_q_heads(sft), sft_get_n_kv_heads(sft),
                         sft_get_head_dim(sft), sft_get_intermediate_size(sft), sft_get_vocab_size(sft), sft_get_n_layers(sft),
                         max_seq_len, 1 };
    InferenceState *s = llmb200_state_begin(&c);
    if (!s) return NULL;
    if (s->tp_size != 1) {
        fprintf(stderr, "[FastGen] sharing weights with an SFT state needs one GPU (tensor parallelism is %d)\n", s->tp_size);
        inference_state_free(s);
        return NULL;
    }
    const int D = s->D, hd = s->hd;
    int rc = take_sft_matrices(s, sft);
    for (int i = 0; i < s->L && !rc; ++i) {
        Layer *ly = &s->layers[i];
        const LayerW *r = &lw[i];
        ly->g_input = clone_f32(r->input_norm_g->dev, (size_t)D);
        ly->g_post_attn = clone_f32(r->post_attn_norm_g->dev, (size_t)D);
        ly->g_qn = r->q_norm_g ? clone_f32(r->q_norm_g->dev, (size_t)hd) : NULL;
        ly->g_kn = r->k_norm_g ? clone_f32(r->k_norm_g->dev, (size_t)hd) : NULL;
        ly->g_pre_ff = r->pre_ff_norm_g ? clone_f32(r->pre_ff_norm_g->dev, (size_t)D) : NULL;      /* Gemma3 */
        ly->g_post_ff = r->post_ff_norm_g ? clone_f32(r->post_ff_norm_g->dev, (size_t)D) : NULL;
        float *f = malloc((size_t)(hd / 2) * sizeof(float));
        if (!f || !ly->g_input || !ly->g_post_attn || (s->mt == MODEL_GEMMA3 && (!ly->g_pre_ff || !ly->g_post_ff))) { free(f); rc = -1; break; }
        for (int d = 0; d < hd / 2; ++d) f[d] = 1.0f / powf(thetas[i], (float)(2 * d) / (float)hd);
        ly->inv_freq = llmb200_upload_f32(f, (size_t)(hd / 2));
        free(f);
        if (!ly->inv_freq) rc = -1;
        ly->rope_theta = thetas[i];
        ly->loaded = 1;
    }
    if (!rc) {
        s->g_final = clone_f32(fg->dev, (size_t)D);
        s->emb = clone_f32(d_emb, (size_t)s->V * D);
        if (!s->g_final || !s->emb) rc = -1;
    }
    if (!rc && cudaStreamSynchronize(g_rt.stream) != cudaSuccess) rc = -1;
    if (rc) {
        fprintf(stderr, "[FastGen] taking over the SFT state's weights failed\n");
        inference_state_free(s);
        return NULL;
    }
    s->finished = 1;
    inference_state_set_lora(s, sft);
    fprintf(stderr, "[FastGen] Created from SFT (weights taken over on the device, no host upload)\n");
    return s;
}

void inference_state_set_lora(InferenceState *s, SFTState *sft)
{
    if (!s || !sft) return;
    const int R = sft_get_lora_rank(sft);
    if (R == 0) return;
    if (s->tp_size != 1) {
        fprintf(stderr, "[FastGen] inference_state_set_lora: not available with tensor parallelism\n");
        return;
    }
    if (R > 64 || sft_get_n_layers(sft) != s->L || sft_get_d_model(sft) != s->D) {
        fprintf(stderr, "[FastGen] inference_state_set_lora: adapter does not match the model (layers %d/%d, d_model %d/%d, rank %d)\n",
                sft_get_n_layers(sft), s->L, sft_get_d_model(sft), s->D, R);
        return;
    }
    if (!s->lora) s->lora = calloc(s->L, sizeof(*s->lora));
    if (!s->xnorm) CU_TRY(cudaMalloc((void **)&s->xnorm, (size_t)s->D * sizeof(float)), return);
    if (!s->lora) return;
    for (int l = 0; l < s->L; ++l) {
        MetalBuf *b[4];
        for (int k = 0; k < 4; ++k) b[k] = sft_get_lora_weight_buf(sft, l, k);
        if (!b[0] || !b[1] || !b[2] || !b[3]) { free(s->lora); s->lora = NULL; return; }
        s->lora[l].A_q = b[0]->dev; s->lora[l].B_q = b[1]->dev; s->lora[l].A_v = b[2]->dev; s->lora[l].B_v = b[3]->dev;
    }
    s->lora_rank = R;
    s->lora_scaling = sft_get_lora_scaling(sft);
    if (g_rt.refs > 0) cudaStreamSynchronize(g_rt.stream);
    free_graphs(s);                      /* the per-token graph gains one kernel per layer */
}

static void free_one(InferenceState *s)
{
    if (!s) return;
    if (g_rt.refs > 0) cudaStreamSynchronize(g_rt.stream);
    free_graphs(s);
    if (s->layers) {
        for (int i = 0; i < s->L; ++i) {
            Layer *ly = &s->layers[i];
            cudaFree(ly->qkv.w); cudaFree(ly->o.w); cudaFree(ly->gateup.w); cudaFree(ly->down.w);
            cudaFree(ly->g_input); cudaFree(ly->g_post_attn); cudaFree(ly->g_pre_ff); cudaFree(ly->g_post_ff);
            cudaFree(ly->g_qn); cudaFree(ly->g_kn); cudaFree(ly->inv_freq);
            cudaFree(ly->k_cache); cudaFree(ly->v_cache);
        }
        free(s->layers);
    }
    cudaFree(s->lm.w); cudaFree(s->g_final); cudaFree(s->emb);
    cudaFree(s->resid[0]); cudaFree(s->resid[1]); cudaFree(s->qkv); cudaFree(s->attn_out); cudaFree(s->act);
    for (int i = 0; i < s->n_rope_tab; ++i) cudaFree(s->rope_tab[i]);
    cudaFree(s->d_tk_layers); cudaFree(s->fl_qkv); cudaFree(s->fl_part); cudaFree(s->fl_attn); cudaFree(s->fl_act);
    cudaFree(s->fl_am); cudaFree(s->d_step_ns);
    cudaFree(s->xnorm);
    free(s->lora);
    cudaFree(s->attn_scratch); cudaFree(s->am_scratch); cudaFree(s->attn_tickets); cudaFree(s->mv_ticket);
    cudaFree(s->d_pos);
    for (int p = 0; p < s->tp_size; ++p)
        if (p != s->tp_rank && s->peer[p] && !s->loopback && !s->local_peers) cudaIpcCloseMemHandle(s->peer[p]);
    cudaFree(s->comm);
    if (s->h_logits) cudaFreeHost(s->h_logits);
    if (s->h_tok) cudaFreeHost(s->h_tok);
    if (s->h_ctl) cudaFreeHost(s->h_ctl);
    for (int i = 0; i < 4; ++i) if (s->tok_ev[i]) cudaEventDestroy(s->tok_ev[i]);
    if (s->ev_a) cudaEventDestroy(s->ev_a);
    if (s->ev_b) cudaEventDestroy(s->ev_b);
    if (s->prof_ev) {
        for (int i = 0; i < s->prof_cap; ++i) cudaEventDestroy(s->prof_ev[i]);
        free(s->prof_ev); free(s->prof_kind);
    }
    free(s);
    fast_metal_shutdown();
}

ModelType inference_state_model_type(InferenceState *s) { return s->mt; }
int inference_state_vocab_size(InferenceState *s) { return s->V; }
void inference_state_reset(InferenceState *s)
{
    if (!s) return;
    s->cur_len = 0;
    for (int r = 1; r < s->group_n; ++r) s->group[r]->cur_len = 0;
}
int llmb200_state_position(InferenceState *s) { return s ? s->cur_len : -1; }
int llmb200_state_graph_kernels(InferenceState *s, int with_lm_head)
{
    if (!s || ensure_graphs(s) != 0) return -1;
    return with_lm_head ? s->kernels_full : s->kernels_nolm;
}
/* Stage trace of the last whole-token launch (needs LLMB200_TRACE=1 at create time), [block][stage][8]
 * words of the nanosecond timer (b200_token_args.d_trace). Returns the number of blocks. */
int llmb200_state_step_trace(InferenceState *s, unsigned long long *out, size_t cap_words)
{
    if (!s || !s->d_step_ns || !out) return 0;
    size_t n = (size_t)s->n_sm * (6 * s->L + 1) * 16;
    if (n > cap_words) n = cap_words;
    if (cudaStreamSynchronize(g_rt.stream) != cudaSuccess) return 0;
    if (cudaMemcpy(out, s->d_step_ns, n * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    return s->n_sm;
}
unsigned long long llmb200_state_weight_bytes(InferenceState *s) { return s ? s->weight_bytes : 0; }
double llmb200_last_decode_ms(InferenceState *s, int *n) { if (n) *n = s->last_n_decoded; return s->last_decode_ms; }
double llmb200_last_prefill_ms(InferenceState *s) { return s->last_prefill_ms; }

void llmb200_state_set_eos(InferenceState *s, const int *eos, int n)
{
    if (!s) return;
    if (n < 0) n = 0;
    if (n > 4) n = 4;
    for (int i = 0; i < n; ++i) s->eos[i] = eos[i];
    s->n_eos = n;
    for (int r = 1; r < s->group_n; ++r) llmb200_state_set_eos(s->group[r], eos, n);
}

int llmb200_state_error(InferenceState *s)
{
    if (!s) return 1;
    int err = 0;
    if (cudaMemcpy(&err, s->d_err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    for (int r = 1; r < s->group_n && !err; ++r) err = llmb200_state_error(s->group[r]);
    return err;
}

int llmb200_state_connect_loopback(InferenceState *s)
{
    if (!s || s->tp_size < 2) return B200_E_BADARG;
    for (int p = 0; p < s->tp_size; ++p) s->peer[p] = s->comm;   /* nothing is opened: inference_state_free closes nothing it did not open */
    s->connected = 1;
    s->loopback = 1;
    free_graphs(s);
    return 0;
}

/* Writes pos / prompt_len (and, when n_tok > 0, token ids starting at tok_at) into the control block. */
static int set_control(InferenceState *s, int pos, int prompt_len, const uint32_t *tok, int tok_at, int n_tok)
{
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1);   /* h_ctl may still be in flight */
    s->h_ctl[0] = pos; s->h_ctl[1] = prompt_len;
    CU_TRY(cudaMemcpyAsync(s->d_pos, s->h_ctl, 8, cudaMemcpyHostToDevice, g_rt.stream), return -1);
    if (n_tok > 0) {
        for (int i = 0; i < n_tok; ++i) s->h_ctl[8 + i] = (int)tok[i];
        CU_TRY(cudaMemcpyAsync(s->d_tokens + tok_at, s->h_ctl + 8, (size_t)n_tok * 4, cudaMemcpyHostToDevice, g_rt.stream),
               return -1);
    }
    return 0;
}

static const float *forward_token_one(InferenceState *s, int token)
{
    follow_sft(s);
    if (!s || ensure_graphs(s) != 0) return NULL;
    if (s->cur_len >= s->max_seq) { fprintf(stderr, "[FastGen] KV cache is full (%d positions)\n", s->max_seq); return NULL; }
    if (token < 0 || token >= s->V) { fprintf(stderr, "[FastGen] token id %d out of range\n", token); return NULL; }
    uint32_t t = (uint32_t)token;
    /* prompt_len beyond pos+1 keeps the graph from overwriting caller-supplied ids */
    if (set_control(s, s->cur_len, s->max_seq + 2, &t, s->cur_len, 1) != 0) return NULL;
    CU_TRY(cudaGraphLaunch(s->g_full, g_rt.stream), return NULL);
    if (s->fused && s->tp_size > 1) {
        /* the whole-token kernel leaves every rank's logits shard on that rank: fetch each from its owner
         * (the pick exchange at the end of the kernel has ordered the peers' stores before this point) */
        for (int p = 0; p < s->tp_size; ++p)
            CU_TRY(cudaMemcpyAsync(s->h_logits + (size_t)p * s->V_l, s->peer[p] + s->off_logits + (size_t)p * s->V_l * 4,
                                   (size_t)s->V_l * 4, cudaMemcpyDeviceToHost, g_rt.stream), return NULL);
    } else {
        CU_TRY(cudaMemcpyAsync(s->h_logits, s->comm + s->off_logits, (size_t)s->V * 4, cudaMemcpyDeviceToHost, g_rt.stream),
               return NULL);
    }
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return NULL);
    s->cur_len++;
    return s->h_logits;
}

static int is_eos(const InferenceState *s, int tok)
{
    for (int e = 0; e < s->n_eos; ++e) if (tok == s->eos[e]) return 1;
    return 0;
}

static int generate_one(InferenceState *s, const uint32_t *prompt, int prompt_len, uint32_t *out, int max_gen_len)
{
    if (!s || !prompt || !out || prompt_len <= 0 || max_gen_len <= 0) return 0;
    follow_sft(s);
    if (ensure_graphs(s) != 0) return 0;
    if (prompt_len > s->max_seq) {
        fprintf(stderr, "[FastGen] prompt of %d tokens exceeds the KV cache (%d)\n", prompt_len, s->max_seq);
        return 0;
    }
    for (int i = 0; i < prompt_len; ++i)
        if (prompt[i] >= (uint32_t)s->V) { fprintf(stderr, "[FastGen] prompt token %u out of range\n", prompt[i]); return 0; }
    s->cur_len = 0;
    const int P = prompt_len;
    if (set_control(s, 0, P, prompt, 0, P) != 0) return 0;

    fprintf(stderr, "[FastGen] Prefilling %d tokens...\n", P);
    double t0 = now_ms();
    for (int i = 0; i < P - 1; ++i) CU_TRY(cudaGraphLaunch(s->g_nolm, g_rt.stream), return 0);
    CU_TRY(cudaGraphLaunch(s->g_full, g_rt.stream), return 0);
    CU_TRY(cudaMemcpyAsync(&s->h_tok[0], s->d_tokens + P, 4, cudaMemcpyDeviceToHost, g_rt.stream), return 0);
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return 0);
    s->cur_len = P;
    s->last_prefill_ms = now_ms() - t0;
    fprintf(stderr, "[FastGen] Prefill: %.0f ms (%.1f tok/s)\n", s->last_prefill_ms, P * 1000.0 / s->last_prefill_ms);

    int next = s->h_tok[0];
    out[0] = (uint32_t)next;
    int n_gen = 1;

    fprintf(stderr, "[FastGen] Decoding...\n");
    t0 = now_ms();
    /* Forward number i (1-based) consumes the id at position P+i-1 and leaves the id for position P+i on the
     * device. The host only needs ids to test for EOS and to fill `out`, so it lets the forwards run ahead and
     * reads the ids back in groups: one small copy and one event per TOK_BATCH forwards (a copy after every
     * forward sits between two launches on the stream and cost 0.8 % of the decode rate), two groups in flight.
     * After an EOS id the forwards already launched are simply not used. */
    enum { TOK_BATCH = 4 };
    int max_fw = max_gen_len - 1;
    if (max_fw > s->max_seq - P) max_fw = s->max_seq - P;
    int launched = 0, done = 0, copied = 0, b_enq = 0, b_done = 0, stop = is_eos(s, next) || max_fw <= 0;
    int batch_n[4] = {0, 0, 0, 0};
    while (!stop) {
        while (launched < max_fw && b_enq - b_done < 2) {
            CU_TRY(cudaGraphLaunch(s->g_full, g_rt.stream), return n_gen);
            launched++;
            if (launched - copied == TOK_BATCH || launched == max_fw) {
                const int slot = b_enq & 3, n = launched - copied;
                CU_TRY(cudaMemcpyAsync(&s->h_tok[8 + slot * TOK_BATCH], s->d_tokens + P + copied + 1, (size_t)n * 4,
                                       cudaMemcpyDeviceToHost, g_rt.stream), return n_gen);
                CU_TRY(cudaEventRecord(s->tok_ev[slot], g_rt.stream), return n_gen);
                batch_n[slot] = n;
                copied = launched;
                b_enq++;
            }
        }
        if (b_done == b_enq) break;                          /* every forward has been launched and read */
        const int slot = b_done & 3;
        CU_TRY(cudaEventSynchronize(s->tok_ev[slot]), return n_gen);
        for (int i = 0; i < batch_n[slot] && !stop; ++i) {
            next = s->h_tok[8 + slot * TOK_BATCH + i];
            done++;
            out[n_gen++] = (uint32_t)next;
            if (n_gen % 10 == 0) {
                double el = now_ms() - t0;
                fprintf(stderr, "[FastGen]   %d tokens, %.1f tok/s\n", n_gen - 1, (n_gen - 1) * 1000.0 / el);
            }
            if (is_eos(s, next)) stop = 1;
        }
        b_done++;
    }
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return n_gen);
    s->cur_len = P + done;
    s->last_decode_ms = now_ms() - t0;
    s->last_n_decoded = n_gen - 1;
    if (s->last_n_decoded > 0)
        fprintf(stderr, "[FastGen] Decode: %d tokens in %.0f ms (%.1f tok/s, %.2f ms/tok)\n", s->last_n_decoded,
                s->last_decode_ms, s->last_n_decoded * 1000.0 / s->last_decode_ms, s->last_decode_ms / s->last_n_decoded);
    if (llmb200_state_error(s)) fprintf(stderr, "[FastGen] a device-side wait timed out; results are invalid\n");
    return n_gen;
}

/* ------------------------------------------------------------ single-process tensor parallelism
 *
 * LLMB200_TP=k (2, 4 or 8) makes the reference's own calls -- inference_state_create, inference_generate,
 * inference_forward_token, ... -- run k-way tensor parallel inside the calling process: one host thread per
 * GPU (the caller's thread drives rank 0 on its current device, devices dev+1 .. dev+k-1 hold the other
 * ranks), each with its own state, stream and upload staging, exactly the states a one-process-per-GPU
 * launch builds. The exchange regions are plain peer pointers (cudaDeviceEnablePeerAccess) instead of IPC
 * mappings. Every rank runs the same host loop on the same prompt and meets the others on the device. */

enum { G_CREATE_QWEN3, G_CREATE_GEMMA3, G_GENERATE, G_FORWARD, G_FREE };

typedef struct {
    int op, rank, world, dev, rc;
    InferenceState *s, **all;
    void *model;
    int max_seq, use_fp16, token;
    const uint32_t *prompt;
    uint32_t *out;
    int prompt_len, max_gen;
    const float *logits;
    pthread_barrier_t *bar;
} GroupJob;

static int single_process_tp(void)
{
    if (g_tp_size > 0 || getenv("LLMB200_TP_SIZE")) return 1;      /* one process per GPU: the caller places the ranks */
    const char *e = getenv("LLMB200_TP");
    const int k = e ? atoi(e) : 1;
    return (k == 2 || k == 4 || k == 8) ? k : 1;
}

static void *group_thread(void *arg)
{
    GroupJob *j = arg;
    j->rc = -1;
    if (cudaSetDevice(j->dev) != cudaSuccess) {
        fprintf(stderr, "[FastGen] rank %d: cannot use device %d\n", j->rank, j->dev);
        if (j->op <= G_CREATE_GEMMA3) { pthread_barrier_wait(j->bar); pthread_barrier_wait(j->bar); }
        return NULL;
    }
    switch (j->op) {
    case G_CREATE_QWEN3:
    case G_CREATE_GEMMA3: {
        g_tp_rank = j->rank; g_tp_size = j->world;
        InferenceState *s = j->op == G_CREATE_QWEN3 ? create_qwen3_one(j->model, j->max_seq, j->use_fp16)
                                                     : create_gemma3_one(j->model, j->max_seq, j->use_fp16);
        g_tp_rank = -1; g_tp_size = -1;
        j->all[j->rank] = s;
        pthread_barrier_wait(j->bar);                    /* every rank has built (or failed to build) its state */
        int ok = 1;
        for (int r = 0; r < j->world; ++r) if (!j->all[r]) ok = 0;
        if (ok) {
            for (int r = 0; r < j->world && ok; ++r) {
                if (r == j->rank) continue;
                int dev_r = 0;
                struct cudaPointerAttributes at;
                if (cudaPointerGetAttributes(&at, j->all[r]->comm) != cudaSuccess) { ok = 0; break; }
                dev_r = at.device;
                cudaError_t e = cudaDeviceEnablePeerAccess(dev_r, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); e = cudaSuccess; }
                if (e != cudaSuccess) {
                    fprintf(stderr, "[FastGen] no peer access from device %d to device %d: %s\n", j->dev, dev_r, cudaGetErrorString(e));
                    ok = 0;
                    break;
                }
                s->peer[r] = j->all[r]->comm;
            }
            if (ok) { s->local_peers = 1; s->connected = 1; free_graphs(s); j->rc = 0; }
        }
        pthread_barrier_wait(j->bar);                    /* nobody launches before everybody is connected */
        j->s = s;
        break;
    }
    case G_GENERATE:
        j->rc = generate_one(j->s, j->prompt, j->prompt_len, j->out, j->max_gen);
        break;
    case G_FORWARD:
        j->logits = forward_token_one(j->s, j->token);
        j->rc = j->logits ? 0 : -1;
        break;
    case G_FREE:
        free_one(j->s);
        j->rc = 0;
        break;
    }
    return NULL;
}

/* Runs jobs[0] on the caller's thread and jobs[1..k-1] on one thread each; the caller's device is restored. */
static void group_run(GroupJob *jobs, int k)
{
    pthread_t th[B200_MAX_PEERS];
    int started[B200_MAX_PEERS] = {0};
    int dev0 = 0;
    cudaGetDevice(&dev0);
    for (int r = 1; r < k; ++r) started[r] = pthread_create(&th[r], NULL, group_thread, &jobs[r]) == 0;
    group_thread(&jobs[0]);
    for (int r = 1; r < k; ++r) {
        if (started[r]) pthread_join(th[r], NULL);
        else {
            /* a rank without a thread would leave the others waiting: run it here (slow, but nothing hangs) */
            group_thread(&jobs[r]);
        }
    }
    cudaSetDevice(dev0);
}

static InferenceState *group_create(int op, void *model, int max_seq_len, int use_fp16, int k)
{
    int dev0 = 0, n_dev = 0;
    if (cudaGetDevice(&dev0) != cudaSuccess || cudaGetDeviceCount(&n_dev) != cudaSuccess || dev0 + k > n_dev) {
        fprintf(stderr, "[FastGen] LLMB200_TP=%d needs devices %d..%d; %d visible\n", k, dev0, dev0 + k - 1, n_dev);
        (void)cudaGetLastError();
        return NULL;
    }
    InferenceState *all[B200_MAX_PEERS] = {0};
    GroupJob jobs[B200_MAX_PEERS];
    pthread_barrier_t bar;
    if (pthread_barrier_init(&bar, NULL, (unsigned)k) != 0) return NULL;
    memset(jobs, 0, sizeof(jobs));
    for (int r = 0; r < k; ++r)
        jobs[r] = (GroupJob){ .op = op, .rank = r, .world = k, .dev = dev0 + r, .all = all, .model = model,
                              .max_seq = max_seq_len, .use_fp16 = use_fp16, .bar = &bar };
    group_run(jobs, k);
    pthread_barrier_destroy(&bar);
    int ok = 1;
    for (int r = 0; r < k; ++r) if (!all[r] || jobs[r].rc != 0) ok = 0;
    if (!ok) {
        for (int r = 0; r < k; ++r)
            if (all[r]) { cudaSetDevice(dev0 + r); free_one(all[r]); }
        cudaSetDevice(dev0);
        fprintf(stderr, "[FastGen] building the %d-way tensor-parallel state failed\n", k);
        return NULL;
    }
    InferenceState *g = all[0];
    g->group_n = k;
    for (int r = 0; r < k; ++r) { g->group[r] = all[r]; g->group_dev[r] = dev0 + r; }
    fprintf(stderr, "[FastGen] %d-way tensor parallel on devices %d..%d, one host thread each\n", k, dev0, dev0 + k - 1);
    return g;
}

InferenceState *inference_state_create(llmb200_qwen3_model *m, int max_seq_len, int use_fp16)
{
    const int k = single_process_tp();
    if (m && k > 1) return group_create(G_CREATE_QWEN3, m, max_seq_len, use_fp16, k);
    return create_qwen3_one(m, max_seq_len, use_fp16);
}

InferenceState *inference_state_create_gemma3(llmb200_gemma3_model *m, int max_seq_len, int use_fp16)
{
    const int k = single_process_tp();
    if (m && k > 1) return group_create(G_CREATE_GEMMA3, m, max_seq_len, use_fp16, k);
    return create_gemma3_one(m, max_seq_len, use_fp16);
}

void inference_state_free(InferenceState *s)
{
    if (!s) return;
    if (s->group_n <= 1) { free_one(s); return; }
    const int k = s->group_n;
    GroupJob jobs[B200_MAX_PEERS];
    memset(jobs, 0, sizeof(jobs));
    for (int r = 0; r < k; ++r) jobs[r] = (GroupJob){ .op = G_FREE, .rank = r, .world = k, .dev = s->group_dev[r], .s = s->group[r] };
    group_run(jobs, k);
}

const float *inference_forward_token(InferenceState *s, int token)
{
    if (!s || s->group_n <= 1) return forward_token_one(s, token);
    const int k = s->group_n;
    GroupJob jobs[B200_MAX_PEERS];
    memset(jobs, 0, sizeof(jobs));
    for (int r = 0; r < k; ++r)
        jobs[r] = (GroupJob){ .op = G_FORWARD, .rank = r, .world = k, .dev = s->group_dev[r], .s = s->group[r], .token = token };
    group_run(jobs, k);
    for (int r = 0; r < k; ++r) if (jobs[r].rc != 0) return NULL;
    return jobs[0].logits;
}

int inference_generate(InferenceState *s, const uint32_t *prompt, int prompt_len, uint32_t *out, int max_gen_len)
{
    if (!s || s->group_n <= 1) return generate_one(s, prompt, prompt_len, out, max_gen_len);
    if (!prompt || !out || prompt_len <= 0 || max_gen_len <= 0) return 0;
    const int k = s->group_n;
    GroupJob jobs[B200_MAX_PEERS];
    uint32_t *tmp = malloc((size_t)(k - 1) * (size_t)max_gen_len * sizeof(uint32_t));
    if (!tmp) return 0;
    memset(jobs, 0, sizeof(jobs));
    for (int r = 0; r < k; ++r)
        jobs[r] = (GroupJob){ .op = G_GENERATE, .rank = r, .world = k, .dev = s->group_dev[r], .s = s->group[r], .prompt = prompt,
                              .prompt_len = prompt_len, .out = r == 0 ? out : tmp + (size_t)(r - 1) * max_gen_len,
                              .max_gen = max_gen_len };
    group_run(jobs, k);
    int n = jobs[0].rc;
    /* every rank folds the same arg-max: a rank that disagrees means the exchange went wrong */
    for (int r = 1; r < k; ++r)
        if (jobs[r].rc != n || memcmp(jobs[r].out, out, (size_t)(n > 0 ? n : 0) * sizeof(uint32_t)) != 0) {
            fprintf(stderr, "[FastGen] rank %d generated different tokens than rank 0; results are invalid\n", r);
            n = 0;
        }
    free(tmp);
    return n;
}

int qwen3_generate_fast(llmb200_qwen3_model *model, const uint32_t *prompt, int prompt_len, uint32_t *out,
                        int max_gen_len, int max_seq_len, int use_fp16)
{
    InferenceState *s = inference_state_create(model, max_seq_len, use_fp16);
    if (!s) return 0;
    int n = inference_generate(s, prompt, prompt_len, out, max_gen_len);
    inference_state_free(s);
    return n;
}

/* Reads the whole file into a NUL-terminated heap buffer (NULL when it cannot be read). */
static char *slurp(const char *path)
{
    FILE *fp = fopen(path, "rb");
    if (!fp) return NULL;
    char *text = NULL;
    long len = -1;
    if (fseek(fp, 0, SEEK_END) == 0) len = ftell(fp);
    if (len >= 0 && len < (16L << 20) && fseek(fp, 0, SEEK_SET) == 0 && (text = malloc((size_t)len + 1)) != NULL) {
        const size_t got = fread(text, 1, (size_t)len, fp);
        text[got] = 0;
    }
    fclose(fp);
    return text;
}

/* The "eos_token_id" member of the config.json that belongs to model_path (the file inside it when it
 * is a directory, else the one beside it): a JSON integer or an array of integers. Stores up to
 * max_eos ids and returns how many; 0 when the file or the member is missing or holds no integer. */
static int parse_eos(const char *model_path, int *eos, int max_eos)
{
    const size_t plen = strlen(model_path);
    char *cfg = malloc(plen + 16);
    if (!cfg) return 0;
    struct stat st;
    size_t dir = plen;                                  /* length of the directory part, without the slash */
    if (!(stat(model_path, &st) == 0 && S_ISDIR(st.st_mode))) {
        while (dir > 0 && model_path[dir - 1] != '/') --dir;
        if (dir > 0) --dir;                             /* "a/b.safetensors" -> "a"; no slash at all -> "" (current directory) */
    }
    memcpy(cfg, model_path, dir);
    strcpy(cfg + dir, dir > 0 || model_path[0] == '/' ? "/config.json" : "config.json");
    char *text = slurp(cfg);
    free(cfg);
    if (!text) return 0;
    int n = 0;
    const char *key = strstr(text, "\"eos_token_id\"");
    if (key) {
        const char *c = key + strlen("\"eos_token_id\"");
        while (*c && *c != ':') ++c;                    /* the member's value follows the colon */
        if (*c == ':') ++c;
        while (*c == ' ' || *c == '\t' || *c == '\r' || *c == '\n') ++c;
        const int is_array = *c == '[';
        if (is_array) ++c;
        /* integers separated by commas and white space, until the array closes (or one integer) */
        while (n < max_eos) {
            while (*c == ' ' || *c == '\t' || *c == '\r' || *c == '\n' || (is_array && *c == ',')) ++c;
            char *after = NULL;
            const long v = strtol(c, &after, 10);
            if (after == c) break;                      /* ']' , end of text or anything that is not a number */
            eos[n++] = (int)v;
            c = after;
            if (!is_array) break;
        }
    }
    free(text);
    return n;
}

void inference_state_load_eos(InferenceState *s, const char *model_path)
{
    if (!s || !model_path) return;
    s->n_eos = parse_eos(model_path, s->eos, 4);
    if (s->n_eos == 0) {
        if (s->mt == MODEL_GEMMA3) { s->eos[0] = 1; s->eos[1] = 106; }
        else { s->eos[0] = 151645; s->eos[1] = 151643; }
        s->n_eos = 2;
    }
    fprintf(stderr, "[FastGen] EOS tokens (%d):", s->n_eos);
    for (int i = 0; i < s->n_eos; ++i) fprintf(stderr, " %d", s->eos[i]);
    fprintf(stderr, "\n");
    for (int r = 1; r < s->group_n; ++r) llmb200_state_set_eos(s->group[r], s->eos, s->n_eos);
}

/* ------------------------------------------------------------ measurement */

float llmb200_state_run_device_steps(InferenceState *s, int n_steps)
{
    if (!s || n_steps <= 0 || ensure_graphs(s) != 0) return -1.0f;
    if (s->cur_len + n_steps > s->max_seq) return -1.0f;
    if (set_control(s, s->cur_len, 0, NULL, 0, 0) != 0) return -1.0f;
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1.0f);
    CU_TRY(cudaEventRecord(s->ev_a, g_rt.stream), return -1.0f);
    for (int i = 0; i < n_steps; ++i) CU_TRY(cudaGraphLaunch(s->g_full, g_rt.stream), return -1.0f);
    CU_TRY(cudaEventRecord(s->ev_b, g_rt.stream), return -1.0f);
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1.0f);
    float ms = -1.0f;
    CU_TRY(cudaEventElapsedTime(&ms, s->ev_a, s->ev_b), return -1.0f);
    s->cur_len += n_steps;
    return ms;
}

float llmb200_state_time_kind(InferenceState *s, int kind, int reps, int *launches)
{
    if (!s || kind < 0 || kind >= K_KINDS || reps <= 0 || ensure_graphs(s) != 0) return -1.0f;
    if (s->cur_len >= s->max_seq) return -1.0f;
    if (set_control(s, s->cur_len, 0, NULL, 0, 0) != 0) return -1.0f;
    s->only_kind = kind;
    int rc = enqueue_token(s, kind == K_LM, 0);                 /* warm-up pass, untimed */
    const unsigned long long before = b200_launch_count(0);
    if (rc == 0) rc = (int)cudaEventRecord(s->ev_a, g_rt.stream);
    for (int i = 0; i < reps && rc == 0; ++i) rc = enqueue_token(s, kind == K_LM, 0);
    if (rc == 0) rc = (int)cudaEventRecord(s->ev_b, g_rt.stream);
    s->only_kind = -1;
    if (launches) *launches = (int)(b200_launch_count(0) - before);
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1.0f);
    if (rc != 0) return -1.0f;
    float ms = -1.0f;
    CU_TRY(cudaEventElapsedTime(&ms, s->ev_a, s->ev_b), return -1.0f);
    return ms;
}

int llmb200_state_profile_token(InferenceState *s, float *ms, int *launches)
{
    if (!s || !ms || !launches || ensure_graphs(s) != 0) return B200_E_BADARG;
    if (s->cur_len + 1 > s->max_seq) return B200_E_STATE;
    const int need = 2 * (5 * s->L + 1);
    if (!s->prof_ev) {
        s->prof_ev = calloc((size_t)need, sizeof(cudaEvent_t));
        s->prof_kind = calloc((size_t)need / 2, sizeof(int));
        if (!s->prof_ev || !s->prof_kind) return -1;
        for (int i = 0; i < need; ++i) CU_TRY(cudaEventCreate(&s->prof_ev[i]), return -1);
        s->prof_cap = need;
    }
    if (set_control(s, s->cur_len, 0, NULL, 0, 0) != 0) return -1;
    s->prof_n = 0;
    cudaEvent_t *ev = s->prof_ev;
    s->prof_on = 1;
    int rc = enqueue_token(s, 1, 0);
    s->prof_on = 0;
    const int n = s->prof_n;
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return -1);
    if (rc != 0) return rc;
    for (int i = 0; i < K_KINDS; ++i) { ms[i] = 0.0f; launches[i] = 0; }
    for (int i = 0; i + 1 < n; i += 2) {
        float t = 0.0f;
        CU_TRY(cudaEventElapsedTime(&t, ev[i], ev[i + 1]), return -1);
        ms[s->prof_kind[i / 2]] += t;
        launches[s->prof_kind[i / 2]]++;
    }
    s->cur_len++;
    return 0;
}

size_t llmb200_state_export_weight(InferenceState *s, int layer, int which, void *buf, size_t cap)
{
    if (!s) return 0;
    const PackedMat *m = NULL;
    if (which == 4) m = &s->lm;
    else if (layer >= 0 && layer < s->L) {
        Layer *ly = &s->layers[layer];
        m = which == 0 ? &ly->qkv : which == 1 ? &ly->o : which == 2 ? &ly->gateup : which == 3 ? &ly->down : NULL;
    }
    if (!m) return 0;
    const size_t bytes = s->wtype == B200_WT_Q8 ? (size_t)m->rows * (m->cols / 32) * 34 : (size_t)m->rows * m->cols * 2;
    if (!buf) return bytes;
    if (cap < bytes) return 0;
    if (s->wtype == B200_WT_Q8) {
        void *d = NULL;
        CU_TRY(cudaMalloc(&d, bytes), return 0);
        int rc = b200_q8_unpack_blocks(m->w, m->stride, m->rows, m->cols, d, g_rt.stream);
        if (rc == 0) rc = (int)cudaMemcpyAsync(buf, d, bytes, cudaMemcpyDeviceToHost, g_rt.stream);
        if (rc == 0) rc = (int)cudaStreamSynchronize(g_rt.stream);
        cudaFree(d);
        return rc == 0 ? bytes : 0;
    }
    CU_TRY(cudaStreamSynchronize(g_rt.stream), return 0);
    CU_TRY(cudaMemcpy2D(buf, (size_t)m->cols * 2, m->w, (size_t)m->stride, (size_t)m->cols * 2, (size_t)m->rows,
                        cudaMemcpyDeviceToHost), return 0);
    return bytes;
}
