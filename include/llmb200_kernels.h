/*
 * llmb200_kernels.h -- thin C ABI over the sm_100a kernels of the decode path.
 *
 * Plain pointers and sizes only. Every pointer named d_* is CUDA device memory
 * on the current device; `stream` is a cudaStream_t passed as void*. Functions
 * return 0 on success, a positive cudaError_t value when CUDA reports one and
 * a negative B200_E_* code for rejected arguments. Nothing here allocates
 * device memory.
 *
 * Each launcher states which reference dispatch(es) it stands in for
 * (src/nn/fast_metal.m line of the metal_enqueue_* function, and the kernel in
 * shaders/q8_kernels.metal).
 *
 * Packed weight layout ("row-sliced"):
 *   Q8_0  row r = cols int8 quants, then cols/32 binary16 scales; rows are
 *         row_stride bytes apart, row_stride = round_up(34*cols/32, 16).
 *   F16   row r = cols binary16 values; row_stride = round_up(2*cols, 16).
 * Values are exactly those of the reference's 34-byte block stream / half
 * array; only the placement differs, so that every 16-byte load of a row is
 * aligned and a warp reads 512 contiguous bytes.
 */
#ifndef LLMB200_KERNELS_H
#define LLMB200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_E_BADARG   (-1)
#define B200_E_TOOLARGE (-2)
#define B200_E_STATE    (-3)

#define B200_WT_Q8  0
#define B200_WT_F16 1

#define B200_MAX_PEERS 8

/* Bytes between consecutive rows of a packed matrix with `cols` columns. */
size_t b200_packed_row_stride(int wtype, int cols);

/* fp32 [rows, cols] (leading dimension ld floats, device) -> packed Q8_0 rows.
 * Source row r lands in packed row dst_row0 + r*dst_row_step.
 * Replaces quantize_row_q8/wmat_create_q8 (src/nn/wmat.c:19-61); bit-exact. */
int b200_q8_pack(const float *d_src, long long ld, int rows, int cols,
                 void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step,
                 void *stream);
/* Same for F16 (src/nn/wmat.c:63-75). */
int b200_f16_pack(const float *d_src, long long ld, int rows, int cols,
                  void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step,
                  void *stream);
/* Packed Q8_0 rows -> the reference's canonical stream of 34-byte blocks
 * {u16 d; i8 qs[32]} (src/nn/wmat.c:14-17), rows*cols/32 blocks, row-major. */
int b200_q8_unpack_blocks(const void *d_packed, long long row_stride, int rows, int cols,
                          void *d_blocks, void *stream);

/* ------------------------------------------------------------------------
 * Fused matrix-vector product  y = W . f(x)
 *
 * One launch covers what the reference enqueues as rms_norm + q8_matvec /
 * f16_matvec (+ residual_add, silu_mul / gelu_mul, CPU embedding copy, CPU
 * argmax): src/nn/fast_metal.m:253-289, 309-341, 428-462 and
 * src/nn/fast_inference.c:386-392, 469-476.
 *
 * Input assembly (in_mode), all in fp32:
 *   B200_IN_VEC    x = in_vec[cols]
 *   B200_IN_RESID  h = resid_in + S, S = sum over n_slots of slots[s][0..cols)
 *                  (if slot_norm_gamma: S <- rmsnorm(S) * slot_norm_gamma first);
 *                  block 0 stores h to resid_out; x = h
 *   B200_IN_EMBED  h = emb[tokens[*pos]][0..cols) * emb_scale; stored to
 *                  resid_out by block 0; x = h
 * then, if norm_gamma != NULL, x <- x * rsqrt(mean(x^2)+eps) * norm_gamma.
 *
 * Output (out_mode):
 *   B200_OUT_STORE  out[p][out_offset + r] = y[r] for every peer p < n_out
 *   B200_OUT_GLU    rows come in (gate, up) pairs: out[0][out_offset + r/2] =
 *                   act(y[r]) * y[r+1], act = SiLU (0) or tanh-GELU (1)
 * With d_argmax_scratch != NULL (B200_OUT_STORE only) the launch also leaves
 * the largest y[r] and its row index plus out_offset (first one on ties, as
 * the reference's argmax) in *d_argmax_val[p] / *d_argmax_idx[p], p < n_argmax_out.
 *
 * Tensor-parallel hand-shake (all optional, n_wait = 0 / n_signal = 0 to
 * disable): before reading `slots` the kernel waits, with an iteration limit,
 * until wait_flags[i] >= E for i < n_wait, E = *epoch * epoch_mul + epoch_add;
 * after its last store it writes E into signal_flags[p][signal_index], p < n_signal. A wait
 * that runs out sets *err = 1 and the kernel carries on without hanging.
 * ---------------------------------------------------------------------- */
enum { B200_IN_VEC = 0, B200_IN_RESID = 1, B200_IN_EMBED = 2 };
enum { B200_OUT_STORE = 0, B200_OUT_GLU = 1 };

typedef struct b200_matvec_args {
    /* weights */
    const void *d_w; long long row_stride; int rows, cols, wtype;
    /* input assembly */
    int in_mode;
    const float *d_in_vec;
    const float *d_resid_in; float *d_resid_out;
    const float *d_slots; int n_slots; long long slot_stride;   /* floats between slots */
    const float *d_slot_norm_gamma;
    const float *d_emb; const int *d_tokens; const int *d_pos; float emb_scale;
    int emb_rows;                  /* rows of d_emb; an id outside [0, emb_rows) is read as id 0 */
    const float *d_norm_gamma; float eps;
    /* output */
    int out_mode, act;
    float *d_out[B200_MAX_PEERS]; int n_out; long long out_offset;
    float *d_argmax_scratch;                       /* 2 words per block, or NULL: no argmax */
    float *d_argmax_val[B200_MAX_PEERS];           /* [0] of each receives the largest y */
    int   *d_argmax_idx[B200_MAX_PEERS];           /* [0] of each receives its row + out_offset */
    int    n_argmax_out;
    /* bookkeeping done by the last block to finish */
    unsigned *d_ticket;            /* one zero-initialised word; required when any of the below is used */
    int advance_pos;               /* (*d_pos_rw)++ */
    int *d_pos_rw;
    int advance_epoch;             /* *d_epoch_rw = *d_epoch + 1 */
    unsigned *d_epoch_rw;
    int *d_next_token; const int *d_prompt_len;   /* tokens[pos+1] = argmax unless pos+1 < *prompt_len */
    /* tensor-parallel flags */
    const unsigned *d_wait_flags; int n_wait;
    unsigned *d_signal_flags[B200_MAX_PEERS]; int n_signal, signal_index;
    const unsigned *d_epoch; int epoch_mul, epoch_add;   /* flag value = *d_epoch * epoch_mul + epoch_add */
    int *d_err;
    /* launch shape: 0 = choose (a multiple of the SM count) */
    int grid;
    int use_pdl;                   /* programmatic dependent launch: prefetch weights under the previous kernel's tail */
    /* optional: block 0 also stores the assembled (summed, normalised) input vector here, cols floats --
     * what a LoRA side path multiplies by A (src/nn/fast_inference.c:406-421 reads mb_ln_out) */
    float *d_in_copy;
    /* iterations of the bounded wait on d_wait_flags before the kernel gives up and sets *d_err = 1
     * (0 = default, about a second) */
    int spin_limit;
} b200_matvec_args;

int b200_matvec(const b200_matvec_args *a, void *stream);

/* ------------------------------------------------------------------------
 * Decode attention for one new token over an F16 KV cache, split over the
 * sequence. One launch covers per_head_rms_norm(q), per_head_rms_norm(k),
 * rope, kv_cache_store and attention of the reference
 * (src/nn/fast_metal.m:343-426; shaders/q8_kernels.metal:165-331).
 *
 *   qkv        fp32 [n_q*hd | n_kv*hd | n_kv*hd] of the new token (unnormalised)
 *   q/k_gamma  [hd] or NULL (no QK-norm)
 *   inv_freq   [hd/2] fp32, 1/theta^(2d/hd); angle = pos * inv_freq[d]
 *   k/v_cache  binary16 [n_kv][max_seq][hd]; row *pos is written by this launch
 *   out        fp32 [n_q*hd]
 *   scratch    fp32, b200_attn_scratch_floats(n_q, hd, n_split) floats
 *   tickets    n_kv zero-initialised words
 * Keys 0..*pos are attended (no window), scores scaled by 1/sqrt(hd). A position outside
 * [0, max_seq) is ignored: nothing is written or read, the output keeps its contents.
 * ---------------------------------------------------------------------- */
typedef struct b200_attn_args {
    const float *d_qkv; const float *d_q_gamma; const float *d_k_gamma; const float *d_inv_freq;
    void *d_k_cache; void *d_v_cache;
    float *d_out; float *d_scratch; unsigned *d_tickets;
    const int *d_pos;
    int n_q, n_kv, hd, max_seq, n_split;
    float eps;
    int use_pdl;
    /* Batched form (several sequences at the same position, one launch): n_items > 1 adds a grid
     * dimension; item i reads d_qkv + i*qkv_item_stride, its own caches at + i*cache_item_stride halves,
     * writes d_out + i*out_item_stride and uses scratch / tickets slice i (b200_attn_scratch_floats and
     * n_kv words per item). 0 or 1 = one sequence. */
    int n_items;
    long long qkv_item_stride, cache_item_stride, out_item_stride;
} b200_attn_args;

size_t b200_attn_scratch_floats(int n_q, int hd, int n_split);
int    b200_attn_decode(const b200_attn_args *a, void *stream);

/* No counterpart in the reference. b200_attn_decode for callers that cannot allocate device memory --
 * a process whose GPU memory was carved up completely at start-up, or a loop that must not risk the
 * device-wide synchronisation a cudaMalloc can cause. a->d_scratch and a->d_tickets are ignored; the
 * partial results go to arrays built into the library (held by every GPU that loads it until the
 * process exits). Limits: n_q * n_split * (hd + 2) <= B200_ATTN_STATIC_SCRATCH_FLOATS and
 * n_kv <= B200_ATTN_STATIC_MAX_KV_HEADS, one sequence per call (n_items <= 1: the batched form indexes
 * scratch and tickets by item); anything larger is refused with B200_E_TOOLARGE and a message on stderr. Calls no cudaMalloc/cudaFree. The first call on a device looks up the arrays'
 * device addresses and should therefore come before any stream capture. All calls share the arrays:
 * two calls whose kernels may overlap on the GPU (different streams) race with each other. */
#define B200_ATTN_STATIC_SCRATCH_FLOATS (1 << 18)      /* 1 MiB */
#define B200_ATTN_STATIC_MAX_KV_HEADS   64
int b200_attn_decode_static(const b200_attn_args *a, void *stream);

/* Last tensor-parallel step of a token: waits for every rank's (value, index)
 * pair, takes the largest (lowest index on ties), stores it as tokens[pos+1]
 * unless that position belongs to the prompt, and advances *pos. */
int b200_tp_argmax_finalize(const float *d_vals, const int *d_idx, int n_ranks,
                            const unsigned *d_wait_flags, const unsigned *d_epoch,
                            int epoch_mul, int epoch_add,
                            int *d_tokens, int *d_pos, const int *d_prompt_len,
                            unsigned *d_epoch_rw, int *d_err, int use_pdl, void *stream);

/* ------------------------------------------------------------------------
 * Whole-token kernel: every matvec and attention step of one token in ONE
 * persistent launch (one block per SM, cooperative). Replaces the reference's
 * single command buffer with its barrier after every dispatch
 * (src/nn/fast_metal.m:223-247; op sequence src/nn/fast_inference.c:394-466).
 *
 * Structure: per layer five stages (q/k/v matvec, attention, o matvec, gate/up
 * matvec, down matvec), then the LM head. A producer warp per block streams
 * the block's share of every stage's weights, in stage order, through one
 * shared-memory ring with bulk copies; it depends on no activation, so it runs
 * ahead across stage boundaries and HBM stays busy while the consumers hand a
 * stage's result over. Hand-over is through "flagged" vectors in global
 * memory: every fp32 value travels as an 8-byte word {value, flag} written
 * with one store, flag = epoch * (n_layers + 1) + layer + 1; a reader polls
 * the word until the flag matches, so data and readiness arrive in the same
 * round trip to L2 and no device-wide barrier exists. The residual stream is
 * kept by every block in its own shared memory and updated from the flagged
 * o / down outputs ("slots", one per tensor-parallel rank, summed in rank
 * order). Every wait is bounded (spin_limit); a wait that runs out raises
 * *d_err and the block's abort flag, after which all later waits fall through.
 *
 * b200_flagged is the 8-byte word: low half the fp32 bits, high half the flag.
 * ---------------------------------------------------------------------- */
typedef unsigned long long b200_flagged;
#define B200_CNT_STRIDE 32
enum { B200_CNT_QKV = 0, B200_CNT_ATTN = 1, B200_CNT_ACT = 2, B200_CNT_SLOTS_O = 3, B200_CNT_SLOTS_DN = 4, B200_CNT_PART = 8 };

/* Pointers of one layer (device table, n_layers entries). Gammas may be NULL where the
 * architecture has none (pre_ff / post_ff outside Gemma3, q/k norm when absent). */
typedef struct b200_token_layer {
    const void *w_qkv, *w_o, *w_gateup, *w_down;     /* packed rows, see the layout note above */
    const float *g_input, *g_post_attn, *g_pre_ff, *g_post_ff, *g_qn, *g_kn;
    /* This layer's rotation for every position: [max_seq][hd/2] pairs (cos, sin) of pos * inv_freq[d], made on
     * the host with the C library's cosf / sinf, i.e. the values the reference's CPU path multiplies with
     * (src/nn/attention.c:757-766). Layers with the same base share one table. */
    const float *rope;
    void *k_cache, *v_cache;                         /* binary16 [n_kv][max_seq][hd] */
} b200_token_layer;

/* Geometry of one matvec stage. rows/cols/row_stride/glu are the caller's; the rest is filled by
 * b200_token_plan. */
typedef struct b200_stage_geom {
    int rows, cols; long long row_stride;
    int glu;                      /* rows are (gate, up) pairs */
    int T, NG, spt;               /* threads per consumer group, groups, 16-byte column slices per thread */
    int rg, rb;                   /* rows per group in a chunk; rows per chunk (one ring slot) = NG * rg */
    int pw;                       /* rows per emission window, a multiple of rb */
    int cta_base, cta_rem;        /* row units per block: base, +1 for the first rem blocks */
    int direct_in;                /* reserved, 0 */
} b200_stage_geom;

enum { B200_ST_QKV = 0, B200_ST_O = 1, B200_ST_GATEUP = 2, B200_ST_DOWN = 3, B200_ST_LM = 4, B200_ST_KINDS = 5 };

typedef struct b200_token_args {
    const b200_token_layer *d_layers; int n_layers;
    int wtype;                                    /* B200_WT_Q8 or B200_WT_F16, all matrices */
    int gemma;                                    /* 1: four-norm block and tanh-GELU (src/nn/fast_inference.c:436-462) */
    b200_stage_geom g[B200_ST_KINDS];
    const void *w_lm; const float *g_final;
    int with_lm;                                  /* 0: stop after the last layer (prompt positions) */
    const float *d_emb; int emb_rows; float emb_scale, eps;
    int d_model, n_q, n_kv, hd, max_seq, n_split;
    /* device control words */
    int *d_pos; int *d_tokens; const int *d_prompt_len; unsigned *d_epoch; int *d_err;
    /* flagged vectors local to this GPU */
    b200_flagged *d_qkv;                          /* [(n_q + 2 n_kv) * hd] */
    b200_flagged *d_attn_part;                    /* [n_q][n_split][hd + 2] */
    b200_flagged *d_attn_out;                     /* [n_q * hd] */
    b200_flagged *d_act;                          /* [g[GATEUP].rows / 2] */
    b200_flagged *d_am;                           /* [2 * blocks]: (best value, row) of each block */
    /* flagged vectors written by every rank: [n_ranks][d_model] each */
    const b200_flagged *d_slots_o, *d_slots_dn;
    b200_flagged *d_peer_slots_o[B200_MAX_PEERS]; /* slot `rank` inside rank p's d_slots_o, p < n_ranks */
    b200_flagged *d_peer_slots_dn[B200_MAX_PEERS];
    const b200_flagged *d_am_rank;                /* [2 * n_ranks] */
    b200_flagged *d_peer_am[B200_MAX_PEERS];      /* entry `rank` inside rank p's d_am_rank */
    int n_ranks, rank;
    /* Arrival counters (hints that spare L2 the polling of 640 threads per block: one thread waits for
     * the count, then everybody reads the flagged words once; the flags stay the proof of validity).
     * Each producer adds the number of words it stored; a reader expects (epoch * n_layers + layer + 1)
     * * words-per-layer. d_counters: B200_CNT_STRIDE words apart: [0] q/k/v rows, [1] attention output,
     * [2] activations, [3] o slots, [4] down slots (all ranks add to these two), [8 + h] partial
     * records of KV head h. Zero-initialised by the caller, never reset. */
    unsigned *d_counters;
    unsigned *d_peer_counters[B200_MAX_PEERS];    /* rank p's d_counters, p < n_ranks */
    float *d_logits; long long logits_offset;     /* logits[logits_offset + r] = row r of this rank's LM-head shard */
    int spin_limit;                               /* iterations of a polling loop before it gives up; 0 = default */
    /* optional trace: 16 words per block and stage, [block][stage][16], 6 stages
     * per layer (q/k/v, attention, o, gate/up, down, one unused) + the LM head: [0] stage entered,
     * [1] input vector complete, [2] first weights in shared memory, [3] thread 0 done with its rows,
     * [4] results stored, [5] producer issued the stage's first copy, [6] its last copy, [7] all warps
     * of the block done with their rows; [8..13] thread 0's first two chunks (data there, rows summed,
     * partials stored), [14] chunks walked, [15] chunks owned. NULL = no trace (a separate kernel instantiation without the
     * timer reads). */
    unsigned long long *d_trace;
    /* filled by b200_token_plan */
    int n_blocks, smem_bytes, scratch_floats;
    int att_keys;                                 /* cache rows the attention stage holds in shared memory at a time */
    /* Bytes of the following stage's weights that a block asks L2 for when it starts streaming a stage
     * (0 = none, the default: the ring alone measured faster on Qwen3-4B). */
    int l2_ahead_bytes;
    /* Iterations one thread per block spends watching an arrival counter before the block polls the flagged
     * words themselves. 0: no counter wait at all, every thread re-reads its own words until their flags
     * match. */
    int counter_spin_limit;
} b200_token_args;

/* Fills the geometry (g[k].T ... direct_in), n_split limits and the launch shape for `n_blocks` blocks
 * (0 = one per SM of the current device). Returns 0, B200_E_BADARG for shapes the kernel does not
 * cover, B200_E_TOOLARGE when a row or the shared-memory budget is exceeded. Host-only arithmetic
 * when n_blocks > 0: callable without a GPU. */
int b200_token_plan(b200_token_args *a, int n_blocks);

/* Host-side replay of the row partition the kernel uses (no GPU needed; for tests): writes up to `cap`
 * triples {first_row, n_rows, window} of block `block`, stage kind `kind`, in the order the producer
 * issues them; returns the number of chunks. */
int b200_token_chunks(const b200_token_args *a, int kind, int block, int *out, int cap);

int b200_decode_token(const b200_token_args *a, void *stream);

/* LoRA side path of one decode token: qkv[0..q_rows) += scaling * B_q (A_q x) and
 * qkv[q_rows + kv_rows ..) += scaling * B_v (A_v x), with x [d_model] the normalised
 * layer input (b200_matvec_args.d_in_copy), A [rank, d_model], B [rows, rank],
 * fp32. Replaces the six per-layer dispatches of src/nn/fast_inference.c:406-421. */
int b200_lora_decode(const float *x, const float *A_q, const float *B_q, const float *A_v, const float *B_v,
                     float *qkv, int d_model, int q_rows, int kv_rows, int rank, float scaling, void *stream);

/* Batched decode: arg-max of each of n_rows logit rows (lowest index on ties,
 * src/nn/fast_inference.c:469-476) written to next_tokens[row] and, when ctl[2]
 * is set, to history[ctl[1]*n_rows + row]; the last row to finish then advances
 * the position ctl[0] (and the step count ctl[1] when recording). done_count is
 * a zeroed scratch word. */
int b200_argmax_rows(const float *logits, int n_rows, int vocab, unsigned *next_tokens, unsigned *history,
                     int max_steps, int *ctl, unsigned *done_count, void *stream);

/* Number of kernel launches issued through this ABI since the last reset
 * (what bench.py reports as gpu_launches). */
unsigned long long b200_launch_count(int reset);
/* For callers that replay captured launches (a CUDA graph): adds the kernel nodes of a replay to the count. */
void b200_launch_count_add(unsigned long long n);

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_KERNELS_H */
