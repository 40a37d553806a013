// Whole-token decode kernel (sm_100a): every matvec and attention stage of one
// token in one persistent, cooperative launch of one block per SM.
//
// Why: a batch-1 token is ~180 dependent stages of a few microseconds of HBM
// time each. As separate kernels each stage pays launch, pipeline fill and
// drain, and the weight stream stops at every boundary. Here
//
//  * a producer warp per block streams the block's rows of EVERY stage, in
//    stage order, through one shared-memory ring (cp.async.bulk + mbarriers).
//    Weights depend on no activation, so the producer runs ahead across stage
//    boundaries: while the consumers hand a stage's result over, the ring is
//    already filling with the next stage's rows and HBM never idles;
//  * results travel between blocks as "flagged" vectors: each fp32 value is
//    stored together with a flag in one 8-byte word, flag = epoch * (L + 1) +
//    layer + 1. A reader polls the word itself, so data and readiness arrive
//    in the same round trip to L2 -- there is no device-wide barrier and no
//    separate "wait, then load" step;
//  * every block keeps the residual stream in its own shared memory and adds
//    the flagged o / down outputs to it (summed in rank order when tensor
//    parallel), so RMSNorm needs no extra exchange;
//  * consumer warps run free of each other inside a stage: each leaves its
//    partial row sums in shared memory and one block-wide barrier per window
//    of rows precedes the fixed-order final sums and the epilogue.
//
// The arithmetic of a row is that of matvec.cu (stream_core.cuh): the
// reference's q8_matvec / f16_matvec (shaders/q8_kernels.metal:10-42, 97-127)
// with rms_norm (:133-157), residual_add (:369-375), silu_mul / gelu_mul
// (:337-363) folded into input assembly and epilogue; the attention stage is
// per_head_rms_norm, rope, kv_cache_store and attention (:165-331) split over
// the sequence as in attention.cu.
//
// Every wait (mbarrier, flagged word) is bounded: when one runs out the block
// raises the error word and its abort flag, after which all later waits return
// at once and the kernel ends; the producer waits (bounded) for its copies in
// flight before it leaves.
#include "stream_core.cuh"
#include "../../include/llmb200_kernels.h"

#include <stdio.h>

extern unsigned long long g_b200_launches;

namespace {

constexpr int TK_NC = 640;                           // consumer threads
constexpr int TK_THREADS = TK_NC + 32;               // + the producer warp
constexpr int TK_NWARP = TK_NC / 32;
constexpr int TK_SLOTS = 7;                          // 7 x 21.25 KB in flight per SM; the rest of shared memory holds activations
constexpr int TK_SLOT_BYTES = 21760;                 // 170 * 128
constexpr int TK_PART = 1024;                        // floats per partial-sum buffer (two buffers)
constexpr int ATT_T = 512;                           // consumer threads that work on an attention item
constexpr int TK_SPIN_DEFAULT = 1 << 20;
constexpr int TK_TRACE_WORDS = 16;



// ---------------------------------------------------------------------------
// Row partition, shared by the producer, the consumers and the host-side replay.
// A stage's rows (in units of `ralign` rows: 2 for gate/up pairs) go to the blocks in contiguous,
// nearly equal ranges; a block's range is cut into windows of at most `pw` rows (pw a multiple of rb);
// a window is cut into chunks of rb = NG * rg consecutive rows (the last one may be short). A chunk
// is one bulk copy into one ring slot; inside a chunk consumer group g owns rows g*rg .. g*rg + rg-1,
// so every warp of the block works on every chunk.
// ---------------------------------------------------------------------------
struct RowRange { int r0, r1; };

__host__ __device__ inline RowRange block_rows(const b200_stage_geom &g, int block)
{
    const int ralign = g.glu ? 2 : 1;
    RowRange r;
    r.r0 = (block * g.cta_base + (block < g.cta_rem ? block : g.cta_rem)) * ralign;
    r.r1 = r.r0 + (g.cta_base + (block < g.cta_rem ? 1 : 0)) * ralign;
    return r;
}

// ---------------------------------------------------------------------------
// Shared-memory layout (byte offsets from the 128-aligned base).
// ---------------------------------------------------------------------------
struct Layout {
    int ring, bars, part, red, flags, layers, resid, scratch, total;
};

__host__ __device__ inline Layout make_layout(int n_layers, int d_model, int scratch_floats)
{
    Layout l;
    int o = 0;
    l.ring = o;    o += TK_SLOTS * TK_SLOT_BYTES;
    l.bars = o;    o += (2 * TK_SLOTS + 2) * 8;      // full[], empty[], the attention stage's K/V barrier
    l.part = o;    o += 2 * TK_PART * 4;
    l.red = o;     o += 2 * 32 * 4 + 2 * 32 * 4;      // two sum buffers, one (value, index) buffer
    l.flags = o;   o += 64;
    l.layers = o;  o += ((n_layers * (int)sizeof(b200_token_layer) + 15) / 16) * 16;
    l.resid = o;   o += ((d_model * 4 + 15) / 16) * 16;
    l.scratch = o; o += ((scratch_floats * 4 + 15) / 16) * 16;
    l.total = o;
    return l;
}

// Scratch floats the attention stage needs besides its K/V staging area: rotated queries, new key and
// value, the per-warp merge buffer and the new q/k/v rows as produced. The staging area (att_keys rows
// of K and of V in binary16 = att_keys * hd floats) follows; the split-merge records reuse it.
__host__ __device__ inline int attention_fixed_floats(int G, int hd)
{
    const int wph = (ATT_T / G) / 32;
    return G * hd + 2 * hd + G * wph * (hd + 2) + (G + 2) * hd;
}

// ---------------------------------------------------------------------------
// Device side. Two rules shape it:
//  * no local memory. With ~220 KB of shared memory per block the L1 that backs the stack is a few
//    KB, so every stack access is a round trip to L2 (about a microsecond while the weights stream).
//    Hence: no structures or arrays passed by reference to out-of-line functions, no dynamically
//    indexed register arrays, no spills; block-wide constants are recomputed from the kernel
//    parameters (constant bank) and the shared-memory base; running counters travel by value.
//  * one layer's code stays resident in the instruction cache (every stage runs its code once per
//    layer, so nothing amortises a miss): loops outside the row loop are kept rolled.
// ---------------------------------------------------------------------------
extern __shared__ __align__(128) unsigned char tk_smem[];

struct Smem {
    unsigned char *ring;
    uint64_t *full, *empty, *att_bar;
    float *part, *red, *resid, *scratch;
    volatile int *flags;                             // [0] abort, [1] always 0
    const b200_token_layer *layers;
};

__device__ __forceinline__ Smem smem_of(const b200_token_args &p)
{
    const Layout lo = make_layout(p.n_layers, p.d_model, p.scratch_floats);
    Smem m;
    m.ring = tk_smem + lo.ring;
    m.full = reinterpret_cast<uint64_t *>(tk_smem + lo.bars);
    m.empty = m.full + TK_SLOTS;
    m.att_bar = m.full + 2 * TK_SLOTS;
    m.part = reinterpret_cast<float *>(tk_smem + lo.part);
    m.red = reinterpret_cast<float *>(tk_smem + lo.red);
    m.resid = reinterpret_cast<float *>(tk_smem + lo.resid);
    m.scratch = reinterpret_cast<float *>(tk_smem + lo.scratch);
    m.flags = reinterpret_cast<volatile int *>(tk_smem + lo.flags);
    m.layers = reinterpret_cast<const b200_token_layer *>(tk_smem + lo.layers);
    return m;
}

__device__ __forceinline__ int spin_of(const b200_token_args &p) { return p.spin_limit > 0 ? p.spin_limit : TK_SPIN_DEFAULT; }
// Iteration limit of a wait on an arrival counter: none at all when the readers poll the data directly.
__device__ __forceinline__ int cspin_of(const b200_token_args &p) { return p.counter_spin_limit; }

// Where element i of a stage's input vector (residual, norm weights, flagged input) lives in shared memory.
// A consumer thread later pulls 16 consecutive elements (64 bytes) into registers with 16-byte loads; with
// the elements in natural order the eight lanes of a load phase would hit the same two bank groups (four-way
// conflict, ~1 us per stage). Exchanging the 16-byte chunks inside each 64-byte group by a pattern that
// changes every 128 bytes spreads them over all banks. i and swz(i) share their 16-byte chunk offset, so
// float2/float4 accesses stay whole; the pattern repeats every 128 elements.
__device__ __forceinline__ int swz(int i) { return i ^ (((i >> 5) & 3) << 2); }

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void raise(volatile int *flags, int *d_err, int code)
{
    flags[0] = 1;
    if (d_err) *d_err = code;
}

// mbarrier wait that ends as soon as the block's abort flag is up.
__device__ __forceinline__ bool mbar_wait_abort(uint64_t *b, unsigned parity, volatile int *abort_flag, int limit)
{
#pragma unroll 1
    for (int it = 0; it < limit; ++it) {
        if (mbar_try_wait(b, parity)) return true;
        if ((it & 63) == 63 && *abort_flag) return false;
    }
    return false;
}

// Flag-carrying words, arrival counters: relaxed accesses at device scope, or at system scope (MULTI)
// when other GPUs write into this one's vectors and counters.
template <bool MULTI>
__device__ __forceinline__ void fl_store(b200_flagged *p, float v, unsigned flag)
{
    const unsigned long long w = ((unsigned long long)flag << 32) | (unsigned long long)__float_as_uint(v);
    if (MULTI) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
    else asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

// Arrival counters: a producer adds the number of words it has stored, one thread of a reading block
// waits for the expected total. The counter is only a hint that keeps hundreds of threads from
// polling L2 while nothing is there yet -- validity is proved by the flags of the words themselves, so
// no fence orders the stores before the count and a wait that runs out simply falls through to the
// flagged polls (whose limit raises the error).
template <bool MULTI>
__device__ __forceinline__ void cnt_add(unsigned *cnt, unsigned n)
{
    if (MULTI) asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(n) : "memory");
    else asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(n) : "memory");
}
template <bool MULTI>
__device__ __forceinline__ void cnt_wait(const unsigned *cnt, unsigned target, volatile int *flags, int spin)
{
#pragma unroll 1
    for (int it = 0; it < spin; ++it) {
        unsigned v;
        if (MULTI) asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        else asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        if ((int)(v - target) >= 0) return;
        if ((it & 31) == 31 && flags[0]) return;
        __nanosleep(20);
    }
}

// Reads N pairs of flagged words: pair k sits (k / INNER) * STEP + (k % INNER) * 2 words after the first
// (INNER = 1: one pair every STEP words; INNER = 2: two adjacent pairs, i.e. four consecutive words, every
// STEP words). Only the first `count` pairs exist (the others read as zero). All loads of a round are
// issued before the first flag is looked at, so a ready vector costs one round trip to L2 however many
// words a thread needs; a round with a stale flag is repeated as a whole. On a timeout the abort flag goes
// up and the values read as zero.
template <int N, int STEP, bool MULTI, int INNER = 1>
__device__ __forceinline__ void fl_poll(const b200_flagged *base, int count, unsigned flag, float (&a)[N], float (&b)[N],
                                        volatile int *flags, int *d_err, int spin)
{
#pragma unroll 1
    for (int it = 0;; ++it) {
        unsigned long long v0[N], v1[N];
#pragma unroll
        for (int k = 0; k < N; ++k) {
            v0[k] = 0ull; v1[k] = 0ull;
            if (k < count) {
                const b200_flagged *src = base + (size_t)(k / INNER) * STEP + (k % INNER) * 2;
                if (MULTI) asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(v0[k]), "=l"(v1[k]) : "l"(src) : "memory");
                else asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(v0[k]), "=l"(v1[k]) : "l"(src) : "memory");
            }
        }
        bool ok = true;
#pragma unroll
        for (int k = 0; k < N; ++k) {
            ok = ok && (k >= count || ((unsigned)(v0[k] >> 32) == flag && (unsigned)(v1[k] >> 32) == flag));
            a[k] = __uint_as_float((unsigned)v0[k]);
            b[k] = __uint_as_float((unsigned)v1[k]);
        }
        if (ok) return;
        if (it >= spin || ((it & 31) == 0 && flags[0])) break;       // an aborted block no longer waits
        if (it > 4) __nanosleep(40);
    }
    raise(flags, d_err, 5);
#pragma unroll
    for (int k = 0; k < N; ++k) { a[k] = 0.0f; b[k] = 0.0f; }
}

// The same with the distance between groups of INNER pairs given at run time (the slots of the tensor-
// parallel ranks lie d_model words apart).
template <int N, bool MULTI, int INNER>
__device__ __forceinline__ void fl_poll_step(const b200_flagged *base, size_t step, int count, unsigned flag, float (&a)[N], float (&b)[N],
                                             volatile int *flags, int *d_err, int spin)
{
#pragma unroll 1
    for (int it = 0;; ++it) {
        unsigned long long v0[N], v1[N];
#pragma unroll
        for (int k = 0; k < N; ++k) {
            v0[k] = 0ull; v1[k] = 0ull;
            if (k < count) {
                const b200_flagged *src = base + (size_t)(k / INNER) * step + (k % INNER) * 2;
                if (MULTI) asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(v0[k]), "=l"(v1[k]) : "l"(src) : "memory");
                else asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(v0[k]), "=l"(v1[k]) : "l"(src) : "memory");
            }
        }
        bool ok = true;
#pragma unroll
        for (int k = 0; k < N; ++k) {
            ok = ok && (k >= count || ((unsigned)(v0[k] >> 32) == flag && (unsigned)(v1[k] >> 32) == flag));
            a[k] = __uint_as_float((unsigned)v0[k]);
            b[k] = __uint_as_float((unsigned)v1[k]);
        }
        if (ok) return;
        if (it >= spin || ((it & 31) == 0 && flags[0])) break;       // an aborted block no longer waits
        if (it > 4) __nanosleep(40);
    }
    raise(flags, d_err, 5);
#pragma unroll
    for (int k = 0; k < N; ++k) { a[k] = 0.0f; b[k] = 0.0f; }
}

// Sum over the consumer threads; every thread gets it. One block-wide barrier. `buf` (0 or 1) picks
// the exchange buffer: two calls on the same buffer must have another consumer barrier between them.
__device__ __forceinline__ float cons_sum(float v, float *red, int buf, int tid)
{
    v = warp_sum(v);
    float *r = red + buf * 32;
    if ((tid & 31) == 0) r[tid >> 5] = v;
    named_barrier(1, TK_NC);
    // 20 partials, fetched with five 16-byte loads and added in warp order
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < TK_NWARP; w += 4) {
        const float4 v4 = *reinterpret_cast<const float4 *>(r + w);
        tot += v4.x; tot += v4.y; tot += v4.z; tot += v4.w;
    }
    return tot;
}
static_assert(TK_NWARP % 4 == 0, "cons_sum reads the warp partials four at a time");

// Sum of the nwg warp partials of one row, in warp order; the loads go out four at a time.
__device__ __forceinline__ float row_sum(const float *pr, int nwg)
{
    float y = 0.0f;
#pragma unroll 1
    for (int w = 0; w < nwg; w += 4) {
        const float a = pr[w], b = w + 1 < nwg ? pr[w + 1] : 0.0f, c = w + 2 < nwg ? pr[w + 2] : 0.0f, d = w + 3 < nwg ? pr[w + 3] : 0.0f;
        y += a; y += b; y += c; y += d;
    }
    return y;
}

// ---------------------------------------------------------------------------
// A matvec stage, consumer side, in three out-of-line pieces that exchange nothing but scalars and
// shared memory: (1) the input vector: stage_residual (residual update + RMS statistics; the norm
// weights are parked in shared memory) or stage_vector (a flagged vector fetched once per block);
// (2) stage_rows: this thread's slices of x from shared memory into registers, then the block's rows
// of one window from the ring, warp partials into shared memory; (3) stage_emit: final sums and the
// epilogue of the window. kind selects what is read and written (l is the layer, n_layers for the
// LM head).
// ---------------------------------------------------------------------------

// Residual update of the q/k/v, gate/up and LM-head stages:
//   residual <- embedding row (first stage of a token) | residual + sum over ranks of the slots
// (the sum is RMS-normalised first where the architecture has post norms), and the RMS statistics of
// the new residual. Leaves the stage's norm weights in scratch[D .. 2D). Returns 1/sqrt(mean(r^2)+eps).
template <bool MULTI>
__device__ __forceinline__ float stage_residual(const b200_token_args &p, int kind, int l, unsigned ep, unsigned long long *trace)
{
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const int tid = threadIdx.x, D = p.d_model, L = p.n_layers;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    const unsigned cnt_mul = ep * (unsigned)L + (unsigned)l + 1u;
    const unsigned words_slots = (unsigned)(D * p.n_ranks);
    const b200_token_layer *ly = sm.layers + (l < L ? l : L - 1);
    const float *norm_gamma, *slot_gamma;
    const b200_flagged *slots;
    const unsigned *in_cnt;
    unsigned slots_flag, target;
    if (kind == B200_ST_GATEUP) {
        norm_gamma = p.gemma ? ly->g_pre_ff : ly->g_post_attn;
        slot_gamma = p.gemma ? ly->g_post_attn : nullptr;
        slots = p.d_slots_o; slots_flag = flag;
        in_cnt = p.d_counters + B200_CNT_SLOTS_O * B200_CNT_STRIDE; target = cnt_mul * words_slots;
    } else {
        // q/k/v of layer l, or the LM head (l == L): the down slots of the layer before
        norm_gamma = kind == B200_ST_LM ? p.g_final : ly->g_input;
        slot_gamma = (p.gemma && l > 0) ? sm.layers[l - 1].g_post_ff : nullptr;
        slots = p.d_slots_dn; slots_flag = flag - 1u;
        in_cnt = p.d_counters + B200_CNT_SLOTS_DN * B200_CNT_STRIDE; target = (cnt_mul - 1u) * words_slots;
    }
    float *gam = sm.scratch + D;
    float ss = 0.0f;
    if (kind == B200_ST_QKV && l == 0) {
        long long tok = p.d_tokens[*p.d_pos];
        if (tok < 0 || tok >= p.emb_rows) tok = 0;   // never index outside the table
        const float *er = p.d_emb + tok * (long long)D;
#pragma unroll 1
        for (int i = tid * 4; i < D; i += TK_NC * 4) {
            float4 v = *reinterpret_cast<const float4 *>(er + i);
            const float4 g4 = *reinterpret_cast<const float4 *>(norm_gamma + i);
            v.x *= p.emb_scale; v.y *= p.emb_scale; v.z *= p.emb_scale; v.w *= p.emb_scale;
            *reinterpret_cast<float4 *>(sm.resid + swz(i)) = v;
            *reinterpret_cast<float4 *>(gam + swz(i)) = g4;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        // Up to 4 pairs per thread and round, all in flight together; the norm weights of the first round's
        // elements are requested before the wait, so that their round trip hides behind it. Every thread
        // reaches the barrier, whether or not it owns elements.
        constexpr int NB = 4;
        float sq = 0.0f;
        float2 gq[NB];
        {
            const int cnt0 = tid * 2 < D ? (D - tid * 2 + TK_NC * 2 - 1) / (TK_NC * 2) : 0;
#pragma unroll
            for (int u = 0; u < NB; ++u) gq[u] = u < cnt0 ? *reinterpret_cast<const float2 *>(norm_gamma + tid * 2 + u * TK_NC * 2) : make_float2(0, 0);
        }
        const int cspin = cspin_of(p);
        if (tid == 0) { cnt_wait<MULTI>(in_cnt, target, sm.flags, cspin); if (trace) trace[8] = global_ns(); }
        named_barrier(1, TK_NC);
        if (trace && tid == 0) trace[9] = global_ns();
#pragma unroll 1
        for (int i0 = tid * 2; i0 < D; i0 += TK_NC * 2 * NB) {
            const int cnt = (D - i0 + TK_NC * 2 - 1) / (TK_NC * 2);
            if (i0 != tid * 2) {
#pragma unroll
                for (int u = 0; u < NB; ++u) gq[u] = u < cnt ? *reinterpret_cast<const float2 *>(norm_gamma + i0 + u * TK_NC * 2) : make_float2(0, 0);
            }
            float s0[NB], s1[NB];
#pragma unroll
            for (int u = 0; u < NB; ++u) { s0[u] = 0.0f; s1[u] = 0.0f; }
#pragma unroll 1
            for (int k = 0; k < p.n_ranks; ++k) {
                float a[NB], b[NB];
                fl_poll<NB, TK_NC * 2, MULTI>(slots + (size_t)k * D + i0, cnt, slots_flag, a, b, sm.flags, p.d_err, spin);
#pragma unroll
                for (int u = 0; u < NB; ++u) { s0[u] += a[u]; s1[u] += b[u]; }
            }
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                const int i = swz(i0 + u * TK_NC * 2);
                if (u < cnt) {
                    *reinterpret_cast<float2 *>(gam + i) = gq[u];
                    if (slot_gamma) {
                        sm.scratch[i] = s0[u]; sm.scratch[i + 1] = s1[u];
                        sq = fmaf(s0[u], s0[u], sq); sq = fmaf(s1[u], s1[u], sq);
                    } else {
                        const float r0 = sm.resid[i] + s0[u], r1 = sm.resid[i + 1] + s1[u];
                        sm.resid[i] = r0; sm.resid[i + 1] = r1;
                        ss = fmaf(r0, r0, ss); ss = fmaf(r1, r1, ss);
                    }
                }
            }
        }
        if (trace && tid == 0) trace[10] = global_ns();
        if (slot_gamma) {
            // the sum of the slots is normalised before it joins the residual (Gemma3's post norms)
            const float inv_s = rsqrtf(cons_sum(sq, sm.red, 0, tid) / (float)D + p.eps);
#pragma unroll 1
            for (int n = tid * 2; n < D; n += TK_NC * 2) {
                const int i = swz(n);
                const float r0 = sm.resid[i] + slot_gamma[n] * sm.scratch[i] * inv_s;
                const float r1 = sm.resid[i + 1] + slot_gamma[n + 1] * sm.scratch[i + 1] * inv_s;
                sm.resid[i] = r0; sm.resid[i + 1] = r1;
                ss = fmaf(r0, r0, ss); ss = fmaf(r1, r1, ss);
            }
        }
    }
    const float tot = cons_sum(ss, sm.red, 1, tid);
    if (trace && tid == 0) trace[11] = global_ns();
    return rsqrtf(tot / (float)D + p.eps);       // 2 ulp, as the shader's rsqrt (q8_kernels.metal:156)
}

// Input vector of the o and down stages: the flagged vector, fetched once per block with coalesced
// loads into scratch[0 .. cols).
template <bool MULTI>
__device__ __forceinline__ void stage_vector(const b200_token_args &p, int kind, int l, unsigned ep, unsigned long long *trace)
{
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const int tid = threadIdx.x, L = p.n_layers, cols = p.g[kind].cols;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    const unsigned cnt_mul = ep * (unsigned)L + (unsigned)l + 1u;
    const b200_flagged *in_vec = kind == B200_ST_O ? p.d_attn_out : p.d_act;
    const unsigned *in_cnt = p.d_counters + (kind == B200_ST_O ? B200_CNT_ATTN : B200_CNT_ACT) * B200_CNT_STRIDE;
    if (tid == 0) { cnt_wait<false>(in_cnt, cnt_mul * (unsigned)cols, sm.flags, cspin_of(p)); if (trace) trace[8] = global_ns(); }
    named_barrier(1, TK_NC);
    if (trace && tid == 0) trace[9] = global_ns();
    constexpr int NB = 4;
#pragma unroll 1
    for (int i0 = tid * 2; i0 < cols; i0 += TK_NC * 2 * NB) {
        float a[NB], b[NB];
        fl_poll<NB, TK_NC * 2, false>(in_vec + i0, (cols - i0 + TK_NC * 2 - 1) / (TK_NC * 2), flag, a, b, sm.flags, p.d_err, spin);
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int i = i0 + u * TK_NC * 2;
            if (i < cols) *reinterpret_cast<float2 *>(sm.scratch + swz(i)) = make_float2(a[u], b[u]);
        }
    }
    if (trace && tid == 0) trace[10] = global_ns();
    named_barrier(1, TK_NC);
    if (trace && tid == 0) trace[11] = global_ns();
}

// Q8_0 stages multiply in integers: the input vector is rewritten once per stage as block fixed point.
// Each 16-column slice (what one consumer thread owns) gets a scale s = max|x| / 2^22 and its values
// X = round(x / s), |X| <= 2^22, split into three signed bytes X = a + 256 b + 65536 c (a, b in
// [-128, 127], |c| <= 64). A row's share of the slice is then three dp4a sums per four weights, exact in
// int32, recombined in fp32 -- the rounding of x is 2^-23 of the slice's largest element, below what the
// fp32 accumulation of the same products loses. One thread converts one slice; the 64-byte record
// [a0..a3][b0..b3][c0..c3][s, -, -, -] (byte k of word j = element 4j + k, the order of the weight bytes)
// replaces the slice in scratch[0 .. cols), chunks swizzled like the vector they come from. Normalised
// stages read residual * norm weight * inv from shared memory; the others convert scratch in place.
// One work item of that conversion: four consecutive elements v4 (element 4 * it .. 4 * it + 3; one word
// of each byte plane). The four items of a slice sit in adjacent lanes and agree on the slice's maximum by
// two shuffles, so every lane of the warp must call this (lanes past the end of the vector with on = false).
__device__ __forceinline__ void quantize_item(uint32_t *rec, int it, float4 v4, bool on)
{
    float amax = fmaxf(fmaxf(fabsf(v4.x), fabsf(v4.y)), fmaxf(fabsf(v4.z), fabsf(v4.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = amax * (1.0f / 4194304.0f);
    const float rinv = amax > 1e-30f ? 4194304.0f * __frcp_rn(amax) : 0.0f;     // a slice of zeros (or denormals) reads as zero
    // round to nearest through the 1.5 * 2^23 constant: exact for |X| <= 2^22
    const int X0 = __float_as_int(fmaf(v4.x, rinv, 12582912.0f)) - 0x4B400000;
    const int X1 = __float_as_int(fmaf(v4.y, rinv, 12582912.0f)) - 0x4B400000;
    const int X2 = __float_as_int(fmaf(v4.z, rinv, 12582912.0f)) - 0x4B400000;
    const int X3 = __float_as_int(fmaf(v4.w, rinv, 12582912.0f)) - 0x4B400000;
    const int Y0 = (X0 + 128) >> 8, Y1 = (X1 + 128) >> 8, Y2 = (X2 + 128) >> 8, Y3 = (X3 + 128) >> 8;
    const int Z0 = (Y0 + 128) >> 8, Z1 = (Y1 + 128) >> 8, Z2 = (Y2 + 128) >> 8, Z3 = (Y3 + 128) >> 8;
    const uint32_t wa = __byte_perm(__byte_perm(X0, X1, 0x0040), __byte_perm(X2, X3, 0x0040), 0x5410);
    const uint32_t wb = __byte_perm(__byte_perm(Y0, Y1, 0x0040), __byte_perm(Y2, Y3, 0x0040), 0x5410);
    const uint32_t wc = __byte_perm(__byte_perm(Z0, Z1, 0x0040), __byte_perm(Z2, Z3, 0x0040), 0x5410);
    if (on) {
        const int base = (it >> 2) * 16, j = it & 3;         // the slice's record, this item's word in each plane
        rec[swz(base + j)] = wa;
        rec[swz(base + 4 + j)] = wb;
        rec[swz(base + 8 + j)] = wc;
        if (j == 0) rec[swz(base + 12)] = __float_as_uint(scale);
    }
}

// The conversion as a pass of its own over a vector that is already in shared memory (stages whose
// residual update goes through a post norm first; see stage_residual). cols is a multiple of 32, so a
// warp's items are all inside the vector or all outside. In-place stages: the items of a slice read their
// chunks before any of them writes (the shuffles are in between), and no other slice shares those 64 bytes.
__device__ __forceinline__ void quantize_input(const b200_token_args &p, int kind, float inv)
{
    const Smem sm = smem_of(p);
    const int tid = threadIdx.x, cols = p.g[kind].cols;
    const bool normed = kind != B200_ST_O && kind != B200_ST_DOWN;
    const float *xv = normed ? sm.resid : sm.scratch;
    const float *gam = sm.scratch + p.d_model;
    uint32_t *rec = reinterpret_cast<uint32_t *>(sm.scratch);
#pragma unroll 1
    for (int it = tid; it * 4 < ((cols + 127) & ~127); it += TK_NC) {
        const int e0 = it * 4;
        const bool on = e0 < cols;
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (on) {
            v4 = *reinterpret_cast<const float4 *>(xv + swz(e0));
            if (normed) {
                const float4 g4 = *reinterpret_cast<const float4 *>(gam + swz(e0));
                v4.x = g4.x * v4.x * inv; v4.y = g4.y * v4.y * inv; v4.z = g4.z * v4.z * inv; v4.w = g4.w * v4.w * inv;
            }
        }
        quantize_item(rec, it, v4, on);
    }
    named_barrier(1, TK_NC);
}

// Q8_0 stages without a post norm: the input is converted while it is assembled, four consecutive
// elements per thread, straight from the polled words -- no fp32 copy in shared memory, no second pass.
//
// Residual stages (q/k/v, gate/up, LM head): residual <- embedding row | residual + sum of the slots; the
// records hold residual * norm weight WITHOUT the 1/rms factor, which is a scalar known only after the
// block-wide sum: it is returned and multiplies the stage's outputs instead.
template <bool MULTI>
__device__ __forceinline__ float fused_residual_q8(const b200_token_args &p, int kind, int l, unsigned ep, unsigned long long *trace)
{
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const int tid = threadIdx.x, D = p.d_model, L = p.n_layers;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    const unsigned cnt_mul = ep * (unsigned)L + (unsigned)l + 1u;
    const b200_token_layer *ly = sm.layers + (l < L ? l : L - 1);
    const float *norm_gamma;
    const b200_flagged *slots;
    const unsigned *in_cnt;
    unsigned slots_flag, target;
    if (kind == B200_ST_GATEUP) {
        norm_gamma = p.gemma ? ly->g_pre_ff : ly->g_post_attn;
        slots = p.d_slots_o; slots_flag = flag;
        in_cnt = p.d_counters + B200_CNT_SLOTS_O * B200_CNT_STRIDE; target = cnt_mul * (unsigned)(D * p.n_ranks);
    } else {
        norm_gamma = kind == B200_ST_LM ? p.g_final : ly->g_input;
        slots = p.d_slots_dn; slots_flag = flag - 1u;
        in_cnt = p.d_counters + B200_CNT_SLOTS_DN * B200_CNT_STRIDE; target = (cnt_mul - 1u) * (unsigned)(D * p.n_ranks);
    }
    const bool from_emb = kind == B200_ST_QKV && l == 0;
    uint32_t *rec = reinterpret_cast<uint32_t *>(sm.scratch);
    const float *er = nullptr;
    if (from_emb) {
        long long tok = p.d_tokens[*p.d_pos];
        if (tok < 0 || tok >= p.emb_rows) tok = 0;   // never index outside the table
        er = p.d_emb + tok * (long long)D;
    } else {
        const int cspin = cspin_of(p);
        if (tid == 0) { cnt_wait<MULTI>(in_cnt, target, sm.flags, cspin); if (trace) trace[8] = global_ns(); }
        named_barrier(1, TK_NC);
    }
    if (trace && tid == 0) trace[9] = global_ns();
    float ss = 0.0f;
#pragma unroll 1
    for (int it = tid; it * 4 < ((D + 127) & ~127); it += TK_NC) {
        const int e0 = it * 4;
        const bool on = e0 < D;
        float4 g4 = make_float4(0.f, 0.f, 0.f, 0.f), r4 = g4;
        if (on) g4 = *reinterpret_cast<const float4 *>(norm_gamma + e0);     // in flight while the slots are polled
        if (from_emb) {
            if (on) {
                r4 = *reinterpret_cast<const float4 *>(er + e0);
                r4.x *= p.emb_scale; r4.y *= p.emb_scale; r4.z *= p.emb_scale; r4.w *= p.emb_scale;
            }
        } else {
            if (on) r4 = *reinterpret_cast<const float4 *>(sm.resid + swz(e0));
            if (MULTI) {
                // the slots of up to four ranks per round, all loads in flight together; added in rank order
#pragma unroll 1
                for (int k0 = 0; k0 < p.n_ranks; k0 += 4) {
                    const int nk = p.n_ranks - k0 < 4 ? p.n_ranks - k0 : 4;
                    float a[8], b[8];
                    fl_poll_step<8, true, 2>(slots + (size_t)k0 * D + e0, (size_t)D, on ? 2 * nk : 0, slots_flag, a, b, sm.flags, p.d_err, spin);
#pragma unroll
                    for (int k = 0; k < 4; ++k) { r4.x += a[2 * k]; r4.y += b[2 * k]; r4.z += a[2 * k + 1]; r4.w += b[2 * k + 1]; }
                }
            } else {
                float a[2], b[2];
                fl_poll<2, 2, false>(slots + e0, on ? 2 : 0, slots_flag, a, b, sm.flags, p.d_err, spin);
                r4.x += a[0]; r4.y += b[0]; r4.z += a[1]; r4.w += b[1];
            }
        }
        if (on) *reinterpret_cast<float4 *>(sm.resid + swz(e0)) = r4;
        ss = fmaf(r4.x, r4.x, ss); ss = fmaf(r4.y, r4.y, ss); ss = fmaf(r4.z, r4.z, ss); ss = fmaf(r4.w, r4.w, ss);
        quantize_item(rec, it, make_float4(r4.x * g4.x, r4.y * g4.y, r4.z * g4.z, r4.w * g4.w), on);
    }
    if (trace && tid == 0) trace[10] = global_ns();
    const float tot = cons_sum(ss, sm.red, 1, tid);       // its barrier also publishes the records
    if (trace && tid == 0) trace[11] = global_ns();
    return rsqrtf(tot / (float)D + p.eps);
}

// Vector stages (o, down): the flagged input vector, polled and converted in one go.
template <bool MULTI>
__device__ __forceinline__ void fused_vector_q8(const b200_token_args &p, int kind, int l, unsigned ep, unsigned long long *trace)
{
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const int tid = threadIdx.x, L = p.n_layers, cols = p.g[kind].cols;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    const unsigned cnt_mul = ep * (unsigned)L + (unsigned)l + 1u;
    const b200_flagged *in_vec = kind == B200_ST_O ? p.d_attn_out : p.d_act;
    const unsigned *in_cnt = p.d_counters + (kind == B200_ST_O ? B200_CNT_ATTN : B200_CNT_ACT) * B200_CNT_STRIDE;
    uint32_t *rec = reinterpret_cast<uint32_t *>(sm.scratch);
    if (tid == 0) { cnt_wait<false>(in_cnt, cnt_mul * (unsigned)cols, sm.flags, cspin_of(p)); if (trace) trace[8] = global_ns(); }
    named_barrier(1, TK_NC);
    if (trace && tid == 0) trace[9] = global_ns();
    // Up to four items per thread and round, all eight loads in flight together (one round trip, not four).
    constexpr int NI = 4;
    const int lim = (cols + 127) & ~127;
#pragma unroll 1
    for (int it0 = tid; it0 * 4 < lim; it0 += TK_NC * NI) {
        const int left = cols - it0 * 4;                                 // elements from this thread's first item on
        const int n_on = left <= 0 ? 0 : (left + TK_NC * 4 - 1) / (TK_NC * 4);       // its items inside the vector
        float a[2 * NI], b[2 * NI];
        fl_poll<2 * NI, TK_NC * 4, false, 2>(in_vec + it0 * 4, 2 * (n_on < NI ? n_on : NI), flag, a, b, sm.flags, p.d_err, spin);
#pragma unroll
        for (int k = 0; k < NI; ++k) {
            const int it = it0 + k * TK_NC;
            if (it * 4 < lim)                                            // the same for every lane of a warp
                quantize_item(rec, it, make_float4(a[2 * k], b[2 * k], a[2 * k + 1], b[2 * k + 1]), k < n_on);
        }
    }
    if (trace && tid == 0) trace[10] = global_ns();
    named_barrier(1, TK_NC);
    if (trace && tid == 0) trace[11] = global_ns();
}

// Rows [w0, w1) of the block: every warp works on every chunk. A thread owns SPT 16-byte column
// slices (its slices of x stay in registers) and, in each chunk, the RG rows of its group; eight row
// partials are collected in registers (8 / RG chunks) and then folded across the warp's lanes by one
// transposing shuffle reduction; the warp partial of each row goes to part[]. `state` is the running
// chunk number; returned advanced.
template <int WT, int SPT, int RG, int NACC, bool TRACE>
__device__ __forceinline__ unsigned stage_rows(const b200_token_args &p, int kind, float inv, int w0, int w1, unsigned state, unsigned win,
                                            unsigned long long *trace)
{
    constexpr int E = (WT == B200_WT_Q8) ? 16 : 8;
    const b200_stage_geom &G = p.g[kind];
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    if (TRACE && trace && threadIdx.x == 0) trace[13] = global_ns();
    const int tid = threadIdx.x, T = G.T, NG = G.NG, RB = G.rb;
    const int g = tid / T, t = tid - g * T, lane = tid & 31, wg = t >> 5, nwgp = (T >> 5) | 1;
    const bool active = g < NG;

    // ---------------- this thread's slices of the input vector -> registers ----------------
    if (TRACE && trace && tid == 0) trace[14] = (unsigned long long)g + global_ns();
    float x[WT == B200_WT_Q8 ? 1 : SPT][WT == B200_WT_Q8 ? 1 : E];   // F16 weights: the slices as fp32
    uint4 xa[SPT], xb[SPT], xc[SPT];                                  // Q8_0 weights: the slices' three byte planes
    float xs[SPT];                                                    //   and scales (see quantize_input)
    uint32_t qoff[SPT], soff[SPT];
    {
        const bool normed = kind != B200_ST_O && kind != B200_ST_DOWN;
        const float *xv = normed ? sm.resid : sm.scratch;
        const float *gam = sm.scratch + p.d_model;
#pragma unroll
        for (int s = 0; s < SPT; ++s) {
            const int col = (s * T + t) * E;
            const bool on = active && col < G.cols;
            if (WT == B200_WT_Q8) {
                const uint32_t *rec = reinterpret_cast<const uint32_t *>(sm.scratch);
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                xa[s] = on ? *reinterpret_cast<const uint4 *>(rec + swz(col)) : z;
                xb[s] = on ? *reinterpret_cast<const uint4 *>(rec + swz(col + 4)) : z;
                xc[s] = on ? *reinterpret_cast<const uint4 *>(rec + swz(col + 8)) : z;
                xs[s] = on ? __uint_as_float(rec[swz(col + 12)]) : 0.0f;
            } else {
#pragma unroll
                for (int e = 0; e < E; e += 4) {
                    float4 v4 = make_float4(0, 0, 0, 0);
                    if (on) {
                        v4 = *reinterpret_cast<const float4 *>(xv + swz(col + e));
                        if (normed) {
                            const float4 g4 = *reinterpret_cast<const float4 *>(gam + swz(col + e));
                            v4.x = g4.x * v4.x * inv; v4.y = g4.y * v4.y * inv; v4.z = g4.z * v4.z * inv; v4.w = g4.w * v4.w * inv;
                        }
                    }
                    x[WT == B200_WT_Q8 ? 0 : s][WT == B200_WT_Q8 ? 0 : e] = v4.x;
                    x[WT == B200_WT_Q8 ? 0 : s][WT == B200_WT_Q8 ? 0 : e + 1] = v4.y;
                    x[WT == B200_WT_Q8 ? 0 : s][WT == B200_WT_Q8 ? 0 : e + 2] = v4.z;
                    x[WT == B200_WT_Q8 ? 0 : s][WT == B200_WT_Q8 ? 0 : e + 3] = v4.w;
                }
            }
            // Byte offsets of the slice inside a row. Threads past the end of the row read slice 0 (valid
            // memory) against a zero input slice.
            const int cc = on ? col : 0;
            qoff[s] = (uint32_t)(WT == B200_WT_Q8 ? cc : 2 * cc);
            soff[s] = (uint32_t)G.cols + (uint32_t)(cc >> 5) * 2u;   // Q8: scales follow the quants of a row
        }
    }
    if (TRACE && trace && tid == 0) trace[1] = global_ns();

    const uint32_t ring_s = smem_u32(sm.ring), stride = (uint32_t)G.row_stride;
    const uint32_t grow = (uint32_t)(g * RG) * stride;           // this group's first row inside a chunk
    float *part = sm.part + (win & 1u) * TK_PART;
    const int nrows = w1 - w0;
    unsigned seq = state;
    bool first = true;
    // NV = RG * NACC row partials (NACC chunks) are folded across the lanes per pass: measured on Qwen3-4B,
    // eight per pass (fewer shuffles per weight) beat one chunk per pass (smaller loop body) by 3 %.
    constexpr int NV = RG * NACC;
#pragma unroll 1
    for (int r0 = 0; r0 < nrows; r0 += RB * NACC) {
        float v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = 0.0f;
#pragma unroll
        for (int u = 0; u < NACC; ++u) {
            if (r0 + u * RB < nrows) {
                const unsigned slot = seq % TK_SLOTS, par = (seq / TK_SLOTS) & 1u;
                ++seq;
                if (!mbar_wait_abort(&sm.full[slot], par, sm.flags, spin) && !sm.flags[0]) raise(sm.flags, p.d_err, 3);
                if (TRACE && trace && tid == 0 && first) { trace[2] = global_ns(); first = false; }
                if (active) {
                    // rows past the end of a short chunk hold bytes of an earlier chunk: computed, never stored
                    const uint32_t sb = ring_s + slot * TK_SLOT_BYTES + grow;
                    // at most four rows' slices in flight per thread (eight cost registers ptxas found on the stack)
                    constexpr int JB = RG < 4 ? RG : 4;
#pragma unroll
                    for (int j0 = 0; j0 < RG; j0 += JB) {
                        uint4 wq[JB][SPT];
                        uint32_t ws[JB][SPT];
#pragma unroll
                        for (int j = 0; j < JB; ++j)
#pragma unroll
                            for (int s = 0; s < SPT; ++s) {
                                wq[j][s] = lds_128(sb + (uint32_t)(j0 + j) * stride + qoff[s]);
                                if (WT == B200_WT_Q8) ws[j][s] = lds_u16(sb + (uint32_t)(j0 + j) * stride + soff[s]);
                            }
#pragma unroll
                        for (int j = 0; j < JB; ++j) {
                            float acc = 0.0f;
#pragma unroll
                            for (int s = 0; s < SPT; ++s) {
                                float d;
                                if (WT == B200_WT_Q8) d = (__half2float(__ushort_as_half((unsigned short)ws[j][s])) * xs[s]) * dot16_q8_planes(wq[j][s], xa[s], xb[s], xc[s]);
                                else d = dot8_f16(wq[j][s], x[WT == B200_WT_Q8 ? 0 : s]);
                                acc += d;
                            }
                            v[u * RG + j0 + j] = acc;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.empty[slot]);      // this warp no longer reads the slot
            }
        }
        if (active) {
            // lane i < NV ends up with the warp's total of partial i: chunk i / RG of this pass, row g*RG + i % RG of it
            const float tot = reduce_rows<NV>(v, lane);
            const int rin = g * RG + lane % RG;
            const int lrow = r0 + (lane / RG) * RB + rin;
            if (lane < NV && lrow < nrows && rin < RB) part[lrow * nwgp + wg] = tot;
        }
    }
    if (TRACE && trace && tid == 0) trace[3] = global_ns();
    return seq;
}

// Final sums and epilogue of rows [w0, w1): thread i adds the warp partials of row i in warp order.
// best (value bits | row << 32) carries the LM head's running arg-max of this thread.
template <bool TRACE, bool MULTI>
__device__ __forceinline__ unsigned long long stage_emit(const b200_token_args &p, int kind, int l, unsigned ep, int w0, int w1, unsigned win,
                                                      unsigned long long best, float oscale, unsigned long long *trace)
{
    const b200_stage_geom &G = p.g[kind];
    const Smem sm = smem_of(p);
    const int tid = threadIdx.x, lane = tid & 31, L = p.n_layers;
    const int nwg = G.T >> 5, nwgp = nwg | 1;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    unsigned *const cn = p.d_counters;
    const float *part = sm.part + (win & 1u) * TK_PART;
    named_barrier(1, TK_NC);
    if (TRACE && trace && tid == 0) trace[7] = global_ns();
    const int n = w1 - w0;
    unsigned stored = 0;
    if (kind == B200_ST_GATEUP) {
#pragma unroll 1
        for (int i = tid; i < n / 2; i += TK_NC) {
            const float gte = oscale * row_sum(part + (2 * i) * nwgp, nwg), up = oscale * row_sum(part + (2 * i + 1) * nwgp, nwg);
            const float a = p.gemma ? act_gelu_tanh(gte) : act_silu(gte);
            fl_store<false>(p.d_act + (w0 >> 1) + i, a * up, flag);
            ++stored;
        }
        stored = (unsigned)__reduce_add_sync(0xffffffffu, stored);
        if (lane == 0 && stored && cspin_of(p) > 0) cnt_add<false>(cn + B200_CNT_ACT * B200_CNT_STRIDE, stored);
        return best;
    }
    float best_v = __uint_as_float((unsigned)best);
    int best_i = (int)(best >> 32);
#pragma unroll 1
    for (int i = tid; i < n; i += TK_NC) {
        const float y = oscale * row_sum(part + i * nwgp, nwg);     // oscale: the 1/rms of a converted input, else 1
        const int row = w0 + i;
        if (kind == B200_ST_QKV) fl_store<false>(p.d_qkv + row, y, flag);
        else if (kind == B200_ST_LM) {
            p.d_logits[p.logits_offset + row] = y;
            if (better(y, row, best_v, best_i)) { best_v = y; best_i = row; }
        } else {
            // partial sums into slot `rank` of every rank
#pragma unroll 1
            for (int q = 0; q < p.n_ranks; ++q) fl_store<MULTI>((kind == B200_ST_O ? p.d_peer_slots_o[q] : p.d_peer_slots_dn[q]) + row, y, flag);
        }
        ++stored;
    }
    if (kind != B200_ST_LM && cspin_of(p) > 0) {       // nobody watches the counters when the readers poll the words themselves
        // one add per warp and receiver: the words this warp has stored
        stored = (unsigned)__reduce_add_sync(0xffffffffu, stored);
        if (lane == 0 && stored) {
            if (kind == B200_ST_QKV) cnt_add<false>(cn + B200_CNT_QKV * B200_CNT_STRIDE, stored);
            else {
#pragma unroll 1
                for (int q = 0; q < p.n_ranks; ++q)
                    cnt_add<MULTI>(p.d_peer_counters[q] + (kind == B200_ST_O ? B200_CNT_SLOTS_O : B200_CNT_SLOTS_DN) * B200_CNT_STRIDE, stored);
            }
        }
    }
    return ((unsigned long long)(unsigned)best_i << 32) | (unsigned long long)__float_as_uint(best_v);
}

// One matvec stage. `state`: running chunk number (low word) and window number (high word).
template <int WT, bool TRACE, bool MULTI>
__device__ __forceinline__ unsigned run_matvec(const b200_token_args &p, int kind, int l, unsigned ep, unsigned state,
                                                      unsigned long long *trace)
{
    const b200_stage_geom &G = p.g[kind];
    const int tid = threadIdx.x;
    if (TRACE && trace && tid == 0) trace[0] = global_ns();
    float inv = 0.0f, oscale = 1.0f;
    const bool vec = kind == B200_ST_O || kind == B200_ST_DOWN;
    // a residual update that goes through a post norm (Gemma3, except the embedding of layer 0) takes two passes
    const bool post_norm = p.gemma && !(kind == B200_ST_QKV && l == 0);
    if (WT == B200_WT_Q8 && (vec || !post_norm)) {
        if (vec) fused_vector_q8<MULTI>(p, kind, l, ep, TRACE ? trace : nullptr);
        else oscale = fused_residual_q8<MULTI>(p, kind, l, ep, TRACE ? trace : nullptr);
        if (TRACE && trace && tid == 0) trace[12] = global_ns();
        if (kind == B200_ST_LM && !p.with_lm) return state;      // only the residual update that ends a prompt position
    } else {
        if (vec) stage_vector<MULTI>(p, kind, l, ep, TRACE ? trace : nullptr);
        else inv = stage_residual<MULTI>(p, kind, l, ep, TRACE ? trace : nullptr);
        if (TRACE && trace && tid == 0) trace[12] = global_ns();
        if (kind == B200_ST_LM && !p.with_lm) return state;      // only the residual update that ends a prompt position
        if (WT == B200_WT_Q8) quantize_input(p, kind, inv);
    }
    unsigned seq = state & 0x7fffffffu, win = state >> 31;        // only the parity of the window number is ever used
    unsigned long long best = ((unsigned long long)0x7fffffffu << 32) | (unsigned long long)__float_as_uint(-INFINITY);
    const RowRange br = block_rows(G, blockIdx.x);
#pragma unroll 1
    for (int w0 = br.r0; w0 < br.r1; w0 += G.pw) {
        const int w1 = w0 + G.pw < br.r1 ? w0 + G.pw : br.r1;
        if (G.spt == 1) {
            if (G.rg == 2) seq = stage_rows<WT, 1, 2, 4, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
            else if (G.rg == 4) seq = stage_rows<WT, 1, 4, 1, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
            else if (G.rg == 8) seq = stage_rows<WT, 1, 8, 1, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
            else seq = stage_rows<WT, 1, 1, 8, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
        } else if (WT == B200_WT_F16) {
            // two slices per thread exist for binary16 rows only (more than 5120 columns); a Q8_0 thread with two
            // slices would carry 26 registers of input planes and push ptxas over the 80-register cap
            if (G.rg == 2) seq = stage_rows<B200_WT_F16, 2, 2, 4, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
            else seq = stage_rows<B200_WT_F16, 2, 1, 8, TRACE>(p, kind, inv, w0, w1, seq, win, trace);
        }
        best = stage_emit<TRACE, MULTI>(p, kind, l, ep, w0, w1, win, best, oscale, trace);
        ++win;
    }
    if (TRACE && trace && tid == 0) trace[4] = global_ns();
    if (kind == B200_ST_LM) {
        // best row of the block -> flagged pair (folded over the blocks by block 0)
        const Smem sm = smem_of(p);
        const int lane = tid & 31, warp = tid >> 5, L = p.n_layers;
        const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
        float best_v = __uint_as_float((unsigned)best);
        int best_i = (int)(best >> 32);
#pragma unroll 1
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
        }
        float *am_v = sm.red + 64;
        int *am_i = reinterpret_cast<int *>(sm.red + 96);
        if (lane == 0) { am_v[warp] = best_v; am_i[warp] = best_i; }
        named_barrier(1, TK_NC);
        if (tid == 0) {
#pragma unroll 1
            for (int ww = 1; ww < TK_NWARP; ++ww) if (better(am_v[ww], am_i[ww], best_v, best_i)) { best_v = am_v[ww]; best_i = am_i[ww]; }
            if (p.n_ranks > 1) __threadfence_system();   // this block's logits are visible before its pair is
            fl_store<false>(p.d_am + 2 * blockIdx.x, best_v, flag);
            fl_store<false>(p.d_am + 2 * blockIdx.x + 1, __int_as_float(best_i), flag);
        }
    }
    return ((win & 1u) << 31) | seq;
}

// ---------------------------------------------------------------------------
// Attention stage: item (kv head, sequence split) = block index. The block rebuilds the normalised,
// rotated query heads of its KV head and the new key/value row, stores the row to the cache (split 0),
// attends over its slice with one online softmax per key lane and leaves (max, sum, output) as a
// flagged record; block (kv head, split g) then merges all splits of query head g of that KV head.
// ---------------------------------------------------------------------------
// OWNROW: the row of the new position joins the staged rows (written by the block itself) instead of being
// selected element by element in the key loop. Shorter and faster; the instantiations with binary16 weights keep
// the select, where the other form pushed ptxas over its register cap.
template <int HD, bool TRACE, bool MULTI, bool OWNROW>
__device__ __forceinline__ void attention_stage(const b200_token_args &p, int l, unsigned ep, unsigned long long *trace)
{
    constexpr int DPT = 8;                           // head-dim values per thread
    constexpr int DLN = HD / DPT;                    // threads that share one key (a key lane): 8, 16 or 32
    constexpr int HALF = HD / 2;
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const b200_token_layer &ly = sm.layers[l];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.n_q / p.n_kv, L = p.n_layers;
    const unsigned flag = ep * (unsigned)(L + 1) + (unsigned)l + 1u;
    const unsigned cnt_mul = ep * (unsigned)L + (unsigned)l + 1u;
    const int item = blockIdx.x;
    if (TRACE && trace && tid == 0) trace[0] = global_ns();
    if (item < p.n_kv * p.n_split && tid < ATT_T) {
        const int kvh = item / p.n_split, split = item - kvh * p.n_split;
        const int TPH = ATT_T / G, WPH = TPH / 32, KL = TPH / DLN;
        const int g = tid / TPH, r = tid - g * TPH, kl = r / DLN, dl = r - kl * DLN;
        const int pos = sm.flags[3], n = pos + 1;
        const int chunk = (n + p.n_split - 1) / p.n_split;
        const int j0 = min(split * chunk, n), j1 = min(j0 + chunk, n);
        const int KCH = p.att_keys;                  // cache rows staged in shared memory at a time
        const int nsub = (chunk + KCH - 1) / KCH;    // the same for every block and layer of this token

        float *q_s = sm.scratch;                     // [G][HD]
        float *k_new = q_s + G * HD;                 // [HD] the new key row (OWNROW: as binary16, see k_new_h)
        float *v_new = k_new + HD;                   // [HD] the new value row
        __half *k_new_h = reinterpret_cast<__half *>(k_new), *v_new_h = reinterpret_cast<__half *>(v_new);
        float *mrg = v_new + HD;                     // [G][WPH][HD + 2]
        float *raw = mrg + G * WPH * (HD + 2);       // [(G + 2) * HD] new q heads, k row, v row as produced
        __half *ks = reinterpret_cast<__half *>(raw + (G + 2) * HD);   // [KCH][HD] staged keys
        __half *vs = ks + (size_t)KCH * HD;                            // [KCH][HD] staged values
        float *stg = reinterpret_cast<float *>(ks);  // [n_split][HD + 2]: the staging area again, once the keys are done

        const __half *kc = static_cast<const __half *>(ly.k_cache) + (size_t)kvh * p.max_seq * HD;
        const __half *vc = static_cast<const __half *>(ly.v_cache) + (size_t)kvh * p.max_seq * HD;

        // The block's slice of the cache is two contiguous byte ranges: one bulk copy each into shared
        // memory, started before the wait for q/k/v so that its latency hides behind that wait. The row
        // of the new position (not in the cache yet) is copied like the others and never read, or (OWNROW)
        // left out and written by the block itself.
        auto stage_rows = [&](int c0, int c1) {
            if (OWNROW && c1 > pos) c1 = pos;        // the block writes that row itself (below)
            const unsigned bytes = c1 > c0 ? (unsigned)(c1 - c0) * HD * 2u : 0u;
            mbar_expect_tx(sm.att_bar, 2u * bytes);
            if (bytes) {
                bulk_load(ks, kc + (size_t)c0 * HD, bytes, sm.att_bar);
                bulk_load(vs, vc + (size_t)c0 * HD, bytes, sm.att_bar);
            }
        };
        if (tid == 0) stage_rows(j0, min(j0 + KCH, j1));

        // ---- what the rotation needs and does not depend on q/k/v: cos/sin of this position (from the layer's
        // table) and the two
        // norm weight vectors, fetched by the threads that have no row to poll, while the rows are awaited.
        // The table lives in the merge buffer, which is not used before the keys are done. ----
        float *rot_c = mrg, *rot_s = mrg + HALF, *gam_q = mrg + 2 * HALF, *gam_k = gam_q + HD;
        {
            const int first = ((G + 2) * HD / 2 + 31) & ~31;            // threads below poll the rows
            const int nt = ATT_T - first > 0 ? ATT_T - first : ATT_T;     // helpers (all threads if every one polls)
            const int r0 = ATT_T - first > 0 ? tid - first : tid;
            if (r0 >= 0) {
#pragma unroll 1
                for (int d = r0; d < HALF; d += nt) {
                    const float2 cs = *reinterpret_cast<const float2 *>(ly.rope + ((size_t)pos * HALF + d) * 2);
                    rot_c[d] = cs.x; rot_s[d] = cs.y;
                }
#pragma unroll 1
                for (int d = r0; d < HD; d += nt) {
                    gam_q[d] = ly.g_qn ? ly.g_qn[d] : 1.0f;
                    gam_k[d] = ly.g_kn ? ly.g_kn[d] : 1.0f;
                }
            }
        }

        // ---- the new rows of this KV head (with arrival counters: one thread watches, the others wait for it;
        // without, everybody polls at once and the table work above overlaps the wait) ----
        if (cspin_of(p) > 0) {
            if (tid == 0) cnt_wait<false>(p.d_counters + B200_CNT_QKV * B200_CNT_STRIDE, cnt_mul * (unsigned)((p.n_q + 2 * p.n_kv) * HD), sm.flags, cspin_of(p));
            named_barrier(2, ATT_T);
        }
        {
            // q heads of this KV head are contiguous; its k row and v row follow at their own offsets
            const int nq = G * HD;
#pragma unroll 1
            for (int i = tid * 2; i < (G + 2) * HD; i += ATT_T * 2) {
                const int src = i < nq ? kvh * nq + i
                              : i < nq + HD ? p.n_q * HD + kvh * HD + (i - nq)
                                            : (p.n_q + p.n_kv) * HD + kvh * HD + (i - nq - HD);
                float a[1], b[1];
                fl_poll<1, 2, false>(p.d_qkv + src, 1, flag, a, b, sm.flags, p.d_err, spin);
                *reinterpret_cast<float2 *>(raw + i) = make_float2(a[0], b[0]);
            }
        }
        named_barrier(2, ATT_T);
        if (TRACE && trace && tid == 0) trace[1] = global_ns();

        // ---- normalise + rotate: warp vi < G takes query head vi, warp G the new key, warp G + 1 the new value ----
        if (warp <= G) {
            const bool is_k = (warp == G);
            const float *src = raw + warp * HD;
            const bool has_norm = is_k ? ly.g_kn != nullptr : ly.g_qn != nullptr;
            const float *gamma = is_k ? gam_k : gam_q;
            float ss = 0.0f;
#pragma unroll 1
            for (int d = lane; d < HD; d += 32) ss = fmaf(src[d], src[d], ss);
            ss = warp_sum(ss);
            const float inv = has_norm ? rsqrtf(ss / (float)HD + p.eps) : 1.0f;
            __half *kdst = const_cast<__half *>(kc) + (size_t)pos * HD;
#pragma unroll 1
            for (int d = lane; d < HALF; d += 32) {
                float ra = src[d], rb = src[d + HALF];
                if (has_norm) { ra = gamma[d] * ra * inv; rb = gamma[d + HALF] * rb * inv; }
                const float sn = rot_s[d], cs = rot_c[d];
                const float r0 = ra * cs - rb * sn;
                const float r1 = ra * sn + rb * cs;
                if (is_k) {
                    const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
                    if (OWNROW) { k_new_h[d] = h0; k_new_h[d + HALF] = h1; }
                    else { k_new[d] = __half2float(h0); k_new[d + HALF] = __half2float(h1); }
                    if (split == 0) { kdst[d] = h0; kdst[d + HALF] = h1; }
                } else {
                    q_s[warp * HD + d] = r0; q_s[warp * HD + d + HALF] = r1;
                }
            }
        } else if (warp == G + 1) {
            // the new value row: rounded to the cache's binary16 by a warp of its own
            const float *vsrc = raw + (G + 1) * HD;
            __half *vdst = const_cast<__half *>(vc) + (size_t)pos * HD;
#pragma unroll 1
            for (int d = lane; d < HD; d += 32) {
                const __half h = __float2half_rn(vsrc[d]);
                if (OWNROW) v_new_h[d] = h; else v_new[d] = __half2float(h);
                if (split == 0) vdst[d] = h;
            }
        }
        named_barrier(2, ATT_T);
        if (TRACE && trace && tid == 0) trace[5] = global_ns();

        // ---- the keys of this lane, from shared memory: online softmax in registers ----
        float q[DPT], acc[DPT];
#pragma unroll
        for (int e = 0; e < DPT; ++e) { q[e] = q_s[g * HD + dl * DPT + e]; acc[e] = 0.0f; }
        const float scale = 1.0f / sqrtf((float)HD);
        float m = -INFINITY, lsum = 0.0f;
#pragma unroll 1
        for (int sub = 0; sub < nsub; ++sub) {
            const int c0 = min(j0 + sub * KCH, j1), c1 = min(c0 + KCH, j1);
            if (sub > 0) {
                named_barrier(2, ATT_T);             // everybody is done with the rows staged before
                if (tid == 0) stage_rows(c0, c1);
            }
            if (OWNROW && pos >= c0 && pos < c1) {   // the same for the whole block: the last split only
                // the row of this position joins the staged rows (the bulk copies leave its place alone)
                if (tid < HD / 8) {
                    reinterpret_cast<uint4 *>(ks + (size_t)(pos - c0) * HD)[tid] = reinterpret_cast<const uint4 *>(k_new_h)[tid];
                    reinterpret_cast<uint4 *>(vs + (size_t)(pos - c0) * HD)[tid] = reinterpret_cast<const uint4 *>(v_new_h)[tid];
                }
                named_barrier(2, ATT_T);
            }
            if (!mbar_wait_abort(sm.att_bar, (unsigned)(l * nsub + sub) & 1u, sm.flags, spin) && !sm.flags[0]) raise(sm.flags, p.d_err, 6);
            if (TRACE && trace && tid == 0 && sub == 0) trace[8] = global_ns();
            // same trip count for every key lane of the block, so that the warp-wide shuffles stay convergent
            const int rounds = (c1 - c0 + KL - 1) / KL;
#pragma unroll 1
            for (int it = 0, j = c0 + kl; it < rounds; ++it, j += KL) {
                const bool valid = j < c1;           // every lane of the warp runs the shuffles; only valid keys count
                // One unconditional 16-byte load of the staged key and value (row 0 for an idle lane); both stay
                // packed until they are used, and the row of the new position, which is not in the cache yet,
                // is selected element by element: unpacked copies of both rows, or separate branches filling
                // them, cost registers that ptxas could only find on the stack.
                const int jj = valid ? j - c0 : 0;
                const uint4 ku = *reinterpret_cast<const uint4 *>(ks + (size_t)jj * HD + dl * DPT);
                const uint4 vu = *reinterpret_cast<const uint4 *>(vs + (size_t)jj * HD + dl * DPT);
                const uint32_t kw[4] = {ku.x, ku.y, ku.z, ku.w}, vw[4] = {vu.x, vu.y, vu.z, vu.w};
                const bool fresh = !OWNROW && j == pos;
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float k0 = __half2float(__ushort_as_half((unsigned short)(kw[i] & 0xffffu)));
                    float k1 = __half2float(__ushort_as_half((unsigned short)(kw[i] >> 16)));
                    if (fresh) { k0 = k_new[dl * DPT + 2 * i]; k1 = k_new[dl * DPT + 2 * i + 1]; }
                    s = fmaf(q[2 * i], k0, s);
                    s = fmaf(q[2 * i + 1], k1, s);
                }
#pragma unroll
                for (int o = 1; o < DLN; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                s *= scale;
                if (valid) {
                    const float mn = fmaxf(m, s);
                    const float corr = __expf(m - mn), pj = __expf(s - mn);
                    lsum = fmaf(lsum, corr, pj);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float v0 = __half2float(__ushort_as_half((unsigned short)(vw[i] & 0xffffu)));
                        float v1 = __half2float(__ushort_as_half((unsigned short)(vw[i] >> 16)));
                        if (fresh) { v0 = v_new[dl * DPT + 2 * i]; v1 = v_new[dl * DPT + 2 * i + 1]; }
                        acc[2 * i] = fmaf(acc[2 * i], corr, pj * v0);
                        acc[2 * i + 1] = fmaf(acc[2 * i + 1], corr, pj * v1);
                    }
                    m = mn;
                }
            }
        }

        if (TRACE && trace && tid == 0) trace[6] = global_ns();
        // ---- merge the key lanes of a head: inside the warp, then across the head's warps ----
#pragma unroll 1
        for (int o = DLN; o < 32; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, lsum, o);
            const float mn = fmaxf(m, mo);
            const float ca = (m == -INFINITY) ? 0.0f : __expf(m - mn), cb = (mo == -INFINITY) ? 0.0f : __expf(mo - mn);
            lsum = lsum * ca + lo * cb;
#pragma unroll
            for (int e = 0; e < DPT; ++e) acc[e] = acc[e] * ca + __shfl_xor_sync(0xffffffffu, acc[e], o) * cb;
            m = mn;
        }
        const int wh = r >> 5;                       // warp index inside the head group
        if ((r & 31) < DLN) {                        // key lane 0 of each warp holds the warp's state
            float *dst = mrg + ((size_t)g * WPH + wh) * (HD + 2);
#pragma unroll
            for (int e = 0; e < DPT; ++e) dst[dl * DPT + e] = acc[e];
            if (dl == 0) { dst[HD] = m; dst[HD + 1] = lsum; }
        }
        named_barrier(2, ATT_T);
        if (TRACE && trace && tid == 0) trace[7] = global_ns();
        // record of (head, split): unnormalised output [HD], running max, sum. One pass: thread (head, d)
        // folds the head's warps for output element d; the thread of d = 0 also leaves the max and the sum.
        unsigned nst = 0;
#pragma unroll 1
        for (int o = tid; o < G * HD; o += ATT_T) {
            const int gg = o / HD, d = o - gg * HD;
            const float *src = mrg + (size_t)gg * WPH * (HD + 2);
            float M = -INFINITY;
#pragma unroll 1
            for (int w = 0; w < WPH; ++w) M = fmaxf(M, src[w * (HD + 2) + HD]);
            float v = 0.0f, lt = 0.0f;
#pragma unroll 1
            for (int w = 0; w < WPH; ++w) {
                const float mw = src[w * (HD + 2) + HD];
                const float cf = (mw == -INFINITY) ? 0.0f : __expf(mw - M);
                v = fmaf(src[w * (HD + 2) + d], cf, v);
                lt = fmaf(src[w * (HD + 2) + HD + 1], cf, lt);
            }
            b200_flagged *rec = p.d_attn_part + ((size_t)(kvh * G + gg) * p.n_split + split) * (HD + 2);
            fl_store<false>(rec + d, v, flag);
            ++nst;
            if (d == 0) { fl_store<false>(rec + HD, M, flag); fl_store<false>(rec + HD + 1, lt, flag); nst += 2; }
        }
        nst = (unsigned)__reduce_add_sync(0xffffffffu, nst);
        if (lane == 0 && nst && cspin_of(p) > 0) cnt_add<false>(p.d_counters + (B200_CNT_PART + kvh) * B200_CNT_STRIDE, nst);
        if (TRACE && trace && tid == 0) trace[3] = global_ns();

        // ---- this block merges the splits of query heads split, split + n_split, ... of its KV head ----
#pragma unroll 1
        for (int gm = split; gm < G; gm += p.n_split) {
            const int head = kvh * G + gm;
            const b200_flagged *rec = p.d_attn_part + (size_t)head * p.n_split * (HD + 2);
            if (tid == 0)
                cnt_wait<false>(p.d_counters + (B200_CNT_PART + kvh) * B200_CNT_STRIDE, cnt_mul * (unsigned)(p.n_split * G * (HD + 2)), sm.flags, cspin_of(p));
            named_barrier(2, ATT_T);                 // also: the staging area is free (keys done, previous head merged)
            {
                constexpr int NB = 4;
                const int tot = p.n_split * (HD + 2);
#pragma unroll 1
                for (int i0 = tid * 2; i0 < tot; i0 += ATT_T * 2 * NB) {
                    float a[NB], b[NB];
                    fl_poll<NB, ATT_T * 2, false>(rec + i0, (tot - i0 + ATT_T * 2 - 1) / (ATT_T * 2), flag, a, b, sm.flags, p.d_err, spin);
#pragma unroll
                    for (int u = 0; u < NB; ++u) {
                        const int i = i0 + u * ATT_T * 2;
                        if (i < tot) *reinterpret_cast<float2 *>(stg + i) = make_float2(a[u], b[u]);
                    }
                }
            }
            named_barrier(2, ATT_T);
            // One warp turns the (max, sum) pairs of the splits into normalised weights, left where the
            // maxima were; every output element is then a plain weighted sum over the splits.
            if (warp == 0) {
                const bool has = lane < p.n_split;
                const float ms = stg[(has ? lane : 0) * (HD + 2) + HD];
                const float ls = has ? stg[lane * (HD + 2) + HD + 1] : 0.0f;
                const float M = warp_max(ls > 0.0f ? ms : -INFINITY);
                const float wgt = ls > 0.0f ? __expf(ms - M) : 0.0f;
                const float Lsum = warp_sum(ls * wgt);
                if (has) stg[lane * (HD + 2) + HD] = wgt / Lsum;
            }
            named_barrier(2, ATT_T);
            unsigned nout = 0;
#pragma unroll 1
            for (int d = tid; d < HD; d += ATT_T) {
                float O = 0.0f;
#pragma unroll 1
                for (int s = 0; s < p.n_split; ++s) O = fmaf(stg[s * (HD + 2) + d], stg[s * (HD + 2) + HD], O);
                fl_store<false>(p.d_attn_out + (size_t)head * HD + d, O, flag);
                ++nout;
            }
            nout = (unsigned)__reduce_add_sync(0xffffffffu, nout);
            if (lane == 0 && nout && cspin_of(p) > 0) cnt_add<false>(p.d_counters + B200_CNT_ATTN * B200_CNT_STRIDE, nout);
        }
    }
    // the o stage reuses the scratch area: nobody goes on before the attention threads are done with it
    named_barrier(1, TK_NC);
    if (TRACE && trace && tid == 0) trace[4] = global_ns();
}

// ---------------------------------------------------------------------------
// Producer: one thread issues every bulk copy of the block, stage after stage. Returns the advanced
// chunk number; bit 31 set = gave up.
// ---------------------------------------------------------------------------
// Asks L2 for this block's rows of a stage that the ring will only reach later: while the consumers
// hand results over (and the ring is full) HBM keeps working, and the ring later fills at L2 speed.
__device__ __forceinline__ void prefetch_share(const b200_token_args &p, int kind, const void *d_w)
{
    const b200_stage_geom &G = p.g[kind];
    const RowRange br = block_rows(G, blockIdx.x);
    const unsigned char *a = static_cast<const unsigned char *>(d_w) + (size_t)br.r0 * G.row_stride;
    long long left = (long long)(br.r1 - br.r0) * G.row_stride;
    if (left > (long long)p.l2_ahead_bytes) left = p.l2_ahead_bytes;
#pragma unroll 1
    for (; left > 0; left -= 16384, a += 16384) {
        const unsigned n = left < 16384 ? (unsigned)left : 16384u;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a), "r"(n) : "memory");
    }
}

__device__ __noinline__ unsigned produce_stage(const b200_token_args &p, int kind, const void *d_w, unsigned seq, unsigned long long *trace)
{
    const b200_stage_geom &G = p.g[kind];
    const Smem sm = smem_of(p);
    const int spin = spin_of(p);
    const int rb = G.rb;
    const RowRange br = block_rows(G, blockIdx.x);
    const unsigned char *wbase = static_cast<const unsigned char *>(d_w);
    const unsigned stride = (unsigned)G.row_stride;
    const uint32_t ring_s = smem_u32(sm.ring), full_s = smem_u32(sm.full);
    bool first = true;
#pragma unroll 1
    for (int w0 = br.r0; w0 < br.r1; w0 += G.pw) {
        const int w1 = w0 + G.pw < br.r1 ? w0 + G.pw : br.r1;
#pragma unroll 1
        for (int row0 = w0; row0 < w1; row0 += rb) {
            const unsigned slot = seq % TK_SLOTS;
            if (seq >= TK_SLOTS && !mbar_wait_abort(&sm.empty[slot], (seq / TK_SLOTS - 1u) & 1u, sm.flags, spin)) {
                if (!sm.flags[0]) raise(sm.flags, p.d_err, 2);
                return seq | 0x80000000u;
            }
            const unsigned bytes = (unsigned)(w1 - row0 < rb ? w1 - row0 : rb) * stride;
            const uint32_t bar = full_s + slot * 8u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(ring_s + slot * (unsigned)TK_SLOT_BYTES), "l"(wbase + (size_t)row0 * stride), "r"(bytes), "r"(bar) : "memory");
            if (trace) { const unsigned long long t = global_ns(); if (first) { trace[5] = t; first = false; } trace[6] = t; }
            ++seq;
        }
    }
    return sm.flags[0] ? (seq | 0x80000000u) : seq;
}

template <int WT, bool TRACE, bool MULTI>
__global__ void __launch_bounds__(TK_THREADS, 1)
decode_token_kernel(const __grid_constant__ b200_token_args p)
{
    const Smem sm = smem_of(p);
    const int tid = threadIdx.x;
    const int spin = spin_of(p);
    const int L = p.n_layers;

    if (tid == 0) {
        for (int i = 0; i < TK_SLOTS; ++i) { mbar_init(&sm.full[i], 1); mbar_init(&sm.empty[i], TK_NWARP); }
        mbar_init(sm.att_bar, 1);
        sm.flags[0] = 0; sm.flags[1] = 0;
        sm.flags[2] = (int)*p.d_epoch;               // read back from shared memory wherever it is needed: one
        sm.flags[3] = *p.d_pos;                      // register less to carry through every stage
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    {   // the layer table, once per token: every later pointer read is a shared-memory load
        const int words = L * (int)(sizeof(b200_token_layer) / 8);
        const unsigned long long *src = reinterpret_cast<const unsigned long long *>(p.d_layers);
        unsigned long long *dst = reinterpret_cast<unsigned long long *>(const_cast<b200_token_layer *>(sm.layers));
        for (int i = tid; i < words; i += TK_THREADS) dst[i] = src[i];
    }
    __syncthreads();
    unsigned long long *tr = (TRACE && p.d_trace) ? p.d_trace + (size_t)blockIdx.x * (6 * L + 1) * TK_TRACE_WORDS : nullptr;

    // ---------------- producer warp ----------------
    if (tid >= TK_NC) {
        if (tid == TK_NC) {
            unsigned seq = 0;
#pragma unroll 1
            for (int l = 0; l < L && !(seq >> 31); ++l) {
#pragma unroll 1
                for (int kind = 0; kind < 4 && !(seq >> 31); ++kind) {
                    const b200_token_layer &ly = sm.layers[l];
                    const void *w = kind == B200_ST_QKV ? ly.w_qkv : kind == B200_ST_O ? ly.w_o : kind == B200_ST_GATEUP ? ly.w_gateup : ly.w_down;
                    if (p.l2_ahead_bytes > 0) {
                        // the stage after this one
                        const int nk = kind == 3 ? (l + 1 < L ? B200_ST_QKV : (p.with_lm ? B200_ST_LM : -1)) : kind + 1;
                        if (nk >= 0) {
                            const b200_token_layer &nl = sm.layers[kind == 3 && l + 1 < L ? l + 1 : l];
                            const void *nw = nk == B200_ST_QKV ? nl.w_qkv : nk == B200_ST_O ? nl.w_o : nk == B200_ST_GATEUP ? nl.w_gateup
                                           : nk == B200_ST_DOWN ? nl.w_down : p.w_lm;
                            prefetch_share(p, nk, nw);
                        }
                    }
                    seq = produce_stage(p, kind, w, seq, tr ? tr + (size_t)(6 * l + (kind == 0 ? 0 : kind + 1)) * TK_TRACE_WORDS : nullptr);
                }
            }
            if (!(seq >> 31) && p.with_lm) seq = produce_stage(p, B200_ST_LM, p.w_lm, seq, tr ? tr + (size_t)(6 * L) * TK_TRACE_WORDS : nullptr);
            seq &= 0x7fffffffu;
            // copies still in flight must land before the block may leave: wait for the last fill of every slot
            const unsigned nfill = seq < TK_SLOTS ? seq : TK_SLOTS;
#pragma unroll 1
            for (unsigned i = 0; i < nfill; ++i) {
                const unsigned s = seq - 1u - i;
                mbar_wait_abort(&sm.full[s % TK_SLOTS], (s / TK_SLOTS) & 1u, sm.flags + 1, spin);   // flags[1] stays 0: a plain bounded wait
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // One loop over the stages with a single (inlined) call site per stage type: no function calls,
    // hence nothing saved to and restored from the stack between stages.
    unsigned state = 0;                              // chunk number | parity of the window number << 31
    const bool tail = p.with_lm || p.n_ranks > 1;    // the LM head, or the residual update that ends a prompt position
#pragma unroll 1
    for (int l = 0; l <= L; ++l) {
        if (l == L && !tail) break;
#pragma unroll 1
        for (int k = 0; k < 5; ++k) {
            if (l == L && k > 0) break;
            unsigned long long *t = tr ? tr + (size_t)(6 * l + k) * TK_TRACE_WORDS : nullptr;
            if (k == 1) {
                constexpr bool OWN = WT == B200_WT_Q8;
                if (p.hd == 128) attention_stage<128, TRACE, MULTI, OWN>(p, l, (unsigned)sm.flags[2], t);
                else if (p.hd == 64) attention_stage<64, TRACE, MULTI, OWN>(p, l, (unsigned)sm.flags[2], t);
                else attention_stage<256, TRACE, MULTI, OWN>(p, l, (unsigned)sm.flags[2], t);
            } else {
                const int kind = l == L ? B200_ST_LM : k == 0 ? B200_ST_QKV : k - 1;     // 2, 3, 4 -> o, gate/up, down
                state = run_matvec<WT, TRACE, MULTI>(p, kind, l, (unsigned)sm.flags[2], state, t);
            }
        }
    }

    const unsigned ep = (unsigned)sm.flags[2];
    const int pos = sm.flags[3];
    const unsigned flag_lm = ep * (unsigned)(L + 1) + (unsigned)L + 1u;
    if (p.with_lm) {
        // --- block 0 folds the best rows of all blocks (and all ranks) ---
        if (blockIdx.x == 0 && tid < 32) {
            const int lane = tid;
            float bv = -INFINITY; int bi = 0x7fffffff;
#pragma unroll 1
            for (int b0 = lane; b0 < (int)gridDim.x; b0 += 32 * 4) {
                float v[4], fi[4];
                const int cnt = ((int)gridDim.x - b0 + 31) / 32;
                fl_poll<4, 64, false>(p.d_am + 2 * b0, cnt, flag_lm, v, fi, sm.flags, p.d_err, spin);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (u < cnt && better(v[u], __float_as_int(fi[u]), bv, bi)) { bv = v[u]; bi = __float_as_int(fi[u]); }
            }
#pragma unroll 1
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (bi == 0x7fffffff) bi = 0;            // nothing compared greater (all NaN): index 0, as the reference's loop
            bi += (int)p.logits_offset;              // global row of a sharded LM head
            if (p.n_ranks > 1) {
                // (value, row) to every rank, then the best of all ranks, lowest row on ties
                __threadfence_system();
                if (lane < p.n_ranks) {
                    fl_store<true>(p.d_peer_am[lane], bv, flag_lm);
                    fl_store<true>(p.d_peer_am[lane] + 1, __int_as_float(bi), flag_lm);
                }
                float gv[1], gf[1];
                fl_poll<1, 2, true>(p.d_am_rank + 2 * (lane < p.n_ranks ? lane : 0), lane < p.n_ranks ? 1 : 0, flag_lm, gv, gf, sm.flags, p.d_err, spin);
                float xv = lane < p.n_ranks ? gv[0] : -INFINITY;
                int xi = lane < p.n_ranks ? __float_as_int(gf[0]) : 0x7fffffff;
#pragma unroll 1
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, xv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, xi, o);
                    if (better(ov, oi, xv, xi)) { xv = ov; xi = oi; }
                }
                if (xi == 0x7fffffff) xi = 0;
                bi = xi;
                __threadfence_system();
            }
            if (lane == 0 && pos + 1 >= *p.d_prompt_len) p.d_tokens[pos + 1] = bi;
        }
    }
    if (blockIdx.x == 0 && tid == 0) {
        *p.d_pos = pos + 1;
        *p.d_epoch = ep + 1u;
    }
}

int g_tk_sm_count = 0;

int tk_sm_count()
{
    if (!g_tk_sm_count) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            return 0;
        g_tk_sm_count = n;
    }
    return g_tk_sm_count;
}

int plan_stage(b200_stage_geom &g, int wtype, int n_blocks, int xin_floats)
{
    if (g.rows <= 0 || g.cols <= 0 || g.row_stride <= 0 || (g.row_stride % 16)) return B200_E_BADARG;
    if (wtype == B200_WT_Q8 ? (g.cols % 32) : (g.cols % 8)) return B200_E_BADARG;
    if (g.row_stride < (long long)b200_packed_row_stride(wtype, g.cols)) return B200_E_BADARG;
    const int ralign = g.glu ? 2 : 1;
    if (g.rows % ralign) return B200_E_BADARG;
    const int E = wtype == B200_WT_Q8 ? 16 : 8;
    const int nsl = (g.cols + E - 1) / E;
    // One 16-byte slice per thread up to 640 slices; two per thread beyond that, for binary16 rows only
    // (Q8_0 rows of more than 10240 columns are refused: the caller keeps its per-stage kernels).
    g.spt = nsl <= TK_NC ? 1 : 2;
    if (g.spt == 2 && wtype == B200_WT_Q8) return B200_E_TOOLARGE;
    g.T = (((nsl + g.spt - 1) / g.spt) + 31) / 32 * 32;
    if (g.T > TK_NC) return B200_E_TOOLARGE;
    g.NG = TK_NC / g.T;
    if (g.NG > TK_NWARP) g.NG = TK_NWARP;
    // a chunk (one ring slot) holds rg rows for each group: as many as fit, a power of two up to 8
    // (2 with two slices per thread: the row partials of a chunk live in registers)
    const int fit = (int)(TK_SLOT_BYTES / g.row_stride);          // rows per slot
    if (fit < ralign) return B200_E_TOOLARGE;
    while (g.NG > 1 && g.NG * ralign > fit) --g.NG;               // a slot must hold at least one row (pair) per group
    int rg = g.spt == 1 ? 8 : 2;
    while (rg > ralign && rg * g.NG > fit) rg >>= 1;
    if (rg * g.NG > fit || rg < ralign) return B200_E_TOOLARGE;
    g.rg = rg;
    g.rb = rg * g.NG;
    const int nwgp = (g.T / 32) | 1;
    int pw = TK_PART / nwgp;                           // rows whose warp partials fit one buffer
    pw -= pw % g.rb;                                   // whole chunks in a full window
    if (pw < g.rb) return B200_E_TOOLARGE;
    g.pw = pw;
    const int units = g.rows / ralign;
    g.cta_base = units / n_blocks;
    g.cta_rem = units % n_blocks;
    if (g.cols > xin_floats) return B200_E_TOOLARGE;   // the input vector is held in shared memory once per block
    g.direct_in = 0;
    return 0;
}

} // namespace

extern "C" int b200_token_plan(b200_token_args *a, int n_blocks)
{
    if (!a || a->n_layers <= 0 || a->d_model <= 0 || (a->d_model % 4)) return B200_E_BADARG;
    if (a->wtype != B200_WT_Q8 && a->wtype != B200_WT_F16) return B200_E_BADARG;
    if (a->n_kv <= 0 || a->n_q <= 0 || a->n_q % a->n_kv || (a->hd != 64 && a->hd != 128 && a->hd != 256)) return B200_E_BADARG;
    const int G = a->n_q / a->n_kv;
    if (G != 1 && G != 2 && G != 4 && G != 8) return B200_E_BADARG;
    if (a->n_ranks < 1 || a->n_ranks > B200_MAX_PEERS || a->rank < 0 || a->rank >= a->n_ranks) return B200_E_BADARG;
    if (n_blocks <= 0) n_blocks = tk_sm_count();
    if (n_blocks <= 0) return B200_E_STATE;
    // sequence splits: items (kv head, split) must fit the blocks; at least 32 cache rows per split at full
    // length; by default few enough that the block merging a head reads little (18, or 9 for wide heads)
    int ns = a->n_split > 0 ? a->n_split : (a->hd > 128 ? 9 : 18);
    if (ns > n_blocks / a->n_kv) ns = n_blocks / a->n_kv;
    if (ns > (a->max_seq + 31) / 32) ns = (a->max_seq + 31) / 32;
    if (ns > 32) ns = 32;
    if (ns < 1) return B200_E_TOOLARGE;                // more KV heads than blocks
    a->n_split = ns;
    // Shared memory beyond the ring and the fixed areas is one scratch area: the block-wide input vector
    // of the o and down stages, the slot sums of a normalised residual update, and the attention stage's
    // buffers with as many staged cache rows as fit.
    const Layout fixed = make_layout(a->n_layers, a->d_model, 0);
    int scratch = (232448 - 128 - fixed.total) / 4;
    scratch -= scratch % 4;
    const int att_fixed = attention_fixed_floats(G, a->hd);
    const int chunk_cap = (a->max_seq + ns - 1) / ns;
    int keys = scratch > att_fixed ? (scratch - att_fixed) / a->hd : 0;
    if (keys > chunk_cap) keys = chunk_cap;
    if (keys * a->hd < ns * (a->hd + 2) || keys < 1 || scratch < 2 * a->d_model) return B200_E_TOOLARGE;
    a->att_keys = keys;
    int need = att_fixed + keys * a->hd;               // what is actually used: the rest is left to L1
    if (need < 2 * a->d_model) need = 2 * a->d_model;  // slot sums and the stage's norm weights
    for (int k = 0; k < B200_ST_KINDS; ++k) {
        int rc = plan_stage(a->g[k], a->wtype, n_blocks, scratch);
        if (rc) return rc;
        if ((k == B200_ST_O || k == B200_ST_DOWN) && !a->g[k].direct_in && a->g[k].cols > need) need = a->g[k].cols;
    }
    scratch = (need + 3) / 4 * 4;
    if (a->l2_ahead_bytes < 0) a->l2_ahead_bytes = 0;     // default 0: measured slower than leaving the order of HBM requests to the ring
    if (a->g[B200_ST_QKV].cols != a->d_model || a->g[B200_ST_GATEUP].cols != a->d_model || !a->g[B200_ST_GATEUP].glu ||
        a->g[B200_ST_QKV].rows != (a->n_q + 2 * a->n_kv) * a->hd || a->g[B200_ST_O].cols != a->n_q * a->hd ||
        a->g[B200_ST_O].rows != a->d_model || a->g[B200_ST_DOWN].rows != a->d_model ||
        a->g[B200_ST_DOWN].cols != a->g[B200_ST_GATEUP].rows / 2 || a->g[B200_ST_QKV].glu || a->g[B200_ST_O].glu ||
        a->g[B200_ST_DOWN].glu || a->g[B200_ST_LM].cols != a->d_model || a->g[B200_ST_LM].glu)
        return B200_E_BADARG;
    a->scratch_floats = scratch;
    a->n_blocks = n_blocks;
    const Layout lo = make_layout(a->n_layers, a->d_model, scratch);
    a->smem_bytes = lo.total;
    if (a->smem_bytes > 232448) return B200_E_TOOLARGE;
    return 0;
}

extern "C" int b200_token_chunks(const b200_token_args *a, int kind, int block, int *out, int cap)
{
    if (!a || kind < 0 || kind >= B200_ST_KINDS || block < 0 || block >= a->n_blocks) return B200_E_BADARG;
    const b200_stage_geom &G = a->g[kind];
    const RowRange br = block_rows(G, block);
    int n = 0;
    for (int w0 = br.r0; w0 < br.r1; w0 += G.pw) {
        const int w1 = w0 + G.pw < br.r1 ? w0 + G.pw : br.r1;
        for (int row0 = w0; row0 < w1; row0 += G.rb) {
            if (out && n < cap) { out[3 * n] = row0; out[3 * n + 1] = min(G.rb, w1 - row0); out[3 * n + 2] = (w0 - br.r0) / G.pw; }
            ++n;
        }
    }
    return n;
}

extern "C" int b200_decode_token(const b200_token_args *ap, void *stream)
{
    if (!ap || !ap->d_layers || !ap->d_pos || !ap->d_tokens || !ap->d_prompt_len || !ap->d_epoch || !ap->d_err || !ap->d_emb ||
        !ap->d_qkv || !ap->d_attn_part || !ap->d_attn_out || !ap->d_act || !ap->d_slots_o || !ap->d_slots_dn || !ap->d_counters)
        return B200_E_BADARG;
    if (ap->n_blocks <= 0 || ap->smem_bytes <= 0 || ap->scratch_floats <= 0) return B200_E_STATE;   // b200_token_plan first
    if (ap->with_lm && (!ap->w_lm || !ap->g_final || !ap->d_logits || !ap->d_am || ap->g[B200_ST_LM].rows <= 0)) return B200_E_BADARG;
    if (ap->n_ranks > 1 && ap->with_lm && !ap->d_am_rank) return B200_E_BADARG;
    for (int q = 0; q < ap->n_ranks; ++q)
        if (!ap->d_peer_slots_o[q] || !ap->d_peer_slots_dn[q] || !ap->d_peer_counters[q] || (ap->n_ranks > 1 && ap->with_lm && !ap->d_peer_am[q])) return B200_E_BADARG;
    if (ap->n_kv * ap->n_split > ap->n_blocks || B200_CNT_PART + ap->n_kv > 72) return B200_E_BADARG;
    const int sms = tk_sm_count();
    if (sms <= 0) return B200_E_STATE;
    if (ap->n_blocks > sms) return B200_E_TOOLARGE;    // all blocks must be resident at once
    void (*kern)(const b200_token_args);
    const bool multi = ap->n_ranks > 1, trace = ap->d_trace != nullptr;
#define TK_PICK(WT_) (multi ? (trace ? decode_token_kernel<WT_, true, true> : decode_token_kernel<WT_, false, true>) \
                            : (trace ? decode_token_kernel<WT_, true, false> : decode_token_kernel<WT_, false, false>))
    kern = ap->wtype == B200_WT_Q8 ? TK_PICK(B200_WT_Q8) : TK_PICK(B200_WT_F16);
#undef TK_PICK
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ap->smem_bytes);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ap->n_blocks);
    cfg.blockDim = dim3(TK_THREADS);
    cfg.dynamicSmemBytes = ap->smem_bytes;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // all blocks resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, kern, *ap);
}
