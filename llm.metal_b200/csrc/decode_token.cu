// Whole-token decode kernel (sm_100a): every matvec and attention step of one
// token in one persistent, cooperative launch of one block per SM.
//
// Why: a batch-1 token is ~180 dependent steps of a few microseconds of HBM
// time each. As separate kernels each step pays launch, pipeline fill and
// drain; here the steps are separated by device-wide barriers only, and the
// producer warp of every block runs ahead of the consumers through the whole
// step list, so the next steps' weights are already in shared memory when a
// barrier opens. Weights stream through a ring of 8 slots filled by bulk
// asynchronous copies (TMA) and released through mbarriers; the arithmetic of
// a stage is the one of matvec.cu (stream_core.cuh), the attention step is the
// split-sequence scheme of attention.cu.
//
// Every wait (mbarrier, device-wide barrier, peer flag) is bounded: when one
// runs out the block raises the error word and a shared abort flag, after
// which all loops fall through and the kernel ends.
#include "stream_core.cuh"
#include "../../include/llmb200_kernels.h"

#include <stdio.h>

extern unsigned long long g_b200_launches;

namespace {

constexpr int TK_CONSUMERS = 640;
constexpr int TK_THREADS = TK_CONSUMERS + 32;
constexpr int TK_SLOTS = 8;
constexpr int TK_SLOT_BYTES = 22016;                 // 172 * 128; >= rb * row_stride of every step
constexpr int TK_ATT_BYTES = 43008;                  // attention scratch; the shared input vector aliases it
constexpr int TK_XS_FLOATS = 4096;                   // largest input vector handed over through shared memory
constexpr int TK_MAX_WARPS = TK_CONSUMERS / 32;
constexpr int ATT_T = 256;                           // consumer threads that work on an attention item

struct Smem {
    unsigned char *ring;
    uint64_t *full, *empty;
    float *wpart;        // [TK_SLOTS][TK_MAX_WARPS][8] partial row sums of the stage in each slot
    int *cnt;            // [TK_SLOTS] warps that have delivered their partials
    float *red;          // [8][32]
    float *am_v; int *am_i;   // [TK_MAX_WARPS * 8] each
    int *flags;          // [0] abort, [1] last-block
    float *att;          // TK_ATT_BYTES, also xs
};

__device__ __forceinline__ Smem carve(unsigned char *base)
{
    Smem s;
    s.ring = base;
    unsigned char *p = base + (size_t)TK_SLOTS * TK_SLOT_BYTES;
    s.full = reinterpret_cast<uint64_t *>(p); p += TK_SLOTS * 8;
    s.empty = reinterpret_cast<uint64_t *>(p); p += TK_SLOTS * 8;
    s.wpart = reinterpret_cast<float *>(p); p += TK_SLOTS * TK_MAX_WARPS * 8 * 4;
    s.cnt = reinterpret_cast<int *>(p); p += TK_SLOTS * 4 + 32;
    s.red = reinterpret_cast<float *>(p); p += 8 * 32 * 4;
    s.am_v = reinterpret_cast<float *>(p); p += TK_MAX_WARPS * 8 * 4;
    s.am_i = reinterpret_cast<int *>(p); p += TK_MAX_WARPS * 8 * 4;
    s.flags = reinterpret_cast<int *>(p); p += 64;
    s.att = reinterpret_cast<float *>(p);
    return s;
}
constexpr size_t TK_SMEM_BYTES = (size_t)TK_SLOTS * TK_SLOT_BYTES + TK_SLOTS * 16 + TK_SLOTS * TK_MAX_WARPS * 8 * 4 + (TK_SLOTS * 4 + 32) +
                                 8 * 32 * 4 + TK_MAX_WARPS * 8 * 8 + 64 + TK_ATT_BYTES;
static_assert(TK_SMEM_BYTES <= 232448, "more shared memory than an sm_100 block can have");

// Rows of a step owned by this block, and by each of its consumer groups.
struct RowSplit { int r0, r1; };
__device__ __forceinline__ RowSplit block_rows(const b200_op &op)
{
    const int ralign = op.out_mode == B200_OUT_GLU ? 2 : 1;
    const long long units = op.rows / ralign;
    RowSplit r;
    r.r0 = (int)(units * blockIdx.x / gridDim.x) * ralign;
    r.r1 = (int)(units * (blockIdx.x + 1) / gridDim.x) * ralign;
    return r;
}
__device__ __forceinline__ RowSplit group_rows(const b200_op &op, const RowSplit &b, int g)
{
    const int ralign = op.out_mode == B200_OUT_GLU ? 2 : 1;
    const int units = (b.r1 - b.r0) / ralign;
    RowSplit r;
    r.r0 = b.r0 + (int)((long long)units * g / op.NG) * ralign;
    r.r1 = b.r0 + (int)((long long)units * (g + 1) / op.NG) * ralign;
    return r;
}

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// mbarrier wait that also ends as soon as the block's abort flag is up, so that after one failed wait
// every later wait returns at once and the block still walks through all its barriers.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t *b, unsigned parity, volatile int *abort_flag)
{
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_try_wait(b, parity)) return true;
        if ((it & 63) == 63 && *abort_flag) return false;
    }
    return false;
}

// Device-wide barrier over the consumer threads of all blocks. `target` is the total number of
// arrivals expected so far. Returns false when the wait ran out.
__device__ __forceinline__ bool grid_barrier(unsigned *counter, unsigned target, int tid, volatile int *abort_flag)
{
    named_barrier(1, TK_CONSUMERS);
    if (tid == 0) {
        __threadfence();
        atomicAdd(counter, 1u);                         // always arrive, so that the other blocks are not held up
        bool ok = *abort_flag != 0;
        for (int it = 0; it < B200_SPIN_LIMIT / 2 && !ok; ++it) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if ((int)(v - target) >= 0) ok = true;
        }
        if (!ok) *abort_flag = 1;
        abort_flag[3] = *abort_flag;                    // the block's decision, read by everyone after the barrier
        __threadfence();
    }
    named_barrier(1, TK_CONSUMERS);
    return !abort_flag[3];
}

// ---------------------------------------------------------------------------
// One matvec step, consumer side.
// ---------------------------------------------------------------------------
template <int WT, int SPT, int RB>
__device__ __forceinline__ void matvec_step(const b200_op &op, const b200_token_args &p, const Smem &sm, int tid, int pos,
                                            unsigned &fill_parity, float &best_v, int &best_i, unsigned long long *trace)
{
    constexpr int E = (WT == B200_WT_Q8) ? 16 : 8;
    const int T = op.T, NG = op.NG, spg = TK_SLOTS / NG;
    const int g = tid / T, t = tid - g * T, lane = t & 31, wg = t >> 5, nwg = T >> 5;
    const bool active = g < NG;                        // threads beyond NG*T sit this step out
    const RowSplit br = block_rows(op);

    if (active) {
        int col[SPT];
        bool on[SPT];
#pragma unroll
        for (int s = 0; s < SPT; ++s) { col[s] = (s * T + t) * E; on[s] = col[s] < op.cols; }
        float *gred = sm.red + g * 32;
        float *xs = sm.att;
        const bool share_x = NG > 1 && (op.in_mode != B200_IN_VEC || op.d_norm_gamma) && SPT * T * E <= TK_XS_FLOATS;

        // ---------------- input assembly ----------------
        float x[SPT][E];
        if (!share_x || g == 0) {
            if (op.in_mode == B200_IN_VEC) {
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; e += 4) {
                        // produced earlier in this same kernel by other SMs: read from L2
                        float4 v4 = on[s] ? __ldcg(reinterpret_cast<const float4 *>(op.d_in_vec + col[s] + e)) : make_float4(0, 0, 0, 0);
                        x[s][e] = v4.x; x[s][e + 1] = v4.y; x[s][e + 2] = v4.z; x[s][e + 3] = v4.w;
                    }
            } else {
                if (op.in_mode == B200_IN_EMBED) {
                    long long tok = p.d_tokens[pos];
                    if (tok < 0 || tok >= p.emb_rows) tok = 0;
                    const float *er = p.d_emb + tok * (long long)op.cols;
#pragma unroll
                    for (int s = 0; s < SPT; ++s)
#pragma unroll
                        for (int e = 0; e < E; e += 4) {
                            float4 v4 = on[s] ? *reinterpret_cast<const float4 *>(er + col[s] + e) : make_float4(0, 0, 0, 0);
                            x[s][e] = v4.x * p.emb_scale; x[s][e + 1] = v4.y * p.emb_scale;
                            x[s][e + 2] = v4.z * p.emb_scale; x[s][e + 3] = v4.w * p.emb_scale;
                        }
                } else {
                    float sacc[SPT][E];
#pragma unroll
                    for (int s = 0; s < SPT; ++s)
#pragma unroll
                        for (int e = 0; e < E; ++e) sacc[s][e] = 0.0f;
                    for (int k = 0; k < op.n_slots; ++k) {
                        const float *sl = op.d_slots + (long long)k * op.slot_stride;
#pragma unroll
                        for (int s = 0; s < SPT; ++s)
#pragma unroll
                            for (int e = 0; e < E; e += 4)
                                if (on[s]) {
                                    float4 v4 = __ldcg(reinterpret_cast<const float4 *>(sl + col[s] + e));
                                    sacc[s][e] += v4.x; sacc[s][e + 1] += v4.y; sacc[s][e + 2] += v4.z; sacc[s][e + 3] += v4.w;
                                }
                    }
                    if (op.d_slot_norm_gamma) {
                        float ss = 0.0f;
#pragma unroll
                        for (int s = 0; s < SPT; ++s)
#pragma unroll
                            for (int e = 0; e < E; ++e) ss = fmaf(sacc[s][e], sacc[s][e], ss);
                        ss = group_sum(ss, gred, 2 + g, T, t);
                        const float inv = 1.0f / sqrtf(ss / (float)op.cols + p.eps);
#pragma unroll
                        for (int s = 0; s < SPT; ++s)
#pragma unroll
                            for (int e = 0; e < E; ++e)
                                if (on[s]) sacc[s][e] = op.d_slot_norm_gamma[col[s] + e] * sacc[s][e] * inv;
                    }
#pragma unroll
                    for (int s = 0; s < SPT; ++s)
#pragma unroll
                        for (int e = 0; e < E; e += 4) {
                            float4 v4 = on[s] ? __ldcg(reinterpret_cast<const float4 *>(op.d_resid_in + col[s] + e)) : make_float4(0, 0, 0, 0);
                            x[s][e] = v4.x + sacc[s][e]; x[s][e + 1] = v4.y + sacc[s][e + 1];
                            x[s][e + 2] = v4.z + sacc[s][e + 2]; x[s][e + 3] = v4.w + sacc[s][e + 3];
                        }
                }
                if (blockIdx.x == 0 && g == 0 && op.d_resid_out) {
#pragma unroll
                    for (int s = 0; s < SPT; ++s)
#pragma unroll
                        for (int e = 0; e < E; e += 4)
                            if (on[s])
                                *reinterpret_cast<float4 *>(op.d_resid_out + col[s] + e) =
                                    make_float4(x[s][e], x[s][e + 1], x[s][e + 2], x[s][e + 3]);
                }
            }
            if (op.d_norm_gamma) {
                float gm[SPT][E];
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; e += 4) {
                        float4 v4 = on[s] ? *reinterpret_cast<const float4 *>(op.d_norm_gamma + col[s] + e) : make_float4(0, 0, 0, 0);
                        gm[s][e] = v4.x; gm[s][e + 1] = v4.y; gm[s][e + 2] = v4.z; gm[s][e + 3] = v4.w;
                    }
                float ss = 0.0f;
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; ++e) ss = fmaf(x[s][e], x[s][e], ss);
                ss = group_sum(ss, gred, 2 + g, T, t);
                const float inv = 1.0f / sqrtf(ss / (float)op.cols + p.eps);
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; ++e) x[s][e] = gm[s][e] * x[s][e] * inv;
            }
        }
        if (share_x) {
            if (g == 0) {
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; e += 4)
                        *reinterpret_cast<float4 *>(xs + (size_t)(s * T + t) * E + e) = make_float4(x[s][e], x[s][e + 1], x[s][e + 2], x[s][e + 3]);
            }
            named_barrier(10, NG * T);
            if (g != 0) {
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; e += 4) {
                        const float4 v4 = *reinterpret_cast<const float4 *>(xs + (size_t)(s * T + t) * E + e);
                        x[s][e] = v4.x; x[s][e + 1] = v4.y; x[s][e + 2] = v4.z; x[s][e + 3] = v4.w;
                    }
            }
        }

        if (trace && tid == 0) trace[2] = global_ns();
        // ---------------- this group's stages ----------------
        uint32_t qoff[SPT], soff[SPT];
#pragma unroll
        for (int s = 0; s < SPT; ++s) {
            const int c = on[s] ? col[s] : 0;
            qoff[s] = (uint32_t)(WT == B200_WT_Q8 ? c : 2 * c);
            soff[s] = (uint32_t)op.cols + (uint32_t)(c >> 5) * 2u;
        }
        const uint32_t ring_s = smem_u32(sm.ring), stride = (uint32_t)op.row_stride;
        const RowSplit gr = group_rows(op, br, g);
        const int nst = (gr.r1 - gr.r0 + RB - 1) / RB;
        for (int k = 0; k < nst; ++k) {
            const int slot = g * spg + (k % spg);
            const unsigned par = ((fill_parity >> slot) + (unsigned)(k / spg)) & 1u;
            if (!mbar_wait_or_abort(&sm.full[slot], par, sm.flags)) { sm.flags[0] = 1; if (p.d_err) *p.d_err = 3; }
            if (trace && tid == 0 && k == 0) trace[3] = global_ns();
            const uint32_t sb = ring_s + (uint32_t)slot * TK_SLOT_BYTES;
            const int row0 = gr.r0 + k * RB;
            const int nr = min(RB, gr.r1 - row0);
            // rows are fetched from the slot four at a time: enough loads in flight, few live registers
            constexpr int CH = RB < 4 ? RB : 4;
            float v[RB];
#pragma unroll
            for (int jb = 0; jb < RB; jb += CH) {
                uint4 wq[CH][SPT];
                uint32_t ws[CH][SPT];
#pragma unroll
                for (int j = 0; j < CH; ++j)
#pragma unroll
                    for (int s = 0; s < SPT; ++s) {
                        wq[j][s] = lds_128(sb + (uint32_t)(jb + j) * stride + qoff[s]);
                        if (WT == B200_WT_Q8) ws[j][s] = lds_u16(sb + (uint32_t)(jb + j) * stride + soff[s]);
                    }
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    float acc = 0.0f;
#pragma unroll
                    for (int s = 0; s < SPT; ++s) {
                        float d;
                        if (WT == B200_WT_Q8) d = __half2float(__ushort_as_half((unsigned short)ws[j][s])) * dot16_q8(wq[j][s], x[s]);
                        else d = dot8_f16(wq[j][s], x[s]);
                        acc += d;
                    }
                    v[jb + j] = acc;
                }
            }
            // Warps run free of each other: each leaves its partial sums of the stage's rows in shared memory
            // and counts itself in; the warp that arrives last (no waiting involved) adds the partials in warp
            // order, emits the rows and hands the slot back to the producer.
            const float tot = reduce_rows<RB>(v, lane);
            float *wp = sm.wpart + (size_t)slot * TK_MAX_WARPS * 8;
            if (lane < RB) wp[wg * 8 + lane] = tot;
            __threadfence_block();
            int last = 0;
            if (lane == 0) last = (atomicAdd(&sm.cnt[slot], 1) == nwg - 1);
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
                float y = 0.0f;
                if (lane < RB)
                    for (int w = 0; w < nwg; ++w) y += wp[w * 8 + lane];
                __syncwarp();
                if (lane == 0) { sm.cnt[slot] = 0; mbar_arrive(&sm.empty[slot]); }
                const int row = row0 + lane;
                if (op.out_mode == B200_OUT_GLU) {
                    const float u = __shfl_down_sync(0xffffffffu, y, 1);
                    if (lane < nr && !(lane & 1)) {
                        const float a = op.act == 0 ? act_silu(y) : act_gelu_tanh(y);
                        op.d_out[0][op.out_offset + (row >> 1)] = a * u;
                    }
                } else if (lane < nr) {
                    for (int q = 0; q < op.n_out; ++q) op.d_out[q][op.out_offset + row] = y;
                    if (op.argmax && better(y, row, best_v, best_i)) { best_v = y; best_i = row; }
                }
            }
        }
    }
    // every consumer thread advances the fill parities of all slots by this step's stage counts
    for (int gg = 0; gg < NG; ++gg) {
        const RowSplit gr = group_rows(op, br, gg);
        const int nst = (gr.r1 - gr.r0 + RB - 1) / RB;
        for (int j = 0; j < spg; ++j) {
            const int fills = nst > j ? (nst - j + spg - 1) / spg : 0;
            fill_parity ^= (unsigned)(fills & 1) << (gg * spg + j);
        }
    }
}

// ---------------------------------------------------------------------------
// One attention step: items (kv head, sequence split) are dealt to the blocks;
// the first ATT_T consumer threads of a block work on an item. Scheme and math
// as in attention.cu; the last block to finish a KV head merges its splits.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void halves8_to_float(const uint4 &u, float *f)
{
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

template <int HD, int G>
__device__ __forceinline__ void attention_step(const b200_op &op, const b200_token_args &p, const Smem &sm, int tid, int pos)
{
    constexpr int TPK = HD / 8;                 // threads per key row in the PV pass
    constexpr int KPW = 32 / TPK;               // key rows a warp handles side by side
    constexpr int HALF = HD / 2;
    constexpr int NW = ATT_T / 32;
    if (tid >= ATT_T) return;
    const int chunk_cap = (p.max_seq + p.n_split - 1) / p.n_split;
    float *q_s = sm.att;                        // [G][HD]
    float *k_new = q_s + G * HD;                // [HD]
    float *v_new = k_new + HD;                  // [HD]
    float *ml = v_new + HD;                     // [2*G]
    float *scores = ml + 16;                    // [G][chunk_cap]
    float *ored = scores + (size_t)G * chunk_cap;  // [NW][G][HD]
    const int lane = tid & 31, warp = tid >> 5;
    const int n = pos + 1;
    const int chunk = (n + p.n_split - 1) / p.n_split;
    const int n_items = p.n_kv * p.n_split;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int kvh = item / p.n_split, split = item - kvh * p.n_split;
        const int j0 = min(split * chunk, n), j1 = min(j0 + chunk, n);
        const int len = j1 - j0;
        __half *kc = static_cast<__half *>(op.d_k_cache) + (size_t)kvh * p.max_seq * HD;
        __half *vc = static_cast<__half *>(op.d_v_cache) + (size_t)kvh * p.max_seq * HD;

        for (int vi = warp; vi <= G; vi += NW) {
            const bool is_k = (vi == G);
            const float *src = is_k ? op.d_qkv + (size_t)p.n_q * HD + (size_t)kvh * HD : op.d_qkv + (size_t)(kvh * G + vi) * HD;
            const float *gamma = is_k ? op.d_k_gamma : op.d_q_gamma;
            float a[HALF / 32], b[HALF / 32];
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < HALF / 32; ++j) {
                const int d = lane + 32 * j;
                a[j] = __ldcg(src + d); b[j] = __ldcg(src + d + HALF);
                ss = fmaf(a[j], a[j], ss); ss = fmaf(b[j], b[j], ss);
            }
            ss = warp_sum(ss);
            if (gamma) {
                const float inv = 1.0f / sqrtf(ss / (float)HD + p.eps);
#pragma unroll
                for (int j = 0; j < HALF / 32; ++j) {
                    const int d = lane + 32 * j;
                    a[j] = gamma[d] * a[j] * inv; b[j] = gamma[d + HALF] * b[j] * inv;
                }
            }
#pragma unroll
            for (int j = 0; j < HALF / 32; ++j) {
                const int d = lane + 32 * j;
                float sn, cs;
                sincosf((float)pos * op.d_inv_freq[d], &sn, &cs);
                const float r0 = a[j] * cs - b[j] * sn, r1 = a[j] * sn + b[j] * cs;
                if (is_k) {
                    const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
                    k_new[d] = __half2float(h0); k_new[d + HALF] = __half2float(h1);
                    if (split == 0) { kc[(size_t)pos * HD + d] = h0; kc[(size_t)pos * HD + d + HALF] = h1; }
                } else {
                    q_s[vi * HD + d] = r0; q_s[vi * HD + d + HALF] = r1;
                }
            }
            if (is_k) {
                const float *vsrc = op.d_qkv + (size_t)(p.n_q + p.n_kv) * HD + (size_t)kvh * HD;
                for (int d = lane; d < HD; d += 32) {
                    const __half h = __float2half_rn(__ldcg(vsrc + d));
                    v_new[d] = __half2float(h);
                    if (split == 0) vc[(size_t)pos * HD + d] = h;
                }
            }
        }
        named_barrier(11, ATT_T);

        const float scale = 1.0f / sqrtf((float)HD);
        for (int j = j0 + tid; j < j1; j += ATT_T) {
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.0f;
            if (j == pos) {
                for (int d = 0; d < HD; ++d) {
                    const float kv = k_new[d];
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g] = fmaf(q_s[g * HD + d], kv, acc[g]);
                }
            } else {
                const uint4 *kr = reinterpret_cast<const uint4 *>(kc + (size_t)j * HD);
#pragma unroll 4
                for (int c = 0; c < HD / 8; ++c) {
                    float kf[8];
                    halves8_to_float(__ldcg(kr + c), kf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float4 qa = *reinterpret_cast<const float4 *>(q_s + g * HD + 8 * c);
                        const float4 qb = *reinterpret_cast<const float4 *>(q_s + g * HD + 8 * c + 4);
                        float t = acc[g];
                        t = fmaf(qa.x, kf[0], t); t = fmaf(qa.y, kf[1], t); t = fmaf(qa.z, kf[2], t); t = fmaf(qa.w, kf[3], t);
                        t = fmaf(qb.x, kf[4], t); t = fmaf(qb.y, kf[5], t); t = fmaf(qb.z, kf[6], t); t = fmaf(qb.w, kf[7], t);
                        acc[g] = t;
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) scores[(size_t)g * chunk_cap + (j - j0)] = acc[g] * scale;
        }
        named_barrier(11, ATT_T);

        for (int g = warp; g < G; g += NW) {
            float *sc = scores + (size_t)g * chunk_cap;
            float m = -INFINITY;
            for (int i = lane; i < len; i += 32) m = fmaxf(m, sc[i]);
            m = warp_max(m);
            float l = 0.0f;
            for (int i = lane; i < len; i += 32) { const float e = expf(sc[i] - m); sc[i] = e; l += e; }
            l = warp_sum(l);
            if (lane == 0) { ml[2 * g] = m; ml[2 * g + 1] = l; }
        }
        named_barrier(11, ATT_T);

        {
            const int kl = lane / TPK, dl = lane % TPK;
            float acc[G][8];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
            for (int j = j0 + warp * KPW + kl; j < j1; j += NW * KPW) {
                float vf[8];
                if (j == pos) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) vf[e] = v_new[8 * dl + e];
                } else {
                    halves8_to_float(__ldcg(reinterpret_cast<const uint4 *>(vc + (size_t)j * HD) + dl), vf);
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = scores[(size_t)g * chunk_cap + (j - j0)];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj, vf[e], acc[g][e]);
                }
            }
#pragma unroll
            for (int o = TPK; o < 32; o <<= 1)
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
            if (lane < TPK) {
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int e = 0; e < 8; ++e) ored[((size_t)warp * G + g) * HD + 8 * dl + e] = acc[g][e];
            }
        }
        named_barrier(11, ATT_T);
        for (int o = tid; o < G * HD; o += ATT_T) {
            const int g = o / HD, d = o % HD;
            float v = 0.0f;
#pragma unroll
            for (int k = 0; k < NW; ++k) v += ored[((size_t)k * G + g) * HD + d];
            p.d_attn_scratch[((size_t)(kvh * G + g) * p.n_split + split) * (HD + 2) + d] = v;
        }
        if (tid < 2 * G) {
            const int g = tid >> 1;
            p.d_attn_scratch[((size_t)(kvh * G + g) * p.n_split + split) * (HD + 2) + HD + (tid & 1)] = ml[tid];
        }
        __threadfence();
        named_barrier(11, ATT_T);
        if (tid == 0) sm.flags[1] = (atomicAdd(p.d_attn_tickets + kvh, 1u) == (unsigned)p.n_split - 1u);
        named_barrier(11, ATT_T);
        if (sm.flags[1]) {
            __threadfence();
            for (int o = tid; o < G * HD; o += ATT_T) {
                const int g = o / HD, d = o % HD;
                const float *base = p.d_attn_scratch + (size_t)(kvh * G + g) * p.n_split * (HD + 2);
                float M = -INFINITY;
                for (int s = 0; s < p.n_split; ++s) M = fmaxf(M, __ldcg(base + (size_t)s * (HD + 2) + HD));
                float Lsum = 0.0f, acc = 0.0f;
                for (int s = 0; s < p.n_split; ++s) {
                    const float m = __ldcg(base + (size_t)s * (HD + 2) + HD);
                    const float l = __ldcg(base + (size_t)s * (HD + 2) + HD + 1);
                    if (l > 0.0f) {
                        const float w = expf(m - M);
                        Lsum = fmaf(l, w, Lsum);
                        acc = fmaf(__ldcg(base + (size_t)s * (HD + 2) + d), w, acc);
                    }
                }
                op.d_attn_out[(size_t)(kvh * G + g) * HD + d] = acc / Lsum;
            }
            if (tid == 0) p.d_attn_tickets[kvh] = 0u;
            __threadfence();
        }
        named_barrier(11, ATT_T);               // smem is reused by the next item
    }
}

// WIDE: the plan contains rows so long that a thread owns two slices (more registers); kept out of the
// common instantiation so that it does not cost the narrow steps their registers.
template <int WT, bool WIDE>
__global__ void __launch_bounds__(TK_THREADS, 1)
decode_token_kernel(const __grid_constant__ b200_token_args p)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ b200_op s_op;
    const Smem sm = carve(smem_raw);
    const int tid = threadIdx.x;

    if (tid == 0) {
        for (int i = 0; i < TK_SLOTS; ++i) { mbar_init(&sm.full[i], 1); mbar_init(&sm.empty[i], 1); }
        sm.flags[0] = 0; sm.flags[1] = 0; sm.flags[2] = 0; sm.flags[3] = 0;
        for (int i = 0; i < TK_SLOTS; ++i) sm.cnt[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ---------------- producer warp: runs ahead through the whole step list ----------------
    if (tid >= TK_CONSUMERS) {
        if (tid == TK_CONSUMERS) {
            int fills[TK_SLOTS];
            for (int i = 0; i < TK_SLOTS; ++i) fills[i] = 0;
            bool dead = false;
            for (int oi = 0; oi < p.n_ops && !dead; ++oi) {
                const b200_op &op = p.d_ops[oi];
                if (op.type != B200_OP_MATVEC) continue;
                const int rb = op.rb, NG = op.NG, spg = TK_SLOTS / NG;
                const RowSplit br = block_rows(op);
                // per-group row ranges once per step: the issue loop below must stay a handful of instructions per copy
                int g0[TK_SLOTS], g1[TK_SLOTS], maxk = 0;
                for (int g = 0; g < NG; ++g) {
                    const RowSplit gr = group_rows(op, br, g);
                    g0[g] = gr.r0; g1[g] = gr.r1;
                    maxk = max(maxk, (gr.r1 - gr.r0 + rb - 1) / rb);
                }
                const unsigned char *wbase = static_cast<const unsigned char *>(op.d_w);
                const unsigned stride = (unsigned)op.row_stride;
                for (int k = 0; k < maxk && !dead; ++k) {
                    for (int g = 0; g < NG; ++g) {
                        const int row0 = g0[g] + k * rb;
                        if (row0 >= g1[g]) continue;
                        const int slot = g * spg + (k % spg);
                        if (fills[slot] > 0 && !mbar_wait_or_abort(&sm.empty[slot], (unsigned)(fills[slot] - 1) & 1u, sm.flags)) {
                            sm.flags[0] = 1; if (p.d_err) *p.d_err = 2; dead = true; break;
                        }
                        if (*(volatile int *)sm.flags) { dead = true; break; }
                        const unsigned bytes = (unsigned)min(rb, g1[g] - row0) * stride;
                        mbar_expect_tx(&sm.full[slot], bytes);
                        bulk_load(sm.ring + (size_t)slot * TK_SLOT_BYTES, wbase + (size_t)row0 * stride, bytes, &sm.full[slot]);
                        ++fills[slot];
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int pos = *p.d_pos;
    const unsigned ep = *p.d_epoch;
    unsigned fill_parity = 0, arrivals = 0;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    volatile int *abort_flag = sm.flags;

    for (int oi = 0; oi <= p.n_ops; ++oi) {
        if (oi > 0) {
            // everything the previous step wrote must be visible device-wide (and to the peers) before anyone goes on
            arrivals += gridDim.x;
            if (!grid_barrier(p.d_grid_barrier, arrivals, tid, abort_flag)) { if (tid == 0 && p.d_err) *p.d_err = 4; break; }
            if (s_op.n_signal > 0 && blockIdx.x == 0 && tid == 0) {
                __threadfence_system();
                const unsigned val = ep * (unsigned)p.epoch_mul + (unsigned)s_op.signal_add;
                for (int q = 0; q < s_op.n_signal; ++q) st_release_sys(s_op.d_signal_flags[q] + s_op.signal_index, val);
            }
            named_barrier(1, TK_CONSUMERS);                 // s_op is about to be overwritten
        }
        if (oi == p.n_ops) break;
        if (tid == 0) sm.flags[2] = sm.flags[0];            // one thread decides for the block whether to go on
        if (tid < (int)(sizeof(b200_op) / 4))
            reinterpret_cast<uint32_t *>(&s_op)[tid] = reinterpret_cast<const uint32_t *>(p.d_ops + oi)[tid];
        named_barrier(1, TK_CONSUMERS);
        if (s_op.n_wait > 0) {
            if (tid < s_op.n_wait) {
                const unsigned want = ep * (unsigned)p.epoch_mul + (unsigned)s_op.wait_add;
                if (!wait_flag_ge(s_op.d_wait_flags + tid, want)) { *abort_flag = 1; if (p.d_err) *p.d_err = 1; }
            }
            named_barrier(1, TK_CONSUMERS);
        }
        if (sm.flags[2]) break;
        unsigned long long *trace = (p.d_step_ns && blockIdx.x == 0) ? p.d_step_ns + 4 * oi : nullptr;
        if (trace && tid == 0) trace[0] = global_ns();
        if (s_op.type == B200_OP_MATVEC) {
#define TK_MV(SPT_, RB_) matvec_step<WT, SPT_, RB_>(s_op, p, sm, tid, pos, fill_parity, best_v, best_i, trace)
            if (s_op.spt == 1) {
                switch (s_op.rb) {
                case 8: TK_MV(1, 8); break;
                case 4: TK_MV(1, 4); break;
                case 2: TK_MV(1, 2); break;
                default: TK_MV(1, 1); break;
                }
            } else if (WIDE) {
                if (s_op.rb == 2) TK_MV(2, 2); else TK_MV(2, 1);
            }
#undef TK_MV
            if (s_op.n_out > 1 || s_op.n_signal > 0) __threadfence_system(); else __threadfence();
        } else {
            if (p.hd == 128) attention_step<128, 4>(s_op, p, sm, tid, pos);
            else if (p.hd == 64) attention_step<64, 4>(s_op, p, sm, tid, pos);
            else attention_step<256, 4>(s_op, p, sm, tid, pos);
            __threadfence();
        }
        if (trace && tid == 0) trace[1] = global_ns();
        if (oi == p.n_ops - 1 && p.pick_token) {
            // this block's best row of the last step -> scratch, before the closing barrier
            const int T = s_op.T, g = tid / T, t = tid - g * T;
            if ((tid & 31) < 8) {
                const bool act = g < s_op.NG;
                sm.am_v[(tid >> 5) * 8 + (tid & 31)] = act ? best_v : -INFINITY;
                sm.am_i[(tid >> 5) * 8 + (tid & 31)] = act ? best_i : 0x7fffffff;
            }
            named_barrier(1, TK_CONSUMERS);
            if (tid == 0) {
                float bv = -INFINITY; int bi = 0x7fffffff;
                for (int k = 0; k < TK_MAX_WARPS * 8; ++k) if (better(sm.am_v[k], sm.am_i[k], bv, bi)) { bv = sm.am_v[k]; bi = sm.am_i[k]; }
                p.d_argmax_scratch[2 * blockIdx.x] = bv;
                reinterpret_cast<int *>(p.d_argmax_scratch)[2 * blockIdx.x + 1] = bi;
                __threadfence();
            }
        }
    }

    // ---------------- closing work of block 0, warp 0 ----------------
    if (blockIdx.x == 0 && tid < 32 && !sm.flags[2]) {
        const int lane = tid;
        int tok = 0;
        if (p.pick_token) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int b = lane; b < (int)gridDim.x; b += 32) {
                const float v = __ldcg(p.d_argmax_scratch + 2 * b);
                const int i = __ldcg(reinterpret_cast<const int *>(p.d_argmax_scratch) + 2 * b + 1);
                if (better(v, i, bv, bi)) { bv = v; bi = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi2 = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi2, bv, bi)) { bv = ov; bi = oi2; }
            }
            if (bi == 0x7fffffff) bi = 0;               // nothing compared greater (all NaN): index 0, as the reference's loop
            bi += (int)s_op.out_offset;
            if (p.n_ranks > 1) {
                // push (value, row) to every rank, raise the flag, then take the best of all ranks
                if (lane < p.n_ranks) { p.d_argmax_val[lane][0] = bv; p.d_argmax_idx[lane][0] = bi; }
                __threadfence_system();
                __syncwarp();
                const unsigned val = ep * (unsigned)p.epoch_mul + (unsigned)p.argmax_add;
                if (lane < p.n_ranks) st_release_sys(p.d_argmax_signal_flags[lane] + p.rank, val);
                bool ok = true;
                if (lane < p.n_ranks) ok = wait_flag_ge(p.d_argmax_wait_flags + lane, val);
                if (!ok && p.d_err) *p.d_err = 1;
                __syncwarp();
                float gv = -INFINITY; int gi = 0x7fffffff;
                for (int r = 0; r < p.n_ranks; ++r) {
                    const float v = __ldcv(p.d_rank_vals + r);
                    const int i = __ldcv(p.d_rank_idx + r);
                    if (better(v, i, gv, gi)) { gv = v; gi = i; }
                }
                if (gi == 0x7fffffff) gi = 0;
                bi = gi;
            }
            tok = bi;
        }
        if (lane == 0) {
            if (p.pick_token && pos + 1 >= *p.d_prompt_len) p.d_tokens[pos + 1] = tok;
            *p.d_pos = pos + 1;
            *p.d_epoch = ep + 1u;
        }
    }
    // the last block to get here re-arms the barrier counters for the next launch
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.d_grid_barrier + 1, 1u) == gridDim.x - 1) {
            p.d_grid_barrier[0] = 0u;
            p.d_grid_barrier[1] = 0u;
            __threadfence();
        }
    }
}

int g_tk_sm_count = 0;

} // namespace

extern "C" int b200_op_plan_matvec(b200_op *op, int wtype)
{
    if (!op || op->rows <= 0 || op->cols <= 0 || op->row_stride <= 0) return B200_E_BADARG;
    const int E = wtype == B200_WT_Q8 ? 16 : 8;
    const int nsl = (op->cols + E - 1) / E;
    int spt = nsl <= TK_CONSUMERS ? 1 : 2;
    int T = (((nsl + spt - 1) / spt) + 31) / 32 * 32;
    if (T > TK_CONSUMERS) return B200_E_TOOLARGE;
    int ng = TK_CONSUMERS / T;                               // power of two <= 8: slots are split evenly between groups
    int p2 = 1;
    while (p2 * 2 <= ng && p2 * 2 <= TK_SLOTS) p2 *= 2;
    const int ralign = op->out_mode == B200_OUT_GLU ? 2 : 1;
    int rb = spt == 1 ? 8 : 2;
    while (rb > 1 && (long long)rb * op->row_stride > TK_SLOT_BYTES) rb >>= 1;
    if ((long long)rb * op->row_stride > TK_SLOT_BYTES || rb < ralign) return B200_E_TOOLARGE;
    op->spt = spt; op->T = T; op->NG = p2; op->rb = rb;
    return 0;
}

extern "C" int b200_decode_token(const b200_token_args *ap, void *stream)
{
    if (!ap || !ap->d_ops || ap->n_ops <= 0 || !ap->d_pos || !ap->d_tokens || !ap->d_prompt_len || !ap->d_epoch ||
        !ap->d_grid_barrier || !ap->d_emb || !ap->d_attn_scratch || !ap->d_attn_tickets || !ap->d_argmax_scratch)
        return B200_E_BADARG;
    if (ap->wtype != B200_WT_Q8 && ap->wtype != B200_WT_F16) return B200_E_BADARG;
    if (ap->n_kv <= 0 || ap->n_q != 4 * ap->n_kv || (ap->hd != 64 && ap->hd != 128 && ap->hd != 256) || ap->n_split <= 0 ||
        ap->n_ranks < 1 || ap->n_ranks > B200_MAX_PEERS)
        return B200_E_BADARG;
    const int chunk_cap = (ap->max_seq + ap->n_split - 1) / ap->n_split;
    const size_t att = ((size_t)4 * ap->hd + 2 * ap->hd + 16 + (size_t)4 * chunk_cap + (size_t)(ATT_T / 32) * 4 * ap->hd) * sizeof(float);
    if (att > TK_ATT_BYTES) return B200_E_TOOLARGE;
    if (!g_tk_sm_count) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_tk_sm_count = n;
    }
    void (*kern)(const b200_token_args) =
        ap->wtype == B200_WT_Q8 ? (ap->wide ? decode_token_kernel<B200_WT_Q8, true> : decode_token_kernel<B200_WT_Q8, false>)
                                : (ap->wide ? decode_token_kernel<B200_WT_F16, true> : decode_token_kernel<B200_WT_F16, false>);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TK_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g_tk_sm_count);
    cfg.blockDim = dim3(TK_THREADS);
    cfg.dynamicSmemBytes = TK_SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;          // all blocks resident at once: the in-kernel barriers need it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, kern, *ap);
}
