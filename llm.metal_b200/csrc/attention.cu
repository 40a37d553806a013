// Decode attention for one new token over an F16 KV cache, split over the
// sequence (sm_100a).
//
// grid = (n_split, n_kv). A block serves the G = n_q/n_kv query heads that
// share one KV head, so every cached K/V row is read once per token instead of
// G times, and works on keys [s*chunk, (s+1)*chunk) of the 0..pos range. Each
// block first rebuilds, redundantly and identically, the normalised + rotated
// query heads and the new key/value row (per-head RMSNorm, half-split RoPE with
// angle = pos * inv_freq[d] in fp32); block 0 of a KV head stores that row to
// the cache in binary16. Partial results (running max, sum of exponentials,
// unnormalised output) go to scratch; the last block of a KV head to finish
// merges them.
//
// Math follows per_head_rms_norm, rope, kv_cache_store and attention in
// shaders/q8_kernels.metal:165-331: fp32 throughout, scores = (q.k)/sqrt(hd),
// softmax over keys 0..pos, out = sum p_j v_j. The only change of value is the
// cache precision (binary16 instead of fp32).
#include "common.cuh"
#include "../../include/llmb200_kernels.h"

#include <stdio.h>

extern unsigned long long g_b200_launches;

namespace {

constexpr int ATT_THREADS = 512;

__device__ __forceinline__ void halves8_to_float(const uint4 &u, float *f)
{
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}

// Thread layout: the block's threads are split into G head groups; a head group is KL key lanes of
// 8 threads (16 for head dimensions above 128); the threads of a key lane split the head dimension
// (DPT = 16 values each at head dimension 128 and 256). A key lane
// walks keys kl, kl+KL, ... of the block's slice with its own online softmax (running max, sum and
// output), so nothing is exchanged between threads while keys stream in; K and V rows are prefetched
// two keys ahead, the first ones before the query is even normalised. At the end the key lanes of a
// head are merged (shuffles inside a warp, shared memory across warps).
template <int HD, int G>
__global__ void __launch_bounds__(ATT_THREADS)
attn_decode_kernel(const __grid_constant__ b200_attn_args pa, const int chunk_cap)
{
    // batched form: blockIdx.z selects the sequence; its buffers are slices of the shared ones
    b200_attn_args p = pa;
    if (pa.n_items > 1) {
        const long long it = blockIdx.z;
        p.d_qkv = pa.d_qkv + it * pa.qkv_item_stride;
        p.d_k_cache = static_cast<__half *>(pa.d_k_cache) + it * pa.cache_item_stride;
        p.d_v_cache = static_cast<__half *>(pa.d_v_cache) + it * pa.cache_item_stride;
        p.d_out = pa.d_out + it * pa.out_item_stride;
        p.d_scratch = pa.d_scratch + it * (long long)pa.n_q * pa.n_split * (HD + 2);
        p.d_tickets = pa.d_tickets + it * pa.n_kv;
    }
    constexpr int DLN = HD > 128 ? 16 : 8;      // threads that share one key (a key lane)
    constexpr int DPT = HD / DLN;               // head-dim values per thread (at most 16: no register spills)
    constexpr int NV = DPT / 8;                 // 16-byte loads per K (and per V) row per thread
    constexpr int TPH = ATT_THREADS / G;        // threads per head group
    constexpr int KL = TPH / DLN;               // key lanes per head
    constexpr int WPH = TPH / 32;               // warps per head
    constexpr int HALF = HD / 2;
    constexpr int PF = 2;                       // keys in flight per key lane
    extern __shared__ __align__(16) float sm[];
    float *q_s = sm;                            // [G][HD]
    float *k_new = q_s + G * HD;                // [HD]
    float *v_new = k_new + HD;                  // [HD]
    float *mrg = v_new + HD;                    // [G][WPH][HD + 2] merge buffer across warps
    __shared__ int s_last;
    (void)chunk_cap;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = ATT_THREADS / 32;
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int g = tid / TPH, r = tid - g * TPH, kl = r / DLN, dl = r % DLN;

    pdl_launch_dependents();
    // Norm weights and rotation frequencies are constants: fetch them before waiting for the kernel
    // that produces q/k/v, so that their round trip is not part of the dependent chain.
    float gq_a[HALF / 32], gq_b[HALF / 32], gk_a[HALF / 32], gk_b[HALF / 32], fr[HALF / 32];
#pragma unroll
    for (int j = 0; j < HALF / 32; ++j) {
        const int d = lane + 32 * j;
        gq_a[j] = p.d_q_gamma ? p.d_q_gamma[d] : 1.0f; gq_b[j] = p.d_q_gamma ? p.d_q_gamma[d + HALF] : 1.0f;
        gk_a[j] = p.d_k_gamma ? p.d_k_gamma[d] : 1.0f; gk_b[j] = p.d_k_gamma ? p.d_k_gamma[d + HALF] : 1.0f;
        fr[j] = p.d_inv_freq[d];
    }
    pdl_wait();

    // The new q/k/v rows do not depend on the position: their loads go out before the position is read,
    // so that the two round trips overlap. Warp vi < G takes query head vi, warp G the new key and value.
    static_assert(ATT_THREADS / 32 > G, "one warp per new row");
    const bool row_k = (warp == G);
    float ra[HALF / 32], rb[HALF / 32], rv[HD / 32];
    if (warp <= G) {
        const float *src = row_k ? p.d_qkv + (size_t)p.n_q * HD + (size_t)kvh * HD
                                 : p.d_qkv + (size_t)(kvh * G + warp) * HD;
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) { ra[j] = src[lane + 32 * j]; rb[j] = src[lane + 32 * j + HALF]; }
        if (row_k) {
            const float *vsrc = p.d_qkv + (size_t)(p.n_q + p.n_kv) * HD + (size_t)kvh * HD;
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) rv[j] = vsrc[lane + 32 * j];
        }
    }

    const int pos = *p.d_pos;
    // A position outside the cache writes and reads nothing: the block leaves (all its threads take the
    // same branch) and the output keeps its previous contents. The engine checks positions on the host.
    if (pos < 0 || pos >= p.max_seq) return;
    const int n = pos + 1;
    const int chunk = (n + p.n_split - 1) / p.n_split;
    const int j0 = min(split * chunk, n), j1 = min(j0 + chunk, n);

    __half *kc = static_cast<__half *>(p.d_k_cache) + (size_t)kvh * p.max_seq * HD;
    __half *vc = static_cast<__half *>(p.d_v_cache) + (size_t)kvh * p.max_seq * HD;

    // ---- start the first K/V rows of this key lane on their way ----
    static_assert(PF == 2, "the key loop below is unrolled for two slots");
    uint4 kq0[NV], vq0[NV], kq1[NV], vq1[NV];
    auto fetch = [&](uint4 (&kq)[NV], uint4 (&vq)[NV], int j) {
        if (j < j1 && j != pos) {
            const uint4 *kr = reinterpret_cast<const uint4 *>(kc + (size_t)j * HD + dl * DPT);
            const uint4 *vr = reinterpret_cast<const uint4 *>(vc + (size_t)j * HD + dl * DPT);
#pragma unroll
            for (int i = 0; i < NV; ++i) { kq[i] = kr[i]; vq[i] = vr[i]; }
        }
    };
    fetch(kq0, vq0, j0 + kl);
    fetch(kq1, vq1, j0 + kl + KL);

    // ---- normalise + rotate the G query heads and the new key; fetch the new value ----
    if (warp <= G) {
        const int vi = warp;
        const bool is_k = row_k;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) { ss = fmaf(ra[j], ra[j], ss); ss = fmaf(rb[j], rb[j], ss); }
        ss = warp_sum(ss);
        if (is_k ? p.d_k_gamma != nullptr : p.d_q_gamma != nullptr) {
            const float inv = 1.0f / sqrtf(ss / (float)HD + p.eps);
#pragma unroll
            for (int j = 0; j < HALF / 32; ++j) {
                ra[j] = (is_k ? gk_a[j] : gq_a[j]) * ra[j] * inv; rb[j] = (is_k ? gk_b[j] : gq_b[j]) * rb[j] * inv;
            }
        }
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) {
            const int d = lane + 32 * j;
            float sn, cs;
            sincosf((float)pos * fr[j], &sn, &cs);
            const float r0 = ra[j] * cs - rb[j] * sn;
            const float r1 = ra[j] * sn + rb[j] * cs;
            if (is_k) {
                const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
                k_new[d] = __half2float(h0); k_new[d + HALF] = __half2float(h1);
                if (split == 0) { kc[(size_t)pos * HD + d] = h0; kc[(size_t)pos * HD + d + HALF] = h1; }
            } else {
                q_s[vi * HD + d] = r0; q_s[vi * HD + d + HALF] = r1;
            }
        }
        if (is_k) {
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) {
                const int d = lane + 32 * j;
                const __half h = __float2half_rn(rv[j]);
                v_new[d] = __half2float(h);
                if (split == 0) vc[(size_t)pos * HD + d] = h;
            }
        }
    }
    __syncthreads();

    // ---- stream the keys of this lane: online softmax in registers ----
    float q[DPT], acc[DPT];
#pragma unroll
    for (int e = 0; e < DPT; ++e) { q[e] = q_s[g * HD + dl * DPT + e]; acc[e] = 0.0f; }
    const float scale = 1.0f / sqrtf((float)HD);
    float m = -INFINITY, l = 0.0f;
    auto one_key = [&](uint4 (&kq)[NV], uint4 (&vq)[NV], int j) {
        const bool valid = j < j1;              // every lane of the warp runs the shuffles; only valid keys count
        float kf[DPT], vf[DPT];
        if (!valid) {
#pragma unroll
            for (int e = 0; e < DPT; ++e) { kf[e] = 0.0f; vf[e] = 0.0f; }
        } else if (j == pos) {
#pragma unroll
            for (int e = 0; e < DPT; ++e) { kf[e] = k_new[dl * DPT + e]; vf[e] = v_new[dl * DPT + e]; }
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                halves8_to_float(kq[i], kf + 8 * i);
                halves8_to_float(vq[i], vf + 8 * i);
            }
        }
        fetch(kq, vq, j + PF * KL);             // refill these registers with the key two rounds ahead
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < DPT; ++e) s = fmaf(q[e], kf[e], s);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (DLN == 16) s += __shfl_xor_sync(0xffffffffu, s, 8);
        s *= scale;
        if (valid) {
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn), pj = expf(s - mn);
            l = fmaf(l, corr, pj);
#pragma unroll
            for (int e = 0; e < DPT; ++e) acc[e] = fmaf(acc[e], corr, pj * vf[e]);
            m = mn;
        }
    };
    // same trip count for every key lane of the block, so that the warp-wide shuffles stay convergent
    const int rounds = (j1 - j0 + PF * KL - 1) / (PF * KL);
    for (int it = 0, j = j0 + kl; it < rounds; ++it, j += PF * KL) {
        one_key(kq0, vq0, j);
        one_key(kq1, vq1, j + KL);
    }

    // ---- merge the key lanes of a head: inside the warp, then across the head's warps ----
#pragma unroll
    for (int o = DLN; o < 32; o <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo = __shfl_xor_sync(0xffffffffu, l, o);
        const float mn = fmaxf(m, mo);
        const float ca = (m == -INFINITY) ? 0.0f : expf(m - mn), cb = (mo == -INFINITY) ? 0.0f : expf(mo - mn);
        l = l * ca + lo * cb;
#pragma unroll
        for (int e = 0; e < DPT; ++e) acc[e] = acc[e] * ca + __shfl_xor_sync(0xffffffffu, acc[e], o) * cb;
        m = mn;
    }
    const int wh = r >> 5;                      // warp index inside the head group
    if ((r & 31) < DLN) {                       // key lane 0 of each warp holds the warp's state
        float *dst = mrg + ((size_t)g * WPH + wh) * (HD + 2);
#pragma unroll
        for (int e = 0; e < DPT; ++e) dst[dl * DPT + e] = acc[e];
        if (dl == 0) { dst[HD] = m; dst[HD + 1] = l; }
    }
    __syncthreads();
    // scratch: [n_q][n_split][HD + 2] = unnormalised output, running max, sum
    for (int o = tid; o < G * (HD + 2); o += ATT_THREADS) {
        const int gg = o / (HD + 2), d = o - gg * (HD + 2);
        const float *src = mrg + (size_t)gg * WPH * (HD + 2);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WPH; ++w) M = fmaxf(M, src[w * (HD + 2) + HD]);
        float v = 0.0f;
        if (d == HD) v = M;
        else {
#pragma unroll
            for (int w = 0; w < WPH; ++w) {
                const float mw = src[w * (HD + 2) + HD];
                const float c = (mw == -INFINITY) ? 0.0f : expf(mw - M);
                v = fmaf(src[w * (HD + 2) + (d == HD + 1 ? HD + 1 : d)], c, v);
            }
        }
        p.d_scratch[((size_t)(kvh * G + gg) * p.n_split + split) * (HD + 2) + d] = v;
    }

    // ---- the last block of this KV head merges the splits ----
    // The barrier orders every thread's partials before thread 0; its fence (cumulative) then makes
    // them visible device-wide before the ticket is taken.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(p.d_tickets + kvh, 1u) == (unsigned)p.n_split - 1u);
        __threadfence();
    }
    __syncthreads();
    if (!s_last) return;
    // Every output element folds the splits with its own running (max, sum, value): the three loads of
    // a split depend on nothing, so the unrolled loop keeps a batch of them in flight and the whole merge
    // costs two round trips to L2 instead of one pass for the weights and another for the values.
    constexpr int NO = (G * HD + ATT_THREADS - 1) / ATT_THREADS;    // outputs per thread, folded side by side
    constexpr int UN = NO > 1 ? 9 : 18;
    const float *base[NO];
    int od[NO];
    float M[NO], L[NO], O[NO];
#pragma unroll
    for (int k = 0; k < NO; ++k) {
        const int o = min(tid + k * ATT_THREADS, G * HD - 1);      // surplus threads repeat the last output
        const int gg = o / HD;
        od[k] = o % HD;
        base[k] = p.d_scratch + (size_t)(kvh * G + gg) * p.n_split * (HD + 2);
        M[k] = -INFINITY; L[k] = 0.0f; O[k] = 0.0f;
    }
    // Batches of UN splits, all loads of a batch issued before the first use; a short last batch repeats
    // the final split's addresses (valid memory) and drops the values.
    if (p.n_split == UN) {
        // the usual split count (one split per SM at 8 KV heads): no clamping, no predicates
#pragma unroll
        for (int s = 0; s < UN; ++s) {
#pragma unroll
            for (int k = 0; k < NO; ++k) {
                const float *rec = base[k] + (size_t)s * (HD + 2);
                const float ms = __ldcg(rec + HD), ls = __ldcg(rec + HD + 1), as = __ldcg(rec + od[k]);
                const float Mn = fmaxf(M[k], ms);
                const float c0 = (M[k] == -INFINITY) ? 0.0f : expf(M[k] - Mn);
                const float c1 = ls > 0.0f ? expf(ms - Mn) : 0.0f;
                L[k] = fmaf(L[k], c0, ls * c1);
                O[k] = fmaf(O[k], c0, as * c1);
                M[k] = Mn;
            }
        }
    } else
    for (int s0 = 0; s0 < p.n_split; s0 += UN) {
        float2 ml[UN][NO];
        float av[UN][NO];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int sc = min(s0 + u, p.n_split - 1);
#pragma unroll
            for (int k = 0; k < NO; ++k) {
                const float *rec = base[k] + (size_t)sc * (HD + 2);
                ml[u][k] = __ldcg(reinterpret_cast<const float2 *>(rec + HD));
                av[u][k] = __ldcg(rec + od[k]);
            }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const bool valid = s0 + u < p.n_split;
#pragma unroll
            for (int k = 0; k < NO; ++k) {
                const float ms = ml[u][k].x, ls = valid ? ml[u][k].y : 0.0f;
                const float Mn = ls > 0.0f ? fmaxf(M[k], ms) : M[k];
                const float c0 = (M[k] == -INFINITY) ? 0.0f : expf(M[k] - Mn);
                const float c1 = ls > 0.0f ? expf(ms - Mn) : 0.0f;
                L[k] = fmaf(L[k], c0, ls * c1);
                O[k] = fmaf(O[k], c0, av[u][k] * c1);
                M[k] = Mn;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NO; ++k) {
        const int o = tid + k * ATT_THREADS;
        if (o < G * HD) p.d_out[(size_t)(kvh * G) * HD + o] = O[k] / L[k];
    }
    if (tid == 0) p.d_tickets[kvh] = 0u;
}

template <int HD, int G>
int launch_attn(const b200_attn_args &a, cudaStream_t st)
{
    const int chunk_cap = (a.max_seq + a.n_split - 1) / a.n_split;
    const int WPH = ATT_THREADS / G / 32;
    size_t mrg_floats = (size_t)G * WPH * (HD + 2);
    if (mrg_floats < (size_t)2 * G * a.n_split) mrg_floats = (size_t)2 * G * a.n_split;
    const size_t smem = ((size_t)G * HD + 2 * HD + mrg_floats) * sizeof(float);
    auto kern = attn_decode_kernel<HD, G>;
    if (smem > 200 * 1024) return B200_E_TOOLARGE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_split, a.n_kv, a.n_items > 1 ? a.n_items : 1);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, kern, a, chunk_cap);
}

} // namespace

extern "C" size_t b200_attn_scratch_floats(int n_q, int hd, int n_split)
{
    if (n_q <= 0 || hd <= 0 || n_split <= 0) return 0;
    return (size_t)n_q * n_split * (hd + 2);
}

extern "C" int b200_attn_decode(const b200_attn_args *ap, void *stream)
{
    if (!ap) return B200_E_BADARG;
    const b200_attn_args &a = *ap;
    if (!a.d_qkv || !a.d_inv_freq || !a.d_k_cache || !a.d_v_cache || !a.d_out || !a.d_scratch || !a.d_tickets || !a.d_pos)
        return B200_E_BADARG;
    if (a.n_q <= 0 || a.n_kv <= 0 || a.n_q % a.n_kv || a.max_seq <= 0 || a.n_split <= 0 || a.n_split > 1024)
        return B200_E_BADARG;
    if (((uintptr_t)a.d_k_cache % 16) || ((uintptr_t)a.d_v_cache % 16)) return B200_E_BADARG;
    if ((uintptr_t)a.d_scratch % 8) return B200_E_BADARG;       // (max, sum) pairs are read as one 8-byte load
    const int G = a.n_q / a.n_kv;
    cudaStream_t st = (cudaStream_t)stream;
#define B200_ATT(HD_, G_) if (a.hd == HD_ && G == G_) return launch_attn<HD_, G_>(a, st)
    B200_ATT(64, 1);  B200_ATT(64, 2);  B200_ATT(64, 4);  B200_ATT(64, 8);
    B200_ATT(128, 1); B200_ATT(128, 2); B200_ATT(128, 4); B200_ATT(128, 8);
    B200_ATT(256, 1); B200_ATT(256, 2); B200_ATT(256, 4); B200_ATT(256, 8);
#undef B200_ATT
    return B200_E_BADARG;   // unsupported head_dim / group size
}

// ---------------------------------------------------------------------------
// Tensor-parallel greedy pick: every rank has pushed (best value, global row)
// of its vocabulary shard into vals[r] / idx[r]; take the largest, lowest row
// on ties, exactly what one argmax over the whole vocabulary returns.
// ---------------------------------------------------------------------------
__global__ void tp_argmax_finalize_kernel(const float *vals, const int *idx, int n_ranks,
                                          const unsigned *wait_flags, const unsigned *epoch,
                                          int epoch_mul, int epoch_add,
                                          int *tokens, int *pos_rw, const int *prompt_len,
                                          unsigned *epoch_rw, int *err)
{
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0) return;
    const unsigned ep = *epoch;
    const unsigned want = ep * (unsigned)epoch_mul + (unsigned)epoch_add;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int r = 0; r < n_ranks; ++r) {
        if (!wait_flag_ge(wait_flags + r, want)) *err = 1;
        const float v = __ldcv(vals + r);
        const int i = __ldcv(idx + r);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    if (bi == 0x7fffffff) bi = 0;
    const int pos = *pos_rw;
    if (pos + 1 >= *prompt_len) tokens[pos + 1] = bi;
    *pos_rw = pos + 1;
    *epoch_rw = ep + 1u;
}

extern "C" int b200_tp_argmax_finalize(const float *d_vals, const int *d_idx, int n_ranks,
                                       const unsigned *d_wait_flags, const unsigned *d_epoch,
                                       int epoch_mul, int epoch_add,
                                       int *d_tokens, int *d_pos, const int *d_prompt_len,
                                       unsigned *d_epoch_rw, int *d_err, int use_pdl, void *stream)
{
    if (!d_vals || !d_idx || n_ranks < 1 || n_ranks > B200_MAX_PEERS || !d_wait_flags || !d_epoch ||
        !d_tokens || !d_pos || !d_prompt_len || !d_epoch_rw || !d_err)
        return B200_E_BADARG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, tp_argmax_finalize_kernel, d_vals, d_idx, n_ranks, d_wait_flags, d_epoch,
                                   epoch_mul, epoch_add, d_tokens, d_pos, d_prompt_len, d_epoch_rw, d_err);
}

// ---------------------------------------------------------------------------
// b200_attn_decode_static: the same attention launch for callers that can
// neither allocate device memory themselves nor let a library do it for them
// -- for instance a serving process whose device memory was handed out in full
// at start-up, or a latency-critical loop in which a cudaMalloc (which may
// synchronise the whole device) is not acceptable. The split-sequence partials
// and the per-KV-head tickets, which b200_attn_decode takes from the caller,
// live here in two arrays that are part of the library image. They exist once
// per GPU that loads the library and stay there until the process exits.
//
// In host code the names of these arrays are only stand-ins; the kernel needs
// their device addresses, which cudaGetSymbolAddress returns for the device
// that is current at the time. That look-up happens on the first call on each
// device, so that first call should be made before any stream capture.
// ---------------------------------------------------------------------------
static __device__ __align__(256) float g_attn_static_scratch[B200_ATTN_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned g_attn_static_tickets[B200_ATTN_STATIC_MAX_KV_HEADS];

namespace {
constexpr int kMaxDevices = 64;
float *g_static_scratch_addr[kMaxDevices];
unsigned *g_static_tickets_addr[kMaxDevices];
bool g_static_ready[kMaxDevices];
}

extern "C" int b200_attn_decode_static(const b200_attn_args *ap, void *stream)
{
    if (!ap) return B200_E_BADARG;
    const size_t need = b200_attn_scratch_floats(ap->n_q, ap->hd, ap->n_split);
    if (need == 0 || ap->n_kv <= 0) return B200_E_BADARG;
    if (ap->n_items > 1) {
        // the batched form indexes scratch and tickets by item: the built-in arrays hold one item
        fprintf(stderr, "[llmb200] b200_attn_decode_static: one sequence per call (n_items = %d); use b200_attn_decode with "
                        "caller-provided scratch for the batched form\n", ap->n_items);
        return B200_E_TOOLARGE;
    }
    if (need > (size_t)B200_ATTN_STATIC_SCRATCH_FLOATS || ap->n_kv > B200_ATTN_STATIC_MAX_KV_HEADS) {
        fprintf(stderr, "[llmb200] b200_attn_decode_static: n_q*n_split*(hd+2) = %zu floats / %d KV heads exceed the built-in "
                        "scratch (%d floats, %d KV heads); use b200_attn_decode with caller-provided scratch\n",
                need, ap->n_kv, B200_ATTN_STATIC_SCRATCH_FLOATS, B200_ATTN_STATIC_MAX_KV_HEADS);
        return B200_E_TOOLARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return B200_E_BADARG;
    if (!g_static_ready[dev]) {
        // once per device, with that device current: host-side symbol -> device address
        void *ps = nullptr, *pt = nullptr;
        e = cudaGetSymbolAddress(&ps, g_attn_static_scratch);
        if (e != cudaSuccess) return (int)e;
        e = cudaGetSymbolAddress(&pt, g_attn_static_tickets);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_addr[dev] = static_cast<float *>(ps);
        g_static_tickets_addr[dev] = static_cast<unsigned *>(pt);
        g_static_ready[dev] = true;
    }
    // The arrays keep whatever the last call left. The partials are fully rewritten by every launch;
    // the tickets must start at zero, so they are cleared on the caller's stream first.
    e = cudaMemsetAsync(g_static_tickets_addr[dev], 0, sizeof(unsigned) * (size_t)ap->n_kv, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    b200_attn_args a = *ap;
    a.d_scratch = g_static_scratch_addr[dev];
    a.d_tickets = g_static_tickets_addr[dev];
    return b200_attn_decode(&a, stream);
}
