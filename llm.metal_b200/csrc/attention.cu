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

constexpr int ATT_THREADS = 256;

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
__global__ void __launch_bounds__(ATT_THREADS)
attn_decode_kernel(const __grid_constant__ b200_attn_args p, const int chunk_cap)
{
    constexpr int TPK = HD / 8;                 // threads that share one key row in the PV pass
    constexpr int KG = ATT_THREADS / TPK;       // key rows processed side by side
    constexpr int HALF = HD / 2;
    extern __shared__ __align__(16) float sm[];
    float *q_s = sm;                            // [G][HD]
    float *k_new = q_s + G * HD;                // [HD]
    float *v_new = k_new + HD;                  // [HD]
    float *ml = v_new + HD;                     // [2*G] running max, sum
    float *scores = ml + 2 * G;                 // [G][chunk_cap]
    float *ored = scores + (size_t)G * chunk_cap;  // [KG][G][HD]
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = ATT_THREADS / 32;
    const int split = blockIdx.x, kvh = blockIdx.y;

    pdl_launch_dependents();
    pdl_wait();

    const int pos = *p.d_pos;
    const int n = pos + 1;
    const int chunk = (n + p.n_split - 1) / p.n_split;
    const int j0 = min(split * chunk, n), j1 = min(j0 + chunk, n);
    const int len = j1 - j0;

    __half *kc = static_cast<__half *>(p.d_k_cache) + (size_t)kvh * p.max_seq * HD;
    __half *vc = static_cast<__half *>(p.d_v_cache) + (size_t)kvh * p.max_seq * HD;

    // ---- normalise + rotate the G query heads and the new key; fetch the new value ----
    for (int vi = warp; vi <= G; vi += nw) {
        const bool is_k = (vi == G);
        const float *src = is_k ? p.d_qkv + (size_t)p.n_q * HD + (size_t)kvh * HD
                                : p.d_qkv + (size_t)(kvh * G + vi) * HD;
        const float *gamma = is_k ? p.d_k_gamma : p.d_q_gamma;
        float a[HALF / 32 > 0 ? HALF / 32 : 1], b[HALF / 32 > 0 ? HALF / 32 : 1];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) {
            const int d = lane + 32 * j;
            a[j] = src[d]; b[j] = src[d + HALF];
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
            const float ang = (float)pos * p.d_inv_freq[d];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            const float r0 = a[j] * cs - b[j] * sn;
            const float r1 = a[j] * sn + b[j] * cs;
            if (is_k) {
                const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
                k_new[d] = __half2float(h0); k_new[d + HALF] = __half2float(h1);
                if (split == 0) { kc[(size_t)pos * HD + d] = h0; kc[(size_t)pos * HD + d + HALF] = h1; }
            } else {
                q_s[vi * HD + d] = r0; q_s[vi * HD + d + HALF] = r1;
            }
        }
        if (is_k) {
            const float *vsrc = p.d_qkv + (size_t)(p.n_q + p.n_kv) * HD + (size_t)kvh * HD;
            for (int d = lane; d < HD; d += 32) {
                const __half h = __float2half_rn(vsrc[d]);
                v_new[d] = __half2float(h);
                if (split == 0) vc[(size_t)pos * HD + d] = h;
            }
        }
    }
    __syncthreads();

    // ---- scores: one thread per key row ----
    const float scale = 1.0f / sqrtf((float)HD);
    for (int j = j0 + tid; j < j1; j += ATT_THREADS) {
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
                halves8_to_float(kr[c], kf);
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
    __syncthreads();

    // ---- per head: max, exponentials, sum ----
    for (int g = warp; g < G; g += nw) {
        float *sc = scores + (size_t)g * chunk_cap;
        float m = -INFINITY;
        for (int i = lane; i < len; i += 32) m = fmaxf(m, sc[i]);
        m = warp_max(m);
        float l = 0.0f;
        for (int i = lane; i < len; i += 32) { const float e = expf(sc[i] - m); sc[i] = e; l += e; }
        l = warp_sum(l);
        if (lane == 0) { ml[2 * g] = m; ml[2 * g + 1] = l; }
    }
    __syncthreads();

    // ---- unnormalised output: KG key rows side by side, 8 dims per thread ----
    {
        const int kg = tid / TPK, dl = tid % TPK;
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
        for (int j = j0 + kg; j < j1; j += KG) {
            float vf[8];
            if (j == pos) {
#pragma unroll
                for (int e = 0; e < 8; ++e) vf[e] = v_new[8 * dl + e];
            } else {
                halves8_to_float(reinterpret_cast<const uint4 *>(vc + (size_t)j * HD)[dl], vf);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pj = scores[(size_t)g * chunk_cap + (j - j0)];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj, vf[e], acc[g][e]);
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) ored[((size_t)kg * G + g) * HD + 8 * dl + e] = acc[g][e];
    }
    __syncthreads();
    // scratch: [n_q][n_split][HD + 2]
    for (int o = tid; o < G * HD; o += ATT_THREADS) {
        const int g = o / HD, d = o % HD;
        float v = 0.0f;
#pragma unroll 4
        for (int k = 0; k < KG; ++k) v += ored[((size_t)k * G + g) * HD + d];
        p.d_scratch[((size_t)(kvh * G + g) * p.n_split + split) * (HD + 2) + d] = v;
    }
    if (tid < 2 * G) {
        const int g = tid >> 1;
        p.d_scratch[((size_t)(kvh * G + g) * p.n_split + split) * (HD + 2) + HD + (tid & 1)] = ml[tid];
    }

    // ---- the last block of this KV head merges the splits ----
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.d_tickets + kvh, 1u) == (unsigned)p.n_split - 1u);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int o = tid; o < G * HD; o += ATT_THREADS) {
        const int g = o / HD, d = o % HD;
        const float *base = p.d_scratch + (size_t)(kvh * G + g) * p.n_split * (HD + 2);
        float M = -INFINITY;
        for (int s = 0; s < p.n_split; ++s) M = fmaxf(M, __ldcg(base + (size_t)s * (HD + 2) + HD));
        float L = 0.0f, acc = 0.0f;
        for (int s = 0; s < p.n_split; ++s) {
            const float m = __ldcg(base + (size_t)s * (HD + 2) + HD);
            const float l = __ldcg(base + (size_t)s * (HD + 2) + HD + 1);
            if (l > 0.0f) {
                const float w = expf(m - M);
                L = fmaf(l, w, L);
                acc = fmaf(__ldcg(base + (size_t)s * (HD + 2) + d), w, acc);
            }
        }
        p.d_out[(size_t)(kvh * G + g) * HD + d] = acc / L;
    }
    if (tid == 0) p.d_tickets[kvh] = 0u;
}

template <int HD, int G>
int launch_attn(const b200_attn_args &a, cudaStream_t st)
{
    const int chunk_cap = (a.max_seq + a.n_split - 1) / a.n_split;
    const int KG = ATT_THREADS / (HD / 8);
    const size_t smem = ((size_t)G * HD + 2 * HD + 2 * G + (size_t)G * chunk_cap + (size_t)KG * G * HD) * sizeof(float);
    auto kern = attn_decode_kernel<HD, G>;
    if (smem > 200 * 1024) return B200_E_TOOLARGE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_split, a.n_kv);
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
