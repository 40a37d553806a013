// Fused weight-streaming matrix-vector product for batch-1 decode (sm_100a).
//
// One block per SM slot owns a contiguous range of rows. A producer warp
// streams that range through a shared-memory ring with bulk asynchronous
// copies (TMA, cp.async.bulk + mbarrier): rows of a packed matrix are
// contiguous, so one copy instruction moves a whole stage (RB rows, 16-24 KB)
// and the ring keeps ~100 KB per block in flight without holding registers.
// Consumer threads own fixed 16-byte column slices (16 int8 quants or 8
// halves) of every row, so their slice of the input vector stays in registers
// for the whole kernel; consumer groups take stages round-robin, finish the RB
// rows of a stage with one transposing shuffle reduction per warp plus a
// fixed-order sum over the group's warps (reproducible run to run).
//
// Launched with programmatic dependent launch, a block of the NEXT kernel in
// the stream starts as soon as an SM has room for it (with the default 192 KB
// ring that is when a block of this kernel has left), fills its own ring with
// weights and only then waits for its input.
//
// The math is the reference's q8_matvec / f16_matvec
// (shaders/q8_kernels.metal:10-42, 97-127): fp32 activations, integer quants
// converted to fp32, fp32 multiply-accumulate, partial block sums scaled by
// the binary16 block scale. Input assembly and the epilogues fold in rms_norm
// (:133-157), residual_add (:369-375), silu_mul / gelu_mul (:337-363), the
// embedding copy (src/nn/fast_inference.c:386-392) and argmax (:469-476).
#include "stream_core.cuh"
#include "../../include/llmb200_kernels.h"

#include <stdlib.h>

unsigned long long g_b200_launches = 0;

extern "C" unsigned long long b200_launch_count(int reset)
{
    unsigned long long v = g_b200_launches;
    if (reset) g_b200_launches = 0;
    return v;
}

extern "C" void b200_launch_count_add(unsigned long long n) { g_b200_launches += n; }

namespace {

struct Geometry {
    int T;              // threads per consumer group (a multiple of 32)
    int NG;             // consumer groups
    int nstage;         // ring slots
    unsigned slot_bytes;  // bytes per slot (RB rows, rounded up to 128)
    int share_x;        // 1: group 0 assembles the input vector and hands it to the other groups through shared memory
};

// blockDim.x = NG*T consumers + 32 producer threads.
template <int WT, int SPT, int RB, int MAXT>
__global__ void __launch_bounds__(MAXT)
matvec_kernel(const __grid_constant__ b200_matvec_args p, const Geometry geo)
{
    constexpr int E = (WT == B200_WT_Q8) ? 16 : 8;       // elements per 16-byte slice
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int T = geo.T, NG = geo.NG, nstage = geo.nstage, nwg = T >> 5, nC = NG * T;
    unsigned char *ring = smem_raw;
    uint64_t *full = reinterpret_cast<uint64_t *>(ring + (size_t)nstage * geo.slot_bytes);
    uint64_t *empty = full + nstage;
    float *wpart = reinterpret_cast<float *>(empty + nstage);   // [NG][2][nwg][RB]
    float *red = wpart + (size_t)NG * 2 * nwg * RB;             // [NG][32]
    float *am_v = red + NG * 32;                                // [NG*RB]
    int *am_i = reinterpret_cast<int *>(am_v + NG * RB);        // [NG*RB]
    float *xs = reinterpret_cast<float *>(am_i + NG * RB);      // [SPT*T*E] when geo.share_x
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int ralign = (p.out_mode == B200_OUT_GLU) ? 2 : 1;
    const long long units = p.rows / ralign;
    const int r0 = (int)(units * blockIdx.x / gridDim.x) * ralign;
    const int r1 = (int)(units * (blockIdx.x + 1) / gridDim.x) * ralign;
    const int nst = (r1 - r0 + RB - 1) / RB;

    if (tid == 0) {
        for (int i = 0; i < nstage; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], T); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Every thread signals: the next kernel in the stream may be scheduled now and start
    // filling its own ring beside this block.
    pdl_launch_dependents();

    // ---------------- producer warp: weights depend on no earlier kernel ----------------
    if (tid >= nC) {
        if (tid == nC) {
            const unsigned char *wbase = static_cast<const unsigned char *>(p.d_w);
            for (int i = 0; i < nst; ++i) {
                const int slot = i % nstage;
                if (i >= nstage && !mbar_wait(&empty[slot], ((i / nstage) - 1) & 1)) {
                    if (p.d_err) *p.d_err = 2;
                    break;
                }
                const int row0 = r0 + i * RB;
                const int nr = min(RB, r1 - row0);
                const unsigned bytes = (unsigned)nr * (unsigned)p.row_stride;
                mbar_expect_tx(&full[slot], bytes);
                bulk_load(ring + (size_t)slot * geo.slot_bytes, wbase + (long long)row0 * p.row_stride, bytes, &full[slot]);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = tid / T, t = tid - g * T, lane = t & 31, wg = t >> 5;
    float *gred = red + g * 32;
    int col[SPT];
    bool on[SPT];
#pragma unroll
    for (int s = 0; s < SPT; ++s) { col[s] = (s * T + t) * E; on[s] = col[s] < p.cols; }

    // The norm weights are constants: their round trip is taken before the wait for the previous
    // kernel, not after it.
    float gm[SPT][E];
    const bool pre_gamma = p.d_norm_gamma && (!geo.share_x || g == 0);
    if (pre_gamma) {
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; e += 4) {
                float4 v4 = on[s] ? *reinterpret_cast<const float4 *>(p.d_norm_gamma + col[s] + e) : make_float4(0, 0, 0, 0);
                gm[s][e] = v4.x; gm[s][e + 1] = v4.y; gm[s][e + 2] = v4.z; gm[s][e + 3] = v4.w;
            }
    }

    pdl_wait();

    // Tensor parallel: every rank's partial vector must have landed in `slots`
    // (and, for the first kernel of a token, every rank must be done reading the
    // previous token's slots) before this block goes on.
    if (p.n_wait > 0) {
        if (tid < p.n_wait) {
            const unsigned want = (*p.d_epoch) * (unsigned)p.epoch_mul + (unsigned)p.epoch_add;
            if (!wait_flag_ge(p.d_wait_flags + tid, want, p.spin_limit > 0 ? p.spin_limit : B200_SPIN_LIMIT)) *p.d_err = 1;
        }
        named_barrier(1, nC);
    }

    // ---------------- input assembly ----------------
    // Every SM needs the whole input vector. When it has to be assembled (slot sums, norms), one group
    // per block does it and passes it on through shared memory: the few KB involved are read by all
    // SMs at once, and every extra reader of the same L2 lines queues behind the others.
    float x[SPT][E];
    if (!geo.share_x || g == 0) {
    if (p.in_mode == B200_IN_VEC) {
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; e += 4) {
                float4 v4 = on[s] ? *reinterpret_cast<const float4 *>(p.d_in_vec + col[s] + e) : make_float4(0, 0, 0, 0);
                x[s][e] = v4.x; x[s][e + 1] = v4.y; x[s][e + 2] = v4.z; x[s][e + 3] = v4.w;
            }
    } else {
        if (p.in_mode == B200_IN_EMBED) {
            long long tok = p.d_tokens[*p.d_pos];
            if (tok < 0 || tok >= p.emb_rows) tok = 0;      // never index outside the table
            const float *er = p.d_emb + tok * (long long)p.cols;
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
            for (int k = 0; k < p.n_slots; ++k) {
                const float *sl = p.d_slots + (long long)k * p.slot_stride;
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; e += 4) {
                        if (on[s]) {
                            // slots may be written by other GPUs: read them from L2, the point of coherence, never from L1
                            float4 v4 = __ldcg(reinterpret_cast<const float4 *>(sl + col[s] + e));
                            sacc[s][e] += v4.x; sacc[s][e + 1] += v4.y; sacc[s][e + 2] += v4.z; sacc[s][e + 3] += v4.w;
                        }
                    }
            }
            if (p.d_slot_norm_gamma) {
                float ss = 0.0f;
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; ++e) ss = fmaf(sacc[s][e], sacc[s][e], ss);
                ss = group_sum(ss, gred, 2 + g, T, t);
                const float inv = 1.0f / sqrtf(ss / (float)p.cols + p.eps);
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; ++e)
                        if (on[s]) sacc[s][e] = p.d_slot_norm_gamma[col[s] + e] * sacc[s][e] * inv;
            }
#pragma unroll
            for (int s = 0; s < SPT; ++s)
#pragma unroll
                for (int e = 0; e < E; e += 4) {
                    float4 v4 = on[s] ? *reinterpret_cast<const float4 *>(p.d_resid_in + col[s] + e) : make_float4(0, 0, 0, 0);
                    x[s][e] = v4.x + sacc[s][e]; x[s][e + 1] = v4.y + sacc[s][e + 1];
                    x[s][e + 2] = v4.z + sacc[s][e + 2]; x[s][e + 3] = v4.w + sacc[s][e + 3];
                }
        }
        if (blockIdx.x == 0 && g == 0 && p.d_resid_out) {
#pragma unroll
            for (int s = 0; s < SPT; ++s)
#pragma unroll
                for (int e = 0; e < E; e += 4)
                    if (on[s])
                        *reinterpret_cast<float4 *>(p.d_resid_out + col[s] + e) =
                            make_float4(x[s][e], x[s][e + 1], x[s][e + 2], x[s][e + 3]);
        }
    }
    if (p.d_norm_gamma) {
        float ss = 0.0f;
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; ++e) ss = fmaf(x[s][e], x[s][e], ss);
        ss = group_sum(ss, gred, 2 + g, T, t);
        const float inv = 1.0f / sqrtf(ss / (float)p.cols + p.eps);
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; ++e) x[s][e] = gm[s][e] * x[s][e] * inv;
    }
    }
    if (p.d_in_copy && blockIdx.x == 0 && g == 0) {
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; e += 4)
                if (on[s])
                    *reinterpret_cast<float4 *>(p.d_in_copy + col[s] + e) = make_float4(x[s][e], x[s][e + 1], x[s][e + 2], x[s][e + 3]);
    }
    if (geo.share_x) {
        if (g == 0) {
#pragma unroll
            for (int s = 0; s < SPT; ++s)
#pragma unroll
                for (int e = 0; e < E; e += 4)
                    *reinterpret_cast<float4 *>(xs + (size_t)(s * T + t) * E + e) = make_float4(x[s][e], x[s][e + 1], x[s][e + 2], x[s][e + 3]);
        }
        named_barrier(1, nC);
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

    // ---------------- consume the ring: group g takes stages g, g+NG, ... ----------------
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    // Byte offsets of this thread's slices inside a row. Threads past the end of the row read slice 0
    // (valid memory) against a zero input slice and drop the result.
    uint32_t qoff[SPT], soff[SPT];
#pragma unroll
    for (int s = 0; s < SPT; ++s) {
        const int c = on[s] ? col[s] : 0;
        qoff[s] = (uint32_t)(WT == B200_WT_Q8 ? c : 2 * c);
        soff[s] = (uint32_t)p.cols + (uint32_t)(c >> 5) * 2u;   // Q8: scales follow the quants of a row
    }
    const uint32_t ring_s = smem_u32(ring), stride = (uint32_t)p.row_stride;
    for (int i = g, it = 0; i < nst; i += NG, ++it) {
        const int slot = i % nstage;
        if (!mbar_wait(&full[slot], (i / nstage) & 1) && p.d_err) *p.d_err = 3;
        const uint32_t sb = ring_s + (uint32_t)slot * geo.slot_bytes;
        const int row0 = r0 + i * RB;
        const int nr = min(RB, r1 - row0);
        // Rows past nr hold stale bytes; they are computed like the others (no predicates in the
        // hot loop), stay in their own reduction lane and are never emitted.
        uint4 wq[RB][SPT];
        uint32_t ws[RB][SPT];
#pragma unroll
        for (int j = 0; j < RB; ++j)
#pragma unroll
            for (int s = 0; s < SPT; ++s) {
                wq[j][s] = lds_128(sb + (uint32_t)j * stride + qoff[s]);
                if (WT == B200_WT_Q8) ws[j][s] = lds_u16(sb + (uint32_t)j * stride + soff[s]);
            }
        float v[RB];
#pragma unroll
        for (int j = 0; j < RB; ++j) {
            float acc = 0.0f;
#pragma unroll
            for (int s = 0; s < SPT; ++s) {
                float d;
                if (WT == B200_WT_Q8) d = __half2float(__ushort_as_half((unsigned short)ws[j][s])) * dot16_q8(wq[j][s], x[s]);
                else d = dot8_f16(wq[j][s], x[s]);
                acc += d;                      // threads past the end of the row hold a zero input slice
            }
            v[j] = acc;
        }
        mbar_arrive(&empty[slot]);             // this thread no longer reads the slot

        const float tot = reduce_rows<RB>(v, lane);
        float *wp = wpart + (size_t)((g * 2 + (it & 1)) * nwg) * RB;
        if (lane < RB) wp[wg * RB + lane] = tot;
        named_barrier(2 + g, T);
        if (wg == 0) {
            float y = 0.0f;
            if (lane < RB)
                for (int w = 0; w < nwg; ++w) y += wp[w * RB + lane];
            const int row = row0 + lane;
            if (p.out_mode == B200_OUT_GLU) {
                const float u = __shfl_down_sync(0xffffffffu, y, 1);
                if (lane < nr && !(lane & 1)) {
                    const float a = p.act == 0 ? act_silu(y) : act_gelu_tanh(y);
                    p.d_out[0][p.out_offset + (row >> 1)] = a * u;
                }
            } else if (lane < nr) {
                for (int q = 0; q < p.n_out; ++q) p.d_out[q][p.out_offset + row] = y;
                if (better(y, row, best_v, best_i)) { best_v = y; best_i = row; }
            }
        }
    }

    if (!p.d_ticket) return;

    // ---------------- last-block bookkeeping ----------------
    if (p.d_argmax_scratch && wg == 0 && lane < RB) { am_v[g * RB + lane] = best_v; am_i[g * RB + lane] = best_i; }
    // The barrier orders every thread's stores (peers' slots included) before thread 0; its system-wide
    // fence is cumulative, so one fence per block publishes them all before the ticket is taken.
    named_barrier(1, nC);
    if (tid == 0) {
        __threadfence_system();
        if (p.d_argmax_scratch) {
            float bv = am_v[0]; int bi = am_i[0];
            for (int k = 1; k < NG * RB; ++k) if (better(am_v[k], am_i[k], bv, bi)) { bv = am_v[k]; bi = am_i[k]; }
            p.d_argmax_scratch[2 * blockIdx.x] = bv;
            reinterpret_cast<int *>(p.d_argmax_scratch)[2 * blockIdx.x + 1] = bi;
            __threadfence();
        }
        s_last = (atomicAdd(p.d_ticket, 1u) == gridDim.x - 1);
    }
    named_barrier(1, nC);
    if (!s_last || tid >= 32) return;
    __threadfence_system();
    {
        float bv = -INFINITY; int bi = 0x7fffffff;
        if (p.d_argmax_scratch) {
            for (int b = lane; b < (int)gridDim.x; b += 32) {
                const float v = *reinterpret_cast<volatile float *>(p.d_argmax_scratch + 2 * b);
                const int i = *reinterpret_cast<volatile int *>(p.d_argmax_scratch + 2 * b + 1);
                if (better(v, i, bv, bi)) { bv = v; bi = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (bi == 0x7fffffff) bi = 0;         // nothing compared greater (all NaN): index 0, as the reference's loop
            bi += (int)p.out_offset;              // global row index of a sharded matrix
            if (lane < p.n_argmax_out) { p.d_argmax_val[lane][0] = bv; p.d_argmax_idx[lane][0] = bi; }
        }
        __syncwarp();
        if (lane == 0) {
            const int pos = p.d_pos_rw ? *p.d_pos_rw : 0;
            if (p.d_next_token && pos + 1 >= *p.d_prompt_len) p.d_next_token[pos + 1] = bi;
            if (p.advance_pos) *p.d_pos_rw = pos + 1;
            const unsigned ep = p.d_epoch ? *p.d_epoch : 0u;
            if (p.advance_epoch) *p.d_epoch_rw = ep + 1u;
            *p.d_ticket = 0u;
            if (p.n_signal > 0) {
                __threadfence_system();
                const unsigned want = ep * (unsigned)p.epoch_mul + (unsigned)p.epoch_add;
                for (int q = 0; q < p.n_signal; ++q) st_release_sys(p.d_signal_flags[q] + p.signal_index, want);
            }
        }
    }
}

int g_sm_count = 0;
int sm_count()
{
    if (!g_sm_count) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sm_count = n;
    }
    return g_sm_count;
}

// Tuning knobs from the environment, read once per process: consumer threads per block and the ring
// budget in KB (defaults measured on Qwen3-4B shapes).
struct Knobs { int group_threads, ring_kb; };
const Knobs &knobs()
{
    static const Knobs k = [] {
        auto env_int = [](const char *name, int dflt) { const char *e = getenv(name); return e && *e ? atoi(e) : dflt; };
        Knobs v;
        v.group_threads = env_int("LLMB200_MV_GROUP_THREADS", 640);
        v.ring_kb = env_int("LLMB200_MV_RING_KB", 192);
        return v;
    }();
    return k;
}

template <int WT, int SPT, int RB, int MAXT>
int launch(const b200_matvec_args &a, const Geometry &geo, int grid, cudaStream_t st)
{
    const int nwg = geo.T / 32;
    const size_t smem = (size_t)geo.nstage * geo.slot_bytes + (size_t)geo.nstage * 16 +
                        ((size_t)geo.NG * 2 * nwg * RB + (size_t)geo.NG * 32 + (size_t)geo.NG * RB * 2) * sizeof(float) +
                        (geo.share_x ? (size_t)SPT * geo.T * (WT == B200_WT_Q8 ? 16 : 8) * sizeof(float) : 0);
    auto kern = matvec_kernel<WT, SPT, RB, MAXT>;
    if (smem > 220 * 1024) return B200_E_TOOLARGE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(geo.NG * geo.T + 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, kern, a, geo);
}

template <int WT, int SPT, int RB>
int launch_by_size(const b200_matvec_args &a, const Geometry &geo, int grid, cudaStream_t st)
{
    const int threads = geo.NG * geo.T + 32;
    if (threads <= 672) return launch<WT, SPT, RB, 672>(a, geo, grid, st);
    return launch<WT, SPT, RB, 1024>(a, geo, grid, st);
}

template <int WT, int SPT>
int launch_by_rows(const b200_matvec_args &a, const Geometry &geo, int rb, int grid, cudaStream_t st)
{
    switch (rb) {
    case 8: return launch_by_size<WT, SPT, 8>(a, geo, grid, st);
    case 4: return launch_by_size<WT, SPT, 4>(a, geo, grid, st);
    case 2: return launch_by_size<WT, SPT, 2>(a, geo, grid, st);
    default: return launch_by_size<WT, SPT, 1>(a, geo, grid, st);
    }
}

} // namespace

extern "C" int b200_matvec(const b200_matvec_args *ap, void *stream)
{
    if (!ap) return B200_E_BADARG;
    const b200_matvec_args &a = *ap;
    if (!a.d_w || a.rows <= 0 || a.cols <= 0 || (a.row_stride % 16) || ((uintptr_t)a.d_w % 16)) return B200_E_BADARG;
    if (a.wtype != B200_WT_Q8 && a.wtype != B200_WT_F16) return B200_E_BADARG;
    if (a.wtype == B200_WT_Q8 ? (a.cols % 32) : (a.cols % 8)) return B200_E_BADARG;
    if (a.row_stride < (long long)b200_packed_row_stride(a.wtype, a.cols)) return B200_E_BADARG;
    if (a.in_mode == B200_IN_VEC ? !a.d_in_vec
        : a.in_mode == B200_IN_RESID ? (!a.d_resid_in || a.n_slots < 0 || (a.n_slots > 0 && !a.d_slots))
        : a.in_mode == B200_IN_EMBED ? (!a.d_emb || !a.d_tokens || !a.d_pos || a.emb_rows <= 0) : true)
        return B200_E_BADARG;
    if (a.out_mode == B200_OUT_GLU ? (a.rows % 2 || !a.d_out[0]) : (a.out_mode != B200_OUT_STORE || a.n_out < 1 || a.n_out > B200_MAX_PEERS))
        return B200_E_BADARG;
    if (a.n_wait < 0 || a.n_wait > B200_MAX_PEERS || a.n_signal < 0 || a.n_signal > B200_MAX_PEERS ||
        a.n_argmax_out < 0 || a.n_argmax_out > B200_MAX_PEERS)
        return B200_E_BADARG;
    if ((a.n_wait > 0 || a.n_signal > 0) && (!a.d_epoch || !a.d_err)) return B200_E_BADARG;
    if ((a.n_signal > 0 || a.advance_pos || a.advance_epoch || a.d_next_token || a.d_argmax_scratch) && !a.d_ticket)
        return B200_E_BADARG;
    if ((a.advance_pos || a.d_next_token) && !a.d_pos_rw) return B200_E_BADARG;
    if (a.d_next_token && (!a.d_prompt_len || !a.d_argmax_scratch)) return B200_E_BADARG;
    if (a.advance_epoch && (!a.d_epoch || !a.d_epoch_rw)) return B200_E_BADARG;
    if (a.d_argmax_scratch && a.out_mode != B200_OUT_STORE) return B200_E_BADARG;

    const int E = a.wtype == B200_WT_Q8 ? 16 : 8;
    const int nsl = (a.cols + E - 1) / E;
    // Up to two slices per thread: keeps a group at <= 320 threads for rows of up to 640 slices, so that
    // two blocks (this kernel's and the next one's) fit on an SM; 960 consumers + the producer warp at most.
    // Measured on the 2560 x 9728 down projection: two slices per thread 12.3 us, one slice 16.3 us.
    const int spt = nsl <= 320 ? 1 : 2;
    if ((nsl + spt - 1) / spt > 960) return B200_E_TOOLARGE;
    Geometry geo;
    geo.T = (((nsl + spt - 1) / spt) + 31) / 32 * 32;
    const int ralign = a.out_mode == B200_OUT_GLU ? 2 : 1;
    const int units = a.rows / ralign;

    // rows per stage: 16-24 KB per bulk copy
    int rb = 8;
    while (rb > 1 && (long long)rb * a.row_stride > 24576) rb >>= 1;
    if (rb < ralign) rb = ralign;
    geo.slot_bytes = (unsigned)(((long long)rb * a.row_stride + 127) / 128 * 128);
    geo.NG = knobs().group_threads / geo.T;
    if (geo.NG > 8) geo.NG = 8;
    if (geo.NG < 1) geo.NG = 1;
    // Ring slots: a multiple of the group count, so that a slot is always consumed by the same group.
    // A group works through its stages in order, hence never waits on a slot whose previous phase is
    // still open -- mbarrier parity waits cannot tell phase k from phase k-2.
    const int ring_budget = knobs().ring_kb * 1024;
    while (geo.NG > 1 && (long long)geo.NG * geo.slot_bytes > ring_budget) --geo.NG;
    int per_group = ring_budget / (int)(geo.NG * geo.slot_bytes);
    if (per_group < 1) per_group = 1;
    while (per_group > 1 && per_group * geo.NG > 12) --per_group;
    geo.nstage = per_group * geo.NG;
    geo.share_x = geo.NG > 1 && (a.in_mode != B200_IN_VEC || a.d_norm_gamma) && (size_t)spt * geo.T * E * 4 <= 16384;

    int grid = a.grid;
    if (grid <= 0) grid = sm_count();                // one block per SM
    if (grid > units) grid = units;
    cudaStream_t st = (cudaStream_t)stream;
    if (a.wtype == B200_WT_Q8)
        return spt == 1 ? launch_by_rows<B200_WT_Q8, 1>(a, geo, rb, grid, st) : launch_by_rows<B200_WT_Q8, 2>(a, geo, rb, grid, st);
    return spt == 1 ? launch_by_rows<B200_WT_F16, 1>(a, geo, rb, grid, st) : launch_by_rows<B200_WT_F16, 2>(a, geo, rb, grid, st);
}
