// Fused weight-streaming matrix-vector product for batch-1 decode (sm_100a).
//
// Work split: a block owns a contiguous range of rows; its threads own fixed
// 16-byte column slices (16 int8 quants or 8 halves) of every row. The input
// vector slice of a thread therefore lives in registers for the whole kernel,
// a warp reads 512 contiguous bytes of a row per load instruction, and a row's
// dot product is completed by one pass over per-thread partials kept in shared
// memory (fixed summation order, so results are reproducible run to run).
// Grids are sized to a multiple of the SM count with all blocks resident.
//
// The math is the reference's q8_matvec / f16_matvec
// (shaders/q8_kernels.metal:10-42, 97-127): fp32 activations, integer quants
// converted to fp32, fp32 multiply-accumulate, block sum scaled by the
// binary16 block scale. Input assembly and the epilogues fold in rms_norm
// (:133-157), residual_add (:369-375), silu_mul / gelu_mul (:337-363), the
// embedding copy (src/nn/fast_inference.c:386-392) and argmax (:469-476).
#include "common.cuh"
#include "../../include/llmb200_kernels.h"

unsigned long long g_b200_launches = 0;

extern "C" unsigned long long b200_launch_count(int reset)
{
    unsigned long long v = g_b200_launches;
    if (reset) g_b200_launches = 0;
    return v;
}

namespace {

// int8 -> fp32 through the 2^23 trick: byte b (biased by 128) is dropped into
// the low mantissa byte of 0x4B000000 (= 8388608.0f); subtracting 8388736.0f
// leaves the signed value exactly. One PRMT + one FADD per element.
__device__ __forceinline__ float q8_to_f32(uint32_t biased_word, int k)
{
    return __uint_as_float(__byte_perm(biased_word, 0x4B000000u, 0x7650u + k)) - 8388736.0f;
}

__device__ __forceinline__ float dot16_q8(const uint4 &w, const float *x)
{
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s0 = fmaf(q8_to_f32(u[i], 0), x[4 * i + 0], s0);
        s1 = fmaf(q8_to_f32(u[i], 1), x[4 * i + 1], s1);
        s2 = fmaf(q8_to_f32(u[i], 2), x[4 * i + 2], s2);
        s3 = fmaf(q8_to_f32(u[i], 3), x[4 * i + 3], s3);
    }
    return (s0 + s1) + (s2 + s3);
}

__device__ __forceinline__ float dot8_f16(const uint4 &w, const float *x)
{
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
        s0 = fmaf(f.x, x[2 * i + 0], s0);
        s1 = fmaf(f.y, x[2 * i + 1], s1);
    }
    return s0 + s1;
}

__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float act_gelu_tanh(float g)
{
    float inner = 0.7978845608f * (g + 0.044715f * g * g * g);
    inner = fminf(fmaxf(inner, -15.0f), 15.0f);
    return 0.5f * g * (1.0f + tanhf(inner));
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi)
{
    return v > bv || (v == bv && i < bi);
}

template <int WT, int SPT, int RB, int MAXT>
__global__ void __launch_bounds__(MAXT)
matvec_kernel(const __grid_constant__ b200_matvec_args p, const int rmax)
{
    constexpr int E = (WT == B200_WT_Q8) ? 16 : 8;       // elements per 16-byte slice
    extern __shared__ __align__(16) float smem[];
    const int T = blockDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = T >> 5;
    float *part = smem;                  // [rmax][T]
    float *red = smem + (size_t)rmax * T;  // 40 floats of reduction scratch, then argmax scratch
    __shared__ int s_last;

    const int ralign = (p.out_mode == B200_OUT_GLU) ? 2 : 1;
    const long long units = p.rows / ralign;
    const int r0 = (int)(units * blockIdx.x / gridDim.x) * ralign;
    const int r1 = (int)(units * (blockIdx.x + 1) / gridDim.x) * ralign;

    int col[SPT];
    bool on[SPT];
#pragma unroll
    for (int s = 0; s < SPT; ++s) { col[s] = (s * T + tid) * E; on[s] = col[s] < p.cols; }

    const uint8_t *wbase = static_cast<const uint8_t *>(p.d_w);
    const long long scale_off = (long long)p.cols;        // Q8: scales follow the quants of a row

    uint4 wq[RB][SPT];
    unsigned short ws[RB][SPT];
    auto load_batch = [&](int r, int rend) {
#pragma unroll
        for (int i = 0; i < RB; ++i) {
            if (r + i < rend) {
                const uint8_t *row = wbase + (long long)(r + i) * p.row_stride;
#pragma unroll
                for (int s = 0; s < SPT; ++s) {
                    if (on[s]) {
                        if (WT == B200_WT_Q8) {
                            wq[i][s] = ldg_stream_16(row + col[s]);
                            ws[i][s] = ldg_stream_u16(row + scale_off + (col[s] >> 5) * 2);
                        } else {
                            wq[i][s] = ldg_stream_16(row + (long long)col[s] * 2);
                        }
                    }
                }
            }
        }
    };

    // Weights depend on no earlier kernel: start streaming them, and let the
    // next kernel in the stream start doing the same, before waiting.
    pdl_launch_dependents();
    load_batch(r0, min(r0 + rmax, r1));
    pdl_wait();

    // Tensor parallel: every rank's partial vector must have landed in `slots`
    // (and, for the first kernel of a token, every rank must be done reading the
    // previous token's slots) before this block goes on.
    if (p.n_wait > 0) {
        if (tid < p.n_wait) {
            const unsigned want = (*p.d_epoch) * (unsigned)p.epoch_mul + (unsigned)p.epoch_add;
            if (!wait_flag_ge(p.d_wait_flags + tid, want)) *p.d_err = 1;
        }
        __syncthreads();
    }

    // ---------------- input assembly ----------------
    float x[SPT][E];
    if (p.in_mode == B200_IN_VEC) {
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; e += 4) {
                float4 t = on[s] ? *reinterpret_cast<const float4 *>(p.d_in_vec + col[s] + e) : make_float4(0, 0, 0, 0);
                x[s][e] = t.x; x[s][e + 1] = t.y; x[s][e + 2] = t.z; x[s][e + 3] = t.w;
            }
    } else {
        if (p.in_mode == B200_IN_EMBED) {
            const long long tok = p.d_tokens[*p.d_pos];
            const float *er = p.d_emb + tok * (long long)p.cols;
#pragma unroll
            for (int s = 0; s < SPT; ++s)
#pragma unroll
                for (int e = 0; e < E; e += 4) {
                    float4 t = on[s] ? *reinterpret_cast<const float4 *>(er + col[s] + e) : make_float4(0, 0, 0, 0);
                    x[s][e] = t.x * p.emb_scale; x[s][e + 1] = t.y * p.emb_scale;
                    x[s][e + 2] = t.z * p.emb_scale; x[s][e + 3] = t.w * p.emb_scale;
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
                            // slots may be written by other GPUs: read them past L1
                            float4 t = __ldcv(reinterpret_cast<const float4 *>(sl + col[s] + e));
                            sacc[s][e] += t.x; sacc[s][e + 1] += t.y; sacc[s][e + 2] += t.z; sacc[s][e + 3] += t.w;
                        }
                    }
            }
            if (p.d_slot_norm_gamma) {
                float ss = 0.0f;
#pragma unroll
                for (int s = 0; s < SPT; ++s)
#pragma unroll
                    for (int e = 0; e < E; ++e) ss = fmaf(sacc[s][e], sacc[s][e], ss);
                ss = block_sum(ss, red);
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
                    float4 t = on[s] ? *reinterpret_cast<const float4 *>(p.d_resid_in + col[s] + e) : make_float4(0, 0, 0, 0);
                    x[s][e] = t.x + sacc[s][e]; x[s][e + 1] = t.y + sacc[s][e + 1];
                    x[s][e + 2] = t.z + sacc[s][e + 2]; x[s][e + 3] = t.w + sacc[s][e + 3];
                }
        }
        if (blockIdx.x == 0 && p.d_resid_out) {
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
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)p.cols + p.eps);
#pragma unroll
        for (int s = 0; s < SPT; ++s)
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (on[s]) x[s][e] = p.d_norm_gamma[col[s] + e] * x[s][e] * inv;
    }

    // ---------------- stream the rows ----------------
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    for (int rb = r0; rb < r1; rb += rmax) {
        const int rend = min(rb + rmax, r1);
        for (int r = rb; r < rend; r += RB) {
            if (r != r0) load_batch(r, rend);
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                if (r + i < rend) {
                    float v = 0.0f;
#pragma unroll
                    for (int s = 0; s < SPT; ++s) {
                        if (on[s]) {
                            if (WT == B200_WT_Q8)
                                v = fmaf(__half2float(__ushort_as_half(ws[i][s])), dot16_q8(wq[i][s], x[s]), v);
                            else
                                v += dot8_f16(wq[i][s], x[s]);
                        }
                    }
                    part[(size_t)(r + i - rb) * T + tid] = v;
                }
            }
        }
        __syncthreads();
        // one warp finishes one row (or one gate/up pair): fixed order over the T partials
        const int nrows = rend - rb;
        for (int lr = warp * ralign; lr < nrows; lr += nw * ralign) {
            float v0 = 0.0f, v1 = 0.0f;
            for (int t = lane; t < T; t += 32) v0 += part[(size_t)lr * T + t];
            v0 = warp_sum(v0);
            if (ralign == 2) {
                for (int t = lane; t < T; t += 32) v1 += part[(size_t)(lr + 1) * T + t];
                v1 = warp_sum(v1);
            }
            const int row = rb + lr;
            if (p.out_mode == B200_OUT_GLU) {
                if (lane == 0) {
                    const float a = p.act == 0 ? act_silu(v0) : act_gelu_tanh(v0);
                    p.d_out[0][p.out_offset + (row >> 1)] = a * v1;
                }
            } else {
                if (lane < p.n_out) p.d_out[lane][p.out_offset + row] = v0;
                if (better(v0, row, best_v, best_i)) { best_v = v0; best_i = row; }
            }
        }
        __syncthreads();
    }

    if (!p.d_ticket) return;

    // ---------------- last-block bookkeeping ----------------
    float *am_v = red + 40;                       // [32] per-warp best value
    int *am_i = reinterpret_cast<int *>(red + 72);  // [32] per-warp best row
    if (p.d_argmax_scratch) {
        if (lane == 0) { am_v[warp] = best_v; am_i[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
            float bv = am_v[0]; int bi = am_i[0];
            for (int w = 1; w < nw; ++w) if (better(am_v[w], am_i[w], bv, bi)) { bv = am_v[w]; bi = am_i[w]; }
            p.d_argmax_scratch[2 * blockIdx.x] = bv;
            reinterpret_cast<int *>(p.d_argmax_scratch)[2 * blockIdx.x + 1] = bi;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.d_ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (warp == 0) {
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

template <int WT, int SPT, int RB, int MAXT>
int launch(const b200_matvec_args &a, int T, int grid, int rmax, cudaStream_t st)
{
    const size_t smem = ((size_t)rmax * T + 40 + 64) * sizeof(float);
    auto kern = matvec_kernel<WT, SPT, RB, MAXT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(T);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    ++g_b200_launches;
    return (int)cudaLaunchKernelEx(&cfg, kern, a, rmax);
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
        : a.in_mode == B200_IN_EMBED ? (!a.d_emb || !a.d_tokens || !a.d_pos) : true)
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

    const int E = a.wtype == B200_WT_Q8 ? 16 : 8;
    const int nsl = (a.cols + E - 1) / E;
    const int spt = (nsl + 1023) / 1024;
    if (spt > 2) return B200_E_TOOLARGE;
    const int T = (((nsl + spt - 1) / spt) + 31) / 32 * 32;
    const int ralign = a.out_mode == B200_OUT_GLU ? 2 : 1;
    const int units = a.rows / ralign;

    int grid = a.grid;
    if (grid <= 0) {
        int per_sm = 640 / T;
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 16) per_sm = 16;
        grid = sm_count() * per_sm;
    }
    if (grid > units) grid = units;
    const int RB = (spt == 1 && T <= 640) ? 8 : 4;
    int rows_cta = ((units + grid - 1) / grid) * ralign;
    int cap = (int)(40960 / (4 * (size_t)T)) / RB * RB;
    if (cap < RB) cap = RB;
    int rmax = (rows_cta + RB - 1) / RB * RB;
    if (rmax > cap) rmax = cap;
    cudaStream_t st = (cudaStream_t)stream;

#define B200_MV(WT_, SPT_, RB_, MAXT_) return launch<WT_, SPT_, RB_, MAXT_>(a, T, grid, rmax, st)
    if (a.wtype == B200_WT_Q8) {
        if (spt == 1) {
            if (T <= 256) B200_MV(B200_WT_Q8, 1, 8, 256);
            if (T <= 640) B200_MV(B200_WT_Q8, 1, 8, 640);
            B200_MV(B200_WT_Q8, 1, 4, 1024);
        }
        B200_MV(B200_WT_Q8, 2, 4, 1024);
    } else {
        if (spt == 1) {
            if (T <= 256) B200_MV(B200_WT_F16, 1, 8, 256);
            if (T <= 640) B200_MV(B200_WT_F16, 1, 8, 640);
            B200_MV(B200_WT_F16, 1, 4, 1024);
        }
        B200_MV(B200_WT_F16, 2, 4, 1024);
    }
#undef B200_MV
}
