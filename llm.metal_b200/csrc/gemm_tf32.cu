// Tensor-core GEMM for the frozen projections of the LoRA-SFT step (sm_100a only).
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T (+ R),  C, R fp32 row-major; A and B contiguous along k, either
//   binary16 (b200_gemm_f16: tcgen05.mma kind::f16) or fp32 read as TF32 (b200_gemm_tf32: kind::tf32).
//
// Replaces the reference's scalar tiled products f16_matmul / f16_matmul_nt
// (shaders/q8_kernels.metal:383-435) for the seven projections and the LM head,
// forward and backward (the backward product reads a transposed weight copy so
// that it has the same operand layout). The weights hold binary16 values and are
// exact in either operand format; the activation operand is rounded once per
// product (11 significant bits either way); accumulation is fp32 in tensor memory.
//
// Structure per CTA (one 128 x bn output tile, bn chosen per launch; 192 threads):
//   warp 0      producer: TMA (cp.async.bulk.tensor.2d, 128B swizzle) of a 128-row A tile and a bn-row
//               B tile, 128 bytes of k wide, one to three of each per slot of a ring guarded by
//               full/empty mbarriers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M=128, N=bn, 32 bytes of k per
//               instruction, four per sub-tile) and tcgen05.commit to release ring slots and, at the end,
//               to publish the accumulator
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (lane = row), alpha / residual, stores; with
//               split-k the CTAs of a tile add into C one after the other in split order
// Every wait is bounded; on a timeout the CTA raises *d_err, lets copies in
// flight land, frees its tensor memory and returns.
#include "stream_core.cuh"
#include "../../include/llmb200_train_kernels.h"

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

extern unsigned long long g_b200_launches;

namespace {

constexpr int BM = 128;          // rows of A per tile = TMEM lanes
constexpr int BK = 32;           // fp32 elements per stage along k = one 128-byte swizzle row
constexpr int UMMA_K = 8;        // k extent of one tcgen05.mma kind::tf32
constexpr int GEMM_THREADS = 192;

struct EpiArgs {
    float *C; long long ldc;
    const float *R; long long ldr;
    int M, N, K;
    float alpha;
    unsigned *d_err;
    int bn;            // columns of the output tile = N of one tcgen05.mma (a multiple of 16, 64..256)
    int stages;        // ring slots
    int tmem_cols;     // tensor-memory columns to allocate: the power of two >= bn
    int f16;           // 0: fp32 operands read as TF32 (32 per 128-byte row); 1: binary16 operands (64 per row)
    int ksub;          // 128-byte-wide k sub-tiles per ring slot (each its own 128-byte-swizzled block)
    int splits;        // CTAs sharing one output tile along k (gridDim.z); 1 = none
    unsigned *flags;   // one turn counter per output tile, zero between launches
};

// Turn counters of the serial split-k epilogue (see the kernel): one word per output tile.
constexpr int MAX_SPLIT_TILES = 1024;
__device__ unsigned g_split_flags[MAX_SPLIT_TILES];

constexpr int MAX_STAGES = 8;

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// K-major, 128-byte swizzle: rows 128 bytes apart, groups of 8 rows 1024 bytes apart (stride byte offset),
// leading byte offset unused (1), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Bounded wait that also gives up as soon as another role of the CTA has.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, unsigned parity, volatile int *abort_flag)
{
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63 && *abort_flag) return false;
    }
    return false;
}

__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const EpiArgs p)
{
    constexpr uint32_t A_BYTES = BM * BK * 4;
    const int BN = p.bn, STAGES = p.stages;
    const int KSUB = p.ksub;
    const uint32_t B_BYTES = (uint32_t)BN * BK * 4;                                     // both multiples of 1024
    const uint32_t STAGE_BYTES = (A_BYTES + B_BYTES) * KSUB;                            // [A_0 .. A_ksub-1][B_0 .. B_ksub-1]
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_bar;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;

    // the swizzle pattern of TMA and of the MMA descriptors is a function of the address: 1024-byte aligned tiles
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    // k-blocks of this CTA: the whole contraction, or its share when several CTAs split one tile along k
    const int BKE = p.f16 ? 2 * BK : BK;                         // elements per 128-byte operand row
    const int nkb_all = (p.K + BKE * KSUB - 1) / (BKE * KSUB);
    const int per_split = (nkb_all + p.splits - 1) / p.splits;
    const int kb0 = blockIdx.z * per_split;
    const int nkb = min(per_split, nkb_all - kb0);               // > 0: the host never launches an empty split
    volatile int *abort_flag = &abort_sh;

    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_sh;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES, it = kb / STAGES;
                if (!wait_or_abort(&empty_bar[s], (it & 1) ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.d_err) atomicExch(p.d_err, 0x7101u); }
                    break;
                }
                uint8_t *a_dst = tiles + (size_t)s * STAGE_BYTES, *b_dst = a_dst + A_BYTES * KSUB;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                for (int u = 0; u < KSUB; ++u) {     // a sub-tile past the end of k is all fill (zeros)
                    const int x = ((kb0 + kb) * KSUB + u) * BKE;
                    tma_load_2d(a_dst + (size_t)u * A_BYTES, &map_a, x, m0, &full_bar[s]);
                    tma_load_2d(b_dst + (size_t)u * B_BYTES, &map_b, x, n0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B TF32, both K-major, N = BN, M = 128
            // (operand format field: 2 = TF32, 0 = F16; an MMA covers 32 bytes of k either way: 8 or 16 elements)
            const uint32_t fmt = p.f16 ? 0u : 2u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % STAGES, it = kb / STAGES;
                if (!wait_or_abort(&full_bar[s], it & 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.d_err) atomicExch(p.d_err, 0x7102u); }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES), b_addr = a_addr + A_BYTES * KSUB;
                for (int u = 0; u < KSUB; ++u) {
                    const uint64_t adesc = smem_desc_sw128(a_addr + u * A_BYTES), bdesc = smem_desc_sw128(b_addr + u * B_BYTES);
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {     // 32 bytes along k per step: +2 in 16-byte units
                        if (p.f16) umma_f16(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | u | j) != 0);
                        else umma_tf32(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | u | j) != 0);
                    }
                }
                umma_commit(&empty_bar[s]);                     // slot reusable once these MMAs have read it
            }
            if (ok) umma_commit(&acc_bar);                      // accumulator complete
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32*(warp%4) .. +31
        const int lane_base = 32 * (warp & 3);
        const int row = m0 + lane_base + lane;
        bool ok = wait_or_abort(&acc_bar, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0 && !*abort_flag) { *abort_flag = 1; if (p.d_err) atomicExch(p.d_err, 0x7103u); }
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // Serial split-k: the CTAs of a tile add their partial sums into C one after the other, in split
            // order (deterministic), handing over through a turn counter. All of them are resident at once
            // (the host keeps tiles * splits <= SMs), so the wait cannot deadlock; it is bounded anyway.
            const int split = blockIdx.z;
            unsigned *turn = p.flags + (blockIdx.y * gridDim.x + blockIdx.x);
            if (p.splits > 1 && split > 0) {
                bool mine = true;
                if (lane == 0) {
                    mine = false;
                    for (int it = 0; it < (1 << 22); ++it) {
                        unsigned v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(turn) : "memory");
                        if (v == (unsigned)split) { mine = true; break; }
                        if ((it & 63) == 63 && *abort_flag) break;
                    }
                }
                mine = __shfl_sync(0xffffffffu, mine, 0);
                if (!mine) {
                    if (lane == 0 && !*abort_flag) { *abort_flag = 1; if (p.d_err) atomicExch(p.d_err, 0x7104u); }
                    ok = false;
                }
            }
            const bool first = split == 0;
            float *crow = p.C + (long long)row * p.ldc;
            // split 0 adds the residual; later splits add what is already in C
            const float *rrow = !first ? crow : p.R ? p.R + (long long)row * p.ldr : nullptr;
            const bool vec = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                             (!p.R || (((p.ldr & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0)));
#pragma unroll 1
            for (int c = 0; ok && c < BN; c += 32) {
                if (n0 + c >= p.N) break;                       // uniform across the warp
                const int cw = min(32, BN - c);                 // columns of this chunk that belong to the tile
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c, r);
                if (row < p.M) {
                    if (vec && cw == 32 && n0 + c + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 v = make_float4(p.alpha * __uint_as_float(r[j]), p.alpha * __uint_as_float(r[j + 1]),
                                                   p.alpha * __uint_as_float(r[j + 2]), p.alpha * __uint_as_float(r[j + 3]));
                            if (rrow) {
                                const float4 q = __ldcg(reinterpret_cast<const float4 *>(rrow + n0 + c + j));
                                v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                            }
                            *reinterpret_cast<float4 *>(crow + n0 + c + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int n = n0 + c + j;
                            if (j < cw && n < p.N) {
                                float v = p.alpha * __uint_as_float(r[j]);
                                if (rrow) v += __ldcg(rrow + n);
                                crow[n] = v;
                            }
                        }
                    }
                }
            }
        }
        if (p.splits > 1) {
            // every epilogue warp comes here on every path, so the barrier always has its 128 threads
            named_barrier(1, 128);                              // the four warps have stored their rows
            if (threadIdx.x == 64 && !*abort_flag) {
                __threadfence();
                const int split = blockIdx.z;
                unsigned *turn = p.flags + (blockIdx.y * gridDim.x + blockIdx.x);
                const unsigned next = split + 1 == p.splits ? 0u : (unsigned)(split + 1);
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(turn), "r"(next) : "memory");
            }
        }
    }

    // Teardown. After an abort, give copies already issued time to land before the memory is released.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------

typedef CUresult (*encode_fn_t)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_fn_t encode_fn()
{
    static encode_fn_t fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_fn_t>(p);
    }
    return fn;
}

// [rows, K] fp32 matrix with row stride ld elements; box = 32 x box_rows, 128-byte swizzle, zero fill outside.
bool make_map(CUtensorMap *map, const void *base, long long rows, long long K, long long ld, int box_rows, int f16)
{
    encode_fn_t enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * (f16 ? 2 : 4)};
    const cuuint32_t box[2] = {(cuuint32_t)(f16 ? 2 * BK : BK), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base),
               dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count_tc()
{
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// Tile choice, from measurements on B200. A CTA stages (128 + bn) * 128 bytes per 32 elements of k; an SM
// takes them in at <= ~117 GB/s (its 64 B/clk L2 port) and all SMs together at <= ~12 TB/s, and that, not
// the tensor pipe, bounds the kernel -- fewer bytes per flop (wide tiles) win as long as the tiles fill the
// machine.
//  * 128-wide tiles fit in one wave: take them, with two k sub-tiles per ring slot (three 64 KB slots
//    hide the per-slot hand-over better than six 32 KB ones: 0.27 us instead of 0.40 us per 32 of k);
//    96-wide tiles with three sub-tiles per slot when those fit one wave too (more CTAs at work).
//    With a very long contraction on top (the LM-head backward, K = vocabulary), three CTAs split a
//    256-wide tile along k; their epilogues run one after the other, which only pays when k is long.
//  * otherwise the width (a multiple of 16 up to 256) that minimises waves * (128 + bn).
void pick_tile(int M, int N, int K, int f16, int *bn_out, int *ksub_out, int *splits_out)
{
    const int bke = f16 ? 2 * BK : BK;
    const int mt = (M + BM - 1) / BM, sms = sm_count_tc(), nkb = (K + bke - 1) / bke;
    *splits_out = 1;
    if ((long long)mt * ((N + 127) / 128) <= sms) {
        const long long tiles256 = (long long)mt * ((N + 255) / 256);
        static int split_nkb = -1;
        if (split_nkb < 0) {
            const char *t = getenv("LLMB200_GEMM_SPLIT_NKB");
            split_nkb = t ? atoi(t) : 1024;
        }
        if (nkb >= split_nkb && tiles256 * 3 <= sms && tiles256 <= MAX_SPLIT_TILES) {
            *bn_out = 256; *ksub_out = 1; *splits_out = 3;
        } else if ((long long)mt * ((N + 95) / 96) <= sms) {
            *bn_out = 96; *ksub_out = 3;      // measured ~10 % faster than 128 x 2 when it still fits one wave
                                              // (80-wide tiles, 128 CTAs instead of 108 at N = 2560, measured 0.8 % slower)
        } else {
            *bn_out = 128; *ksub_out = 2;
        }
        return;
    }
    long long best = -1;
    for (int bn = 144; bn <= 256; bn += 16) {
        const long long tiles = (long long)mt * ((N + bn - 1) / bn);
        const long long cost = ((tiles + sms - 1) / sms) * (BM + bn);
        if (best < 0 || cost < best || (cost == best && bn > *bn_out)) { best = cost; *bn_out = bn; }
    }
    *ksub_out = *bn_out <= 192 ? 2 : 1;       // two sub-tiles per slot as long as two slots still fit
}

int launch(const CUtensorMap &ma, const CUtensorMap &mb, EpiArgs e, cudaStream_t st)
{
    static int ksub_env = -1;
    if (ksub_env < 0) {
        const char *t = getenv("LLMB200_GEMM_KSUB");
        ksub_env = t ? atoi(t) : 0;
        if (ksub_env < 0 || ksub_env > 4) ksub_env = 0;
    }
    if (ksub_env) e.ksub = ksub_env;
    // One CTA per SM with a 200 KB ring; two resident CTAs with 100 KB rings each (the epilogue of one under the
    // mainloop of the other) measured 2.5 % slower on the multi-wave products: the shallower ring costs more.
    while (e.ksub > 1 && (size_t)(BM + e.bn) * BK * 4 * e.ksub * 2 > 200 * 1024) --e.ksub;
    const size_t stage = (size_t)(BM + e.bn) * BK * 4 * e.ksub;
    int stages = (int)((200 * 1024) / stage);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) return B200_E_UNSUPPORTED;
    e.stages = stages;
    e.tmem_cols = e.bn <= 64 ? 64 : e.bn <= 128 ? 128 : 256;
    const size_t smem = stage * stages + 1024;
    static size_t attr_set = 0;
    if (smem > attr_set) {
        cudaError_t rc = cudaFuncSetAttribute(gemm_tf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc != cudaSuccess) return (int)rc;
        attr_set = smem;
    }
    static unsigned *flags_addr = nullptr;       // looked up once (the first launch must not be inside a stream capture)
    if (!flags_addr && cudaGetSymbolAddress((void **)&flags_addr, g_split_flags) != cudaSuccess) return B200_E_UNSUPPORTED;
    e.flags = flags_addr;
    dim3 grid((e.M + BM - 1) / BM, (e.N + e.bn - 1) / e.bn, e.splits);
    gemm_tf32_kernel<<<grid, GEMM_THREADS, smem, st>>>(ma, mb, e);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}

}  // namespace

static int gemm_tc(const b200_gemm_args *a, int f16, void *stream)
{
    if (!a || !a->A || !a->B || !a->C || a->M <= 0 || a->N <= 0 || a->K <= 0) return B200_E_BADARG;
    if (a->a_col != 1 || a->b_row != 1) return B200_E_UNSUPPORTED;
    const long long lda = a->a_row, ldb = a->b_col;
    const int gran = f16 ? 7 : 3;                                  // 16-byte granularity of rows and of k
    if ((a->K & gran) || (lda & gran) || (ldb & gran) || lda < a->K || ldb < a->K) return B200_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15)) return B200_E_UNSUPPORTED;
    if (a->N < 64) return B200_E_UNSUPPORTED;                     // the CUDA-core kernel is the better fit
    if ((a->N + 63) / 64 > 65535) return B200_E_UNSUPPORTED;

    CUtensorMap ma, mb;
    EpiArgs e = {a->C, a->ldc, a->R, a->ldr, a->M, a->N, a->K, a->alpha, a->d_err, 128, 0, 0, f16, 1, 1, nullptr};
    // LLMB200_GEMM_BN=<n> overrides the tile width for experiments
    static int forced = -1;
    if (forced < 0) {
        const char *t = getenv("LLMB200_GEMM_BN");
        forced = t ? atoi(t) : 0;
        if (forced < 0 || forced > 256 || (forced % 16)) forced = 0;
    }
    pick_tile(a->M, a->N, a->K, f16, &e.bn, &e.ksub, &e.splits);
    if (forced >= 64) { e.bn = forced; e.splits = 1; }
    if (!make_map(&ma, a->A, a->M, a->K, lda, BM, f16)) return B200_E_UNSUPPORTED;
    if (!make_map(&mb, a->B, a->N, a->K, ldb, e.bn, f16)) return B200_E_UNSUPPORTED;
    return launch(ma, mb, e, (cudaStream_t)stream);
}

extern "C" int b200_gemm_tf32(const b200_gemm_args *a, void *stream) { return gemm_tc(a, 0, stream); }
extern "C" int b200_gemm_f16(const b200_gemm_args *a, void *stream) { return gemm_tc(a, 1, stream); }
