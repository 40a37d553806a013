// Tensor-core GEMM for the frozen projections of the LoRA-SFT step (sm_100a only).
//
//   C[M,N] = alpha * A[M,K] * B[N,K]^T (+ R),  A, B, C, R fp32 row-major, A and B contiguous along k.
//
// Replaces the reference's scalar tiled products f16_matmul / f16_matmul_nt
// (shaders/q8_kernels.metal:383-435) for the seven projections and the LM head,
// forward and backward (the backward product reads a transposed weight copy so
// that it has the same operand layout). Operands are fp32 in memory; the tensor
// core reads them as TF32 (10-bit mantissa): weights holding binary16 values
// are exact, activations are rounded once per product, accumulation is fp32.
//
// Structure per CTA (one 128 x BN output tile, 192 threads):
//   warp 0      producer: TMA (cp.async.bulk.tensor.2d, 128B swizzle) of a 128 x 32 A tile and a
//               BN x 32 B tile per stage into a ring guarded by full/empty mbarriers
//   warp 1      allocates BN columns of tensor memory; one lane issues tcgen05.mma
//               (kind::tf32, M=128, N=BN, K=8; four per stage) and tcgen05.commit to
//               release ring slots and, at the end, to publish the accumulator
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (lane = row), alpha / residual, stores
// Every wait is bounded; on a timeout the CTA raises *d_err, lets copies in
// flight land, frees its tensor memory and returns.
#include "stream_core.cuh"
#include "../../include/llmb200_train_kernels.h"

#include <cuda.h>

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
};

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

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const EpiArgs p)
{
    constexpr uint32_t A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4, STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_sh;

    // the swizzle pattern of TMA and of the MMA descriptors is a function of the address: 1024-byte aligned tiles
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int nkb = (p.K + BK - 1) / BK;
    volatile int *abort_flag = &abort_sh;

    if (threadIdx.x == 0) {
        abort_sh = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"((uint32_t)BN) : "memory");
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
                uint8_t *a_dst = tiles + (size_t)s * STAGE_BYTES, *b_dst = a_dst + A_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, kb * BK, m0, &full_bar[s]);
                tma_load_2d(b_dst, &map_b, kb * BK, n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B TF32, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % STAGES, it = kb / STAGES;
                if (!wait_or_abort(&full_bar[s], it & 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; if (p.d_err) atomicExch(p.d_err, 0x7102u); }
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
                const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(b_addr);
#pragma unroll
                for (int j = 0; j < BK / UMMA_K; ++j)           // 32 bytes along k per step: +2 in 16-byte units
                    umma_tf32(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, (kb | j) != 0);
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
            float *crow = p.C + (long long)row * p.ldc;
            const float *rrow = p.R ? p.R + (long long)row * p.ldr : nullptr;
            const bool vec = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                             (!p.R || (((p.ldr & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0)));
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                if (n0 + c >= p.N) break;                       // uniform across the warp
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c, r);
                if (row < p.M) {
                    if (vec && n0 + c + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 v = make_float4(p.alpha * __uint_as_float(r[j]), p.alpha * __uint_as_float(r[j + 1]),
                                                   p.alpha * __uint_as_float(r[j + 2]), p.alpha * __uint_as_float(r[j + 3]));
                            if (rrow) {
                                const float4 q = *reinterpret_cast<const float4 *>(rrow + n0 + c + j);
                                v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                            }
                            *reinterpret_cast<float4 *>(crow + n0 + c + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int n = n0 + c + j;
                            if (n < p.N) {
                                float v = p.alpha * __uint_as_float(r[j]);
                                if (rrow) v += rrow[n];
                                crow[n] = v;
                            }
                        }
                    }
                }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
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
bool make_map(CUtensorMap *map, const float *base, long long rows, long long K, long long ld, int box_rows)
{
    encode_fn_t enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const EpiArgs &e, cudaStream_t st)
{
    constexpr size_t smem = (size_t)STAGES * (BM + BN) * BK * 4 + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t rc = cudaFuncSetAttribute(gemm_tf32_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)smem);
        if (rc != cudaSuccess) return (int)rc;
        set = true;
    }
    dim3 grid((e.M + BM - 1) / BM, (e.N + BN - 1) / BN);
    gemm_tf32_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, e);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}

}  // namespace

extern "C" int b200_gemm_tf32(const b200_gemm_args *a, void *stream)
{
    if (!a || !a->A || !a->B || !a->C || a->M <= 0 || a->N <= 0 || a->K <= 0) return B200_E_BADARG;
    if (a->a_col != 1 || a->b_row != 1) return B200_E_UNSUPPORTED;
    const long long lda = a->a_row, ldb = a->b_col;
    if ((a->K & 3) || (lda & 3) || (ldb & 3) || lda < a->K || ldb < a->K) return B200_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15)) return B200_E_UNSUPPORTED;
    if (a->N < 64 || a->M < 16) return B200_E_UNSUPPORTED;        // the CUDA-core kernel is the better fit
    if ((a->M + BM - 1) / BM > 2147483647 || (a->N + 127) / 128 > 65535) return B200_E_UNSUPPORTED;

    CUtensorMap ma, mb;
    EpiArgs e = {a->C, a->ldc, a->R, a->ldr, a->M, a->N, a->K, a->alpha, a->d_err};
    if (!make_map(&ma, a->A, a->M, a->K, lda, BM)) return B200_E_UNSUPPORTED;
    if (!make_map(&mb, a->B, a->N, a->K, ldb, 128)) return B200_E_UNSUPPORTED;
    return launch<128, 6>(ma, mb, e, (cudaStream_t)stream);
}
