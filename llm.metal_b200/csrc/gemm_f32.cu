// CUDA-core fp32 GEMM with arbitrary unit-stride orientation of both operands.
//
// Carries the small and oddly shaped products of the LoRA-SFT step (the rank-R
// LoRA matmuls of src/nn/fast_sft.c:639-643, 946-966: float_matmul,
// float_matmul_tn, float_matmul_nt of shaders/q8_kernels.metal:1043-1152) and is
// the any-shape fallback of the tensor-core GEMM for the frozen projections
// (f16_matmul :383-407, f16_matmul_nt :411-435). fp32 multiply-add throughout,
// k ascending within a thread, like the reference's tiled kernels.
//
// Tile 64 x 64 x 16, 256 threads, 4 x 4 outputs per thread. The loader walks
// whichever dimension of an operand has stride 1 so that global reads coalesce.
#include "common.cuh"
#include "../../include/llmb200_train_kernels.h"

extern unsigned long long g_b200_launches;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// AK: A is contiguous along k (a_col == 1); otherwise along m. BKC: B contiguous along k (b_row == 1).
template <bool AK, bool BKC>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const b200_gemm_args p)
{
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;      // thread's 4 columns start at tx*4, 4 rows at ty*4

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += 256) {
            int m, k;
            if (AK) { k = e % BK; m = e / BK; } else { m = e % BM; k = e / BM; }
            const int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < p.M && gk < p.K) ? __ldg(p.A + (long long)gm * p.a_row + (long long)gk * p.a_col) : 0.f;
        }
#pragma unroll
        for (int e = tid; e < BN * BK; e += 256) {
            int n, k;
            if (BKC) { k = e % BK; n = e / BK; } else { n = e % BN; k = e / BN; }
            const int gn = n0 + n, gk = k0 + k;
            Bs[k][n] = (gn < p.N && gk < p.K) ? __ldg(p.B + (long long)gk * p.b_row + (long long)gn * p.b_col) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4 *>(&As[k][ty * TM]);
            const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[k][tx * TN]);
            const float a[TM] = {a4.x, a4.y, a4.z, a4.w};
            const float b[TN] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= p.N) continue;
            float v = p.alpha * acc[i][j];
            if (p.R) v += p.R[(long long)gm * p.ldr + gn];
            p.C[(long long)gm * p.ldc + gn] = v;
        }
    }
}

}  // namespace

extern "C" int b200_gemm_f32(const b200_gemm_args *a, void *stream)
{
    if (!a || !a->A || !a->B || !a->C || a->M <= 0 || a->N <= 0 || a->K <= 0) return B200_E_BADARG;
    if ((a->a_row != 1 && a->a_col != 1) || (a->b_row != 1 && a->b_col != 1)) return B200_E_BADARG;
    const bool ak = a->a_col == 1, bk = a->b_row == 1;
    dim3 grid((a->N + BN - 1) / BN, (a->M + BM - 1) / BM);
    cudaStream_t st = (cudaStream_t)stream;
    if (ak && bk) gemm_f32_kernel<true, true><<<grid, 256, 0, st>>>(*a);
    else if (ak) gemm_f32_kernel<true, false><<<grid, 256, 0, st>>>(*a);
    else if (bk) gemm_f32_kernel<false, true><<<grid, 256, 0, st>>>(*a);
    else gemm_f32_kernel<false, false><<<grid, 256, 0, st>>>(*a);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}
