// LoRA side path of the decode step (sm_100a): q += s * B_q (A_q x), v += s * B_v (A_v x) for one token.
//
// Stands in for the six dispatches src/nn/fast_inference.c:406-421 adds per layer when an adapter is
// attached (two float_matmul with M = 1 and one add_scaled for q, the same for v; fp32 throughout).
// x is the normalised layer input the fused q/k/v matvec has just consumed (it stores a copy on request).
// Every block recomputes the 2R dot products A x (R*D multiply-adds, the matrices sit in L2) and then
// updates its slice of the q and v rows, so one short launch does all six steps.
#include "common.cuh"
#include "../../include/llmb200_kernels.h"

extern unsigned long long g_b200_launches;

namespace {

constexpr int LORA_MAX_R = 64;

__global__ void __launch_bounds__(256)
lora_decode_kernel(const float *x, const float *A_q, const float *B_q, const float *A_v, const float *B_v, float *qkv,
                   int D, int q_rows, int kv_rows, int R, float sc)
{
    __shared__ float mid[2 * LORA_MAX_R];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < 2 * R; r += 8) {
        const float *a = r < R ? A_q + (size_t)r * D : A_v + (size_t)(r - R) * D;
        float acc = 0.f;
        for (int d = lane; d < D; d += 32) acc = fmaf(a[d], x[d], acc);
        acc = warp_sum(acc);
        if (lane == 0) mid[r] = acc;
    }
    __syncthreads();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;        // 0 .. q_rows + kv_rows - 1
    if (row >= q_rows + kv_rows) return;
    const bool is_q = row < q_rows;
    const float *b = is_q ? B_q + (size_t)row * R : B_v + (size_t)(row - q_rows) * R;
    const float *m = is_q ? mid : mid + R;
    float acc = 0.f;
    for (int r = 0; r < R; ++r) acc = fmaf(m[r], b[r], acc);
    float *dst = is_q ? qkv + row : qkv + q_rows + kv_rows + (row - q_rows);   // v sits after q and k
    *dst += sc * acc;
}

}  // namespace

extern "C" int b200_lora_decode(const float *x, const float *A_q, const float *B_q, const float *A_v, const float *B_v,
                                float *qkv, int d_model, int q_rows, int kv_rows, int rank, float scaling, void *stream)
{
    if (!x || !A_q || !B_q || !A_v || !B_v || !qkv || d_model <= 0 || q_rows <= 0 || kv_rows <= 0 || rank <= 0 ||
        rank > LORA_MAX_R)
        return B200_E_BADARG;
    const unsigned grid = (unsigned)((q_rows + kv_rows + 255) / 256);
    lora_decode_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, A_q, B_q, A_v, B_v, qkv, d_model, q_rows, kv_rows, rank,
                                                                scaling);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}
