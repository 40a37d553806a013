// Upload-time weight conversion: fp32 -> packed Q8_0 / F16 rows, and back to
// the reference's canonical byte stream.
//
// The arithmetic restates quantize_row_q8 (src/nn/wmat.c:19-41) operation by
// operation in IEEE fp32 so that the quantised bytes are identical to the CPU
// quantiser's: amax over 32 values, scale = amax / 127 (correctly rounded
// division), d = binary16(scale) round-to-nearest-even, inv = 1 / scale
// (division again, from the *unrounded* fp32 scale), q = roundf(x * inv)
// (half away from zero) clamped to [-128, 127]. This file must not be built
// with --use_fast_math.
#include "common.cuh"
#include "../../include/llmb200_kernels.h"

extern unsigned long long g_b200_launches;

__global__ void __launch_bounds__(256)
q8_pack_kernel(const float *__restrict__ src, long long ld, int rows, int nb,
               uint8_t *__restrict__ dst, long long dst_stride, int dst_row0, int dst_row_step)
{
    const long long total = (long long)rows * nb;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nb), b = (int)(i % nb);
        const float4 *sp = reinterpret_cast<const float4 *>(src + (long long)r * ld + (long long)b * 32);
        float v[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float4 t = sp[j];
            v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) { float a = fabsf(v[j]); if (a > amax) amax = a; }
        const float scale = __fdiv_rn(amax, 127.0f);
        const __half h = __float2half_rn(scale);
        uint32_t q[8];
        if (scale != 0.0f) {
            const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                uint32_t word = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    int iv = (int)roundf(__fmul_rn(v[4 * w + k], inv));
                    iv = iv < -128 ? -128 : (iv > 127 ? 127 : iv);
                    word |= (uint32_t)(iv & 0xff) << (8 * k);
                }
                q[w] = word;
            }
        } else {
#pragma unroll
            for (int w = 0; w < 8; ++w) q[w] = 0u;
        }
        uint8_t *row = dst + (long long)(dst_row0 + (long long)r * dst_row_step) * dst_stride;
        uint4 *qp = reinterpret_cast<uint4 *>(row + (long long)b * 32);
        qp[0] = make_uint4(q[0], q[1], q[2], q[3]);
        qp[1] = make_uint4(q[4], q[5], q[6], q[7]);
        reinterpret_cast<__half *>(row + (long long)nb * 32)[b] = h;
    }
}

__global__ void __launch_bounds__(256)
f16_pack_kernel(const float *__restrict__ src, long long ld, int rows, int cols,
                uint8_t *__restrict__ dst, long long dst_stride, int dst_row0, int dst_row_step)
{
    const int c4 = cols / 4;                       // cols % 8 == 0 is checked by the launcher
    const long long total = (long long)rows * c4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / c4), c = (int)(i % c4);
        const float4 t = reinterpret_cast<const float4 *>(src + (long long)r * ld)[c];
        __half2 lo = __halves2half2(__float2half_rn(t.x), __float2half_rn(t.y));
        __half2 hi = __halves2half2(__float2half_rn(t.z), __float2half_rn(t.w));
        uint8_t *row = dst + (long long)(dst_row0 + (long long)r * dst_row_step) * dst_stride;
        uint2 o;
        o.x = *reinterpret_cast<uint32_t *>(&lo);
        o.y = *reinterpret_cast<uint32_t *>(&hi);
        reinterpret_cast<uint2 *>(row)[c] = o;
    }
}

// One thread per block: 34 bytes out, written bytewise (the canonical stream is
// only 2-byte aligned).
__global__ void __launch_bounds__(256)
q8_unpack_kernel(const uint8_t *__restrict__ packed, long long row_stride, int rows, int nb,
                 uint8_t *__restrict__ blocks)
{
    const long long total = (long long)rows * nb;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nb), b = (int)(i % nb);
        const uint8_t *row = packed + (long long)r * row_stride;
        uint8_t *o = blocks + i * 34;
        const uint16_t d = reinterpret_cast<const uint16_t *>(row + (long long)nb * 32)[b];
        reinterpret_cast<uint16_t *>(o)[0] = d;
        const uint16_t *q = reinterpret_cast<const uint16_t *>(row + (long long)b * 32);
#pragma unroll
        for (int j = 0; j < 16; ++j) reinterpret_cast<uint16_t *>(o + 2)[j] = q[j];
    }
}

static int grid_for(long long total) {
    long long g = (total + 255) / 256;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return (int)g;
}

extern "C" size_t b200_packed_row_stride(int wtype, int cols)
{
    size_t raw = wtype == B200_WT_Q8 ? (size_t)(cols / 32) * 34 : (size_t)cols * 2;
    return (raw + 15) & ~(size_t)15;
}

extern "C" int b200_q8_pack(const float *d_src, long long ld, int rows, int cols,
                            void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step,
                            void *stream)
{
    if (!d_src || !d_dst || rows < 0 || cols <= 0 || cols % 32 || ld < cols || (ld % 4) ||
        dst_row_stride < (long long)b200_packed_row_stride(B200_WT_Q8, cols) || (dst_row_stride % 16) ||
        ((uintptr_t)d_src % 16) || ((uintptr_t)d_dst % 16))
        return B200_E_BADARG;
    if (rows == 0) return 0;
    const long long total = (long long)rows * (cols / 32);
    q8_pack_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
        d_src, ld, rows, cols / 32, (uint8_t *)d_dst, dst_row_stride, dst_row0, dst_row_step);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}

extern "C" int b200_f16_pack(const float *d_src, long long ld, int rows, int cols,
                             void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step,
                             void *stream)
{
    if (!d_src || !d_dst || rows < 0 || cols <= 0 || cols % 8 || ld < cols || (ld % 4) ||
        dst_row_stride < (long long)b200_packed_row_stride(B200_WT_F16, cols) || (dst_row_stride % 16) ||
        ((uintptr_t)d_src % 16) || ((uintptr_t)d_dst % 16))
        return B200_E_BADARG;
    if (rows == 0) return 0;
    const long long total = (long long)rows * (cols / 4);
    f16_pack_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
        d_src, ld, rows, cols, (uint8_t *)d_dst, dst_row_stride, dst_row0, dst_row_step);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}

extern "C" int b200_q8_unpack_blocks(const void *d_packed, long long row_stride, int rows, int cols,
                                     void *d_blocks, void *stream)
{
    if (!d_packed || !d_blocks || rows < 0 || cols <= 0 || cols % 32 ||
        row_stride < (long long)b200_packed_row_stride(B200_WT_Q8, cols))
        return B200_E_BADARG;
    if (rows == 0) return 0;
    const long long total = (long long)rows * (cols / 32);
    q8_unpack_kernel<<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t *)d_packed, row_stride, rows, cols / 32, (uint8_t *)d_blocks);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}
