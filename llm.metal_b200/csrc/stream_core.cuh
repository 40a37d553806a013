// Device helpers shared by the weight-streaming kernels: mbarrier / bulk-copy (TMA) primitives, the
// int8 / binary16 -> fp32 dot products of one 16-byte slice, activations and small reductions.
#pragma once
#include "common.cuh"

namespace {

// ---- mbarrier / bulk-copy primitives ------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *b, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *b, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *b)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *b, unsigned parity)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded: gives up after ~a second instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *b, unsigned parity)
{
    for (int it = 0; it < (1 << 22); ++it)
        if (mbar_try_wait(b, parity)) return true;
    return false;
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, unsigned bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds_128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void named_barrier(int id, int count)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---- arithmetic -----------------------------------------------------------
// int8 -> fp32 through the 2^23 trick: a byte biased by 128 is dropped into the
// low mantissa byte of 0x4B000000 (= 8388608.0f); subtracting 8388736.0f leaves
// the signed value exactly. Conversion and multiply-add run two elements per
// instruction on the packed fp32 pipe (add.f32x2 / fma.rn.f32x2).
__device__ __forceinline__ float2 q8_pair(uint32_t biased_word, int k)
{
    float2 f;
    f.x = __uint_as_float(__byte_perm(biased_word, 0x4B000000u, 0x7650u + k));
    f.y = __uint_as_float(__byte_perm(biased_word, 0x4B000000u, 0x7651u + k));
    return __fadd2_rn(f, make_float2(-8388736.0f, -8388736.0f));
}

__device__ __forceinline__ float dot16_q8(const uint4 &w, const float *x)
{
    const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
    float2 a = make_float2(0.f, 0.f), b = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a = __ffma2_rn(q8_pair(u[i], 0), make_float2(x[4 * i + 0], x[4 * i + 1]), a);
        b = __ffma2_rn(q8_pair(u[i], 2), make_float2(x[4 * i + 2], x[4 * i + 3]), b);
    }
    return (a.x + a.y) + (b.x + b.y);
}

// 16 int8 weights against a 16-element slice of the input held as three signed byte planes
// (x = scale * (a + 256 b + 65536 c), see quantize_input in decode_token.cu): twelve dp4a, exact in
// int32 (each sum stays below 2^18), then a + 256 b joined in integers and c joined in fp32.
__device__ __forceinline__ float dot16_q8_planes(const uint4 &w, const uint4 &a, const uint4 &b, const uint4 &c)
{
    int sa = __dp4a((int)w.x, (int)a.x, 0), sb = __dp4a((int)w.x, (int)b.x, 0), sc = __dp4a((int)w.x, (int)c.x, 0);
    sa = __dp4a((int)w.y, (int)a.y, sa); sb = __dp4a((int)w.y, (int)b.y, sb); sc = __dp4a((int)w.y, (int)c.y, sc);
    sa = __dp4a((int)w.z, (int)a.z, sa); sb = __dp4a((int)w.z, (int)b.z, sb); sc = __dp4a((int)w.z, (int)c.z, sc);
    sa = __dp4a((int)w.w, (int)a.w, sa); sb = __dp4a((int)w.w, (int)b.w, sb); sc = __dp4a((int)w.w, (int)c.w, sc);
    return fmaf((float)sc, 65536.0f, (float)(sa + (sb << 8)));
}

__device__ __forceinline__ float dot8_f16(const uint4 &w, const float *x)
{
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    float2 a = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        a = __ffma2_rn(__half22float2(*reinterpret_cast<const __half2 *>(&u[i])), make_float2(x[2 * i], x[2 * i + 1]), a);
    return a.x + a.y;
}

// exp through ex2.approx (2 ulp), what the shader's fast-math exp is (q8_kernels.metal:336)
__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + __expf(-g)); }
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

// Sum of v over the T threads of one consumer group; every thread gets it.
__device__ __forceinline__ float group_sum(float v, float *red, int bar_id, int T, int t)
{
    const int lane = t & 31, w = t >> 5, nw = T >> 5;
    v = warp_sum(v);
    named_barrier(bar_id, T);              // protect `red` from a previous use
    if (lane == 0) red[w] = v;
    named_barrier(bar_id, T);
    float tot = 0.0f;
    for (int i = 0; i < nw; ++i) tot += red[i];
    return tot;
}

// v[j] holds this lane's partial of row j. Returns, in every lane, the warp
// total of row (lane & (RB-1)): RB-1 exchanges fold the rows across lane bits,
// the remaining log2(32/RB) butterflies add the lane groups.
template <int RB>
__device__ __forceinline__ float reduce_rows(float (&v)[RB], int lane)
{
#pragma unroll
    for (int h = RB / 2; h >= 1; h >>= 1) {
        const bool up = (lane & h) != 0;
#pragma unroll
        for (int j = 0; j < h; ++j) {
            const float send = up ? v[j] : v[j + h];
            const float keep = up ? v[j + h] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, h);
        }
    }
    float tot = v[0];
#pragma unroll
    for (int o = RB; o < 32; o <<= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    return tot;
}


} // namespace
