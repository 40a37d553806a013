// Shared device helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define B200_WARP 32

// ---- programmatic dependent launch -------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may
// begin while its predecessor drains. Everything before pdl_wait() must touch
// only memory no earlier kernel writes (here: weights); pdl_wait() returns once
// the predecessor grid has completed and its stores are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- memory ------------------------------------------------------------
// Streaming 16-byte load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned short ldg_stream_u16(const void *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// ---- reductions --------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the whole block; every thread gets the result. `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // protect `red` from a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Bounded wait for a flag another GPU writes. Returns false when it gave up.
#define B200_SPIN_LIMIT 4000000
__device__ __forceinline__ bool wait_flag_ge(const unsigned *flag, unsigned want, int limit = B200_SPIN_LIMIT) {
    for (int it = 0; it < limit; ++it) {
        // signed distance so that a wrapped counter still compares correctly
        if ((int)(ld_acquire_sys(flag) - want) >= 0) return true;
        __nanosleep(20);
    }
    return false;
}
