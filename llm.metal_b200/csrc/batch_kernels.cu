// Small kernels of the batched decode step (several sequences sharing one weight read).
//
// The reference takes the arg-max of every sequence's logits on the CPU after each step
// (src/nn/fast_inference.c:469-476, 955-958); here a kernel does it per row, feeds the result back as
// the next step's input tokens, records it, and advances the position, so that a step is one CUDA
// graph with no host in the loop.
#include "common.cuh"
#include "../../include/llmb200_kernels.h"

extern unsigned long long g_b200_launches;

namespace {

// ctl[0] = position, ctl[1] = number of recorded steps, ctl[2] = record flag (0 during the prompt).
// One block per row. The lowest index wins ties, like the reference's strict '>' scan.
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float *logits, int vocab, unsigned *next_tokens, unsigned *history, int n_rows, int max_steps,
                   int *ctl, unsigned *done_count)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    const int row = blockIdx.x;
    const float *lr = logits + (size_t)row * vocab;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = lr[i];
        if (v > best) { best = v; bi = i; }          // ascending i per thread: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = best; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i)
            if (sv[i] > best || (sv[i] == best && si[i] < bi)) { best = sv[i]; bi = si[i]; }
        if (bi < 0 || bi >= vocab) bi = 0;           // all-NaN row: stay inside the table
        next_tokens[row] = (unsigned)bi;
        const int step = ctl[1];
        if (ctl[2] && step < max_steps) history[(size_t)step * n_rows + row] = (unsigned)bi;
        // the last row to finish advances the position (and the step count when recording)
        __threadfence();
        if (atomicAdd(done_count, 1u) == (unsigned)n_rows - 1u) {
            *done_count = 0u;
            ctl[0] += 1;
            if (ctl[2]) ctl[1] = step + 1;
        }
    }
}

}  // namespace

extern "C" int b200_argmax_rows(const float *logits, int n_rows, int vocab, unsigned *next_tokens, unsigned *history,
                                int max_steps, int *ctl, unsigned *done_count, void *stream)
{
    if (!logits || !next_tokens || !history || !ctl || !done_count || n_rows <= 0 || vocab <= 0 || max_steps <= 0)
        return B200_E_BADARG;
    argmax_rows_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, vocab, next_tokens, history, n_rows, max_steps,
                                                                 ctl, done_count);
    ++g_b200_launches;
    return (int)cudaGetLastError();
}
