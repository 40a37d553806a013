// Tensor-core GEMM placeholder: reports "unsupported" so that callers take the CUDA-core path.
#include "common.cuh"
#include "../../include/llmb200_train_kernels.h"

extern "C" int b200_gemm_tf32(const b200_gemm_args *a, void *stream)
{
    (void)a; (void)stream;
    return B200_E_UNSUPPORTED;
}
