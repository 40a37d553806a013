/* Internal declarations shared by the C host files of libllmb200. */
#ifndef LLMB200_INTERNAL_H
#define LLMB200_INTERNAL_H

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/llmb200_kernels.h"
#include "../../include/llmb200_wmat.h"

enum { MB_SHARED = 0, MB_Q8 = 1, MB_F16 = 2, MB_DEVICE = 3 };

struct MetalBuf {
    void *dev;               /* device (or unified) pointer */
    size_t size;             /* bytes at dev */
    int kind;                /* MB_* */
    int rows, cols;          /* packed weights only */
    long long row_stride;
    void *host_mirror;       /* canonical host copy of a packed weight, made on demand */
    int borrowed;            /* dev belongs to someone else: metal_buf_free leaves it alone */
};

#define LLMB200_STAGE_BYTES ((size_t)64 << 20)

typedef struct {
    int refs;
    int device;
    cudaStream_t stream;
    /* double-buffered upload staging: pinned host + device fp32 */
    float *h_stage[2];
    float *d_stage[2];
    cudaEvent_t stage_done[2];
    int stage_next;
} llmb200_runtime;

/* One runtime (stream + staging buffers) per CUDA device. A host thread works with the runtime of its
 * current device, so several devices can be driven from one process -- one thread each. */
#define LLMB200_MAX_DEVICES 16
extern llmb200_runtime g_rts[LLMB200_MAX_DEVICES];
static inline llmb200_runtime *llmb200_rt(void)
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= LLMB200_MAX_DEVICES) { (void)cudaGetLastError(); d = 0; }
    return &g_rts[d];
}
#define g_rt (*llmb200_rt())

#define CU_TRY(call, onfail)                                                          \
    do {                                                                              \
        cudaError_t e__ = (call);                                                     \
        if (e__ != cudaSuccess) {                                                     \
            fprintf(stderr, "[llmb200] %s failed: %s (%s:%d)\n", #call,               \
                    cudaGetErrorString(e__), __FILE__, __LINE__);                     \
            onfail;                                                                   \
        }                                                                             \
    } while (0)

#define K_TRY(call, onfail)                                                           \
    do {                                                                              \
        int e__ = (call);                                                             \
        if (e__ != 0) {                                                               \
            fprintf(stderr, "[llmb200] %s failed: code %d%s%s (%s:%d)\n", #call, e__, \
                    e__ > 0 ? " " : "", e__ > 0 ? cudaGetErrorString((cudaError_t)e__) : "", \
                    __FILE__, __LINE__);                                              \
            onfail;                                                                   \
        }                                                                             \
    } while (0)

/* Convert the sub-matrix src[0..rows) x [col0, col0+cols) of a host fp32 matrix
 * with leading dimension ld into packed rows dst_row0 + r*dst_row_step of a
 * packed device matrix. Returns 0 on success. Asynchronous on g_rt.stream
 * except for the host-side staging copies. */
int llmb200_upload_packed(int wtype, const float *src, long long ld, int rows, int col0, int cols,
                          void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step);

/* Plain fp32 host -> new device allocation (returns NULL on failure). */
float *llmb200_upload_f32(const float *src, size_t n);
/* Plain fp32 host -> existing device memory through the staging buffers. */
int llmb200_upload_f32_into(float *d_dst, const float *src, size_t n);
/* Host fp32 -> existing device memory as binary16 (round to nearest even), through the staging buffers. */
int llmb200_upload_f16_into(void *d_dst, const float *src, size_t n);
/* A MetalBuf handle over device memory the caller keeps owning. metal_buf_ptr
 * on it returns a host copy refreshed by every call. */
MetalBuf *llmb200_buf_wrap(void *dev, size_t size);

/* The embedding table of an SFT state on the device (decode states built from it copy it). */
struct SFTState;
const float *llmb200_sft_device_emb(struct SFTState *s);
/* Full-parameter training changes the matrices a decode state copied from an SFT state: a count of the
 * changes, and the SFT state's weight views brought up to date before they are copied again. */
unsigned long long llmb200_sft_weights_version(struct SFTState *s);
void llmb200_sft_refresh_views(struct SFTState *s);

#endif
