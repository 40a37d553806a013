/*
 * llmb200_wmat.h -- weight containers and device buffers at the drop-in boundary.
 *
 * Declares, with the reference's own symbol names and structure layouts, the
 * part of llm.metal's weight/buffer interface that the decode and SFT engines
 * are built on. libllmb200.so exports every function below; a program that was
 * compiled against the reference's src/nn/wmat.h and src/nn/fast_metal.h links
 * against it unchanged.
 *
 *   MetalBuf, metal_buf_*      replaces src/nn/fast_metal.h:12-17 (src/nn/fast_metal.m:197-217)
 *   fast_metal_init/shutdown   replaces src/nn/fast_metal.h:8-9   (src/nn/fast_metal.m:75-195)
 *   metal_flush                replaces src/nn/fast_metal.h:84    (src/nn/fast_metal.m:239-247)
 *   metal_enqueue_scale, metal_enqueue_grpo_policy_grad
 *                              replace src/nn/fast_metal.h:124, :179-181 (src/nn/fast_metal.m:722-731, 963-981):
 *                              the two dispatches a caller outside the engines issues itself (the GRPO
 *                              step, src/nn/fast_grpo.c:449-457); every other dispatch stays inside the engines
 *   WMat, LayerW, WeightRef, LayerWeightRef, ModelType   src/nn/wmat.h:10-56
 *   wmat_create_q8/f16, wmat_free, layers_convert_upload, layers_free,
 *   wmat_convert, norm_upload  replaces src/nn/wmat.c:47-156
 *
 * What differs underneath: a MetalBuf is CUDA memory on the current device.
 * Generic buffers (metal_buf_create/from_data) are unified-memory allocations,
 * so metal_buf_ptr() stays a pointer both the host and the kernels can use, as
 * on the reference's shared-storage buffers. Weight buffers made by wmat_* are
 * device-only and hold a repacked layout (see llmb200_kernels.h); for those,
 * metal_buf_ptr() materialises, on first use, a host copy in the reference's
 * canonical byte format (34-byte Q8_0 blocks / row-major binary16).
 */
#ifndef LLMB200_WMAT_H
#define LLMB200_WMAT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device runtime (reference counted, like the reference's global Metal state) ---- */
int  fast_metal_init(void);      /* 0 on success; selects the current CUDA device, creates the stream */
void fast_metal_shutdown(void);
void metal_flush(void);          /* wait for everything enqueued on the library's stream */

/* ---- buffers ---- */
typedef struct MetalBuf MetalBuf;
MetalBuf *metal_buf_create(size_t size);                     /* zero-filled */
MetalBuf *metal_buf_from_data(const void *data, size_t sz);  /* copies sz bytes in */
void      metal_buf_free(MetalBuf *b);                       /* NULL is accepted */
void     *metal_buf_ptr(MetalBuf *b);                        /* host-visible pointer */

/* ---- dispatches on buffers (asynchronous on the library's stream, like the reference's encoder) ---- */
void metal_enqueue_scale(MetalBuf *x, float alpha, int n);   /* x[i] *= alpha, fp32 */
/* One position per row of logits [N, V]: writes new_lp [N] and dlogits [N, V] (see llmb200_train_kernels.h). */
void metal_enqueue_grpo_policy_grad(MetalBuf *logits, MetalBuf *actions, MetalBuf *old_lp, MetalBuf *advs, MetalBuf *new_lp,
                                    MetalBuf *dlogits, int N, int V, float clip_eps);

/* ---- containers (layouts as in src/nn/wmat.h:10-56) ---- */
typedef enum { MODEL_QWEN3, MODEL_GEMMA3 } ModelType;

typedef struct WMat {
    MetalBuf *mbuf;
    int rows, cols, nb;          /* nb = cols/32 for Q8_0, 0 for F16 */
} WMat;

typedef struct {
    WMat *q_proj, *k_proj, *v_proj, *o_proj;
    WMat *gate_proj, *up_proj, *down_proj;
    MetalBuf *input_norm_g, *post_attn_norm_g;
    MetalBuf *pre_ff_norm_g, *post_ff_norm_g;   /* Gemma3 only, else NULL */
    MetalBuf *q_norm_g, *k_norm_g;              /* NULL when the model has no QK-norm */
} LayerW;

typedef struct { const float *data; int rows, cols; } WeightRef;

typedef struct {
    WeightRef q_proj, k_proj, v_proj, o_proj;
    WeightRef gate_proj, up_proj, down_proj;
    const float *input_norm_g;
    const float *post_attn_norm_g;
    const float *pre_ff_norm_g;
    const float *post_ff_norm_g;
    const float *q_norm_g;
    const float *k_norm_g;
    int d_model;
    int head_dim;
} LayerWeightRef;

/* ---- conversion + upload ---- */
/* fp32 [rows, cols] row-major -> Q8_0 (cols % 32 == 0): per 32 values
 * amax=max|x|, scale=amax/127 (fp32), d=binary16(scale) round-to-nearest-even,
 * q=clamp(roundf(x * (1.0f/scale)), -128, 127), all-zero block when scale==0.
 * Quantisation runs on the GPU and is bit-identical to src/nn/wmat.c:19-41. */
WMat *wmat_create_q8(const float *src, int rows, int cols);
/* fp32 -> binary16, round-to-nearest-even (src/nn/wmat.c:63-75). */
WMat *wmat_create_f16(const float *src, int rows, int cols);
void  wmat_free(WMat *w);
WMat *wmat_convert(const float *data, int rows, int cols, int use_fp16);
MetalBuf *norm_upload(const float *gamma, int dim);
/* Converts the seven matrices and up to six gamma vectors of every layer.
 * Returns a calloc'd array of n_layers LayerW (NULL on failure). */
LayerW *layers_convert_upload(const LayerWeightRef *refs, int n_layers, int use_fp16);
void    layers_free(LayerW *layers, int n_layers);

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_WMAT_H */
