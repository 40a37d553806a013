/*
 * Device runtime, buffers and weight containers of libllmb200 (host side, C).
 *
 * Stands in for the buffer half of the reference's dispatch shim
 * (src/nn/fast_metal.m:75-247) and for its weight container
 * (src/nn/wmat.c:47-156). The reference quantises on one CPU thread and hands
 * the bytes to a shared-storage buffer; here the fp32 rows go through a
 * double-buffered pinned staging area to the GPU and are quantised there by
 * b200_q8_pack / b200_f16_pack, which reproduce the CPU quantiser bit for bit.
 * There is no CPU path: without a usable CUDA device every entry point fails.
 */
#include "internal.h"
#include "../../include/llmb200_train_kernels.h"

#include <stdlib.h>
#include <string.h>

llmb200_runtime g_rts[LLMB200_MAX_DEVICES] = {{0}};

int fast_metal_init(void)
{
    if (g_rt.refs > 0) { g_rt.refs++; return 0; }
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        fprintf(stderr, "[llmb200] no CUDA device available (%s); this library has no CPU path\n",
                e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
        return -1;
    }
    CU_TRY(cudaGetDevice(&g_rt.device), return -1);
    CU_TRY(cudaStreamCreateWithFlags(&g_rt.stream, cudaStreamNonBlocking), return -1);
    for (int i = 0; i < 2; ++i) {
        CU_TRY(cudaMallocHost((void **)&g_rt.h_stage[i], LLMB200_STAGE_BYTES), return -1);
        CU_TRY(cudaMalloc((void **)&g_rt.d_stage[i], LLMB200_STAGE_BYTES), return -1);
        CU_TRY(cudaEventCreateWithFlags(&g_rt.stage_done[i], cudaEventDisableTiming), return -1);
    }
    g_rt.stage_next = 0;
    g_rt.refs = 1;
    return 0;
}

void fast_metal_shutdown(void)
{
    if (g_rt.refs <= 0) return;
    if (--g_rt.refs > 0) return;
    cudaStreamSynchronize(g_rt.stream);
    for (int i = 0; i < 2; ++i) {
        cudaFreeHost(g_rt.h_stage[i]);
        cudaFree(g_rt.d_stage[i]);
        cudaEventDestroy(g_rt.stage_done[i]);
    }
    cudaStreamDestroy(g_rt.stream);
    memset(&g_rt, 0, sizeof(g_rt));
}

void metal_flush(void)
{
    if (g_rt.refs > 0) CU_TRY(cudaStreamSynchronize(g_rt.stream), return);
}

/* ---------------------------------------------------------------- buffers */

static MetalBuf *mb_new(int kind, size_t size)
{
    MetalBuf *b = calloc(1, sizeof(MetalBuf));
    if (!b) return NULL;
    b->kind = kind;
    b->size = size;
    cudaError_t e = kind == MB_SHARED ? cudaMallocManaged(&b->dev, size ? size : 1, cudaMemAttachGlobal)
                                      : cudaMalloc(&b->dev, size ? size : 1);
    if (e != cudaSuccess) {
        fprintf(stderr, "[llmb200] allocating %zu bytes failed: %s\n", size, cudaGetErrorString(e));
        free(b);
        return NULL;
    }
    return b;
}

MetalBuf *metal_buf_create(size_t size)
{
    if (g_rt.refs <= 0 && fast_metal_init() != 0) return NULL;
    MetalBuf *b = mb_new(MB_SHARED, size);
    if (b) memset(b->dev, 0, size);
    return b;
}

MetalBuf *metal_buf_from_data(const void *data, size_t sz)
{
    if (!data) return NULL;
    MetalBuf *b = metal_buf_create(sz);
    if (b) memcpy(b->dev, data, sz);
    return b;
}

void metal_buf_free(MetalBuf *b)
{
    if (!b) return;
    if (b->dev && !b->borrowed) cudaFree(b->dev);
    free(b->host_mirror);
    free(b);
}

void *metal_buf_ptr(MetalBuf *b)
{
    if (!b) return NULL;
    if (b->kind == MB_SHARED) {
        /* the host may touch unified memory only when no kernel is using it */
        metal_flush();
        return b->dev;
    }
    if (b->host_mirror && b->kind != MB_DEVICE) return b->host_mirror;
    if (b->kind == MB_Q8) {
        /* rebuild the reference's 34-byte block stream from the packed rows */
        size_t bytes = (size_t)b->rows * (b->cols / 32) * 34;
        void *d_blocks = NULL;
        CU_TRY(cudaMalloc(&d_blocks, bytes ? bytes : 1), return NULL);
        b->host_mirror = malloc(bytes ? bytes : 1);
        int rc = b200_q8_unpack_blocks(b->dev, b->row_stride, b->rows, b->cols, d_blocks, g_rt.stream);
        if (rc == 0 && b->host_mirror)
            rc = (int)cudaMemcpyAsync(b->host_mirror, d_blocks, bytes, cudaMemcpyDeviceToHost, g_rt.stream);
        if (rc == 0) rc = (int)cudaStreamSynchronize(g_rt.stream);
        cudaFree(d_blocks);
        if (rc != 0 || !b->host_mirror) { free(b->host_mirror); b->host_mirror = NULL; }
        return b->host_mirror;
    }
    if (b->kind == MB_F16) {
        /* the conversion ran on the library's own (non-blocking) stream: a copy on the default stream does not wait for it */
        metal_flush();
        size_t row_bytes = (size_t)b->cols * 2;
        b->host_mirror = malloc((size_t)b->rows * row_bytes + 1);
        if (!b->host_mirror) return NULL;
        cudaError_t e = cudaMemcpy2D(b->host_mirror, row_bytes, b->dev, (size_t)b->row_stride, row_bytes,
                                     (size_t)b->rows, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { free(b->host_mirror); b->host_mirror = NULL; }
        return b->host_mirror;
    }
    /* plain device memory: the copy is refreshed on every call */
    metal_flush();
    if (!b->host_mirror) b->host_mirror = malloc(b->size ? b->size : 1);
    if (b->host_mirror && cudaMemcpy(b->host_mirror, b->dev, b->size, cudaMemcpyDeviceToHost) != cudaSuccess) {
        free(b->host_mirror);
        b->host_mirror = NULL;
    }
    return b->host_mirror;
}

/* ---------------------------------------------------------------- dispatches on buffers */

/* Size checks against the buffers' own sizes: a wrong count would otherwise write past a device allocation.
 * A refused dispatch says so; the caller's next read of the output sees it unchanged. */
static int buf_holds(const MetalBuf *b, size_t bytes) { return b && b->dev && b->size >= bytes; }

void metal_enqueue_scale(MetalBuf *x, float alpha, int n)
{
    if (n <= 0) return;
    if (!buf_holds(x, (size_t)n * 4)) {
        fprintf(stderr, "[llmb200] metal_enqueue_scale: buffer smaller than %d floats\n", n);
        return;
    }
    K_TRY(b200_scale((float *)x->dev, alpha, (size_t)n, g_rt.stream), return);
}

void metal_enqueue_grpo_policy_grad(MetalBuf *logits, MetalBuf *actions, MetalBuf *old_lp, MetalBuf *advs, MetalBuf *new_lp,
                                    MetalBuf *dlogits, int N, int V, float clip_eps)
{
    if (N <= 0 || V <= 0) return;
    const size_t nv = (size_t)N * (size_t)V * 4, n4 = (size_t)N * 4;
    if (!buf_holds(logits, nv) || !buf_holds(dlogits, nv) || !buf_holds(actions, n4) || !buf_holds(old_lp, n4) ||
        !buf_holds(advs, n4) || !buf_holds(new_lp, n4)) {
        fprintf(stderr, "[llmb200] metal_enqueue_grpo_policy_grad: a buffer is missing or smaller than N = %d, V = %d need\n", N, V);
        return;
    }
    K_TRY(b200_grpo_policy_grad((const float *)logits->dev, (const uint32_t *)actions->dev, (const float *)old_lp->dev,
                                (const float *)advs->dev, (float *)new_lp->dev, (float *)dlogits->dev, N, V, clip_eps,
                                g_rt.stream), return);
}

/* ---------------------------------------------------------------- upload */

int llmb200_upload_packed(int wtype, const float *src, long long ld, int rows, int col0, int cols,
                          void *d_dst, long long dst_row_stride, int dst_row0, int dst_row_step)
{
    if (!src || !d_dst || rows < 0 || cols <= 0) return B200_E_BADARG;
    const size_t row_floats = (size_t)cols;
    long long rows_per_chunk = (long long)(LLMB200_STAGE_BYTES / (row_floats * sizeof(float)));
    if (rows_per_chunk < 1) return B200_E_TOOLARGE;
    for (long long r = 0; r < rows; r += rows_per_chunk) {
        const int nr = (int)((rows - r) < rows_per_chunk ? (rows - r) : rows_per_chunk);
        const int sb = g_rt.stage_next;
        g_rt.stage_next ^= 1;
        CU_TRY(cudaEventSynchronize(g_rt.stage_done[sb]), return -100);
        if (col0 == 0 && ld == cols) {
            memcpy(g_rt.h_stage[sb], src + (size_t)r * ld, (size_t)nr * row_floats * sizeof(float));
        } else {
            for (int i = 0; i < nr; ++i)
                memcpy(g_rt.h_stage[sb] + (size_t)i * row_floats, src + (size_t)(r + i) * ld + col0,
                       row_floats * sizeof(float));
        }
        CU_TRY(cudaMemcpyAsync(g_rt.d_stage[sb], g_rt.h_stage[sb], (size_t)nr * row_floats * sizeof(float),
                               cudaMemcpyHostToDevice, g_rt.stream), return -101);
        int rc = wtype == B200_WT_Q8
            ? b200_q8_pack(g_rt.d_stage[sb], cols, nr, cols, d_dst, dst_row_stride,
                           dst_row0 + (int)r * dst_row_step, dst_row_step, g_rt.stream)
            : b200_f16_pack(g_rt.d_stage[sb], cols, nr, cols, d_dst, dst_row_stride,
                            dst_row0 + (int)r * dst_row_step, dst_row_step, g_rt.stream);
        if (rc != 0) return rc;
        CU_TRY(cudaEventRecord(g_rt.stage_done[sb], g_rt.stream), return -102);
    }
    return 0;
}

int llmb200_upload_f32_into(float *d, const float *src, size_t n)
{
    const size_t chunk = LLMB200_STAGE_BYTES / sizeof(float);
    for (size_t o = 0; o < n; o += chunk) {
        const size_t m = (n - o) < chunk ? (n - o) : chunk;
        const int sb = g_rt.stage_next;
        g_rt.stage_next ^= 1;
        CU_TRY(cudaEventSynchronize(g_rt.stage_done[sb]), return -100);
        memcpy(g_rt.h_stage[sb], src + o, m * sizeof(float));
        CU_TRY(cudaMemcpyAsync(d + o, g_rt.h_stage[sb], m * sizeof(float), cudaMemcpyHostToDevice, g_rt.stream),
               return -101);
        CU_TRY(cudaEventRecord(g_rt.stage_done[sb], g_rt.stream), return -102);
    }
    return 0;
}

float *llmb200_upload_f32(const float *src, size_t n)
{
    float *d = NULL;
    CU_TRY(cudaMalloc((void **)&d, (n ? n : 1) * sizeof(float)), return NULL);
    if (llmb200_upload_f32_into(d, src, n) != 0) { cudaFree(d); return NULL; }
    return d;
}

/* host fp32 -> device binary16 (round to nearest even) through the runtime's staging buffers */
int llmb200_upload_f16_into(void *d_dst, const float *src, size_t n)
{
    const size_t chunk = LLMB200_STAGE_BYTES / sizeof(float);
    for (size_t o = 0; o < n; o += chunk) {
        const size_t m = (n - o) < chunk ? (n - o) : chunk;
        const int sb = g_rt.stage_next;
        g_rt.stage_next ^= 1;
        CU_TRY(cudaEventSynchronize(g_rt.stage_done[sb]), return -100);
        memcpy(g_rt.h_stage[sb], src + o, m * sizeof(float));
        CU_TRY(cudaMemcpyAsync(g_rt.d_stage[sb], g_rt.h_stage[sb], m * sizeof(float), cudaMemcpyHostToDevice, g_rt.stream),
               return -101);
        int rc = b200_f32_to_f16(g_rt.d_stage[sb], m, 1.0f, (char *)d_dst + o * 2, g_rt.stream);
        if (rc) return rc;
        CU_TRY(cudaEventRecord(g_rt.stage_done[sb], g_rt.stream), return -102);
    }
    return 0;
}

MetalBuf *llmb200_buf_wrap(void *dev, size_t size)
{
    MetalBuf *b = calloc(1, sizeof(MetalBuf));
    if (!b) return NULL;
    b->kind = MB_DEVICE;
    b->dev = dev;
    b->size = size;
    b->borrowed = 1;
    return b;
}

/* ---------------------------------------------------------------- WMat */

static WMat *wmat_create(const float *src, int rows, int cols, int wtype)
{
    if (!src || rows <= 0 || cols <= 0 || (wtype == B200_WT_Q8 ? cols % 32 : cols % 8)) {
        fprintf(stderr, "[llmb200] wmat_create: unsupported shape %d x %d for %s\n", rows, cols,
                wtype == B200_WT_Q8 ? "Q8_0 (cols must be a multiple of 32)" : "F16 (cols must be a multiple of 8)");
        return NULL;
    }
    if (g_rt.refs <= 0 && fast_metal_init() != 0) return NULL;
    const size_t stride = b200_packed_row_stride(wtype, cols);
    MetalBuf *b = mb_new(wtype == B200_WT_Q8 ? MB_Q8 : MB_F16, stride * (size_t)rows);
    if (!b) return NULL;
    b->rows = rows; b->cols = cols; b->row_stride = (long long)stride;
    if (llmb200_upload_packed(wtype, src, cols, rows, 0, cols, b->dev, (long long)stride, 0, 1) != 0) {
        metal_buf_free(b);
        return NULL;
    }
    WMat *w = calloc(1, sizeof(WMat));
    if (!w) { metal_buf_free(b); return NULL; }
    w->mbuf = b; w->rows = rows; w->cols = cols; w->nb = wtype == B200_WT_Q8 ? cols / 32 : 0;
    return w;
}

WMat *wmat_create_q8(const float *src, int rows, int cols) { return wmat_create(src, rows, cols, B200_WT_Q8); }
WMat *wmat_create_f16(const float *src, int rows, int cols) { return wmat_create(src, rows, cols, B200_WT_F16); }
WMat *wmat_convert(const float *data, int rows, int cols, int use_fp16)
{
    return wmat_create(data, rows, cols, use_fp16 ? B200_WT_F16 : B200_WT_Q8);
}

void wmat_free(WMat *w)
{
    if (!w) return;
    metal_buf_free(w->mbuf);
    free(w);
}

MetalBuf *norm_upload(const float *gamma, int dim)
{
    return metal_buf_from_data(gamma, (size_t)dim * sizeof(float));
}

LayerW *layers_convert_upload(const LayerWeightRef *refs, int n_layers, int use_fp16)
{
    if (!refs || n_layers <= 0) return NULL;
    LayerW *layers = calloc((size_t)n_layers, sizeof(LayerW));
    if (!layers) return NULL;
    for (int i = 0; i < n_layers; ++i) {
        const LayerWeightRef *r = &refs[i];
        LayerW *lw = &layers[i];
        const WeightRef *src[7] = {&r->q_proj, &r->k_proj, &r->v_proj, &r->o_proj, &r->gate_proj, &r->up_proj, &r->down_proj};
        WMat **dst[7] = {&lw->q_proj, &lw->k_proj, &lw->v_proj, &lw->o_proj, &lw->gate_proj, &lw->up_proj, &lw->down_proj};
        for (int m = 0; m < 7; ++m) {
            *dst[m] = wmat_convert(src[m]->data, src[m]->rows, src[m]->cols, use_fp16);
            if (!*dst[m]) { layers_free(layers, n_layers); return NULL; }
        }
        lw->input_norm_g = norm_upload(r->input_norm_g, r->d_model);
        lw->post_attn_norm_g = norm_upload(r->post_attn_norm_g, r->d_model);
        if (r->pre_ff_norm_g) lw->pre_ff_norm_g = norm_upload(r->pre_ff_norm_g, r->d_model);
        if (r->post_ff_norm_g) lw->post_ff_norm_g = norm_upload(r->post_ff_norm_g, r->d_model);
        if (r->q_norm_g) lw->q_norm_g = norm_upload(r->q_norm_g, r->head_dim);
        if (r->k_norm_g) lw->k_norm_g = norm_upload(r->k_norm_g, r->head_dim);
        if ((i + 1) % 6 == 0) printf("  Converted layers 0-%d\n", i);
    }
    return layers;
}

void layers_free(LayerW *layers, int n_layers)
{
    if (!layers) return;
    for (int i = 0; i < n_layers; ++i) {
        LayerW *lw = &layers[i];
        wmat_free(lw->q_proj); wmat_free(lw->k_proj); wmat_free(lw->v_proj); wmat_free(lw->o_proj);
        wmat_free(lw->gate_proj); wmat_free(lw->up_proj); wmat_free(lw->down_proj);
        metal_buf_free(lw->input_norm_g); metal_buf_free(lw->post_attn_norm_g);
        metal_buf_free(lw->pre_ff_norm_g); metal_buf_free(lw->post_ff_norm_g);
        metal_buf_free(lw->q_norm_g); metal_buf_free(lw->k_norm_g);
    }
    free(layers);
}
