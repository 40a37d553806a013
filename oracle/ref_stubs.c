/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Stand-ins for the two Objective-C translation units the reference's C files
 * link against, so that its CPU code path can be built and run without Metal:
 *
 *   src/core/metal_backend.h  metal_is_initialized() answers 0, which selects
 *                             the CPU branch of every layer (e.g.
 *                             src/nn/layers.c:136-150, 362-377); the dispatch
 *                             functions are then unreachable and abort.
 *   src/nn/fast_metal.h       the four metal_buf_* functions wmat.c uses,
 *                             backed by malloc.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int  metal_init(const char *p) { (void)p; return -1; }
void metal_cleanup(void) {}
int  metal_is_initialized(void) { return 0; }
void metal_synchronize(void) {}
void *metal_create_shared_buffer(size_t bytes) { return calloc(1, bytes ? bytes : 1); }
void  metal_free_buffer(void *b) { free(b); }
void *metal_buffer_contents(void *b) { return b; }

#define UNREACHABLE(name) void name(void) { fprintf(stderr, "oracle: " #name " reached on the CPU path\n"); abort(); }
UNREACHABLE(metal_matmul)
UNREACHABLE(metal_matmul_batched)
UNREACHABLE(metal_layer_norm_residual)
UNREACHABLE(metal_flash_attention)
UNREACHABLE(metal_flash_attention_backward)
UNREACHABLE(metal_layer_norm)
UNREACHABLE(metal_layer_norm_backward)
UNREACHABLE(metal_gelu)
UNREACHABLE(metal_gelu_backward)
UNREACHABLE(metal_rope)
UNREACHABLE(metal_rope_backward)
UNREACHABLE(metal_embedding)
UNREACHABLE(metal_embedding_backward)
UNREACHABLE(metal_softmax_ce_loss)
UNREACHABLE(metal_adamw_update)
UNREACHABLE(metal_add)
UNREACHABLE(metal_mul)
UNREACHABLE(metal_rms_norm)
UNREACHABLE(metal_rms_norm_backward)
UNREACHABLE(metal_silu)
UNREACHABLE(metal_silu_backward)
UNREACHABLE(metal_lora_forward)
UNREACHABLE(metal_dequantize_4bit)

typedef struct MetalBuf { void *p; size_t n; } MetalBuf;
MetalBuf *metal_buf_create(size_t size)
{
    MetalBuf *b = malloc(sizeof(*b));
    b->p = calloc(1, size ? size : 1); b->n = size;
    return b;
}
MetalBuf *metal_buf_from_data(const void *data, size_t sz)
{
    MetalBuf *b = metal_buf_create(sz);
    memcpy(b->p, data, sz);
    return b;
}
void  metal_buf_free(MetalBuf *b) { if (b) { free(b->p); free(b); } }
void *metal_buf_ptr(MetalBuf *b) { return b ? b->p : NULL; }
