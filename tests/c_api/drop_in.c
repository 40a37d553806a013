/*
 * A caller of the reference's fast engines, compiled against the reference's OWN headers
 * (src/nn/qwen3.h, src/nn/fast_inference.h, src/nn/fast_sft.h) and linked against libllmb200.so:
 * the drop-in claim as a program. It does what the reference's main.c does around these calls
 * (run_generate main.c:530-655, run_sft main.c:366-524): build a Qwen3Model with the reference's
 * qwen3_create, hand it to inference_state_create / inference_generate and to sft_state_create /
 * sft_train_step, take a decode state from the SFT state, save the adapter.
 *
 * The model comes from the reference's own C code (oracle/_ref/libllmref.so, linked second so that the
 * engine symbols resolve to libllmb200.so); the same library's CPU decode is the checker for the tokens.
 *
 *     make -C tests/c_api            (where the reference tree is mounted)
 *     tests/c_api/_bin/drop_in       prints "DROP_IN ok" and exits 0; without a GPU it exits 3 after
 *                                    the library's own "no CUDA device" message
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>

#include "nn/qwen3.h"
#include "nn/fast_inference.h"
#include "nn/fast_sft.h"

/* the CPU checker in oracle/ref_driver.c */
void ref_requant_qwen3(Qwen3Model *m, int use_fp16);
int ref_qwen3_generate(Qwen3Model *m, const uint32_t *prompt, int P, uint32_t *out, int max_gen, int max_seq,
                       const int *eos, int n_eos, float *logits, double *ms);

#define P 8
#define G 16
#define N 16

static int fail(const char *what) { fprintf(stderr, "DROP_IN failed: %s\n", what); return 1; }

int main(void)
{
    srand(7);
    Qwen3Config cfg = { .n_layers = 2, .d_model = 256, .n_q_heads = 4, .n_kv_heads = 2, .head_dim = 64,
                        .intermediate_size = 512, .vocab_size = 1024, .rope_theta = 1e6f, .rms_norm_eps = 1e-6f };
    Qwen3Model *model = qwen3_create(cfg);
    if (!model) return fail("qwen3_create");

    uint32_t prompt[P], out[G], want[G];
    for (int i = 0; i < P; ++i) prompt[i] = (uint32_t)(rand() % cfg.vocab_size);

    /* never stop on a token: the reference's own way, a config.json next to the model */
    char dir[] = "/tmp/llmb200_dropin_XXXXXX";
    if (!mkdtemp(dir)) return fail("mkdtemp");
    char path[256];
    snprintf(path, sizeof path, "%s/config.json", dir);
    FILE *fp = fopen(path, "w");
    if (!fp) return fail("config.json");
    fputs("{\"eos_token_id\": -1}\n", fp);
    fclose(fp);

    /* ---- decode: Q8_0 and F16 through the reference's API ---- */
    for (int use_fp16 = 0; use_fp16 < 2; ++use_fp16) {
        InferenceState *st = inference_state_create(model, 64, use_fp16);
        if (!st) return 3;
        inference_state_load_eos(st, dir);
        if (inference_state_model_type(st) != MODEL_QWEN3 || inference_state_vocab_size(st) != cfg.vocab_size)
            return fail("state accessors");
        int n = inference_generate(st, prompt, P, out, G);
        if (n != G) return fail("inference_generate count");
        /* logits through the per-token entry point */
        inference_state_reset(st);
        const float *lg = NULL;
        for (int i = 0; i < P; ++i) lg = inference_forward_token(st, (int)prompt[i]);
        int am = 0;
        for (int v = 1; v < cfg.vocab_size; ++v) if (lg[v] > lg[am]) am = v;
        if ((uint32_t)am != out[0]) return fail("forward_token argmax != first generated token");
        inference_state_free(st);

        /* the checker: the reference's CPU layers on the same (requantised) weights */
        Qwen3Model *copy = qwen3_create(cfg);
        if (!copy) return fail("qwen3_create (copy)");
        for (int l = 0; l < cfg.n_layers; ++l) {
            Qwen3Block *a = model->blocks[l], *b = copy->blocks[l];
            memcpy(b->attn->q_proj->weight->data, a->attn->q_proj->weight->data, sizeof(float) * a->attn->q_proj->weight->size);
            memcpy(b->attn->k_proj->weight->data, a->attn->k_proj->weight->data, sizeof(float) * a->attn->k_proj->weight->size);
            memcpy(b->attn->v_proj->weight->data, a->attn->v_proj->weight->data, sizeof(float) * a->attn->v_proj->weight->size);
            memcpy(b->attn->o_proj->weight->data, a->attn->o_proj->weight->data, sizeof(float) * a->attn->o_proj->weight->size);
            memcpy(b->gate_proj->weight->data, a->gate_proj->weight->data, sizeof(float) * a->gate_proj->weight->size);
            memcpy(b->up_proj->weight->data, a->up_proj->weight->data, sizeof(float) * a->up_proj->weight->size);
            memcpy(b->down_proj->weight->data, a->down_proj->weight->data, sizeof(float) * a->down_proj->weight->size);
            memcpy(b->input_norm->gamma->data, a->input_norm->gamma->data, sizeof(float) * a->input_norm->gamma->size);
            memcpy(b->post_attn_norm->gamma->data, a->post_attn_norm->gamma->data, sizeof(float) * a->post_attn_norm->gamma->size);
            memcpy(b->attn->q_norm->gamma->data, a->attn->q_norm->gamma->data, sizeof(float) * a->attn->q_norm->gamma->size);
            memcpy(b->attn->k_norm->gamma->data, a->attn->k_norm->gamma->data, sizeof(float) * a->attn->k_norm->gamma->size);
        }
        memcpy(copy->token_emb->weight->data, model->token_emb->weight->data, sizeof(float) * model->token_emb->weight->size);
        memcpy(copy->lm_head->weight->data, model->lm_head->weight->data, sizeof(float) * model->lm_head->weight->size);
        memcpy(copy->final_norm->gamma->data, model->final_norm->gamma->data, sizeof(float) * model->final_norm->gamma->size);
        ref_requant_qwen3(copy, use_fp16);
        if (ref_qwen3_generate(copy, prompt, P, want, G, 64, NULL, 0, NULL, NULL) != G) return fail("checker count");
        qwen3_free(copy);
        for (int i = 0; i < G; ++i)
            if (out[i] != want[i]) {
                fprintf(stderr, "token %d: engine %u, reference CPU %u (%s)\n", i, out[i], want[i], use_fp16 ? "F16" : "Q8_0");
                return fail("tokens differ");
            }
        printf("decode %s: %d tokens identical to the reference's CPU path\n", use_fp16 ? "F16" : "Q8_0", G);
    }

    /* ---- the one-call form ---- */
    if (qwen3_generate_fast(model, prompt, P, out, 4, 64, 0) < 1) return fail("qwen3_generate_fast");

    /* ---- LoRA-SFT, then a decode state on the same device weights ---- */
    SFTState *sft = sft_state_create(model, N, 4, 8.0f);
    if (!sft) return fail("sft_state_create");
    uint32_t in[N], tg[N];
    for (int i = 0; i < N; ++i) { in[i] = (uint32_t)(rand() % cfg.vocab_size); tg[i] = (uint32_t)(rand() % cfg.vocab_size); }
    float first = 0, last = 0;
    for (int step = 0; step < 4; ++step) {
        last = sft_train_step(sft, in, tg, 1e-2f);
        if (step == 0) first = last;
        if (!isfinite(last)) return fail("loss not finite");
    }
    if (!(last < first)) return fail("loss did not fall on a repeated batch");
    if (sft_get_step_count(sft) != 4 || sft_get_n_lora_grad_bufs(sft) != 4 * cfg.n_layers || sft_get_seq_len(sft) != N)
        return fail("sft accessors");
    if (sft_get_n_q_heads(sft) != cfg.n_q_heads || sft_get_head_dim(sft) != cfg.head_dim || !sft_get_layers(sft) ||
        sft_get_lm_head(sft)->rows != cfg.vocab_size)
        return fail("weight-sharing accessors");
    InferenceState *shared = inference_state_create_from_sft(sft, 64);
    if (!shared) return fail("inference_state_create_from_sft");
    inference_state_load_eos(shared, dir);
    if (inference_generate(shared, prompt, P, out, G) != G) return fail("generate on the shared state");
    inference_state_free(shared);
    snprintf(path, sizeof path, "%s/adapter.lora", dir);
    sft_save_lora(sft, path);
    struct stat sb;
    const long want_bytes = 12 + 4L * cfg.n_layers * (2 * 4 * cfg.d_model + 4 * (cfg.n_q_heads + cfg.n_kv_heads) * cfg.head_dim);
    if (stat(path, &sb) != 0 || sb.st_size != want_bytes) return fail("adapter file size");
    printf("sft: loss %.4f -> %.4f over 4 steps; adapter %ld bytes\n", first, last, (long)sb.st_size);
    sft_state_free(sft);
    qwen3_free(model);
    printf("DROP_IN ok\n");
    return 0;
}
