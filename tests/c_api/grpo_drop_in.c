/*
 * The reference's GRPO step on top of the drop-in library: src/nn/fast_grpo.c runs unchanged
 * (oracle/_ref/libllmref_grpo.so, see oracle/grpo_caller.c) and everything it calls --
 * sft_state_create, inference_state_create_from_sft, inference_forward_token, forward_to_logits,
 * metal_enqueue_grpo_policy_grad, metal_enqueue_scale, sft_backward, sft_set_lora_grad,
 * sft_lora_update, sft_save_lora -- comes from the library the executable is linked with:
 *
 *     _bin/grpo_b200   libllmb200.so (the CUDA engines)
 *     _bin/grpo_ref    the reference's own engines over the CPU stand-in for its Metal layer
 *
 * Both write the same record file (argv[1]): per step the sampled tokens, their log-probabilities,
 * rewards, advantages and the LoRA gradients summed over the group; then the losses of two plain
 * sft_train_step calls on the same state and the adapter after them. argv[2] picks the mode: "lora" (default), "full" (grpo_state_create_full: every weight stepped by
 * SGD inside each completion's backward pass) or "full-accurate" (gradients accumulated in binary16 over the
 * group, one step at the end); the full-parameter modes go on with two sft_train_step calls on the same
 * state and record a sample of the saved checkpoint instead of an adapter. "gemma" and "gemma-full" are the
 * LoRA and the immediate full-parameter mode on a Gemma3 model (grpo_state_create_gemma3 / _gemma3_full);
 * "gemma-hd256" is the LoRA mode with Gemma3-1B's head layout (four query heads of 256 on one key/value head).
 * tests/golden/grpo_golden*.bin are the records of grpo_ref; the GPU test compares grpo_b200 with them.
 *
 * Exit codes: 0 ok, 3 the state could not be created (no CUDA device), 1 anything else.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nn/qwen3.h"
#include "nn/gemma3.h"
#include "nn/fast_sft.h"
#include "nn/fast_grpo.h"

/* oracle/grpo_caller.c */
int grpo_dbg_gen_len(const GRPOState *g, int i);
const uint32_t *grpo_dbg_tokens(const GRPOState *g, int i);
const float *grpo_dbg_logprobs(const GRPOState *g, int i);
float grpo_dbg_reward(const GRPOState *g, int i);
float grpo_dbg_advantage(const GRPOState *g, int i);
int grpo_dbg_n_grad_bufs(const GRPOState *g);
const float *grpo_dbg_accum_grad(const GRPOState *g, int b, int *size);
const float *grpo_dbg_new_logprobs(GRPOState *g);
SFTState *grpo_dbg_sft(GRPOState *g);

enum { GROUP = 4, MAX_GEN = 8, SEQ = 16, PROMPT = 8, RANK = 4, STEPS = 2 };
enum { K_REWARD = 1, K_LEN = 2, K_TOKENS = 3, K_LOGPROBS = 4, K_REWARDS = 5, K_ADVANTAGES = 6, K_GRADS = 7, K_NEW_LP = 8,
       K_ADAPTER = 9, K_SFT_LOSS = 10, K_CKPT_HEAD = 11, K_CKPT_SAMPLE = 12, K_CKPT_SUMS = 13 };
enum { CKPT_STRIDE = 97 };

static FILE *out;
static void section(int kind, const float *v, int n)
{
    const int32_t head[2] = {kind, n};
    fwrite(head, 4, 2, out);
    fwrite(v, 4, (size_t)n, out);
}

int main(int argc, char **argv)
{
    if (argc < 2) { fprintf(stderr, "usage: %s <record file> [lora|full|full-accurate|gemma|gemma-full|gemma-hd256] [seed]\n", argv[0]); return 1; }
    const char *mode = argc > 2 ? argv[2] : "lora";
    const int gemma = strncmp(mode, "gemma", 5) == 0;
    const int full = strncmp(mode, "full", 4) == 0 || strcmp(mode, "gemma-full") == 0, accurate = strcmp(mode, "full-accurate") == 0;
    srand(11);
    Qwen3Config cfg = { .n_layers = 2, .d_model = 256, .n_q_heads = 4, .n_kv_heads = 2, .head_dim = 64,
                        .intermediate_size = 512, .vocab_size = 64, .rope_theta = 1e6f, .rms_norm_eps = 1e-6f };
    Gemma3Config gcfg = { .n_layers = 2, .d_model = 256, .n_q_heads = 4, .n_kv_heads = 2, .head_dim = 64,
                          .intermediate_size = 512, .vocab_size = 64, .sliding_window = 512, .local_rope_theta = 1e4f,
                          .global_rope_theta = 1e6f, .rms_norm_eps = 1e-6f };
    if (strcmp(mode, "gemma-hd256") == 0) { gcfg.head_dim = 256; gcfg.n_kv_heads = 1; }
    Qwen3Model *model = gemma ? NULL : qwen3_create(cfg);
    Gemma3Model *gmodel = gemma ? gemma3_create(gcfg) : NULL;
    if (!model && !gmodel) return 1;
    GRPOConfig gc = { .group_size = GROUP, .max_gen_len = MAX_GEN, .temperature = 0.7f, .clip_eps = 0.2f,
                      .reward = "combined", .accurate = accurate };
    GRPOState *g = gemma ? (full ? grpo_state_create_gemma3_full(gmodel, gc, SEQ, NULL) : grpo_state_create_gemma3(gmodel, gc, SEQ, RANK, 8.0f, NULL))
                         : (full ? grpo_state_create_full(model, gc, SEQ, NULL) : grpo_state_create(model, gc, SEQ, RANK, 8.0f, NULL));
    if (!g) return 3;
    out = fopen(argv[1], "wb");
    if (!out) return 1;

    /* The sampler draws from rand(). The default seed is one whose rewards differ inside the group in both
     * steps (repeated bigrams, completions ending early on the EOS id 1: the gradients are not all zero) and whose draws stay
     * clear of the far tail of the distribution: multinomial sampling is ill-conditioned there -- a draw that
     * lands between two tokens of probability 1e-3 picks the other one at a logit difference far inside the
     * decode path's 1e-2 tolerance (3 of 42 compared steps over seven seeds and three modes did). */
    srand(argc > 3 ? (unsigned)atoi(argv[3]) : gemma ? 13u : 4u);
    uint32_t prompt[PROMPT];
    for (int i = 0; i < PROMPT; ++i) prompt[i] = (uint32_t)(2 + rand() % (cfg.vocab_size - 2));
    float buf[GROUP * MAX_GEN];
    for (int step = 0; step < STEPS; ++step) {
        const float mean_reward = grpo_train_step(g, prompt, PROMPT, 1e-2f);
        if (!isfinite(mean_reward)) { fprintf(stderr, "GRPO_DROP_IN failed: mean reward not finite\n"); return 1; }
        section(K_REWARD, &mean_reward, 1);
        for (int i = 0; i < GROUP; ++i) buf[i] = (float)grpo_dbg_gen_len(g, i);
        section(K_LEN, buf, GROUP);
        memset(buf, 0, sizeof buf);
        for (int i = 0; i < GROUP; ++i)
            for (int t = 0; t < grpo_dbg_gen_len(g, i); ++t) buf[i * MAX_GEN + t] = (float)grpo_dbg_tokens(g, i)[t];
        section(K_TOKENS, buf, GROUP * MAX_GEN);
        memset(buf, 0, sizeof buf);
        for (int i = 0; i < GROUP; ++i)
            for (int t = 0; t < grpo_dbg_gen_len(g, i); ++t) buf[i * MAX_GEN + t] = grpo_dbg_logprobs(g, i)[t];
        section(K_LOGPROBS, buf, GROUP * MAX_GEN);
        for (int i = 0; i < GROUP; ++i) buf[i] = grpo_dbg_reward(g, i);
        section(K_REWARDS, buf, GROUP);
        for (int i = 0; i < GROUP; ++i) buf[i] = grpo_dbg_advantage(g, i);
        section(K_ADVANTAGES, buf, GROUP);
        for (int b = 0; b < grpo_dbg_n_grad_bufs(g); ++b) {
            int n = 0;
            const float *a = grpo_dbg_accum_grad(g, b, &n);
            section(K_GRADS, a, n);
        }
        section(K_NEW_LP, grpo_dbg_new_logprobs(g), SEQ);
    }

    char path[512];
    if (!full) {
        /* two plain LoRA-SFT steps on the same state (sft_train_step: embedding gather with the model's embedding
         * scale, loss, backward, clip + AdamW), then the adapter as the reference saves it (12-byte header, matrices) */
        SFTState *sft = grpo_dbg_sft(g);
        uint32_t in[SEQ], tg[SEQ];
        const int V = gemma ? gcfg.vocab_size : cfg.vocab_size;
        for (int i = 0; i < SEQ; ++i) { in[i] = (uint32_t)(rand() % V); tg[i] = (uint32_t)(rand() % V); }
        float loss[2];
        for (int k = 0; k < 2; ++k) loss[k] = sft_train_step(sft, in, tg, 1e-3f);
        section(K_SFT_LOSS, loss, 2);
        snprintf(path, sizeof path, "%s.lora", argv[1]);
        grpo_save_lora(g, path);
        FILE *fp = fopen(path, "rb");
        if (!fp) { fprintf(stderr, "GRPO_DROP_IN failed: adapter file\n"); return 1; }
        fseek(fp, 0, SEEK_END);
        const long bytes = ftell(fp) - 12;
        fseek(fp, 12, SEEK_SET);
        float *w = malloc((size_t)bytes);
        if (!w || fread(w, 1, (size_t)bytes, fp) != (size_t)bytes) { fprintf(stderr, "GRPO_DROP_IN failed: adapter read\n"); return 1; }
        fclose(fp);
        remove(path);
        section(K_ADAPTER, w, (int)(bytes / 4));
        free(w);
    } else {
        /* two plain full-parameter SFT steps on the same state (sft_train_step, SGD inside the backward pass) */
        SFTState *sft = grpo_dbg_sft(g);
        uint32_t in[SEQ], tg[SEQ];
        for (int i = 0; i < SEQ; ++i) { in[i] = (uint32_t)(rand() % cfg.vocab_size); tg[i] = (uint32_t)(rand() % cfg.vocab_size); }
        float loss[2];
        for (int k = 0; k < 2; ++k) loss[k] = sft_train_step(sft, in, tg, 5e-3f);
        section(K_SFT_LOSS, loss, 2);
        /* the checkpoint as the reference saves it: nine header words, then every matrix in binary16 */
        snprintf(path, sizeof path, "%s.ckpt", argv[1]);
        grpo_save_full_checkpoint(g, path);
        FILE *fp = fopen(path, "rb");
        if (!fp) { fprintf(stderr, "GRPO_DROP_IN failed: checkpoint file\n"); return 1; }
        uint32_t head[9];
        if (fread(head, 4, 9, fp) != 9) { fprintf(stderr, "GRPO_DROP_IN failed: checkpoint header\n"); return 1; }
        float headf[9];
        for (int i = 0; i < 9; ++i) headf[i] = (float)(head[i] & 0xffffffu);     /* exact in fp32 */
        section(K_CKPT_HEAD, headf, 9);
        fseek(fp, 0, SEEK_END);
        const long n = (ftell(fp) - 36) / 2;
        fseek(fp, 36, SEEK_SET);
        _Float16 *h = malloc((size_t)n * 2);
        if (!h || fread(h, 2, (size_t)n, fp) != (size_t)n) { fprintf(stderr, "GRPO_DROP_IN failed: checkpoint read\n"); return 1; }
        fclose(fp);
        remove(path);
        const long ns = (n + CKPT_STRIDE - 1) / CKPT_STRIDE;
        float *smp = malloc((size_t)ns * 4);
        double sum = 0, sq = 0;
        for (long i = 0; i < n; ++i) { const double v = (double)(float)h[i]; sum += v; sq += v * v; if (i % CKPT_STRIDE == 0) smp[i / CKPT_STRIDE] = (float)h[i]; }
        section(K_CKPT_SAMPLE, smp, (int)ns);
        const float sums[3] = { (float)n, (float)sum, (float)sq };
        section(K_CKPT_SUMS, sums, 3);
        free(h); free(smp);
    }
    fclose(out);

    if (sft_is_full_param(grpo_dbg_sft(g)) != full) { fprintf(stderr, "GRPO_DROP_IN failed: sft_is_full_param\n"); return 1; }
    grpo_state_free(g);
    if (model) qwen3_free(model);
    if (gmodel) gemma3_free(gmodel);
    printf("GRPO_DROP_IN ok\n");
    return 0;
}
