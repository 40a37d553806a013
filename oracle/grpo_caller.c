/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * The reference's GRPO loop (src/nn/fast_grpo.c, unmodified, compiled where it lies) as a shared
 * library with its engine calls left undefined: whatever the executable links next provides
 * sft_*, inference_*, metal_buf_* and the two metal_enqueue_* dispatches the loop issues itself
 * (fast_grpo.c:449-457) -- the reference's own engines over the CPU stand-in for its Metal layer
 * (_ref/libllmref_fast.so), or libllmb200.so. The loop is a CALLER of the path, like main.c; running
 * it unchanged on both sides is the parity test of the GRPO step.
 *
 * GRPOState is private to that file, so the few read-only views a test needs are added here.
 */
#include "nn/fast_grpo.c"

int grpo_dbg_group_size(const GRPOState *g) { return g->cfg.group_size; }
int grpo_dbg_max_gen_len(const GRPOState *g) { return g->cfg.max_gen_len; }
int grpo_dbg_gen_len(const GRPOState *g, int i) { return g->gen_lengths[i]; }
const uint32_t *grpo_dbg_tokens(const GRPOState *g, int i) { return g->gen_tokens[i]; }
const float *grpo_dbg_logprobs(const GRPOState *g, int i) { return g->gen_logprobs[i]; }
float grpo_dbg_reward(const GRPOState *g, int i) { return g->rewards[i]; }
float grpo_dbg_advantage(const GRPOState *g, int i) { return g->advantages[i]; }
int grpo_dbg_n_grad_bufs(const GRPOState *g) { return g->n_grad_bufs; }
/* the LoRA gradients summed over the group (what the step hands to sft_set_lora_grad) */
const float *grpo_dbg_accum_grad(const GRPOState *g, int b, int *size) { if (size) *size = g->grad_buf_sizes[b]; return g->accum_grads[b]; }
/* new log-probabilities written by the policy-gradient dispatch of the last completion */
const float *grpo_dbg_new_logprobs(GRPOState *g) { return (const float *)metal_buf_ptr(g->mb_new_lp); }
SFTState *grpo_dbg_sft(GRPOState *g) { return g->sft; }
