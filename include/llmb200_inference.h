/*
 * llmb200_inference.h -- the decode engine at the drop-in boundary.
 *
 * Part 1 declares, under the reference's own names and with the same argument
 * meaning and error behaviour, the public interface of llm.metal's fast
 * inference engine (src/nn/fast_inference.h:12-72; implementation
 * src/nn/fast_inference.c:171-692). A program compiled against the reference
 * header links against libllmb200.so unchanged.
 *
 * Part 2 is additive: tensor-parallel set-up, layer-by-layer construction for
 * callers that cannot hold the whole fp32 model in host memory, and
 * measurement hooks. Existing callers never need it (defaults: one GPU).
 */
#ifndef LLMB200_INFERENCE_H
#define LLMB200_INFERENCE_H

#include <stdint.h>
#include "llmb200_model_abi.h"
#include "llmb200_wmat.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ========================= Part 1: reference interface ==================== */

typedef struct InferenceState InferenceState;

/* Builds the persistent decode state: converts every matrix to Q8_0
 * (use_fp16 = 0) or F16 (use_fp16 = 1), uploads it, allocates the KV cache for
 * max_seq_len positions (values above 4096 are clamped with a warning, as in
 * the reference) and captures the per-token CUDA graph. Returns NULL with a
 * message on stderr on any failure. The model is only read during this call:
 * the embedding table is copied to the device, so the model may be freed
 * afterwards (the reference keeps borrowing it).
 * Replaces inference_state_create (src/nn/fast_inference.c:277-296). */
InferenceState *inference_state_create(llmb200_qwen3_model *model, int max_seq_len, int use_fp16);
/* Gemma3: tied LM head, embedding scaled by sqrt(d_model), four norms per
 * block, GeGLU, per-layer RoPE base. Replaces inference_state_create_gemma3
 * (src/nn/fast_inference.c:298-318). */
InferenceState *inference_state_create_gemma3(llmb200_gemma3_model *model, int max_seq_len, int use_fp16);
/* Frees everything the state owns and drops one reference on the runtime.
 * Replaces inference_state_free (src/nn/fast_inference.c:344-370). */
void inference_state_free(InferenceState *state);

/* One greedy request: token-by-token prefill of the prompt, first output token
 * = argmax of the last prompt position, then one forward per further token
 * until max_gen_len tokens, an EOS token or the end of the KV cache. Returns
 * the number of tokens written to output_tokens (>= 1).
 * Replaces inference_generate (src/nn/fast_inference.c:614-675). */
int inference_generate(InferenceState *state, const uint32_t *prompt_tokens, int prompt_len,
                       uint32_t *output_tokens, int max_gen_len);

ModelType inference_state_model_type(InferenceState *state);   /* src/nn/fast_inference.c:320-322 */
int  inference_state_vocab_size(InferenceState *state);        /* :482-484 */
void inference_state_reset(InferenceState *state);             /* :486-488 */
/* Forward one token at the current position and advance it. The returned
 * pointer addresses vocab_size fp32 logits in pinned host memory, valid until
 * the next call on this state. Replaces inference_forward_token (:490-494). */
const float *inference_forward_token(InferenceState *state, int token);
/* Reads "eos_token_id" (int or array of up to 4 ints) from config.json next to
 * or inside model_path; falls back to the model-type defaults.
 * Replaces inference_state_load_eos (:324-342). */
void inference_state_load_eos(InferenceState *state, const char *model_path);
/* Create, generate, free. Replaces qwen3_generate_fast (:681-692). */
int qwen3_generate_fast(llmb200_qwen3_model *model, const uint32_t *prompt_tokens, int prompt_len,
                        uint32_t *output_tokens, int max_gen_len, int max_seq_len, int use_fp16);

/* Batched F16 generation: batch_size (1..32) sequences start from the same
 * prompt and advance one position per step, sharing one read of the weights.
 * output_tokens is [batch_size][max_gen_len]; returns the number of tokens
 * generated per sequence (0 on failure). Stops when every sequence has
 * produced an EOS id (151645, 151643 or 0, the reference's list) or the cache
 * is full. Replaces qwen3_generate_fast_batch
 * (src/nn/fast_inference.c:895-985; fast_inference.h:66-72). */
int qwen3_generate_fast_batch(llmb200_qwen3_model *model, const uint32_t *prompt_tokens, int prompt_len,
                              uint32_t *output_tokens, int max_gen_len, int max_seq_len, int batch_size);

/* Attaches the LoRA matrices of an SFT state (Q and V projections, read in
 * place on the device) to the decode step: q += s B_q (A_q ln), v += s B_v (A_v ln)
 * per layer. One GPU only. Replaces inference_state_set_lora
 * (src/nn/fast_inference.c:496-520; declared in fast_inference.h:56-58). */
struct SFTState;
void inference_state_set_lora(InferenceState *state, struct SFTState *sft);

/* A decode state over the weights an SFT state already holds on the device,
 * with that state's LoRA attached. F16 weights, one GPU; the frozen matrices
 * are re-laid for the decode kernels by device-to-device copies (they never
 * change in LoRA training), the LoRA matrices are read in place. The SFT state
 * must outlive the decode state. Replaces inference_state_create_from_sft
 * (src/nn/fast_inference.c:526-608; declared in fast_inference.h:50). */
InferenceState *inference_state_create_from_sft(struct SFTState *sft, int max_seq_len);

/* ========================= Part 2: additions ============================== */

/* Tensor parallelism. One process per GPU; rank r of `world` holds the r-th
 * slice of every column-parallel matrix (rows of Q/K/V, gate, up, LM head) and
 * of every row-parallel matrix (input columns of O and down), plus the KV
 * cache of its own KV heads. Call before creating a state (or set
 * LLMB200_TP_RANK / LLMB200_TP_SIZE); world must divide the KV-head count. */
int llmb200_set_tp(int rank, int world);
/* The ranks exchange these handles out of band (bench.py uses
 * torch.distributed) and hand the full table, world * LLMB200_HANDLE_BYTES
 * bytes ordered by rank, to llmb200_state_connect before the first token. */
#define LLMB200_HANDLE_BYTES 64
int llmb200_state_comm_handle(InferenceState *state, void *out_handle);
int llmb200_state_connect(InferenceState *state, const void *all_handles, int world);

/* Layer-by-layer construction (same conversions as inference_state_create). */
typedef struct {
    int model_type;                 /* MODEL_QWEN3 / MODEL_GEMMA3 */
    int d_model, n_q_heads, n_kv_heads, head_dim, intermediate_size, vocab_size, n_layers;
    int max_seq_len, use_fp16;
} llmb200_config;
InferenceState *llmb200_state_begin(const llmb200_config *cfg);
/* refs holds full (unsharded) matrices; rope_theta is this layer's RoPE base. */
int llmb200_state_load_layer(InferenceState *state, int layer, const LayerWeightRef *refs, float rope_theta);
/* lm_head [vocab, d_model], final_norm_gamma [d_model], token_emb [vocab, d_model]. */
int llmb200_state_finish(InferenceState *state, const float *lm_head, const float *final_norm_gamma,
                         const float *token_emb);

/* Overrides the EOS list (n = 0: never stop on a token). */
void llmb200_state_set_eos(InferenceState *state, const int *eos, int n);
/* Decode-loop wall time of the last inference_generate, in milliseconds, and
 * the number of forwards it covers (the figures the reference prints). */
double llmb200_last_decode_ms(InferenceState *state, int *n_decoded);
double llmb200_last_prefill_ms(InferenceState *state);
/* Non-zero once a bounded device-side wait ran out or a launch failed. */
int llmb200_state_error(InferenceState *state);
/* Fault injection on the host, for tests of the bounded waits: "connects" a tensor-parallel state
 * (world > 1) to itself instead of to its peers, i.e. to ranks that never arrive. The next token then
 * waits for partial sums nobody writes; every such wait gives up after its iteration limit
 * (LLMB200_SPIN_LIMIT at create time), the launch completes, llmb200_state_error turns non-zero and
 * the state is dead. Nothing on the GPU faults or hangs. */
int llmb200_state_connect_loopback(InferenceState *state);
/* Device-resident timing: starting from the current position, replay the
 * per-token graph n_steps times back to back with every input already in
 * device memory, timed by CUDA events on the launching stream. Returns the
 * elapsed milliseconds (negative on error); the position advances. */
float llmb200_state_run_device_steps(InferenceState *state, int n_steps);
/* Instrumented pass: one token launched kernel by kernel with an event pair
 * around each launch. ms[6] receives the summed milliseconds of: 0 qkv matvec,
 * 1 attention, 2 o matvec, 3 gate/up matvec, 4 down matvec, 5 LM head;
 * launches[6] the launch counts. The position advances by one. */
int llmb200_state_profile_token(InferenceState *state, float *ms, int *launches);
/* Times one kind of kernel (numbering as above) in isolation: `reps` passes over all layers' launches
 * of that kind, back to back on the library stream between two CUDA events; every launch reads a
 * different layer's weights, so nothing is served from L2. Returns the elapsed milliseconds for
 * *launches launches (negative on error). The token state is left untouched. */
float llmb200_state_time_kind(InferenceState *state, int kind, int reps, int *launches);
/* Stage trace of the last whole-token launch (only when LLMB200_TRACE=1 was set at create time): for
 * every block and stage 16 words (b200_token_args.d_trace), laid out
 * [block][stage][16], stages = 6 per layer (q/k/v, attention, o, gate/up, down, one unused) + the LM head.
 * Copies at most cap_words words; returns the number of blocks, 0 when there is no trace. */
int llmb200_state_step_trace(InferenceState *state, unsigned long long *out, size_t cap_words);
/* Bytes of weights one token streams on this rank (all matrices + LM head). */
unsigned long long llmb200_state_weight_bytes(InferenceState *state);
int llmb200_state_position(InferenceState *state);
/* Kernel nodes in the per-token graph (with or without the LM head launch). */
int llmb200_state_graph_kernels(InferenceState *state, int with_lm_head);
/* Copies the packed device weights of one matrix back as the reference's
 * canonical bytes (Q8_0 34-byte blocks or binary16), for parity checks.
 * which: 0 qkv (this rank's q rows, then k rows, then v rows), 1 o, 2 gate/up
 * (interleaved rows g0,u0,g1,u1,...), 3 down, 4 LM head (layer ignored).
 * Returns the byte count, or 0 on error; buf may be NULL to query the size. */
size_t llmb200_state_export_weight(InferenceState *state, int layer, int which, void *buf, size_t cap);

/* Batched decode state, built layer by layer (cfg->use_fp16 is ignored: weights
 * are binary16; cfg->max_seq_len is clamped to 4096). Sequences may have
 * different prompts of one common length: prompts is [batch][prompt_len],
 * output_tokens [batch][max_gen_len]. */
typedef struct llmb200_batch_state llmb200_batch_state;
llmb200_batch_state *llmb200_batch_begin(const llmb200_config *cfg, int batch_size, int max_gen_len);
int llmb200_batch_load_layer(llmb200_batch_state *state, int layer, const LayerWeightRef *refs, float rope_theta);
int llmb200_batch_finish(llmb200_batch_state *state, const float *lm_head, const float *final_norm_gamma,
                         const float *token_emb);
void llmb200_batch_set_eos(llmb200_batch_state *state, const int *eos, int n);
int llmb200_batch_generate(llmb200_batch_state *state, const uint32_t *prompts, int prompt_len,
                           uint32_t *output_tokens, int max_gen_len);
/* Wall time of the decode loop of the last llmb200_batch_generate and its step count. */
double llmb200_batch_last_decode_ms(llmb200_batch_state *state, int *n_steps);
/* Kernel nodes in the per-step CUDA graph (0 before the first generate). */
int llmb200_batch_graph_kernels(llmb200_batch_state *state);
/* The logits [batch][vocab] of the last step, copied to dst (cap floats); NULL if it does not fit. */
const float *llmb200_batch_logits(llmb200_batch_state *state, float *dst, size_t cap);
void llmb200_batch_free(llmb200_batch_state *state);

#ifdef __cplusplus
}
#endif
#endif /* LLMB200_INFERENCE_H */
