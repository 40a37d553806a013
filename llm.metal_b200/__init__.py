"""Python bindings (ctypes) over libllmb200's C ABI.

The product is the C library: `include/*.h` declares its entry points and this
module binds exactly those, so that tests and benchmarks read like calls into
the reference (`inference_state_create`, `inference_generate`, `wmat_create_q8`
...). There is no Python or CPU implementation behind any of them: loading
fails loudly when the CUDA library is missing and every compute call needs a
GPU.
"""
import ctypes as C
import os

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))

c_float_p = C.POINTER(C.c_float)
c_int_p = C.POINTER(C.c_int)
c_uint_p = C.POINTER(C.c_uint)
c_u32_p = C.POINTER(C.c_uint32)

B200_MAX_PEERS = 8
B200_WT_Q8, B200_WT_F16 = 0, 1
B200_IN_VEC, B200_IN_RESID, B200_IN_EMBED = 0, 1, 2
B200_OUT_STORE, B200_OUT_GLU = 0, 1
MODEL_QWEN3, MODEL_GEMMA3 = 0, 1
LLMB200_HANDLE_BYTES = 64


class MatvecArgs(C.Structure):
    """b200_matvec_args (include/llmb200_kernels.h)."""
    _fields_ = [
        ("d_w", C.c_void_p), ("row_stride", C.c_longlong), ("rows", C.c_int), ("cols", C.c_int), ("wtype", C.c_int),
        ("in_mode", C.c_int),
        ("d_in_vec", C.c_void_p),
        ("d_resid_in", C.c_void_p), ("d_resid_out", C.c_void_p),
        ("d_slots", C.c_void_p), ("n_slots", C.c_int), ("slot_stride", C.c_longlong),
        ("d_slot_norm_gamma", C.c_void_p),
        ("d_emb", C.c_void_p), ("d_tokens", C.c_void_p), ("d_pos", C.c_void_p), ("emb_scale", C.c_float),
        ("emb_rows", C.c_int),
        ("d_norm_gamma", C.c_void_p), ("eps", C.c_float),
        ("out_mode", C.c_int), ("act", C.c_int),
        ("d_out", C.c_void_p * B200_MAX_PEERS), ("n_out", C.c_int), ("out_offset", C.c_longlong),
        ("d_argmax_scratch", C.c_void_p),
        ("d_argmax_val", C.c_void_p * B200_MAX_PEERS),
        ("d_argmax_idx", C.c_void_p * B200_MAX_PEERS),
        ("n_argmax_out", C.c_int),
        ("d_ticket", C.c_void_p),
        ("advance_pos", C.c_int), ("d_pos_rw", C.c_void_p),
        ("advance_epoch", C.c_int), ("d_epoch_rw", C.c_void_p),
        ("d_next_token", C.c_void_p), ("d_prompt_len", C.c_void_p),
        ("d_wait_flags", C.c_void_p), ("n_wait", C.c_int),
        ("d_signal_flags", C.c_void_p * B200_MAX_PEERS), ("n_signal", C.c_int), ("signal_index", C.c_int),
        ("d_epoch", C.c_void_p), ("epoch_mul", C.c_int), ("epoch_add", C.c_int),
        ("d_err", C.c_void_p),
        ("grid", C.c_int), ("use_pdl", C.c_int),
        ("d_in_copy", C.c_void_p), ("spin_limit", C.c_int),
    ]


class AttnArgs(C.Structure):
    """b200_attn_args (include/llmb200_kernels.h)."""
    _fields_ = [
        ("d_qkv", C.c_void_p), ("d_q_gamma", C.c_void_p), ("d_k_gamma", C.c_void_p), ("d_inv_freq", C.c_void_p),
        ("d_k_cache", C.c_void_p), ("d_v_cache", C.c_void_p),
        ("d_out", C.c_void_p), ("d_scratch", C.c_void_p), ("d_tickets", C.c_void_p),
        ("d_pos", C.c_void_p),
        ("n_q", C.c_int), ("n_kv", C.c_int), ("hd", C.c_int), ("max_seq", C.c_int), ("n_split", C.c_int),
        ("eps", C.c_float), ("use_pdl", C.c_int),
        ("n_items", C.c_int), ("qkv_item_stride", C.c_longlong), ("cache_item_stride", C.c_longlong),
        ("out_item_stride", C.c_longlong),
    ]


class StageGeom(C.Structure):
    """b200_stage_geom (include/llmb200_kernels.h)."""
    _fields_ = [("rows", C.c_int), ("cols", C.c_int), ("row_stride", C.c_longlong), ("glu", C.c_int),
                ("T", C.c_int), ("NG", C.c_int), ("spt", C.c_int), ("rg", C.c_int), ("rb", C.c_int), ("pw", C.c_int),
                ("cta_base", C.c_int), ("cta_rem", C.c_int), ("direct_in", C.c_int)]


class TokenLayer(C.Structure):
    """b200_token_layer (include/llmb200_kernels.h)."""
    _fields_ = [(n, C.c_void_p) for n in ("w_qkv", "w_o", "w_gateup", "w_down", "g_input", "g_post_attn", "g_pre_ff",
                                          "g_post_ff", "g_qn", "g_kn", "rope", "k_cache", "v_cache")]


B200_ST_QKV, B200_ST_O, B200_ST_GATEUP, B200_ST_DOWN, B200_ST_LM, B200_ST_KINDS = 0, 1, 2, 3, 4, 5


class TokenArgs(C.Structure):
    """b200_token_args (include/llmb200_kernels.h)."""
    _fields_ = [
        ("d_layers", C.c_void_p), ("n_layers", C.c_int), ("wtype", C.c_int), ("gemma", C.c_int),
        ("g", StageGeom * B200_ST_KINDS),
        ("w_lm", C.c_void_p), ("g_final", C.c_void_p), ("with_lm", C.c_int),
        ("d_emb", C.c_void_p), ("emb_rows", C.c_int), ("emb_scale", C.c_float), ("eps", C.c_float),
        ("d_model", C.c_int), ("n_q", C.c_int), ("n_kv", C.c_int), ("hd", C.c_int), ("max_seq", C.c_int), ("n_split", C.c_int),
        ("d_pos", C.c_void_p), ("d_tokens", C.c_void_p), ("d_prompt_len", C.c_void_p), ("d_epoch", C.c_void_p), ("d_err", C.c_void_p),
        ("d_qkv", C.c_void_p), ("d_attn_part", C.c_void_p), ("d_attn_out", C.c_void_p), ("d_act", C.c_void_p), ("d_am", C.c_void_p),
        ("d_slots_o", C.c_void_p), ("d_slots_dn", C.c_void_p),
        ("d_peer_slots_o", C.c_void_p * B200_MAX_PEERS), ("d_peer_slots_dn", C.c_void_p * B200_MAX_PEERS),
        ("d_am_rank", C.c_void_p), ("d_peer_am", C.c_void_p * B200_MAX_PEERS),
        ("n_ranks", C.c_int), ("rank", C.c_int),
        ("d_counters", C.c_void_p), ("d_peer_counters", C.c_void_p * B200_MAX_PEERS),
        ("d_logits", C.c_void_p), ("logits_offset", C.c_longlong),
        ("spin_limit", C.c_int),
        ("d_trace", C.c_void_p),
        ("n_blocks", C.c_int), ("smem_bytes", C.c_int), ("scratch_floats", C.c_int), ("att_keys", C.c_int), ("l2_ahead_bytes", C.c_int),
        ("counter_spin_limit", C.c_int),
    ]


class Config(C.Structure):
    """llmb200_config (include/llmb200_inference.h)."""
    _fields_ = [("model_type", C.c_int), ("d_model", C.c_int), ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("intermediate_size", C.c_int), ("vocab_size", C.c_int), ("n_layers", C.c_int),
                ("max_seq_len", C.c_int), ("use_fp16", C.c_int)]


class WeightRef(C.Structure):
    _fields_ = [("data", c_float_p), ("rows", C.c_int), ("cols", C.c_int)]


class LayerWeightRef(C.Structure):
    _fields_ = [("q_proj", WeightRef), ("k_proj", WeightRef), ("v_proj", WeightRef), ("o_proj", WeightRef),
                ("gate_proj", WeightRef), ("up_proj", WeightRef), ("down_proj", WeightRef),
                ("input_norm_g", c_float_p), ("post_attn_norm_g", c_float_p),
                ("pre_ff_norm_g", c_float_p), ("post_ff_norm_g", c_float_p),
                ("q_norm_g", c_float_p), ("k_norm_g", c_float_p),
                ("d_model", C.c_int), ("head_dim", C.c_int)]


class GemmArgs(C.Structure):
    """b200_gemm_args (include/llmb200_train_kernels.h)."""
    _fields_ = [("A", C.c_void_p), ("a_row", C.c_longlong), ("a_col", C.c_longlong),
                ("B", C.c_void_p), ("b_row", C.c_longlong), ("b_col", C.c_longlong),
                ("C", C.c_void_p), ("ldc", C.c_longlong),
                ("R", C.c_void_p), ("ldr", C.c_longlong),
                ("M", C.c_int), ("N", C.c_int), ("K", C.c_int), ("alpha", C.c_float), ("d_err", C.c_void_p)]


class WMat(C.Structure):
    _fields_ = [("mbuf", C.c_void_p), ("rows", C.c_int), ("cols", C.c_int), ("nb", C.c_int)]


class LayerW(C.Structure):
    """LayerW (include/llmb200_wmat.h): seven WMat pointers and six norm buffers."""
    _fields_ = [(n, C.POINTER(WMat)) for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")] + \
               [(n, C.c_void_p) for n in ("input_norm_g", "post_attn_norm_g", "pre_ff_norm_g", "post_ff_norm_g", "q_norm_g", "k_norm_g")]


class SynthSpec(C.Structure):
    """llmb200_synth_spec (include/llmb200_synth.h)."""
    _fields_ = [("seed", C.c_uint64),
                ("n_layers", C.c_int), ("d_model", C.c_int), ("n_q_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("intermediate_size", C.c_int), ("vocab_size", C.c_int),
                ("rope_theta", C.c_float), ("local_rope_theta", C.c_float), ("sliding_window", C.c_int),
                ("weight_std", C.c_float), ("gamma_jitter", C.c_float)]


# Every symbol include/*.h declares, by header. the ABI test under tests/ checks the lists against the
# headers and against the built libraries.
SYMBOLS_MAIN = {
    "llmb200_wmat.h": ["fast_metal_init", "fast_metal_shutdown", "metal_flush", "metal_buf_create", "metal_buf_from_data",
                       "metal_buf_free", "metal_buf_ptr", "wmat_create_q8", "wmat_create_f16", "wmat_free", "wmat_convert",
                       "norm_upload", "layers_convert_upload", "layers_free", "metal_enqueue_scale", "metal_enqueue_grpo_policy_grad"],
    "llmb200_kernels.h": ["b200_packed_row_stride", "b200_q8_pack", "b200_f16_pack", "b200_q8_unpack_blocks", "b200_matvec",
                          "b200_attn_scratch_floats", "b200_attn_decode", "b200_attn_decode_static", "b200_tp_argmax_finalize", "b200_token_plan", "b200_token_chunks", "b200_decode_token", "b200_lora_decode", "b200_argmax_rows",
                          "b200_launch_count", "b200_launch_count_add"],
    "llmb200_inference.h": ["inference_state_create", "inference_state_create_gemma3", "inference_state_free",
                            "inference_generate", "inference_state_model_type", "inference_state_vocab_size",
                            "inference_state_reset", "inference_forward_token", "inference_state_load_eos",
                            "qwen3_generate_fast", "qwen3_generate_fast_batch", "inference_state_set_lora", "inference_state_create_from_sft", "llmb200_set_tp", "llmb200_state_comm_handle", "llmb200_state_connect",
                            "llmb200_state_begin", "llmb200_state_load_layer", "llmb200_state_finish",
                            "llmb200_state_set_eos", "llmb200_last_decode_ms", "llmb200_last_prefill_ms",
                            "llmb200_state_error", "llmb200_state_connect_loopback", "llmb200_state_run_device_steps", "llmb200_state_profile_token",
                            "llmb200_state_time_kind", "llmb200_state_step_trace",
                            "llmb200_state_weight_bytes", "llmb200_state_position", "llmb200_state_graph_kernels",
                            "llmb200_state_export_weight", "llmb200_batch_begin", "llmb200_batch_load_layer",
                            "llmb200_batch_finish", "llmb200_batch_set_eos", "llmb200_batch_generate",
                            "llmb200_batch_last_decode_ms", "llmb200_batch_graph_kernels", "llmb200_batch_logits", "llmb200_batch_free"],
    "llmb200_train_kernels.h": ["b200_gemm_f32", "b200_gemm_tf32", "b200_gemm_f16", "b200_f32_to_f16", "b200_transpose_f16", "b200_lora_pack_f16", "b200_embed_rows", "b200_round_f16",
                                "b200_transpose_f32", "b200_rms_norm_rows", "b200_rms_norm_bwd_rows",
                                "b200_qk_norm_rope", "b200_qk_norm_rope_bwd", "b200_attn_train_fwd",
                                "b200_attn_train_bwd", "b200_silu_mul_rows", "b200_silu_mul_bwd_rows", "b200_lora_add", "b200_lora_pack", "b200_xty_skinny",
                                "b200_softmax_ce_rows", "b200_sumsq_partials", "b200_clip_adamw",
                                "b200_rms_norm_rows_h", "b200_rms_norm_bwd_rows_h", "b200_attn_train_fwd_h",
                                "b200_silu_mul_rows_h", "b200_silu_mul_bwd_rows_h", "b200_softmax_ce_rows_h",
                                "b200_grpo_policy_grad", "b200_scale", "b200_sgd_apply_f16", "b200_gelu_mul_rows", "b200_gelu_mul_bwd_rows", "b200_add"],
    "llmb200_sft.h": ["sft_state_create", "sft_state_free", "sft_train_step", "forward_to_logits", "sft_backward",
                      "sft_get_logits", "sft_get_dlogits", "sft_get_x_cpu", "sft_get_losses_cpu", "sft_get_seq_len",
                      "sft_get_vocab_size", "sft_get_d_model", "sft_get_lora_rank", "sft_get_n_layers",
                      "sft_get_emb_scale", "sft_get_token_emb", "sft_get_step_count", "sft_set_step_count",
                      "sft_get_n_lora_grad_bufs", "sft_get_lora_grad_ptr", "sft_set_lora_grad", "sft_lora_update",
                      "sft_save_lora", "sft_get_lora_weight_buf", "sft_get_lora_scaling", "sft_sync_lora_to_model",
                      "sft_get_layers", "sft_get_lm_head", "sft_get_final_norm_g", "sft_get_model_type", "sft_get_n_q_heads",
                      "sft_get_n_kv_heads", "sft_get_head_dim", "sft_get_intermediate_size", "sft_get_rope_thetas",
                      "llmb200_sft_begin", "llmb200_sft_load_layer", "llmb200_sft_finish",
                      "llmb200_sft_forward_backward", "llmb200_sft_apply_update", "llmb200_sft_train_batch",
                      "llmb200_sft_grad_vector", "llmb200_sft_param_vector", "llmb200_sft_last_grad_norm",
                      "llmb200_sft_last_step_ms", "llmb200_sft_use_tensor_cores", "llmb200_sft_error",
                      "llmb200_sft_export",
                      "sft_state_create_gemma3", "sft_state_create_full", "sft_state_create_gemma3_full", "sft_is_full_param",
                      "sft_backward_sgd", "sft_alloc_grad_accum", "sft_backward_accum", "sft_apply_grad_sgd",
                      "sft_save_full_checkpoint", "sft_sync_lora_to_gemma3"],
}
SYMBOLS_SYNTH = {
    "llmb200_synth.h": ["llmb200_synth_tensor_id", "llmb200_synth_normal_range", "llmb200_synth_normal",
                        "llmb200_synth_tokens", "llmb200_synth_qwen3", "llmb200_synth_free_qwen3", "llmb200_synth_gemma3",
                        "llmb200_synth_free_gemma3", "llmb200_abi_layout"],
}

_lib = None
_synth = None


def lib():
    """libllmb200.so with argument types set. Raises if it cannot be built or loaded."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if not os.path.exists(path):
        _build.build_main()
    L = C.CDLL(path)
    vp, i, ll, sz, fl = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t, C.c_float
    sig = {
        "fast_metal_init": (i, []), "fast_metal_shutdown": (None, []), "metal_flush": (None, []),
        "metal_buf_create": (vp, [sz]), "metal_buf_from_data": (vp, [vp, sz]), "metal_buf_free": (None, [vp]),
        "metal_buf_ptr": (vp, [vp]),
        "wmat_create_q8": (C.POINTER(WMat), [c_float_p, i, i]), "wmat_create_f16": (C.POINTER(WMat), [c_float_p, i, i]),
        "wmat_free": (None, [C.POINTER(WMat)]), "wmat_convert": (C.POINTER(WMat), [c_float_p, i, i, i]),
        "norm_upload": (vp, [c_float_p, i]),
        "layers_convert_upload": (vp, [C.POINTER(LayerWeightRef), i, i]), "layers_free": (None, [vp, i]),
        "b200_packed_row_stride": (sz, [i, i]),
        "b200_q8_pack": (i, [vp, ll, i, i, vp, ll, i, i, vp]), "b200_f16_pack": (i, [vp, ll, i, i, vp, ll, i, i, vp]),
        "b200_q8_unpack_blocks": (i, [vp, ll, i, i, vp, vp]),
        "b200_matvec": (i, [C.POINTER(MatvecArgs), vp]),
        "b200_attn_scratch_floats": (sz, [i, i, i]), "b200_attn_decode": (i, [C.POINTER(AttnArgs), vp]),
        "b200_attn_decode_static": (i, [C.POINTER(AttnArgs), vp]),
        "b200_tp_argmax_finalize": (i, [vp, vp, i, vp, vp, i, i, vp, vp, vp, vp, vp, i, vp]),
        "b200_token_plan": (i, [C.POINTER(TokenArgs), i]), "b200_token_chunks": (i, [C.POINTER(TokenArgs), i, i, c_int_p, i]),
        "b200_decode_token": (i, [C.POINTER(TokenArgs), vp]),
        "b200_lora_decode": (i, [vp, vp, vp, vp, vp, vp, i, i, i, i, fl, vp]),
        "b200_argmax_rows": (i, [vp, i, i, vp, vp, i, vp, vp, vp]),
        "b200_launch_count": (C.c_ulonglong, [i]), "b200_launch_count_add": (None, [C.c_ulonglong]),
        "inference_state_create": (vp, [vp, i, i]), "inference_state_create_gemma3": (vp, [vp, i, i]),
        "inference_state_free": (None, [vp]),
        "inference_generate": (i, [vp, c_u32_p, i, c_u32_p, i]),
        "inference_state_model_type": (i, [vp]), "inference_state_vocab_size": (i, [vp]),
        "inference_state_reset": (None, [vp]), "inference_forward_token": (c_float_p, [vp, i]),
        "inference_state_load_eos": (None, [vp, C.c_char_p]),
        "qwen3_generate_fast": (i, [vp, c_u32_p, i, c_u32_p, i, i, i]),
        "inference_state_set_lora": (None, [vp, vp]),
        "inference_state_create_from_sft": (vp, [vp, i]),
        "qwen3_generate_fast_batch": (i, [vp, c_u32_p, i, c_u32_p, i, i, i]),
        "llmb200_batch_begin": (vp, [C.POINTER(Config), i, i]),
        "llmb200_batch_load_layer": (i, [vp, i, C.POINTER(LayerWeightRef), C.c_float]),
        "llmb200_batch_finish": (i, [vp, c_float_p, c_float_p, c_float_p]),
        "llmb200_batch_set_eos": (None, [vp, c_int_p, i]),
        "llmb200_batch_generate": (i, [vp, c_u32_p, i, c_u32_p, i]),
        "llmb200_batch_last_decode_ms": (C.c_double, [vp, c_int_p]),
        "llmb200_batch_graph_kernels": (i, [vp]),
        "llmb200_batch_logits": (c_float_p, [vp, c_float_p, sz]),
        "llmb200_batch_free": (None, [vp]),
        "llmb200_set_tp": (i, [i, i]), "llmb200_state_comm_handle": (i, [vp, vp]),
        "llmb200_state_connect": (i, [vp, vp, i]),
        "llmb200_state_begin": (vp, [C.POINTER(Config)]),
        "llmb200_state_load_layer": (i, [vp, i, C.POINTER(LayerWeightRef), C.c_float]),
        "llmb200_state_finish": (i, [vp, c_float_p, c_float_p, c_float_p]),
        "llmb200_state_set_eos": (None, [vp, c_int_p, i]),
        "llmb200_last_decode_ms": (C.c_double, [vp, c_int_p]), "llmb200_last_prefill_ms": (C.c_double, [vp]),
        "llmb200_state_error": (i, [vp]), "llmb200_state_connect_loopback": (i, [vp]), "llmb200_state_run_device_steps": (C.c_float, [vp, i]),
        "llmb200_state_profile_token": (i, [vp, c_float_p, c_int_p]),
        "llmb200_state_time_kind": (C.c_float, [vp, i, i, c_int_p]),
        "llmb200_state_step_trace": (i, [vp, C.POINTER(C.c_ulonglong), sz]),
        "llmb200_state_weight_bytes": (C.c_ulonglong, [vp]), "llmb200_state_position": (i, [vp]),
        "llmb200_state_graph_kernels": (i, [vp, i]),
        "llmb200_state_export_weight": (sz, [vp, i, i, vp, sz]),
        # ---- llmb200_train_kernels.h
        "b200_gemm_f32": (i, [C.POINTER(GemmArgs), vp]), "b200_gemm_tf32": (i, [C.POINTER(GemmArgs), vp]),
        "b200_gemm_f16": (i, [C.POINTER(GemmArgs), vp]), "b200_f32_to_f16": (i, [vp, sz, fl, vp, vp]),
        "b200_transpose_f16": (i, [vp, i, i, vp, vp]),
        "b200_lora_pack_f16": (i, [vp, vp, vp, vp, vp, vp, i, i, i, i, i, fl, vp]),
        "b200_embed_rows": (i, [vp, vp, i, i, i, fl, vp, vp]),
        "b200_round_f16": (i, [vp, sz, vp]), "b200_transpose_f32": (i, [vp, i, i, vp, vp]),
        "b200_rms_norm_rows": (i, [vp, vp, vp, i, i, fl, vp]),
        "b200_rms_norm_bwd_rows": (i, [vp, vp, ll, vp, vp, i, i, fl, i, fl, vp]),
        "b200_qk_norm_rope": (i, [vp, ll, vp, vp, vp, i, i, i, i, i, fl, vp, vp, vp]),
        "b200_qk_norm_rope_bwd": (i, [vp, vp, ll, ll, vp, vp, vp, i, i, i, i, i, fl, vp]),
        "b200_attn_train_fwd": (i, [vp, vp, vp, ll, i, i, i, i, i, fl, vp, vp, vp]),
        "b200_attn_train_bwd": (i, [vp, vp, vp, vp, vp, ll, i, i, i, i, i, fl, vp, vp, ll, vp]),
        "b200_silu_mul_rows": (i, [vp, i, i, vp, vp]), "b200_silu_mul_bwd_rows": (i, [vp, vp, i, i, vp, vp]),
        "b200_lora_add": (i, [vp, ll, i, i, vp, ll, vp, i, fl, i, vp]),
        "b200_lora_pack": (i, [vp, vp, vp, vp, vp, vp, i, i, i, i, i, fl, vp]),
        "b200_xty_skinny": (i, [vp, ll, vp, ll, i, i, i, fl, vp, ll, ll, vp]),
        "b200_softmax_ce_rows": (i, [vp, vp, i, i, fl, vp, vp, vp]),
        "b200_sumsq_partials": (i, [vp, sz, vp, i, vp]),
        "b200_clip_adamw": (i, [vp, vp, vp, vp, sz, vp, i, fl, fl, fl, fl, fl, fl, fl, fl, i, vp, vp]),
        "b200_rms_norm_rows_h": (i, [vp, vp, vp, vp, i, i, fl, vp]),
        "b200_rms_norm_bwd_rows_h": (i, [vp, vp, ll, vp, vp, i, i, fl, i, fl, vp, fl, vp]),
        "b200_attn_train_fwd_h": (i, [vp, vp, vp, ll, i, i, i, i, i, fl, vp, vp, vp, vp]),
        "b200_silu_mul_rows_h": (i, [vp, i, i, vp, vp, vp]),
        "b200_silu_mul_bwd_rows_h": (i, [vp, vp, i, i, vp, vp, fl, vp]),
        "b200_softmax_ce_rows_h": (i, [vp, vp, i, i, fl, vp, vp, vp, fl, vp]),
        "b200_grpo_policy_grad": (i, [vp, vp, vp, vp, vp, vp, i, i, fl, vp]),
        "b200_scale": (i, [vp, fl, sz, vp]),
        "b200_sgd_apply_f16": (i, [vp, vp, sz, fl, vp]),
        "b200_gelu_mul_rows": (i, [vp, i, i, vp, vp]), "b200_gelu_mul_bwd_rows": (i, [vp, vp, i, i, vp, vp]),
        "b200_add": (i, [vp, vp, vp, sz, vp]),
        # ---- llmb200_sft.h
        "sft_state_create": (vp, [vp, i, i, fl]), "sft_state_free": (None, [vp]),
        "sft_train_step": (fl, [vp, c_u32_p, c_u32_p, fl]),
        "forward_to_logits": (None, [vp]), "sft_backward": (None, [vp]),
        "sft_get_logits": (vp, [vp]), "sft_get_dlogits": (vp, [vp]),
        "sft_get_x_cpu": (c_float_p, [vp]), "sft_get_losses_cpu": (c_float_p, [vp]),
        "sft_get_seq_len": (i, [vp]), "sft_get_vocab_size": (i, [vp]), "sft_get_d_model": (i, [vp]),
        "sft_get_lora_rank": (i, [vp]), "sft_get_n_layers": (i, [vp]), "sft_get_emb_scale": (fl, [vp]),
        "sft_get_token_emb": (c_float_p, [vp]), "sft_get_step_count": (i, [vp]), "sft_set_step_count": (None, [vp, i]),
        "sft_get_n_lora_grad_bufs": (i, [vp]), "sft_get_lora_grad_ptr": (c_float_p, [vp, i, c_int_p]),
        "sft_set_lora_grad": (None, [vp, i, c_float_p, i]), "sft_lora_update": (None, [vp, fl]),
        "sft_save_lora": (None, [vp, C.c_char_p]), "sft_get_lora_weight_buf": (vp, [vp, i, i]),
        "sft_get_lora_scaling": (fl, [vp]), "sft_sync_lora_to_model": (None, [vp, vp]),
        "sft_get_layers": (vp, [vp]), "sft_get_lm_head": (vp, [vp]), "sft_get_final_norm_g": (vp, [vp]),
        "sft_get_model_type": (i, [vp]), "sft_get_n_q_heads": (i, [vp]), "sft_get_n_kv_heads": (i, [vp]),
        "sft_get_head_dim": (i, [vp]), "sft_get_intermediate_size": (i, [vp]), "sft_get_rope_thetas": (c_float_p, [vp]),
        "llmb200_sft_begin": (vp, [C.POINTER(Config), i, i, i, fl]),
        "llmb200_sft_load_layer": (i, [vp, i, C.POINTER(LayerWeightRef), fl, C.POINTER(c_float_p * 4)]),
        "llmb200_sft_finish": (i, [vp, c_float_p, c_float_p, c_float_p, i]),
        "llmb200_sft_forward_backward": (fl, [vp, c_u32_p, c_u32_p]),
        "llmb200_sft_apply_update": (None, [vp, fl]),
        "llmb200_sft_train_batch": (fl, [vp, c_u32_p, c_u32_p, fl]),
        "llmb200_sft_grad_vector": (sz, [vp, C.POINTER(vp)]), "llmb200_sft_param_vector": (sz, [vp, C.POINTER(vp)]),
        "llmb200_sft_last_grad_norm": (fl, [vp]), "llmb200_sft_last_step_ms": (fl, [vp, c_float_p]),
        "llmb200_sft_use_tensor_cores": (i, [vp, i]), "llmb200_sft_error": (i, [vp]),
        "llmb200_sft_export": (sz, [vp, i, i, vp, sz]),
        "sft_state_create_gemma3": (vp, [vp, i, i, fl]), "sft_state_create_full": (vp, [vp, i]),
        "sft_state_create_gemma3_full": (vp, [vp, i]), "sft_is_full_param": (i, [vp]),
        "sft_backward_sgd": (None, [vp, fl]), "sft_alloc_grad_accum": (None, [vp]), "sft_backward_accum": (None, [vp]),
        "sft_apply_grad_sgd": (None, [vp, fl]), "sft_save_full_checkpoint": (None, [vp, C.c_char_p]),
        "sft_sync_lora_to_gemma3": (None, [vp, vp]),
        "metal_enqueue_scale": (None, [vp, fl, i]),
        "metal_enqueue_grpo_policy_grad": (None, [vp, vp, vp, vp, vp, vp, i, i, fl]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def synth():
    """libllmb200_synth.so (host only)."""
    global _synth
    if _synth is not None:
        return _synth
    path = _build.LIB_SYNTH
    if not os.path.exists(path):
        _build.build_synth()
    S = C.CDLL(path)
    vp, i, sz, u64, f = C.c_void_p, C.c_int, C.c_size_t, C.c_uint64, C.c_float
    S.llmb200_synth_tensor_id.restype, S.llmb200_synth_tensor_id.argtypes = u64, [i, i]
    S.llmb200_synth_normal_range.restype, S.llmb200_synth_normal_range.argtypes = None, [vp, sz, sz, u64, u64, f, f, i]
    S.llmb200_synth_normal.restype, S.llmb200_synth_normal.argtypes = None, [vp, sz, u64, u64, f, f, i]
    S.llmb200_synth_tokens.restype, S.llmb200_synth_tokens.argtypes = None, [vp, sz, u64, C.c_uint32]
    S.llmb200_synth_qwen3.restype, S.llmb200_synth_qwen3.argtypes = vp, [C.POINTER(SynthSpec), i]
    S.llmb200_synth_free_qwen3.restype, S.llmb200_synth_free_qwen3.argtypes = None, [vp]
    S.llmb200_synth_gemma3.restype, S.llmb200_synth_gemma3.argtypes = vp, [C.POINTER(SynthSpec), i]
    S.llmb200_synth_free_gemma3.restype, S.llmb200_synth_free_gemma3.argtypes = None, [vp]
    S.llmb200_abi_layout.restype, S.llmb200_abi_layout.argtypes = i, [C.POINTER(sz), i]
    _synth = S
    return S


# ---- the architectures the benchmarks and tests use ------------------------------------------------

def spec(name, seed=1234, gamma_jitter=0.0, **over):
    """SynthSpec of a named architecture. All matrices N(0, 0.02)."""
    table = {
        # hidden 512, 4 layers, 8/2 heads, head_dim 64, ffn 1536, vocab 4096
        "tiny-qwen3": dict(n_layers=4, d_model=512, n_q_heads=8, n_kv_heads=2, head_dim=64, intermediate_size=1536,
                           vocab_size=4096, rope_theta=1e6),
        # Qwen3-4B: src/nn/qwen3.c:13-25
        "qwen3-4b": dict(n_layers=36, d_model=2560, n_q_heads=32, n_kv_heads=8, head_dim=128, intermediate_size=9728,
                         vocab_size=151936, rope_theta=1e6),
        # Gemma3-1B: src/nn/gemma3.c:11-25
        "gemma3-1b": dict(n_layers=26, d_model=1152, n_q_heads=4, n_kv_heads=1, head_dim=256, intermediate_size=6912,
                          vocab_size=262144, rope_theta=1e6, local_rope_theta=1e4, sliding_window=512),
        "tiny-gemma3": dict(n_layers=7, d_model=384, n_q_heads=4, n_kv_heads=1, head_dim=256, intermediate_size=1152,
                            vocab_size=2048, rope_theta=1e6, local_rope_theta=1e4, sliding_window=512),
    }
    d = dict(table[name])
    d.update(over)
    s = SynthSpec()
    s.seed = seed
    s.weight_std = 0.02
    s.gamma_jitter = gamma_jitter
    s.local_rope_theta = 1e4
    for k, v in d.items():
        setattr(s, k, v)
    return s


def config_of(sp, model_type, max_seq_len, use_fp16):
    return Config(model_type, sp.d_model, sp.n_q_heads, sp.n_kv_heads, sp.head_dim, sp.intermediate_size, sp.vocab_size,
                  sp.n_layers, max_seq_len, use_fp16)
