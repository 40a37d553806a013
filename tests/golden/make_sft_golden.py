"""Generates tests/golden/sft_golden.npz, sft_golden_gemma3.npz, sft_golden_full.npz and fast_decode_golden.npz by running the reference's
own fast engines -- src/nn/fast_sft.c and src/nn/fast_inference.c, compiled unmodified into
oracle/_ref/libllmref_fast.so over a CPU stand-in for their Metal dispatch layer (oracle/fast_metal_cpu.c).

    python tests/golden/make_sft_golden.py [lora] [decode] [gemma3] [full]       (where the reference tree is mounted)

sft_golden.npz -- three sft_train_step calls (fast_sft.c:1113-1157) on the tiny Qwen3 configuration
(hidden 512, 4 layers, 8/2 heads, head_dim 64, ffn 1536, vocab 4096; seeded weights 1234, norm gammas
N(1, 0.1)), one sequence of 16 tokens, LoRA rank 4, alpha 8, lr 1e-3. The state is created by
sft_state_create; its A matrices are then overwritten in place, through the CPU pointer the reference
exposes for exactly that (sft_get_lora_weight_buf + metal_buf_ptr), with the seeded N(0, 0.01) values
tests/_sft_common.make_lora produces (libc rand() is not reproducible across platforms); B starts at 0 as
in the reference. Kept per step: the returned loss, the per-position losses, and the 4*L gradient buffers
as sft_train_step leaves them (after clip_grad_norm at 1.0); after the third step: the LoRA weights and the
bytes sft_save_lora writes.

fast_decode_golden.npz -- inference_generate (fast_inference.c:614-675) and inference_forward_token on the
tiny Qwen3 and tiny Gemma3 models, Q8_0 and F16: prompt 16, 32 generated tokens, the logits of the last
prompt position. This is the reference's own forward_token (:376-467), Gemma3 block order included.
"""
import ctypes as C
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import _sft_common as sc  # noqa: E402

RANK, ALPHA, N, LR, STEPS = 4, 8.0, 16, 1e-3, 3
P, G, MAX_SEQ = 16, 32, 64
KEYS = ("A_q", "B_q", "A_v", "B_v")


def fast_ref():
    r = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libllmref_fast.so"))
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    r.sft_state_create.restype, r.sft_state_create.argtypes = vp, [vp, i32, i32, f32]
    r.sft_state_free.argtypes = [vp]
    r.sft_train_step.restype, r.sft_train_step.argtypes = f32, [vp, vp, vp, f32]
    r.sft_get_lora_grad_ptr.restype, r.sft_get_lora_grad_ptr.argtypes = C.POINTER(f32), [vp, i32, C.POINTER(i32)]
    r.sft_get_lora_weight_buf.restype, r.sft_get_lora_weight_buf.argtypes = vp, [vp, i32, i32]
    r.sft_get_losses_cpu.restype, r.sft_get_losses_cpu.argtypes = C.POINTER(f32), [vp]
    r.metal_buf_ptr.restype, r.metal_buf_ptr.argtypes = C.POINTER(f32), [vp]
    r.sft_save_lora.argtypes = [vp, C.c_char_p]
    r.inference_state_create.restype, r.inference_state_create.argtypes = vp, [vp, i32, i32]
    r.inference_state_create_gemma3.restype, r.inference_state_create_gemma3.argtypes = vp, [vp, i32, i32]
    r.inference_state_free.argtypes = [vp]
    r.inference_state_reset.argtypes = [vp]
    r.inference_generate.restype, r.inference_generate.argtypes = i32, [vp, vp, i32, vp, i32]
    r.inference_forward_token.restype, r.inference_forward_token.argtypes = C.POINTER(f32), [vp, i32]
    r.inference_state_load_eos.argtypes = [vp, C.c_char_p]
    return r


def sft_golden(pkg, R):
    S = pkg.synth()
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    cfg = dict(sc.TINY)
    model = S.llmb200_synth_qwen3(C.byref(sp), 4)
    st = R.sft_state_create(model, N, RANK, ALPHA)
    assert st
    shapes = dict(A_q=(RANK, cfg["d_model"]), B_q=(cfg["n_q_heads"] * cfg["head_dim"], RANK),
                  A_v=(RANK, cfg["d_model"]), B_v=(cfg["n_kv_heads"] * cfg["head_dim"], RANK))

    def weight(L, sub):
        k = KEYS[sub]
        return np.ctypeslib.as_array(R.metal_buf_ptr(R.sft_get_lora_weight_buf(st, L, sub)), shape=shapes[k])

    start = sc.make_lora(pkg, cfg, RANK)
    for L in range(cfg["n_layers"]):
        for sub, k in enumerate(KEYS):
            w = weight(L, sub)
            if k.startswith("B"):
                assert not w.any()                       # the reference's own start
            w[...] = start[L][k]
    toks = sc.tokens(pkg, N + 1, 4321, cfg["vocab_size"])
    x, y = np.ascontiguousarray(toks[:-1]), np.ascontiguousarray(toks[1:])
    out = dict(rank=np.array(RANK), alpha=np.array(ALPHA, np.float32), seq_len=np.array(N), lr=np.array(LR, np.float32),
               inputs=x, targets=y)
    for step in range(STEPS):
        loss = R.sft_train_step(st, x.ctypes.data, y.ctypes.data, LR)
        out[f"loss_{step}"] = np.array(loss, np.float32)
        out[f"losses_{step}"] = np.ctypeslib.as_array(R.sft_get_losses_cpu(st), shape=(N,)).copy()
        for L in range(cfg["n_layers"]):
            for sub, k in enumerate(KEYS):
                n = C.c_int(0)
                p = R.sft_get_lora_grad_ptr(st, 4 * L + sub, C.byref(n))
                assert n.value == int(np.prod(shapes[k]))
                out[f"grad_{step}_{L}_{k}"] = np.ctypeslib.as_array(p, shape=shapes[k]).copy()
        print(f"step {step}: loss {loss:.6f}")
    for L in range(cfg["n_layers"]):
        for sub, k in enumerate(KEYS):
            out[f"weight_{L}_{k}"] = weight(L, sub).copy()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "adapter.lora")
        R.sft_save_lora(st, path.encode())
        out["save_lora_bytes"] = np.frombuffer(open(path, "rb").read(), dtype=np.uint8)
    R.sft_state_free(st)
    S.llmb200_synth_free_qwen3(model)
    path = os.path.join(HERE, "sft_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def decode_golden(pkg, R):
    S = pkg.synth()
    out = dict(prompt_len=np.array(P), gen_len=np.array(G), max_seq=np.array(MAX_SEQ))
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "config.json"), "w").write('{"eos_token_id": -1}')       # never stop on a token
        for arch, gemma in (("tiny-qwen3", False), ("tiny-gemma3", True)):
            sp = pkg.spec(arch, gamma_jitter=0.1)
            prompt = np.zeros(P, dtype=np.uint32)
            S.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
            out[f"{arch}_prompt"] = prompt
            for use_fp16 in (0, 1):
                model = (S.llmb200_synth_gemma3 if gemma else S.llmb200_synth_qwen3)(C.byref(sp), 4)
                st = (R.inference_state_create_gemma3 if gemma else R.inference_state_create)(model, MAX_SEQ, use_fp16)
                assert st
                R.inference_state_load_eos(st, d.encode())
                toks = np.zeros(G, dtype=np.uint32)
                n = R.inference_generate(st, prompt.ctypes.data, P, toks.ctypes.data, G)
                assert n == G, n
                R.inference_state_reset(st)
                for t in prompt:
                    p = R.inference_forward_token(st, int(t))
                lg = np.ctypeslib.as_array(p, shape=(sp.vocab_size,)).copy()
                assert int(lg.argmax()) == int(toks[0])
                tag = f"{arch}_{'f16' if use_fp16 else 'q8'}"
                out[f"{tag}_tokens"], out[f"{tag}_logits"] = toks, lg
                print(tag, toks[:8])
                R.inference_state_free(st)
                (S.llmb200_synth_free_gemma3 if gemma else S.llmb200_synth_free_qwen3)(model)
    path = os.path.join(HERE, "fast_decode_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def sft_golden_gemma3(pkg, R):
    """sft_golden_gemma3.npz -- the same three sft_train_step calls on a Gemma3 state (sft_state_create_gemma3,
    fast_sft.c:284-396): the tiny Gemma3 configuration cut to two layers (hidden 384, four query heads of 256 on
    one key/value head, ffn 1152, vocab 2048; layer 0 takes the global RoPE base, layer 1 the local one), LoRA
    rank 4, alpha 8, lr 1e-3, A overwritten with the seeded values as above."""
    S = pkg.synth()
    sp = pkg.spec("tiny-gemma3", gamma_jitter=0.1, n_layers=2)
    cfg = sc.gemma_cfg(sp)
    model = S.llmb200_synth_gemma3(C.byref(sp), 4)
    R.sft_state_create_gemma3.restype, R.sft_state_create_gemma3.argtypes = C.c_void_p, [C.c_void_p, C.c_int, C.c_int, C.c_float]
    st = R.sft_state_create_gemma3(model, N, RANK, ALPHA)
    assert st
    shapes = dict(A_q=(RANK, cfg["d_model"]), B_q=(cfg["n_q_heads"] * cfg["head_dim"], RANK),
                  A_v=(RANK, cfg["d_model"]), B_v=(cfg["n_kv_heads"] * cfg["head_dim"], RANK))

    def weight(L, sub):
        return np.ctypeslib.as_array(R.metal_buf_ptr(R.sft_get_lora_weight_buf(st, L, sub)), shape=shapes[KEYS[sub]])

    start = sc.make_lora(pkg, cfg, RANK)
    for L in range(cfg["n_layers"]):
        for sub, k in enumerate(KEYS):
            weight(L, sub)[...] = start[L][k]
    toks = sc.tokens(pkg, N + 1, 4321, cfg["vocab_size"])
    x, y = np.ascontiguousarray(toks[:-1]), np.ascontiguousarray(toks[1:])
    out = dict(rank=np.array(RANK), alpha=np.array(ALPHA, np.float32), seq_len=np.array(N), lr=np.array(LR, np.float32),
               inputs=x, targets=y)
    for step in range(STEPS):
        loss = R.sft_train_step(st, x.ctypes.data, y.ctypes.data, LR)
        out[f"loss_{step}"] = np.array(loss, np.float32)
        out[f"losses_{step}"] = np.ctypeslib.as_array(R.sft_get_losses_cpu(st), shape=(N,)).copy()
        for L in range(cfg["n_layers"]):
            for sub, k in enumerate(KEYS):
                n = C.c_int(0)
                p = R.sft_get_lora_grad_ptr(st, 4 * L + sub, C.byref(n))
                out[f"grad_{step}_{L}_{k}"] = np.ctypeslib.as_array(p, shape=shapes[k]).copy()
        print(f"gemma3 step {step}: loss {loss:.6f}")
    for L in range(cfg["n_layers"]):
        for sub, k in enumerate(KEYS):
            out[f"weight_{L}_{k}"] = weight(L, sub).copy()
    R.sft_state_free(st)
    S.llmb200_synth_free_gemma3(model)
    path = os.path.join(HERE, "sft_golden_gemma3.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


FULL_STRIDE = 211
MATS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def sft_golden_full(pkg, R):
    """sft_golden_full.npz -- full-parameter training (sft_state_create_full, fast_sft.c:402-501) on the tiny Qwen3
    configuration cut to two layers, one sequence of 16 tokens, lr 1e-3. State one: three sft_train_step calls (SGD
    inside the backward pass). State two: sft_alloc_grad_accum, two sft_train_step calls (which then accumulate),
    sft_apply_grad_sgd. Kept: the losses of every step and, for both states, every FULL_STRIDE-th element of every
    matrix after the last call (binary16, in the order q k v o gate up down per layer, then the LM head)."""
    S = pkg.synth()
    vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
    R.sft_state_create_full.restype, R.sft_state_create_full.argtypes = vp, [vp, i32]
    R.sft_get_layers.restype, R.sft_get_layers.argtypes = C.POINTER(pkg.LayerW), [vp]
    R.sft_get_lm_head.restype, R.sft_get_lm_head.argtypes = C.POINTER(pkg.WMat), [vp]
    R.sft_alloc_grad_accum.argtypes = [vp]
    R.sft_apply_grad_sgd.argtypes = [vp, f32]
    half_p = C.POINTER(C.c_uint16)

    def sample(st, n_layers):
        lw = R.sft_get_layers(st)
        parts = []
        mats = [getattr(lw[L], m).contents for L in range(n_layers) for m in MATS] + [R.sft_get_lm_head(st).contents]
        for wm in mats:
            a = np.ctypeslib.as_array(C.cast(R.metal_buf_ptr(wm.mbuf), half_p), shape=(wm.rows * wm.cols,))
            parts.append(a[::FULL_STRIDE].copy())
        return np.concatenate(parts).view(np.float16)

    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1, n_layers=2)
    toks = sc.tokens(pkg, N + 1, 4321, sp.vocab_size)
    x, y = np.ascontiguousarray(toks[:-1]), np.ascontiguousarray(toks[1:])
    out = dict(seq_len=np.array(N), lr=np.array(LR, np.float32), stride=np.array(FULL_STRIDE), inputs=x, targets=y)
    for tag in ("sgd", "accum"):
        model = S.llmb200_synth_qwen3(C.byref(sp), 4)
        st = R.sft_state_create_full(model, N)
        assert st
        start = sample(st, sp.n_layers)
        if tag == "accum":
            R.sft_alloc_grad_accum(st)
        losses = []
        for step in range(3 if tag == "sgd" else 2):
            losses.append(R.sft_train_step(st, x.ctypes.data, y.ctypes.data, LR))
            out[f"{tag}_losses_{step}"] = np.ctypeslib.as_array(R.sft_get_losses_cpu(st), shape=(N,)).copy()
        if tag == "accum":
            R.sft_apply_grad_sgd(st, LR)
        out[f"{tag}_loss"] = np.array(losses, np.float32)
        out[f"{tag}_weights"] = sample(st, sp.n_layers)
        print(tag, losses, "changed", float((out[f"{tag}_weights"] != start).mean()))
        R.sft_state_free(st)
        S.llmb200_synth_free_qwen3(model)
    path = os.path.join(HERE, "sft_golden_full.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    pkg = entry.load_package()
    R = fast_ref()
    which = sys.argv[1:] or ["lora", "decode", "gemma3", "full"]
    if "lora" in which:
        sft_golden(pkg, R)
    if "decode" in which:
        decode_golden(pkg, R)
    if "gemma3" in which:
        sft_golden_gemma3(pkg, R)
    if "full" in which:
        sft_golden_full(pkg, R)
