"""Generates tests/golden/decode_golden.npz from the reference's own C code (oracle/_ref).

Run in a container where the reference tree is mounted (oracle/Makefile builds
oracle/_ref/libllmref.so from it):

    python tests/golden/make_golden.py

What is recorded (all on seeded synthetic models, see llmb200_synth.h):
  * Q8_0 blocks and binary16 bits the reference's wmat.c produces for a small
    matrix with edge-case values, plus SHA-256 of the blocks of a whole layer
    matrix of the tiny Qwen3 model;
  * greedy tokens (prompt 16, generate 32) and the logits of three steps of the
    tiny Qwen3 configuration, Q8_0 and F16, computed by the reference's CPU
    layers (rms_norm_forward, gqa_forward_cached, linear_forward, ...);
  * the same for a small Gemma3-shaped model (F16).
"""
import ctypes as C
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import _oracle as O  # noqa: E402

LOGIT_STEPS = [0, 15, 31]


def edge_matrix(S):
    w = np.empty((4, 96), dtype=np.float32)
    S.llmb200_synth_normal(w.ctypes.data, w.size, 77, 3, 0.0, 0.02, 1)
    w[1, :32] = 0.0
    w[2, 32:41] = [127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5]
    w[2, 41:64] = 0.0
    w[3, 70] = 3.0e38
    w[0, 5] = 1e-41
    return w


def main():
    pkg = entry.load_package()
    S = pkg.synth()
    R = O.ref()
    out = {}

    w = edge_matrix(S)
    blocks = np.zeros(4 * 3 * 34, dtype=np.uint8)
    R.ref_q8_blocks(w.ctypes.data, 4, 96, blocks.ctypes.data)
    bits = np.zeros((4, 96), dtype=np.uint16)
    R.ref_f16_bits(w.ctypes.data, 4, 96, bits.ctypes.data)
    out["edge_w"], out["edge_q8"], out["edge_f16"] = w, blocks, bits

    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    q = np.empty((sp.n_q_heads * sp.head_dim, sp.d_model), dtype=np.float32)
    S.llmb200_synth_normal(q.ctypes.data, q.size, sp.seed, S.llmb200_synth_tensor_id(0, 0), 0.0, 0.02, 1)
    qb = np.zeros(q.size // 32 * 34, dtype=np.uint8)
    R.ref_q8_blocks(q.ctypes.data, q.shape[0], q.shape[1], qb.ctypes.data)
    out["tiny_q0_weight_sha256"] = np.frombuffer(hashlib.sha256(q.tobytes()).digest(), dtype=np.uint8)
    out["tiny_q0_q8_sha256"] = np.frombuffer(hashlib.sha256(qb.tobytes()).digest(), dtype=np.uint8)

    prompt = np.zeros(16, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, 16, 4321, sp.vocab_size)
    out["tiny_prompt"] = prompt
    for use_fp16, tag in ((0, "q8"), (1, "f16")):
        model = S.llmb200_synth_qwen3(C.byref(sp), 4)
        R.ref_requant_qwen3(model, use_fp16)
        toks = np.zeros(32, dtype=np.uint32)
        lg = np.zeros((32, sp.vocab_size), dtype=np.float32)
        n = R.ref_qwen3_generate(model, prompt.ctypes.data, 16, toks.ctypes.data, 32, 64, None, 0, lg.ctypes.data, None)
        assert n == 32
        # cross-check the cached driver against the reference's full causal recompute
        seq = np.concatenate([prompt, toks[:4]]).astype(np.uint32)
        full = np.zeros(sp.vocab_size, dtype=np.float32)
        R.ref_qwen3_forward_full(model, seq.ctypes.data, len(seq), full.ctypes.data)
        assert np.abs(full - lg[4]).max() < 1e-4, np.abs(full - lg[4]).max()
        out[f"tiny_{tag}_tokens"] = toks
        out[f"tiny_{tag}_logits"] = lg[LOGIT_STEPS]
        S.llmb200_synth_free_qwen3(model)

    gsp = pkg.spec("tiny-gemma3", gamma_jitter=0.1)
    gprompt = np.zeros(24, dtype=np.uint32)
    S.llmb200_synth_tokens(gprompt.ctypes.data, 24, 4321, gsp.vocab_size)
    gm = S.llmb200_synth_gemma3(C.byref(gsp), 4)
    R.ref_requant_gemma3(gm, 1)
    toks = np.zeros(32, dtype=np.uint32)
    lg = np.zeros((32, gsp.vocab_size), dtype=np.float32)
    n = R.ref_gemma3_generate(gm, 1, gprompt.ctypes.data, 24, toks.ctypes.data, 32, 96, None, 0, lg.ctypes.data, None)
    assert n == 32
    out["gemma_prompt"], out["gemma_f16_tokens"], out["gemma_f16_logits"] = gprompt, toks, lg[LOGIT_STEPS]
    S.llmb200_synth_free_gemma3(gm)

    out["logit_steps"] = np.array(LOGIT_STEPS)
    path = os.path.join(HERE, "decode_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
