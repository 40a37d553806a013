"""Generates tests/golden/wide_golden.npz: greedy decodes of "wide cuts" -- two layers of the benchmarked
architectures at their full widths -- computed by the reference's own C code (oracle/_ref).

    python tests/golden/make_wide_golden.py        (where the reference tree is mounted)

  wide-qwen3   Qwen3-4B widths (hidden 2560, 32/8 heads, head_dim 128, ffn 9728, vocab 151936), 2 layers,
               Q8_0, prompt 16, generate 32, through qwen3_block_forward_cached's call sequence
  wide-gemma3  Gemma3-1B widths (hidden 1152, 4/1 heads, head_dim 256, ffn 6912, vocab 262144 tied), 2
               layers, F16, prompt 16, generate 32, block order of src/nn/fast_inference.c:386-466 on the
               reference's CPU primitives
These are the shapes the benchmarks run (row lengths 2560 / 4096 / 9728, 1152 / 1024 / 6912, the
151936- and 262144-row LM heads with the arg-max across all blocks); the tiny models never reach them.
Per generated step the file keeps the token, the largest |logit|, the gap between the two largest logits
and every 251st logit -- enough for "tokens identical, logits within 1e-2 of max|logit|" without storing
32 x 262144 floats.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import _oracle as O  # noqa: E402

P, G, MAX_SEQ, STRIDE, LAYERS = 16, 32, 64, 251, 2


def summarise(out, tag, prompt, toks, lg):
    srt = np.sort(lg, axis=1)
    out[f"{tag}_prompt"] = prompt
    out[f"{tag}_tokens"] = toks
    out[f"{tag}_logit_absmax"] = np.abs(lg).max(axis=1).astype(np.float32)
    out[f"{tag}_top2_gap"] = (srt[:, -1] - srt[:, -2]).astype(np.float32)
    out[f"{tag}_logit_sample"] = lg[:, ::STRIDE].astype(np.float32)


def main():
    pkg = entry.load_package()
    S = pkg.synth()
    R = O.ref()
    out = {"stride": np.array(STRIDE), "layers": np.array(LAYERS), "max_seq": np.array(MAX_SEQ)}

    sp = pkg.spec("qwen3-4b", gamma_jitter=0.1, n_layers=LAYERS)
    prompt = np.zeros(P, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
    model = S.llmb200_synth_qwen3(C.byref(sp), 8)
    R.ref_requant_qwen3(model, 0)
    toks = np.zeros(G, dtype=np.uint32)
    lg = np.zeros((G, sp.vocab_size), dtype=np.float32)
    n = R.ref_qwen3_generate(model, prompt.ctypes.data, P, toks.ctypes.data, G, MAX_SEQ, None, 0, lg.ctypes.data, None)
    assert n == G
    summarise(out, "qwen3", prompt, toks, lg)
    S.llmb200_synth_free_qwen3(model)
    print("wide-qwen3 tokens", toks[:8], "min top-2 gap", out["qwen3_top2_gap"].min())

    gsp = pkg.spec("gemma3-1b", gamma_jitter=0.1, n_layers=LAYERS)
    gprompt = np.zeros(P, dtype=np.uint32)
    S.llmb200_synth_tokens(gprompt.ctypes.data, P, 4321, gsp.vocab_size)
    gm = S.llmb200_synth_gemma3(C.byref(gsp), 8)
    R.ref_requant_gemma3(gm, 1)
    toks = np.zeros(G, dtype=np.uint32)
    lg = np.zeros((G, gsp.vocab_size), dtype=np.float32)
    n = R.ref_gemma3_generate(gm, 1, gprompt.ctypes.data, P, toks.ctypes.data, G, MAX_SEQ, None, 0, lg.ctypes.data, None)
    assert n == G
    summarise(out, "gemma3", gprompt, toks, lg)
    S.llmb200_synth_free_gemma3(gm)
    print("wide-gemma3 tokens", toks[:8], "min top-2 gap", out["gemma3_top2_gap"].min())

    path = os.path.join(HERE, "wide_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
