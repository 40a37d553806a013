"""Worker of tests/test_gpu_tp.py: tensor parallelism inside ONE process (LLMB200_TP=k in the environment).

The reference's own calls -- inference_state_create, inference_generate, inference_forward_token -- are used
exactly as a single-GPU caller uses them; the library spreads the model over k GPUs with one host thread
each. Tokens and logits must equal the CPU oracle's (or the reference-made vectors for the wide cut).
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import _oracle as O  # noqa: E402


def main():
    arch, use_fp16 = sys.argv[1], int(sys.argv[2])
    k = int(os.environ["LLMB200_TP"])
    pkg = entry.load_package()
    L, S = pkg.lib(), pkg.synth()
    wide = arch == "wide-qwen3"
    golden = np.load(os.path.join(ROOT, "tests", "golden", "wide_golden.npz")) if wide else None
    sp = pkg.spec("qwen3-4b", gamma_jitter=0.1, n_layers=int(golden["layers"])) if wide else pkg.spec(arch, gamma_jitter=0.1)
    gemma = arch.endswith("gemma3")
    model = (S.llmb200_synth_gemma3 if gemma else S.llmb200_synth_qwen3)(C.byref(sp), 4)
    max_seq, P, G = (int(golden["max_seq"]) if wide else 96), 16, 32
    st = (L.inference_state_create_gemma3 if gemma else L.inference_state_create)(model, max_seq, use_fp16)
    assert st, "state create failed"
    L.llmb200_state_set_eos(st, None, 0)
    prompt = np.zeros(P, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
    out = np.zeros(G, dtype=np.uint32)
    for _ in range(2):                                  # the second request reuses slots, flags and epochs
        n = L.inference_generate(st, prompt.ctypes.data_as(pkg.c_u32_p), P, out.ctypes.data_as(pkg.c_u32_p), G)
        assert n == G and L.llmb200_state_error(st) == 0, (n, L.llmb200_state_error(st))
    L.inference_state_reset(st)
    lg = None
    for t in prompt[:4]:
        p = L.inference_forward_token(st, int(t))
        assert p
        lg = np.ctypeslib.as_array(p, shape=(sp.vocab_size,)).copy()
    if wide:
        ref = golden["qwen3_tokens"]
        ok = list(out) == list(ref)
        err = 0.0
    else:
        om = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, max_seq, vocab=sp.vocab_size)
        ref, _ = O.generate(om, prompt, G)
        om2 = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, max_seq, vocab=sp.vocab_size)
        ref_lg = None
        for i, t in enumerate(prompt[:4]):
            ref_lg = O.forward_token(om2, t, i)
        err = float(np.abs(lg - ref_lg).max() / np.abs(ref_lg).max())
        ok = list(out) == list(ref) and err <= 1e-2
    L.inference_state_free(st)
    print("TP_SINGLE", k, "ok" if ok else "MISMATCH", list(out[:8]), list(ref[:8]), err, flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
