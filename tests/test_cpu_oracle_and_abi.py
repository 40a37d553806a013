"""CPU-side checks: the oracle against the golden vectors and the compiled reference, the synthetic-weight
generator, and the C-ABI surface (every declared symbol is exported; no compute call is made here)."""
import ctypes as C
import hashlib
import os
import re
import subprocess

import numpy as np
import pytest

import _oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "decode_golden.npz"))
needs_ref = pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref was not built (reference tree absent)")


# ---------------------------------------------------------------- quantiser golden vectors

def test_q8_and_f16_edge_vectors():
    w = GOLD["edge_w"]
    assert np.array_equal(O.q8_quantize(w), GOLD["edge_q8"])
    assert np.array_equal(O.f16_bits(w), GOLD["edge_f16"])
    blk = GOLD["edge_q8"].reshape(4, 3, 34)
    assert not blk[1, 0].any()                                    # all-zero block: zero scale, zero quants
    assert list(blk[2, 1, 2:11].view(np.int8)) == [127, 1, -1, 2, -2, 3, -3, 127, -127]   # ties away from zero
    assert blk[3, 2, :2].view(np.uint16)[0] == 0x7C00             # scale overflows binary16 to +inf


def test_q8_dequant_and_matvec_definitions():
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((16, 256)) * 0.02).astype(np.float32)
    x = rng.standard_normal(256).astype(np.float32)
    blocks = O.q8_quantize(w)
    deq = O.q8_dequantize(blocks, 16, 256)
    b = blocks.reshape(-1, 34)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    q = b[:, 2:].copy().view(np.int8).astype(np.float32)
    assert np.array_equal(deq.reshape(-1, 32), q * d)             # w = (float)q * f16(d)
    assert np.abs(deq - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-6
    y_blockwise = O.q8_matvec(blocks, x, 16, 256)                  # GPU-kernel association
    y_dequant = O.linear(deq, x)                                   # CPU-reference association
    assert np.allclose(y_blockwise, y_dequant, rtol=0, atol=2e-5 * np.abs(y_dequant).max())


def test_synth_generator_is_reproducible(pkg, synth):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    n = sp.n_q_heads * sp.head_dim * sp.d_model
    a = np.empty(n, dtype=np.float32)
    synth.llmb200_synth_normal(a.ctypes.data, n, sp.seed, synth.llmb200_synth_tensor_id(0, 0), 0.0, 0.02, 1)
    assert hashlib.sha256(a.tobytes()).digest() == GOLD["tiny_q0_weight_sha256"].tobytes()
    b = np.empty(n, dtype=np.float32)
    synth.llmb200_synth_normal(b.ctypes.data, n, sp.seed, synth.llmb200_synth_tensor_id(0, 0), 0.0, 0.02, 7)
    assert np.array_equal(a, b)                                    # thread count does not matter
    c = np.empty(1001, dtype=np.float32)
    synth.llmb200_synth_normal_range(c.ctypes.data, 12345, 1001, sp.seed, synth.llmb200_synth_tensor_id(0, 0), 0.0, 0.02, 1)
    assert np.array_equal(c, a[12345:12345 + 1001])                # any sub-range can be generated on its own
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    z = a / 0.02
    assert abs(float((z ** 4).mean()) - 3.0) < 0.1                 # normal kurtosis
    assert hashlib.sha256(O.q8_quantize(a.reshape(-1, sp.d_model)).tobytes()).digest() == GOLD["tiny_q0_q8_sha256"].tobytes()
    t = np.zeros(16, dtype=np.uint32)
    synth.llmb200_synth_tokens(t.ctypes.data, 16, 4321, sp.vocab_size)
    assert np.array_equal(t, GOLD["tiny_prompt"])


# ---------------------------------------------------------------- decode golden vectors

@pytest.mark.parametrize("use_fp16,tag", [(0, "q8"), (1, "f16")])
def test_oracle_reproduces_reference_tiny_qwen3(pkg, synth, use_fp16, tag):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    om = O.model_qwen3(model, use_fp16, 64, vocab=sp.vocab_size)
    toks, lg = O.generate(om, GOLD["tiny_prompt"], 32, want_logits=True)
    assert list(toks) == list(GOLD[f"tiny_{tag}_tokens"])
    gold = GOLD[f"tiny_{tag}_logits"]
    assert np.abs(lg[GOLD["logit_steps"]] - gold).max() <= 1e-5 * np.abs(gold).max()
    del om
    synth.llmb200_synth_free_qwen3(model)


def test_oracle_reproduces_reference_tiny_gemma3(pkg, synth):
    sp = pkg.spec("tiny-gemma3", gamma_jitter=0.1)
    model = synth.llmb200_synth_gemma3(C.byref(sp), 4)
    om = O.model_gemma3(model, 1, 96, vocab=sp.vocab_size)
    toks, lg = O.generate(om, GOLD["gemma_prompt"], 32, want_logits=True)
    assert list(toks) == list(GOLD["gemma_f16_tokens"])
    gold = GOLD["gemma_f16_logits"]
    assert np.abs(lg[GOLD["logit_steps"]] - gold).max() <= 1e-5 * np.abs(gold).max()
    del om
    synth.llmb200_synth_free_gemma3(model)


def test_oracle_generate_semantics(pkg, synth):
    sp = pkg.spec("tiny-qwen3", n_layers=1, vocab_size=256)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 2)
    om = O.model_qwen3(model, 0, 24, vocab=sp.vocab_size)
    prompt = np.arange(8, dtype=np.uint32)
    full, _ = O.generate(om, prompt, 64)
    assert len(full) == 17                                           # 8 prompt + 16 forwards fill the 24-slot cache
    eos_tok = int(full[4])
    cut, _ = O.generate(om, prompt, 64, eos=[eos_tok])
    assert list(cut) == list(full[:list(full).index(eos_tok) + 1])   # EOS is emitted, nothing after it
    one, _ = O.generate(om, prompt, 1)
    assert list(one) == [full[0]]
    # F16 KV cache option: small, bounded change of the logits
    om16 = O.model_qwen3(model, 0, 24, vocab=sp.vocab_size, kv_f16=True)
    a = O.forward_token(om, 3, 0)
    b = O.forward_token(om16, 3, 0)
    assert 0 < np.abs(a - b).max() <= 5e-3 * np.abs(a).max() or np.array_equal(a, b)
    del om, om16
    synth.llmb200_synth_free_qwen3(model)


# ---------------------------------------------------------------- the compiled reference itself

@needs_ref
def test_oracle_matches_compiled_reference_quantiser(synth):
    for rows, cols, tid in ((64, 2560, 1), (5, 9728, 2), (300, 512, 3)):
        w = np.empty((rows, cols), dtype=np.float32)
        synth.llmb200_synth_normal(w.ctypes.data, w.size, 9, tid, 0.0, 0.02, 2)
        w[0, :64] *= 1e-6
        blocks = np.zeros(rows * (cols // 32) * 34, dtype=np.uint8)
        O.ref().ref_q8_blocks(w.ctypes.data, rows, cols, blocks.ctypes.data)
        assert np.array_equal(blocks, O.q8_quantize(w))
        bits = np.zeros((rows, cols), dtype=np.uint16)
        O.ref().ref_f16_bits(w.ctypes.data, rows, cols, bits.ctypes.data)
        assert np.array_equal(bits, O.f16_bits(w))
        x = np.empty(cols, dtype=np.float32)
        synth.llmb200_synth_normal(x.ctypes.data, cols, 9, 50 + tid, 0.0, 1.0, 1)
        y = np.zeros(rows, dtype=np.float32)
        O.ref().ref_linear(w.ctypes.data, x.ctypes.data, y.ctypes.data, rows, cols)
        assert np.array_equal(y, O.linear(w, x))


@needs_ref
def test_oracle_matches_compiled_reference_decode(pkg, synth):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1, n_layers=2, seed=77)
    prompt = np.zeros(12, dtype=np.uint32)
    synth.llmb200_synth_tokens(prompt.ctypes.data, 12, 5, sp.vocab_size)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    om = O.model_qwen3(model, 0, 32, vocab=sp.vocab_size)
    toks, lg = O.generate(om, prompt, 12, want_logits=True)
    O.ref().ref_requant_qwen3(model, 0)
    rt = np.zeros(12, dtype=np.uint32)
    rl = np.zeros((12, sp.vocab_size), dtype=np.float32)
    n = O.ref().ref_qwen3_generate(model, prompt.ctypes.data, 12, rt.ctypes.data, 12, 32, None, 0, rl.ctypes.data, None)
    assert n == 12 and list(rt) == list(toks)
    assert np.array_equal(rl, lg)
    del om
    synth.llmb200_synth_free_qwen3(model)


@needs_ref
def test_boundary_struct_layouts_match_reference_headers(synth):
    a, b = (C.c_size_t * 128)(), (C.c_size_t * 128)()
    na, nb = synth.llmb200_abi_layout(a, 128), O.ref().ref_abi_layout(b, 128)
    assert na == nb and na > 60
    assert list(a[:na]) == list(b[:nb])


# ---------------------------------------------------------------- the C-ABI surface

def declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    text = re.sub(r"typedef\s+struct[^;{]*\{.*?\}[^;]*;", "", text, flags=re.S)
    text = re.sub(r"typedef\s+enum[^;{]*\{.*?\}[^;]*;", "", text, flags=re.S)
    text = re.sub(r"enum\s*\{.*?\};", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)))


def exported(path):
    out = subprocess.run(["nm", "-D", "--defined-only", path], check=True, stdout=subprocess.PIPE, text=True).stdout
    return {line.split()[-1] for line in out.splitlines() if " T " in line}


def test_every_declared_symbol_is_exported_and_bound(pkg):
    main_syms, synth_syms = exported(pkg.build.LIB), exported(pkg.build.LIB_SYNTH)
    for header, names in pkg.SYMBOLS_MAIN.items():
        assert declared_functions(header) == sorted(names), header
        assert not [n for n in names if n not in main_syms], header
    for header, names in pkg.SYMBOLS_SYNTH.items():
        assert declared_functions(header) == sorted(names), header
        assert not [n for n in names if n not in synth_syms], header
    L = pkg.lib()                                                   # loads without a GPU
    for names in pkg.SYMBOLS_MAIN.values():
        for n in names:
            assert getattr(L, n).argtypes is not None


def test_library_refuses_to_run_without_a_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = pkg.lib()
    assert L.fast_metal_init() != 0                                 # no CPU fallback: init fails loudly
    assert not L.metal_buf_create(16)
    cfg = pkg.config_of(pkg.spec("tiny-qwen3"), pkg.MODEL_QWEN3, 32, 0)
    assert not L.llmb200_state_begin(C.byref(cfg))
    w = np.zeros((2, 32), dtype=np.float32)
    assert not L.wmat_create_q8(w.ctypes.data_as(pkg.c_float_p), 2, 32)


def test_product_never_touches_the_oracle():
    bad = []
    for base, _, files in os.walk(os.path.join(ROOT, "llm.metal_b200")):
        if os.path.basename(base) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".c", ".cu", ".cuh", ".h")):
                if re.search(r"oracle/|liboracle|_oracle|libllmref|_work/", open(os.path.join(base, f), errors="ignore").read()):
                    bad.append(f)
    assert not bad


# ---------------------------------------------------------------- the drop-in program

DROP_IN = os.path.join(ROOT, "tests", "c_api", "_bin", "drop_in")


@pytest.mark.skipif(not os.path.exists(DROP_IN), reason="tests/c_api/_bin/drop_in was not built (reference tree absent)")
def test_drop_in_program_links_and_fails_loudly_without_a_gpu():
    """tests/c_api/drop_in.c includes the reference's own headers and links against libllmb200.so: every
    engine symbol it uses resolved at build time. Without a CUDA device it must stop at the first engine
    call with the library's message -- there is no CPU path to fall back to."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU suite runs the program for real")
    r = subprocess.run([DROP_IN], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert r.returncode == 3, (r.returncode, r.stderr[-500:])
    assert "no CUDA device available" in r.stderr and "no CPU path" in r.stderr
    assert "DROP_IN ok" not in r.stdout
