"""End-to-end parity of the decode engine (through the reference-facing C API) against the CPU oracle.

Bars (the north-star's): Q8_0 bytes on the device bit-exact; logits within 1e-2 of max|logit| at every
step; greedy tokens identical over the first 32 generated.
"""
import ctypes as C
import os

import numpy as np
import pytest

import _oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def make_prompt(synth, n, vocab, seed=4321):
    p = np.zeros(n, dtype=np.uint32)
    synth.llmb200_synth_tokens(p.ctypes.data, n, seed, vocab)
    return p


def gpu_generate(lib, pkg, state, prompt, max_gen):
    out = np.zeros(max_gen, dtype=np.uint32)
    n = lib.inference_generate(state, prompt.ctypes.data_as(pkg.c_u32_p), len(prompt), out.ctypes.data_as(pkg.c_u32_p), max_gen)
    assert lib.llmb200_state_error(state) == 0
    return out[:n]


def gpu_logits_trace(lib, state, tokens, vocab):
    """Feeds `tokens` one by one through inference_forward_token; returns logits [len(tokens), V]."""
    lib.inference_state_reset(state)
    rows = []
    for t in tokens:
        p = lib.inference_forward_token(state, int(t))
        assert p
        rows.append(np.ctypeslib.as_array(p, shape=(vocab,)).copy())
    return np.stack(rows)


def check_against_oracle(lib, pkg, synth, model, omodel, state, vocab, P, G, max_seq):
    prompt = make_prompt(synth, P, vocab)
    lib.llmb200_state_set_eos(state, None, 0)
    got = gpu_generate(lib, pkg, state, prompt, G)
    ref_tok, ref_lg = O.generate(omodel, prompt, G, vocab=vocab, want_logits=True)
    assert len(got) == G == len(ref_tok)
    # logits along the *reference's* token path, so a single flipped token cannot hide later errors
    seq = np.concatenate([prompt, ref_tok[:-1]])
    lg = gpu_logits_trace(lib, state, seq, vocab)[P - 1:]
    rel = np.abs(lg - ref_lg).max(axis=1) / np.abs(ref_lg).max(axis=1)
    assert rel.max() <= 1e-2, f"logit error {rel.max():.3e}"
    if list(got) != list(ref_tok):
        k = next(i for i in range(G) if got[i] != ref_tok[i])
        top2 = np.sort(ref_lg[k])[-2:]
        pytest.fail(f"greedy token {k} differs: gpu {got[k]} vs oracle {ref_tok[k]}; oracle top-2 gap {top2[1] - top2[0]:.3e}, "
                    f"logit error at that step {np.abs(lg[k] - ref_lg[k]).max():.3e}")
    return rel.max()


@pytest.mark.parametrize("use_fp16", [0, 1])
def test_tiny_qwen3_matches_oracle(lib, pkg, synth, use_fp16):
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    state = lib.inference_state_create(model, 64, use_fp16)
    assert state
    try:
        omodel = O.model_qwen3(model, use_fp16, 64, vocab=sp.vocab_size)
        check_against_oracle(lib, pkg, synth, model, omodel, state, sp.vocab_size, 16, 32, 64)
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)


def test_tiny_qwen3_device_weights_bit_exact(lib, pkg, synth):
    sp = pkg.spec("tiny-qwen3")
    model_p = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    state = lib.inference_state_create(model_p, 32, 0)
    assert state
    try:
        D, hd, IS = sp.d_model, sp.head_dim, sp.intermediate_size

        def gen(layer, which, rows, cols):
            w = np.empty((rows, cols), dtype=np.float32)
            synth.llmb200_synth_normal(w.ctypes.data, w.size, sp.seed, synth.llmb200_synth_tensor_id(layer, which), 0.0, 0.02, 4)
            return w

        def export(layer, which):
            n = lib.llmb200_state_export_weight(state, layer, which, None, 0)
            buf = np.zeros(n, dtype=np.uint8)
            assert lib.llmb200_state_export_weight(state, layer, which, buf.ctypes.data, n) == n
            return buf
        for layer in (0, sp.n_layers - 1):
            q, k, v = gen(layer, 0, sp.n_q_heads * hd, D), gen(layer, 1, sp.n_kv_heads * hd, D), gen(layer, 2, sp.n_kv_heads * hd, D)
            assert np.array_equal(export(layer, 0), O.q8_quantize(np.concatenate([q, k, v])))
            assert np.array_equal(export(layer, 1), O.q8_quantize(gen(layer, 3, D, sp.n_q_heads * hd)))
            g, u = gen(layer, 4, IS, D), gen(layer, 5, IS, D)
            gu = np.empty((2 * IS, D), dtype=np.float32)
            gu[0::2], gu[1::2] = g, u
            assert np.array_equal(export(layer, 2), O.q8_quantize(gu))
            assert np.array_equal(export(layer, 3), O.q8_quantize(gen(layer, 6, D, IS)))
        lm = gen(0, 101, sp.vocab_size, D)
        assert np.array_equal(export(0, 4), O.q8_quantize(lm))
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model_p)


@pytest.mark.parametrize("use_fp16", [1, 0])
def test_tiny_gemma3_matches_oracle(lib, pkg, synth, use_fp16):
    sp = pkg.spec("tiny-gemma3", gamma_jitter=0.1)
    model = synth.llmb200_synth_gemma3(C.byref(sp), 8)
    state = lib.inference_state_create_gemma3(model, 96, use_fp16)
    assert state
    try:
        assert lib.inference_state_model_type(state) == pkg.MODEL_GEMMA3
        omodel = O.model_gemma3(model, use_fp16, 96, vocab=sp.vocab_size)
        check_against_oracle(lib, pkg, synth, model, omodel, state, sp.vocab_size, 24, 32, 96)
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_gemma3(model)


FAST = np.load(os.path.join(ROOT, "tests", "golden", "fast_decode_golden.npz"))


@pytest.mark.parametrize("arch", ["tiny-qwen3", "tiny-gemma3"])
@pytest.mark.parametrize("use_fp16", [0, 1])
def test_tiny_models_match_the_reference_engine_vectors(lib, pkg, synth, arch, use_fp16):
    """Tokens and logits the reference's own fast_inference.c produced (tests/golden/make_sft_golden.py)."""
    gemma = arch.endswith("gemma3")
    sp = pkg.spec(arch, gamma_jitter=0.1)
    model = (synth.llmb200_synth_gemma3 if gemma else synth.llmb200_synth_qwen3)(C.byref(sp), 8)
    state = (lib.inference_state_create_gemma3 if gemma else lib.inference_state_create)(model, int(FAST["max_seq"]), use_fp16)
    assert state
    try:
        tag = f"{arch}_{'f16' if use_fp16 else 'q8'}"
        prompt = FAST[f"{arch}_prompt"]
        lib.llmb200_state_set_eos(state, None, 0)
        got = gpu_generate(lib, pkg, state, prompt, int(FAST["gen_len"]))
        lg = gpu_logits_trace(lib, state, prompt, sp.vocab_size)[-1]
        ref = FAST[f"{tag}_logits"]
        assert np.abs(lg - ref).max() <= 1e-2 * np.abs(ref).max()
        assert list(got) == list(FAST[f"{tag}_tokens"])
    finally:
        lib.inference_state_free(state)
        (synth.llmb200_synth_free_gemma3 if gemma else synth.llmb200_synth_free_qwen3)(model)


def test_generate_semantics(lib, pkg, synth):
    """Count, EOS and cache-limit behaviour of inference_generate (src/nn/fast_inference.c:614-675)."""
    sp = pkg.spec("tiny-qwen3")
    model = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    state = lib.inference_state_create(model, 40, 0)
    assert state
    try:
        assert lib.inference_state_vocab_size(state) == sp.vocab_size
        assert lib.inference_state_model_type(state) == pkg.MODEL_QWEN3
        prompt = make_prompt(synth, 16, sp.vocab_size)
        lib.llmb200_state_set_eos(state, None, 0)
        full = gpu_generate(lib, pkg, state, prompt, 64)
        # stops when the KV cache is full: 16 prompt + 24 forwards = 40 positions, 25 tokens out
        assert len(full) == 25
        again = gpu_generate(lib, pkg, state, prompt, 64)
        assert list(full) == list(again)               # the request resets the state
        # EOS: the EOS token is returned as the last token and nothing follows it
        eos = (C.c_int * 1)(int(full[5]))
        lib.llmb200_state_set_eos(state, eos, 1)
        cut = gpu_generate(lib, pkg, state, prompt, 64)
        first = list(full).index(full[5])
        assert list(cut) == list(full[:first + 1])
        # max_gen_len = 1: only the prefill argmax
        lib.llmb200_state_set_eos(state, None, 0)
        assert list(gpu_generate(lib, pkg, state, prompt, 1)) == [full[0]]
        # one-token prompt
        one = gpu_generate(lib, pkg, state, prompt[:1], 4)
        om = O.model_qwen3(model, 0, 40, vocab=sp.vocab_size)
        ref, _ = O.generate(om, prompt[:1], 4)
        assert list(one) == list(ref)
        # bad input is refused without touching the device
        assert lib.inference_generate(state, prompt.ctypes.data_as(pkg.c_u32_p), 0, full.ctypes.data_as(pkg.c_u32_p), 4) == 0
        big = np.full(41, 1, dtype=np.uint32)
        assert lib.inference_generate(state, big.ctypes.data_as(pkg.c_u32_p), 41, full.ctypes.data_as(pkg.c_u32_p), 4) == 0
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)


def test_max_seq_is_clamped_and_long_context(lib, pkg, synth):
    """max_seq_len > 4096 is clamped (src/nn/fast_inference.c:183-186); attention over a long cache stays exact."""
    sp = pkg.spec("tiny-qwen3", n_layers=1, vocab_size=512)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    state = lib.inference_state_create(model, 5000, 0)
    assert state
    try:
        P = 700
        prompt = make_prompt(synth, P, sp.vocab_size)
        lib.llmb200_state_set_eos(state, None, 0)
        got = gpu_generate(lib, pkg, state, prompt, 8)
        om = O.model_qwen3(model, 0, P + 8, vocab=sp.vocab_size)
        ref, _ = O.generate(om, prompt, 8)
        assert list(got) == list(ref)
        big = np.zeros(4097, dtype=np.uint32)
        out = np.zeros(2, dtype=np.uint32)
        assert lib.inference_generate(state, big.ctypes.data_as(pkg.c_u32_p), 4097, out.ctypes.data_as(pkg.c_u32_p), 2) == 0
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)


def test_load_eos_from_config(lib, pkg, synth, tmp_path):
    sp = pkg.spec("tiny-qwen3", n_layers=1, vocab_size=512)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    state = lib.inference_state_create(model, 32, 0)
    assert state
    try:
        prompt = make_prompt(synth, 8, sp.vocab_size)
        lib.llmb200_state_set_eos(state, None, 0)
        full = gpu_generate(lib, pkg, state, prompt, 12)
        (tmp_path / "config.json").write_text('{"model_type": "qwen3", "eos_token_id": [%d, 999999]}' % int(full[3]))
        lib.inference_state_load_eos(state, str(tmp_path).encode())
        cut = gpu_generate(lib, pkg, state, prompt, 12)
        assert list(cut) == list(full[:list(full).index(full[3]) + 1])
        (tmp_path / "config.json").write_text('{"eos_token_id": -1}')
        lib.inference_state_load_eos(state, str(tmp_path / "model.safetensors").encode())
        assert list(gpu_generate(lib, pkg, state, prompt, 12)) == list(full)
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)


def test_wmat_api_roundtrip(lib, pkg, synth):
    """wmat_create_q8 / metal_buf_ptr give back the reference's canonical bytes (src/nn/wmat.c:47-75)."""
    rows, cols = 96, 512
    w = np.empty((rows, cols), dtype=np.float32)
    synth.llmb200_synth_normal(w.ctypes.data, w.size, 1, 2, 0.0, 0.02, 1)
    wm = lib.wmat_create_q8(w.ctypes.data_as(pkg.c_float_p), rows, cols)
    assert wm and wm.contents.rows == rows and wm.contents.cols == cols and wm.contents.nb == cols // 32
    p = lib.metal_buf_ptr(wm.contents.mbuf)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(rows * (cols // 32) * 34,)).copy()
    assert np.array_equal(got, O.q8_quantize(w))
    lib.wmat_free(wm)
    wf = lib.wmat_convert(w.ctypes.data_as(pkg.c_float_p), rows, cols, 1)
    assert wf and wf.contents.nb == 0
    p = lib.metal_buf_ptr(wf.contents.mbuf)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=(rows, cols)).copy()
    assert np.array_equal(got, O.f16_bits(w))
    lib.wmat_free(wf)
    b = lib.metal_buf_from_data(w.ctypes.data, w.nbytes)
    got = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(b), C.POINTER(C.c_float)), shape=(rows, cols)).copy()
    assert np.array_equal(got, w)
    lib.metal_buf_free(b)
    lib.metal_buf_free(None)
    assert not lib.wmat_create_q8(w.ctypes.data_as(pkg.c_float_p), rows, 40)     # cols % 32 != 0


def test_whole_token_kernel_gives_the_same_tokens(lib, pkg, synth, monkeypatch):
    """The persistent whole-token kernel (the default) and the graph of one kernel per stage (LLMB200_TOKEN_KERNEL=0)
    must produce the same tokens."""
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    prompt = make_prompt(synth, 16, sp.vocab_size)
    outs = []
    try:
        for flag in ("0", "1"):
            monkeypatch.setenv("LLMB200_TOKEN_KERNEL", flag)
            state = lib.inference_state_create(model, 64, 0)
            assert state
            lib.llmb200_state_set_eos(state, None, 0)
            outs.append(list(gpu_generate(lib, pkg, state, prompt, 32)))
            assert lib.llmb200_state_graph_kernels(state, 1) == (1 if flag == "1" else 5 * sp.n_layers + 1)
            lib.inference_state_free(state)
    finally:
        synth.llmb200_synth_free_qwen3(model)
    assert outs[0] == outs[1]


# ---------------------------------------------------------------------------------------------------
# Wide cuts: two layers of the benchmarked architectures at full width, against vectors the reference's
# own C code produced (tests/golden/wide_golden.npz, made by tests/golden/make_wide_golden.py). These are
# the kernel configurations the benchmarks run: rows of 2560 / 4096 / 9728 (Q8_0) and 1152 / 1024 / 6912
# (F16) columns, head_dim 128 and 256, the 151936- and 262144-row LM heads with the arg-max over all blocks.
# ---------------------------------------------------------------------------------------------------
WIDE = np.load(os.path.join(ROOT, "tests", "golden", "wide_golden.npz"))


def check_wide(lib, pkg, state, tag, vocab):
    prompt, ref_tok = WIDE[f"{tag}_prompt"], WIDE[f"{tag}_tokens"]
    absmax, gap, sample, stride = WIDE[f"{tag}_logit_absmax"], WIDE[f"{tag}_top2_gap"], WIDE[f"{tag}_logit_sample"], int(WIDE["stride"])
    P, G = len(prompt), len(ref_tok)
    lib.llmb200_state_set_eos(state, None, 0)
    got = gpu_generate(lib, pkg, state, prompt, G)
    # logits along the reference's token path
    seq = np.concatenate([prompt, ref_tok[:-1]])
    lg = gpu_logits_trace(lib, state, seq, vocab)[P - 1:]
    rel = np.abs(lg[:, ::stride] - sample).max(axis=1) / absmax
    assert rel.max() <= 1e-2, f"logit error {rel.max():.3e}"
    assert np.abs(np.abs(lg).max(axis=1) - absmax).max() <= 1e-2 * absmax.max()
    if list(got) != list(ref_tok):
        k = next(i for i in range(G) if got[i] != ref_tok[i])
        pytest.fail(f"greedy token {k} differs: gpu {got[k]} vs reference {ref_tok[k]}; reference top-2 gap {gap[k]:.3e}, "
                    f"sampled logit error at that step {rel[k] * absmax[k]:.3e}")


@pytest.mark.parametrize("token_kernel", ["1", "0"])
def test_wide_cut_qwen3_matches_reference_golden(lib, pkg, synth, monkeypatch, token_kernel):
    monkeypatch.setenv("LLMB200_TOKEN_KERNEL", token_kernel)
    sp = pkg.spec("qwen3-4b", gamma_jitter=0.1, n_layers=int(WIDE["layers"]))
    model = synth.llmb200_synth_qwen3(C.byref(sp), 8)
    state = lib.inference_state_create(model, int(WIDE["max_seq"]), 0)
    lib.metal_flush()
    synth.llmb200_synth_free_qwen3(model)              # the state keeps its own device copies
    assert state
    try:
        assert lib.llmb200_state_graph_kernels(state, 1) == (1 if token_kernel == "1" else 5 * sp.n_layers + 1)
        check_wide(lib, pkg, state, "qwen3", sp.vocab_size)
    finally:
        lib.inference_state_free(state)


@pytest.mark.parametrize("token_kernel", ["1", "0"])
def test_wide_cut_gemma3_matches_reference_golden(lib, pkg, synth, monkeypatch, token_kernel):
    monkeypatch.setenv("LLMB200_TOKEN_KERNEL", token_kernel)
    sp = pkg.spec("gemma3-1b", gamma_jitter=0.1, n_layers=int(WIDE["layers"]))
    model = synth.llmb200_synth_gemma3(C.byref(sp), 8)
    state = lib.inference_state_create_gemma3(model, int(WIDE["max_seq"]), 1)
    lib.metal_flush()
    synth.llmb200_synth_free_gemma3(model)
    assert state
    try:
        check_wide(lib, pkg, state, "gemma3", sp.vocab_size)
    finally:
        lib.inference_state_free(state)


def test_a_rank_that_never_arrives_runs_into_the_bounded_waits(lib, pkg, synth, monkeypatch):
    """Failure detection without a GPU fault: a two-rank state connected to itself waits for partial sums nobody
    writes. Every wait must give up after its iteration limit, the launch must complete and the error word must be
    set; the process and the device stay usable (the next test creates a fresh state)."""
    monkeypatch.setenv("LLMB200_SPIN_LIMIT", "2000")
    sp = pkg.spec("tiny-qwen3")
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    assert lib.llmb200_set_tp(0, 2) == 0
    try:
        state = lib.inference_state_create(model, 32, 0)
    finally:
        assert lib.llmb200_set_tp(0, 1) == 0
    assert state
    try:
        assert lib.llmb200_state_connect_loopback(state) == 0
        assert lib.llmb200_state_error(state) == 0
        p = lib.inference_forward_token(state, 5)          # completes: nothing hangs
        assert p
        assert lib.llmb200_state_error(state) != 0
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)
    # a healthy state afterwards: the device context is intact
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    state = lib.inference_state_create(model, 32, 0)
    assert state
    try:
        assert lib.inference_forward_token(state, 5) and lib.llmb200_state_error(state) == 0
    finally:
        lib.inference_state_free(state)
        synth.llmb200_synth_free_qwen3(model)


def test_layer_containers_roundtrip(lib, pkg, synth):
    """layers_convert_upload / norm_upload / layers_free (src/nn/wmat.c:87-156): seven matrices and the norm weights of
    every layer, converted and uploaded in bulk; the device bytes are the reference quantiser's."""
    D, hd, Hq, Hkv, IS, n_layers = 256, 64, 4, 2, 512, 2
    shapes = dict(q_proj=(Hq * hd, D), k_proj=(Hkv * hd, D), v_proj=(Hkv * hd, D), o_proj=(D, Hq * hd),
                  gate_proj=(IS, D), up_proj=(IS, D), down_proj=(D, IS))
    refs = (pkg.LayerWeightRef * n_layers)()
    keep = []
    fp = pkg.c_float_p
    for l in range(n_layers):
        for i, (name, (r, c)) in enumerate(shapes.items()):
            w = np.empty((r, c), dtype=np.float32)
            synth.llmb200_synth_normal(w.ctypes.data, w.size, 5, 100 * l + i, 0.0, 0.02, 1)
            keep.append((l, name, w))
            setattr(refs[l], name, pkg.WeightRef(w.ctypes.data_as(fp), r, c))
        g = (1.0 + 0.1 * np.arange(D, dtype=np.float32) / D).astype(np.float32)
        gq = np.linspace(0.5, 1.5, hd).astype(np.float32)
        keep += [(l, "g", g), (l, "gq", gq)]
        refs[l].input_norm_g, refs[l].post_attn_norm_g = g.ctypes.data_as(fp), g.ctypes.data_as(fp)
        refs[l].q_norm_g, refs[l].k_norm_g = gq.ctypes.data_as(fp), gq.ctypes.data_as(fp)
        refs[l].d_model, refs[l].head_dim = D, hd

    class LayerW(C.Structure):                       # LayerW of include/llmb200_wmat.h
        _fields_ = [(n, C.POINTER(pkg.WMat)) for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")] + \
                   [(n, C.c_void_p) for n in ("input_norm_g", "post_attn_norm_g", "pre_ff_norm_g", "post_ff_norm_g", "q_norm_g", "k_norm_g")]

    for use_fp16 in (0, 1):
        lw = lib.layers_convert_upload(refs, n_layers, use_fp16)
        assert lw
        arr = C.cast(lw, C.POINTER(LayerW))
        for l, name, w in keep:
            if name in shapes:
                m = getattr(arr[l], name).contents
                assert (m.rows, m.cols) == w.shape and m.nb == (0 if use_fp16 else w.shape[1] // 32)
                p = lib.metal_buf_ptr(m.mbuf)
                if use_fp16:
                    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=w.shape).copy()
                    assert np.array_equal(got, O.f16_bits(w))
                else:
                    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(w.size // 32 * 34,)).copy()
                    assert np.array_equal(got, O.q8_quantize(w))
        g0 = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(arr[0].input_norm_g), fp), shape=(D,)).copy()
        assert np.array_equal(g0, keep[7][2])
        assert not arr[0].pre_ff_norm_g and not arr[0].post_ff_norm_g        # absent norms stay NULL
        lib.layers_free(lw, n_layers)
    nb = lib.norm_upload(keep[7][2].ctypes.data_as(fp), D)
    assert nb
    assert np.array_equal(np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(nb), fp), shape=(D,)), keep[7][2])
    lib.metal_buf_free(nb)


def test_drop_in_program_built_against_the_reference_headers():
    """tests/c_api/drop_in.c: a caller compiled against the reference's own qwen3.h / fast_inference.h /
    fast_sft.h, with a model made by the reference's qwen3_create, linked against libllmb200.so. Decodes in
    Q8_0 and F16 (tokens identical to the reference's CPU path), trains four LoRA steps, takes a decode state
    from the SFT state and saves the adapter."""
    import subprocess
    exe = os.path.join(ROOT, "tests", "c_api", "_bin", "drop_in")
    if not os.path.exists(exe):
        pytest.skip("tests/c_api/_bin/drop_in was not built (reference tree absent at build time)")
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0 and "DROP_IN ok" in r.stdout, r.stdout[-2000:]
