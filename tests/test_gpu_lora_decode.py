"""Decode with a LoRA adapter attached (inference_state_set_lora): the per-token logits must equal the
full-sequence forward of the SFT restatement with the same adapter, position by position, and follow
the adapter as training changes it (it is read in place on the device)."""
import ctypes as C

import numpy as np
import pytest

import _sft_common as sc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
o = sc.sft_oracle

RANK, ALPHA, N = 8, 16.0, 12


def build_decode_state(pkg, lib, cfg, w, max_seq):
    keep = []
    c = pkg.Config(pkg.MODEL_QWEN3, cfg["d_model"], cfg["n_q_heads"], cfg["n_kv_heads"], cfg["head_dim"],
                   cfg["intermediate_size"], cfg["vocab_size"], cfg["n_layers"], max_seq, 1)       # F16 weights
    st = lib.llmb200_state_begin(C.byref(c))
    assert st
    D, Hq, Hkv, hd, IS = (cfg[k] for k in ("d_model", "n_q_heads", "n_kv_heads", "head_dim", "intermediate_size"))
    for i, l in enumerate(w["layers"]):
        r = pkg.LayerWeightRef()
        for name, rows, cols in (("q", Hq * hd, D), ("k", Hkv * hd, D), ("v", Hkv * hd, D), ("o", D, Hq * hd),
                                 ("gate", IS, D), ("up", IS, D), ("down", D, IS)):
            a = np.ascontiguousarray(l[name], dtype=np.float32)
            keep.append(a)
            setattr(r, name + "_proj", pkg.WeightRef(sc.fptr(a), rows, cols))
        for name, field in (("input_norm", "input_norm_g"), ("post_attn_norm", "post_attn_norm_g"),
                            ("q_norm", "q_norm_g"), ("k_norm", "k_norm_g")):
            a = np.ascontiguousarray(l[name], dtype=np.float32)
            keep.append(a)
            setattr(r, field, sc.fptr(a))
        r.d_model, r.head_dim = D, hd
        assert lib.llmb200_state_load_layer(st, i, C.byref(r), C.c_float(cfg["rope_theta"])) == 0
        lib.metal_flush()
    lm, fn, emb = (np.ascontiguousarray(w[k], dtype=np.float32) for k in ("lm_head", "final_norm", "emb"))
    assert lib.llmb200_state_finish(st, sc.fptr(lm), sc.fptr(fn), sc.fptr(emb)) == 0
    return st


def decode_logits(lib, st, toks, V):
    lib.inference_state_reset(st)
    out = []
    for t in toks:
        p = lib.inference_forward_token(st, int(t))
        assert p
        out.append(np.ctypeslib.as_array(p, shape=(V,)).copy())
    assert lib.llmb200_state_error(st) == 0
    return np.stack(out)


def test_decode_with_adapter_matches_the_sft_forward(pkg, lib):
    cfg = dict(sc.TINY, n_layers=2, vocab_size=1024)
    V = cfg["vocab_size"]
    w = sc.make_weights(pkg, cfg)
    ow = sc.oracle_model(cfg, w)
    toks = sc.tokens(pkg, N + 1, 99, V)
    x, y = toks[:-1], toks[1:]
    init = sc.make_lora(pkg, cfg, RANK, b_std=0.05)
    lora = o.LoRA(init, RANK, ALPHA)
    eng = sc.Engine(pkg, cfg, w, init, N, 1, RANK, ALPHA, tensor_cores=False)
    st = build_decode_state(pkg, lib, cfg, w, 32)
    try:
        base = decode_logits(lib, st, x, V)
        lib.inference_state_set_lora(st, eng.h)
        got = decode_logits(lib, st, x, V)
        want, _ = o.forward(ow, lora, x)
        scale = np.abs(want).max()
        assert np.abs(got - want).max() < 1e-2 * scale
        assert np.abs(base - want).max() > 5e-2 * scale            # the adapter does change the logits
        zero = o.LoRA(sc.make_lora(pkg, cfg, RANK), RANK, ALPHA)     # B = 0: the plain model
        plain, _ = o.forward(ow, zero, x)
        assert np.abs(base - plain).max() < 1e-2 * np.abs(plain).max()

        # two training steps on the SFT state: the attached decode state follows without any further call
        for _ in range(2):
            eng.train(x, y, 5e-2)
            o.train_step(ow, lora, x, y, 5e-2)
        got2 = decode_logits(lib, st, x, V)
        want2, _ = o.forward(ow, lora, x)
        assert np.abs(got2 - want2).max() < 1e-2 * np.abs(want2).max()
        assert np.abs(got2 - got).max() > 1e-3 * scale

        # greedy generation with the adapter: each token is the argmax of the restatement's logits at that point
        prompt = x[:4].copy()
        outt = np.zeros(6, dtype=np.uint32)
        lib.llmb200_state_set_eos(st, None, 0)
        n = lib.inference_generate(st, prompt.ctypes.data_as(pkg.c_u32_p), 4, outt.ctypes.data_as(pkg.c_u32_p), 6)
        assert n == 6
        seq = list(prompt)
        for t in outt:
            lg, _ = o.forward(ow, lora, np.asarray(seq, dtype=np.uint32))
            top = np.sort(lg[-1])[-2:]
            assert int(np.argmax(lg[-1])) == int(t) or (top[1] - top[0]) < 1e-3 * np.abs(lg[-1]).max()
            seq.append(int(t))
    finally:
        lib.inference_state_free(st)
        eng.close()


@pytest.mark.parametrize("tensor_cores", [True, False])
def test_decode_state_made_from_the_sft_state(pkg, lib, tensor_cores):
    """inference_state_create_from_sft: the decode state takes its weights from the SFT state's device memory
    (binary16 views in tensor-core mode, narrowed fp32 copies in CUDA-core mode) and follows its LoRA."""
    cfg = dict(sc.TINY, n_layers=2, vocab_size=1024)
    V = cfg["vocab_size"]
    w = sc.make_weights(pkg, cfg)
    ow = sc.oracle_model(cfg, w)
    toks = sc.tokens(pkg, N + 1, 99, V)
    x, y = toks[:-1], toks[1:]
    init = sc.make_lora(pkg, cfg, RANK, b_std=0.05)
    lora = o.LoRA(init, RANK, ALPHA)
    eng = sc.Engine(pkg, cfg, w, init, N, 1, RANK, ALPHA, tensor_cores=tensor_cores)
    st = lib.inference_state_create_from_sft(eng.h, 32)
    assert st
    try:
        assert lib.inference_state_model_type(st) == pkg.MODEL_QWEN3 and lib.inference_state_vocab_size(st) == V
        assert lib.sft_get_n_q_heads(eng.h) == cfg["n_q_heads"] and lib.sft_get_n_kv_heads(eng.h) == cfg["n_kv_heads"]
        assert lib.sft_get_head_dim(eng.h) == cfg["head_dim"] and lib.sft_get_intermediate_size(eng.h) == cfg["intermediate_size"]
        th = lib.sft_get_rope_thetas(eng.h)
        assert [th[i] for i in range(cfg["n_layers"])] == [cfg["rope_theta"]] * cfg["n_layers"]
        # the shared containers hold the reference's canonical bytes: row-major binary16 of the fp32 matrix
        lw = C.cast(lib.sft_get_layers(eng.h), C.POINTER(pkg.LayerW))
        for name, field in (("q", "q_proj"), ("k", "k_proj"), ("v", "v_proj"), ("o", "o_proj"), ("gate", "gate_proj"),
                            ("up", "up_proj"), ("down", "down_proj")):
            wm = getattr(lw[1], field).contents
            want_bits = w["layers"][1][name].astype(np.float16)
            assert (wm.rows, wm.cols, wm.nb) == (want_bits.shape[0], want_bits.shape[1], 0)
            got_bits = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(wm.mbuf), C.POINTER(C.c_uint16)), shape=want_bits.shape)
            assert np.array_equal(got_bits, want_bits.view(np.uint16)), name
        got = decode_logits(lib, st, x, V)
        want, _ = o.forward(ow, lora, x)
        assert np.abs(got - want).max() < 1e-2 * np.abs(want).max()
        # one training step: the decode state reads the SFT state's LoRA in place, so it must now follow the
        # engine's own updated matrices (taken back from the device: the tensor-core step rounds activations to
        # binary16, so its update differs a little from an fp32 restatement of the step)
        eng.train(x, y, 5e-2)
        got2 = decode_logits(lib, st, x, V)
        want2, _ = o.forward(ow, o.LoRA(eng.params(), RANK, ALPHA), x)
        assert np.abs(got2 - want2).max() < 1e-2 * np.abs(want2).max()
        assert np.abs(got2 - got).max() > 1e-3 * np.abs(want).max()
    finally:
        lib.inference_state_free(st)
        eng.close()


def test_lora_decode_kernel(lib):
    rng = np.random.default_rng(2)
    D, qr, kr, R = 200, 96, 32, 5
    x = rng.standard_normal(D).astype(np.float32)
    Aq, Av = (rng.standard_normal((R, D)).astype(np.float32) for _ in range(2))
    Bq, Bv = rng.standard_normal((qr, R)).astype(np.float32), rng.standard_normal((kr, R)).astype(np.float32)
    qkv = rng.standard_normal(qr + 2 * kr).astype(np.float32)
    d = [torch.from_numpy(a).cuda() for a in (x, Aq, Bq, Av, Bv, qkv)]
    assert lib.b200_lora_decode(*[t.data_ptr() for t in d], D, qr, kr, R, 0.5, None) == 0
    torch.cuda.synchronize()
    want = qkv.astype(np.float64).copy()
    want[:qr] += 0.5 * (Bq.astype(np.float64) @ (Aq.astype(np.float64) @ x))
    want[qr + kr:] += 0.5 * (Bv.astype(np.float64) @ (Av.astype(np.float64) @ x))
    assert np.abs(d[5].cpu().numpy() - want).max() < 1e-4
