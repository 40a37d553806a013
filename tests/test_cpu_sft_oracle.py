"""The LoRA-SFT restatement (oracle/sft_oracle.py) checked without the reference's Metal path:
against an independent float64 autograd model, by finite differences, against closed-form AdamW,
and -- for the forward half -- against the decode oracle, which is pinned to the reference's C code."""
import struct

import numpy as np
import pytest

import _oracle
import _sft_common as sc

torch = pytest.importorskip("torch")
o = sc.sft_oracle

RANK, ALPHA = 4, 8.0


@pytest.fixture(scope="module")
def small(pkg):
    cfg = sc.SMALL
    w = sc.make_weights(pkg, cfg)
    ow = sc.oracle_model(cfg, w)
    n = 12
    toks = sc.tokens(pkg, 2 * (n + 1), 4321, cfg["vocab_size"]).reshape(2, n + 1)
    return cfg, w, ow, toks[:, :-1], toks[:, 1:]


def test_gradients_match_autograd_float64(pkg, small):
    cfg, w, ow, x, y = small
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    loss, grads, _ = o.loss_and_grads(ow, lora, x, y, dtype=np.float64)
    tloss, tgrads = sc.torch_loss_and_grads(cfg, ow, lora.p, float(lora.scaling), x, y)
    assert abs(loss - tloss) < 1e-9 * abs(tloss)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            # the restatement scales by float32(1/N) as the reference does; autograd by the exact 1/N
            assert sc.rel_err(grads[L][k], tgrads[L][k]) < 2e-7, (L, k)


def test_float32_pass_is_close_to_float64(pkg, small):
    cfg, w, ow, x, y = small
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    l32, g32, _ = o.loss_and_grads(ow, lora, x, y, dtype=np.float32)
    l64, g64, _ = o.loss_and_grads(ow, lora, x, y, dtype=np.float64)
    assert abs(l32 - l64) < 1e-5 * abs(l64)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            assert sc.rel_err(g32[L][k], g64[L][k]) < 2e-4, (L, k)


def test_gradient_by_finite_differences(pkg, small):
    cfg, w, ow, x, y = small
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    _, grads, _ = o.loss_and_grads(ow, lora, x[:1], y[:1], dtype=np.float64)
    rng = np.random.default_rng(5)
    for L, k in ((0, "A_q"), (1, "B_v"), (1, "B_q"), (0, "A_v")):
        p = lora.p[L][k]
        i, j = rng.integers(p.shape[0]), rng.integers(p.shape[1])
        keep, h = p[i, j], 1e-3
        p[i, j] = keep + h
        lp, _, _ = o.loss_and_grads(ow, lora, x[:1], y[:1], dtype=np.float64)
        p[i, j] = keep - h
        lm, _, _ = o.loss_and_grads(ow, lora, x[:1], y[:1], dtype=np.float64)
        p[i, j] = keep
        num = (lp - lm) / (float(np.float32(keep + h)) - float(np.float32(keep - h)))
        assert abs(num - grads[L][k][i, j]) < 1e-4 * max(abs(num), 1e-6) + 1e-9, (L, k, num, grads[L][k][i, j])


def test_zero_B_gives_zero_A_gradient_and_base_logits(pkg, small):
    cfg, w, ow, x, y = small
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK), RANK, ALPHA)
    _, grads, _ = o.loss_and_grads(ow, lora, x[:1], y[:1])
    for g in grads:
        assert not g["A_q"].any() and not g["A_v"].any()
        assert g["B_q"].any() and g["B_v"].any()


def test_forward_logits_equal_the_pinned_decode_oracle(pkg, synth):
    """With B = 0 the SFT forward is the plain F16-weight forward: position by position it must give
    the logits of the decode restatement (itself bit-pinned to the reference's C code)."""
    spec = pkg.spec("tiny-qwen3", n_layers=2)
    m = synth.llmb200_synth_qwen3(spec, 4)
    try:
        model = _oracle.model_qwen3(m, 1, 32, vocab=spec.vocab_size)
        cfg = dict(sc.TINY, n_layers=2)
        w = sc.make_weights(pkg, cfg, seed=1234, gamma_jitter=0.0)
        ow = sc.oracle_model(cfg, w)
        n = 8
        toks = sc.tokens(pkg, n, 4321, cfg["vocab_size"])
        lora = o.LoRA(sc.make_lora(pkg, cfg, RANK), RANK, ALPHA)
        logits, _ = o.forward(ow, lora, toks)
        for pos in range(n):
            ref = _oracle.forward_token(model, int(toks[pos]), pos)
            assert sc.rel_err(logits[pos], ref) < 2e-4, pos
    finally:
        synth.llmb200_synth_free_qwen3(m)


def test_clip_and_adamw_closed_form(pkg, small):
    cfg = small[0]
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    before = [{k: v.copy() for k, v in l.items()} for l in lora.p]
    rng = np.random.default_rng(1)
    grads = [{k: rng.standard_normal(v.shape).astype(np.float32) for k, v in l.items()} for l in lora.p]
    total = np.sqrt(sum(float((g[k].astype(np.float64) ** 2).sum()) for g in grads for k in o.KEYS))
    clipped, norm = o.clip_grad_norm(grads, 1.0)
    assert abs(norm - total) < 1e-6 * total
    new = np.sqrt(sum(float((g[k].astype(np.float64) ** 2).sum()) for g in clipped for k in o.KEYS))
    assert abs(new - 1.0) < 1e-5
    small_g = [{k: v * np.float32(1e-4) for k, v in g.items()} for g in clipped]
    same, _ = o.clip_grad_norm(small_g, 1.0)
    assert all(np.array_equal(a[k], b[k]) for a, b in zip(small_g, same) for k in o.KEYS)
    # first AdamW step: m_hat = g, v_hat = g^2 -> p -= lr * (g / (|g| + eps) + wd * p)
    lora.step_count = 1
    o.adamw(lora, clipped, 1e-3)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            g, p0 = clipped[L][k].astype(np.float64), before[L][k].astype(np.float64)
            want = p0 - 1e-3 * (g / (np.abs(g) + 1e-8) + 0.01 * p0)
            assert np.abs(lora.p[L][k] - want).max() < 1e-6


def test_train_step_lowers_the_loss(pkg, small):
    cfg, w, ow, x, y = small
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK), RANK, ALPHA)
    losses = [o.train_step(ow, lora, x[:1], y[:1], 1e-2)[0] for _ in range(4)]
    assert lora.step_count == 4
    assert losses[-1] < losses[0]
    assert abs(losses[0] - np.log(cfg["vocab_size"])) < 0.5        # random init: about uniform


def test_adapter_file_layout(pkg, small):
    cfg = small[0]
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    blob = o.save_lora_bytes(lora)
    magic, nl, rank = struct.unpack_from("<Iii", blob)
    assert (magic, nl, rank) == (0x4C4F5241, cfg["n_layers"], RANK)
    per = sum(v.size for v in lora.p[0].values())
    assert len(blob) == 12 + 4 * per * nl
    first = np.frombuffer(blob, dtype="<f4", count=lora.p[0]["A_q"].size, offset=12)
    assert np.array_equal(first, lora.p[0]["A_q"].ravel())
