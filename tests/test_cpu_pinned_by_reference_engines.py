"""The restatements held to what the reference's own fast engines computed.

tests/golden/sft_golden.npz, sft_golden_gemma3.npz, sft_golden_full.npz and fast_decode_golden.npz were produced by src/nn/fast_sft.c and
src/nn/fast_inference.c themselves (compiled unmodified over a CPU stand-in for their Metal dispatch
layer, see tests/golden/make_sft_golden.py). Here the LoRA-SFT restatement (oracle/sft_oracle.py) must
reproduce the reference's losses, gradient buffers, updated weights and adapter file, and the decode
restatement (oracle/oracle.c) the reference's tokens and logits -- Gemma3 block order included.
"""
import ctypes as C
import os

import numpy as np
import pytest

import _oracle as O
import _sft_common as sc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SFT = np.load(os.path.join(ROOT, "tests", "golden", "sft_golden.npz"))
DEC = np.load(os.path.join(ROOT, "tests", "golden", "fast_decode_golden.npz"))
o = sc.sft_oracle
TOL = 1e-5          # max |a-b| / max |b|, fp32 against fp32 with different summation orders


def test_sft_restatement_reproduces_three_reference_steps(pkg):
    """Loss and gradients of every step, then the optimizer, each within 1e-5 of the reference.

    AdamW divides by sqrt(v) + 1e-8, so entries whose gradient is at rounding level (|g| ~ 1e-8) move by an
    amount that depends on the last bits of g; two fp32 programs with different summation orders therefore
    drift apart by ~1e-3 of a weight after a step, which says nothing about either. The steps are checked
    one at a time instead: the restatement computes loss and gradients at the reference's weights, and its
    optimizer is then fed the reference's own gradient buffers, which must land on the reference's weights.
    """
    cfg = dict(sc.TINY)
    rank, alpha, lr = int(SFT["rank"]), float(SFT["alpha"]), float(SFT["lr"])
    ow = sc.oracle_model(cfg, sc.make_weights(pkg, cfg))
    lora = o.LoRA(sc.make_lora(pkg, cfg, rank), rank, alpha)
    x, y = SFT["inputs"], SFT["targets"]
    assert len(x) == int(SFT["seq_len"])
    for step in range(3):
        loss, grads, logits = o.loss_and_grads(ow, lora, x, y)
        losses, _ = o.softmax_ce(logits, y.astype(np.int64))
        assert sc.rel_err(losses, SFT[f"losses_{step}"]) < TOL
        assert abs(loss - float(SFT[f"loss_{step}"])) < TOL * abs(loss), (step, loss)
        grads = [{k: g[k].astype(np.float32) for k in o.KEYS} for g in grads]
        clipped, _ = o.clip_grad_norm(grads, 1.0)                 # the buffers hold the clipped values
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                want = SFT[f"grad_{step}_{L}_{k}"]
                if not want.any():
                    assert not clipped[L][k].any(), (step, L, k)  # dA is exactly zero while B is
                    continue
                assert sc.rel_err(clipped[L][k], want) < TOL, (step, L, k, sc.rel_err(clipped[L][k], want))
        lora.step_count += 1                                      # fast_sft.c:1152
        o.adamw(lora, [{k: SFT[f"grad_{step}_{L}_{k}"] for k in o.KEYS} for L in range(cfg["n_layers"])], lr)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            assert sc.rel_err(lora.p[L][k], SFT[f"weight_{L}_{k}"]) < TOL, (L, k)
    # adapter file: header and layout byte for byte, payload as above
    mine, ref = o.save_lora_bytes(lora), SFT["save_lora_bytes"].tobytes()
    assert len(mine) == len(ref) and mine[:12] == ref[:12]
    a, b = np.frombuffer(mine[12:], dtype="<f4"), np.frombuffer(ref[12:], dtype="<f4")
    assert np.abs(a - b).max() < TOL * np.abs(b).max()


def test_free_running_steps_stay_close(pkg):
    """Without the hand-over of gradients: three restated steps in a row against the reference's three."""
    cfg = dict(sc.TINY)
    rank = int(SFT["rank"])
    ow = sc.oracle_model(cfg, sc.make_weights(pkg, cfg))
    lora = o.LoRA(sc.make_lora(pkg, cfg, rank), rank, float(SFT["alpha"]))
    for step in range(3):
        loss, grads, _ = o.train_step(ow, lora, SFT["inputs"], SFT["targets"], float(SFT["lr"]))
        assert abs(loss - float(SFT[f"loss_{step}"])) < 1e-6 * abs(loss)
        clipped, _ = o.clip_grad_norm(grads, 1.0)
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                want = SFT[f"grad_{step}_{L}_{k}"]
                if want.any():
                    assert sc.rel_err(clipped[L][k], want) < 1e-4, (step, L, k)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            assert sc.rel_err(lora.p[L][k], SFT[f"weight_{L}_{k}"]) < 1e-2, (L, k)


def test_sft_golden_saw_every_gradient(pkg):
    # by the second step B is non-zero, so all four matrices of every layer carry gradient
    for L in range(sc.TINY["n_layers"]):
        for k in o.KEYS:
            assert SFT[f"grad_2_{L}_{k}"].any() and np.isfinite(SFT[f"grad_2_{L}_{k}"]).all()
    assert float(SFT["loss_2"]) < float(SFT["loss_0"])


def test_gemma3_sft_restatement_reproduces_three_reference_steps(pkg):
    """The Gemma3 block order of the restatement (four norms per layer, GeGLU, scaled and tied embeddings, a RoPE
    base per layer) against sft_state_create_gemma3 + sft_train_step of the reference, step by step as above."""
    G3 = np.load(os.path.join(ROOT, "tests", "golden", "sft_golden_gemma3.npz"))
    sp = pkg.spec("tiny-gemma3", gamma_jitter=0.1, n_layers=2)
    cfg = sc.gemma_cfg(sp)
    rank, alpha, lr = int(G3["rank"]), float(G3["alpha"]), float(G3["lr"])
    ow = sc.oracle_model(cfg, sc.make_weights_gemma(pkg, cfg))
    lora = o.LoRA(sc.make_lora(pkg, cfg, rank), rank, alpha)
    x, y = G3["inputs"], G3["targets"]
    for step in range(3):
        loss, grads, logits = o.loss_and_grads(ow, lora, x, y)
        losses, _ = o.softmax_ce(logits, y.astype(np.int64))
        assert sc.rel_err(losses, G3[f"losses_{step}"]) < TOL
        assert abs(loss - float(G3[f"loss_{step}"])) < TOL * abs(loss), (step, loss)
        grads = [{k: g[k].astype(np.float32) for k in o.KEYS} for g in grads]
        clipped, _ = o.clip_grad_norm(grads, 1.0)
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                want = G3[f"grad_{step}_{L}_{k}"]
                if not want.any():
                    assert not clipped[L][k].any(), (step, L, k)
                    continue
                assert sc.rel_err(clipped[L][k], want) < TOL, (step, L, k, sc.rel_err(clipped[L][k], want))
        lora.step_count += 1
        o.adamw(lora, [{k: G3[f"grad_{step}_{L}_{k}"] for k in o.KEYS} for L in range(cfg["n_layers"])], lr)
    for L in range(cfg["n_layers"]):
        for k in o.KEYS:
            assert sc.rel_err(lora.p[L][k], G3[f"weight_{L}_{k}"]) < TOL, (L, k)
    assert float(G3["loss_2"]) < float(G3["loss_0"]) and all(G3[f"grad_2_{L}_{k}"].any() for L in range(2) for k in o.KEYS)


def full_sample(ow, stride):
    parts = []
    for lw in ow.layers:
        parts += [lw[k].reshape(-1)[::stride] for k in ("q", "k", "v", "o", "gate", "up", "down")]
    parts.append(ow.lm_head.reshape(-1)[::stride])
    return np.concatenate(parts).astype(np.float32)


@pytest.mark.parametrize("mode", ["sgd", "accum"])
def test_full_parameter_restatement_reproduces_the_reference_steps(pkg, mode):
    """sft_state_create_full + sft_train_step (every matrix stepped inside the backward pass, q/k/v before the
    gradient goes on through them), and the accumulate-then-apply form. Losses to 1e-5; the binary16 weights after
    the last call equal the reference's except where a sum in another order lands on the other side of a rounding
    (one unit in the last place, a small fraction of the elements)."""
    FG = np.load(os.path.join(ROOT, "tests", "golden", "sft_golden_full.npz"))
    cfg = dict(sc.TINY, n_layers=2)
    stride, lr = int(FG["stride"]), float(FG["lr"])
    ow = sc.oracle_model(cfg, sc.make_weights(pkg, cfg))
    x, y = FG["inputs"], FG["targets"]
    start = full_sample(ow, stride)
    acc = o.new_accum(ow) if mode == "accum" else None
    for step in range(3 if mode == "sgd" else 2):
        loss, losses = o.full_train_step(ow, x, y, lr, acc)
        assert sc.rel_err(losses, FG[f"{mode}_losses_{step}"]) < TOL, step
        assert abs(loss - float(FG[f"{mode}_loss"][step])) < TOL * abs(loss)
    if mode == "accum":
        assert (full_sample(ow, stride) == start).all()           # nothing moves before the apply
        o.apply_accum(ow, acc, lr)
    got, want = full_sample(ow, stride), FG[f"{mode}_weights"].astype(np.float32)
    assert got.shape == want.shape
    assert (want != start).mean() > 0.1                           # the steps did move the weights
    assert (got == want).mean() > 0.995, float((got == want).mean())
    assert np.abs(got - want).max() <= 2.0 ** -10 * np.abs(want).max()
    if mode == "sgd":
        assert FG["sgd_loss"][2] < FG["sgd_loss"][0]
    else:
        assert FG["accum_loss"][1] == FG["accum_loss"][0]


@pytest.mark.parametrize("arch", ["tiny-qwen3", "tiny-gemma3"])
@pytest.mark.parametrize("use_fp16", [0, 1])
def test_decode_restatement_reproduces_the_reference_engine(pkg, synth, arch, use_fp16):
    gemma = arch.endswith("gemma3")
    sp = pkg.spec(arch, gamma_jitter=0.1)
    model = (synth.llmb200_synth_gemma3 if gemma else synth.llmb200_synth_qwen3)(C.byref(sp), 4)
    try:
        prompt = DEC[f"{arch}_prompt"]
        tag = f"{arch}_{'f16' if use_fp16 else 'q8'}"
        om = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, int(DEC["max_seq"]), vocab=sp.vocab_size)
        toks, _ = O.generate(om, prompt, int(DEC["gen_len"]))
        assert list(toks) == list(DEC[f"{tag}_tokens"])
        om2 = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, int(DEC["max_seq"]), vocab=sp.vocab_size)
        lg = None
        for i, t in enumerate(prompt):
            lg = O.forward_token(om2, t, i)
        ref = DEC[f"{tag}_logits"]
        assert np.abs(lg - ref).max() < 1e-4 * np.abs(ref).max()
    finally:
        (synth.llmb200_synth_free_gemma3 if gemma else synth.llmb200_synth_free_qwen3)(model)
