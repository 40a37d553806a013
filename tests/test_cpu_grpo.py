"""The GRPO step (the reference's src/nn/fast_grpo.c as a caller of the drop-in library), CPU side: the
committed record of the reference run is what the reference produces here, it exercises the step (rewards
differ inside the groups, gradients are not zero), the numpy restatement of the policy-gradient kernel has the
properties its formula implies, and the CUDA build of the same program stops loudly without a GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import sft_oracle as o  # noqa: E402
import _grpo_record as gr  # noqa: E402

GOLDEN = os.path.join(ROOT, "tests", "golden", "grpo_golden.bin")
REF_BIN = os.path.join(ROOT, "tests", "c_api", "_bin", "grpo_ref")
B200_BIN = os.path.join(ROOT, "tests", "c_api", "_bin", "grpo_b200")


def test_golden_record_exercises_the_step():
    steps, tail = gr.by_step(gr.read(GOLDEN))
    adapter, loss = tail[gr.ADAPTER], tail[gr.SFT_LOSS]
    assert len(steps) == gr.STEPS and np.abs(adapter).max() > 0
    assert np.isfinite(loss).all() and loss[1] < loss[0]       # two LoRA-SFT steps on one batch after the GRPO steps
    for st in steps:
        assert st[gr.REWARDS].std() > 0, "equal rewards give zero advantages and an all-zero gradient"
        assert abs(float(st[gr.ADVANTAGES].mean())) < 1e-5
        assert abs(float(st[gr.REWARD][0]) - float(st[gr.REWARDS].mean())) < 1e-6
        lens = st[gr.LEN].astype(int)
        assert ((lens >= 1) & (lens <= gr.MAX_GEN)).all()
        assert max(float(np.abs(g).max()) for g in st[gr.GRADS]) > 1e-2
        lp = st[gr.LOGPROBS].reshape(gr.GROUP, gr.MAX_GEN)
        for i, n in enumerate(lens):
            assert (lp[i, :n] < 0).all() and (lp[i, n:] == 0).all()
    # B starts at zero: the first step has no gradient on A (dA = (dq B^T ...)), the second has
    assert all(np.abs(g).max() == 0 for g in steps[0][gr.GRADS][0::2])
    assert all(np.abs(g).max() > 0 for g in steps[1][gr.GRADS])


MODES = {"lora": GOLDEN, "full": GOLDEN.replace(".bin", "_full.bin"), "full-accurate": GOLDEN.replace(".bin", "_full_accurate.bin"),
         "gemma": GOLDEN.replace(".bin", "_gemma.bin"), "gemma-full": GOLDEN.replace(".bin", "_gemma_full.bin"),
         "gemma-hd256": GOLDEN.replace(".bin", "_gemma_hd256.bin")}


@pytest.mark.skipif(not os.path.exists(REF_BIN), reason="tests/c_api/_bin/grpo_ref was not built (reference tree absent)")
@pytest.mark.parametrize("mode", sorted(MODES))
def test_golden_record_is_what_the_reference_run_writes(tmp_path, mode):
    """The reference's own fast_grpo.c, fast_sft.c and fast_inference.c over the CPU stand-in for the Metal layer."""
    out = str(tmp_path / "ref.bin")
    r = subprocess.run([REF_BIN, out, mode], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert r.returncode == 0 and "GRPO_DROP_IN ok" in r.stdout, r.stderr[-800:]
    assert open(out, "rb").read() == open(MODES[mode], "rb").read()


@pytest.mark.parametrize("mode", ["gemma", "gemma-hd256"])
def test_gemma3_lora_record_exercises_the_step(mode):
    steps, tail = gr.by_step(gr.read(MODES[mode]))
    assert len(steps) == gr.STEPS and np.abs(tail[gr.ADAPTER]).max() > 0
    assert np.isfinite(tail[gr.SFT_LOSS]).all() and tail[gr.SFT_LOSS][1] < tail[gr.SFT_LOSS][0]
    assert all(st[gr.REWARDS].std() > 0 for st in steps)
    assert all(max(float(np.abs(g).max()) for g in st[gr.GRADS]) > 1e-3 for st in steps)
    assert (steps[0][gr.TOKENS] != gr.by_step(gr.read(GOLDEN))[0][0][gr.TOKENS]).any()      # another model, another seed


@pytest.mark.parametrize("mode", ["full", "full-accurate", "gemma-full"])
def test_full_parameter_records_exercise_the_step(mode):
    """Full-parameter modes: rewards differ inside the groups, the second step samples from changed weights, the
    two SFT steps on the same batch lower the loss (immediate mode), and the checkpoint has the reference's header."""
    steps, tail = gr.by_step(gr.read(MODES[mode]))
    lora_steps, _ = gr.by_step(gr.read(MODES["gemma"] if mode.startswith("gemma") else GOLDEN))
    assert len(steps) == gr.STEPS and all(st[gr.REWARDS].std() > 0 for st in steps)
    assert not steps[0][gr.GRADS]                                          # no adapter, no LoRA gradient buffers
    assert (steps[0][gr.TOKENS] == lora_steps[0][gr.TOKENS]).all()        # first samples: the untouched base model
    assert (steps[1][gr.TOKENS] != lora_steps[1][gr.TOKENS]).any()
    loss = tail[gr.SFT_LOSS]
    assert np.isfinite(loss).all()
    if mode != "full-accurate":
        assert loss[1] < loss[0]
    else:
        assert loss[1] == loss[0]          # accumulators allocated: the reference's step accumulates and moves no weight
    assert tail[gr.CKPT_HEAD].astype(int).tolist() == [0x46554C4C & 0xffffff, int(mode.startswith("gemma")), 2, 256, 4, 2, 64, 512, 64]
    n = int(tail[gr.CKPT_SUMS][0])
    assert n == 2 * (512 * 256 + 256 * 256 + 1024 * 256 + 256 * 512) + 64 * 256
    assert len(tail[gr.CKPT_SAMPLE]) == (n + 96) // 97


def test_policy_gradient_restatement_properties():
    """oracle.grpo_policy_grad: rows sum to zero, clipped positions and zero advantages give zero rows, the
    unclipped gradient is -advantage * ratio * d(log p_action)/d(logits)."""
    rng = np.random.default_rng(3)
    n, v = 12, 50
    logits = rng.standard_normal((n, v)).astype(np.float32) * 3
    actions = rng.integers(0, v, n)
    logp = logits - np.log(np.exp(logits.astype(np.float64)).sum(1, keepdims=True))
    true_lp = logp[np.arange(n), actions].astype(np.float32)
    old = true_lp.copy()
    adv = rng.standard_normal(n).astype(np.float32)
    old[0] -= 0.5; adv[0] = 1.0        # ratio 1.65 > 1.2, positive advantage: clipped away
    old[1] += 0.5; adv[1] = -1.0       # ratio 0.61 < 0.8, negative advantage: clipped away
    old[2] -= 0.5; adv[2] = -1.0       # ratio high, negative advantage: kept
    old[3] += 0.5; adv[3] = 1.0        # ratio low, positive advantage: kept
    adv[4] = 0.0
    new_lp, d = o.grpo_policy_grad(logits, actions, old, adv, 0.2)
    assert np.abs(new_lp - true_lp).max() < 1e-5
    assert np.abs(d.sum(1)).max() < 1e-5
    assert (d[0] == 0).all() and (d[1] == 0).all() and (d[4] == 0).all()
    for r in (2, 3, 5, 6):
        ratio = np.exp(true_lp[r] - old[r])
        want = -adv[r] * ratio * (-np.exp(logp[r]))
        want[actions[r]] += -adv[r] * ratio
        assert np.abs(d[r] + want).max() < 1e-5 * max(1.0, np.abs(want).max()), r


@pytest.mark.skipif(not os.path.exists(B200_BIN), reason="tests/c_api/_bin/grpo_b200 was not built (reference tree absent)")
def test_cuda_build_of_the_program_fails_loudly_without_a_gpu(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU suite runs the program for real")
    r = subprocess.run([B200_BIN, str(tmp_path / "x.bin")], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert r.returncode == 3, (r.returncode, r.stderr[-500:])
    assert "no CUDA device available" in r.stderr and "no CPU path" in r.stderr
    assert "GRPO_DROP_IN ok" not in r.stdout


def test_geglu_restatement_backward_matches_finite_differences():
    rng = np.random.default_rng(9)
    g = (rng.standard_normal(200) * 2).astype(np.float32)
    u = rng.standard_normal(200).astype(np.float32)
    dy = rng.standard_normal(200).astype(np.float32)
    dg, du = o.gelu_mul_backward(dy, g, u)
    h = 1e-3
    f = lambda gg, uu: o.gelu_mul(gg.astype(np.float32), uu.astype(np.float32)).astype(np.float64)
    num_g = (f(g + h, u) - f(g - h, u)) / (2 * h) * dy
    num_u = (f(g, u + h) - f(g, u - h)) / (2 * h) * dy
    assert np.abs(dg - num_g).max() < 2e-3 and np.abs(du - num_u).max() < 2e-3
