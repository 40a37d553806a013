"""The GRPO step on the GPU: the policy-gradient and scale kernels against the numpy restatement
(oracle/sft_oracle.py), then the reference's own src/nn/fast_grpo.c running unchanged on top of
libllmb200.so (tests/c_api/grpo_drop_in.c) against the record of the same program over the reference's
engines on the CPU (tests/golden/grpo_golden.bin). Sampled tokens must be identical; log-probabilities
within 1e-2 (the decode path's logits tolerance; they are logits / temperature - logsumexp); LoRA gradients within 1e-2 of the largest element with binary16 operands on the tensor cores
(the engine's default) and within 1e-3 on the fp32 CUDA-core path."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import sft_oracle as o  # noqa: E402
import _grpo_record as gr  # noqa: E402

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(ROOT, "tests", "golden", "grpo_golden.bin")
B200_BIN = os.path.join(ROOT, "tests", "c_api", "_bin", "grpo_b200")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n,v", [(16, 64), (5, 1023), (64, 4096), (3, 151936)])
def test_policy_gradient_kernel(lib, n, v):
    rng = np.random.default_rng(n * 7 + v)
    logits = (rng.standard_normal((n, v)) * 4).astype(np.float32)
    actions = rng.integers(0, v, n).astype(np.uint32)
    lp64 = logits.astype(np.float64) - np.log(np.exp(logits.astype(np.float64)).sum(1, keepdims=True))
    old = lp64[np.arange(n), actions].astype(np.float32) + (rng.standard_normal(n) * 0.3).astype(np.float32)
    adv = rng.standard_normal(n).astype(np.float32)
    adv[0] = 0.0                                                # a prompt position
    want_lp, want_d = o.grpo_policy_grad(logits, actions, old, adv, 0.2)
    assert (np.abs(want_d).max(1) == 0).sum() >= 1 and (np.abs(want_d).max(1) > 0).sum() >= 1
    d_logits, d_act, d_old, d_adv = dev(logits), dev(actions.view(np.int32)), dev(old), dev(adv)
    d_new = torch.full((n,), 7.0, dtype=torch.float32, device="cuda")
    d_out = torch.full((n, v), 7.0, dtype=torch.float32, device="cuda")
    rc = lib.b200_grpo_policy_grad(d_logits.data_ptr(), d_act.data_ptr(), d_old.data_ptr(), d_adv.data_ptr(), d_new.data_ptr(),
                                   d_out.data_ptr(), n, v, 0.2, None)
    torch.cuda.synchronize()
    assert rc == 0
    got_lp, got_d = d_new.cpu().numpy(), d_out.cpu().numpy()
    assert np.abs(got_lp - want_lp).max() < 1e-4
    # rows the clip removes are exact zeros on both sides; the others agree to fp32 rounding of exp/log
    zero = np.abs(want_d).max(1) == 0
    assert (got_d[zero] == 0).all()
    assert np.abs(got_d - want_d).max() < 2e-5 * max(1.0, float(np.abs(want_d).max()))
    # scale in place, odd length and an unaligned start
    x = rng.standard_normal(4099).astype(np.float32)
    d_x = dev(x)
    assert lib.b200_scale(d_x.data_ptr() + 4, 0.25, 4098, None) == 0
    torch.cuda.synchronize()
    want = x.copy(); want[1:] *= np.float32(0.25)
    assert (d_x.cpu().numpy() == want).all()
    assert lib.b200_grpo_policy_grad(None, d_act.data_ptr(), d_old.data_ptr(), d_adv.data_ptr(), d_new.data_ptr(),
                                     d_out.data_ptr(), n, v, 0.2, None) != 0


def run_program(tmp_path, env_extra):
    out = str(tmp_path / "b200.bin")
    env = dict(os.environ, **env_extra)
    r = subprocess.run([B200_BIN, out], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "GRPO_DROP_IN ok" in r.stdout, (r.returncode, r.stderr[-1500:])
    return gr.by_step(gr.read(out))


def compare_step(got, want, grad_tol):
    assert (got[gr.LEN] == want[gr.LEN]).all()
    assert (got[gr.TOKENS] == want[gr.TOKENS]).all(), "sampled tokens differ from the reference run"
    assert np.abs(got[gr.LOGPROBS] - want[gr.LOGPROBS]).max() < 1e-2
    assert (got[gr.REWARDS] == want[gr.REWARDS]).all() and np.abs(got[gr.ADVANTAGES] - want[gr.ADVANTAGES]).max() < 1e-5
    assert abs(float(got[gr.REWARD][0]) - float(want[gr.REWARD][0])) < 1e-6
    assert np.abs(got[gr.NEW_LP] - want[gr.NEW_LP]).max() < 1e-2
    assert len(got[gr.GRADS]) == len(want[gr.GRADS])
    gmax = max(float(np.abs(g).max()) for g in want[gr.GRADS])
    for a, b in zip(got[gr.GRADS], want[gr.GRADS]):
        assert a.shape == b.shape
        assert np.abs(a - b).max() < grad_tol * gmax, (float(np.abs(a - b).max()), gmax)


@pytest.mark.skipif(not os.path.exists(B200_BIN), reason="tests/c_api/_bin/grpo_b200 was not built (reference tree absent)")
def test_reference_grpo_loop_on_the_cuda_engines_fp32_path(tmp_path):
    """LLMB200_SFT_TC=0: every product in fp32 on the CUDA cores, as the reference computes. Both steps are
    compared: the second one generates with the adapter the first one trained."""
    want, want_adapter = gr.by_step(gr.read(GOLDEN))
    got, got_adapter = run_program(tmp_path, {"LLMB200_SFT_TC": "0"})
    assert len(got) == len(want) == gr.STEPS
    for g, w in zip(got, want):
        compare_step(g, w, 1e-3)
    # AdamW turns a gradient element into a step of about lr whatever its size, so an element whose gradient is
    # rounding noise may move the other way: nearly all elements must agree closely, none by more than two steps
    diff = np.abs(got_adapter - want_adapter)
    assert diff.max() <= 2 * gr.STEPS * 1e-2 * 1.01
    assert (diff < 1e-4).mean() > 0.97, float((diff < 1e-4).mean())


@pytest.mark.skipif(not os.path.exists(B200_BIN), reason="tests/c_api/_bin/grpo_b200 was not built (reference tree absent)")
def test_reference_grpo_loop_on_the_cuda_engines_default_path(tmp_path):
    """The engine's default: frozen products on the tensor cores with binary16 operands. The first step samples
    from the untouched base model (B = 0), so its tokens must be the reference's; its gradients carry the
    operand rounding. The second step's samples depend on an adapter trained from those gradients and are not
    compared element by element."""
    want, _ = gr.by_step(gr.read(GOLDEN))
    got, got_adapter = run_program(tmp_path, {})
    assert len(got) == gr.STEPS
    compare_step(got[0], want[0], 1e-2)
    assert np.isfinite(got_adapter).all() and np.abs(got_adapter).max() > 0
    assert np.isfinite(got[1][gr.REWARD]).all()
