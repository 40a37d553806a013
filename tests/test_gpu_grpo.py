"""The GRPO step on the GPU: the policy-gradient and scale kernels against the numpy restatement
(oracle/sft_oracle.py), then the reference's own src/nn/fast_grpo.c running unchanged on top of
libllmb200.so (tests/c_api/grpo_drop_in.c) against the record of the same program over the reference's
engines on the CPU (tests/golden/grpo_golden*.bin). Sampled tokens must be identical; log-probabilities
within 1e-2 (the decode path's logits tolerance; they are logits / temperature - logsumexp). The gradient is
proportional to ratio = exp(new - old log-probability), and the old one comes from the decode path, so its
tolerance carries over: LoRA gradients within 5e-3 of the largest element on the fp32 CUDA-core path (measured
1e-3) and within 2e-2 with binary16 operands on the tensor cores (the engine's default)."""
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


def run_program(tmp_path, env_extra, mode="lora"):
    out = str(tmp_path / "b200.bin")
    env = dict(os.environ, **env_extra)
    r = subprocess.run([B200_BIN, out, mode], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600, env=env)
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
@pytest.mark.parametrize("mode", ["lora", "gemma", "gemma-hd256"])
def test_reference_grpo_loop_on_the_cuda_engines_fp32_path(tmp_path, mode):
    """LLMB200_SFT_TC=0: every product in fp32 on the CUDA cores, as the reference computes (the Gemma3 block
    order always runs that way). Both steps are compared: the second one generates with the adapter the first one
    trained. "gemma": grpo_state_create_gemma3 -- four norms per layer, GeGLU, scaled and tied embeddings, a RoPE
    base per layer; "gemma-hd256": the same with Gemma3-1B's head layout, four query heads of 256 on one key/value head."""
    want, want_tail = gr.by_step(gr.read(GOLDEN.replace(".bin", {"lora": ".bin", "gemma": "_gemma.bin",
                                                                 "gemma-hd256": "_gemma_hd256.bin"}[mode])))
    got, got_tail = run_program(tmp_path, {"LLMB200_SFT_TC": "0"}, mode)
    want_adapter, got_adapter = want_tail[gr.ADAPTER], got_tail[gr.ADAPTER]
    # the two LoRA-SFT steps after the GRPO steps (sft_train_step on the same state)
    assert np.abs(got_tail[gr.SFT_LOSS] - want_tail[gr.SFT_LOSS]).max() < 2e-3
    assert len(got) == len(want) == gr.STEPS
    for g, w in zip(got, want):
        compare_step(g, w, 5e-3)
    # AdamW turns a gradient element into a step of about lr whatever its size, so an element whose gradient is
    # rounding noise may move the other way: nearly all elements must agree closely, none by more than two steps
    diff = np.abs(got_adapter - want_adapter)
    assert diff.max() <= 2 * (gr.STEPS * 1e-2 + 2 * 1e-3) * 1.01
    assert (diff < 1e-4).mean() > 0.97, float((diff < 1e-4).mean())


@pytest.mark.skipif(not os.path.exists(B200_BIN), reason="tests/c_api/_bin/grpo_b200 was not built (reference tree absent)")
def test_reference_grpo_loop_on_the_cuda_engines_default_path(tmp_path):
    """The engine's default: frozen products on the tensor cores with binary16 operands. The first step samples
    from the untouched base model (B = 0), so its tokens must be the reference's; its gradients carry the
    operand rounding. The second step's samples depend on an adapter trained from those gradients and are not
    compared element by element."""
    want, _ = gr.by_step(gr.read(GOLDEN))
    got, got_tail = run_program(tmp_path, {})
    got_adapter = got_tail[gr.ADAPTER]
    assert len(got) == gr.STEPS
    compare_step(got[0], want[0], 2e-2)
    assert np.isfinite(got_adapter).all() and np.abs(got_adapter).max() > 0
    assert np.isfinite(got_tail[gr.SFT_LOSS]).all() and got_tail[gr.SFT_LOSS][1] < got_tail[gr.SFT_LOSS][0]
    assert np.isfinite(got[1][gr.REWARD]).all()


def test_sgd_apply_kernel(lib):
    """f16_sgd_apply on fp32 holders of binary16 values: w <- half(w - lr g), g <- 0."""
    rng = np.random.default_rng(5)
    n = 10007
    w = rng.standard_normal(n).astype(np.float16).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float16).astype(np.float32)
    d_w, d_g = dev(w), dev(g)
    assert lib.b200_sgd_apply_f16(d_w.data_ptr(), d_g.data_ptr(), n, 0.01, None) == 0
    torch.cuda.synchronize()
    got = d_w.cpu().numpy()
    exact = w.astype(np.float64) - 0.01 * g.astype(np.float64)
    assert (got == got.astype(np.float16).astype(np.float32)).all()               # binary16 values
    assert np.abs(got - exact).max() <= np.abs(exact).max() * 2.0 ** -11 + 1e-7   # half an ulp of binary16
    assert (d_g.cpu().numpy() == 0).all()


@pytest.mark.skipif(not os.path.exists(B200_BIN), reason="tests/c_api/_bin/grpo_b200 was not built (reference tree absent)")
@pytest.mark.parametrize("mode", ["full", "full-accurate", "gemma-full"])
def test_reference_grpo_loop_full_parameter_modes(tmp_path, mode):
    """grpo_state_create_full: every projection and the LM head stepped by SGD inside the backward passes
    ("full": at once, completion by completion; "full-accurate": accumulated in binary16 over the group, applied
    once), the decode state following the changed weights, then two sft_train_step calls and the checkpoint.
    Tokens must be the reference's in both steps (the second step samples from the stepped weights); the
    checkpoint must hold the reference's binary16 values up to single roundings."""
    want, want_tail = gr.by_step(gr.read(GOLDEN.replace(".bin", {"full": "_full.bin", "full-accurate": "_full_accurate.bin",
                                                                 "gemma-full": "_gemma_full.bin"}[mode])))
    got, got_tail = run_program(tmp_path, {}, mode)
    assert len(got) == len(want) == gr.STEPS
    for k, (g, w) in enumerate(zip(got, want)):
        assert (g[gr.TOKENS] == w[gr.TOKENS]).all(), ("sampled tokens differ from the reference run", k,
                                                       g[gr.TOKENS].astype(int).tolist(), w[gr.TOKENS].astype(int).tolist(),
                                                       g[gr.LOGPROBS].tolist(), w[gr.LOGPROBS].tolist())
        assert (g[gr.LEN] == w[gr.LEN]).all()
        # SGD steps of this size make the logits grow; the decode tolerance is relative to them, so the bound on a
        # log-probability scales with its size (measured: 0.018 at a log-probability of -5.6)
        for kind in (gr.LOGPROBS, gr.NEW_LP):
            assert (np.abs(g[kind] - w[kind]) <= 1e-2 * np.maximum(1.0, np.abs(w[kind]))).all(), kind
        assert (g[gr.REWARDS] == w[gr.REWARDS]).all()
        assert not g[gr.GRADS]
    assert np.abs(got_tail[gr.SFT_LOSS] - want_tail[gr.SFT_LOSS]).max() < 2e-3
    assert (got_tail[gr.CKPT_HEAD] == want_tail[gr.CKPT_HEAD]).all()
    a, b = got_tail[gr.CKPT_SAMPLE], want_tail[gr.CKPT_SAMPLE]
    assert a.shape == b.shape
    # binary16 weights: a product summed in another order may round a step the other way (one ulp, 2^-10 relative)
    assert np.abs(a - b).max() <= 2.0 ** -9 * np.abs(b).max()
    assert (a == b).mean() > 0.9, float((a == b).mean())
    assert got_tail[gr.CKPT_SUMS][0] == want_tail[gr.CKPT_SUMS][0]
    assert abs(float(got_tail[gr.CKPT_SUMS][2]) - float(want_tail[gr.CKPT_SUMS][2])) < 1e-3 * float(want_tail[gr.CKPT_SUMS][2])


def test_geglu_and_add_kernels(lib):
    rng = np.random.default_rng(11)
    rows, inter = 37, 300
    gu = (rng.standard_normal((rows, 2 * inter)) * 2).astype(np.float32)
    gu[0, :4] = [40.0, -40.0, 0.0, 1e-4]                       # the clamp region and the origin
    dy = rng.standard_normal((rows, inter)).astype(np.float32)
    g, u = gu[:, :inter], gu[:, inter:]
    d_gu, d_dy = dev(gu), dev(dy)
    act = torch.empty(rows, inter, dtype=torch.float32, device="cuda")
    dgu = torch.empty(rows, 2 * inter, dtype=torch.float32, device="cuda")
    assert lib.b200_gelu_mul_rows(d_gu.data_ptr(), rows, inter, act.data_ptr(), None) == 0
    assert lib.b200_gelu_mul_bwd_rows(d_dy.data_ptr(), d_gu.data_ptr(), rows, inter, dgu.data_ptr(), None) == 0
    torch.cuda.synchronize()
    want = o.gelu_mul(g, u)
    wg, wu = o.gelu_mul_backward(dy, g, u)
    assert np.abs(act.cpu().numpy() - want).max() < 1e-5 * max(1.0, np.abs(want).max())
    got = dgu.cpu().numpy()
    assert np.abs(got[:, :inter] - wg).max() < 1e-5 * max(1.0, np.abs(wg).max())
    assert np.abs(got[:, inter:] - wu).max() < 1e-5 * max(1.0, np.abs(wu).max())
    a, b = rng.standard_normal(1001).astype(np.float32), rng.standard_normal(1001).astype(np.float32)
    d_a, d_b = dev(a), dev(b)
    assert lib.b200_add(d_a.data_ptr(), d_b.data_ptr(), d_a.data_ptr(), 1001, None) == 0      # in place
    torch.cuda.synchronize()
    assert (d_a.cpu().numpy() == a + b).all()
