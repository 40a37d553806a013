"""LoRA-SFT on the GPU against the CPU restatement (oracle/sft_oracle.py): the kernels one by one,
then the engine end to end through the C ABI. Tolerances are the stated ones: loss and LoRA gradients
within 1e-2 relative, LoRA weights after one step within 1e-3 relative (the CUDA-core path is far
tighter and is held to 1e-4)."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import _sft_common as sc

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
o = sc.sft_oracle


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def gemm(pkg, lib, fn, A, a_row, a_col, B, b_row, b_col, M, N, K, alpha=1.0, R=None):
    g = pkg.GemmArgs()
    dA, dB = dev(A), dev(B)
    dC = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    g.A, g.a_row, g.a_col = dA.data_ptr(), a_row, a_col
    g.B, g.b_row, g.b_col = dB.data_ptr(), b_row, b_col
    g.C, g.ldc = dC.data_ptr(), N
    dR = dev(R) if R is not None else None
    g.R, g.ldr = (dR.data_ptr() if R is not None else None), N
    g.M, g.N, g.K, g.alpha = M, N, K, alpha
    rc = fn(C.byref(g), None)
    return rc, (host(dC) if rc == 0 else None)


@pytest.mark.parametrize("M,N,K", [(64, 64, 64), (70, 33, 45), (512, 16, 128), (16, 130, 512), (3, 5, 7)])
def test_gemm_f32_all_orientations(pkg, lib, M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    R = rng.standard_normal((M, N)).astype(np.float32)
    want = (A.astype(np.float64) @ B.astype(np.float64))
    for a_t in (False, True):
        for b_t in (False, True):
            Am = np.ascontiguousarray(A.T) if a_t else A           # stored [K, M] when a_t
            Bm = np.ascontiguousarray(B.T) if b_t else B           # stored [N, K] when b_t
            a_row, a_col = (1, M) if a_t else (K, 1)
            b_row, b_col = (1, K) if b_t else (N, 1)
            rc, got = gemm(pkg, lib, lib.b200_gemm_f32, Am, a_row, a_col, Bm, b_row, b_col, M, N, K, 0.5, R)
            assert rc == 0
            assert np.abs(got - (0.5 * want + R)).max() < 1e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (128, 128, 256), (70, 200, 100), (512, 384, 1024), (64, 640, 2560),
                                   (300, 64, 36),
                                   # tile widths the wave-aware choice picks for the SFT shapes: 80, 176, 112, 144
                                   (512, 2560, 128), (512, 6176, 64), (512, 4096, 96), (512, 9728, 32),
                                   # few tiles: several CTAs split a tile along k and add in turn (3 and 8 splits)
                                   (512, 2560, 4096), (128, 256, 2048), (100, 300, 1000)])
def test_gemm_tf32_tensor_cores(pkg, lib, M, N, K):
    """A = activations (rounded to TF32 by the tensor core), B = weights holding binary16 values
    (exact in TF32): the error is that of rounding A once, ~2^-11 relative per product."""
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = o.f16_round(rng.standard_normal((N, K)) * 0.02)
    R = rng.standard_normal((M, N)).astype(np.float32)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = pkg.GemmArgs()
    dA, dB, dR = dev(A), dev(B), dev(R)
    dC = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    g.A, g.a_row, g.a_col = dA.data_ptr(), K, 1
    g.B, g.b_row, g.b_col = dB.data_ptr(), 1, K
    g.C, g.ldc, g.R, g.ldr = dC.data_ptr(), N, dR.data_ptr(), N
    g.M, g.N, g.K, g.alpha, g.d_err = M, N, K, 0.5, err.data_ptr()
    assert lib.b200_gemm_tf32(C.byref(g), None) == 0
    got = host(dC)
    assert int(host(err)[0]) == 0
    want = 0.5 * (A.astype(np.float64) @ B.astype(np.float64).T) + R
    scale = np.abs(A.astype(np.float64)) @ np.abs(B.astype(np.float64)).T        # per-element error bound basis
    assert (np.abs(got - want) <= 2.0 ** -10 * 0.5 * scale + 1e-6).all()
    # and on average far better than the bound
    assert np.abs(got - want).mean() < 1e-3 * np.abs(want - R).mean() + 1e-6


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (70, 200, 104), (512, 2560, 4096), (512, 6176, 256), (512, 19456, 128),
                                   (128, 256, 4096), (64, 640, 2560),
                                   # few rows (batched decode: one row per sequence)
                                   (5, 768, 512), (32, 2560, 9728), (32, 19456, 256), (17, 300, 1000)])
def test_gemm_f16_tensor_cores(pkg, lib, M, N, K):
    """binary16 operands (the activation copy scaled by a power of two, as the engine does for gradients),
    fp32 accumulate: against float64 on the same rounded operands the only error is the accumulation's."""
    rng = np.random.default_rng(M + N + K + 1)
    A = (rng.standard_normal((M, K)) * 1e-4).astype(np.float32)          # gradient-sized values
    B = o.f16_round(rng.standard_normal((N, K)) * 0.02)
    R = rng.standard_normal((M, N)).astype(np.float32)
    scale = 4096.0
    dA32, dB32, dR = dev(A), dev(B), dev(R)
    dAh = torch.zeros(M, K, dtype=torch.float16, device="cuda")
    dBh = torch.zeros(N, K, dtype=torch.float16, device="cuda")
    assert lib.b200_f32_to_f16(dA32.data_ptr(), A.size, scale, dAh.data_ptr(), None) == 0
    assert lib.b200_f32_to_f16(dB32.data_ptr(), B.size, 1.0, dBh.data_ptr(), None) == 0
    Ah = host(dAh)
    assert np.array_equal(Ah, (A * np.float32(scale)).astype(np.float16))          # round to nearest even
    assert np.array_equal(host(dBh).astype(np.float32), B)                          # binary16 values are kept exactly
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    dC = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    g = pkg.GemmArgs()
    g.A, g.a_row, g.a_col = dAh.data_ptr(), K, 1
    g.B, g.b_row, g.b_col = dBh.data_ptr(), 1, K
    g.C, g.ldc, g.R, g.ldr = dC.data_ptr(), N, dR.data_ptr(), N
    g.M, g.N, g.K, g.alpha, g.d_err = M, N, K, 1.0 / scale, err.data_ptr()
    assert lib.b200_gemm_f16(C.byref(g), None) == 0
    got = host(dC)
    assert int(host(err)[0]) == 0
    want = (Ah.astype(np.float64) @ B.astype(np.float64).T) / scale + R
    bound = (np.abs(Ah.astype(np.float64)) @ np.abs(B.astype(np.float64)).T) / scale
    assert (np.abs(got - want) <= 1e-5 * bound + 1e-6).all()
    # transposed copy
    dT = torch.zeros(K, N, dtype=torch.float16, device="cuda")
    assert lib.b200_transpose_f16(dBh.data_ptr(), N, K, dT.data_ptr(), None) == 0
    assert np.array_equal(host(dT), host(dBh).T)


def test_gemm_tf32_refuses_what_it_cannot_do(pkg, lib):
    g = pkg.GemmArgs()
    x = torch.zeros(256 * 256, device="cuda")
    g.A, g.B, g.C = x.data_ptr(), x.data_ptr(), x.data_ptr()
    g.M, g.N, g.K, g.alpha, g.ldc = 128, 128, 128, 1.0, 128
    g.a_row, g.a_col, g.b_row, g.b_col = 1, 128, 1, 128          # A contiguous along m
    assert lib.b200_gemm_tf32(C.byref(g), None) == -4
    g.a_row, g.a_col, g.K = 130, 1, 130                          # K not a multiple of 4
    assert lib.b200_gemm_tf32(C.byref(g), None) == -4


def test_round_f16_is_bit_exact_and_transpose(pkg, lib):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((70, 45)) * 0.02).astype(np.float32)
    w[0, :4] = [0.0, 1e-8, 65519.0, -3.0e-5]
    d = dev(w)
    assert lib.b200_round_f16(d.data_ptr(), w.size, None) == 0
    got = host(d)
    assert np.array_equal(got.view(np.uint32), o.f16_round(w).view(np.uint32))
    t = torch.zeros(45, 70, dtype=torch.float32, device="cuda")
    assert lib.b200_transpose_f32(d.data_ptr(), 70, 45, t.data_ptr(), None) == 0
    assert np.array_equal(host(t), got.T)


@pytest.mark.parametrize("rows,dim", [(37, 200), (19, 2560)])
def test_rms_norm_rows_forward_and_backward(lib, rows, dim):
    rng = np.random.default_rng(4)
    eps = 1e-6
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    dy = rng.standard_normal((rows, dim)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    dx0 = rng.standard_normal((rows, dim)).astype(np.float32)
    dx, dg, dout = dev(x), dev(g), torch.zeros(rows, dim, device="cuda")
    assert lib.b200_rms_norm_rows(dx.data_ptr(), dg.data_ptr(), dout.data_ptr(), rows, dim, eps, None) == 0
    assert sc.rel_err(host(dout), o.rms_norm(x, g, eps)) < 1e-5
    ddy, dacc = dev(dy), dev(dx0)
    assert lib.b200_rms_norm_bwd_rows(dx.data_ptr(), ddy.data_ptr(), dim, dg.data_ptr(), dacc.data_ptr(), rows, dim, eps,
                                      1, 0.0, None) == 0
    assert sc.rel_err(host(dacc), dx0 + o.rms_norm_backward(x, dy, g, eps)) < 1e-5
    assert lib.b200_rms_norm_bwd_rows(dx.data_ptr(), ddy.data_ptr(), dim, dg.data_ptr(), dacc.data_ptr(), rows, dim, eps,
                                      0, 0.5, None) == 0
    assert sc.rel_err(host(dacc), np.clip(o.rms_norm_backward(x, dy, g, eps), -0.5, 0.5)) < 1e-5


@pytest.mark.parametrize("hd,N", [(64, 9), (128, 9), (256, 9), (128, 64), (64, 33), (128, 70)])
def test_qk_norm_rope_and_attention(lib, hd, N):
    """N <= 64 with head_dim <= 128 takes the one-block-per-head kernels, the rest the per-query kernels."""
    rng = np.random.default_rng(hd + N)
    S, Hq, Hkv, eps, theta = 2, 4, 2, 1e-6, 1e6
    M, QKV = S * N, (Hq + 2 * Hkv) * hd
    qkv = rng.standard_normal((M, QKV)).astype(np.float32)
    qg = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kg = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    d = np.arange(hd // 2, dtype=np.float32)
    inv_freq = (np.float32(1) / np.power(np.float32(theta), 2 * d / np.float32(hd), dtype=np.float32)).astype(np.float32)
    cos, sin = o.rope_angles(N, hd, theta, np.float32)
    scale = np.float32(1 / np.sqrt(hd))

    # ---- oracle, sequence by sequence
    q_want, k_want = np.zeros((M, Hq * hd), np.float32), np.zeros((M, Hkv * hd), np.float32)
    probs_want = np.zeros((S, Hq, N, N), np.float32)
    out_want = np.zeros((M, Hq * hd), np.float32)
    d_out = rng.standard_normal((M, Hq * hd)).astype(np.float32)
    dqkv_want = np.zeros((M, QKV), np.float32)
    for s in range(S):
        r = slice(s * N, (s + 1) * N)
        q_t = o.heads_fwd(qkv[r, :Hq * hd], Hq, hd)
        k_t = o.heads_fwd(qkv[r, Hq * hd:(Hq + Hkv) * hd], Hkv, hd)
        v_t = o.heads_fwd(qkv[r, (Hq + Hkv) * hd:], Hkv, hd)
        q_f = o.rope(o.rms_norm(q_t, qg, eps), cos, sin)
        k_f = o.rope(o.rms_norm(k_t, kg, eps), cos, sin)
        q_want[r], k_want[r] = o.heads_rev(q_f), o.heads_rev(k_f)
        G = Hq // Hkv
        k_e, v_e = np.repeat(k_f, G, axis=0), np.repeat(v_t, G, axis=0)
        att, p = o.attn_fwd(q_f, k_e, v_e, scale)
        probs_want[s], out_want[r] = p, o.heads_rev(att)
        dq, dk_e, dv_e = o.attn_bwd(o.heads_fwd(d_out[r], Hq, hd), p, q_f, k_e, v_e, scale)
        dk = dk_e.reshape(Hkv, G, N, hd).sum(axis=1)
        dv = dv_e.reshape(Hkv, G, N, hd).sum(axis=1)
        dq = o.rms_norm_backward(q_t, o.rope(dq, cos, sin, inverse=True), qg, eps)
        dk = o.rms_norm_backward(k_t, o.rope(dk, cos, sin, inverse=True), kg, eps)
        dqkv_want[r] = np.concatenate([o.heads_rev(dq), o.heads_rev(dk), o.heads_rev(dv)], axis=1)

    # ---- device
    dqkv_in, dqg, dkg, dfr = dev(qkv), dev(qg), dev(kg), dev(inv_freq)
    dq_f = torch.zeros(M, Hq * hd, device="cuda")
    dk_f = torch.zeros(M, Hkv * hd, device="cuda")
    assert lib.b200_qk_norm_rope(dqkv_in.data_ptr(), QKV, dqg.data_ptr(), dkg.data_ptr(), dfr.data_ptr(), M, N, Hq, Hkv,
                                 hd, eps, dq_f.data_ptr(), dk_f.data_ptr(), None) == 0
    assert sc.rel_err(host(dq_f), q_want) < 2e-5
    assert sc.rel_err(host(dk_f), k_want) < 2e-5
    probs = torch.full((S, Hq, N, N), 7.0, device="cuda")
    out = torch.zeros(M, Hq * hd, device="cuda")
    v_ptr = dqkv_in.data_ptr() + 4 * (Hq + Hkv) * hd
    assert lib.b200_attn_train_fwd(dq_f.data_ptr(), dk_f.data_ptr(), v_ptr, QKV, S, N, Hq, Hkv, hd, float(scale),
                                   probs.data_ptr(), out.data_ptr(), None) == 0
    assert np.abs(host(probs) - probs_want).max() < 2e-6
    assert sc.rel_err(host(out), out_want) < 2e-5
    d_score = torch.zeros(S * Hq * N * max(N, 2 * hd), device="cuda")
    dgrad = torch.zeros(M, QKV, device="cuda")
    ddo = dev(d_out)
    assert lib.b200_attn_train_bwd(ddo.data_ptr(), probs.data_ptr(), dq_f.data_ptr(), dk_f.data_ptr(), v_ptr, QKV, S, N,
                                   Hq, Hkv, hd, float(scale), d_score.data_ptr(), dgrad.data_ptr(), QKV, None) == 0
    assert lib.b200_qk_norm_rope_bwd(dgrad.data_ptr(), dqkv_in.data_ptr(), QKV, QKV, dqg.data_ptr(), dkg.data_ptr(),
                                     dfr.data_ptr(), M, N, Hq, Hkv, hd, eps, None) == 0
    assert sc.rel_err(host(dgrad), dqkv_want) < 5e-5


def test_silu_lora_add_softmax_ce(lib):
    rng = np.random.default_rng(8)
    rows, inter = 11, 70
    gu = rng.standard_normal((rows, 2 * inter)).astype(np.float32)
    dy = rng.standard_normal((rows, inter)).astype(np.float32)
    dgu, dact = dev(gu), torch.zeros(rows, inter, device="cuda")
    assert lib.b200_silu_mul_rows(dgu.data_ptr(), rows, inter, dact.data_ptr(), None) == 0
    assert sc.rel_err(host(dact), o.silu_mul(gu[:, :inter], gu[:, inter:])) < 1e-5
    ddy, dd = dev(dy), torch.zeros(rows, 2 * inter, device="cuda")
    assert lib.b200_silu_mul_bwd_rows(ddy.data_ptr(), dgu.data_ptr(), rows, inter, dd.data_ptr(), None) == 0
    dg, du = o.silu_mul_backward(dy, gu[:, :inter], gu[:, inter:])
    assert sc.rel_err(host(dd), np.concatenate([dg, du], axis=1)) < 1e-5

    for R in (16, 8, 40):                       # ranks below the kernel's register tile read no stale shared memory
        ld, col0, n_cols = 300, 40, 130
        y = rng.standard_normal((rows, ld)).astype(np.float32)
        mid = rng.standard_normal((rows, R + 3)).astype(np.float32)          # strided rows
        B = rng.standard_normal((n_cols, R)).astype(np.float32)
        dyy, dmid, dB = dev(y), dev(mid), dev(B)
        assert lib.b200_lora_add(dyy.data_ptr(), ld, col0, n_cols, dmid.data_ptr(), R + 3, dB.data_ptr(), R, 2.0, rows,
                                 None) == 0
        want = y.copy()
        want[:, col0:col0 + n_cols] += 2.0 * (mid[:, :R] @ B.T)
        assert sc.rel_err(host(dyy), want) < 1e-5

    for V in (5000, 5003):                      # four-at-a-time and scalar paths
        logits = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
        tg = rng.integers(0, V, rows).astype(np.uint32)
        dl, dt = dev(logits), dev(tg.view(np.int32))
        losses, dlog = torch.zeros(rows, device="cuda"), torch.zeros(rows, V, device="cuda")
        dlog_h = torch.zeros(rows, V, dtype=torch.float16, device="cuda")
        assert lib.b200_softmax_ce_rows_h(dl.data_ptr(), dt.data_ptr(), rows, V, 0.25, losses.data_ptr(), dlog.data_ptr(),
                                          dlog_h.data_ptr(), 64.0, None) == 0
        wl, wd = o.softmax_ce(logits.astype(np.float64), tg.astype(np.int64))
        assert np.abs(host(losses) - wl).max() < 1e-5
        got = host(dlog)
        assert np.abs(got - 0.25 * wd).max() < 1e-6
        assert np.array_equal(host(dlog_h), (got * np.float32(64.0)).astype(np.float16))
        dlog2 = torch.zeros(rows, V, device="cuda")
        assert lib.b200_softmax_ce_rows(dl.data_ptr(), dt.data_ptr(), rows, V, 0.25, losses.data_ptr(), dlog2.data_ptr(),
                                        None) == 0
        assert np.array_equal(host(dlog2), got)


@pytest.mark.parametrize("rows,P,R", [(512, 4096, 16), (37, 130, 8), (300, 2560, 16), (64, 2560, 3)])
def test_xty_skinny_lora_gradients(lib, rows, P, R):
    rng = np.random.default_rng(P + R)
    X = rng.standard_normal((rows, P + 5)).astype(np.float32)
    Y = rng.standard_normal((rows, R + 3)).astype(np.float32)
    dX, dY = dev(X), dev(Y)
    want = 0.5 * (X[:, :P].astype(np.float64).T @ Y[:, :R].astype(np.float64))
    c1 = torch.zeros(P, R, device="cuda")
    assert lib.b200_xty_skinny(dX.data_ptr(), P + 5, dY.data_ptr(), R + 3, rows, P, R, 0.5, c1.data_ptr(), R, 1, None) == 0
    assert sc.rel_err(host(c1), want) < 1e-5
    c2 = torch.zeros(R, P, device="cuda")
    assert lib.b200_xty_skinny(dX.data_ptr(), P + 5, dY.data_ptr(), R + 3, rows, P, R, 0.5, c2.data_ptr(), 1, P, None) == 0
    assert sc.rel_err(host(c2), want.T) < 1e-5


def test_clip_and_adamw_kernels(lib):
    rng = np.random.default_rng(9)
    n = 100003
    for gscale in (3.0, 1e-4):                      # clipped, not clipped
        p = rng.standard_normal(n).astype(np.float32)
        g = (rng.standard_normal(n) * gscale).astype(np.float32)
        m = (rng.standard_normal(n) * 0.01).astype(np.float32)
        v = (rng.random(n) * 0.01).astype(np.float32)
        lora = o.LoRA([dict(A_q=p.reshape(1, -1), B_q=np.zeros((1, 1), np.float32), A_v=np.zeros((1, 1), np.float32),
                            B_v=np.zeros((1, 1), np.float32))], 1, 1.0)
        lora.m[0]["A_q"], lora.v[0]["A_q"] = m.reshape(1, -1).copy(), v.reshape(1, -1).copy()
        lora.step_count = 3
        grads = [dict(A_q=g.reshape(1, -1), B_q=np.zeros((1, 1), np.float32), A_v=np.zeros((1, 1), np.float32),
                      B_v=np.zeros((1, 1), np.float32))]
        clipped, norm = o.clip_grad_norm(grads, 1.0)
        o.adamw(lora, clipped, 1e-2)
        dp, dg, dm, dv = dev(p), dev(g), dev(m), dev(v)
        parts = torch.zeros(256, dtype=torch.float64, device="cuda")
        dn = torch.zeros(1, device="cuda")
        assert lib.b200_sumsq_partials(dg.data_ptr(), n, parts.data_ptr(), 256, None) == 0
        bc1 = float(np.float32(1) - np.power(np.float32(0.9), np.float32(3), dtype=np.float32))
        bc2 = float(np.float32(1) - np.power(np.float32(0.999), np.float32(3), dtype=np.float32))
        assert lib.b200_clip_adamw(dp.data_ptr(), dg.data_ptr(), dm.data_ptr(), dv.data_ptr(), n, parts.data_ptr(), 256,
                                   1.0, 1e-2, 0.9, 0.999, 1e-8, 0.01, bc1, bc2, 1, dn.data_ptr(), None) == 0
        assert abs(float(host(dn)[0]) - norm) < 1e-6 * norm
        assert sc.rel_err(host(dg), clipped[0]["A_q"].ravel()) < 1e-6
        assert sc.rel_err(host(dp), lora.p[0]["A_q"].ravel()) < 1e-6
        assert sc.rel_err(host(dm), lora.m[0]["A_q"].ravel()) < 1e-6
        assert sc.rel_err(host(dv), lora.v[0]["A_q"].ravel()) < 1e-6


# ---- the engine ------------------------------------------------------------------------------------------

RANK, ALPHA = 8, 16.0


def run_case(pkg, cfg, n, S, b_std, tensor_cores, tol_grad, tol_param, steps=1, lr=1e-3):
    w = sc.make_weights(pkg, cfg)
    ow = sc.oracle_model(cfg, w)
    toks = sc.tokens(pkg, S * (n + 1), 4321, cfg["vocab_size"]).reshape(S, n + 1)
    x, y = toks[:, :-1], toks[:, 1:]
    init = sc.make_lora(pkg, cfg, RANK, b_std=b_std)
    lora = o.LoRA(init, RANK, ALPHA)
    eng = sc.Engine(pkg, cfg, w, init, n, S, RANK, ALPHA, tensor_cores=tensor_cores)
    try:
        for step in range(steps):
            want_loss, want_g, want_norm = o.train_step(ow, lora, x, y, lr)
            loss = eng.forward_backward(x, y)
            got_g = eng.grads()
            assert abs(loss - want_loss) < tol_grad * abs(want_loss), (step, loss, want_loss)
            for L in range(cfg["n_layers"]):
                for k in o.KEYS:
                    if np.abs(want_g[L][k]).max() == 0:
                        assert np.abs(got_g[L][k]).max() == 0, (step, L, k)
                    else:
                        assert sc.rel_err(got_g[L][k], want_g[L][k]) < tol_grad, (step, L, k)
            eng.L.llmb200_sft_apply_update(eng.h, lr)
            assert abs(eng.L.llmb200_sft_last_grad_norm(eng.h) - want_norm) < tol_grad * want_norm
            got_p = eng.params()
            for L in range(cfg["n_layers"]):
                for k in o.KEYS:
                    if np.abs(lora.p[L][k]).max() == 0:
                        assert np.abs(got_p[L][k]).max() == 0
                    else:
                        # AdamW's first steps move a weight by lr*g/(|g|+1e-8): where |g| is near 1e-8 the
                        # step depends on the last bits of g, so single elements of a matrix that started
                        # at zero can be off by more than the matrix as a whole
                        d = got_p[L][k].astype(np.float64) - lora.p[L][k]
                        rel_l2 = np.sqrt((d * d).sum() / (lora.p[L][k].astype(np.float64) ** 2).sum())
                        assert rel_l2 < tol_param, (step, L, k, rel_l2)
                        assert sc.rel_err(got_p[L][k], lora.p[L][k]) < 30 * tol_param, (step, L, k)
        return eng, lora, ow, (x, y)
    except Exception:
        eng.close()
        raise


def test_engine_small_one_sequence_cuda_cores(pkg):
    eng, *_ = run_case(pkg, sc.SMALL, 12, 1, 0.02, False, 1e-4, 1e-4, steps=2)
    eng.close()


def test_engine_tiny_qwen3_two_sequences_three_steps(pkg):
    """hidden 512, 4 layers, 8/2 heads, seq 64: the architecture of the CPU-runnable decode case.
    B starts at zero, as configured, so the first step has dA = 0 exactly. The first AdamW step
    moves every weight by lr * g/(|g| + 1e-8): where |g| is near 1e-8 the step depends on the last
    bits of g, hence the stated 1e-3 on the weights while the gradients are held to 1e-4."""
    eng, *_ = run_case(pkg, sc.TINY, 64, 2, 0.0, False, 1e-4, 1e-3, steps=3, lr=1e-2)
    eng.close()


def test_engine_tensor_core_path_within_stated_tolerance(pkg):
    # lr as configured for the SFT workload (1e-4): TF32 rounding of the activations moves small gradients by
    # up to a percent, and AdamW turns that into a few percent of a step of size lr where |g| is near its epsilon
    eng, *_ = run_case(pkg, sc.TINY, 64, 2, 0.02, True, 1e-2, 1e-3, steps=2, lr=1e-4)
    eng.close()


def test_engine_against_the_reference_engine_vectors(pkg):
    """Three steps on the tiny configuration against what the reference's own fast_sft.c computed
    (tests/golden/sft_golden.npz, made by tests/golden/make_sft_golden.py): loss and the clipped gradient
    buffers of every step, the weights after the third."""
    import os
    G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sft_golden.npz"))
    cfg = dict(sc.TINY)
    rank, alpha, lr, n = int(G["rank"]), float(G["alpha"]), float(G["lr"]), int(G["seq_len"])
    w = sc.make_weights(pkg, cfg)
    init = sc.make_lora(pkg, cfg, rank)
    eng = sc.Engine(pkg, cfg, w, init, n, 1, rank, alpha, tensor_cores=False)
    try:
        for step in range(3):
            loss = eng.forward_backward(G["inputs"], G["targets"])
            assert abs(loss - float(G[f"loss_{step}"])) < 1e-4 * abs(loss), (step, loss)
            assert sc.rel_err(eng.export(sc.LOSSES, 0, n), G[f"losses_{step}"]) < 1e-4
            got = eng.grads()
            norm = np.sqrt(sum(float((got[L][k].astype(np.float64) ** 2).sum()) for L in range(cfg["n_layers"]) for k in o.KEYS))
            scale = 1.0 / norm if norm > 1.0 else 1.0             # the reference's buffers hold the clipped values
            for L in range(cfg["n_layers"]):
                for k in o.KEYS:
                    want = G[f"grad_{step}_{L}_{k}"]
                    if not want.any():
                        assert not got[L][k].any(), (step, L, k)
                    else:
                        # free-running: from the second step on the weights carry AdamW's amplified rounding
                        assert sc.rel_err(got[L][k] * scale, want) < (1e-4 if step == 0 else 2e-3), (step, L, k)
            eng.L.llmb200_sft_apply_update(eng.h, lr)
        got_p = eng.params()
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                want = G[f"weight_{L}_{k}"]
                d = got_p[L][k].astype(np.float64) - want
                assert np.sqrt((d * d).sum() / (want.astype(np.float64) ** 2).sum()) < 1e-3, (L, k)
    finally:
        eng.close()


def test_gemma3_engine_against_the_reference_engine_vectors(pkg):
    """The Gemma3 block order of the engine (fp32 path) against sft_state_create_gemma3 + sft_train_step of the
    reference (tests/golden/sft_golden_gemma3.npz): two layers, four query heads of 256 on one key/value head, a
    global and a local RoPE base."""
    import os
    G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sft_golden_gemma3.npz"))
    sp = pkg.spec("tiny-gemma3", gamma_jitter=0.1, n_layers=2)
    cfg = sc.gemma_cfg(sp)
    rank, alpha, lr, n = int(G["rank"]), float(G["alpha"]), float(G["lr"]), int(G["seq_len"])
    eng = sc.Engine(pkg, cfg, sc.make_weights_gemma(pkg, cfg), sc.make_lora(pkg, cfg, rank), n, 1, rank, alpha)
    try:
        for step in range(3):
            loss = eng.forward_backward(G["inputs"], G["targets"])
            assert abs(loss - float(G[f"loss_{step}"])) < 1e-4 * abs(loss), (step, loss)
            assert sc.rel_err(eng.export(sc.LOSSES, 0, n), G[f"losses_{step}"]) < 1e-4
            got = eng.grads()
            norm = np.sqrt(sum(float((got[L][k].astype(np.float64) ** 2).sum()) for L in range(cfg["n_layers"]) for k in o.KEYS))
            scale = 1.0 / norm if norm > 1.0 else 1.0
            for L in range(cfg["n_layers"]):
                for k in o.KEYS:
                    want = G[f"grad_{step}_{L}_{k}"]
                    if not want.any():
                        assert not got[L][k].any(), (step, L, k)
                    else:
                        assert sc.rel_err(got[L][k] * scale, want) < (1e-4 if step == 0 else 2e-3), (step, L, k)
            eng.L.llmb200_sft_apply_update(eng.h, lr)
        got_p = eng.params()
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                want = G[f"weight_{L}_{k}"]
                d = got_p[L][k].astype(np.float64) - want
                assert np.sqrt((d * d).sum() / (want.astype(np.float64) ** 2).sum()) < 1e-3, (L, k)
    finally:
        eng.close()


@pytest.mark.parametrize("mode", ["sgd", "accum"])
def test_full_parameter_engine_against_the_reference_engine_vectors(pkg, lib, synth, mode):
    """sft_state_create_full through the reference's calls: three sft_train_step calls that step every matrix
    inside the backward pass, or accumulators, two accumulating steps and one apply
    (tests/golden/sft_golden_full.npz). Losses to 1e-4; the sampled binary16 weights equal the reference's except
    for single roundings."""
    import ctypes as C
    import os
    G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sft_golden_full.npz"))
    stride, lr, n = int(G["stride"]), float(G["lr"]), int(G["seq_len"])
    sp = pkg.spec("tiny-qwen3", gamma_jitter=0.1, n_layers=2)
    model = synth.llmb200_synth_qwen3(C.byref(sp), 4)
    st = lib.sft_state_create_full(model, n)
    assert st and lib.sft_is_full_param(st) == 1 and lib.sft_get_lora_rank(st) == 0
    try:
        x = np.ascontiguousarray(G["inputs"], dtype=np.uint32)
        y = np.ascontiguousarray(G["targets"], dtype=np.uint32)
        if mode == "accum":
            lib.sft_alloc_grad_accum(st)
        for step in range(3 if mode == "sgd" else 2):
            loss = lib.sft_train_step(st, x.ctypes.data_as(pkg.c_u32_p), y.ctypes.data_as(pkg.c_u32_p), lr)
            assert abs(loss - float(G[f"{mode}_loss"][step])) < 1e-4 * abs(loss), (step, loss)
            losses = np.ctypeslib.as_array(lib.sft_get_losses_cpu(st), shape=(n,)).copy()
            assert sc.rel_err(losses, G[f"{mode}_losses_{step}"]) < 1e-4
        if mode == "accum":
            lib.sft_apply_grad_sgd(st, lr)
        lw = C.cast(lib.sft_get_layers(st), C.POINTER(pkg.LayerW))
        mats = [getattr(lw[L], m).contents for L in range(sp.n_layers)
                for m in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")]
        mats.append(C.cast(lib.sft_get_lm_head(st), C.POINTER(pkg.WMat)).contents)
        parts = []
        for wm in mats:
            a = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(wm.mbuf), C.POINTER(C.c_uint16)), shape=(wm.rows * wm.cols,))
            parts.append(a[::stride].copy())
        got = np.concatenate(parts).view(np.float16).astype(np.float32)
        want = G[f"{mode}_weights"].astype(np.float32)
        assert got.shape == want.shape
        assert (got == want).mean() > 0.97, float((got == want).mean())
        assert np.abs(got - want).max() <= 2.0 ** -10 * np.abs(want).max()
    finally:
        lib.sft_state_free(st)
        synth.llmb200_synth_free_qwen3(model)


def test_saved_activations_and_logits(pkg):
    cfg, n = sc.SMALL, 12
    eng, lora, ow, (x, y) = run_case(pkg, cfg, n, 1, 0.02, False, 1e-4, 1e-4, steps=1)
    try:
        loss = eng.forward_backward(x, y)                      # second pass with the updated LoRA
        logits, (saves, fin) = o.forward(ow, lora, x[0])
        D, V = cfg["d_model"], cfg["vocab_size"]
        assert sc.rel_err(eng.export(sc.LOGITS, 0, n * V), logits.ravel()) < 1e-4
        for L in range(cfg["n_layers"]):
            assert sc.rel_err(eng.export(sc.X_IN, L, n * D), saves[L]["x_in"].ravel()) < 1e-4
            assert sc.rel_err(eng.export(sc.LN2, L, n * D), saves[L]["ln2"].ravel()) < 1e-4
            pr = eng.export(sc.PROBS, L, cfg["n_q_heads"] * n * n)
            assert np.abs(pr - saves[L]["probs"].ravel()).max() < 1e-5
            assert sc.rel_err(eng.export(sc.MID_Q, L, n * RANK), saves[L]["q_mid"].ravel()) < 1e-4
        losses, _ = o.softmax_ce(logits, y[0].astype(np.int64))
        assert np.abs(eng.export(sc.LOSSES, 0, n) - losses).max() < 1e-4
        assert abs(loss - float(losses.mean())) < 1e-4
    finally:
        eng.close()


def test_batch_gradient_is_the_mean_of_single_sequence_gradients(pkg):
    cfg, n = sc.SMALL, 12
    w = sc.make_weights(pkg, cfg)
    toks = sc.tokens(pkg, 3 * (n + 1), 99, cfg["vocab_size"]).reshape(3, n + 1)
    init = sc.make_lora(pkg, cfg, RANK, b_std=0.02)
    one = sc.Engine(pkg, cfg, w, init, n, 1, RANK, ALPHA, tensor_cores=False)
    three = sc.Engine(pkg, cfg, w, init, n, 3, RANK, ALPHA, tensor_cores=False)
    try:
        acc, losses = None, []
        for s in range(3):
            losses.append(one.forward_backward(toks[s, :-1], toks[s, 1:]))
            g = one.grads()
            acc = g if acc is None else [{k: a[k] + b[k] for k in o.KEYS} for a, b in zip(acc, g)]
        loss = three.forward_backward(toks[:, :-1], toks[:, 1:])
        got = three.grads()
        assert abs(loss - np.mean(losses)) < 1e-5
        for L in range(cfg["n_layers"]):
            for k in o.KEYS:
                assert sc.rel_err(got[L][k], acc[L][k] / 3) < 1e-4
    finally:
        one.close()
        three.close()


def test_reference_api_surface(pkg, lib, synth, tmp_path):
    """sft_state_create on a model struct, sft_train_step, the gradient accessors, sft_lora_update,
    sft_save_lora and forward_to_logits from caller-supplied embeddings."""
    spec = pkg.spec("tiny-qwen3", n_layers=2, vocab_size=1024)
    m = synth.llmb200_synth_qwen3(spec, 4)
    n, R = 16, 4
    st = lib.sft_state_create(m, n, R, 8.0)
    assert st
    try:
        assert lib.sft_get_seq_len(st) == n and lib.sft_get_vocab_size(st) == 1024 and lib.sft_get_d_model(st) == 512
        assert lib.sft_get_lora_rank(st) == R and lib.sft_get_n_layers(st) == 2
        assert lib.sft_get_emb_scale(st) == 1.0 and lib.sft_get_lora_scaling(st) == 2.0
        assert lib.sft_get_n_lora_grad_bufs(st) == 8 and lib.sft_get_step_count(st) == 0
        D, V = 512, 1024
        # default init: A uniform within +-1/sqrt(D), B zero
        a = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(lib.sft_get_lora_weight_buf(st, 0, 0)),
                                         C.POINTER(C.c_float)), shape=(R * D,)).copy()
        b = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(lib.sft_get_lora_weight_buf(st, 1, 1)),
                                         C.POINTER(C.c_float)), shape=(8 * 64 * R,)).copy()
        assert np.abs(a).max() <= 1 / np.sqrt(D) and a.std() > 0.01 and not b.any()
        toks = sc.tokens(pkg, n + 1, 5, V)
        x, y = toks[:-1].copy(), toks[1:].copy()
        px, py = x.ctypes.data_as(C.POINTER(C.c_uint32)), y.ctypes.data_as(C.POINTER(C.c_uint32))
        l0 = lib.sft_train_step(st, px, py, 1e-2)
        assert lib.sft_get_step_count(st) == 1
        assert abs(l0 - np.log(V)) < 0.5
        losses = [lib.sft_train_step(st, px, py, 1e-2) for _ in range(5)]
        assert losses[-1] < l0
        per_pos = np.ctypeslib.as_array(lib.sft_get_losses_cpu(st), shape=(n,))
        assert abs(per_pos.mean() - losses[-1]) < 1e-5

        # gradient accessors: read, scale on the host, write back, update
        sz = C.c_int()
        g = lib.sft_get_lora_grad_ptr(st, 1, C.byref(sz))                 # layer 0, dB_q
        assert sz.value == 8 * 64 * R
        ga = np.ctypeslib.as_array(g, shape=(sz.value,)).copy()
        assert ga.any()
        half = (ga * 0.5).astype(np.float32)
        lib.sft_set_lora_grad(st, 1, half.ctypes.data_as(C.POINTER(C.c_float)), sz.value)
        again = np.ctypeslib.as_array(lib.sft_get_lora_grad_ptr(st, 1, None), shape=(sz.value,)).copy()
        assert np.array_equal(again, half)
        before = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(lib.sft_get_lora_weight_buf(st, 0, 1)),
                                              C.POINTER(C.c_float)), shape=(sz.value,)).copy()
        lib.sft_lora_update(st, 1e-2)
        assert lib.sft_get_step_count(st) == 6                              # not incremented by sft_lora_update
        after = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(lib.sft_get_lora_weight_buf(st, 0, 1)),
                                             C.POINTER(C.c_float)), shape=(sz.value,)).copy()
        assert not np.array_equal(before, after)

        # adapter file
        path = str(tmp_path / "adapter.lora")
        lib.sft_save_lora(st, path.encode())
        blob = open(path, "rb").read()
        assert struct.unpack_from("<Iii", blob) == (0x4C4F5241, 2, R)
        per = R * D + 8 * 64 * R + R * D + 2 * 64 * R
        assert len(blob) == 12 + 4 * per * 2
        file_b = np.frombuffer(blob, dtype="<f4", count=sz.value, offset=12 + 4 * R * D)
        assert np.array_equal(file_b, after)

        # forward_to_logits from embeddings the caller wrote
        emb = np.ctypeslib.as_array(lib.sft_get_token_emb(st), shape=(V, D))
        xc = np.ctypeslib.as_array(lib.sft_get_x_cpu(st), shape=(n, D))
        xc[:] = emb[x.astype(np.int64)]
        lib.forward_to_logits(st)
        lg = np.ctypeslib.as_array(C.cast(lib.metal_buf_ptr(lib.sft_get_logits(st)), C.POINTER(C.c_float)),
                                   shape=(n, V)).copy()
        ref = np.empty(n * V, dtype=np.float32)
        lib.sft_train_step(st, px, py, 0.0)          # same LoRA (lr 0 leaves p unchanged up to weight decay 0)
        assert lib.llmb200_sft_export(st, sc.LOGITS, 0, ref.ctypes.data, ref.size) == ref.size
        assert sc.rel_err(lg.ravel(), ref) < 1e-5
        assert lib.llmb200_sft_error(st) == 0
    finally:
        lib.sft_state_free(st)
        synth.llmb200_synth_free_qwen3(m)
