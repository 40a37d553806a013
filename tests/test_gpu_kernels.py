"""GPU parity of the individual kernels, called through the C ABI, against the CPU oracle.

Bars: Q8_0 / F16 conversion bit-exact; matvec within 2e-4 of max|y| (fp32
accumulation in a different order); attention within 2e-3 of max|out| (the KV
cache is binary16, the oracle is run with the same cache rounding).
"""
import ctypes as C

import numpy as np
import pytest

import _oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SWEEP = [(4096, 2560), (1024, 2560), (2560, 4096), (9728, 2560), (2560, 9728)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def weights(synth, rows, cols, tid, std=0.02):
    w = np.empty((rows, cols), dtype=np.float32)
    synth.llmb200_synth_normal(w.ctypes.data, w.size, 1234, tid, 0.0, std, 8)
    return w


def pack(lib, pkg, w, wtype, dst_row0=0, step=1, total_rows=None):
    rows, cols = w.shape
    total_rows = total_rows or rows
    stride = lib.b200_packed_row_stride(wtype, cols)
    d_src = dev(w)
    d_dst = torch.zeros(stride * total_rows, dtype=torch.uint8, device="cuda")
    fn = lib.b200_q8_pack if wtype == pkg.B200_WT_Q8 else lib.b200_f16_pack
    rc = fn(d_src.data_ptr(), cols, rows, cols, d_dst.data_ptr(), stride, dst_row0, step, None)
    assert rc == 0
    torch.cuda.synchronize()
    return d_dst, stride


@pytest.mark.parametrize("rows,cols", [(8, 32), (3, 96), (64, 2560), (1024, 2560), (257, 9728)])
def test_q8_pack_bit_exact(lib, pkg, synth, rows, cols):
    w = weights(synth, rows, cols, 7)
    if rows >= 3:
        w[1, :32] = 0.0            # all-zero block
        w[2, 5] = 3.0e38           # huge magnitude
        w[0, 0] = -1e-30           # denormal-ish scale
    d_packed, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    d_blocks = torch.zeros(rows * (cols // 32) * 34, dtype=torch.uint8, device="cuda")
    assert lib.b200_q8_unpack_blocks(d_packed.data_ptr(), stride, rows, cols, d_blocks.data_ptr(), None) == 0
    got = d_blocks.cpu().numpy()
    assert np.array_equal(got, O.q8_quantize(w))


def test_q8_pack_rounding_ties(lib, pkg):
    # values that land exactly on .5 after scaling: roundf rounds half away from zero
    w = np.zeros((1, 32), dtype=np.float32)
    w[0, 0] = 127.0
    w[0, 1:9] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5]
    d_packed, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    d_blocks = torch.zeros(34, dtype=torch.uint8, device="cuda")
    assert lib.b200_q8_unpack_blocks(d_packed.data_ptr(), stride, 1, 32, d_blocks.data_ptr(), None) == 0
    got = d_blocks.cpu().numpy()
    assert np.array_equal(got, O.q8_quantize(w))
    assert list(got[2:11].view(np.int8)) == [127, 1, -1, 2, -2, 3, -3, 127, -127]


@pytest.mark.parametrize("rows,cols", [(5, 8), (64, 1152), (33, 6912)])
def test_f16_pack_bit_exact(lib, pkg, synth, rows, cols):
    w = weights(synth, rows, cols, 9)
    w[0, 0] = 65520.0          # rounds to inf in binary16
    w[0, 1] = 6.0e-8           # subnormal half
    d_packed, stride = pack(lib, pkg, w, pkg.B200_WT_F16)
    got = d_packed.cpu().numpy().reshape(rows, stride)[:, :cols * 2].copy().view(np.uint16)
    assert np.array_equal(got, O.f16_bits(w))


def run_matvec(lib, pkg, d_w, stride, rows, cols, wtype, x, **kw):
    a = pkg.MatvecArgs()
    a.d_w, a.row_stride, a.rows, a.cols, a.wtype = d_w.data_ptr(), stride, rows, cols, wtype
    a.in_mode = pkg.B200_IN_VEC
    d_x = dev(x)
    a.d_in_vec = d_x.data_ptr()
    a.out_mode = pkg.B200_OUT_STORE
    d_y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    a.d_out[0] = d_y.data_ptr()
    a.n_out = 1
    a.eps = 1e-6
    for k, v in kw.items():
        setattr(a, k, v)
    assert lib.b200_matvec(C.byref(a), None) == 0
    torch.cuda.synchronize()
    return d_y.cpu().numpy()


@pytest.mark.parametrize("rows,cols", SWEEP + [(768, 512), (512, 1536), (40, 32), (7, 16384)])
def test_q8_matvec_vs_oracle(lib, pkg, synth, rows, cols):
    w = weights(synth, rows, cols, 11)
    x = weights(synth, 1, cols, 99, std=1.0)[0]
    d_w, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    y = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x)
    ref = O.q8_matvec(O.q8_quantize(w), x, rows, cols)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()
    # the CPU reference path multiplies dequantised fp32 weights instead (src/nn/layers.c:136-150)
    ref2 = O.linear(O.q8_dequantize(O.q8_quantize(w), rows, cols), x)
    assert np.abs(y - ref2).max() <= 2e-4 * np.abs(ref2).max()


@pytest.mark.parametrize("grid", [1, 3, 148, 1000])
def test_q8_matvec_any_grid(lib, pkg, synth, grid):
    rows, cols = 777, 2560
    w = weights(synth, rows, cols, 12)
    x = weights(synth, 1, cols, 98, std=1.0)[0]
    d_w, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    y = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x, grid=grid)
    ref = O.q8_matvec(O.q8_quantize(w), x, rows, cols)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()


@pytest.mark.parametrize("rows,cols", [(1024, 1152), (1152, 1024), (6912, 1152), (1152, 6912), (2560, 9728), (9, 8)])
def test_f16_matvec_vs_oracle(lib, pkg, synth, rows, cols):
    w = weights(synth, rows, cols, 13)
    x = weights(synth, 1, cols, 97, std=1.0)[0]
    d_w, stride = pack(lib, pkg, w, pkg.B200_WT_F16)
    y = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_F16, x)
    ref = O.f16_matvec(O.f16_bits(w), x)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()


def test_matvec_is_linear_and_deterministic(lib, pkg, synth):
    rows, cols = 9728, 2560
    w = weights(synth, rows, cols, 14)
    x1 = weights(synth, 1, cols, 96, std=1.0)[0]
    x2 = weights(synth, 1, cols, 95, std=1.0)[0]
    d_w, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    y1 = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x1)
    y1b = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x1)
    y2 = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x2)
    y12 = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x1 + x2)
    assert np.array_equal(y1, y1b)
    assert np.abs(y12 - (y1 + y2)).max() <= 1e-4 * np.abs(y12).max()


def test_matvec_fused_norm_glu_and_argmax(lib, pkg, synth):
    # rms_norm prologue + interleaved gate/up + SiLU*up epilogue, then argmax over a plain matvec
    D, IS = 512, 1536
    wg, wu = weights(synth, IS, D, 20), weights(synth, IS, D, 21)
    x = weights(synth, 1, D, 94, std=1.0)[0]
    gamma = (1.0 + 0.1 * weights(synth, 1, D, 93, std=1.0)[0]).astype(np.float32)
    stride = lib.b200_packed_row_stride(pkg.B200_WT_Q8, D)
    d_w = torch.zeros(stride * 2 * IS, dtype=torch.uint8, device="cuda")
    for src, r0 in ((wg, 0), (wu, 1)):
        d_src = dev(src)
        assert lib.b200_q8_pack(d_src.data_ptr(), D, IS, D, d_w.data_ptr(), stride, r0, 2, None) == 0
    torch.cuda.synchronize()
    a = pkg.MatvecArgs()
    a.d_w, a.row_stride, a.rows, a.cols, a.wtype = d_w.data_ptr(), stride, 2 * IS, D, pkg.B200_WT_Q8
    a.in_mode = pkg.B200_IN_RESID
    d_x, d_g = dev(x), dev(gamma)
    d_res = torch.zeros(D, dtype=torch.float32, device="cuda")
    a.d_resid_in, a.d_resid_out, a.n_slots = d_x.data_ptr(), d_res.data_ptr(), 0
    a.d_norm_gamma, a.eps = d_g.data_ptr(), 1e-6
    a.out_mode, a.act = pkg.B200_OUT_GLU, 0
    d_act = torch.zeros(IS, dtype=torch.float32, device="cuda")
    a.d_out[0], a.n_out = d_act.data_ptr(), 1
    assert lib.b200_matvec(C.byref(a), None) == 0
    torch.cuda.synchronize()
    xn = np.zeros(D, dtype=np.float32)
    O.lib().oracle_rms_norm(x.ctypes.data, gamma.ctypes.data, xn.ctypes.data, D, 1e-6)
    g = O.q8_matvec(O.q8_quantize(wg), xn, IS, D)
    u = O.q8_matvec(O.q8_quantize(wu), xn, IS, D)
    ref = (g / (1.0 + np.exp(-g))) * u
    got = d_act.cpu().numpy()
    assert np.abs(got - ref).max() <= 3e-4 * np.abs(ref).max()
    assert np.array_equal(d_res.cpu().numpy(), x)

    # argmax with ties: duplicate the winning row so that the first index must win
    rows, cols = 4096, 512
    w = weights(synth, rows, cols, 22)
    xv = weights(synth, 1, cols, 92, std=1.0)[0]
    y0 = O.q8_matvec(O.q8_quantize(w), xv, rows, cols)
    best = int(np.argmax(y0))
    w[(best + 1000) % rows] = w[best]
    d_w2, stride2 = pack(lib, pkg, w, pkg.B200_WT_Q8)
    b = pkg.MatvecArgs()
    b.d_w, b.row_stride, b.rows, b.cols, b.wtype = d_w2.data_ptr(), stride2, rows, cols, pkg.B200_WT_Q8
    b.in_mode = pkg.B200_IN_VEC
    d_xv = dev(xv)
    b.d_in_vec = d_xv.data_ptr()
    b.out_mode = pkg.B200_OUT_STORE
    d_y = torch.zeros(rows, dtype=torch.float32, device="cuda")
    b.d_out[0], b.n_out = d_y.data_ptr(), 1
    d_scr = torch.zeros(2 * 148 * 32, dtype=torch.float32, device="cuda")
    d_val = torch.zeros(1, dtype=torch.float32, device="cuda")
    d_idx = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    b.d_argmax_scratch = d_scr.data_ptr()
    b.d_argmax_val[0], b.d_argmax_idx[0], b.n_argmax_out = d_val.data_ptr(), d_idx.data_ptr(), 1
    b.d_ticket = d_ticket.data_ptr()
    for _ in range(2):                              # second run: the ticket must have been reset
        assert lib.b200_matvec(C.byref(b), None) == 0
        torch.cuda.synchronize()
        y = d_y.cpu().numpy()
        assert int(d_idx.item()) == int(np.argmax(y)) == min(best, (best + 1000) % rows)
        assert float(d_val.item()) == float(y.max())


@pytest.mark.parametrize("rows,cols,wtype", [(151936, 2560, 0), (262144, 1152, 1)])
def test_lm_head_shapes_with_argmax_across_all_blocks(lib, pkg, synth, rows, cols, wtype):
    """The two LM heads of the benchmarked architectures: the longest streams (413 MB Q8_0, 604 MB F16), ~1000+ rows per
    block, the device arg-max folded over every block."""
    w = weights(synth, rows, cols, 31)
    x = weights(synth, 1, cols, 91, std=1.0)[0]
    d_w, stride = pack(lib, pkg, w, wtype)
    d_scr = torch.zeros(2 * 1024 * 32, dtype=torch.float32, device="cuda")
    d_val = torch.zeros(1, dtype=torch.float32, device="cuda")
    d_idx = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    kw = dict(d_argmax_scratch=d_scr.data_ptr(), n_argmax_out=1, d_ticket=d_ticket.data_ptr())
    a_val, a_idx = (C.c_void_p * pkg.B200_MAX_PEERS)(), (C.c_void_p * pkg.B200_MAX_PEERS)()
    a_val[0], a_idx[0] = d_val.data_ptr(), d_idx.data_ptr()
    y = run_matvec(lib, pkg, d_w, stride, rows, cols, wtype, x, d_argmax_val=a_val, d_argmax_idx=a_idx, **kw)
    if wtype == pkg.B200_WT_Q8:
        ref = O.q8_matvec(O.q8_quantize(w), x, rows, cols)
    else:
        ref = O.f16_matvec(O.f16_bits(w), x)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()
    assert int(d_idx.item()) == int(np.argmax(y)) and float(d_val.item()) == float(y.max())


def test_matvec_wait_on_a_flag_nobody_raises_gives_up(lib, pkg, synth):
    """Bounded wait of the per-stage kernels: n_wait = 1 on a flag that stays 0. The launch must complete with
    *d_err == 1 (and the product computed from whatever the slots held); nothing hangs."""
    rows, cols = 64, 512
    w = weights(synth, rows, cols, 41)
    d_w, stride = pack(lib, pkg, w, pkg.B200_WT_Q8)
    d_flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    d_epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    d_err = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = weights(synth, 1, cols, 90, std=1.0)[0]
    run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x, d_wait_flags=d_flags.data_ptr(), n_wait=1,
               d_epoch=d_epoch.data_ptr(), epoch_mul=1, epoch_add=0, d_err=d_err.data_ptr(), spin_limit=1000)
    assert int(d_err.item()) == 1
    d_err.zero_()
    d_flags[0] = 1                                   # raised: the same launch goes through
    y = run_matvec(lib, pkg, d_w, stride, rows, cols, pkg.B200_WT_Q8, x, d_wait_flags=d_flags.data_ptr(), n_wait=1,
                   d_epoch=d_epoch.data_ptr(), epoch_mul=1, epoch_add=0, d_err=d_err.data_ptr(), spin_limit=1000)
    assert int(d_err.item()) == 0
    ref = O.q8_matvec(O.q8_quantize(w), x, rows, cols)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).max()


def test_matvec_rejects_bad_arguments(lib, pkg):
    a = pkg.MatvecArgs()
    assert lib.b200_matvec(C.byref(a), None) < 0
    assert lib.b200_matvec(None, None) < 0
    d = torch.zeros(64, dtype=torch.uint8, device="cuda")
    a.d_w, a.row_stride, a.rows, a.cols, a.wtype = d.data_ptr(), 48, 1, 40, pkg.B200_WT_Q8   # cols not a multiple of 32
    assert lib.b200_matvec(C.byref(a), None) < 0
    assert lib.b200_q8_pack(d.data_ptr(), 40, 1, 40, d.data_ptr(), 48, 0, 1, None) < 0


def attn_reference(qkv, qg, kg, theta, Kc, Vc, pos, n_q, n_kv, hd):
    """fp32 restatement of QK-norm + RoPE + attention over a cache that already holds rows < pos (binary16 values)."""
    def norm(v, g):
        return (g * v * (1.0 / np.sqrt(np.float32((v * v).sum(dtype=np.float32) / hd + 1e-6)))).astype(np.float32)

    def rope(v):
        half = hd // 2
        d = np.arange(half, dtype=np.float32)
        freq = (1.0 / np.power(np.float32(theta), (2 * d) / np.float32(hd))).astype(np.float32)
        ang = (np.float32(pos) * freq).astype(np.float32)
        c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        o = v.copy()
        o[:half] = v[:half] * c - v[half:] * s
        o[half:] = v[:half] * s + v[half:] * c
        return o
    q = qkv[:n_q * hd].reshape(n_q, hd)
    k = qkv[n_q * hd:(n_q + n_kv) * hd].reshape(n_kv, hd)
    v = qkv[(n_q + n_kv) * hd:].reshape(n_kv, hd)
    out = np.zeros((n_q, hd), dtype=np.float32)
    G = n_q // n_kv
    for h in range(n_kv):
        kn = rope(norm(k[h], kg)).astype(np.float16).astype(np.float32)
        Kc[h, pos] = kn
        Vc[h, pos] = v[h].astype(np.float16).astype(np.float32)
    for h in range(n_q):
        qn = rope(norm(q[h], qg))
        sc = (Kc[h // G, :pos + 1] @ qn) / np.float32(np.sqrt(hd))
        p = np.exp(sc - sc.max())
        p /= p.sum()
        out[h] = p @ Vc[h // G, :pos + 1]
    return out.reshape(-1)


@pytest.mark.parametrize("n_q,n_kv,hd,max_seq,n_split,positions", [
    (8, 2, 64, 64, 1, [0, 1, 17, 63]),
    (32, 8, 128, 1024, 18, [0, 5, 300, 1023]),
    (4, 1, 256, 512, 8, [0, 7, 511]),
    (4, 4, 128, 256, 4, [3, 255]),
])
def test_attention_vs_fp32_restatement(lib, pkg, synth, n_q, n_kv, hd, max_seq, n_split, positions):
    rng = np.random.default_rng(5)
    theta = 1e6
    qg = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kg = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    inv_freq = np.array([1.0 / np.power(np.float32(theta), np.float32(2 * d) / np.float32(hd)) for d in range(hd // 2)],
                        dtype=np.float32)
    Kc = (rng.standard_normal((n_kv, max_seq, hd)) * 0.5).astype(np.float16)
    Vc = (rng.standard_normal((n_kv, max_seq, hd)) * 0.5).astype(np.float16)
    d_k, d_v = dev(Kc), dev(Vc)
    Kf, Vf = Kc.astype(np.float32), Vc.astype(np.float32)
    d_qg, d_kg, d_if = dev(qg), dev(kg), dev(inv_freq)
    d_out = torch.zeros(n_q * hd, dtype=torch.float32, device="cuda")
    d_scr = torch.zeros(lib.b200_attn_scratch_floats(n_q, hd, n_split), dtype=torch.float32, device="cuda")
    d_tk = torch.zeros(n_kv, dtype=torch.int32, device="cuda")
    for pos in positions:
        qkv = rng.standard_normal((n_q + 2 * n_kv) * hd).astype(np.float32)
        d_qkv = dev(qkv)
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        a = pkg.AttnArgs(d_qkv.data_ptr(), d_qg.data_ptr(), d_kg.data_ptr(), d_if.data_ptr(), d_k.data_ptr(), d_v.data_ptr(),
                         d_out.data_ptr(), d_scr.data_ptr(), d_tk.data_ptr(), d_pos.data_ptr(),
                         n_q, n_kv, hd, max_seq, n_split, 1e-6, 0)
        assert lib.b200_attn_decode(C.byref(a), None) == 0
        torch.cuda.synchronize()
        ref = attn_reference(qkv, qg, kg, theta, Kf, Vf, pos, n_q, n_kv, hd)
        got = d_out.cpu().numpy()
        assert np.abs(got - ref).max() <= 2e-3 * np.abs(ref).max(), f"pos {pos}"
        # the new row must now be in the cache, in binary16
        # (norm and rotation are re-done here in numpy: allow one binary16 ulp on K; V is a plain rounding)
        assert np.allclose(d_k.cpu().numpy()[:, pos].astype(np.float32), Kf[:, pos], rtol=2e-3, atol=1e-6)
        assert np.array_equal(d_v.cpu().numpy()[:, pos].astype(np.float32), Vf[:, pos])
        assert int(d_tk.abs().sum().item()) == 0
