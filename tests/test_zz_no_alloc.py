"""b200_attn_decode_static: the attention launch that allocates nothing.

Some callers of this library cannot allocate device memory at the point where they need attention -- their
memory was handed out in full at start-up, or a cudaMalloc would stall the whole device in the middle of
a latency-critical loop. For them the split-sequence scratch lives inside the library. This test calls that
entry point through the C ABI, twice in a row (the built-in arrays keep the previous call's contents), and
checks each result against b200_attn_decode with caller-provided scratch (the two run the same kernel, so
the results must be identical) and against the fp32 restatement of the attention the kernel tests use; the
bar is the attention tests' 2e-3 of max|out|.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_matches_caller_scratch_twice(lib, pkg):
    n_q, n_kv, hd, max_seq, n_split = 32, 8, 128, 1024, 18
    rng = np.random.default_rng(11)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    d_qg = dev((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32))
    d_kg = dev((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32))
    d_if = dev(np.array([1.0 / 1e6 ** (2 * d / hd) for d in range(hd // 2)], dtype=np.float32))
    kc = (rng.standard_normal((n_kv, max_seq, hd)) * 0.5).astype(np.float16)
    vc = (rng.standard_normal((n_kv, max_seq, hd)) * 0.5).astype(np.float16)
    d_scr = torch.zeros(lib.b200_attn_scratch_floats(n_q, hd, n_split), dtype=torch.float32, device="cuda")
    d_tk = torch.zeros(n_kv, dtype=torch.int32, device="cuda")
    for pos in (700, 33):                                   # two calls in a row, different lengths
        qkv = dev(rng.standard_normal((n_q + 2 * n_kv) * hd).astype(np.float32))
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        outs = []
        for static in (False, True):
            d_k, d_v = dev(kc), dev(vc)                     # each variant writes row `pos` of its own copy
            d_out = torch.zeros(n_q * hd, dtype=torch.float32, device="cuda")
            a = pkg.AttnArgs(qkv.data_ptr(), d_qg.data_ptr(), d_kg.data_ptr(), d_if.data_ptr(), d_k.data_ptr(), d_v.data_ptr(),
                             d_out.data_ptr(), None if static else d_scr.data_ptr(), None if static else d_tk.data_ptr(),
                             d_pos.data_ptr(), n_q, n_kv, hd, max_seq, n_split, 1e-6, 0)
            fn = lib.b200_attn_decode_static if static else lib.b200_attn_decode
            assert fn(C.byref(a), None) == 0
            torch.cuda.synchronize()
            outs.append((d_out.cpu().numpy(), d_k.cpu().numpy()[:, pos].copy(), d_v.cpu().numpy()[:, pos].copy()))
        (o0, k0, v0), (o1, k1, v1) = outs
        assert np.isfinite(o1).all() and np.abs(o1).max() > 0
        assert np.abs(o1 - o0).max() <= 2e-3 * np.abs(o0).max()
        assert np.array_equal(k0, k1) and np.array_equal(v0, v1)
        # and directly against the restatement: cache rows below pos as binary16 values, row pos from q/k/v
        from test_gpu_kernels import attn_reference
        want = attn_reference(qkv.cpu().numpy(), d_qg.cpu().numpy(), d_kg.cpu().numpy(), 1e6, kc.astype(np.float32),
                              vc.astype(np.float32), pos, n_q, n_kv, hd)
        assert np.abs(o1 - want).max() <= 2e-3 * np.abs(want).max()


def test_static_scratch_refuses_oversized_requests(lib, pkg):
    a = pkg.AttnArgs()
    a.n_q, a.n_kv, a.hd, a.max_seq, a.n_split = 64, 8, 256, 4096, 64        # 64*64*258 floats > 2^18
    assert lib.b200_attn_decode_static(C.byref(a), None) == -2              # B200_E_TOOLARGE
    a.n_q, a.n_kv, a.n_split = 128, 128, 1                                   # too many KV heads
    assert lib.b200_attn_decode_static(C.byref(a), None) == -2
    # the batched form needs scratch and tickets per item: refused, nothing is launched
    a.n_q, a.n_kv, a.hd, a.n_split, a.n_items = 32, 8, 128, 18, 2
    assert lib.b200_attn_decode_static(C.byref(a), None) == -2
    assert lib.b200_attn_decode_static(None, None) == -1
