"""Host logic of the whole-token kernel, no GPU: b200_token_plan's geometry and the row partition that its
producer and consumers both walk (replayed on the host by b200_token_chunks).

Properties checked for every benchmarked architecture, both weight types and every tensor-parallel
degree the engine accepts: each row of each stage belongs to exactly one chunk of exactly one block;
chunks fit a ring slot and hold the same number of rows for every consumer group; (gate, up) pairs are
never split; blocks differ by at most one row unit; emission windows never hold more warp partials than
the shared-memory buffer.
"""
import ctypes as C

import numpy as np
import pytest

SLOT_BYTES = 21760
PART_FLOATS = 1024
CONSUMERS = 640

ARCHS = {
    "tiny-qwen3": dict(D=512, Hq=8, Hkv=2, hd=64, IS=1536, V=4096, L=4),
    "qwen3-4b": dict(D=2560, Hq=32, Hkv=8, hd=128, IS=9728, V=151936, L=36),
    "gemma3-1b": dict(D=1152, Hq=4, Hkv=1, hd=256, IS=6912, V=262144, L=26),
    "tiny-gemma3": dict(D=384, Hq=4, Hkv=1, hd=256, IS=1152, V=2048, L=7),
}


def planned(lib, pkg, arch, wtype, tp, n_blocks=148, max_seq=4096):
    a = pkg.TokenArgs()
    d = ARCHS[arch]
    hq, hkv, isz, v = d["Hq"] // tp, d["Hkv"] // tp, d["IS"] // tp, d["V"] // tp
    shapes = [((hq + 2 * hkv) * d["hd"], d["D"], 0), (d["D"], hq * d["hd"], 0), (2 * isz, d["D"], 1),
              (d["D"], isz, 0), (v, d["D"], 0)]
    for k, (rows, cols, glu) in enumerate(shapes):
        a.g[k].rows, a.g[k].cols, a.g[k].glu = rows, cols, glu
        a.g[k].row_stride = lib.b200_packed_row_stride(wtype, cols)
    a.n_layers, a.wtype, a.d_model = d["L"], wtype, d["D"]
    a.n_q, a.n_kv, a.hd, a.max_seq = hq, hkv, d["hd"], max_seq
    a.n_ranks, a.rank = tp, 0
    rc = lib.b200_token_plan(C.byref(a), n_blocks)
    return rc, a


CASES = [("tiny-qwen3", 1), ("tiny-qwen3", 2), ("qwen3-4b", 1), ("qwen3-4b", 2), ("qwen3-4b", 4), ("qwen3-4b", 8),
         ("gemma3-1b", 1), ("tiny-gemma3", 1)]


@pytest.mark.parametrize("arch,tp", CASES)
@pytest.mark.parametrize("wtype", [0, 1])
def test_partition_covers_every_row_once(lib, pkg, arch, tp, wtype):
    rc, a = planned(lib, pkg, arch, wtype, tp)
    assert rc == 0, f"plan refused {arch} tp{tp} wtype{wtype}: {rc}"
    assert a.n_blocks == 148 and 0 < a.smem_bytes <= 232448
    assert a.n_kv * a.n_split <= a.n_blocks
    buf = (C.c_int * (3 * 4096))()
    for kind in range(pkg.B200_ST_KINDS):
        g = a.g[kind]
        ralign = 2 if g.glu else 1
        assert g.T % 32 == 0 and g.T * g.NG <= CONSUMERS and g.spt in (1, 2) and g.rg in (1, 2, 4, 8)
        assert g.rb == g.rg * g.NG and g.rb * g.row_stride <= SLOT_BYTES and g.rg % ralign == 0 and g.pw % g.rb == 0
        elems = 16 if wtype == 0 else 8
        assert g.T * g.spt * elems >= g.cols                      # every column has an owner
        assert g.pw * ((g.T // 32) | 1) <= PART_FLOATS
        seen = np.zeros(g.rows, dtype=np.int32)
        per_block = []
        for b in range(a.n_blocks):
            n = lib.b200_token_chunks(C.byref(a), kind, b, buf, 4096)
            assert 0 <= n <= 4096
            rows_b = 0
            for i in range(n):
                r0, nr, win = buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]
                assert 0 < nr <= g.rb and win >= 0
                assert r0 % ralign == 0 and nr % ralign == 0          # pairs stay together
                seen[r0:r0 + nr] += 1
                rows_b += nr
            per_block.append(rows_b)
        assert (seen == 1).all(), f"kind {kind}: rows covered {seen.min()}..{seen.max()} times"
        assert max(per_block) - min(per_block) <= ralign


def test_plan_refuses_what_the_kernel_cannot_run(lib, pkg):
    rc, a = planned(lib, pkg, "qwen3-4b", 0, 1)
    assert rc == 0
    # a row longer than a ring slot
    b = pkg.TokenArgs.from_buffer_copy(a)
    b.g[3].cols = 32768
    b.g[3].row_stride = lib.b200_packed_row_stride(0, 32768)
    b.g[2].rows = 2 * 32768
    assert lib.b200_token_plan(C.byref(b), 148) == -2
    # head grouping outside 1/2/4/8
    b = pkg.TokenArgs.from_buffer_copy(a)
    b.n_q, b.n_kv = 24, 8
    assert lib.b200_token_plan(C.byref(b), 148) == -1
    # more KV heads than blocks
    b = pkg.TokenArgs.from_buffer_copy(a)
    assert lib.b200_token_plan(C.byref(b), 4) == -2
    # launching without a plan is refused before anything touches the GPU
    c = pkg.TokenArgs()
    assert lib.b200_decode_token(C.byref(c), None) != 0


def test_token_kernel_has_no_register_spills():
    """The whole-token kernel keeps ~220 KB of shared memory per block, which leaves the L1 that backs the
    stack a few KB: a spilled register costs a round trip to L2 (about a microsecond) every time it is
    touched, and ptxas sits at the 80-register cap of a 672-thread block. The instantiations the engine
    launches (no trace) must compile without spill code."""
    import os
    import re
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "llm.metal_b200", "csrc", "decode_token.cu")
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xptxas", "-v",
                        "-c", src, "-o", os.devnull], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:]
    lines = r.stdout.splitlines()
    seen = 0
    for i, line in enumerate(lines):
        m = re.search(r"Function properties for (\S*decode_token_kernelILi(\d)ELb(\d)ELb(\d)E\S*)", line)
        if not m:
            continue
        trace = m.group(3) == "1"                                                  # <WT, TRACE, MULTI>
        spill = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", lines[i + 1])
        assert spill, lines[i + 1]
        if not trace:
            seen += 1
            assert spill.group(1) == "0" and spill.group(2) == "0", (m.group(1), lines[i + 1])
    assert seen == 4          # Q8_0 / F16 x one GPU / several GPUs
