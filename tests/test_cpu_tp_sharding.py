"""Tensor-parallel partitioning, checked on CPU with two gloo ranks.

The engine cuts column-parallel matrices by rows and row-parallel matrices by input columns, every cut a
multiple of 32. This test redoes those cuts with the oracle on two processes: the Q8_0 bytes of a shard are
the corresponding slice of the unsharded quantisation, the sum of the row-parallel partial products over
ranks reproduces the full product, and the (value, index) exchange picks the same token as one argmax.
"""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def worker(rank, world, port, ret):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import _oracle as O
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(3)                       # same weights on every rank
    D, IS, V = 512, 1536, 4096
    w_up = (rng.standard_normal((IS, D)) * 0.02).astype(np.float32)       # column-parallel: rows are cut
    w_down = (rng.standard_normal((D, IS)) * 0.02).astype(np.float32)     # row-parallel: input columns are cut
    w_lm = (rng.standard_normal((V, D)) * 0.02).astype(np.float32)
    x = rng.standard_normal(D).astype(np.float32)
    ok = True
    # 1. shard bytes are slices of the unsharded quantisation
    full_up = O.q8_quantize(w_up).reshape(IS, D // 32, 34)
    il = IS // world
    mine_up = O.q8_quantize(w_up[rank * il:(rank + 1) * il]).reshape(il, D // 32, 34)
    ok &= np.array_equal(mine_up, full_up[rank * il:(rank + 1) * il])
    full_dn = O.q8_quantize(w_down).reshape(D, IS // 32, 34)
    mine_dn = O.q8_quantize(np.ascontiguousarray(w_down[:, rank * il:(rank + 1) * il])).reshape(D, il // 32, 34)
    ok &= np.array_equal(mine_dn, full_dn[:, rank * il // 32:(rank + 1) * il // 32])
    # 2. up (local rows) -> down (partial over local columns) -> all-reduce == unsharded result
    act_full = O.q8_matvec(full_up.reshape(-1), x, IS, D)
    act_mine = O.q8_matvec(mine_up.reshape(-1), x, il, D)
    ok &= np.array_equal(act_mine, act_full[rank * il:(rank + 1) * il])
    part = torch.from_numpy(O.q8_matvec(mine_dn.reshape(-1), act_mine, D, il))
    dist.all_reduce(part, op=dist.ReduceOp.SUM)
    ref = O.q8_matvec(full_dn.reshape(-1), act_full, D, IS)
    ok &= bool(np.abs(part.numpy() - ref).max() <= 1e-5 * np.abs(ref).max())
    # 3. vocabulary-sharded greedy pick: lowest index wins ties
    w_lm[V // 2 + 7] = w_lm[5]                            # a tie across the two shards
    logits = O.q8_matvec(O.q8_quantize(w_lm), x, V, D)
    logits[5] = logits[V // 2 + 7] = logits.max() + 1.0
    vl = V // world
    loc = logits[rank * vl:(rank + 1) * vl]
    pair = torch.tensor([float(loc.max()), float(rank * vl + int(np.argmax(loc)))], dtype=torch.float64)
    pairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(pairs, pair)
    best = min(pairs, key=lambda p: (-p[0].item(), p[1].item()))
    ok &= int(best[1].item()) == int(np.argmax(logits)) == 5
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(int(flag.item()))
    dist.destroy_process_group()


def test_two_rank_partitioning_matches_unsharded():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 1
