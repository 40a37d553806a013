"""Data-parallel LoRA-SFT, checked on CPU with two gloo ranks and the restatement.

The ranks hold the same frozen base and the same LoRA, take different sequences, all-reduce (mean) the
flat LoRA gradient vector and then run the same clip + AdamW: the result must equal one process stepping
on all sequences at once, and the ranks must end bit-identical (no weight broadcast is needed).
This is the exchange bench.py performs with NCCL on the engine's gradient vector.
"""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
RANK, ALPHA, N, PER_RANK = 4, 8.0, 10, 2


def flat(grads, keys):
    return np.concatenate([g[k].ravel() for g in grads for k in keys]).astype(np.float32)


def unflat(vec, like, keys):
    out, o = [], 0
    for g in like:
        d = {}
        for k in keys:
            n = g[k].size
            d[k] = vec[o:o + n].reshape(g[k].shape).copy()
            o += n
        out.append(d)
    return out


def worker(rank, world, port, ret):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import _sft_common as sc
    o = sc.sft_oracle
    pkg = sc.package()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = sc.SMALL
    ow = sc.oracle_model(cfg, sc.make_weights(pkg, cfg))
    toks = sc.tokens(pkg, world * PER_RANK * (N + 1), 4321, cfg["vocab_size"]).reshape(world * PER_RANK, N + 1)
    mine = toks[rank * PER_RANK:(rank + 1) * PER_RANK]
    lora = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
    ok = True
    for step in range(2):
        loss, grads, _ = o.loss_and_grads(ow, lora, mine[:, :-1], mine[:, 1:])
        vec = torch.from_numpy(flat(grads, o.KEYS))
        dist.all_reduce(vec, op=dist.ReduceOp.SUM)
        vec /= world
        lt = torch.tensor([loss], dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        lora.step_count += 1
        clipped, norm = o.clip_grad_norm(unflat(vec.numpy(), grads, o.KEYS), 1.0)
        o.adamw(lora, clipped, 1e-3)
        if rank == 0:
            # the same step on one process over all sequences
            if step == 0:
                single = o.LoRA(sc.make_lora(pkg, cfg, RANK, b_std=0.02), RANK, ALPHA)
            want_loss, want_g, want_norm = o.train_step(ow, single, toks[:, :-1], toks[:, 1:], 1e-3)
            ok &= abs(lt.item() / world - want_loss) < 1e-5
            ok &= abs(norm - want_norm) < 1e-5 * want_norm
            for L in range(cfg["n_layers"]):
                for k in o.KEYS:
                    ok &= sc.rel_err(lora.p[L][k], single.p[L][k]) < 1e-5
    # every rank holds the same weights, bit for bit
    mine_p = torch.from_numpy(flat(lora.p, o.KEYS))
    both = [torch.zeros_like(mine_p) for _ in range(world)]
    dist.all_gather(both, mine_p)
    ok &= all(torch.equal(both[0], b) for b in both)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(int(flag.item()))
    dist.destroy_process_group()


def test_two_rank_gradient_mean_equals_one_batch():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 31000 + os.getpid() % 2000
    procs = [ctx.Process(target=worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    assert ret.get(timeout=5) == 1
