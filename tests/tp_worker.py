"""Worker of tests/test_gpu_tp.py: one rank of a tensor-parallel greedy decode, checked against the CPU oracle.

Launched by torch.distributed.run with one process per GPU. Every rank builds the same seeded model, keeps its
own shard (llmb200_set_tp), connects to its peers and generates; all ranks must return the oracle's tokens.
Architecture "wide-qwen3" is the two-layer cut of Qwen3-4B at full width (8 KV heads: shards over 2, 4 and 8
ranks) and is checked against tests/golden/wide_golden.npz, vectors the reference's own C code produced.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import __graft_entry__ as entry  # noqa: E402
import _oracle as O  # noqa: E402


def main():
    arch, use_fp16 = sys.argv[1], int(sys.argv[2])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry.load_package()
    L, S = pkg.lib(), pkg.synth()
    wide = arch == "wide-qwen3"
    golden = np.load(os.path.join(ROOT, "tests", "golden", "wide_golden.npz")) if wide else None
    sp = pkg.spec("qwen3-4b", gamma_jitter=0.1, n_layers=int(golden["layers"])) if wide else pkg.spec(arch, gamma_jitter=0.1)
    gemma = arch.endswith("gemma3")
    model = (S.llmb200_synth_gemma3 if gemma else S.llmb200_synth_qwen3)(C.byref(sp), 4)
    assert L.llmb200_set_tp(rank, world) == 0
    max_seq, P, G = (int(golden["max_seq"]) if wide else 96), 16, 32
    st = (L.inference_state_create_gemma3 if gemma else L.inference_state_create)(model, max_seq, use_fp16)
    assert st, "state create failed"
    h = (C.c_ubyte * pkg.LLMB200_HANDLE_BYTES)()
    assert L.llmb200_state_comm_handle(st, h) == 0
    mine = torch.tensor(list(h), dtype=torch.uint8, device="cuda")
    allh = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    assert L.llmb200_state_connect(st, bytes(torch.cat(allh).cpu().numpy().tobytes()), world) == 0
    dist.barrier()
    L.llmb200_state_set_eos(st, None, 0)
    prompt = np.zeros(P, dtype=np.uint32)
    S.llmb200_synth_tokens(prompt.ctypes.data, P, 4321, sp.vocab_size)
    out = np.zeros(G, dtype=np.uint32)
    for _ in range(2):                                  # twice: the second request reuses slots, flags and epochs
        n = L.inference_generate(st, prompt.ctypes.data_as(pkg.c_u32_p), P, out.ctypes.data_as(pkg.c_u32_p), G)
        assert n == G and L.llmb200_state_error(st) == 0, (n, L.llmb200_state_error(st))
    # logits through inference_forward_token: every rank must hold the full, identical vector
    L.inference_state_reset(st)
    lg = None
    for t in prompt[:4]:
        p = L.inference_forward_token(st, int(t))
        assert p
        lg = np.ctypeslib.as_array(p, shape=(sp.vocab_size,)).copy()
    dist.barrier()
    if wide:
        # reference vectors: tokens of the greedy decode; the fourth prompt position's logits are not in the file,
        # so the logits check runs along the generated path instead (sampled every `stride`-th logit)
        ref = golden["qwen3_tokens"]
        assert list(prompt) == list(golden["qwen3_prompt"])
        L.inference_state_reset(st)
        seq = np.concatenate([prompt, ref[:1]])
        for t in seq:
            p = L.inference_forward_token(st, int(t))
            lg = np.ctypeslib.as_array(p, shape=(sp.vocab_size,)).copy()
        stride = int(golden["stride"])
        err = np.abs(lg[::stride] - golden["qwen3_logit_sample"][1]).max() / golden["qwen3_logit_absmax"][1]
        ok = list(out) == list(ref) and err <= 1e-2
        ref_lg = lg if ok else lg + 1.0
    else:
        om = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, max_seq, vocab=sp.vocab_size)
        ref, _ = O.generate(om, prompt, G)
        ref_lg = None
        om2 = (O.model_gemma3 if gemma else O.model_qwen3)(model, use_fp16, max_seq, vocab=sp.vocab_size)
        for i, t in enumerate(prompt[:4]):
            ref_lg = O.forward_token(om2, t, i)
        ok = list(out) == list(ref) and np.abs(lg - ref_lg).max() <= 1e-2 * np.abs(ref_lg).max()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_RESULT", "ok" if int(flag.item()) == 1 else "MISMATCH", list(out[:8]), list(ref[:8]),
              float(np.abs(lg - ref_lg).max() / np.abs(ref_lg).max()), flush=True)
    L.inference_state_free(st)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
