"""Tensor-parallel decode on 2, 4 and 8 GPUs (as far as the box has them): same greedy tokens as the checker on every rank."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("arch,use_fp16,world", [("tiny-qwen3", 0, 2), ("tiny-qwen3", 1, 2), ("wide-qwen3", 0, 2),
                                                 ("wide-qwen3", 0, 4), ("wide-qwen3", 0, 8)])
def test_tp_matches_oracle(arch, use_fp16, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
                        "--master-port", "29731", os.path.join(HERE, "tp_worker.py"), arch, str(use_fp16)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "TP_RESULT ok" in r.stdout, r.stdout[-3000:]
