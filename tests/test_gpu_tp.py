"""Tensor-parallel decode on 2 GPUs (when the box has them): same greedy tokens as the CPU oracle on every rank."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("arch,use_fp16", [("tiny-qwen3", 0), ("tiny-qwen3", 1)])
def test_tp2_matches_oracle(arch, use_fp16):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29731", os.path.join(HERE, "tp_worker.py"), arch, str(use_fp16)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "TP_RESULT ok" in r.stdout, r.stdout[-3000:]
