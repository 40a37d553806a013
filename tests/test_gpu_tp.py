"""Tensor-parallel decode on 2, 4 and 8 GPUs (as far as the box has them): same greedy tokens as the checker on
every rank, launched as one process per GPU and as one process with one host thread per GPU (LLMB200_TP=k)."""
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


@pytest.mark.parametrize("arch,use_fp16,world", [("tiny-qwen3", 0, 2), ("wide-qwen3", 0, 2),
                                                 ("wide-qwen3", 0, 4), ("wide-qwen3", 0, 8)])
def test_single_process_tp_through_the_reference_calls(arch, use_fp16, world):
    """LLMB200_TP=k: inference_state_create / inference_generate / inference_forward_token, called as on one
    GPU, run k-way tensor parallel inside the calling process."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, LLMB200_TP=str(world))
    r = subprocess.run([sys.executable, os.path.join(HERE, "tp_single_process_worker.py"), arch, str(use_fp16)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=600)
    assert r.returncode == 0 and f"TP_SINGLE {world} ok" in r.stdout, r.stdout[-3000:]


def test_drop_in_program_with_single_process_tp():
    """The C program built against the reference's headers, unchanged, on two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    exe = os.path.join(os.path.dirname(HERE), "tests", "c_api", "_bin", "drop_in")
    if not os.path.exists(exe):
        pytest.skip("tests/c_api/_bin/drop_in was not built (reference tree absent at build time)")
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600,
                       env=dict(os.environ, LLMB200_TP="2"))
    assert r.returncode == 0 and "DROP_IN ok" in r.stdout and "2-way tensor parallel" in r.stdout, r.stdout[-3000:]
