"""The benchmark's contract on its small workloads: exactly one JSON line on stdout with the agreed keys.

Every workload family runs once (decode Q8_0, Gemma3 binary16 decode, LoRA SFT step, batched binary16
decode) so that a change that breaks a family's timing path or its reporting shows up as a test failure.
"""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

KEYS = ["metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "roofline", "clocks"]


def run_bench(*extra):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "1", "--no-cpu-baseline", *extra]
    r = subprocess.run(cmd, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, f"stdout must hold one JSON line, got {len(lines)}: {r.stdout[:500]}"
    return json.loads(lines[0])


@pytest.mark.gpu
@pytest.mark.parametrize("workload,metric", [
    ("tiny-qwen3-q8", "decode_tokens_per_s"),
    ("tiny-gemma3-f16", "decode_tokens_per_s"),
    ("tiny-qwen3-sft-lora", "sft_tokens_per_s"),
    ("tiny-qwen3-f16-batch8", "batched_decode_tokens_per_s"),
])
def test_one_json_line_with_the_contract_keys(workload, metric):
    d = run_bench("--workload", workload)
    for k in KEYS:
        assert k in d, f"{workload}: key {k} missing"
    assert d["metric"] == metric and d["n_gpus"] == 1 and d["data"] == "synthetic"
    assert d["value"] > 0 and d["e2e"]["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0
    assert d["gpu_launches"] > 0, "the timed region must launch this library's kernels"
    assert d["roofline"]["bound"] in ("hbm", "tensor") and d["roofline"]["frac"] > 0
    assert "workload" in d["config"] and "model" not in d["config"]


@pytest.mark.gpu
def test_reference_arm_line():
    d = run_bench("--workload", "tiny-qwen3-q8", "--impl", "reference")
    assert d["impl"] == "reference" and d["metric"] == "decode_tokens_per_s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
