"""The benchmark's command line without a GPU: the reference arm (the CPU restatement timed on
the host's cores) prints one JSON line with the keys the harness reads, and the product arm
refuses loudly instead of falling back to a CPU path."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="the CPU-only behaviour of bench.py")


def _run(*args: str, timeout: int = 300) -> subprocess.CompletedProcess[str]:
    env = dict(os.environ, OMP_NUM_THREADS=os.environ.get("OMP_NUM_THREADS", "4"))
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=ROOT, env=env)


@pytest.mark.parametrize("workload, metric, unit", [("c2", "bf16 GEMM TFLOP/s", "TFLOP/s"), ("c4", "softmax/norm HBM GB/s", "GB/s")])
def test_reference_arm_prints_the_contract_line(workload: str, metric: str, unit: str) -> None:
    done = _run("--impl", "reference", "--workload", workload, "--steps", "1", "--warmup", "1")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == metric and line["unit"] == unit
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 1
    assert line["higher_is_better"] is True and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert isinstance(line["config"]["workload"], str) and "model" not in line["config"]
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["sample"] and baseline["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == unit
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_product_arm_needs_a_gpu_and_says_so() -> None:
    done = _run("--steps", "1", "--warmup", "1", timeout=120)
    assert done.returncode != 0
    assert "needs a CUDA device" in (done.stderr + done.stdout)
    assert not [line for line in done.stdout.splitlines() if line.startswith("{")]  # no figure from a CPU path
