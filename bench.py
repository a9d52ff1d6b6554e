"""Benchmark of the hot path: the fused bf16 linear  y = GELU(x @ W^T + b), with the
other four configurations of the baseline timed beside it in the same line.

    python bench.py --gpus N --steps K --warmup W [--workload c2|c4|c1|c3|c5|attn|c2n|c2n_fused|kernels]
                    [--only-main] [--impl reference] [--row-lengths N,N,...]

A step is one pass of the hot path over one batch of synthetic input. The default
workload is the configuration the headline metric is quoted on: x [8192,4096],
W [4096,4096], b [4096] bf16, f32 accumulation, GELU, bf16 output. With N GPUs each
rank runs its own batch of 8192 rows (rows are independent: no collective on the
data path) and `value` is the whole-job TFLOP/s over the slowest rank's time.

One JSON line is printed by rank 0. Besides the driver's keys it carries
  roofline      algorithmic FLOPs or bytes over the CUDA-event time of the dominant
                kernel, against the measured peak
  cpu_baseline  the CPU restatement of the reference's operator timed on this host's
                cores on a bounded sample
  e2e           the same metric through the public operator with host buffers: pinned
                host -> device copy of x, the kernel, device -> host copy of y, every step
  parity_*      the result of one step on the same seeded tensors against the CPU
                oracle, on samples, outside the timed region
  sustained     the same step back to back for two seconds (the K-step figure of a
                short run is a burst figure), against the measured sustained peak
  linear_entry  the same step entered through linear(x, layer, F.gelu, cache)
  configs       one block per other configuration (C1, C3, C4, C5), each timed for a
                few hundred milliseconds of device time by an inner repeat count that
                does not depend on --steps, with its own roofline, parity and clocks

`--impl reference` times the CPU implementation of the path instead (the
reference's own pipeline needs Helion + an MLIR toolchain, which are not
installed, so the restatement under oracle/ stands in for it).
"""

from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path
import statistics
import subprocess
import sys
import threading
import time

ROOT = Path(__file__).resolve().parent
for _path in (ROOT, ROOT / "helion-mlir-xsmm_b200"):
    if str(_path) not in sys.path:
        sys.path.insert(0, str(_path))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 * 1024 * 1024
BLOCK_TARGET_MS = 300.0  # device time each configuration block is timed for
SUSTAINED_SECONDS = 2.0


def measured_peaks() -> tuple[dict[str, float], str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return {k: float(data[k]) for k in FALLBACK_PEAKS if k in data} | {}, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the whole run; a timed
    region asks for the samples that arrived inside its window."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[tuple[float, str]] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return

        def pump() -> None:
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.lines.append((time.monotonic(), line.strip()))

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=5)

    def window(self, t0: float, t1: float) -> dict[str, object]:
        """Clocks seen between ``t0`` and ``t1`` (time.monotonic); a sample is the state at the
        moment nvidia-smi printed it, so the window is widened by one period at its end."""
        clocks, power, max_clock, reasons = [], [], None, set()
        for stamp, line in list(self.lines):
            if stamp < t0 or stamp > t1 + 0.1:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, value in zip(self.NAMES, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "power_w": max(power) if power else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


# --------------------------------------------------------------------------- workloads


class Workload:
    """One benchmark configuration: device buffers, the step, its algorithmic work,
    the parity check of one step, and the CPU restatement of the same step."""

    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "tensor"
    scaling = "weak"  # per-GPU work is fixed as N grows ("strong": total work is fixed)
    collective = False  # the step holds a collective: every rank must run every call of it
    traffic: float | None = None  # DRAM bytes per launch of the dominant kernel (ncu, profiles/)

    def setup(self, device: torch.device, rank: int) -> None:
        raise NotImplementedError

    def step(self, index: int) -> torch.Tensor:
        raise NotImplementedError

    def e2e_step(self, index: int) -> tuple[int, int] | None:
        """One step through host buffers; returns (h2d bytes, d2h bytes), or None when the
        workload has no host-buffer leg."""
        return None

    def work_per_step(self) -> float:
        """FLOPs (tensor-bound) or bytes (HBM-bound) of one step on one GPU."""
        raise NotImplementedError

    def config(self) -> dict[str, object]:
        raise NotImplementedError

    def parity(self) -> dict[str, object]:
        """One step on the seeded tensors against the CPU oracle (sampled)."""
        raise NotImplementedError

    def cpu_setup(self) -> str:
        """Host tensors of a bounded sample of the workload; returns its description."""
        raise NotImplementedError

    def cpu_step(self) -> float:
        """Runs the CPU restatement on the sample; returns the work done (FLOPs or bytes)."""
        raise NotImplementedError

    def launches_per_step(self) -> int | None:
        """Kernels per step when they do not pass the library's launch counter (graph replays)."""
        return None

    def teardown(self) -> None:
        """Gives back what setup() took beyond tensors (collective where setup() was)."""


def _rotating(count: int, make):
    return [make(i) for i in range(count)]


class LinearGelu(Workload):
    """C2: y = GELU(x @ W^T + b), bf16, f32 accumulate."""

    name, metric, unit, dtype, bound = "c2_linear_gelu_8192x4096x4096", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    M, N, K, SETS = 8192, 4096, 4096, 3
    traffic = 153.4e6  # gemm_umma_bf16_kernel<2>: 107.0 MB read + 46.4 MB written (algorithmic 167.8 MB)
    via_linear = False

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops
        from oracle import inputs

        self.ops, self.device = ops, device
        data = inputs.c2_linear(self.M, self.N, self.K, rank=rank)
        self.host = data
        self.w, self.b = data["w"].to(device), data["b"].to(device)
        # Rotating input sets: 3 x (x + y) = 403 MB, beyond the 126 MB L2.
        self.xs = _rotating(self.SETS, lambda i: data["x"].roll(i, 0).to(device))
        self.x_pinned = data["x"].pin_memory()
        self.y_pinned = torch.empty(self.M, self.N, dtype=torch.bfloat16).pin_memory()
        self.layer = torch.nn.Linear(self.K, self.N, dtype=torch.bfloat16, device=device)
        with torch.no_grad():
            self.layer.weight.copy_(self.w)
            self.layer.bias.copy_(self.b)
        self.cache = None

    def step(self, index: int) -> torch.Tensor:
        if self.via_linear:
            return self.linear_step(index)
        return self.ops.matmul(self.xs[index % self.SETS], self.w, trans_b=True, bias=self.b, epilogue=F.gelu)

    def linear_step(self, index: int) -> torch.Tensor:
        """The reference's stock entry for this configuration: linear() with the weight cache."""
        y, self.cache = self.ops.linear(self.xs[index % self.SETS], self.layer, F.gelu, self.cache)
        return y

    def e2e_step(self, index: int) -> tuple[int, int]:
        # Host rows in, host rows out (b200_gemm_host_rows): copy-in, GEMM and copy-out
        # of neighbouring row chunks overlap on three streams.
        self.ops.matmul_host(self.x_pinned, self.w, self.y_pinned, trans_b=True, bias=self.b, epilogue=F.gelu)
        return self.x_pinned.numel() * 2, self.y_pinned.numel() * 2

    def work_per_step(self) -> float:
        return 2.0 * self.M * self.N * self.K

    def config(self) -> dict[str, object]:
        return {
            "workload": self.name, "m_per_gpu": self.M, "n": self.N, "k": self.K, "epilogue": "bias+gelu_erf",
            "accumulate": "f32", "out": "bf16", "sharding": "rows (M) per GPU, no collective",
            "entry": "linear(x, layer, F.gelu, cache)" if self.via_linear else "matmul(x, W, trans_b=True, bias=b, epilogue=F.gelu)",
            "l2": f"inputs rotated over {self.SETS} buffer sets (403 MB) > 126 MB L2",
        }

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        rows = sampled.rows_of_interest(self.M, extra=4)
        y = self.step(0)
        return sampled.c2_rows(self.host["x"], self.host["w"], self.host["b"], y[rows.to(self.device)], rows)

    CPU_ROWS = 1024

    def cpu_setup(self) -> str:
        from oracle import inputs

        data = getattr(self, "host", None) or inputs.c2_linear(self.CPU_ROWS, self.N, self.K)
        self.cpu = (data["x"][: self.CPU_ROWS].contiguous(), data["w"], data["b"])
        return f"{self.CPU_ROWS} of {self.M} rows per step, f32-accumulate torch CPU restatement"

    def cpu_step(self) -> float:
        from oracle import ops as ref

        x, w, b = self.cpu
        ref.matmul(x, w, trans_b=True, bias=b, epilogue=F.gelu, acc_dtype=torch.float32)
        return 2.0 * x.shape[0] * self.N * self.K


class RowNorms(Workload):
    """C4: softmax, layer_norm and rms_norm of x [32768, 4096], f32 and bf16 (six kernels per step)."""

    name, metric, unit, dtype, bound = "c4_softmax_layernorm_rmsnorm_32768x4096", "softmax/norm HBM GB/s", "GB/s", "f32+bf16", "hbm"
    M, N = 32768, 4096
    traffic = 860.1e6  # f32 softmax, scaled x4 from the 8192-row capture (134.26 MB read + 80.77 MB written)

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops
        from oracle import inputs

        self.ops, self.device = ops, device
        data = inputs.c4_rows(self.M, self.N, torch.float32, rank=rank)
        self.host = data
        self.x32 = data["x"].to(device)
        self.x16 = self.x32.bfloat16()
        self.g32, self.b32 = data["gamma"].to(device), data["beta"].to(device)
        self.g16, self.b16 = self.g32.bfloat16(), self.b32.bfloat16()
        self.x_pinned = data["x"].pin_memory()
        self.y_pinned = torch.empty(self.M, self.N).pin_memory()

    def kernels(self):
        ops = self.ops
        return [
            ("softmax_f32", 4, lambda: ops.softmax(self.x32)),
            ("layer_norm_f32", 4, lambda: ops.layer_norm(self.x32, self.g32, self.b32, 1e-5)),
            ("rms_norm_f32", 4, lambda: ops.rms_norm(self.x32, self.g32, 1e-5)),
            ("softmax_bf16", 2, lambda: ops.softmax(self.x16)),
            ("layer_norm_bf16", 2, lambda: ops.layer_norm(self.x16, self.g16, self.b16, 1e-5)),
            ("rms_norm_bf16", 2, lambda: ops.rms_norm(self.x16, self.g16, 1e-5)),
        ]

    def step(self, index: int) -> torch.Tensor:
        out = None
        for _, _, run in self.kernels():
            out = run()
        return out

    def e2e_step(self, index: int) -> tuple[int, int]:
        self.ops.stream_rows(self.ops.softmax, self.x_pinned, self.y_pinned)
        return self.x_pinned.numel() * 4, self.y_pinned.numel() * 4

    def work_per_step(self) -> float:
        return 3 * (2.0 * self.M * self.N * 4) + 3 * (2.0 * self.M * self.N * 2)

    def config(self) -> dict[str, object]:
        return {
            "workload": self.name, "rows_per_gpu": self.M, "n": self.N,
            "kernels_per_step": "softmax, layer_norm, rms_norm in f32 then bf16",
            "sharding": "rows per GPU, no collective",
            "l2": "each kernel streams 0.5-1 GiB, beyond the 126 MB L2",
            "e2e": "softmax f32 only",
        }

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        ops = self.ops
        rows = sampled.rows_of_interest(self.M, tile_rows=148, group_tiles=64, extra=24)
        pick = rows.to(self.device)
        reports = []
        for x, g, b in ((self.x32, self.g32, self.b32), (self.x16, self.g16, self.b16)):
            soft = ops.softmax(x)
            run = {
                "softmax": soft[pick],
                "layer_norm": ops.layer_norm(x, g, b, 1e-5)[pick],
                "rms_norm": ops.rms_norm(x, g, 1e-5)[pick],
                "chained": ops.layer_norm(soft, g, b, 1e-5)[pick],
            }
            del soft
            reports.append(sampled.c4_rows(x[pick].cpu(), g.cpu(), b.cpu(), run, self.M))
        return sampled.worst(reports)

    CPU_ROWS = 4096

    def cpu_setup(self) -> str:
        from oracle import inputs

        data = getattr(self, "host", None) or inputs.c4_rows(self.CPU_ROWS, self.N)
        x = data["x"][: self.CPU_ROWS].contiguous()
        g, b = data["gamma"], data["beta"]
        self.cpu = ((x, g, b), (x.bfloat16(), g.bfloat16(), b.bfloat16()))
        return f"{self.CPU_ROWS} of {self.M} rows per step, six kernels, f32-compute torch CPU restatement"

    def cpu_step(self) -> float:
        for t, gg, bb in self.cpu:
            tf = t.float()
            torch.softmax(tf, -1).to(t.dtype)
            F.layer_norm(tf, (self.N,), gg.float(), bb.float(), 1e-5).to(t.dtype)
            F.rms_norm(tf, (self.N,), gg.float(), 1e-5).to(t.dtype)
        rows = self.cpu[0][0].shape[0]
        return 3 * 2.0 * rows * self.N * 4 + 3 * 2.0 * rows * self.N * 2


class F32Matmul(Workload):
    """C1: f32 C = A @ B, 1024^3, block_sizes=[64,64,64]."""

    name, metric, unit, dtype, bound = "c1_f32_matmul_1024", "f32 GEMM TFLOP/s", "TFLOP/s", "f32", "tensor"
    SIZE, SETS = 1024, 12

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops
        from oracle import inputs

        self.ops, self.device = ops, device
        data = inputs.c1_f32_matmul(self.SIZE)
        self.host = data
        # 12 rotating (A, B) pairs = 101 MB + outputs: beyond L2 together with the results.
        self.a = _rotating(self.SETS, lambda i: data["a"].roll(i, 0).to(device))
        self.b = _rotating(self.SETS, lambda i: data["b"].roll(i, 1).to(device))
        self.a_pinned, self.b_pinned = data["a"].pin_memory(), data["b"].pin_memory()
        self.c_pinned = torch.empty(self.SIZE, self.SIZE).pin_memory()
        self.a_stage, self.b_stage = torch.empty_like(self.a[0]), torch.empty_like(self.b[0])

        # The call is a few short kernels (operand splits, the GEMM, the ordered sum of its K
        # chunks): replayed as one CUDA graph per operand pair, which takes the host out of the loop.
        from helion_mlir_backend import graphed

        self.calls = [graphed(lambda a, b: ops.matmul(a, b, block_sizes=(64, 64, 64)), a, b)
                      for a, b in zip(self.a, self.b)]

    def step(self, index: int) -> torch.Tensor:
        return self.calls[index % self.SETS]()

    def launches_per_step(self) -> int:
        return self.calls[0].kernels

    def e2e_step(self, index: int) -> tuple[int, int]:
        self.a_stage.copy_(self.a_pinned, non_blocking=True)
        self.b_stage.copy_(self.b_pinned, non_blocking=True)
        self.c_pinned.copy_(self.ops.matmul(self.a_stage, self.b_stage, block_sizes=(64, 64, 64)), non_blocking=True)
        return 2 * self.SIZE * self.SIZE * 4, self.SIZE * self.SIZE * 4

    def work_per_step(self) -> float:
        return 2.0 * self.SIZE**3

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "block_sizes": [64, 64, 64], "sharding": "replicas only",
                "launch": f"one CUDA graph replay per call ({self.calls[0].kernels} kernels)" if hasattr(self, "calls") else "one CUDA graph replay per call",
                "l2": f"{self.SETS} rotating operand pairs (101 MB) plus outputs > 126 MB L2"}

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        out = self.calls[0]()  # the replayed graph is what is timed
        return sampled.c1_whole(self.host["a"], self.host["b"], out)

    def cpu_setup(self) -> str:
        from oracle import inputs

        data = getattr(self, "host", None) or inputs.c1_f32_matmul(self.SIZE)
        self.cpu = (data["a"], data["b"])
        return "the full 1024^3 f32 torch CPU matmul per step"

    def cpu_step(self) -> float:
        a, b = self.cpu
        a @ b
        return 2.0 * self.SIZE**3


class BlockedMatmul(Workload):
    """C3: A [M/32,K/32,32,32] x VNNI B [N/32,K/32,16,32,2] -> f32 [M,N], 8192^3."""

    name, metric, unit, dtype, bound = "c3_blocked_vnni_matmul_8192", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    SIZE = 8192
    traffic = 1506.0e6  # gemm_umma_bf16_kernel<2, blocked A>: 1252.1 MB read + 253.9 MB written (operands streamed 4.7 times)

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops
        from oracle import inputs

        self.ops, self.device = ops, device
        data = inputs.c3_blocked(self.SIZE)
        self.host = data
        a, b = data["a"].to(device), data["b"].to(device)
        self.a4 = ops.pack_a_blocked(a)
        self.b5 = ops.pack_b_blocked_vnni(b)
        del a, b

    def step(self, index: int) -> torch.Tensor:
        s = self.SIZE
        return self.ops.matmul_blocked(self.a4, self.b5, s, s, s, out_dtype=torch.float32)

    def work_per_step(self) -> float:
        return 2.0 * self.SIZE**3

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "out": "f32", "sharding": "block rows of A per GPU, no collective",
                "l2": "operands 268 MB + output 268 MB > 126 MB L2"}

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        rows = sampled.rows_of_interest(self.SIZE, extra=8)
        out = self.step(0)
        return sampled.c3_rows(self.host["a"][rows], self.host["b"], out[rows.to(self.device)], self.SIZE)

    CPU_ROWS = 1024

    def cpu_setup(self) -> str:
        from oracle import inputs

        data = getattr(self, "host", None) or inputs.c3_blocked(self.SIZE)
        self.cpu = (data["a"][: self.CPU_ROWS].float(), data["b"].float())
        return f"{self.CPU_ROWS} of {self.SIZE} rows per step, torch CPU f32 matmul on unpacked operands"

    def cpu_step(self) -> float:
        a, b = self.cpu
        a @ b
        return 2.0 * a.shape[0] * self.SIZE**2


class SplitKBmm(Workload):
    """C5: batch=64, M=N=512, K=16384 bf16, split_k=8 in order, f32 output."""

    name, metric, unit, dtype, bound = "c5_split_k_bmm_64x512x512x16384", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    B, M, N, K = 64, 512, 512, 16384
    traffic = 2217.6e6  # 37-batch capture (1258.5 MB read + 23.5 MB written) scaled to 64 batches

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops, self.device = ops, device
        gen = torch.Generator(device=device).manual_seed(1005 + rank)
        self.a = (torch.rand(self.B, self.M, self.K, generator=gen, device=device) * 2 - 1).bfloat16()
        self.b = (torch.rand(self.B, self.K, self.N, generator=gen, device=device) * 2 - 1).bfloat16()

    def step(self, index: int) -> torch.Tensor:
        return self.ops.bmm(self.a, self.b, split_k=8, out_dtype=torch.float32)

    def work_per_step(self) -> float:
        return 2.0 * self.B * self.M * self.N * self.K

    def hbm_bytes_per_step(self) -> float:
        return 2.0 * self.B * self.K * (self.M + self.N) + 4.0 * self.B * self.M * self.N

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "split_k": 8, "out": "f32", "sharding": "batches per GPU, no collective",
                "l2": "operands 2.1 GB > 126 MB L2"}

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        batches = sorted({0, self.B - 10, self.B - 9, self.B - 1} & set(range(self.B))) or [0]
        out = self.step(0)
        return sampled.c5_batches(self.a[batches].cpu(), self.b[batches].cpu(), out[batches], batches, self.B)

    CPU_BATCHES = 2

    def cpu_setup(self) -> str:
        gen = torch.Generator().manual_seed(1005)
        a = (torch.rand(self.CPU_BATCHES, self.M, self.K, generator=gen) * 2 - 1).bfloat16().float()
        b = (torch.rand(self.CPU_BATCHES, self.K, self.N, generator=gen) * 2 - 1).bfloat16().float()
        self.cpu = (a, b)
        return f"{self.CPU_BATCHES} of {self.B} batches per step, torch CPU f32 bmm"

    def cpu_step(self) -> float:
        a, b = self.cpu
        torch.bmm(a, b)
        return 2.0 * a.shape[0] * self.M * self.N * self.K


class Attention(Workload):
    """Softmax attention of 128 heads (4 sequences x 32 heads) of 4096 x 128, bf16."""

    name, metric, unit, dtype, bound = "attention_128x4096x128", "bf16 attention TFLOP/s", "TFLOP/s", "bf16", "tensor"
    H, S, D, SETS = 128, 4096, 128, 2

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops, self.device = ops, device
        gen = torch.Generator().manual_seed(1006 + rank)
        host = [torch.randn(self.H, self.S, self.D, generator=gen).bfloat16() for _ in range(3)]
        self.host = host
        # Two rotating operand sets: 2 x 4 x 134 MB, beyond the 126 MB L2.
        self.sets = _rotating(self.SETS, lambda i: [t.roll(i, 1).to(device) for t in host])
        self.pinned = [t.pin_memory() for t in host]
        self.out_pinned = torch.empty(self.H, self.S, self.D, dtype=torch.bfloat16).pin_memory()
        self.stage = [torch.empty_like(t) for t in self.sets[0]]

    def step(self, index: int) -> torch.Tensor:
        q, k, v = self.sets[index % self.SETS]
        return self.ops.attention(q, k, v)

    def e2e_step(self, index: int) -> tuple[int, int]:
        for dst, src in zip(self.stage, self.pinned):
            dst.copy_(src, non_blocking=True)
        self.out_pinned.copy_(self.ops.attention(*self.stage), non_blocking=True)
        return 3 * self.pinned[0].numel() * 2, self.out_pinned.numel() * 2

    def work_per_step(self) -> float:
        return 4.0 * self.H * self.S * self.S * self.D

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "heads": self.H, "seq": self.S, "dim": self.D, "scale": "dim ** -0.5",
                "sharding": "heads per GPU, no collective", "l2": "operands rotated over 2 sets (1.07 GB) > 126 MB L2"}

    def parity(self) -> dict[str, object]:
        from oracle import ops as ref
        from oracle import sampled

        heads = [0, self.H - 1]
        out = self.step(0)[heads]
        q, k, v = (t[heads] for t in self.host)
        expect = ref.attention(q, k, v, self.D ** -0.5)
        return sampled._report(torch.bfloat16, out, expect, f"heads {heads} of {self.H}, whole")

    CPU_HEADS = 2

    def cpu_setup(self) -> str:
        self.cpu = tuple(torch.randn(self.CPU_HEADS, self.S, self.D).bfloat16().float() for _ in range(3))
        return f"{self.CPU_HEADS} of {self.H} heads per step, torch CPU restatement (f64 scores)"

    def cpu_step(self) -> float:
        from oracle import ops as ref

        ref.attention(*self.cpu, self.D ** -0.5)
        return 4.0 * self.CPU_HEADS * self.S * self.S * self.D


class BandwidthKernels(Workload):
    """The bandwidth-bound kernel families beside C4's three: reductions, element-wise
    operators, layout conversions, long-row softmax. One launch of each per step; the line's
    `kernels` block times each alone (bytes read + written over the CUDA-event time)."""

    name, metric, unit, dtype, bound = "bandwidth_kernels", "reduction / element-wise / pack HBM GB/s", "GB/s", "f32+bf16", "hbm"
    only: str | None = None  # --kernel NAME: that one kernel only (profiler captures)
    row_lengths: list[int] | None = None  # --row-lengths: the row-wise kernels and row reductions at these lengths instead

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops, self.device = ops, device
        gen = torch.Generator(device=device).manual_seed(1007 + rank)
        if self.row_lengths:
            # softmax / layer_norm / rms_norm / row_sum / row_dot over about 0.5 GB of rows of each length
            self.items = []
            for n in self.row_lengths:
                for dtype, name, size in ((torch.float32, "f32", 4), (torch.bfloat16, "bf16", 2)):
                    m = max(1, (1 << 29) // (n * size))
                    x = torch.randn(m, n, generator=gen, device=device).to(dtype)
                    g, b = torch.randn(n, device=device).to(dtype), torch.randn(n, device=device).to(dtype)
                    v = torch.randn(n, device=device)
                    both, once = 2.0 * m * n * size, 1.0 * m * n * size
                    tag = f"{name}_{m}x{n}"
                    self.items += [
                        (f"softmax_{tag}", both, lambda x=x: ops.softmax(x)),
                        (f"layer_norm_{tag}", both, lambda x=x, g=g, b=b: ops.layer_norm(x, g, b, 1e-5)),
                        (f"rms_norm_{tag}", both, lambda x=x, g=g: ops.rms_norm(x, g, 1e-5)),
                        (f"row_sum_{tag}", once, lambda x=x: ops.row_sum(x)),
                        (f"row_dot_{tag}", once, lambda x=x, v=v: ops.row_dot(x, v)),
                    ]
            if self.only:
                self.items = [item for item in self.items if item[0] == self.only]
                if not self.items:
                    raise SystemExit(f"--kernel {self.only}: no such kernel in this workload")
            return
        m, n = 32768, 4096
        x32 = torch.randn(m, n, generator=gen, device=device)
        x16 = x32.bfloat16()
        tall32 = torch.randn(1 << 20, 64, generator=gen, device=device)
        tall16 = tall32.bfloat16()
        v = torch.randn(n, generator=gen, device=device)
        v16 = v.bfloat16().reshape(n, 1)
        long32 = torch.randn(2048, 65536, generator=gen, device=device)
        sq16 = torch.randn(8192, 8192, generator=gen, device=device).bfloat16()
        sq32 = torch.randn(8192, 8192, generator=gen, device=device)
        # rows that no power-of-two number of threads covers: 12288 = 192 threads x 64 values,
        # 768 = 32 x 24, 11008 has only a cover with a tail
        r12k = torch.randn(16384, 12288, generator=gen, device=device).bfloat16()
        g12k, b12k = torch.randn(12288, device=device).bfloat16(), torch.randn(12288, device=device).bfloat16()
        r768 = torch.randn(262144, 768, generator=gen, device=device).bfloat16()
        g768, b768 = torch.randn(768, device=device).bfloat16(), torch.randn(768, device=device).bfloat16()
        r11k = torch.randn(12288, 11008, generator=gen, device=device)
        f4, f2 = 4.0 * m * n, 2.0 * m * n
        t4, t2 = 4.0 * (1 << 20) * 64, 2.0 * (1 << 20) * 64
        s2, s4 = 2.0 * 8192 * 8192, 4.0 * 8192 * 8192
        # (name, bytes read + written, call)
        self.items = [
            ("row_sum_f32_32768x4096", f4, lambda: ops.row_sum(x32)),
            ("row_sum_bf16_32768x4096", f2, lambda: ops.row_sum(x16)),
            ("row_dot_f32_32768x4096", f4, lambda: ops.row_dot(x32, v)),
            ("row_dot_bf16_32768x4096", f2, lambda: ops.row_dot(x16, v)),
            ("matvec_bf16_32768x4096", f2, lambda: ops.matvec(x16, v16)),
            ("column_sum_f32_32768x4096", f4, lambda: ops.column_sum(x32)),
            ("column_sum_bf16_32768x4096", f2, lambda: ops.column_sum(x16)),
            ("row_sum_f32_1048576x64", t4, lambda: ops.row_sum(tall32)),
            ("row_sum_bf16_1048576x64", t2, lambda: ops.row_sum(tall16)),
            ("column_sum_f32_1048576x64", t4, lambda: ops.column_sum(tall32)),
            ("column_sum_bf16_1048576x64", t2, lambda: ops.column_sum(tall16)),
            ("relu_f32_32768x4096", 2 * f4, lambda: ops.relu(x32)),
            ("leaky_relu_bf16_32768x4096", 2 * f2, lambda: ops.leaky_relu(x16)),
            ("scalar_mul_f32_32768x4096", 2 * f4, lambda: ops.scalar_mul(x32, 1.5)),
            ("softmax_long_rows_f32_2048x65536", 2 * 4.0 * 2048 * 65536, lambda: ops.softmax(long32)),
            ("layer_norm_bf16_16384x12288", 2 * 2.0 * 16384 * 12288, lambda: ops.layer_norm(r12k, g12k, b12k, 1e-5)),
            ("layer_norm_bf16_262144x768", 2 * 2.0 * 262144 * 768, lambda: ops.layer_norm(r768, g768, b768, 1e-5)),
            ("softmax_f32_12288x11008", 2 * 4.0 * 12288 * 11008, lambda: ops.softmax(r11k)),
            ("pack_a_blocked_bf16_8192", 2 * s2, lambda: ops.pack_a_blocked(sq16)),
            ("pack_a_blocked_t_bf16_8192", 2 * s2, lambda: ops.pack_a_blocked_t(sq16)),
            ("pack_b_blocked_vnni_bf16_8192", 2 * s2, lambda: ops.pack_b_blocked_vnni(sq16)),
            ("pack_b_blocked_t_f32_8192", 2 * s4, lambda: ops.pack_b_blocked_t(sq32)),
            ("pack_b_vnni_t_bf16_8192", 2 * s2, lambda: ops.pack_b_vnni_t(sq16, 128)),
        ]
        if self.only:
            self.items = [item for item in self.items if item[0] == self.only]
            if not self.items:
                raise SystemExit(f"--kernel {self.only}: no such kernel in this workload")

    def step(self, index: int) -> torch.Tensor:
        out = None
        for _, _, call in self.items:
            out = call()
        return out

    def work_per_step(self) -> float:
        return float(sum(nbytes for _, nbytes, _ in self.items))

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "kernels": [name for name, _, _ in getattr(self, "items", [])],
                "l2": "every operand is 0.13-1 GiB, beyond the 126 MB L2"}

    def parity(self) -> dict[str, object]:
        return {"parity_metric": None, "parity_pass": None,
                "checked": "these kernels are compared with the oracle and the fixtures by tests/test_gpu_golden.py, test_gpu_packs.py"}

    def cpu_setup(self) -> str:
        self.cpu = torch.randn(4096, 4096)
        return "row sums, column sums and relu of 4096 of 32768 rows, torch CPU"

    def cpu_step(self) -> float:
        x = self.cpu
        x.sum(1), x.sum(0), torch.relu(x)
        return 4.0 * x.numel() * 4


class ColumnShardedLinear(Workload):
    """C2-N: the C2 linear with W split along N over the ranks; every rank holds all of x,
    computes its columns of y and the column shards are all-gathered (NCCL) into the whole
    y on every rank. The total work is C2's whatever the number of GPUs (strong scaling)."""

    name, metric, unit, dtype, bound = "c2n_column_sharded_linear_8192x4096x4096", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    scaling = "strong"
    collective = True
    M, N, K, SETS = 8192, 4096, 4096, 3
    fused = False

    def setup(self, device: torch.device, rank: int) -> None:
        import torch.distributed as dist

        import helion_mlir_utils as ops
        from helion_mlir_utils import sharding
        from oracle import inputs

        self.ops, self.device, self.sharding = ops, device, sharding
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if self.N % self.world:
            raise SystemExit(f"c2n: {self.N} columns do not divide over {self.world} ranks")
        data = inputs.c2_linear(self.M, self.N, self.K)  # the same x, W, b on every rank
        self.host = data
        n0, n1 = sharding.shard_bounds(self.N, self.world, self.rank)
        self.w, self.b = data["w"][n0:n1].contiguous().to(device), data["b"][n0:n1].contiguous().to(device)
        self.xs = _rotating(self.SETS, lambda i: data["x"].roll(i, 0).to(device))
        self.fused_call = None
        if self.fused:
            self.fused_call = sharding.FusedColumnShardedLinear(self.M, self.N, self.K, torch.bfloat16, device)

    def step(self, index: int) -> torch.Tensor:
        x = self.xs[index % self.SETS]
        if self.fused_call is not None:
            return self.fused_call(x, self.w, self.b, F.gelu)
        if self.world == 1:
            return self.ops.matmul(x, self.w, trans_b=True, bias=self.b, epilogue=F.gelu)
        return self.sharding.column_sharded_linear(x, self.w, self.b, self.N, F.gelu)

    def teardown(self) -> None:
        if self.fused_call is not None:
            self.fused_call.close()
            self.fused_call = None

    def gemm_only(self, index: int) -> torch.Tensor:
        return self.ops.matmul(self.xs[index % self.SETS], self.w, trans_b=True, bias=self.b, epilogue=F.gelu)

    def work_per_step(self) -> float:
        return 2.0 * self.M * self.N * self.K / self.world

    def config(self) -> dict[str, object]:
        return {
            "workload": self.name, "m": self.M, "n": self.N, "k": self.K, "epilogue": "bias+gelu_erf",
            "sharding": f"W split along N over {getattr(self, 'world', 1)} ranks, x replicated",
            "collective": ("epilogue stores into every rank's y over NVLink peer memory, then one flag per rank pair"
                           if self.fused else "NCCL all-gather of the [M, N/G] column shards, then one strided copy"),
            "l2": f"inputs rotated over {self.SETS} buffer sets",
        }

    def parity(self) -> dict[str, object]:
        from oracle import sampled

        rows = sampled.rows_of_interest(self.M, extra=4)
        y = self.step(0)
        torch.cuda.synchronize()
        return sampled.c2_rows(self.host["x"], self.host["w"], self.host["b"], y[rows.to(self.device)], rows)

    CPU_ROWS = 1024

    def cpu_setup(self) -> str:
        return LinearGelu.cpu_setup(self)  # the same arithmetic as C2

    def cpu_step(self) -> float:
        return LinearGelu.cpu_step(self)


class FusedColumnShardedLinear(ColumnShardedLinear):
    name = "c2n_fused_column_sharded_linear_8192x4096x4096"
    fused = True


WORKLOADS = {"c1": F32Matmul, "c2": LinearGelu, "c3": BlockedMatmul, "c4": RowNorms, "c5": SplitKBmm, "attn": Attention,
             "c2n": ColumnShardedLinear, "c2n_fused": FusedColumnShardedLinear, "kernels": BandwidthKernels}
BLOCKS = ["c4", "c1", "c3", "c5"]  # timed beside the main line, in this order


# --------------------------------------------------------------------------- driver


def env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def cpu_baseline(workload: Workload, threads: int, budget_s: float = 6.0) -> dict[str, object]:
    """The CPU restatement on a bounded sample: one warm-up step, then steps until
    ``budget_s`` has passed (three at least); the rate is work over the median step."""
    torch.set_num_threads(threads)
    sample = workload.cpu_setup()
    workload.cpu_step()
    times, work = [], 0.0
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        work = workload.cpu_step()
        times.append(time.perf_counter() - t0)
    scale = 1e12 if workload.unit == "TFLOP/s" else 1e9
    return {"value": work / statistics.median(times) / scale, "unit": workload.unit, "cores": threads, "kind": "port",
            "sample": f"{sample}; median of {len(times)} steps"}


def run_reference(args: argparse.Namespace, workload: Workload, rank: int) -> None:
    """The CPU implementation of the path on this host's cores (rank 0 only): a step is
    one run of the restatement on the bounded sample its description names."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = workload.cpu_setup()
    for _ in range(max(args.warmup, 1)):
        workload.cpu_step()
    times, work = [], 0.0
    t_all = time.perf_counter()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        work = workload.cpu_step()
        times.append(time.perf_counter() - t0)
    elapsed = time.perf_counter() - t_all
    scale = 1e12 if workload.unit == "TFLOP/s" else 1e9
    value = work * args.steps / elapsed / scale
    line = {
        "impl": "reference", "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic",
        "config": workload.config(),
        "cpu_baseline": {"value": value, "unit": workload.unit, "cores": threads, "kind": "port",
                         "sample": f"{sample}; {args.steps} steps after {max(args.warmup, 1)} warm-up"},
        "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's own pipeline needs Helion + MLIR/lighthouse (not installed): the CPU restatement under oracle/ is timed; a step is one run on the bounded sample, the rate is per unit of work",
    }
    print(json.dumps(line), flush=True)


class Harness:
    """Timing plumbing shared by the main line and the configuration blocks."""

    def __init__(self, device: torch.device, rank: int, world: int, sampler: ClockSampler | None) -> None:
        self.device, self.rank, self.world, self.sampler = device, rank, world, sampler
        self.distributed = world > 1
        self.peaks, self.peak_kind = measured_peaks()
        self.start, self.stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def barrier(self) -> None:
        if self.distributed:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize(self.device)

    def max_over_ranks(self, *values: float) -> list[float]:
        t = torch.tensor(values, device=self.device, dtype=torch.float64)
        if self.distributed:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def timed(self, step, steps: int) -> tuple[float, dict[str, object], int]:
        """``steps`` calls of ``step(i)`` between two events on the launch stream, a barrier and a
        synchronise on both sides; returns (ms of the slowest rank, clocks in the window, launches)."""
        from helion_mlir_backend import native

        self.barrier()
        before = native.counters()["launches"]
        t0 = time.monotonic()
        self.start.record()
        for i in range(steps):
            step(i)
        self.stop.record()
        self.barrier()
        t1 = time.monotonic()
        ms = self.max_over_ranks(self.start.elapsed_time(self.stop))[0]
        clocks = self.sampler.window(t0, t1) if self.sampler is not None else {}
        return ms, clocks, int(native.counters()["launches"] - before)

    def roofline(self, workload: Workload, per_gpu: float) -> dict[str, object]:
        if workload.bound == "tensor":
            peak, unit, what = self.peaks["bf16_tflops"], "TFLOP/s", "burst cuBLAS bf16"
        else:
            peak, unit, what = self.peaks["hbm_gbs"], "GB/s", "copy bandwidth"
        return {"bound": workload.bound, "achieved": per_gpu, "peak": peak, "unit": unit, "frac": per_gpu / peak,
                "peak_source": f"{self.peak_kind} ({what})", "traffic": workload.traffic}


def host_copy_ceiling(harness: Harness, nbytes: int = 64 << 20, rounds: int = 8) -> dict[str, object]:
    """What the box's host side can move with every rank copying at once: each rank copies
    `nbytes` of pinned memory to its GPU and as much back, on two streams at the same time
    (plain cudaMemcpyAsync through torch, one copy per direction per round). The end-to-end
    leg can be no faster than its bytes over this rate."""
    device = harness.device
    up_src, down_dst = torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    up_dst, down_src = torch.empty(nbytes, dtype=torch.uint8, device=device), torch.zeros(nbytes, dtype=torch.uint8, device=device)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)
    start, stop_up, stop_down = (torch.cuda.Event(enable_timing=True) for _ in range(3))

    def run(count: int) -> float:
        harness.barrier()
        start.record()
        up.wait_event(start)
        down.wait_event(start)
        for _ in range(count):
            with torch.cuda.stream(up):
                up_dst.copy_(up_src, non_blocking=True)
            with torch.cuda.stream(down):
                down_dst.copy_(down_src, non_blocking=True)
        stop_up.record(up)
        stop_down.record(down)
        harness.barrier()
        up.synchronize()
        down.synchronize()
        return max(start.elapsed_time(stop_up), start.elapsed_time(stop_down))

    run(2)
    ms = harness.max_over_ranks(run(rounds))[0]
    per_rank = nbytes * rounds / (ms * 1e-3) / 1e9
    return {"per_rank_gbs_each_direction": per_rank, "aggregate_gbs_each_direction": per_rank * harness.world,
            "how": f"{harness.world} ranks at once, {rounds} x {nbytes >> 20} MiB pinned host -> device and as much back concurrently, slowest rank"}


def exchange_details(workload: "ColumnShardedLinear", harness: Harness, step_ms: float, steps: int) -> dict[str, object]:
    """Where a column-sharded step's time goes (the local GEMM timed alone; the rest is the
    exchange) and the floor it is held against: a step can be no faster than the slower of
    this rank's FLOPs at the measured GEMM peak and the bytes it must send over NVLink (its
    shard, once to every other rank) at the measured peer-copy rate of this pool, 770 GB/s per
    direction per GPU."""
    g_ms, _, _ = harness.timed(workload.gemm_only, steps)
    g_ms /= steps
    world = harness.world
    flops_ms = workload.work_per_step() / (harness.peaks["bf16_tflops"] * 1e12) * 1e3
    link_bytes = 2.0 * workload.M * (workload.N / world) * (world - 1)
    link_ms = link_bytes / 770e9 * 1e3
    floor_ms = max(flops_ms, link_ms)
    return {
        "split": {"gemm_ms_per_step": g_ms, "exchange_ms_per_step": max(step_ms - g_ms, 0.0),
                  "exchange_share": max(step_ms - g_ms, 0.0) / step_ms,
                  "note": "local GEMM of this rank's columns timed alone; the remainder of the step is the exchange"},
        "roofline_exchange": {"bound": "tensor" if flops_ms >= link_ms else "nvlink", "flops_ms": flops_ms,
                              "nvlink_ms": link_ms, "nvlink_bytes_out_per_rank": link_bytes, "nvlink_gbs_assumed": 770.0,
                              "floor_ms": floor_ms, "frac": floor_ms / step_ms},
    }


def run_block(key: str, harness: Harness, rank: int, with_cpu: bool) -> dict[str, object]:
    """One of the other configurations: set up, warm up, size the inner repeat count from a
    pilot so that the timed region is BLOCK_TARGET_MS of device time, time it, check parity."""
    workload: Workload = WORKLOADS[key]()
    workload.setup(harness.device, rank)
    for i in range(5):
        workload.step(i)
    pilot_ms, _, _ = harness.timed(workload.step, 10)
    repeats = int(min(20000, max(20, math.ceil(BLOCK_TARGET_MS / max(pilot_ms / 10, 1e-3)))))
    ms, clocks, launches = harness.timed(workload.step, repeats)
    graph_kernels = workload.launches_per_step()
    if graph_kernels is not None:
        launches = graph_kernels * repeats
    scale = 1e12 if workload.unit == "TFLOP/s" else 1e9
    work = workload.work_per_step()
    per_gpu = work * repeats / (ms * 1e-3) / scale
    block: dict[str, object] = {
        "metric": workload.metric, "value": per_gpu * harness.world, "unit": workload.unit, "per_gpu": per_gpu,
        "ms_per_step": ms / repeats, "inner_repeats": repeats,
        "burst": {"per_gpu": work * 10 / (pilot_ms * 1e-3) / scale, "steps": 10, "ms_per_step": pilot_ms / 10,
                  "note": "the 10 pilot steps after 5 warm-up steps, before the power cap bites; `value` is the 300 ms run"},
        "timing": f"{repeats} steps back to back (sized for {BLOCK_TARGET_MS:.0f} ms of device time, independent of --steps), CUDA events, max over ranks",
        "dtype": workload.dtype, "config": workload.config(), "roofline": harness.roofline(workload, per_gpu),
        "gpu_launches": launches, "clocks": clocks,
    }
    if isinstance(workload, SplitKBmm):
        gbs = workload.hbm_bytes_per_step() * repeats / (ms * 1e-3) / 1e9
        block["roofline_hbm"] = {"bound": "hbm", "achieved": gbs, "peak": harness.peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / harness.peaks["hbm_gbs"],
                                 "note": "the configuration is bound by the larger of its two fractions"}
    if isinstance(workload, RowNorms):
        # each of the six kernels alone, 20 launches back to back
        per_kernel = {}
        for name, size, run in workload.kernels():
            k_ms, _, _ = harness.timed(lambda i, run=run: run(), 20)
            gbs = 2.0 * workload.M * workload.N * size * 20 / (k_ms * 1e-3) / 1e9
            per_kernel[name] = {"GB/s": gbs, "frac": gbs / harness.peaks["hbm_gbs"]}
        block["kernels"] = per_kernel
        e2e = workload.e2e_step(0)
        if e2e is not None:
            e2e_ms, _, _ = harness.timed(workload.e2e_step, 5)
            block["e2e"] = {"value": 2.0 * workload.M * workload.N * 4 * 5 * harness.world / (e2e_ms * 1e-3) / 1e9,
                            "unit": "GB/s", "what": "stream_rows(softmax) f32 through pinned host buffers",
                            "h2d_bytes_per_step": e2e[0], "d2h_bytes_per_step": e2e[1], "ms_per_step": e2e_ms / 5}
    if isinstance(workload, ColumnShardedLinear):
        block.update(exchange_details(workload, harness, ms / repeats, 50))
    if rank == 0 or workload.collective:
        try:
            block.update(workload.parity())
        except Exception as exc:  # a parity leg that cannot run is a failed parity, not a crashed benchmark
            block.update({"parity_metric": None, "parity_pass": False, "parity_error": f"{type(exc).__name__}: {exc}"})
        if with_cpu:
            block["cpu_baseline"] = cpu_baseline(workload, os.cpu_count() or 1, budget_s=3.0)
    harness.barrier()
    workload.teardown()
    del workload
    from helion_mlir_utils import host_io

    host_io.release()
    torch.cuda.empty_cache()
    return block


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    parser.add_argument("--rows", type=int, default=0, help="rows per GPU of the c2/c4 workloads, heads per GPU of attn, batches per GPU of c5 (default: the configuration's; smaller sizes are for profiler captures, not for reported numbers)")
    parser.add_argument("--kernel", default=None, help="kernels workload: run this one kernel only (profiler captures)")
    parser.add_argument("--row-lengths", default=None,
                        help="kernels workload: time softmax, layer_norm, rms_norm, row_sum and row_dot over rows of these "
                             "lengths (comma separated) in f32 and bf16 instead of the fixed list")
    parser.add_argument("--only-main", action="store_true", help="skip the blocks of the other configurations, the sustained leg and the linear() leg")
    parser.add_argument("--via-linear", action="store_true", help="c2: time linear(x, layer, F.gelu, cache) as the main step")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 0)

    rank, world, local_rank = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    workload: Workload = WORKLOADS[args.workload]()
    if args.rows > 0:
        # the one size of the workload that shards: batches, else heads, else rows
        for name in ("B", "H", "M"):
            if hasattr(workload, name):
                setattr(workload, name, args.rows)
                break
    if isinstance(workload, BandwidthKernels):
        workload.only = args.kernel
        if args.row_lengths:
            workload.row_lengths = [int(v) for v in args.row_lengths.split(",") if v]
    if args.via_linear and isinstance(workload, LinearGelu):
        workload.via_linear = True
    if args.impl == "reference":
        run_reference(args, workload, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator set has no CPU path (use --impl reference for the CPU port)")
    warmup = max(args.warmup, 3)
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from helion_mlir_backend import native

    sampler = None
    if rank == 0:
        sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local_rank)
        sampler.start()
    harness = Harness(device, rank, world, sampler)
    workload.setup(device, rank)

    # The warm-up is the same load as the timed region and is inside the clock window: a
    # timed region of a few milliseconds alone would see no 100 ms sample.
    t_warm = time.monotonic()
    time.sleep(0.12)
    for i in range(warmup):
        workload.step(i)
    device_ms, clocks, launches = harness.timed(workload.step, args.steps)
    if sampler is not None:
        clocks = sampler.window(t_warm, time.monotonic())
    graph_kernels = workload.launches_per_step()
    if graph_kernels is not None:
        launches = graph_kernels * args.steps

    e2e_ms, h2d, d2h = None, 0, 0
    first = None if args.no_e2e else workload.e2e_step(0)
    if first is not None:
        h2d, d2h = first
        workload.e2e_step(1)
        e2e_ms, _, _ = harness.timed(workload.e2e_step, args.steps)
    ceiling = host_copy_ceiling(harness) if first is not None else None

    main_only = args.only_main or args.workload != "c2"
    extras: dict[str, object] = {}
    if not main_only and isinstance(workload, LinearGelu):
        # first the other entry point, at the same (burst) clocks as the main timed region
        for i in range(3):
            workload.linear_step(i)
        l_ms, _, _ = harness.timed(workload.linear_step, args.steps)
        l_per_gpu = workload.work_per_step() * args.steps / (l_ms * 1e-3) / 1e12
        extras["linear_entry"] = {
            "value": l_per_gpu * world, "unit": "TFLOP/s", "ms_per_step": l_ms / args.steps,
            "entry": "linear(x, layer, F.gelu, cache): the weight cache's prepared call; `value` of the line is matmul(x, W, trans_b=True, bias=b, epilogue=F.gelu) unless --via-linear",
        }

        # the same step back to back for SUSTAINED_SECONDS: the power-capped, steady figure
        count = int(min(50000, max(args.steps, math.ceil(SUSTAINED_SECONDS * 1e3 / max(device_ms / args.steps, 1e-3)))))
        s_ms, s_clocks, _ = harness.timed(workload.step, count)
        s_per_gpu = workload.work_per_step() * count / (s_ms * 1e-3) / 1e12
        extras["sustained"] = {
            "value": s_per_gpu * world, "per_gpu": s_per_gpu, "unit": "TFLOP/s", "steps": count, "ms_per_step": s_ms / count,
            "peak": harness.peaks["bf16_tflops_sustained"], "frac": s_per_gpu / harness.peaks["bf16_tflops_sustained"],
            "peak_source": f"{harness.peak_kind} (cuBLAS bf16 back to back for seconds)", "clocks": s_clocks,
        }
    if isinstance(workload, ColumnShardedLinear):
        extras.update(exchange_details(workload, harness, device_ms / args.steps, args.steps))
    if isinstance(workload, BandwidthKernels):
        table = {}
        for name, nbytes, call in workload.items:
            k_ms, _, _ = harness.timed(lambda i, call=call: call(), 20)
            gbs = nbytes * 20 / (k_ms * 1e-3) / 1e9
            table[name] = {"GB/s": round(gbs, 1), "frac": round(gbs / harness.peaks["hbm_gbs"], 3)}
        extras["kernels"] = table

    status = native.kernel_status(device)
    parity: dict[str, object] = {}
    if rank == 0 or workload.collective:
        try:
            parity = workload.parity()
        except Exception as exc:
            parity = {"parity_metric": None, "parity_pass": False, "parity_error": f"{type(exc).__name__}: {exc}"}
    harness.barrier()

    blocks: dict[str, object] = {}
    if not main_only:
        del workload.xs
        torch.cuda.empty_cache()
        for key in BLOCKS + (["c2n", "c2n_fused"] if world > 1 else []):
            blocks[key] = run_block(key, harness, rank, with_cpu=(world == 1 and not args.no_cpu_baseline and key == "c4"))
        status |= native.kernel_status(device)

    if sampler is not None:
        sampler.stop()
    if rank == 0:
        scale = 1e12 if workload.unit == "TFLOP/s" else 1e9
        work = workload.work_per_step()
        value = work * args.steps * world / (device_ms * 1e-3) / scale
        per_gpu = value / world
        line: dict[str, object] = {
            "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": device_ms / args.steps, "higher_is_better": True,
            "scaling": workload.scaling, "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic",
            "config": workload.config(), "roofline": harness.roofline(workload, per_gpu),
            "gpu_launches": int(launches),
            "clocks": clocks,
            "kernel_status": status,
        }
        line.update(parity)
        if e2e_ms is not None:
            line["e2e"] = {
                "value": work * args.steps * world / (e2e_ms * 1e-3) / scale, "unit": workload.unit,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
            }
            if ceiling is not None:
                # the step's larger transfer at the rate every rank gets when all copy both ways at once
                floor_ms = max(h2d, d2h) / (float(ceiling["per_rank_gbs_each_direction"]) * 1e9) * 1e3
                line["e2e"].update({"host_ceiling": ceiling, "floor_ms_per_step": floor_ms,
                                    "frac_of_host_ceiling": floor_ms / (e2e_ms / args.steps)})
        else:
            line["e2e"] = None  # this workload has no host-buffer leg
        line.update(extras)
        if blocks:
            line["configs"] = blocks
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(workload, os.cpu_count() or 1)
        print(json.dumps(line), flush=True)
    workload.teardown()
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
