"""Benchmark of the hot path: the fused bf16 linear  y = GELU(x @ W^T + b).

    python bench.py --gpus N --steps K --warmup W [--workload c2|c4|c1|c3|c5|attn] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input. The default
workload is the configuration the headline metric is quoted on: x [8192,4096],
W [4096,4096], b [4096] bf16, f32 accumulation, GELU, bf16 output. With N GPUs each
rank runs its own batch of 8192 rows (rows are independent: no collective on the
data path) and `value` is the whole-job TFLOP/s over the slowest rank's time.

One JSON line is printed by rank 0. Besides the driver's keys it carries
`roofline` (algorithmic FLOPs or bytes over the CUDA-event time of the dominant
kernel, against the measured peak), `cpu_baseline` (the CPU restatement of the
reference's operator timed on this host's cores on a bounded sample) and `e2e`
(the same metric through the public operator with host buffers: pinned host ->
device copy of x, the kernel, device -> host copy of y, every step).

`--impl reference` times the CPU implementation of the path instead (the
reference's own pipeline needs Helion + an MLIR toolchain, which are not
installed, so the restatement under oracle/ stands in for it).
"""

from __future__ import annotations

import argparse
import json
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[str] = []
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
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict[str, object]:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=5)
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


# --------------------------------------------------------------------------- workloads


class Workload:
    """One benchmark configuration: device buffers, the step, its algorithmic work."""

    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "tensor"

    def setup(self, device: torch.device, rank: int) -> None:
        raise NotImplementedError

    def step(self, index: int) -> torch.Tensor:
        raise NotImplementedError

    def e2e_step(self, index: int) -> tuple[int, int]:
        raise NotImplementedError

    def work_per_step(self) -> float:
        """FLOPs (tensor-bound) or bytes (HBM-bound) of one step on one GPU."""
        raise NotImplementedError

    def config(self) -> dict[str, object]:
        raise NotImplementedError

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        """Seconds per unit of work measure on the CPU port: returns (value in `unit`, description)."""
        raise NotImplementedError


def _rotating(count: int, make):
    return [make(i) for i in range(count)]


class LinearGelu(Workload):
    """C2: y = GELU(x @ W^T + b), bf16, f32 accumulate."""

    name, metric, unit, dtype, bound = "c2_linear_gelu_8192x4096x4096", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    M, N, K, SETS = 8192, 4096, 4096, 3

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

    def step(self, index: int) -> torch.Tensor:
        return self.ops.matmul(self.xs[index % self.SETS], self.w, trans_b=True, bias=self.b, epilogue=F.gelu)

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
            "l2": f"inputs rotated over {self.SETS} buffer sets (403 MB) > 126 MB L2",
        }

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        from oracle import ops as ref

        rows = 1024
        x, w, b = self.host["x"][:rows], self.host["w"], self.host["b"]
        ref.matmul(x[:64], w, trans_b=True, bias=b, epilogue=F.gelu, acc_dtype=torch.float32)
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            ref.matmul(x, w, trans_b=True, bias=b, epilogue=F.gelu, acc_dtype=torch.float32)
            times.append(time.perf_counter() - t0)
        flops = 2.0 * rows * self.N * self.K
        return flops / min(times) / 1e12, f"{rows} of {self.M} rows, f32-accumulate torch CPU restatement, best of 3"


class RowNorms(Workload):
    """C4: softmax, layer_norm and rms_norm of x [32768, 4096], f32 and bf16 (six kernels per step)."""

    name, metric, unit, dtype, bound = "c4_softmax_layernorm_rmsnorm_32768x4096", "softmax/norm HBM GB/s", "GB/s", "f32+bf16", "hbm"
    M, N = 32768, 4096

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

    def step(self, index: int) -> torch.Tensor:
        ops = self.ops
        ops.softmax(self.x32)
        ops.layer_norm(self.x32, self.g32, self.b32, 1e-5)
        ops.rms_norm(self.x32, self.g32, 1e-5)
        ops.softmax(self.x16)
        ops.layer_norm(self.x16, self.g16, self.b16, 1e-5)
        return ops.rms_norm(self.x16, self.g16, 1e-5)

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

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        rows = 4096
        x = self.host["x"][:rows]
        g, b = self.host["gamma"], self.host["beta"]
        xb = x.bfloat16()

        def run() -> None:
            for t, gg, bb in ((x, g, b), (xb, g.bfloat16(), b.bfloat16())):
                tf = t.float()
                torch.softmax(tf, -1).to(t.dtype)
                F.layer_norm(tf, (self.N,), gg.float(), bb.float(), 1e-5).to(t.dtype)
                F.rms_norm(tf, (self.N,), gg.float(), 1e-5).to(t.dtype)

        run()
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            run()
            times.append(time.perf_counter() - t0)
        moved = 3 * 2.0 * rows * self.N * 4 + 3 * 2.0 * rows * self.N * 2
        return moved / min(times) / 1e9, f"{rows} of {self.M} rows, f32-compute torch CPU restatement, best of 3"


class F32Matmul(Workload):
    """C1: f32 C = A @ B, 1024^3, block_sizes=[64,64,64]."""

    name, metric, unit, dtype, bound = "c1_f32_matmul_1024", "f32 GEMM TFLOP/s", "TFLOP/s", "f32", "tensor"
    SIZE, SETS = 1024, 12

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops
        from oracle import inputs

        self.ops = ops
        data = inputs.c1_f32_matmul(self.SIZE)
        self.host = data
        # 12 rotating (A, B) pairs = 101 MB + outputs: beyond L2 together with the results.
        self.a = _rotating(self.SETS, lambda i: data["a"].roll(i, 0).to(device))
        self.b = _rotating(self.SETS, lambda i: data["b"].roll(i, 1).to(device))
        self.a_pinned, self.b_pinned = data["a"].pin_memory(), data["b"].pin_memory()
        self.c_pinned = torch.empty(self.SIZE, self.SIZE).pin_memory()
        self.a_stage, self.b_stage = torch.empty_like(self.a[0]), torch.empty_like(self.b[0])

        # The call is three short kernels (two operand splits and the GEMM): replayed as
        # one CUDA graph per operand pair, which takes the host out of the timed loop.
        from helion_mlir_backend import graphed

        self.calls = [graphed(lambda a, b: ops.matmul(a, b, block_sizes=(64, 64, 64)), a, b)
                      for a, b in zip(self.a, self.b)]
        self.graph_launches = 0

    def step(self, index: int) -> torch.Tensor:
        call = self.calls[index % self.SETS]
        self.graph_launches += call.kernels  # replays do not pass the library's launch counter
        return call()

    def e2e_step(self, index: int) -> tuple[int, int]:
        self.a_stage.copy_(self.a_pinned, non_blocking=True)
        self.b_stage.copy_(self.b_pinned, non_blocking=True)
        self.c_pinned.copy_(self.ops.matmul(self.a_stage, self.b_stage, block_sizes=(64, 64, 64)), non_blocking=True)
        return 2 * self.SIZE * self.SIZE * 4, self.SIZE * self.SIZE * 4

    def work_per_step(self) -> float:
        return 2.0 * self.SIZE**3

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "block_sizes": [64, 64, 64], "sharding": "replicas only",
                "launch": "one CUDA graph replay per call (split A, split B, GEMM)",
                "l2": f"{self.SETS} rotating operand pairs (101 MB) plus outputs > 126 MB L2"}

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        a, b = self.host["a"], self.host["b"]
        a @ b
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            a @ b
            times.append(time.perf_counter() - t0)
        return 2.0 * self.SIZE**3 / min(times) / 1e12, "full 1024^3 f32 torch CPU matmul, best of 5"


class BlockedMatmul(Workload):
    """C3: A [M/32,K/32,32,32] x VNNI B [N/32,K/32,16,32,2] -> f32 [M,N], 8192^3."""

    name, metric, unit, dtype, bound = "c3_blocked_vnni_matmul_8192", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    SIZE = 8192

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops = ops
        gen = torch.Generator(device="cpu").manual_seed(1003 + rank)
        a = torch.randn(self.SIZE, self.SIZE, generator=gen).bfloat16().to(device)
        b = torch.randn(self.SIZE, self.SIZE, generator=gen).bfloat16().to(device)
        self.a4 = ops.pack_a_blocked(a)
        self.b5 = ops.pack_b_blocked_vnni(b)
        del a, b

    def step(self, index: int) -> torch.Tensor:
        s = self.SIZE
        return self.ops.matmul_blocked(self.a4, self.b5, s, s, s, out_dtype=torch.float32)

    def e2e_step(self, index: int) -> tuple[int, int]:
        self.step(index)
        return 0, 0

    def work_per_step(self) -> float:
        return 2.0 * self.SIZE**3

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "out": "f32", "l2": "operands 268 MB + output 268 MB > 126 MB L2"}

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        rows = 1024
        a = torch.randn(rows, self.SIZE).bfloat16().float()
        b = torch.randn(self.SIZE, self.SIZE).bfloat16().float()
        t0 = time.perf_counter()
        a @ b
        return 2.0 * rows * self.SIZE**2 / (time.perf_counter() - t0) / 1e12, f"{rows} of {self.SIZE} rows, torch CPU f32 matmul on unpacked operands"


class SplitKBmm(Workload):
    """C5: batch=64, M=N=512, K=16384 bf16, split_k=8 in order, f32 output."""

    name, metric, unit, dtype, bound = "c5_split_k_bmm_64x512x512x16384", "bf16 GEMM TFLOP/s", "TFLOP/s", "bf16", "tensor"
    B, M, N, K = 64, 512, 512, 16384

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops = ops
        gen = torch.Generator(device=device).manual_seed(1005 + rank)
        self.a = (torch.rand(self.B, self.M, self.K, generator=gen, device=device) * 2 - 1).bfloat16()
        self.b = (torch.rand(self.B, self.K, self.N, generator=gen, device=device) * 2 - 1).bfloat16()

    def step(self, index: int) -> torch.Tensor:
        return self.ops.bmm(self.a, self.b, split_k=8, out_dtype=torch.float32)

    def e2e_step(self, index: int) -> tuple[int, int]:
        self.step(index)
        return 0, 0

    def work_per_step(self) -> float:
        return 2.0 * self.B * self.M * self.N * self.K

    def config(self) -> dict[str, object]:
        return {"workload": self.name, "split_k": 8, "out": "f32", "l2": "operands 2.1 GB > 126 MB L2"}

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        a = (torch.rand(2, self.M, self.K) * 2 - 1).bfloat16().float()
        b = (torch.rand(2, self.K, self.N) * 2 - 1).bfloat16().float()
        t0 = time.perf_counter()
        torch.bmm(a, b)
        return 2.0 * 2 * self.M * self.N * self.K / (time.perf_counter() - t0) / 1e12, "2 of 64 batches, torch CPU f32 bmm"


class Attention(Workload):
    """Softmax attention of 128 heads (4 sequences x 32 heads) of 4096 x 128, bf16."""

    name, metric, unit, dtype, bound = "attention_128x4096x128", "bf16 attention TFLOP/s", "TFLOP/s", "bf16", "tensor"
    H, S, D, SETS = 128, 4096, 128, 2

    def setup(self, device: torch.device, rank: int) -> None:
        import helion_mlir_utils as ops

        self.ops = ops
        gen = torch.Generator().manual_seed(1006 + rank)
        host = [torch.randn(self.H, self.S, self.D, generator=gen).bfloat16() for _ in range(3)]
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

    def cpu_sample(self, threads: int) -> tuple[float, str]:
        from oracle import ops as ref

        heads = 2
        q, k, v = (torch.randn(heads, self.S, self.D).bfloat16() for _ in range(3))
        t0 = time.perf_counter()
        ref.attention(q.float(), k.float(), v.float(), self.D ** -0.5)
        return 4.0 * heads * self.S * self.S * self.D / (time.perf_counter() - t0) / 1e12, f"{heads} of {self.H} heads, torch CPU restatement (f64 scores)"


WORKLOADS = {"c1": F32Matmul, "c2": LinearGelu, "c3": BlockedMatmul, "c4": RowNorms, "c5": SplitKBmm, "attn": Attention}


# --------------------------------------------------------------------------- driver


def env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def run_reference(args: argparse.Namespace, workload: Workload, rank: int) -> None:
    """The CPU implementation of the path on this host's cores (rank 0 only)."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    workload.host = None  # type: ignore[attr-defined]
    # Host tensors only: build them without touching a device.
    from oracle import inputs

    if isinstance(workload, LinearGelu):
        workload.host = inputs.c2_linear(1024, workload.N, workload.K)
        workload.host["x"] = workload.host["x"]
    elif isinstance(workload, RowNorms):
        workload.host = inputs.c4_rows(4096, workload.N)
    elif isinstance(workload, F32Matmul):
        workload.host = inputs.c1_f32_matmul(workload.SIZE)
    values = []
    for _ in range(args.warmup):
        workload.cpu_sample(threads)
    t0 = time.perf_counter()
    sample = ""
    for _ in range(args.steps):
        value, sample = workload.cpu_sample(threads)
        values.append(value)
    elapsed = time.perf_counter() - t0
    value = statistics.median(values)
    line = {
        "impl": "reference", "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic",
        "config": workload.config(),
        "cpu_baseline": {"value": value, "unit": workload.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's own pipeline needs Helion + MLIR/lighthouse (not installed): the CPU restatement under oracle/ is timed",
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    parser.add_argument("--rows", type=int, default=0, help="rows per GPU of the c2/c4 workloads, heads per GPU of attn, batches per GPU of c5 (default: the configuration's; smaller sizes are for profiler captures, not for reported numbers)")
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

    workload.setup(device, rank)
    peaks, peak_kind = measured_peaks()

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize(device)

    # The clock sampler covers warm-up and timed region (100 ms period: a timed region
    # of a few milliseconds alone would see no sample); the warm-up is the same load.
    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.12)
    for i in range(warmup):
        workload.step(i)
    barrier()
    launches_before = native.counters()["launches"]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph_before = getattr(workload, "graph_launches", 0)
    barrier()
    start.record()
    for i in range(args.steps):
        workload.step(i)
    stop.record()
    barrier()
    launches = native.counters()["launches"] - launches_before + getattr(workload, "graph_launches", 0) - graph_before
    device_ms = start.elapsed_time(stop)
    clocks = sampler.stop() if rank == 0 else {}

    e2e_ms, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        for i in range(2):
            workload.e2e_step(i)
        barrier()
        start.record()
        for i in range(args.steps):
            h2d, d2h = workload.e2e_step(i)
        stop.record()
        barrier()
        e2e_ms = start.elapsed_time(stop)

    status = native.kernel_status(device)
    times = torch.tensor([device_ms, e2e_ms if e2e_ms is not None else 0.0], device=device, dtype=torch.float64)
    if distributed:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    device_ms, e2e_max = float(times[0]), float(times[1])

    if rank == 0:
        scale = 1e12 if workload.unit == "TFLOP/s" else 1e9
        work = workload.work_per_step()
        value = work * args.steps * world / (device_ms * 1e-3) / scale
        per_gpu = work * args.steps / (device_ms * 1e-3) / scale
        if workload.bound == "tensor":
            peak, peak_unit = peaks["bf16_tflops"], "TFLOP/s"
        else:
            peak, peak_unit = peaks["hbm_gbs"], "GB/s"
        line: dict[str, object] = {
            "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic", "config": workload.config(),
            "roofline": {
                "bound": workload.bound, "achieved": per_gpu, "peak": peak, "unit": peak_unit, "frac": per_gpu / peak,
                "peak_source": f"{peak_kind} ({'burst cuBLAS bf16' if workload.bound == 'tensor' else 'copy bandwidth'})",
                "traffic": TRAFFIC.get(args.workload),
            },
            "gpu_launches": int(launches),
            "clocks": clocks,
            "kernel_status": status,
        }
        if e2e_ms is not None and h2d + d2h == 0:
            # this workload has no host-buffer leg: say so instead of repeating the device-resident number
            line["e2e"] = None
        elif e2e_ms is not None:
            line["e2e"] = {
                "value": work * args.steps * world / (e2e_max * 1e-3) / scale, "unit": workload.unit,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_max / args.steps,
            }
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            cpu_value, sample = workload.cpu_sample(threads)
            line["cpu_baseline"] = {"value": cpu_value, "unit": workload.unit, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


# DRAM bytes (read + write) per launch of each workload's dominant kernel, from
# the ncu captures summarised under profiles/ (None until captured).
TRAFFIC: dict[str, float | None] = {
    "c1": None,
    "c2": 158.1e6,  # gemm_umma_bf16_kernel<2>: 111.7 MB read + 46.5 MB written (algorithmic 167.8 MB)
    "c3": 1509.7e6,  # gemm_umma_bf16_kernel<2> of the step: 1256 MB read + 253.7 MB written (operands streamed 4.7 times)
    "c4": 860.1e6,  # f32 softmax, scaled x4 from the 8192-row capture (134.26 MB read + 80.77 MB written)
    "c5": 2216.6e6,  # 37-batch capture (1258.5 MB read + 23.0 MB written) scaled to 64 batches
    "attn": None,
}


if __name__ == "__main__":
    main()
