"""What needs two GPUs on one box: the column-sharded linear over NCCL (the one exchange
the operator set has) and its fused form (epilogue stores into every rank's copy of y through peer memory, flag words, bounded
wait), and the allocation-free column sum on a device other than 0.
Skipped on a single-GPU machine; the host logic of the exchange is also covered on CPU
by two gloo ranks (tests/test_sharding_gloo.py)."""

from __future__ import annotations

import os
from pathlib import Path
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys
sys.path[:0] = [r"{root}", r"{root}/helion-mlir-xsmm_b200", r"{root}/tests"]
import torch, torch.distributed as dist, torch.nn.functional as F
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
import helion_mlir_utils as ops
from helion_mlir_utils import sharding
from oracle import inputs, checks
from oracle import ops as ref
data = inputs.c2_linear(m=1024, n=768, k=512)
x = data["x"].cuda()
n0, n1 = sharding.shard_bounds(768, world, rank)
w, b = data["w"][n0:n1].contiguous().cuda(), data["b"][n0:n1].contiguous().cuda()
y = sharding.column_sharded_linear(x, w, b, 768, F.gelu)
expect = ref.linear(data["x"], data["w"], data["b"], F.gelu)
checks.assert_parity(torch.bfloat16, y.cpu(), expect, f"rank {{rank}} column-sharded linear")
whole = ops.matmul(x, data["w"].cuda(), trans_b=True, bias=data["b"].cuda(), epilogue=F.gelu)
assert torch.equal(y, whole), "the gathered shards are the unsharded result, bit for bit"
# the fused form: every rank's epilogue stores its columns into all copies of y over peer memory
from helion_mlir_backend import native
fused = sharding.FusedColumnShardedLinear(1024, 768, 512, torch.bfloat16, torch.device("cuda", rank))
for call in range(5):  # the two copies of y alternate
    yf = fused(x, w, b, F.gelu)
    torch.cuda.synchronize()
    assert torch.equal(yf, whole), f"fused call {{call}} on rank {{rank}}"
assert native.kernel_status() == 0, "a bounded wait ran out"
# back to back without host synchronisation, results used in stream order
acc = torch.zeros(1024, 768, device="cuda")
for call in range(6):
    acc += fused(x, w, b, F.gelu).float()
torch.cuda.synchronize()
assert torch.equal(acc, whole.float() * 6)
assert native.kernel_status() == 0
fused.close()
# ragged shares (770 columns over 2 ranks would be equal; 771 is not): the general gather
data = inputs.c2_linear(m=256, n=771, k=256)
n0, n1 = sharding.shard_bounds(771, world, rank)
y = sharding.column_sharded_linear(data["x"].cuda(), data["w"][n0:n1].contiguous().cuda(), data["b"][n0:n1].contiguous().cuda(), 771, F.gelu)
checks.assert_parity(torch.bfloat16, y.cpu(), ref.linear(data["x"], data["w"], data["b"], F.gelu), "ragged shares")
{extra}
dist.barrier()
dist.destroy_process_group()
print(f"rank {{rank}} ok")
"""


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(tmp_path: Path, world: int, extra: str = "") -> None:
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, extra=extra))
    env = {**os.environ, "MASTER_ADDR": "127.0.0.1", "NCCL_DEBUG": "WARN"}
    done = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)],
        capture_output=True, text=True, timeout=280, env=env,
    )
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    for rank in range(world):
        assert f"rank {rank} ok" in done.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_sharded_linear_over_nccl(tmp_path: Path) -> None:
    run_ranks(tmp_path, 2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_static_column_sum_on_the_second_device() -> None:
    """The fixed scratch array's device address is looked up per device: a first call on
    device 1 (with device 1 current) must not use device 0's address."""
    from helion_mlir_backend import native

    lib = native.module()
    dev = torch.device("cuda", 1)
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(20000, 96, generator=gen).to(dev)
    out = torch.full((96,), float("nan"), device=dev)
    with native.on_device(dev):
        rc = lib.b200_column_sum_static(native.F32, x.data_ptr(), out.data_ptr(), 20000, 96, 96, native.stream_ptr(dev))
    assert rc == 0, native.strerror(rc)
    torch.cuda.synchronize(dev)
    expect = x.double().sum(0).float()
    assert float(((out - expect).abs().max() / expect.abs().max())) < 1e-5
    x0 = x.to("cuda:0")
    out0 = torch.full((96,), float("nan"), device="cuda:0")
    with native.on_device(torch.device("cuda", 0)):
        assert lib.b200_column_sum_static(native.F32, x0.data_ptr(), out0.data_ptr(), 20000, 96, 96,
                                          native.stream_ptr(torch.device("cuda", 0))) == 0
    torch.cuda.synchronize()
    assert torch.equal(out0.cpu(), out.cpu())
