"""The five benchmark configurations at their full sizes against the oracle.

Reduced sizes run other launch plans than the benchmark does (one K chunk instead
of parallel chunks plus the ordered reduction for C1, no peeled tail batches for
C5, no raster groups for C3), so every configuration is also checked at the size it
is timed at, on samples the oracle finishes in seconds (``oracle/sampled.py``).
Tolerances: relative Frobenius error <= 1e-5 for f32 results, max-abs error
<= 1e-2 * max|ref| for bf16 results (the reference's own bars:
``tests/test_cpu_utils_f32_fused.py:58-140``, ``tests/test_cpu_utils_split_k_bmm.py:33-69``,
``tests/test_cpu_utils_softmax.py:18-76``).
"""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from helpers import cuda
from oracle import inputs, sampled
from oracle import ops as ref

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


def _passes(report: dict[str, object]) -> None:
    assert report["parity_pass"], report


def test_c1_f32_1024_whole(ops) -> None:
    """1024^3 f32 with block_sizes=[64,64,64]: the widened product runs as parallel K
    chunks with an ordered reduction at this size only."""
    data = inputs.c1_f32_matmul(1024)
    a, b = cuda(data["a"], data["b"])
    text = str(ops.matmul.explain(a, b, block_sizes=(64, 64, 64)))
    assert "umma" in text, text
    out = ops.matmul(a, b, block_sizes=(64, 64, 64))
    _passes(sampled.c1_whole(data["a"], data["b"], out))
    assert torch.equal(out, ops.matmul(a, b, block_sizes=(64, 64, 64)))  # ordered reduction: same bits every run
    from helion_mlir_backend import graphed

    call = graphed(lambda p, q: ops.matmul(p, q, block_sizes=(64, 64, 64)), a, b)
    assert torch.equal(call(), out)  # the replayed graph (what the benchmark times) gives the same bits


def test_c2_linear_8192_rows(ops) -> None:
    data = inputs.c2_linear()
    x, w, b = cuda(data["x"], data["w"], data["b"])
    rows = sampled.rows_of_interest(8192)
    y = ops.matmul(x, w, trans_b=True, bias=b, epilogue=F.gelu)
    _passes(sampled.c2_rows(data["x"], data["w"], data["b"], y[rows.cuda()], rows))
    layer = torch.nn.Linear(4096, 4096, dtype=BF16, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(w)
        layer.bias.copy_(b)
    y2, cache = ops.linear(x, layer, F.gelu, cache=None)
    assert torch.equal(y2, y)  # the layer entry point runs the same kernel on the same operands
    y3, _ = ops.linear(x, layer, F.gelu, cache=cache)
    assert torch.equal(y3, y)


def test_c3_blocked_vnni_8192_rows(ops) -> None:
    """8192^3: B (128 MB) exceeds the raster threshold, so tiles walk groups of 16 tile
    rows; the samples sit either side of the group boundary (row 4096) and in the tile
    rows whose last columns the final, partly filled round computes."""
    size = 8192
    data = inputs.c3_blocked(size)
    a, b = cuda(data["a"], data["b"])
    a4, b5 = ops.pack_a_blocked(a), ops.pack_b_blocked_vnni(b)
    assert tuple(a4.shape) == (256, 256, 32, 32) and tuple(b5.shape) == (256, 256, 16, 32, 2)
    del a, b
    out = ops.matmul_blocked(a4, b5, size, size, size, out_dtype=F32)
    assert out.dtype == F32 and tuple(out.shape) == (size, size)
    rows = sampled.rows_of_interest(size, extra=12)
    _passes(sampled.c3_rows(data["a"][rows], data["b"], out[rows.cuda()], size))
    # every tile was written: a checksum of all rows against the same sum of the sampled expectation's columns
    # would need the whole product; instead no element may be left at the pool's fill value
    assert bool(torch.isfinite(out).all())
    assert torch.equal(out, ops.matmul_blocked(a4, b5, size, size, size, out_dtype=F32))


@pytest.mark.parametrize("dtype", [F32, BF16], ids=["f32", "bf16"])
def test_c4_rows_32768x4096(ops, dtype: torch.dtype) -> None:
    m, n = 32768, 4096
    data = inputs.c4_rows(m, n)
    x = data["x"].to(dtype)
    gamma, beta = data["gamma"].to(dtype), data["beta"].to(dtype)
    dx, dg, db = cuda(x, gamma, beta)
    rows = sampled.rows_of_interest(m, tile_rows=148, group_tiles=64, extra=40)
    pick = rows.cuda()
    soft = ops.softmax(dx)
    run = {
        "softmax": soft[pick],
        "layer_norm": ops.layer_norm(dx, dg, db, 1e-5)[pick],
        "rms_norm": ops.rms_norm(dx, dg, 1e-5)[pick],
        "chained": ops.layer_norm(soft, dg, db, 1e-5)[pick],
    }
    _passes(sampled.c4_rows(x[rows], gamma, beta, run, m))
    # size-independent: every row of a softmax sums to one
    sums = soft.float().sum(-1)
    assert float((sums - 1).abs().max()) < (1e-5 if dtype == F32 else 2e-2)


def test_c5_split_k_bmm_full(ops) -> None:
    """64 x 512 x 512 x 16384, split_k=8: 256 pair tiles on 74 CTA pairs; the batches of
    the last round run as a second launch with narrower tiles. Whole batches are checked
    from the head, either side of the head / tail boundary, and the very last one."""
    data = inputs.c5_split_k_bmm()
    a, b = cuda(data["a"], data["b"])
    text = str(ops.bmm.explain(a, b, split_k=8, out_dtype=F32)) if hasattr(ops.bmm, "explain") else ""
    out = ops.bmm(a, b, split_k=8, out_dtype=F32)
    assert out.dtype == F32 and tuple(out.shape) == (64, 512, 512)
    batches = [0, 54, 55, 63]
    _passes(sampled.c5_batches(data["a"][batches], data["b"][batches], out[batches], batches, 64))
    # sampled rows of every other batch (a batch the samples above skip would otherwise go unseen)
    rows = torch.tensor([0, 255, 256, 511])
    expect = torch.stack([ref.matmul_split_k(data["a"][i][rows], data["b"][i], 8, F32) for i in range(0, 64, 7)])
    got = out[0:64:7][:, rows.cuda()]
    from oracle import checks

    assert checks.rel_frobenius(got.cpu(), expect) <= 1e-5, text
    assert torch.equal(out, ops.bmm(a, b, split_k=8, out_dtype=F32))  # fixed order: same bits every run
