"""Full-size parity through samples (test infrastructure).

At the benchmark's own sizes the CPU restatement cannot compute a whole result in
seconds, but rows of a GEMM, batches of a batched GEMM and rows of the row-wise
operators are independent of one another: the expectation of a sample of them is
the restatement run on that sample alone. The samples here are placed where the
launch plans of the full sizes differ from those of reduced ones: first and last
rows of tiles, the rows either side of a raster-group boundary, rows and columns
that the last round of tiles computes, the batches a second launch takes.

Every function returns ``{"parity_metric", "parity_value", "parity_bound",
"parity_pass", "checked"}``; the bars are those of :mod:`oracle.checks`: relative
Frobenius error 1e-5 for f32 paths (f32 operands), max-abs 1e-2 of max|ref| for bf16
paths with f32 accumulation (bf16 operands, whatever the result type). For bf16 operands
with an f32 result (C3, C5) the relative Frobenius error is reported beside the bar's own
metric (``rel_frobenius``) and held to ``F32_RESULT_OF_BF16_FROBENIUS``: the tensor core's
f32 accumulation truncates, an error that grows with the length of one running sum
(9e-6 at K = 8192 unsplit, 2e-6 with ordered chunks of 2048).
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor
import torch.nn.functional as F

from . import checks
from . import ops as ref


F32_RESULT_OF_BF16_FROBENIUS = 3e-5


def _report(dtype: torch.dtype, actual: Tensor, expect: Tensor, checked: str, frobenius_too: bool = False) -> dict[str, object]:
    """``dtype`` is the operand type, which names the bar; ``frobenius_too`` adds the relative
    Frobenius error of an f32 result of bf16 operands and holds it to its own ceiling."""
    actual, expect = actual.detach().cpu(), expect.detach().cpu()
    same_nans = bool(torch.equal(actual.isnan(), expect.isnan()))
    keep = ~expect.isnan()
    error, bound = checks.metric_for(dtype, actual[keep], expect[keep])
    report = {
        "parity_metric": "rel_frobenius" if dtype == torch.float32 else "max_abs_over_max_ref",
        "parity_value": error,
        "parity_bound": bound,
        "parity_pass": bool(same_nans and error <= bound),
        "checked": checked,
    }
    if frobenius_too:
        frobenius = checks.rel_frobenius(actual[keep], expect[keep])
        report["rel_frobenius"] = frobenius
        report["rel_frobenius_ceiling"] = F32_RESULT_OF_BF16_FROBENIUS
        report["parity_pass"] = bool(report["parity_pass"] and frobenius <= F32_RESULT_OF_BF16_FROBENIUS)
    return report


def worst(reports: list[dict[str, object]]) -> dict[str, object]:
    """One report for several: the largest error relative to its bound."""
    top = max(reports, key=lambda r: float(r["parity_value"]) / float(r["parity_bound"]))
    merged = dict(top)
    merged["parity_pass"] = all(bool(r["parity_pass"]) for r in reports)
    merged["checked"] = "; ".join(str(r["checked"]) for r in reports)
    return merged


def rows_of_interest(m: int, tile_rows: int = 256, group_tiles: int = 16, extra: int = 8, seed: int = 7) -> Tensor:
    """Row indices: both ends of the first and last tile, either side of every
    raster-group boundary (``group_tiles`` tiles of ``tile_rows`` rows), and a few
    seeded others."""
    rows = {0, 1, tile_rows - 1, tile_rows, m - tile_rows, m - 2, m - 1, m // 2 - 1, m // 2}
    group = tile_rows * group_tiles
    for edge in range(group, m, group):
        rows.update({edge - 1, edge})
    gen = torch.Generator().manual_seed(seed)
    rows.update(int(i) for i in torch.randint(0, m, (extra,), generator=gen))
    return torch.tensor(sorted(r for r in rows if 0 <= r < m))


def c1_whole(a: Tensor, b: Tensor, out: Tensor) -> dict[str, object]:
    """C1: the whole f32 1024^3 product (an f64 product of that size takes a fraction of a second)."""
    return _report(torch.float32, out, ref.matmul(a, b), f"whole {tuple(out.shape)} result")


def c2_rows(x: Tensor, w: Tensor, b: Tensor, y_rows: Tensor, rows: Tensor) -> dict[str, object]:
    """C2: sampled rows of y = GELU(x W^T + b), every column."""
    expect = ref.linear(x[rows], w, b, F.gelu)
    return _report(torch.bfloat16, y_rows, expect, f"{len(rows)} of {x.shape[0]} rows, all columns")


def c3_rows(a_rows: Tensor, b: Tensor, out_rows: Tensor, total_rows: int) -> dict[str, object]:
    """C3: sampled rows of the f32 product of the blocked operands, every column.
    ``a_rows`` are the sampled rows of the unpacked A, ``b`` the unpacked B."""
    expect = ref.matmul(a_rows, b, out_dtype=torch.float32)
    return _report(torch.bfloat16, out_rows, expect, f"{a_rows.shape[0]} of {total_rows} rows, all columns", frobenius_too=True)


def c4_rows(x_rows: Tensor, gamma: Tensor, beta: Tensor, run: dict[str, Tensor], total_rows: int) -> dict[str, object]:
    """C4: sampled rows of softmax, layer_norm, rms_norm (and layer_norm(softmax(x)) when
    ``run`` holds ``chained``) in the type of ``x_rows``."""
    dtype = x_rows.dtype
    expect: dict[str, Callable[[], Tensor]] = {
        "softmax": lambda: ref.softmax(x_rows),
        "layer_norm": lambda: ref.layer_norm(x_rows, gamma, beta, 1e-5),
        "rms_norm": lambda: ref.rms_norm(x_rows, gamma, 1e-5),
        "chained": lambda: ref.layer_norm(ref.softmax(x_rows), gamma, beta, 1e-5),
    }
    name = "f32" if dtype == torch.float32 else "bf16"
    reports = [
        _report(dtype, run[key], expect[key](), f"{key} {name}: {x_rows.shape[0]} of {total_rows} rows")
        for key in run
    ]
    return worst(reports)


def c5_batches(a: Tensor, b: Tensor, out: Tensor, batches: list[int], total: int, split_k: int = 8) -> dict[str, object]:
    """C5: whole sampled batches of the ordered split-K product (f32 result).
    ``a``, ``b``, ``out`` hold the sampled batches only."""
    expect = ref.bmm(a, b, split_k=split_k, out_dtype=torch.float32)
    return _report(torch.bfloat16, out, expect, f"batches {batches} of {total}, whole", frobenius_too=True)
