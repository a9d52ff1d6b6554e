"""Launch plans of the row-wise operators and the reductions, pinned as the reference pins its tile heuristics
(exact values: ``tests/test_cpu_utils_prepacked.py:392-510`` for ``vnni_panel`` and
``whole_row_tiles``). ``explain()`` of softmax / layer_norm / rms_norm / group_norm and of row_sum / row_dot / matvec /
column_sum is host arithmetic in the library (``b200_rowwise_explain``, ``b200_reduce_explain``),
so it runs without a GPU on CPU tensors of the same shape and type."""

from __future__ import annotations

import pytest
import torch

F32, BF16 = torch.float32, torch.bfloat16

PLANS = {
    # rows that a power-of-two number of threads covers
    ("softmax", 4096, F32, None): "rowwise_lean_kernel: 256 threads x 16 values per row, 1 rows per CTA of 256 threads",
    ("softmax", 4096, BF16, None): "rowwise_lean_kernel: 128 threads x 32 values per row, 2 rows per CTA of 256 threads",
    ("softmax", 128, F32, None): "rowwise_lean_kernel: 8 threads x 16 values per row, 32 rows per CTA of 256 threads",
    ("softmax", 16384, BF16, None): "rowwise_lean_kernel: 256 threads x 64 values per row, 1 rows per CTA of 256 threads",
    ("softmax", 32768, BF16, None): "rowwise_lean_kernel: 512 threads x 64 values per row, 1 rows per CTA of 512 threads",
    # whole warps that cover the row exactly, and covers with a tail
    ("softmax", 768, F32, None): "rowwise_lean_kernel: 32 threads x 24 values per row, 8 rows per CTA of 256 threads",
    ("softmax", 12288, BF16, None): "rowwise_lean_kernel: 192 threads x 64 values per row, 1 rows per CTA of 192 threads",
    ("softmax", 11008, F32, None): "rowwise_lean_kernel: 352 threads x 32 values per row, 1 rows per CTA of 352 threads, tail",
    ("softmax", 20000, BF16, None): "rowwise_lean_kernel: 320 threads x 64 values per row, 1 rows per CTA of 320 threads, tail",
    # beyond the registers of 512 threads; rows without 16-byte accesses
    ("softmax", 50304, F32, None): "rowwise_long_kernel: one CTA of 1024 threads per row, 2 sweeps, 16-byte accesses",
    ("softmax", 32776, BF16, None): "rowwise_long_kernel: one CTA of 1024 threads per row, 2 sweeps, 16-byte accesses",
    ("softmax", 129, F32, None): "rowwise_kernel (masked, element accesses): 16 threads x 16 values per row, 16 rows per CTA of 256 threads",
    # the norms: bf16 rows kept in 16 bits, two rows per group with f32 parameters
    ("layer_norm", 4096, F32, F32): "rowwise_lean_kernel: 256 threads x 16 values per row, 1 rows per CTA of 256 threads",
    ("layer_norm", 4096, BF16, BF16): "rowwise_lean_kernel: 128 threads x 32 values per row, 2 rows per CTA of 256 threads, row kept in 16 bits",
    ("layer_norm", 4096, BF16, F32): "rowwise_pair_kernel: two rows per group of 256 threads x 16 values, 1 groups per CTA of 256 threads",
    ("layer_norm", 1000, BF16, F32): "rowwise_pair_kernel: two rows per group of 64 threads x 16 values, 4 groups per CTA of 256 threads, tail",
    ("layer_norm", 8192, BF16, F32): "rowwise_lean_kernel: 256 threads x 32 values per row, 1 rows per CTA of 256 threads, row kept in 16 bits",
    ("layer_norm", 11008, BF16, BF16): "rowwise_lean_kernel: 192 threads x 64 values per row, 1 rows per CTA of 192 threads, tail, row kept in 16 bits",
    ("layer_norm", 25600, BF16, BF16): "rowwise_lean_kernel: 416 threads x 64 values per row, 1 rows per CTA of 416 threads, tail, row kept in 16 bits",
    ("rms_norm", 4096, BF16, BF16): "rowwise_lean_kernel: 128 threads x 32 values per row, 2 rows per CTA of 256 threads, row kept in 16 bits",
    ("rms_norm", 768, BF16, BF16): "rowwise_lean_kernel: 32 threads x 24 values per row, 8 rows per CTA of 256 threads",
    ("rms_norm", 50304, BF16, BF16): "rowwise_long_kernel: one CTA of 1024 threads per row, 2 sweeps, 16-byte accesses",
}


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


@pytest.mark.parametrize("case", list(PLANS), ids=[f"{op}-{n}-{str(dt)[6:]}-{str(pd)[6:] if pd else 'none'}" for op, n, dt, pd in PLANS])
def test_row_plan(ops, case) -> None:
    op, n, dtype, param_dtype = case
    x = torch.zeros(4, n, dtype=dtype)
    if op == "softmax":
        plan = ops.softmax.explain(x)
    elif op == "layer_norm":
        plan = ops.layer_norm.explain(x, torch.zeros(n, dtype=param_dtype), torch.zeros(n, dtype=param_dtype))
    else:
        plan = ops.rms_norm.explain(x, torch.zeros(n, dtype=param_dtype))
    assert plan.native and plan.kernel == PLANS[case]


def test_group_norm_plans(ops) -> None:
    x, w = torch.zeros(4, 4096), torch.zeros(4096)
    # 32 groups of 128 values: rows of 128 that share warps
    assert ops.group_norm.explain(x, 32, w, w, 1e-5).kernel == PLANS[("softmax", 128, F32, None)]
    # an activation after the norm is fused, but in the masked kernel
    assert ops.group_norm.explain(x, 1, w, w, 1e-5, torch.relu).kernel.startswith("rowwise_kernel (masked)")
    # an epilogue the kernels do not know runs as its own pass
    unknown = ops.group_norm.explain(x, 1, w, w, 1e-5, lambda y, e: y * torch.tanh(e), w)
    assert unknown.native and "own device pass" in unknown.kernel


def test_explain_goes_through_the_backend_entry(ops) -> None:
    from helion_mlir_backend import explain

    assert str(explain(ops.softmax, torch.zeros(4, 4096))) == "native: " + PLANS[("softmax", 4096, F32, None)]
    refused = ops.softmax.explain(torch.zeros(4, 8, dtype=torch.float64))
    assert not refused.native and "f32 or bf16" in str(refused)


REDUCTIONS = {
    # (m, n, dtype): (row_sum, row_dot with an f32 vector, matvec)
    (64, 4096, F32): ("row_reduce_kernel: 128 threads per row, 2 rows per CTA of 256 threads, 16-byte accesses",) * 3,
    (64, 4096, BF16): (
        "row_reduce_kernel: 64 threads per row, 4 rows per CTA of 256 threads, 16-byte accesses",
        "row_dot_rows_kernel (four rows per group of threads): 64 threads per row, 16 rows per CTA of 256 threads, 16-byte accesses",
        "row_reduce_kernel: 64 threads per row, 4 rows per CTA of 256 threads, 16-byte accesses",
    ),
    (64, 64, BF16): (
        "row_reduce_kernel: 4 threads per row, 64 rows per CTA of 256 threads, 16-byte accesses",
        "row_dot_rows_kernel (four rows per group of threads): 4 threads per row, 256 rows per CTA of 256 threads, 16-byte accesses",
        "row_reduce_kernel: 4 threads per row, 64 rows per CTA of 256 threads, 16-byte accesses",
    ),
    (64, 333, F32): ("row_reduce_kernel: 64 threads per row, 4 rows per CTA of 256 threads, element accesses",) * 3,
    (64, 12288, F32): ("row_reduce_kernel: 256 threads per row, 1 rows per CTA of 256 threads, 16-byte accesses",) * 3,
}

COLUMN_SUMS = {
    (32768, 4096, BF16): "column_partial_kernel: 8 strips of 512 columns (8 per thread) x 128 chunks of 256 rows, then "
                         "column_final_kernel adds the chunks in order (2097152 bytes of scratch)",
    (1 << 20, 64, BF16): "column_partial_kernel: 1 strips of 64 columns (8 per thread) x 1024 chunks of 1024 rows, then "
                         "column_final_kernel adds the chunks in order (262144 bytes of scratch)",
    (1, 4096, F32): "column_partial_kernel: 8 strips of 512 columns (4 per thread), one chunk of 1 rows",
    (100, 333, F32): "column_partial_kernel: 3 strips of 128 columns (1 per thread), one chunk of 100 rows",
}


@pytest.mark.parametrize("shape", list(REDUCTIONS), ids=[f"{m}x{n}-{str(dt)[6:]}" for m, n, dt in REDUCTIONS])
def test_row_reduction_plans(ops, shape) -> None:
    m, n, dtype = shape
    x = torch.zeros(m, n, dtype=dtype)
    got = (ops.row_sum.explain(x).kernel, ops.row_dot.explain(x, torch.zeros(n)).kernel,
           ops.matvec.explain(x, torch.zeros(n, 1, dtype=dtype)).kernel)
    assert got == REDUCTIONS[shape]


@pytest.mark.parametrize("shape", list(COLUMN_SUMS), ids=[f"{m}x{n}-{str(dt)[6:]}" for m, n, dt in COLUMN_SUMS])
def test_column_sum_plans(ops, shape) -> None:
    """The scratch the plan names is what ``b200_column_sum_workspace_bytes`` asks for at most
    (the query does not know the operand's alignment and takes the largest of the three vector widths)."""
    from helion_mlir_backend import native

    m, n, dtype = shape
    plan = ops.column_sum.explain(torch.zeros(m, n, dtype=dtype))
    assert plan.native and plan.kernel == COLUMN_SUMS[shape]
    need = int(native.module().b200_column_sum_workspace_bytes(m, n))
    if "bytes of scratch" in plan.kernel:
        assert int(plan.kernel.split("(")[-1].split(" bytes")[0]) <= need
