"""The allocation-free column sum (``b200_column_sum_static``) against the
ordinary entry point, through the C ABI.

Some hosts cannot give the library memory at call time: their device memory is
budgeted to the last block at start-up, or they sit on a path where an allocation's
device-wide synchronisation is not acceptable. For them the partial sums of the
two-stage column sum live in a fixed array inside the library. This file runs last
(pytest collects files alphabetically) so that a failure here cannot hide others;
it passes alone in a fresh process as well as after the rest of the suite.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def column_sum_both(lib, native, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    m, n = x.shape
    stream = native.stream_ptr(x.device)
    dtype = native.dtype_code(x.dtype)
    need = int(lib.b200_column_sum_workspace_bytes(m, n))
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=x.device)
    expected = torch.full((n,), float("nan"), device=x.device)
    rc = lib.b200_column_sum(dtype, x.data_ptr(), expected.data_ptr(), m, n, n, scratch.data_ptr(), need, stream)
    assert rc == 0, native.strerror(rc)
    actual = torch.full((n,), float("nan"), device=x.device)
    rc = lib.b200_column_sum_static(dtype, x.data_ptr(), actual.data_ptr(), m, n, n, stream)
    assert rc == 0, native.strerror(rc)
    return actual, expected


def test_static_scratch_matches_ordinary_entry_point_twice() -> None:
    from helion_mlir_backend import native

    lib = native.module()
    gen = torch.Generator().manual_seed(77)
    # Two calls in a row on different shapes: the second finds the first one's leftovers in the array.
    first = torch.randn(20000, 96, generator=gen).cuda()  # many row chunks: the partial sums are used
    second = torch.randn(9000, 520, generator=gen).bfloat16().cuda()
    assert lib.b200_column_sum_workspace_bytes(20000, 96) > 0
    for x in (first, second, first):
        actual, expected = column_sum_both(lib, native, x)
        torch.cuda.synchronize()
        # Same kernels, same plan, same summation order: the same bits.
        assert torch.equal(actual, expected)
        reference = x.double().sum(0).float()
        assert ((actual - reference).abs().max() / reference.abs().max()).item() < 1e-5
    one_row = torch.tensor([[-0.0, 2.5, -1.0]], device="cuda")
    actual, expected = column_sum_both(lib, native, one_row)
    assert torch.equal(actual, expected)


def test_limit_and_refusals() -> None:
    from helion_mlir_backend import native

    lib = native.module()
    limit = 2 << 20  # B200_COLUMN_SUM_STATIC_MAX_BYTES
    # The fixed array holds the partial sums of every shape under the present plan ...
    worst = max(
        int(lib.b200_column_sum_workspace_bytes(m, n))
        for m in (1, 64, 4096, 37888, 1 << 20, 1 << 24)
        for n in (1, 96, 443, 512, 1024, 4096, 65536, 1 << 20)
    )
    assert 0 < worst <= limit
    # ... and other bad arguments are refused before anything is launched.
    x = torch.zeros(8, device="cuda")
    out = torch.zeros(8, device="cuda")
    stream = native.stream_ptr(x.device)
    assert lib.b200_column_sum_static(9, x.data_ptr(), out.data_ptr(), 4, 2, 2, stream) == 1
    assert lib.b200_column_sum_static(native.F32, None, out.data_ptr(), 4, 2, 2, stream) == 6
    assert lib.b200_column_sum_static(native.F32, x.data_ptr(), out.data_ptr(), 4, 2, 1, stream) == 3
    assert "capacity" in native.strerror(11)
