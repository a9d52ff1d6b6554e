"""Contracts of the native call path that the reference pins in tests/test_native_call.py,
restated for planned calls of the C ABI: a plan holds no data pointers, concurrent calls
from several threads are all correct and all counted, and operands may be one tensor."""

from __future__ import annotations

import threading

import pytest
import torch

from helpers import cuda
from oracle import checks
from oracle import ops as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


def test_plan_reads_the_current_storage(ops) -> None:
    """tests/test_native_call.py:162-173: storage swapped through ``set_`` or ``.data`` is what
    the next call reads (a plan records sizes and layouts, never addresses)."""
    gen = torch.Generator().manual_seed(5)
    a1, a2 = (torch.randn(256, 128, generator=gen).bfloat16() for _ in range(2))
    b = torch.randn(128, 192, generator=gen).bfloat16()
    x, w = cuda(a1, b)
    first = ops.matmul(x, w)
    checks.assert_parity(torch.bfloat16, first.cpu(), ref.matmul(a1, b), "first storage")
    x.data = a2.cuda()
    second = ops.matmul(x, w)
    checks.assert_parity(torch.bfloat16, second.cpu(), ref.matmul(a2, b), "after .data swap")
    x.set_(a1.cuda())
    third = ops.matmul(x, w)
    assert torch.equal(third, first)


def test_same_tensor_as_both_operands(ops) -> None:
    """tests/test_native_call.py:233-241 has the reference refuse to plan a call whose two
    arguments are one tensor; inputs may alias here (only the output may not), so the call
    runs natively and is right."""
    gen = torch.Generator().manual_seed(6)
    a = torch.randn(192, 192, generator=gen).bfloat16()
    x = a.cuda()
    checks.assert_parity(torch.bfloat16, ops.matmul(x, x).cpu(), ref.matmul(a, a), "a @ a")
    checks.assert_parity(torch.bfloat16, ops.matmul(x, x, trans_b=True).cpu(), ref.matmul(a, a.T.contiguous()), "a @ a^T")


def test_concurrent_calls_from_eight_threads_are_counted(ops) -> None:
    """tests/test_native_call.py:197-219: 8 threads x 25 calls, every result right, every
    call counted by the library."""
    from helion_mlir_backend import native

    gen = torch.Generator().manual_seed(7)
    a, b = torch.randn(384, 256, generator=gen).bfloat16(), torch.randn(256, 320, generator=gen).bfloat16()
    x, w = cuda(a, b)
    expect = ops.matmul(x, w)
    torch.cuda.synchronize()
    before = native.counters()
    wrong: list[int] = []

    def work(tag: int) -> None:
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(25):
                out = ops.matmul(x, w)
                stream.synchronize()
                if not torch.equal(out, expect):
                    wrong.append(tag)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    after = native.counters()
    assert not wrong
    assert after["calls"] - before["calls"] == 200 and after["launches"] - before["launches"] >= 200
    assert after["refusals"] == before["refusals"]
