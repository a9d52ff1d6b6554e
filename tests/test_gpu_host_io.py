"""Row-streamed calls on pinned host buffers: same bits as the direct device call,
for ragged chunkings, repeated calls, and a second stream."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_library):
    import helion_mlir_utils

    return helion_mlir_utils


def test_linear_rows_match_direct_call(ops) -> None:
    gen = torch.Generator().manual_seed(41)
    x = torch.randn(1000, 256, generator=gen).bfloat16().pin_memory()
    w = (torch.randn(192, 256, generator=gen) / 16).bfloat16().cuda()
    b = torch.randn(192, generator=gen).bfloat16().cuda()

    def fn(rows: torch.Tensor) -> torch.Tensor:
        return ops.matmul(rows, w, trans_b=True, bias=b, epilogue=F.gelu)

    direct = fn(x.cuda()).cpu()
    for chunk in (None, 256, 300, 1000, 4096):  # default, even, ragged, one chunk, larger than the rows
        out = torch.full((1000, 192), float("nan"), dtype=torch.bfloat16).pin_memory()
        assert ops.stream_rows(fn, x, out, chunk_rows=chunk) is out
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out, direct), chunk


def test_repeated_calls_and_other_stream(ops) -> None:
    gen = torch.Generator().manual_seed(42)
    xs = [torch.randn(2048, 512, generator=gen).pin_memory() for _ in range(3)]
    outs = [torch.empty(2048, 512).pin_memory() for _ in range(3)]
    side = torch.cuda.Stream()
    for i, (x, out) in enumerate(zip(xs, outs)):  # back to back, no host sync in between
        if i == 1:
            with torch.cuda.stream(side):
                ops.stream_rows(ops.softmax, x, out, chunk_rows=256, depth=2)
        else:
            ops.stream_rows(ops.softmax, x, out, chunk_rows=256, depth=2)
    torch.cuda.synchronize()
    for x, out in zip(xs, outs):
        assert torch.equal(out, ops.softmax(x.cuda()).cpu())


def test_rejects_what_it_cannot_stream(ops) -> None:
    x = torch.zeros(8, 4)
    with pytest.raises(ValueError, match="pinned"):
        ops.stream_rows(ops.softmax, x, x.clone())
    pinned = x.pin_memory()
    with pytest.raises(ValueError, match="row counts"):
        ops.stream_rows(ops.softmax, pinned, torch.zeros(9, 4).pin_memory())
    with pytest.raises(ValueError, match="host tensors"):
        ops.stream_rows(ops.softmax, pinned.cuda(), pinned)
    with pytest.raises(ValueError, match="depth"):
        ops.stream_rows(ops.softmax, pinned, torch.zeros(8, 4).pin_memory(), depth=1)
    empty = torch.zeros(0, 4).pin_memory()
    assert ops.stream_rows(ops.softmax, empty, torch.zeros(0, 4).pin_memory()).shape == (0, 4)


def test_matmul_host_matches_device_call(ops) -> None:
    gen = torch.Generator().manual_seed(43)
    x = torch.randn(1500, 256, generator=gen).bfloat16().pin_memory()
    w = (torch.randn(320, 256, generator=gen) / 16).bfloat16().cuda()
    b = torch.randn(320, generator=gen).bfloat16().cuda()
    direct = ops.matmul(x.cuda(), w, trans_b=True, bias=b, epilogue=F.gelu).cpu()
    for chunk in (None, 256, 700, 1500):
        out = torch.full((1500, 320), float("nan"), dtype=torch.bfloat16).pin_memory()
        assert ops.matmul_host(x, w, out, trans_b=True, bias=b, epilogue=F.gelu, chunk_rows=chunk) is out
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out, direct), chunk
    # back to back without a host sync, changing chunk sizes (the ring is re-carved), f32 result
    outs = [torch.empty(1500, 320).pin_memory() for _ in range(4)]
    for out, chunk in zip(outs, (256, 512, 256, 1024)):
        ops.matmul_host(x, w, out, trans_b=True, out_dtype=torch.float32, chunk_rows=chunk)
    torch.cuda.synchronize()
    want = ops.matmul(x.cuda(), w, trans_b=True, out_dtype=torch.float32).cpu()
    for out in outs:
        assert torch.equal(out, want)
    # allocates a pinned result when none is given; f32 operands take the widened path
    a32 = torch.randn(512, 384, generator=gen).pin_memory()
    b32 = torch.randn(384, 256, generator=gen).cuda()
    got = ops.matmul_host(a32, b32)
    torch.cuda.current_stream().synchronize()
    assert got.is_pinned() and torch.equal(got, ops.matmul(a32.cuda(), b32).cpu())


def test_matmul_host_refusals(ops) -> None:
    x = torch.zeros(64, 64, dtype=torch.bfloat16).pin_memory()
    w = torch.zeros(64, 64, dtype=torch.bfloat16).cuda()
    with pytest.raises(ValueError, match="host a_host"):
        ops.matmul_host(x.cuda(), w)
    with pytest.raises(ValueError, match="contracted"):
        ops.matmul_host(x, torch.zeros(32, 64, dtype=torch.bfloat16).cuda())
    with pytest.raises(ValueError, match="fuses"):
        ops.matmul_host(x, w, epilogue=lambda t: t * 3)
    with pytest.raises(ValueError, match="out_host"):
        ops.matmul_host(x, w, torch.zeros(64, 32, dtype=torch.bfloat16).pin_memory())


def test_chained_host_calls_read_the_first_result(ops) -> None:
    """The result of one matmul_host call (in host memory) as the input of the next,
    with no host synchronisation in between: the second call's copy-in must wait for the
    first call's copy-out of the rows it reads. Compared with the device path."""
    gen = torch.Generator().manual_seed(43)
    m, k, n1, n2 = 4096, 1024, 2048, 512
    x = torch.randn(m, k, generator=gen).bfloat16().pin_memory()
    w1 = (torch.randn(n1, k, generator=gen) / 32).bfloat16().cuda()
    w2 = (torch.randn(n2, n1, generator=gen) / 32).bfloat16().cuda()
    expect = ops.matmul(ops.matmul(x.cuda(), w1, trans_b=True, epilogue=torch.relu), w2, trans_b=True, epilogue=torch.relu).cpu()
    for round_ in range(3):  # the staging ring and the copy streams persist between rounds
        hidden = torch.full((m, n1), float("nan"), dtype=torch.bfloat16).pin_memory()
        out = torch.full((m, n2), float("nan"), dtype=torch.bfloat16).pin_memory()
        ops.matmul_host(x, w1, hidden, trans_b=True, epilogue=torch.relu, chunk_rows=512)
        ops.matmul_host(hidden, w2, out, trans_b=True, epilogue=torch.relu, chunk_rows=512)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out, expect), round_
