"""The device-side reuse pool: the contracts tests/test_output_pool.py of the
reference pins for the CPU pool, restated for device blocks."""

from __future__ import annotations

import gc
import threading

import pytest
import torch

pytestmark = pytest.mark.gpu
MIB = 1 << 20


@pytest.fixture()
def pool():
    from helion_mlir_backend import output_pool

    output_pool.set_output_pool(2 << 30)
    gc.collect()
    output_pool.release()
    yield output_pool
    gc.collect()
    output_pool.release()
    output_pool.set_output_pool(2 << 30)


def test_freed_block_is_reused(pool) -> None:
    dev = torch.device("cuda", 0)
    t = pool.empty((8 * MIB,), dtype=torch.uint8, device=dev)
    pointer = t.data_ptr()
    before = pool.output_pool_stats()
    del t
    gc.collect()
    mid = pool.output_pool_stats()
    assert mid["free_blocks"] == before["free_blocks"] + 1
    u = pool.empty((2 * MIB,), dtype=torch.float32, device=dev)  # same bytes, other dtype
    after = pool.output_pool_stats()
    assert u.data_ptr() == pointer and after["hits"] == mid["hits"] + 1
    assert after["free_blocks"] == mid["free_blocks"] - 1


def test_plain_tensor_properties(pool) -> None:
    dev = torch.device("cuda", 0)
    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.bool, torch.float16):
        t = pool.empty((3, MIB, 2), dtype=dtype, device=dev)
        assert t.shape == (3, MIB, 2) and t.dtype == dtype and t.is_contiguous()
        assert not t._is_view() and not t.requires_grad and t.stride() == (2 * MIB, 2, 1)
        assert t.data_ptr() % 256 == 0
        t.fill_(1)
        assert bool((t == 1).all())
    like = pool.empty_like(torch.zeros(4 * MIB, device=dev), dtype=torch.bfloat16)
    assert like.shape == (4 * MIB,) and like.dtype == torch.bfloat16


def test_view_keeps_block_out_of_pool(pool) -> None:
    dev = torch.device("cuda", 0)
    t = pool.empty((8 * MIB,), dtype=torch.uint8, device=dev)
    view = t[: MIB]
    base = pool.output_pool_stats()["free_blocks"]
    del t
    gc.collect()
    assert pool.output_pool_stats()["free_blocks"] == base
    del view
    gc.collect()
    assert pool.output_pool_stats()["free_blocks"] == base + 1


def test_small_tensors_bypass(pool) -> None:
    before = pool.output_pool_stats()
    t = pool.empty((1024,), dtype=torch.float32, device=torch.device("cuda", 0))
    after = pool.output_pool_stats()
    assert (before["hits"], before["misses"]) == (after["hits"], after["misses"]) and t.numel() == 1024


def test_limits_and_eviction(pool) -> None:
    dev = torch.device("cuda", 0)
    pool.set_output_pool(16 * MIB)
    blocks = [pool.empty((6 * MIB,), dtype=torch.uint8, device=dev) for _ in range(4)]
    del blocks
    gc.collect()
    stats = pool.output_pool_stats()
    assert stats["free_bytes"] <= 16 * MIB and stats["free_blocks"] == 2
    big = pool.empty((15 * MIB,), dtype=torch.uint8, device=dev)  # takes the pool path (<= limit)
    del big
    gc.collect()
    assert pool.output_pool_stats()["free_bytes"] <= 16 * MIB
    live = pool.empty((6 * MIB,), dtype=torch.uint8, device=dev)
    live.fill_(7)
    pool.set_output_pool(0)
    assert not pool.enabled() and pool.output_pool_stats()["free_blocks"] == 0
    assert int(live[0]) == 7  # live tensors survive
    t = pool.empty((6 * MIB,), dtype=torch.uint8, device=dev)  # pool off: torch's allocator
    assert t.numel() == 6 * MIB
    pool.set_output_pool(1 << 40)
    many = [pool.empty((4 * MIB,), dtype=torch.uint8, device=dev) for _ in range(70)]
    del many
    gc.collect()
    assert pool.output_pool_stats()["free_blocks"] <= 64


def test_reused_block_is_fully_overwritten(pool) -> None:
    import helion_mlir_utils as ops

    x = torch.randn(2048, 1024, device="cuda")
    first = ops.softmax(x)
    expect = first.clone()
    first.fill_(float("nan"))
    pointer = first.data_ptr()
    del first
    gc.collect()
    second = ops.softmax(x)
    assert second.data_ptr() == pointer and torch.equal(second, expect)


def test_threads_never_share_a_block(pool) -> None:
    dev = torch.device("cuda", 0)
    errors: list[str] = []

    def work(tag: int) -> None:
        for _ in range(50):
            t = pool.empty((4 * MIB,), dtype=torch.uint8, device=dev)
            t.fill_(tag)
            torch.cuda.current_stream().synchronize()
            if not bool((t == tag).all()):
                errors.append(f"thread {tag} saw foreign data")

    threads = [threading.Thread(target=work, args=(i + 1,)) for i in range(8)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors


def test_other_stream_waits_for_pending_work(pool) -> None:
    dev = torch.device("cuda", 0)
    side = torch.cuda.Stream()
    t = pool.empty((64 * MIB,), dtype=torch.uint8, device=dev)
    pointer = t.data_ptr()
    for _ in range(20):
        t.add_(1)  # work pending on the current stream when the block is freed
    del t
    gc.collect()
    with torch.cuda.stream(side):
        u = pool.empty((64 * MIB,), dtype=torch.uint8, device=dev)
        # Either the pending work had finished (same block) or a fresh block was taken: never a race.
        if u.data_ptr() == pointer:
            assert torch.cuda.current_stream() == side
    torch.cuda.synchronize()
