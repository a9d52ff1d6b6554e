"""The device-side reuse pool: the contracts tests/test_output_pool.py of the
reference pins for the CPU pool, restated for device blocks."""

from __future__ import annotations

import ctypes
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


def test_blocks_are_whole_aligned_2mib_units(pool) -> None:
    """tests/test_output_pool.py:157-169: blocks of 2 MiB and more are aligned to 2 MiB and
    accounted in whole 2 MiB units."""
    dev = torch.device("cuda", 0)
    pool.set_output_pool(64 * MIB)
    base = pool.output_pool_stats()["free_bytes"]
    t = pool.empty((4 * MIB,), dtype=torch.uint8, device=dev)
    assert t.data_ptr() % (2 * MIB) == 0
    del t
    gc.collect()
    assert pool.output_pool_stats()["free_bytes"] == base + 4 * MIB
    u = pool.empty((4 * MIB + 128 * 1024,), dtype=torch.uint8, device=dev)  # rounded up to 6 MiB
    assert u.data_ptr() % (2 * MIB) == 0
    del u
    gc.collect()
    assert pool.output_pool_stats()["free_bytes"] == base + 10 * MIB


def test_free_block_count_is_bounded_at_64(pool) -> None:
    """tests/test_output_pool.py:214-220: 70 blocks freed, 64 kept."""
    dev = torch.device("cuda", 0)
    pool.set_output_pool(1 << 40)
    held = [pool.empty((4 * MIB,), dtype=torch.uint8, device=dev) for _ in range(70)]
    del held
    gc.collect()
    stats = pool.output_pool_stats()
    assert stats["free_blocks"] == 64 and stats["free_bytes"] == 64 * 4 * MIB


def test_pooled_tensor_behaves_as_a_tensor(pool) -> None:
    """tests/test_output_pool.py:238-258: a pooled storage shrinks but cannot grow, never
    requires grad, and is an inference tensor under inference mode."""
    dev = torch.device("cuda", 0)
    held = pool.empty((1024, 1024), dtype=torch.float32, device=dev)
    held.fill_(3)
    held.resize_(512, 1024)  # within the block
    assert float(held[0, 0]) == 3
    with pytest.raises(RuntimeError, match="not resizable"):
        held.resize_(4096, 4096)
    assert not pool.empty((1024, 1024), dtype=torch.float32, device=dev).requires_grad
    with torch.inference_mode():
        assert pool.empty((1024, 1024), dtype=torch.float32, device=dev).is_inference()
    assert torch.equal(held[:0], held[:0].clone())


def test_deterministic_fill_bypasses_the_pool(pool) -> None:
    """tests/test_output_pool.py:261-275: with deterministic algorithms filling uninitialised
    memory, torch's own empty() runs (and fills); the pool sees no request."""
    dev = torch.device("cuda", 0)
    deterministic = torch.are_deterministic_algorithms_enabled()
    fill = torch.utils.deterministic.fill_uninitialized_memory
    before = pool.output_pool_stats()
    try:
        torch.use_deterministic_algorithms(True)
        torch.utils.deterministic.fill_uninitialized_memory = True
        t = pool.empty((2048, 1024), dtype=torch.float32, device=dev)
        assert bool(t.isnan().all())  # torch's deterministic fill for floats
    finally:
        torch.use_deterministic_algorithms(deterministic)
        torch.utils.deterministic.fill_uninitialized_memory = fill
    after = pool.output_pool_stats()
    assert (after["hits"], after["misses"]) == (before["hits"], before["misses"])


def test_torch_function_mode_falls_through(pool) -> None:
    """tests/test_output_pool.py:444-460: under an active TorchFunctionMode the allocation is
    torch's own empty_like (the mode sees it) and the pool's counters do not move."""
    from torch.overrides import TorchFunctionMode

    seen: list[str] = []

    class Spy(TorchFunctionMode):
        def __torch_function__(self, func, types, args=(), kwargs=None):
            seen.append(getattr(func, "__name__", ""))
            return func(*args, **(kwargs or {}))

    x = torch.zeros(2048, 1024, device="cuda")
    before = pool.output_pool_stats()
    with Spy():
        out = pool.empty_like(x)
    assert "empty_like" in seen and out.shape == x.shape
    after = pool.output_pool_stats()
    assert (after["hits"], after["misses"]) == (before["hits"], before["misses"])


@pytest.mark.parametrize(
    "dtype",
    [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.complex64, torch.complex128, torch.bool,
     torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.uint16, torch.uint32, torch.uint64],
)
def test_every_dtype_is_a_plain_multi_dim_tensor(pool, dtype: torch.dtype) -> None:
    """tests/test_output_pool.py:492-522, on the device."""
    sizes = (4, 1024, 1024)
    made = pool.empty(sizes, dtype=dtype, device=torch.device("cuda", 0))
    plain = torch.empty(sizes, dtype=dtype, device="cuda")
    assert made.shape == plain.shape and made.dtype == dtype and made.is_contiguous()
    assert made.stride() == plain.stride()
    assert made._is_view() is False and made._base is None
    assert made.requires_grad is False and made.grad_fn is None
    made.fill_(1)
    assert bool(made[3, 1023, 1023])


def test_failed_allocation_releases_free_blocks_and_retries(pool) -> None:
    """tests/test_output_pool.py:683-709: an allocation that fails frees every free block and
    is tried once more. The failure is injected on the host (the pool's next device
    allocation reports out-of-memory without reaching the driver)."""
    from helion_mlir_backend import native

    dev = torch.device("cuda", 0)
    lib = native.module()
    held = [pool.empty((4 * MIB,), dtype=torch.uint8, device=dev) for _ in range(3)]
    del held
    gc.collect()
    assert pool.output_pool_stats()["free_blocks"] == 3
    try:
        assert lib.b200_pool_inject_alloc_failures(1) == 0
        t = pool.empty((6 * MIB,), dtype=torch.uint8, device=dev)  # a size no free block has
        t.fill_(5)
        assert int(t[-1]) == 5
        pool_side = native.PoolStats()
        lib.b200_pool_stats(ctypes.byref(pool_side))
        assert pool_side.free_blocks == 0  # released by the retry
        # two failures in a row: the retry fails too and torch's own allocator serves the request
        assert lib.b200_pool_inject_alloc_failures(2) == 0
        u = pool.empty((10 * MIB,), dtype=torch.uint8, device=dev)
        assert u.numel() == 10 * MIB
    finally:
        lib.b200_pool_inject_alloc_failures(0)
    assert lib.b200_pool_inject_alloc_failures(-1) == 7


def test_block_is_returned_on_its_own_stream(pool) -> None:
    """A block used on a side stream and dropped while another stream is current goes back
    on the side stream: the library then orders its next use after the side stream's work,
    and a request on the default stream does not count as a same-stream reuse."""
    from helion_mlir_backend import native

    dev = torch.device("cuda", 0)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        t = pool.empty((32 * MIB,), dtype=torch.uint8, device=dev)
        for _ in range(10):
            t.add_(1)
        side_handle = native.stream_ptr(dev)
    lease_streams = [b.stream for b in pool._blocks if b.storage.data_ptr() == t.data_ptr()]
    assert lease_streams == [side_handle]
    pointer = t.data_ptr()
    del t  # dies while the default stream is current
    gc.collect()
    with torch.cuda.stream(side):
        u = pool.empty((32 * MIB,), dtype=torch.uint8, device=dev)
        assert u.data_ptr() == pointer  # same stream: reused at once, after the pending adds in stream order
    torch.cuda.synchronize()
