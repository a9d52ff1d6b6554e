"""Row-streamed calls on host buffers (an extension; the reference's operators run
on host memory directly, so they have no counterpart of this step).

Every operator of this package is independent per row of its first operand. For
operands that live in pinned host memory, :func:`stream_rows` cuts the rows into
chunks and runs three stages on three CUDA streams, ``depth`` chunks in flight:

    copy-in stream   host rows  -> device staging buffer
    caller's stream  the operator on the staged chunk
    copy-out stream  device result -> host rows

PCIe carries both directions at once, so a call costs about
``max(bytes in, bytes out) / link rate`` instead of their sum plus the kernel.
All ordering is by events; the caller's stream ends up waiting for the last
copy-out, so a ``torch.cuda.current_stream().synchronize()`` (or any later work
on that stream) sees the finished host result.
"""

from __future__ import annotations

import threading
from collections.abc import Callable

import torch
from torch import Tensor

from helion_mlir_backend import native

# Bytes of one staged input chunk the default chunking aims for: long enough that
# per-chunk launch and cross-stream event latency hides behind its copy, short
# enough that the first copy-in and last copy-out (not overlapped) stay small.
_CHUNK_BYTES = 16 << 20


class _Slot:
    __slots__ = ("staged", "copied_in", "computed", "copied_out", "result", "used")

    def __init__(self, staged: Tensor) -> None:
        self.staged = staged
        self.copied_in = torch.cuda.Event()
        self.computed = torch.cuda.Event()
        self.copied_out = torch.cuda.Event()
        self.result: Tensor | None = None
        self.used = False


class _Lanes:
    """Per (device, chunk shape, dtype): the two copy streams and the staging ring."""

    def __init__(self, device: torch.device, chunk_shape: tuple[int, ...], dtype: torch.dtype, depth: int) -> None:
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        self.started = torch.cuda.Event()
        self.finished: torch.cuda.Event | None = None
        self.slots = [_Slot(torch.empty(chunk_shape, dtype=dtype, device=device)) for _ in range(depth)]
        self.lock = threading.Lock()


_LANES: dict[tuple[object, ...], _Lanes] = {}
_LANES_LOCK = threading.Lock()


def default_chunk_rows(x_host: Tensor) -> int:
    """Rows per chunk: about ``_CHUNK_BYTES`` of input, a multiple of 256 rows (whole
    GEMM tiles), at least 4 chunks when the rows allow it."""
    rows = int(x_host.shape[0])
    row_bytes = max(1, x_host[0].numel() * x_host.element_size()) if rows else 1
    chunk = max(256, (_CHUNK_BYTES // row_bytes) // 256 * 256)
    while chunk > 256 and rows // chunk < 4:
        chunk //= 2
    return max(1, min(chunk, rows))


def stream_rows(
    fn: Callable[[Tensor], Tensor],
    x_host: Tensor,
    out_host: Tensor,
    chunk_rows: int | None = None,
    depth: int = 3,
    device: torch.device | int | None = None,
) -> Tensor:
    """``out_host[r] = fn(x_host[r])`` for every row chunk ``r``, the copies of
    neighbouring chunks overlapped with the kernels. ``fn`` takes a device tensor
    of ``[rows, ...]`` and returns a device tensor of ``[rows, ...]`` on the
    current stream (any operator of this package bound to its other arguments).
    ``x_host`` and ``out_host`` must be pinned and contiguous along all but the
    row dimension. Returns ``out_host``; the caller's stream is left waiting for
    the last copy-out, nothing blocks the host."""
    if x_host.is_cuda or out_host.is_cuda:
        raise ValueError("stream_rows() takes host tensors; call the operator directly on device tensors")
    if x_host.dim() < 1 or out_host.dim() < 1 or x_host.shape[0] != out_host.shape[0]:
        raise ValueError(f"row counts differ: {tuple(x_host.shape)} vs {tuple(out_host.shape)}")
    if x_host.shape[0] == 0:
        return out_host
    if not x_host.is_pinned() or not out_host.is_pinned():
        raise ValueError("stream_rows() needs pinned host memory (tensor.pin_memory()) for asynchronous copies")
    if not x_host.is_contiguous() or not out_host.is_contiguous():
        raise ValueError("stream_rows() needs contiguous host tensors")
    if depth < 2:
        raise ValueError("depth must be at least 2 (one chunk copying while another computes)")
    rows = int(x_host.shape[0])
    native.module()  # fails loudly when the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError("stream_rows() needs a CUDA device")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type != "cuda":
        raise ValueError(f"stream_rows() runs on a CUDA device, got {dev}")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    chunk = default_chunk_rows(x_host) if chunk_rows is None else int(chunk_rows)
    if chunk <= 0:
        raise ValueError("chunk_rows must be positive")
    chunk = min(chunk, rows)

    chunk_shape = (chunk, *map(int, x_host.shape[1:]))
    key = (dev.index, chunk_shape, x_host.dtype, depth)
    with _LANES_LOCK:
        lanes = _LANES.get(key)
        if lanes is None:
            lanes = _LANES[key] = _Lanes(dev, chunk_shape, x_host.dtype, depth)

    with lanes.lock, torch.cuda.device(dev):
        compute = torch.cuda.current_stream(dev)
        # Stage buffers may still be read by work the caller enqueued earlier.
        lanes.started.record(compute)
        lanes.copy_in.wait_event(lanes.started)
        if lanes.finished is not None:  # an earlier call may have run on another stream
            lanes.copy_in.wait_event(lanes.finished)
        for index, begin in enumerate(range(0, rows, chunk)):
            end = min(rows, begin + chunk)
            slot = lanes.slots[index % depth]
            staged = slot.staged[: end - begin]
            if slot.used:
                lanes.copy_in.wait_event(slot.computed)  # its previous chunk has been consumed
            with torch.cuda.stream(lanes.copy_in):
                staged.copy_(x_host[begin:end], non_blocking=True)
                slot.copied_in.record(lanes.copy_in)
            compute.wait_event(slot.copied_in)
            if slot.used:
                # The previous result of this slot goes back to the allocator only once
                # its copy-out is ordered before whatever the compute stream does next.
                compute.wait_event(slot.copied_out)
                slot.result = None
            result = fn(staged)
            if result.shape[0] != end - begin:
                raise ValueError(f"fn returned {tuple(result.shape)} for {end - begin} rows")
            slot.computed.record(compute)
            lanes.copy_out.wait_event(slot.computed)
            with torch.cuda.stream(lanes.copy_out):
                out_host[begin:end].copy_(result, non_blocking=True)
                slot.copied_out.record(lanes.copy_out)
            slot.result = result
            slot.used = True
        for slot in lanes.slots:
            if slot.used:
                compute.wait_event(slot.copied_out)
                slot.result = None
                slot.used = False
        if lanes.finished is None:
            lanes.finished = torch.cuda.Event()
        lanes.finished.record(compute)
    return out_host


def release() -> None:
    """Drops the cached copy streams and staging buffers."""
    with _LANES_LOCK:
        _LANES.clear()
