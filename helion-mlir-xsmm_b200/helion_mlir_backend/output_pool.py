"""Device-side reuse pool for kernel outputs.

The reference's ``output_pool`` (``helion_mlir_backend/_compiler/output_pool.py``)
hands CPU kernels fresh tensors from mappings it keeps, so that large outputs
cost no page faults. On a B200 the cost to avoid is ``cudaMalloc``/``cudaFree``
(both synchronise the device), so the blocks kept are device memory, owned by
``libb200ops.so`` (``b200_pool_*``) and shared by every caller of the library.

Kept from the reference: :func:`empty` / :func:`empty_like` are ``torch.empty`` /
``torch.empty_like`` for tensors of :data:`MIN_BYTES` or more on a CUDA device;
a block returns when the last reference to the tensor's *storage* dies and is
reused for the same rounded size (whole 2 MiB units); at most ``max_bytes`` and
64 free blocks are kept, oldest out first; :func:`set_output_pool`,
:func:`release`, :func:`output_pool_stats`, :func:`enabled`;
``HELION_MLIR_OUTPUT_POOL`` (bytes, read at import; 0 turns it off). Everything
else gets torch's function: other devices, dtypes, argument forms, wrapper
tensors, active modes and deterministic fill.

New on the device: reuse is stream-aware. A freed block is handed to a request
on the stream that last used it at once, and to another stream only after the
work that was pending at free time has finished (an event recorded at free).

The storage hook: a block is wrapped once as a torch storage (``torch.as_tensor``
over an object exposing ``__cuda_array_interface__``, whose ``__del__`` returns the
memory to the library's pool when the storage finally dies) and that storage is
kept and re-shaped for every tensor handed out; a block is free when the pool
holds the only reference to its storage.
"""

from __future__ import annotations

import ctypes
import math
import os
import threading
import warnings

import torch

from . import native

OUTPUT_POOL_ENV = "HELION_MLIR_OUTPUT_POOL"
MIN_BYTES = 4 * 1024 * 1024
DEFAULT_MAX_BYTES = 2 << 30
_GRANULE = 2 * 1024 * 1024
_DTYPES = frozenset(
    {
        torch.float16,
        torch.bfloat16,
        torch.float32,
        torch.float64,
        torch.complex64,
        torch.complex128,
        torch.bool,
        torch.int8,
        torch.int16,
        torch.int32,
        torch.int64,
        torch.uint8,
    }
)


class _Lease:
    """A block of the library's device pool on loan to one torch storage."""

    __slots__ = ("__cuda_array_interface__", "device", "pointer", "stream")

    def __init__(self, pointer: int, nbytes: int, device: torch.device, stream: int) -> None:
        self.pointer = pointer
        self.device = device
        # The stream the block was allocated for, and on which every tensor shaped onto it
        # is handed out (a block is only reused for requests on that stream): the library
        # orders the block's next use after the work enqueued there.
        self.stream = stream
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (pointer, False),
            "version": 2,
            "strides": None,
        }

    def __del__(self) -> None:
        # Runs wherever the storage dies (any thread, any current stream, the garbage
        # collector, interpreter exit): never raises, and names the block's own stream,
        # not the one that happens to be current.
        try:
            with native.on_device(self.device):
                native.module().b200_pool_free(self.pointer, self.stream)
        except Exception:  # noqa: BLE001
            pass


class _Block:
    """A pool block wrapped once as a torch storage and handed out many times.

    Wrapping device memory as a storage (``torch.as_tensor`` over the lease) costs
    tens of microseconds; shaping a tensor onto an existing storage costs two. So
    the storage is kept, and a block is free exactly when this record holds the
    only reference to it (``_storage_Use_Count == 1``): tensors, views and anything
    else sharing the storage keep it in use, which is the reference's rule that a
    block returns when the last reference to the *storage* dies."""

    __slots__ = ("device", "nbytes", "storage", "stream")

    def __init__(self, storage: torch.UntypedStorage, nbytes: int, device: torch.device, stream: int) -> None:
        self.storage, self.nbytes, self.device, self.stream = storage, nbytes, device, stream

    def unused(self) -> bool:
        return torch._C._storage_Use_Count(self.storage._cdata) == 1


_MAX_FREE_BLOCKS = 64
_max_bytes = 0
_wrap_failed = False
_limit_applied = False
_lock = threading.Lock()
_blocks: list[_Block] = []  # oldest first
_hits = 0
_misses = 0


def _plain_dispatch() -> bool:
    """No torch-function or dispatch mode, no transform, no trace and no CUDA graph
    capture (a captured allocation must come from torch's capture-aware allocator:
    the pool would query events and may call cudaMalloc, neither of which a capture allows)."""
    return not (
        torch._C._is_torch_function_mode_enabled()
        or torch._C._len_torch_dispatch_stack()
        or torch._C._functorch.peek_interpreter_stack() is not None
        or torch.jit.is_tracing()
        or torch.cuda.is_current_stream_capturing()
    )


def _deterministic_fill() -> bool:
    return torch.are_deterministic_algorithms_enabled() and torch.utils.deterministic.fill_uninitialized_memory


def _takes(count: int, dtype: torch.dtype) -> bool:
    return (
        dtype in _DTYPES
        and MIN_BYTES <= dtype.itemsize * count <= _max_bytes
        and not _wrap_failed
        and not _deterministic_fill()
    )


def _default_strides(sizes: tuple[int, ...]) -> tuple[int, ...]:
    strides = [1] * len(sizes)
    for i in range(len(sizes) - 2, -1, -1):
        strides[i] = strides[i + 1] * max(sizes[i + 1], 1)
    return tuple(strides)


def _settle_locked() -> None:
    """Drop free blocks over the limits, oldest first (their memory goes back to the
    library's pool, which applies the same limit before it frees device memory)."""
    free = [b for b in _blocks if b.unused()]
    free_bytes = sum(b.nbytes for b in free)
    for block in free:
        if free_bytes <= _max_bytes and len(free) <= _MAX_FREE_BLOCKS and block.nbytes <= _max_bytes:
            break
        _blocks.remove(block)
        free_bytes -= block.nbytes
        free = free[1:]


def _wrap(pointer: int, rounded: int, device: torch.device, stream: int) -> torch.UntypedStorage | None:
    lease = _Lease(pointer, rounded, device, stream)  # its __del__ returns the block, also on failure below
    try:
        flat = torch.as_tensor(lease, device=device)
        del lease  # the storage now owns the only reference
        return flat.untyped_storage()
    except (RuntimeError, TypeError, ValueError) as exc:
        global _wrap_failed
        if not _wrap_failed:
            _wrap_failed = True
            warnings.warn(f"output pool: cannot wrap a device block as a tensor ({exc}); using torch.empty", stacklevel=4)
        return None


def _allocate(sizes: tuple[int, ...], count: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor | None:
    global _hits, _misses, _limit_applied
    nbytes = dtype.itemsize * count
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    rounded = -(-nbytes // _GRANULE) * _GRANULE
    stream = native.stream_ptr(device)
    storage = None
    strides = _default_strides(sizes)
    with _lock:
        # Newest first: most likely still in L2. Only blocks last used on this stream:
        # stream order then protects the previous user's pending work.
        for block in reversed(_blocks):
            if block.nbytes == rounded and block.device == device and block.stream == stream and block.unused():
                # The tensor is shaped onto the storage before the lock is given up:
                # that reference is what makes the block "in use" for other threads.
                out = torch.empty(0, dtype=dtype, device=device)
                out.set_(block.storage, 0, sizes, strides)
                _hits += 1
                _blocks.remove(block)
                _blocks.append(block)
                return out
        _misses += 1
    if storage is None:
        lib = native.module()
        if not _limit_applied:  # the limit chosen at import, handed over once the library is loaded
            _limit_applied = True
            lib.b200_pool_set_limit(_max_bytes)
        pointer = ctypes.c_void_p()
        hit = ctypes.c_int32()
        with native.on_device(device):
            code = lib.b200_pool_alloc(nbytes, stream, ctypes.byref(pointer), ctypes.byref(hit))
        if code != 0 or not pointer.value:
            return None  # torch's own attempt raises its error
        storage = _wrap(pointer.value, rounded, device, stream)
        if storage is None:
            return None
        # Shaped in place on the pool's storage: a plain tensor, not a view.
        out = torch.empty(0, dtype=dtype, device=device)
        out.set_(storage, 0, sizes, strides)
        with _lock:
            _blocks.append(_Block(storage, rounded, device, stream))
            _settle_locked()
    return out


def empty(sizes: tuple[int, ...] | list[int], *, dtype: torch.dtype, device: torch.device | str) -> torch.Tensor:
    """``torch.empty(sizes, dtype=dtype, device=device)``, from the pool if it takes the tensor."""
    dev = torch.device(device)
    if dev.type == "cuda" and all(type(size) is int and size >= 0 for size in sizes):
        count = math.prod(sizes)
        if _takes(count, dtype) and _plain_dispatch():
            out = _allocate(tuple(sizes), count, dtype, dev)
            if out is not None:
                return out
    return torch.empty(sizes, dtype=dtype, device=device)


def empty_like(x: torch.Tensor, *, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``torch.empty_like(x, dtype=dtype)``, from the pool if it takes the tensor."""
    kind = x.dtype if dtype is None else dtype
    if (
        not torch.jit.is_tracing()
        and type(x) is torch.Tensor
        and x.device.type == "cuda"
        and x.layout == torch.strided
        and not (x.is_conj() or x.is_neg() or x.is_quantized)
        and x.is_contiguous()
        and x.stride() == _default_strides(tuple(x.shape))
    ):
        count = x.numel()
        if _takes(count, kind) and _plain_dispatch():
            out = _allocate(tuple(x.shape), count, kind, x.device)
            if out is not None:
                return out
    return torch.empty_like(x, dtype=kind)


def set_output_pool(max_bytes: int) -> None:
    """Keep at most ``max_bytes`` of free blocks; 0 turns the pool off and frees
    them. Tensors using a block are unaffected."""
    global _max_bytes, _limit_applied
    _max_bytes = max(0, int(max_bytes))
    with _lock:
        _settle_locked()
    try:
        native.module().b200_pool_set_limit(_max_bytes)
        _limit_applied = True
    except ImportError:
        _limit_applied = False  # library not built yet: applied on first use


def release() -> None:
    """Free every free block now; tensors using a block are unaffected."""
    with _lock:
        for block in [b for b in _blocks if b.unused()]:
            _blocks.remove(block)
    native.module().b200_pool_release()


def output_pool_stats() -> dict[str, int]:
    with _lock:
        _settle_locked()
        free = [b for b in _blocks if b.unused()]
        live = len(_blocks) - len(free)
        live_bytes = sum(b.nbytes for b in _blocks) - sum(b.nbytes for b in free)
        return {
            "hits": _hits,
            "misses": _misses,
            "free_blocks": len(free),
            "free_bytes": sum(b.nbytes for b in free),
            "max_bytes": _max_bytes,
            "live_blocks": live,
            "live_bytes": live_bytes,
        }


def enabled() -> bool:
    return _max_bytes > 0


def _default_max_bytes() -> int:
    default = DEFAULT_MAX_BYTES
    value = os.environ.get(OUTPUT_POOL_ENV, "").strip()
    if not value:
        return default
    try:
        chosen = int(value)
        if chosen < 0:
            raise ValueError
    except ValueError:
        warnings.warn(f"{OUTPUT_POOL_ENV}={value!r} is not a number of bytes: using {default}", stacklevel=2)
        return default
    return chosen


_max_bytes = _default_max_bytes()
