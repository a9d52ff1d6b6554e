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

The storage hook: ``torch.as_tensor`` keeps an object exposing
``__cuda_array_interface__`` alive until the storage dies; that object's
``__del__`` returns the block.
"""

from __future__ import annotations

import ctypes
import math
import os
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
    """A pool block on loan to one tensor storage."""

    __slots__ = ("__cuda_array_interface__", "device", "pointer")

    def __init__(self, pointer: int, nbytes: int, device: torch.device) -> None:
        self.pointer = pointer
        self.device = device
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (pointer, False),
            "version": 2,
            "strides": None,
        }

    def __del__(self) -> None:
        # Runs wherever the storage dies (any thread, the garbage collector,
        # interpreter exit): never raises.
        try:
            stream = torch.cuda.current_stream(self.device).cuda_stream
            with torch.cuda.device(self.device):
                native.module().b200_pool_free(self.pointer, stream)
        except Exception:  # noqa: BLE001
            pass


_max_bytes = 0
_wrap_failed = False
_limit_applied = False


def _plain_dispatch() -> bool:
    """No torch-function or dispatch mode, no transform and no trace."""
    return not (
        torch._C._is_torch_function_mode_enabled()
        or torch._C._len_torch_dispatch_stack()
        or torch._C._functorch.peek_interpreter_stack() is not None
        or torch.jit.is_tracing()
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


def _allocate(sizes: tuple[int, ...], count: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor | None:
    nbytes = dtype.itemsize * count
    pointer = ctypes.c_void_p()
    hit = ctypes.c_int32()
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    lib = native.module()
    global _limit_applied
    if not _limit_applied:  # the limit chosen at import, handed over once the library is loaded
        _limit_applied = True
        lib.b200_pool_set_limit(_max_bytes)
    with torch.cuda.device(device):
        code = lib.b200_pool_alloc(nbytes, native.stream_ptr(device), ctypes.byref(pointer), ctypes.byref(hit))
    if code != 0 or not pointer.value:
        return None  # torch's own attempt raises its error
    rounded = -(-nbytes // _GRANULE) * _GRANULE
    lease = _Lease(pointer.value, rounded, device)  # its __del__ returns the block, also on failure below
    try:
        flat = torch.as_tensor(lease, device=device)
        del lease  # the storage now owns the only reference
        # Shaped in place on the pool's storage: a plain tensor, not a view of `flat`.
        out = torch.empty(0, dtype=dtype, device=device)
        out.set_(flat.untyped_storage(), 0, sizes, _default_strides(sizes))
    except (RuntimeError, TypeError, ValueError) as exc:
        global _wrap_failed
        if not _wrap_failed:
            _wrap_failed = True
            warnings.warn(f"output pool: cannot wrap a device block as a tensor ({exc}); using torch.empty", stacklevel=3)
        return None
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
    try:
        native.module().b200_pool_set_limit(_max_bytes)
        _limit_applied = True
    except ImportError:
        _limit_applied = False  # library not built yet: applied on first use


def release() -> None:
    """Free every free block now; tensors using a block are unaffected."""
    native.module().b200_pool_release()


def output_pool_stats() -> dict[str, int]:
    stats = native.PoolStats()
    native.module().b200_pool_stats(ctypes.byref(stats))
    return {
        "hits": int(stats.hits),
        "misses": int(stats.misses),
        "free_blocks": int(stats.free_blocks),
        "free_bytes": int(stats.free_bytes),
        "max_bytes": _max_bytes,
        "live_blocks": int(stats.live_blocks),
        "live_bytes": int(stats.live_bytes),
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
