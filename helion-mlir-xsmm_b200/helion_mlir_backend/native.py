"""ctypes binding of ``libb200ops.so``: the native call path.

The reference's native path is a CPython extension built at first use
(``helion_mlir_backend/_compiler/native/__init__.py``, ``call.cpp``) that checks
arguments and calls JIT-compiled CPU code. Here the compiled code is a fixed
CUDA library with a C ABI (``include/b200ops.h``); this module loads it, declares
the signatures and offers small helpers to pass torch tensors as pointers. There
is no CPU fallback: if the library is missing, or a call is refused, the caller
gets an exception.
"""

from __future__ import annotations

import contextlib
import ctypes
from ctypes import c_char_p
from ctypes import c_float
from ctypes import c_int
from ctypes import c_int32
from ctypes import c_int64
from ctypes import c_size_t
from ctypes import c_uint64
from ctypes import c_void_p
import os
from pathlib import Path
import threading

import torch

F32, BF16 = 0, 1

ACT_IDENTITY, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SIGMOID, ACT_TANH, ACT_SILU, ACT_LEAKY_RELU = range(8)
LAYOUT_ROW, LAYOUT_COL, LAYOUT_BLOCKED, LAYOUT_BLOCKED_VNNI, LAYOUT_VNNI_PANELS = range(5)
(
    PACK_PAD_2D,
    PACK_A_BLOCKED,
    PACK_A_BLOCKED_T,
    PACK_B_BLOCKED,
    PACK_B_BLOCKED_T,
    PACK_B_VNNI,
    PACK_B_VNNI_T,
    PACK_B_VNNI_PANELS_T,
    UNPACK_B_VNNI_TO_NK,
    UNPACK_B_VNNI_PANELS_TO_NK,
    UNPACK_A_BLOCKED_TO_MK,
    UNPACK_B_BLOCKED_TO_NK,
) = range(12)
NORM_EXTRA_NONE, NORM_EXTRA_ADD, NORM_EXTRA_MUL = range(3)
REDUCE_ROW_SUM, REDUCE_ROW_DOT, REDUCE_MATVEC = range(3)
ELT_RELU, ELT_LEAKY_RELU, ELT_SCALAR_MUL = range(3)
E_DISABLED = 10

LIB_NAME = "libb200ops.so"
LIB_ENV = "B200OPS_LIBRARY"


class NativeCallError(RuntimeError):
    """A b200ops entry point refused the call or CUDA reported an error."""

    def __init__(self, function: str, code: int, message: str) -> None:
        super().__init__(f"{function} failed ({code}): {message}")
        self.function = function
        self.code = code


class GemmDesc(ctypes.Structure):
    """``b200_gemm_desc`` of include/b200ops.h."""

    _fields_ = [
        ("dtype", c_int32),
        ("out_dtype", c_int32),
        ("a_layout", c_int32),
        ("b_layout", c_int32),
        ("b_panel", c_int32),
        ("epilogue", c_int32),
        ("alpha", c_float),
        ("vec_dtype", c_int32),
        ("m", c_int64),
        ("n", c_int64),
        ("k", c_int64),
        ("batch", c_int64),
        ("lda", c_int64),
        ("ldb", c_int64),
        ("ldc", c_int64),
        ("stride_a", c_int64),
        ("stride_b", c_int64),
        ("stride_c", c_int64),
        ("a", c_void_p),
        ("b", c_void_p),
        ("c", c_void_p),
        ("bias", c_void_p),
        ("scale", c_void_p),
        ("shift", c_void_p),
        ("bias_n", c_int64),
        ("scale_n", c_int64),
        ("shift_n", c_int64),
        ("split_k", c_int32),
        ("tile_m", c_int32),
        ("tile_n", c_int32),
        ("tile_k", c_int32),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("force_kernel", c_int32),
        ("reserved_", c_int32),
    ]


class PoolStats(ctypes.Structure):
    _fields_ = [(name, c_uint64) for name in ("hits", "misses", "free_blocks", "free_bytes", "max_bytes", "live_blocks", "live_bytes")]


MAX_PEERS = 8
IPC_HANDLE_BYTES = 64


class PeerOut(ctypes.Structure):
    """``b200_peer_out``: the copies of C of a GEMM stored to every GPU of a group."""

    _fields_ = [
        ("count", c_int32),
        ("rank", c_int32),
        ("epoch", c_int32),
        ("reserved_", c_int32),
        ("c", c_void_p * MAX_PEERS),
        ("flags", c_void_p * MAX_PEERS),
        ("done_counter", c_void_p),
        ("store_maps", c_void_p),
    ]


class Counters(ctypes.Structure):
    _fields_ = [
        ("launches", c_uint64),
        ("calls", c_uint64),
        ("refusals", c_uint64),
        ("cuda_errors", c_uint64),
        ("last_refusal", c_int32),
        ("reserved_", c_int32),
    ]


# name -> (restype, argtypes): every symbol include/b200ops.h declares.
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "b200_gemm": (c_int, [ctypes.POINTER(GemmDesc), c_void_p]),
    "b200_gemm_explain": (c_int, [ctypes.POINTER(GemmDesc), c_char_p, c_size_t]),
    "b200_gemm_workspace_bytes": (c_size_t, [ctypes.POINTER(GemmDesc)]),
    "b200_gemm_host_rows": (c_int, [ctypes.POINTER(GemmDesc), c_void_p, c_void_p, c_int64, c_void_p]),
    "b200_host_rows_release": (c_int, []),
    "b200_attention": (
        c_int,
        [c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p],
    ),
    "b200_pack": (
        c_int,
        [c_int32, c_int32, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int32, c_void_p],
    ),
    "b200_softmax": (c_int, [c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "b200_group_norm": (
        c_int,
        [
            c_int32,
            c_int32,
            c_void_p,
            c_void_p,
            c_int64,
            c_int64,
            c_int64,
            c_void_p,
            c_void_p,
            c_void_p,
            c_int32,
            c_int32,
            c_float,
            c_float,
            c_void_p,
        ],
    ),
    "b200_rms_norm": (c_int, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_float, c_void_p]),
    "b200_rowwise_explain": (
        c_int,
        [c_int32, c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int32,
         c_int32, ctypes.c_char_p, c_size_t],
    ),
    "b200_row_reduce": (
        c_int,
        [c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_float, c_void_p],
    ),
    "b200_reduce_explain": (
        c_int, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, ctypes.c_char_p, c_size_t]),
    "b200_column_sum_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "b200_column_sum": (c_int, [c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p]),
    "b200_column_sum_static": (c_int, [c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "b200_column_sum_static_fits": (c_int, [c_int64, c_int64, c_size_t]),
    "b200_eltwise": (c_int, [c_int32, c_int32, c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "b200_gemm_to_peers": (c_int, [ctypes.POINTER(GemmDesc), ctypes.POINTER(PeerOut), c_void_p]),
    "b200_peer_store_maps": (c_int, [c_void_p, ctypes.POINTER(c_void_p), c_int32, c_int64, c_int64, c_int64]),
    "b200_peer_wait": (c_int, [c_void_p, c_int32, c_int32, c_uint64, c_void_p]),
    "b200_symm_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "b200_symm_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "b200_symm_close": (c_int, [c_void_p]),
    "b200_symm_free": (c_int, [c_void_p]),
    "b200_pool_alloc": (c_int, [c_size_t, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int32)]),
    "b200_pool_free": (c_int, [c_void_p, c_void_p]),
    "b200_pool_set_limit": (c_int, [c_size_t]),
    "b200_pool_release": (c_int, []),
    "b200_pool_stats": (c_int, [ctypes.POINTER(PoolStats)]),
    "b200_pool_inject_alloc_failures": (c_int, [c_int32]),
    "b200_get_counters": (c_int, [ctypes.POINTER(Counters)]),
    "b200_reset_counters": (c_int, []),
    "b200_read_kernel_status": (c_int, [c_void_p, ctypes.POINTER(c_int32)]),
    "b200_selftest_wait_timeout": (c_int, [c_uint64, c_void_p]),
    "b200_strerror": (c_char_p, [c_int]),
    "b200_abi_version": (c_int, []),
    "b200_set_enabled": (c_int, [c_int]),
    "b200_sm_count": (c_int, []),
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_enabled = os.environ.get("HELION_MLIR_NATIVE_CALL", "1").strip().lower() not in ("0", "false", "no")


def library_path() -> Path:
    """Where the built library lives: ``$B200OPS_LIBRARY`` or ``lib/`` beside the packages."""
    override = os.environ.get(LIB_ENV)
    if override:
        return Path(override)
    return Path(__file__).resolve().parent.parent / "lib" / LIB_NAME


def module() -> ctypes.CDLL:
    """The loaded library, with every signature declared. Raises if it is not built:
    there is no other implementation to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = library_path()
            if not path.exists():
                raise ImportError(
                    f"{path} is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                    "(or helion-mlir-xsmm_b200/csrc/build.py). The B200 operator set has no CPU fallback."
                )
            lib = ctypes.CDLL(str(path))
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            if lib.b200_abi_version() != 1:
                raise ImportError(f"{path}: ABI version {lib.b200_abi_version()} != 1")
            lib.b200_set_enabled(1 if _enabled else 0)
            _lib = lib
    return _lib


def set_native_call(enabled: bool) -> None:
    """Turn the native call path on or off (cf. ``set_native_call`` of the reference,
    ``_compiler/native/__init__.py``). Off, every operator raises: the device
    kernels are the only implementation."""
    global _enabled
    _enabled = bool(enabled)
    if _lib is not None:
        _lib.b200_set_enabled(1 if _enabled else 0)


def native_call_enabled() -> bool:
    return _enabled


def strerror(code: int) -> str:
    return module().b200_strerror(code).decode()


def check(function: str, code: int) -> None:
    if code != 0:
        raise NativeCallError(function, code, strerror(code))


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"dtype must be torch.float32 or torch.bfloat16, got {dtype}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _raw_stream_slow(index: int) -> int:
    return torch.cuda.current_stream(index).cuda_stream


# The raw handle without building a Stream object (an order of magnitude cheaper per call).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", _raw_stream_slow)


def stream_ptr(device: torch.device) -> int:
    """The caller's current stream on ``device``: kernels are enqueued there."""
    index = device.index
    if index is None:
        index = torch.cuda.current_device()
    return _raw_stream(index)


_NO_SWITCH = contextlib.nullcontext()


def on_device(device: torch.device):
    """Context in which ``device`` is current: a no-op when it already is (the usual
    case; entering ``torch.cuda.device`` costs microseconds per call)."""
    index = device.index
    if index is None or index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise ValueError(f"operands must be CUDA tensors, got a tensor on {t.device}")
        if device is None:
            device = t.device
        elif t.device != device:
            raise ValueError(f"operands are on different devices: {device} and {t.device}")
    assert device is not None
    return device


def counters() -> dict[str, int]:
    c = Counters()
    module().b200_get_counters(ctypes.byref(c))
    return {name: int(getattr(c, name)) for name, _ in Counters._fields_ if name != "reserved_"}


def kernel_status(device: torch.device | None = None) -> int:
    """Error bits left by kernels whose bounded waits ran out (0: none). Synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    value = c_int32(0)
    with on_device(device):
        check("b200_read_kernel_status", module().b200_read_kernel_status(stream_ptr(device), ctypes.byref(value)))
    return int(value.value)
