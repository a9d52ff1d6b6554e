"""Row and column reductions on the B200: matvec, row_sum, row_dot, column_sum.

Entry points, result shapes and error text follow
``helion_mlir_utils/reduction.py`` of the reference (``matvec`` :44-67,
``row_sum`` :99-121, ``column_sum`` :142-163, ``row_dot`` :188-212). Each is one
pass over the matrix from HBM with f32 accumulation in a fixed order.
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor

from helion_mlir_backend import native
from helion_mlir_backend import output_pool

from . import epilogues
from .epilogues import identity_epilogue


def supports_matvec(a: Tensor, b: Tensor) -> bool:
    """Whether :func:`matvec` can handle this pair of operands."""
    if a.dtype != b.dtype or a.dtype not in (torch.float32, torch.bfloat16):
        return False
    if a.device.type != "cuda" or b.device != a.device:
        return False
    if a.dim() != 2 or b.dim() != 2 or b.shape[1] != 1:
        return False
    return a.shape[1] == b.shape[0]


def _row_reduce(kind: int, x: Tensor, v: Tensor | None, epilogue: Callable[[Tensor], Tensor]) -> Tensor:
    device = native.require_cuda(x, v)
    m, n = map(int, x.shape)
    x = x.contiguous()
    fused = epilogues.resolve(epilogue)
    act, alpha = fused if fused is not None else (native.ACT_IDENTITY, 0.0)
    out_dtype = x.dtype if fused is not None else torch.float32
    src = x
    if fused is None and x.dtype != torch.float32:
        # Unfused epilogue: reduce to f32 first so that the only rounding comes after it.
        src = x.float()
    out = output_pool.empty((m, 1), dtype=out_dtype, device=device)
    if v is not None and kind == native.REDUCE_MATVEC and src.dtype != v.dtype:
        v = v.to(src.dtype)
    with native.on_device(device):
        code = native.module().b200_row_reduce(
            kind, native.dtype_code(src.dtype), src.data_ptr(), native.ptr(v), out.data_ptr(), m, n, n, act, alpha,
            native.stream_ptr(device),
        )
    native.check("b200_row_reduce", code)
    if fused is None:
        return epilogue(out).to(x.dtype)
    return out


def matvec(a: Tensor, b: Tensor) -> Tensor:
    """``A @ b`` for ``A: [M, K]``, ``b: [K, 1]`` -> ``[M, 1]``.

    Raises ``ValueError`` if unsupported (see :func:`supports_matvec`) instead of
    silently falling back to eager PyTorch.
    """
    if not supports_matvec(a, b):
        raise ValueError(
            f"matvec() does not support these operands: a.shape={tuple(a.shape)} "
            f"a.dtype={a.dtype} a.device={a.device}, b.shape={tuple(b.shape)} "
            f"b.dtype={b.dtype} b.device={b.device}. b must be K-by-1, dtype must be "
            "float32 or bfloat16, both on the same cuda device. Check supports_matvec() before "
            "calling, or use torch.matmul directly for unsupported cases."
        )
    k = int(a.shape[1])
    return _row_reduce(native.REDUCE_MATVEC, a, b.reshape(k).contiguous(), identity_epilogue)


def row_sum(x: Tensor, epilogue: Callable[[Tensor], Tensor] = identity_epilogue) -> Tensor:
    """``epilogue(x.sum(1, keepdim=True))`` of a 2-D ``x``, summed in f32."""
    if x.dim() != 2:
        raise ValueError(f"row_sum() expects a 2-D tensor, got {tuple(x.shape)}")
    return _row_reduce(native.REDUCE_ROW_SUM, x, None, epilogue)


def row_dot(x: Tensor, v: Tensor, epilogue: Callable[[Tensor], Tensor] = identity_epilogue) -> Tensor:
    """``epilogue(x @ v)`` of a 2-D ``x`` and an f32 ``[N]``, in f32 and rounded once, as ``[M, 1]``."""
    if x.dim() != 2 or v.dim() != 1 or x.shape[1] != v.shape[0]:
        raise ValueError(f"row_dot() expects [M, N] and [N], got {tuple(x.shape)}, {tuple(v.shape)}")
    if v.dtype != torch.float32:
        raise ValueError(f"row_dot() expects an f32 vector, got {v.dtype}")
    return _row_reduce(native.REDUCE_ROW_DOT, x, v.contiguous(), epilogue)


def column_sum(x: Tensor) -> Tensor:
    """``x.sum(0)`` of a 2-D ``x`` in f32 (``[N]``), summed in a fixed order."""
    if x.dim() != 2:
        raise ValueError(f"column_sum() expects a 2-D tensor, got {tuple(x.shape)}")
    device = native.require_cuda(x)
    m, n = map(int, x.shape)
    if m == 0:
        return torch.zeros((n,), dtype=torch.float32, device=device)
    x = x.contiguous()
    lib = native.module()
    out = output_pool.empty((n,), dtype=torch.float32, device=device)
    need = int(lib.b200_column_sum_workspace_bytes(m, n))
    workspace = output_pool.empty((need,), dtype=torch.uint8, device=device) if need else None
    with native.on_device(device):
        code = lib.b200_column_sum(
            native.dtype_code(x.dtype), x.data_ptr(), out.data_ptr(), m, n, n, native.ptr(workspace), need,
            native.stream_ptr(device),
        )
    native.check("b200_column_sum", code)
    return out


# --------------------------------------------------------------------------- explain()
# What a call would launch: host arithmetic in the library (`b200_reduce_explain`), so it
# also answers for CPU tensors of the same shape and type.

_KIND_ROW_SUM, _KIND_ROW_DOT, _KIND_MATVEC, _KIND_COLUMN_SUM = 0, 1, 2, 3


def _explain_reduction(kind: int, x: Tensor, v: Tensor | None):
    import ctypes

    from helion_mlir_backend.call_trace import CallExplanation

    if x.dim() != 2 or x.dtype not in (torch.float32, torch.bfloat16) or x.numel() == 0:
        return CallExplanation(False, "", f"expects a non-empty 2-D f32 or bf16 tensor, got {tuple(x.shape)} {x.dtype}")
    x = x.contiguous()
    m, n = map(int, x.shape)
    if v is not None:
        v = v.reshape(-1).to(torch.float32 if kind == _KIND_ROW_DOT else x.dtype).contiguous()
    buf = ctypes.create_string_buffer(320)
    code = native.module().b200_reduce_explain(kind, native.dtype_code(x.dtype), x.data_ptr(), native.ptr(v), m, n, n, buf, len(buf))
    return CallExplanation(code == 0, buf.value.decode(), None if code == 0 else native.strerror(code))


row_sum.explain = lambda x, epilogue=identity_epilogue: _explain_reduction(_KIND_ROW_SUM, x, None)  # type: ignore[attr-defined]
row_dot.explain = lambda x, v, epilogue=identity_epilogue: _explain_reduction(_KIND_ROW_DOT, x, v)  # type: ignore[attr-defined]
matvec.explain = lambda a, b: _explain_reduction(_KIND_MATVEC, a, b)  # type: ignore[attr-defined]
column_sum.explain = lambda x: _explain_reduction(_KIND_COLUMN_SUM, x, None)  # type: ignore[attr-defined]
