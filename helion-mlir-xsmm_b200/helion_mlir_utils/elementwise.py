"""Elementwise kernels on the B200: ReLU, LeakyReLU, scalar multiply.

Same entry points as ``helion_mlir_utils/elementwise.py`` of the reference; the
kernel is ``b200_eltwise`` (128-bit vectorised, grid-stride)."""

from __future__ import annotations

import torch
from torch import Tensor

from helion_mlir_backend import native
from helion_mlir_backend import output_pool


def _eltwise(kind: int, x: Tensor, param: float) -> Tensor:
    device = native.require_cuda(x)
    x = x.contiguous()
    out = output_pool.empty_like(x)
    with native.on_device(device):
        code = native.module().b200_eltwise(
            kind, native.dtype_code(x.dtype), x.data_ptr(), out.data_ptr(), x.numel(), float(param),
            native.stream_ptr(device),
        )
    native.check("b200_eltwise", code)
    return out


def relu(x: Tensor) -> Tensor:
    """Elementwise ``max(x, 0)``."""
    return _eltwise(native.ELT_RELU, x, 0.0)


def leaky_relu(x: Tensor, negative_slope: float = 0.01) -> Tensor:
    """Elementwise LeakyReLU: ``x`` where positive, else ``x * negative_slope``."""
    return _eltwise(native.ELT_LEAKY_RELU, x, negative_slope)


def scalar_mul(a: Tensor, s: float | Tensor) -> Tensor:
    """Elementwise ``a * s``; ``s`` may be a 0-d tensor."""
    if isinstance(s, Tensor):
        s = float(s)
    return _eltwise(native.ELT_SCALAR_MUL, a, s)
