"""Fused epilogues: which Python callables the kernels can apply in their epilogue.

The reference traces any callable ``epilogue(acc)`` into the compiled kernel
(``helion_mlir_utils/matmul.py:321-327``). Hand-written kernels carry a fixed set
of activations instead (``B200_ACT_*`` in include/b200ops.h). :func:`resolve`
maps the callables users pass in practice to that set; a callable outside it is
*not* silently dropped: the operator runs the kernel with an f32 result and then
applies the callable on the device before the single rounding (one extra
elementwise pass; ``explain`` reports it as unfused).
"""

from __future__ import annotations

import functools
from typing import Callable

import torch
import torch.nn.functional as F
from torch import Tensor

from helion_mlir_backend import native


def identity_epilogue(x: Tensor) -> Tensor:
    return x


def gelu_tanh(x: Tensor) -> Tensor:
    return F.gelu(x, approximate="tanh")


@functools.cache
def leaky_relu_epilogue(negative_slope: float = 0.01) -> Callable[[Tensor], Tensor]:
    """A LeakyReLU epilogue with the given slope that the kernels fuse."""

    def leaky(x: Tensor) -> Tensor:
        return F.leaky_relu(x, negative_slope)

    leaky._b200_act = (native.ACT_LEAKY_RELU, float(negative_slope))  # type: ignore[attr-defined]
    return leaky


_KNOWN: dict[object, tuple[int, float]] = {
    identity_epilogue: (native.ACT_IDENTITY, 0.0),
    torch.relu: (native.ACT_RELU, 0.0),
    F.relu: (native.ACT_RELU, 0.0),
    torch.relu_: (native.ACT_RELU, 0.0),
    F.gelu: (native.ACT_GELU_ERF, 0.0),
    gelu_tanh: (native.ACT_GELU_TANH, 0.0),
    torch.sigmoid: (native.ACT_SIGMOID, 0.0),
    F.sigmoid: (native.ACT_SIGMOID, 0.0),
    torch.tanh: (native.ACT_TANH, 0.0),
    F.tanh: (native.ACT_TANH, 0.0),
    F.silu: (native.ACT_SILU, 0.0),
    F.leaky_relu: (native.ACT_LEAKY_RELU, 0.01),
}


def resolve(epilogue: Callable[..., Tensor]) -> tuple[int, float] | None:
    """``(activation code, alpha)`` if the kernels can fuse ``epilogue``, else ``None``."""
    tagged = getattr(epilogue, "_b200_act", None)
    if tagged is not None:
        return tagged
    try:
        known = _KNOWN.get(epilogue)
    except TypeError:  # unhashable callable
        known = None
    if known is not None:
        return known
    # the identity of another copy of this operator set (e.g. the reference's own module)
    if getattr(epilogue, "__name__", None) == "identity_epilogue" and "helion_mlir_utils" in (
        getattr(epilogue, "__module__", "") or ""
    ):
        return (native.ACT_IDENTITY, 0.0)
    if isinstance(epilogue, functools.partial) and not epilogue.args:
        if epilogue.func is F.gelu:
            mode = epilogue.keywords.get("approximate", "none")
            if set(epilogue.keywords) <= {"approximate"} and mode in ("none", "tanh"):
                return (native.ACT_GELU_TANH if mode == "tanh" else native.ACT_GELU_ERF, 0.0)
        if epilogue.func is F.leaky_relu and set(epilogue.keywords) <= {"negative_slope"}:
            return (native.ACT_LEAKY_RELU, float(epilogue.keywords.get("negative_slope", 0.01)))
    if isinstance(epilogue, torch.nn.Module):
        if type(epilogue) is torch.nn.ReLU:
            return (native.ACT_RELU, 0.0)
        if type(epilogue) is torch.nn.GELU:
            return (native.ACT_GELU_TANH if epilogue.approximate == "tanh" else native.ACT_GELU_ERF, 0.0)
        if type(epilogue) is torch.nn.Sigmoid:
            return (native.ACT_SIGMOID, 0.0)
        if type(epilogue) is torch.nn.Tanh:
            return (native.ACT_TANH, 0.0)
        if type(epilogue) is torch.nn.SiLU:
            return (native.ACT_SILU, 0.0)
        if type(epilogue) is torch.nn.LeakyReLU:
            return (native.ACT_LEAKY_RELU, float(epilogue.negative_slope))
        if type(epilogue) is torch.nn.Identity:
            return (native.ACT_IDENTITY, 0.0)
    return None
