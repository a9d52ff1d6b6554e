"""Row-wise normalizations on the B200: softmax, GroupNorm, LayerNorm, RMSNorm.

Entry points and error behaviour follow ``helion_mlir_utils/normalization.py``
of the reference (``softmax`` :138-153, ``group_norm`` :156-196). The kernels are
``b200_softmax`` / ``b200_group_norm`` / ``b200_rms_norm``: one read and one
write of ``x`` from HBM, statistics in f32, one rounding to ``x.dtype``.
``layer_norm`` (GroupNorm with one group) and ``rms_norm`` are new names; the
reference has no ``rms_norm``.
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor

import ctypes

from helion_mlir_backend import native
from helion_mlir_backend import output_pool
from helion_mlir_backend.call_trace import CallExplanation

from . import epilogues


def _second_operand(y: Tensor, extra: Tensor) -> Tensor:
    """The default GroupNorm epilogue: ``y`` itself."""
    return y


def add_extra(y: Tensor, extra: Tensor) -> Tensor:
    """GroupNorm epilogue ``y + extra`` (fused)."""
    return y + extra


def mul_extra(y: Tensor, extra: Tensor) -> Tensor:
    """GroupNorm epilogue ``y * extra`` (fused)."""
    return y * extra


_EXTRA_OPS = {
    _second_operand: native.NORM_EXTRA_NONE,
    add_extra: native.NORM_EXTRA_ADD,
    torch.add: native.NORM_EXTRA_ADD,
    mul_extra: native.NORM_EXTRA_MUL,
    torch.mul: native.NORM_EXTRA_MUL,
}


def _out_for(x: Tensor, in_place: bool) -> Tensor:
    return x if in_place else output_pool.empty_like(x)


def softmax(x: Tensor, in_place: bool = False) -> Tensor:
    """Softmax over the last dim of a 2-D ``x``. ``in_place`` may overwrite a
    contiguous ``x`` (the caller's fresh intermediate) instead of allocating an
    output; use the result, not ``x``."""
    if x.dim() != 2:
        raise ValueError(f"softmax() expects a 2-D tensor, got {tuple(x.shape)}")
    device = native.require_cuda(x)
    m, n = map(int, x.shape)
    x = x.contiguous()
    out = _out_for(x, in_place)
    with native.on_device(device):
        code = native.module().b200_softmax(
            native.dtype_code(x.dtype), x.data_ptr(), out.data_ptr(), m, n, n, native.stream_ptr(device)
        )
    native.check("b200_softmax", code)
    return out


def group_norm(
    x: Tensor,
    num_groups: int,
    weight: Tensor | None,
    bias: Tensor | None,
    eps: float,
    epilogue: Callable[[Tensor, Tensor], Tensor] = _second_operand,
    extra: Tensor | None = None,
    in_place: bool = False,
) -> Tensor:
    """``epilogue(GroupNorm(x), extra)`` of ``x`` ``[M, C]``; ``extra`` is an
    optional per-channel ``[C]`` operand of ``epilogue`` (default: identity).
    Fused epilogues: :func:`add_extra`, :func:`mul_extra` (``torch.add`` /
    ``torch.mul``), or a unary activation the GEMM epilogues know (it then
    ignores ``extra``). ``in_place`` may overwrite a contiguous ``x``."""
    if x.dim() != 2 or x.shape[1] % num_groups:
        raise ValueError(
            f"group_norm() expects [M, C] with C divisible by {num_groups} groups, got {tuple(x.shape)}"
        )
    device = native.require_cuda(x, weight, bias, extra)
    m, c = map(int, x.shape)
    extra_op = _EXTRA_OPS.get(epilogue)
    if extra_op is None and getattr(epilogue, "__name__", None) == "_second_operand":
        extra_op = native.NORM_EXTRA_NONE  # another copy of this module's default epilogue
    act, alpha = native.ACT_IDENTITY, 0.0
    unfused = None
    if extra_op is None:
        extra_op = native.NORM_EXTRA_NONE
        unary = epilogues.resolve(epilogue)  # a unary activation applied to y alone
        if unary is not None:
            act, alpha = unary
        else:
            unfused = epilogue
    if extra_op != native.NORM_EXTRA_NONE and extra is None:
        extra = weight  # the reference passes `weight` where no extra is given (normalization.py:190)
    params = [t for t in (weight, bias, extra) if t is not None]
    param_dtype = torch.float32
    if params:
        param_dtype = params[0].dtype if all(t.dtype == params[0].dtype for t in params) else torch.float32
        if param_dtype not in (torch.float32, torch.bfloat16):
            param_dtype = torch.float32
    def prep(t: Tensor | None) -> Tensor | None:
        if t is None:
            return None
        if t.numel() != c:
            raise ValueError(f"group_norm() expects per-channel parameters of {c} elements, got {tuple(t.shape)}")
        return t.to(param_dtype).contiguous()

    weight_c, bias_c, extra_c = prep(weight), prep(bias), prep(extra)
    x = x.contiguous()
    if unfused is not None:
        # Unknown binary epilogue: normalise to f32, apply it on the device, round once.
        y32 = _group_norm_call(x.float(), m, num_groups, c, weight_c, bias_c, None, native.NORM_EXTRA_NONE,
                               native.ACT_IDENTITY, 0.0, eps, param_dtype, device, None)
        channel = (extra_c if extra_c is not None else weight_c)
        y32 = unfused(y32, None if channel is None else channel.float())
        if in_place:
            return x.copy_(y32)
        return y32.to(x.dtype)
    out = _out_for(x, in_place)
    return _group_norm_call(x, m, num_groups, c, weight_c, bias_c,
                            extra_c if extra_op != native.NORM_EXTRA_NONE else None, extra_op, act, alpha, eps,
                            param_dtype, device, out)


def _group_norm_call(x, m, groups, c, weight, bias, extra, extra_op, act, alpha, eps, param_dtype, device, out):
    if out is None:
        out = output_pool.empty_like(x)
    with native.on_device(device):
        code = native.module().b200_group_norm(
            native.dtype_code(x.dtype),
            native.dtype_code(param_dtype),
            x.data_ptr(),
            out.data_ptr(),
            m,
            groups,
            c // groups,
            native.ptr(weight),
            native.ptr(bias),
            native.ptr(extra),
            extra_op,
            act,
            alpha,
            float(eps),
            native.stream_ptr(device),
        )
    native.check("b200_group_norm", code)
    return out


def layer_norm(
    x: Tensor, weight: Tensor | None = None, bias: Tensor | None = None, eps: float = 1e-5, in_place: bool = False
) -> Tensor:
    """LayerNorm over the last dim of a 2-D ``x``: :func:`group_norm` with one group."""
    if x.dim() != 2:
        raise ValueError(f"layer_norm() expects a 2-D tensor, got {tuple(x.shape)}")
    return group_norm(x, 1, weight, bias, eps, in_place=in_place)


def rms_norm(x: Tensor, weight: Tensor | None = None, eps: float = 1e-5, in_place: bool = False) -> Tensor:
    """``x * rsqrt(mean(x^2, -1) + eps) * weight`` of a 2-D ``x``, in f32, rounded once."""
    if x.dim() != 2:
        raise ValueError(f"rms_norm() expects a 2-D tensor, got {tuple(x.shape)}")
    device = native.require_cuda(x, weight)
    m, n = map(int, x.shape)
    if weight is not None and weight.numel() != n:
        raise ValueError(f"rms_norm() expects a weight of {n} elements, got {tuple(weight.shape)}")
    param_dtype = torch.float32
    if weight is not None:
        param_dtype = weight.dtype if weight.dtype in (torch.float32, torch.bfloat16) else torch.float32
        weight = weight.to(param_dtype).contiguous()
    x = x.contiguous()
    out = _out_for(x, in_place)
    with native.on_device(device):
        code = native.module().b200_rms_norm(
            native.dtype_code(x.dtype),
            native.dtype_code(param_dtype),
            x.data_ptr(),
            out.data_ptr(),
            m,
            n,
            native.ptr(weight),
            float(eps),
            native.stream_ptr(device),
        )
    native.check("b200_rms_norm", code)
    return out


# --------------------------------------------------------------------------- explain()
# What a call would launch (kernel family, threads and values per thread per row, rows per
# CTA, tail, row kept in 16 bits, two rows per group): host arithmetic in the library
# (`b200_rowwise_explain`), so it also answers for CPU tensors of the same shape and type.

_OP_SOFTMAX, _OP_GROUP_NORM, _OP_RMS_NORM = 0, 1, 2


def _param_dtype(params: list[Tensor]) -> torch.dtype:
    if params and all(t.dtype == torch.bfloat16 for t in params):
        return torch.bfloat16
    return torch.float32


def _explain_rows(op: int, x: Tensor, n: int, groups: int, weight: Tensor | None, bias: Tensor | None,
                  extra: Tensor | None = None, extra_op: int = native.NORM_EXTRA_NONE,
                  act: int = native.ACT_IDENTITY) -> CallExplanation:
    if x.dim() != 2 or x.dtype not in (torch.float32, torch.bfloat16):
        return CallExplanation(False, "", f"expects a 2-D f32 or bf16 tensor, got {tuple(x.shape)} {x.dtype}")
    x = x.contiguous()
    param_dtype = _param_dtype([t for t in (weight, bias, extra) if t is not None])
    held = [None if t is None else t.to(param_dtype).contiguous() for t in (weight, bias, extra)]
    buf = ctypes.create_string_buffer(256)
    code = native.module().b200_rowwise_explain(
        op, native.dtype_code(x.dtype), native.dtype_code(param_dtype), x.data_ptr(), x.data_ptr(), n, n, groups,
        native.ptr(held[0]), native.ptr(held[1]), native.ptr(held[2]), extra_op, act, buf, len(buf))
    text = buf.value.decode()
    return CallExplanation(code == 0, text, None if code == 0 else native.strerror(code))


def _explain_softmax(x: Tensor, in_place: bool = False) -> CallExplanation:
    return _explain_rows(_OP_SOFTMAX, x, int(x.shape[-1]), 1, None, None)


def _explain_group_norm(x: Tensor, num_groups: int, weight: Tensor | None, bias: Tensor | None, eps: float = 1e-5,
                        epilogue: Callable[[Tensor, Tensor], Tensor] = _second_operand, extra: Tensor | None = None,
                        in_place: bool = False) -> CallExplanation:
    extra_op = _EXTRA_OPS.get(epilogue, native.NORM_EXTRA_NONE)
    act = native.ACT_IDENTITY
    if epilogue not in _EXTRA_OPS and getattr(epilogue, "__name__", None) != "_second_operand":
        unary = epilogues.resolve(epilogue)
        if unary is None:
            return CallExplanation(True, "group_norm in f32 through the row-wise kernel, then the epilogue as its own device pass")
        act = unary[0]
    if extra_op != native.NORM_EXTRA_NONE and extra is None:
        extra = weight
    return _explain_rows(_OP_GROUP_NORM, x, int(x.shape[-1]) // num_groups, num_groups, weight, bias, extra, extra_op, act)


def _explain_layer_norm(x: Tensor, weight: Tensor | None = None, bias: Tensor | None = None, eps: float = 1e-5,
                        in_place: bool = False) -> CallExplanation:
    return _explain_rows(_OP_GROUP_NORM, x, int(x.shape[-1]), 1, weight, bias)


def _explain_rms_norm(x: Tensor, weight: Tensor | None = None, eps: float = 1e-5, in_place: bool = False) -> CallExplanation:
    return _explain_rows(_OP_RMS_NORM, x, int(x.shape[-1]), 1, weight, None)


softmax.explain = _explain_softmax  # type: ignore[attr-defined]
group_norm.explain = _explain_group_norm  # type: ignore[attr-defined]
layer_norm.explain = _explain_layer_norm  # type: ignore[attr-defined]
rms_norm.explain = _explain_rms_norm  # type: ignore[attr-defined]
