"""Softmax attention built on this operator set (an extension of the reference's
30 names: the reference carries the kernel only as a test body,
``tests/harness.py:263-300`` ``_attention`` and ``tests/test_numerics.py:141-158``
``attention``).

``attention(q, k, v, scale)`` computes ``softmax(scale * q @ k^T) @ v`` per head for
``[heads, seq, dim]`` operands. bf16 operands with ``dim`` 64 or 128 run the fused
tensor-core kernel ``b200_attention`` (scores and probabilities never leave the
SM). Everything else (f32, other head sizes) is composed from the operators of
this package: one batched GEMM for the scores, the row softmax, one batched GEMM
with ``v`` -- the scores then pass through HBM once in f32.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from helion_mlir_backend import native
from helion_mlir_backend import output_pool
from helion_mlir_backend.call_trace import trace

_FUSED_DIMS = (64, 128)


def _check(q: Tensor, k: Tensor, v: Tensor) -> tuple[int, int, int, int]:
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError(f"attention() expects [heads, seq, dim] operands, got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    heads, seq_q, dim = map(int, q.shape)
    if int(k.shape[0]) != heads or int(k.shape[2]) != dim or tuple(v.shape) != tuple(k.shape):
        raise ValueError(f"attention() operands do not match: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"attention() requires matching bf16/f32 operands, got {q.dtype}, {k.dtype}, {v.dtype}")
    return heads, seq_q, int(k.shape[1]), dim


def fused(q: Tensor, k: Tensor, v: Tensor, scale: float = 1.0) -> bool:
    """Whether this call takes the fused kernel (else the composed path)."""
    return (q.dtype == torch.bfloat16 and q.dim() == 3 and int(q.shape[2]) in _FUSED_DIMS
            and scale != 0.0 and math.isfinite(scale))


def attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None) -> Tensor:
    """``softmax(scale * q @ k^T, dim=-1) @ v`` per head; ``scale`` defaults to
    ``dim ** -0.5``. Result in ``q.dtype``, shape of ``q``."""
    heads, seq_q, seq_k, dim = _check(q, k, v)
    device = native.require_cuda(q, k, v)
    scale = 1.0 / math.sqrt(dim) if scale is None else float(getattr(scale, "value", scale))
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if fused(q, k, v, scale):
        out = output_pool.empty_like(q)
        with native.on_device(device):
            code = native.module().b200_attention(
                native.BF16, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), heads, seq_q, seq_k, dim,
                scale, native.stream_ptr(device),
            )
        native.check("b200_attention", code)
        trace(f"attention fused {tuple(q.shape)} x {tuple(k.shape)}")
        return out
    return _composed(q, k, v, scale)


def _composed(q: Tensor, k: Tensor, v: Tensor, scale: float) -> Tensor:
    from . import elementwise, normalization
    from .matmul import bmm

    heads, seq_q, dim = map(int, q.shape)
    seq_k = int(k.shape[1])
    if seq_k == 0 or seq_q == 0 or heads == 0:
        return torch.zeros_like(q)
    # scores = (scale * q) @ k^T: the scale rides on the smaller operand
    scaled = elementwise.scalar_mul(q.reshape(heads * seq_q, dim), scale).reshape(heads, seq_q, dim)
    scores = bmm(scaled, k.transpose(1, 2).contiguous(), out_dtype=torch.float32)
    probs = normalization.softmax(scores.reshape(heads * seq_q, seq_k), in_place=True).reshape(heads, seq_q, seq_k)
    trace(f"attention composed {tuple(q.shape)} x {tuple(k.shape)}")
    return bmm(probs.to(q.dtype), v)


def explain_attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None) -> str:
    _check(q, k, v)
    if fused(q, k, v):
        return "native: attention_kernel (tcgen05, 128 queries x 128 keys per step, scores in TMEM)"
    return "native: composed bmm + softmax + bmm (scores pass through HBM once in f32)"


attention.explain = explain_attention  # type: ignore[attr-defined]
