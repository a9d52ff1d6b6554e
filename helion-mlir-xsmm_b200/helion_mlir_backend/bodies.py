"""Kernel bodies this backend recognises by name, and how each is run natively.

A Helion kernel that selects backend ``"mlir"`` reaches
``BoundKernel.compile_config`` (patched by :func:`..inject.install`). The
reference compiles the body there. This backend instead looks the body up: the
Helion kernels of the reference's operator set (``helion_mlir_utils/*.py``, e.g.
``_softmax_kernel`` normalization.py:28, ``_matmul_fused_pack`` matmul.py:259,
``_matmul_prepacked_vnni`` matmul.py:534) are known by function name and parameter
list, and each maps to an adapter that takes the arguments exactly as the
reference's host code passes them (constexpr wrappers included) and calls the
hand-written kernels. So user code that keeps the reference's
``helion_mlir_utils`` sources and only swaps the backend package still runs on the
B200 kernels; the ``block_sizes`` of the kernel's config arrive as tile hints.
"""

from __future__ import annotations

import inspect
from typing import Callable

import torch
from torch import Tensor

Adapter = Callable[..., object]


def _value(x: object) -> object:
    """Unwrap ``hl.constexpr(...)`` (anything with a ``.value``) to the plain value."""
    return getattr(x, "value", x)


def _ops():
    import helion_mlir_utils

    return helion_mlir_utils


def _flat(t: Tensor | None) -> Tensor | None:
    return None if t is None else t.reshape(-1)


def _into(out: Tensor | None, result: Tensor) -> Tensor:
    if out is None:
        return result
    out.copy_(result.view(out.shape))
    return out


def _hint(block_sizes: tuple[int, ...] | None) -> tuple[int, ...] | None:
    return tuple(block_sizes[:3]) if block_sizes and len(block_sizes) >= 3 else None


def _make(block_sizes: tuple[int, ...] | None) -> dict[str, tuple[tuple[str, ...], Adapter]]:
    """``name -> (leading parameter names, adapter)`` for one tile config."""
    ops = _ops()
    hint = _hint(block_sizes)

    def softmax(x, whole=None, in_place=False):
        return ops.softmax(x, in_place=bool(_value(in_place)))

    def group_norm(x3, weight, bias, extra, eps, epilogue, in_place=False):
        m, groups, size = map(int, x3.shape)
        out = ops.group_norm(
            x3.reshape(m, groups * size), groups, _flat(weight), _flat(bias), float(_value(eps)), epilogue,
            _flat(extra), bool(_value(in_place)),
        )
        return out.view(m, groups, size)

    def fused_pack(a, b, bias, scale, shift, epilogue, k_chunked, k_even, trans_a, trans_b, out=None):
        result = ops.matmul(
            a, b, trans_a=bool(_value(trans_a)), trans_b=bool(_value(trans_b)), bias=bias, epilogue=epilogue,
            block_sizes=hint, scale=scale, shift=shift,
        )
        return _into(out, result)

    def f32_fused_pack(a, b, epilogue, trans_a, trans_b):
        return ops.matmul(a, b, trans_a=bool(_value(trans_a)), trans_b=bool(_value(trans_b)), epilogue=epilogue)

    def blocked(a4, b4, epilogue, bias3=None, scale3=None, post_bias3=None):
        mb, kb = int(a4.shape[0]), int(a4.shape[1])
        nb = int(b4.shape[0])
        out = ops.matmul_blocked(
            a4, b4, mb * 32, nb * 32, kb * 32, bias=_flat(bias3), epilogue=epilogue, scale=_flat(scale3),
            shift=_flat(post_bias3),
        )
        return out.view(mb, 32, nb, 32)

    def blocked_bias(a4, b4, bias3, epilogue):
        return blocked(a4, b4, epilogue, bias3)

    def blocked_affine(a4, b4, bias3, scale3, post_bias3, epilogue):
        return blocked(a4, b4, epilogue, bias3, scale3, post_bias3)

    def prepacked_vnni(a3, b4, bias2, scale2, shift2, epilogue, pairs_chunked=None, pairs_even=None, out=None):
        m = int(a3.shape[0])
        panels, _, panel, _ = map(int, b4.shape)
        result = ops.matmul_prepacked_b(
            a3.reshape(m, -1), b4, panels * panel, _flat(bias2), epilogue, _flat(scale2), _flat(shift2)
        )
        return _into(out, result.view(m, panels, panel))

    def prepacked_rows(a, b3, bias2, epilogue, out=None):
        m = int(a.shape[0])
        panels, k, panel = map(int, b3.shape)
        result = ops.matmul_prepacked_b(a, b3.view(panels, k // 32, 32, panel), panels * panel, _flat(bias2), epilogue)
        return _into(out, result.view(m, panels, panel))

    def split_k_partials(a3, b3):
        return ops.bmm(a3.permute(1, 0, 2).contiguous(), b3)  # [S, M, C] x [S, C, N], f32

    def sum_partials(partials, dtype):
        splits, m, n = map(int, partials.shape)
        return ops.column_sum(partials.reshape(splits, m * n)).to(_value(dtype)).view(m, n)

    def bmm_direct(a, b):
        return ops.bmm(a, b)

    def bmm_batched(a, b, out):
        return _into(out, ops.bmm(a, b))

    def matvec(a, x):
        return ops.matvec(a, x.reshape(-1, 1)).reshape(int(a.shape[0]))

    def pack(fn):
        def run(x, first, second):
            return fn(x, int(_value(first)), int(_value(second)))

        return run

    def pack_panels(b3_t, panel):
        n, pairs, _ = map(int, b3_t.shape)
        return ops.pack_b_vnni_t(b3_t.reshape(n, 2 * pairs), int(_value(panel)))

    return {
        "_softmax_kernel": (("x", "whole"), softmax),
        "_softmax_one_kernel": (("x",), lambda x: ops.softmax(x)),
        "_group_norm_kernel": (("x3", "weight", "bias", "extra"), group_norm),
        "_matmul_fused_pack": (("a", "b", "bias", "scale", "shift", "epilogue"), fused_pack),
        "_matmul_f32_fused_pack": (("a", "b", "epilogue", "trans_a"), f32_fused_pack),
        "_matmul_blocked_kernel": (("a4", "b4", "epilogue"), blocked),
        "_matmul_blocked_kernel_bias": (("a4", "b4", "bias3"), blocked_bias),
        "_matmul_blocked_kernel_affine": (("a4", "b4", "bias3", "scale3"), blocked_affine),
        "_matmul_prepacked_vnni": (("a3", "b4", "bias2", "scale2"), prepacked_vnni),
        "_matmul_prepacked_rows": (("a", "b3", "bias2"), prepacked_rows),
        "_split_k_partials": (("a3", "b3"), split_k_partials),
        "_sum_partials": (("partials", "dtype"), sum_partials),
        "_bmm_direct": (("a", "b"), bmm_direct),
        "_bmm_batched": (("a", "b", "out"), bmm_batched),
        "_matvec_kernel": (("a", "x"), matvec),
        "_row_sum_kernel": (("x", "epilogue"), lambda x, epilogue: ops.row_sum(x, epilogue)),
        "_row_dot_kernel": (("x", "v", "epilogue"), lambda x, v, epilogue: ops.row_dot(x, v, epilogue)),
        "_column_sum_kernel": (("x",), lambda x: ops.column_sum(x)),
        "_relu_kernel": (("x",), lambda x: ops.relu(x)),
        "_leaky_relu_kernel": (("x", "negative_slope"), lambda x, slope: ops.leaky_relu(x, float(_value(slope)))),
        "_scalar_mul_kernel": (("a", "s"), lambda a, s: ops.scalar_mul(a, float(_value(s)))),
        "_pad_kernel": (("x", "rows", "cols"), pack(ops.pad_2d)),
        "_pack_a_kernel": (("a", "m_pad", "k_pad"), pack(ops.pack_a_blocked)),
        "_pack_a_kernel_t": (("a_t", "m_pad", "k_pad"), pack(ops.pack_a_blocked_t)),
        "_pack_b_kernel": (("b", "k_pad", "n_pad"), pack(ops.pack_b_blocked)),
        "_pack_b_kernel_t": (("b_t", "k_pad", "n_pad"), pack(ops.pack_b_blocked_t)),
        "_pack_b_vnni_kernel": (("b", "k_pad", "n_pad"), pack(ops.pack_b_blocked_vnni)),
        "_pack_b_vnni_kernel_t": (("b_t", "k_pad", "n_pad"), pack(ops.pack_b_blocked_vnni_t)),
        "_pack_b_vnni_panels_kernel_t": (("b3_t", "panel"), pack_panels),
        # the attention bodies of the reference's tests (tests/harness.py:263, tests/test_numerics.py:141)
        "_attention": (("q", "k", "v", "scale", "vnni"), lambda q, k, v, scale, vnni=False: ops.attention(q, k, v, float(_value(scale)))),
        "attention": (("q", "k", "v"), lambda q, k, v: ops.attention(q, k, v, 1.0)),
        # the two-phase packed GEMM of examples/matmul_packed_mlir.py:40-60 (pack both operands
        # into 32x32 blocks, barrier, blocked contraction): one GEMM on the operands as given
        "_gemm_packed": (("a", "b"), lambda a, b: ops.matmul(a, b)),
    }


KNOWN_BODIES = frozenset(
    """_softmax_kernel _softmax_one_kernel _group_norm_kernel _matmul_fused_pack _matmul_f32_fused_pack
    _matmul_blocked_kernel _matmul_blocked_kernel_bias _matmul_blocked_kernel_affine _matmul_prepacked_vnni
    _matmul_prepacked_rows _split_k_partials _sum_partials _bmm_direct _bmm_batched _matvec_kernel _row_sum_kernel
    _row_dot_kernel _column_sum_kernel _relu_kernel _leaky_relu_kernel _scalar_mul_kernel _pad_kernel _pack_a_kernel
    _pack_a_kernel_t _pack_b_kernel _pack_b_kernel_t _pack_b_vnni_kernel _pack_b_vnni_kernel_t
    _pack_b_vnni_panels_kernel_t _attention attention _gemm_packed""".split()
)


def adapter_for(fn: Callable[..., object], block_sizes: tuple[int, ...] | None) -> Adapter | None:
    """The native adapter for kernel body ``fn`` if its name and leading parameter
    names are those of a known body of the operator set, else ``None``."""
    name = getattr(fn, "__name__", None)
    if name not in KNOWN_BODIES:
        return None
    expected, adapter = _make(block_sizes)[name]
    try:
        parameters = tuple(inspect.signature(fn).parameters)
    except (TypeError, ValueError):
        return None
    if parameters[: len(expected)] != expected:
        return None
    return adapter


def same_role(function: object, name: str) -> bool:
    """Whether ``function`` is this package's or the reference's function of that name
    (e.g. ``identity_epilogue``): user code may hold either module's object."""
    return getattr(function, "__name__", None) == name and "helion_mlir_utils" in (getattr(function, "__module__", "") or "")


__all__ = ["KNOWN_BODIES", "adapter_for", "same_role"]
