"""Parity metrics and the tolerances the hot path is held to.

f32 paths: relative Frobenius error <= 1e-5. bf16 paths with f32 accumulation:
max abs error <= 1e-2 * max|ref|. The reference's own tests use the max-norm
relative error (e.g. ``tests/test_cpu_utils_softmax.py:33``,
``tests/test_cpu_utils_split_k_bmm.py:50``): :func:`max_norm_rel`.
"""

from __future__ import annotations

import torch

F32_REL_FROBENIUS = 1e-5
BF16_MAX_ABS_REL = 1e-2


def rel_frobenius(actual: torch.Tensor, ref: torch.Tensor) -> float:
    a, r = actual.detach().double().cpu(), ref.detach().double().cpu()
    denom = r.norm().item()
    return (a - r).norm().item() / (denom if denom > 0 else 1.0)


def max_norm_rel(actual: torch.Tensor, ref: torch.Tensor) -> float:
    a, r = actual.detach().double().cpu(), ref.detach().double().cpu()
    denom = r.abs().max().item() if r.numel() else 0.0
    if a.numel() == 0:
        return 0.0
    return (a - r).abs().max().item() / (denom if denom > 0 else 1.0)


def metric_for(dtype: torch.dtype, actual: torch.Tensor, ref: torch.Tensor) -> tuple[float, float]:
    """``(error, bound)`` under the bar of the operand type ``dtype``."""
    if dtype == torch.float32:
        return rel_frobenius(actual, ref), F32_REL_FROBENIUS
    return max_norm_rel(actual, ref), BF16_MAX_ABS_REL


def assert_parity(dtype: torch.dtype, actual: torch.Tensor, ref: torch.Tensor, what: str = "") -> float:
    assert actual.shape == ref.shape, f"{what}: shape {tuple(actual.shape)} != {tuple(ref.shape)}"
    a_nan, r_nan = actual.isnan().cpu(), ref.isnan().cpu()
    assert torch.equal(a_nan, r_nan), f"{what}: NaN positions differ"
    if r_nan.any():
        keep = ~r_nan
        actual, ref = actual.cpu()[keep], ref.cpu()[keep]
    error, bound = metric_for(dtype, actual, ref)
    assert error <= bound, f"{what}: error {error:.3e} above {bound:.1e} for {dtype}"
    return error
