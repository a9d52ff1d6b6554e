"""Kernel bodies recognised by structure run on the native GEMM with the epilogue
the store expression spells, against the same expression in f32 on the CPU."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import test_structure as bodies
from helpers import cuda
from oracle import checks

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


def native(fn, block_sizes=(64, 64, 64)):
    from helion_mlir_backend import inject

    run = inject.recognise(fn, {"block_sizes": list(block_sizes)})
    assert run is not None, fn.__name__
    return run


def test_recognised_bodies_match_their_expression(built_library) -> None:
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(200, 160, generator=gen).bfloat16()
    y = torch.randn(160, 136, generator=gen).bfloat16()
    xf, yf = x.float(), y.float()

    out = native(bodies.plain)(*cuda(x, y))
    assert out.dtype == F32 and checks.rel_frobenius(out.cpu(), xf @ yf) < 1e-5

    w = (torch.randn(136, 160, generator=gen) / 12).bfloat16()
    b = torch.randn(136, generator=gen).bfloat16()
    out = native(bodies.linear_gelu)(*cuda(x, w, b))
    want = F.gelu(xf @ w.float().T + b.float(), approximate="tanh")
    assert out.dtype == BF16
    checks.assert_parity(BF16, out.cpu(), want, "linear_gelu body")

    xt = x.t().contiguous()  # stored [K, M]
    gamma, beta, bias = (torch.randn(136, generator=gen).bfloat16() for _ in range(3))
    out = native(bodies.affine)(*cuda(xt, y, gamma, beta, bias), 0.5)  # the body's own slope literal wins
    want = F.leaky_relu((xf @ yf + bias.float()) * gamma.float() + beta.float(), 0.2)
    checks.assert_parity(BF16, out.cpu(), want, "affine body")

    out = native(bodies.scalar_ops)(*cuda(x, y), alpha=0.03)
    checks.assert_parity(BF16, out.cpu(), torch.sigmoid(0.03 * (xf @ yf) - 0.5), "scalar body")


def test_f32_operands_and_unrecognised(built_library) -> None:
    from helion_mlir_backend import inject

    gen = torch.Generator().manual_seed(78)
    x, y = torch.randn(96, 200, generator=gen), torch.randn(200, 72, generator=gen)
    out = native(bodies.plain)(*cuda(x, y))
    assert checks.rel_frobenius(out.cpu(), (x.double() @ y.double()).float()) < 1e-5
    assert inject.recognise(bodies.row_softmax_after, None) is None
    with pytest.raises(TypeError, match="missing"):
        native(bodies.plain)(cuda(x))
