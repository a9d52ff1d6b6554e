"""The adapters that run the reference's Helion kernel bodies natively, called with
the arguments the reference's host code passes (constexpr wrappers, 3-D/4-D operand
views, ``out=`` tensors), against the oracle."""

from __future__ import annotations

import pytest
import torch

from helpers import cuda
from oracle import checks
from oracle import ops as ref

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


class ConstExpr:
    """Stand-in for ``hl.constexpr``: a wrapper with ``.value``."""

    def __init__(self, value) -> None:
        self.value = value


def body(name: str, *params: str):
    """A function with the name and parameter list of one of the reference's bodies."""
    namespace: dict = {}
    exec(f"def {name}({', '.join(params)}):\n    raise AssertionError('bodies never run')", namespace)
    return namespace[name]


def adapter(name: str, *params: str, block_sizes=None):
    from helion_mlir_backend import bodies

    found = bodies.adapter_for(body(name, *params), block_sizes)
    assert found is not None, name
    return found


def identity_epilogue(x):
    return x


identity_epilogue.__module__ = "helion_mlir_utils.matmul"  # as the reference's own object would be


def _second_operand(y, extra):
    return y


def test_rowwise_and_reduction_bodies() -> None:
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(40, 300, generator=gen)
    out = adapter("_softmax_kernel", "x", "whole", "in_place=False")(cuda(x), ConstExpr(256), ConstExpr(False))
    assert checks.max_norm_rel(out.cpu(), ref.softmax(x)) < 1e-6
    w, b = torch.randn(96, generator=gen), torch.randn(96, generator=gen)
    x3 = torch.randn(10, 4, 24, generator=gen)
    run = adapter("_group_norm_kernel", "x3", "weight", "bias", "extra", "eps", "epilogue", "in_place=False")
    out = run(cuda(x3), cuda(w.view(4, 24)), cuda(b.view(4, 24)), cuda(w.view(4, 24)), ConstExpr(1e-5), _second_operand)
    assert out.shape == (10, 4, 24)
    assert checks.rel_frobenius(out.cpu().reshape(10, 96), ref.group_norm(x3.reshape(10, 96), 4, w, b, 1e-5)) < 1e-5
    xr = torch.randn(33, 65, generator=gen)
    assert checks.rel_frobenius(adapter("_row_sum_kernel", "x", "epilogue")(cuda(xr), torch.relu).cpu(), ref.row_sum(xr, torch.relu)) < 1e-5
    assert checks.rel_frobenius(adapter("_column_sum_kernel", "x")(cuda(xr)).cpu(), ref.column_sum(xr)) < 1e-5
    vec = torch.randn(65, generator=gen)
    out = adapter("_matvec_kernel", "a", "x")(cuda(xr), cuda(vec))
    assert out.shape == (33,) and checks.rel_frobenius(out.cpu(), (xr.double() @ vec.double()).float()) < 1e-5
    out = adapter("_scalar_mul_kernel", "a", "s")(cuda(xr), ConstExpr(1.5))
    assert torch.equal(out.cpu(), xr * 1.5)
    out = adapter("_leaky_relu_kernel", "x", "negative_slope")(cuda(xr), ConstExpr(0.2))
    assert torch.equal(out.cpu(), torch.nn.functional.leaky_relu(xr, 0.2))


def test_gemm_bodies() -> None:
    gen = torch.Generator().manual_seed(2)
    a = torch.randn(130, 136, generator=gen).bfloat16()
    b = torch.randn(136, 104, generator=gen).bfloat16()
    bias = torch.randn(104, generator=gen).bfloat16()
    fused = adapter("_matmul_fused_pack", "a", "b", "bias", "scale", "shift", "epilogue", "k_chunked", "k_even", "trans_a",
                    "trans_b", "out=None", block_sizes=(128, 128, 128, 64))
    out_buffer = torch.empty(130, 104, dtype=BF16, device="cuda")
    out = fused(cuda(a), cuda(b.T.contiguous()), cuda(bias), None, None, torch.relu, ConstExpr(128), ConstExpr(128),
                ConstExpr(False), ConstExpr(True), out_buffer)
    assert out.data_ptr() == out_buffer.data_ptr()
    checks.assert_parity(BF16, out.cpu(), ref.matmul(a, b, bias=bias, epilogue=torch.relu), "fused_pack")

    af, bf = a.float(), b.float()
    a4, b4 = ref.pack_a_blocked(af), ref.pack_b_blocked(bf)
    bias3 = ref.pad_2d(bias.float().reshape(1, -1), 1, 128).reshape(4, 1, 32)
    out = adapter("_matmul_blocked_kernel_bias", "a4", "b4", "bias3", "epilogue")(cuda(a4), cuda(b4), cuda(bias3), identity_epilogue)
    assert out.shape == (5, 32, 4, 32)
    expect = ref.matmul(af, bf, bias=bias.float())
    assert checks.rel_frobenius(out.cpu().reshape(160, 128)[:130, :104], expect) < 1e-5

    packed = ref.pack_b_vnni_t(b.T.contiguous(), 64)  # [2, 80, 64, 2]: N padded to 128, K to 160
    a3 = a.reshape(130, 68, 2)
    bias2 = ref.pad_2d(bias.reshape(1, -1), 1, 128).reshape(2, 64)
    run = adapter("_matmul_prepacked_vnni", "a3", "b4", "bias2", "scale2", "shift2", "epilogue", "pairs_chunked",
                  "pairs_even", "out=None")
    out = run(cuda(a3), cuda(packed), cuda(bias2), None, None, identity_epilogue, ConstExpr(64), ConstExpr(64))
    assert out.shape == (130, 2, 64)
    checks.assert_parity(BF16, out.cpu().reshape(130, 128)[:, :104], ref.matmul(a, b, bias=bias), "prepacked_vnni")

    a32 = torch.randn(64, 512, generator=gen)
    b32 = torch.randn(512, 128, generator=gen)
    partials = adapter("_split_k_partials", "a3", "b3")(cuda(a32.view(64, 4, 128)), cuda(b32.view(4, 128, 128)))
    assert partials.shape == (4, 64, 128) and partials.dtype == F32
    total = adapter("_sum_partials", "partials", "dtype")(partials, F32)
    assert checks.rel_frobenius(total.cpu(), ref.matmul_split_k(a32, b32, 4)) < 1e-5

    ab = torch.randn(3, 64, 128, generator=gen).bfloat16()
    bb = torch.randn(3, 128, 96, generator=gen).bfloat16()
    out_buffer = torch.empty(3, 64, 96, dtype=BF16, device="cuda")
    out = adapter("_bmm_batched", "a", "b", "out")(cuda(ab), cuda(bb), out_buffer)
    checks.assert_parity(BF16, out.cpu(), ref.bmm(ab, bb), "bmm_batched")


def test_pack_bodies() -> None:
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(70, 45, generator=gen)
    out = adapter("_pack_a_kernel", "a", "m_pad", "k_pad")(cuda(x), ConstExpr(96), ConstExpr(64))
    assert torch.equal(out.cpu(), ref.pack_a_blocked(x))
    out = adapter("_pack_b_vnni_kernel", "b", "k_pad", "n_pad")(cuda(x), ConstExpr(96), ConstExpr(64))
    assert torch.equal(out.cpu(), ref.pack_b_blocked_vnni(x))
    out = adapter("_pad_kernel", "x", "rows", "cols")(cuda(x), ConstExpr(96), ConstExpr(64))
    assert torch.equal(out.cpu(), ref.pad_2d(x, 96, 64))
    w = torch.randn(128, 64, generator=gen).bfloat16()
    out = adapter("_pack_b_vnni_panels_kernel_t", "b3_t", "panel")(cuda(w.view(128, 32, 2)), ConstExpr(64))
    assert torch.equal(out.cpu(), ref.pack_b_vnni_t(w, 64))
