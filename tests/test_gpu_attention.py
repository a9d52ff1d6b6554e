"""Attention on the device: the fused tensor-core kernel (bf16, head size 64/128)
and the composed path (f32, other head sizes) against the reference body's
fixtures and the CPU oracle, with ragged sequence lengths and growing maxima."""

from __future__ import annotations

import pytest
import torch

from helpers import cuda, load_golden
from oracle import checks
from oracle import ops as ref

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def ops(built_library):
    import helion_mlir_utils

    return helion_mlir_utils


@pytest.mark.parametrize("tag", ["d64", "d128", "peaky", "f32"])
def test_golden(ops, tag: str) -> None:
    g = load_golden("attention")
    q, k, v, want = (g[f"{tag}_{name}"] for name in ("q", "k", "v", "out"))
    out = ops.attention(*cuda(q, k, v), float(g[f"{tag}_scale"]))
    assert out.dtype == want.dtype
    checks.assert_parity(q.dtype, out.cpu(), want.float(), f"attention {tag}")


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("seq_q,seq_k", [(1, 1), (5, 130), (128, 128), (200, 77), (257, 511), (384, 1024)])
def test_fused_ragged_lengths(ops, dim: int, seq_q: int, seq_k: int) -> None:
    gen = torch.Generator().manual_seed(seq_q * 1000 + seq_k + dim)
    heads = 3
    q = torch.randn(heads, seq_q, dim, generator=gen).bfloat16()
    k = torch.randn(heads, seq_k, dim, generator=gen).bfloat16()
    v = torch.randn(heads, seq_k, dim, generator=gen).bfloat16()
    scale = dim ** -0.5
    out = ops.attention(*cuda(q, k, v), scale)
    assert "attention_kernel" in ops.attention.explain(*cuda(q, k, v))
    checks.assert_parity(BF16, out.cpu(), ref.attention(q, k, v, scale).float(), f"{seq_q}x{seq_k}x{dim}")


def test_growing_maxima_rescale_the_accumulator(ops) -> None:
    """Keys sorted so that every block's maximum tops the previous one by far more than 2^8."""
    gen = torch.Generator().manual_seed(9)
    heads, seq, dim = 2, 1024, 64
    q = torch.randn(heads, seq, dim, generator=gen).bfloat16()
    k = torch.randn(heads, seq, dim, generator=gen)
    k = (k * torch.linspace(0.1, 12.0, seq).view(1, seq, 1)).bfloat16()  # later keys score ever larger
    v = torch.randn(heads, seq, dim, generator=gen).bfloat16()
    out = ops.attention(*cuda(q, k, v), 1.0)
    assert torch.isfinite(out).all()
    checks.assert_parity(BF16, out.cpu(), ref.attention(q, k, v, 1.0).float(), "growing maxima")
    # default scale and determinism
    a = ops.attention(*cuda(q, k, v))
    assert torch.equal(a, ops.attention(*cuda(q, k, v)))
    checks.assert_parity(BF16, a.cpu(), ref.attention(q, k, v, dim ** -0.5).float(), "default scale")


def test_composed_path_and_edges(ops) -> None:
    gen = torch.Generator().manual_seed(10)
    q, k, v = (torch.randn(2, 70, 48, generator=gen) for _ in range(3))
    out = ops.attention(*cuda(q, k, v), 0.2)
    assert "composed" in ops.attention.explain(*cuda(q, k, v))
    assert checks.rel_frobenius(out.cpu(), ref.attention(q, k, v, 0.2)) < 1e-5
    qb, kb, vb = q.bfloat16(), k.bfloat16(), v.bfloat16()  # bf16 with a head size the fused kernel lacks
    checks.assert_parity(BF16, ops.attention(*cuda(qb, kb, vb), 0.2).cpu(), ref.attention(qb, kb, vb, 0.2).float(), "bf16 d48")
    # no keys: zeros; no queries: empty
    empty_k = torch.zeros(2, 0, 64, dtype=BF16)
    out = ops.attention(*cuda(torch.ones(2, 5, 64, dtype=BF16), empty_k, empty_k), 1.0)
    assert out.shape == (2, 5, 64) and not out.any()
    some_k = torch.ones(2, 9, 64, dtype=BF16)
    assert ops.attention(*cuda(torch.zeros(2, 0, 64, dtype=BF16), some_k, some_k), 1.0).shape == (2, 0, 64)
    with pytest.raises(ValueError, match="do not match"):
        ops.attention(*cuda(q, k[:, :, :32], v), 1.0)
    with pytest.raises(ValueError, match="bf16/f32"):
        ops.attention(*cuda(q.half(), k.half(), v.half()), 1.0)


def test_c_abi_refusals(ops) -> None:
    from helion_mlir_backend import native

    lib = native.module()
    x = torch.zeros(2, 128, 96, dtype=BF16, device="cuda")
    args = (x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr())
    assert lib.b200_attention(native.BF16, *args, 2, 128, 128, 96, 1.0, None) == 2  # head size
    assert lib.b200_attention(native.F32, *args, 2, 128, 128, 64, 1.0, None) == 1  # dtype
    assert lib.b200_attention(native.BF16, None, None, None, None, 2, 128, 128, 64, 1.0, None) == 6  # NULL
    assert lib.b200_attention(native.BF16, x.data_ptr() + 2, *args[1:], 2, 64, 64, 64, 1.0, None) == 4  # alignment
    assert lib.b200_attention(native.BF16, *args, 0, 128, 128, 64, 1.0, None) == 0  # nothing to do


def test_reference_attention_bodies_are_recognised(ops) -> None:
    """A kernel body named and parameterised like the reference's test kernels runs natively."""
    from helion_mlir_backend import inject

    namespace: dict = {}
    exec("def _attention(q, k, v, scale, vnni):\n    raise AssertionError('never run')\n"
         "def attention(q, k, v):\n    raise AssertionError('never run')", namespace)
    g = load_golden("attention")
    q, k, v, want = (g[f"d64_{name}"] for name in ("q", "k", "v", "out"))
    run = inject.recognise(namespace["_attention"], {"block_sizes": [64, 128]})
    assert run is not None
    checks.assert_parity(BF16, run(*cuda(q, k, v), float(g["d64_scale"]), False).cpu(), want.float(), "_attention body")
    plain = inject.recognise(namespace["attention"], None)
    checks.assert_parity(BF16, plain(*cuda(q, k, v)).cpu(), ref.attention(q, k, v, 1.0).float(), "attention body")
