"""Layout conversions at sizes that exercise the tiled kernels: whole tiles, ragged
edges, sources that are not 16-byte aligned row by row; bit-exact against the oracle."""

from __future__ import annotations

import pytest
import torch

from helpers import cuda
from oracle import ops as ref

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def ops(built_library):
    import helion_mlir_utils

    return helion_mlir_utils


SHAPES = [(32, 32), (64, 512), (300, 520), (257, 1031), (1000, 72), (33, 2049)]


@pytest.mark.parametrize("dtype", [BF16, F32])
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_blocked_packs(ops, rows: int, cols: int, dtype) -> None:
    gen = torch.Generator().manual_seed(rows * 7 + cols)
    x = torch.randn(rows, cols, generator=gen).to(dtype)
    dx = cuda(x)
    for name in ("pack_a_blocked", "pack_a_blocked_t", "pack_b_blocked", "pack_b_blocked_t"):
        assert torch.equal(getattr(ops, name)(dx).cpu(), getattr(ref, name)(x)), name
    # explicit padding beyond the rounded-up size
    rp, cp = (rows + 95) // 32 * 32, (cols + 63) // 32 * 32
    assert torch.equal(ops.pack_a_blocked_t(dx, cp, rp).cpu(), ref.pack_a_blocked_t(x, cp, rp))
    assert torch.equal(ops.pack_b_blocked_t(dx, cp, rp).cpu(), ref.pack_b_blocked_t(x, cp, rp))


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_vnni_packs_and_their_inverses(ops, rows: int, cols: int) -> None:
    gen = torch.Generator().manual_seed(rows * 11 + cols)
    x = torch.randn(rows, cols, generator=gen).bfloat16()
    dx = cuda(x)
    assert torch.equal(ops.pack_b_blocked_vnni(dx).cpu(), ref.pack_b_blocked_vnni(x))
    assert torch.equal(ops.pack_b_blocked_vnni_t(dx).cpu(), ref.pack_b_blocked_vnni_t(x))
    for panel in (32, 64, 128):
        if cols % 2:  # the reference refuses an odd K for this layout
            with pytest.raises(ValueError, match="even K"):
                ops.pack_b_vnni_t(dx, panel)
            continue
        packed = ops.pack_b_vnni_t(dx, panel)
        assert torch.equal(packed.cpu(), ref.pack_b_vnni_t(x, panel)), panel
        back = ops.unpack_b_to_nk(packed)  # [N_pad, K_pad], zero beyond the source
        assert torch.equal(back[:rows, :cols].cpu(), x) and not back[rows:].any() and not back[:, cols:].any()
    back = ops.unpack_b_to_nk(ops.pack_b_blocked_vnni_t(dx))
    assert torch.equal(back[:rows, :cols].cpu(), x)


def test_unaligned_sources(ops) -> None:
    """Rows that start off a 16-byte boundary (a column slice of a wider tensor made contiguous
    is aligned again, so the misalignment comes from an odd leading dimension)."""
    gen = torch.Generator().manual_seed(3)
    for dtype, cols in ((BF16, 133), (BF16, 130), (F32, 67)):
        x = torch.randn(70, cols, generator=gen).to(dtype)
        dx = cuda(x)
        assert torch.equal(ops.pack_a_blocked_t(dx).cpu(), ref.pack_a_blocked_t(x))
        assert torch.equal(ops.pack_b_blocked_t(dx).cpu(), ref.pack_b_blocked_t(x))
        if dtype == BF16:
            assert torch.equal(ops.pack_b_blocked_vnni(dx).cpu(), ref.pack_b_blocked_vnni(x))
            assert torch.equal(ops.pack_b_blocked_vnni_t(dx).cpu(), ref.pack_b_blocked_vnni_t(x))
            if cols % 2 == 0:
                assert torch.equal(ops.pack_b_vnni_t(dx, 64).cpu(), ref.pack_b_vnni_t(x, 64))
