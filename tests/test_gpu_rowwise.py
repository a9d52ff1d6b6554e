"""Row-wise kernels, reductions and element-wise kernels against the CPU oracle:
ragged and unaligned rows, one column, long rows, NaN/inf rows, in-place,
both dtypes, and the C4 configuration."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from helpers import bits
from helpers import cuda
from oracle import checks
from oracle import inputs
from oracle import ops as ref

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32
SHAPES = [(32, 128), (64, 256), (16, 129), (33, 257), (2, 65), (1, 127), (5, 2), (7, 1), (3, 4096), (9, 4100),
          (4, 8192), (3, 10000), (2, 40000), (300, 64), (1000, 24),
          # 512 threads per row: 32 values each (f32 and bf16), 64 each (bf16 only; f32 takes two passes)
          (3, 16384), (2, 20000), (3, 32768), (2, 24584)]


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


def tol(dtype) -> float:
    return 1e-6 if dtype == F32 else 1e-2


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", SHAPES)
def test_softmax(ops, shape, dtype) -> None:
    gen = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    x = (torch.randn(*shape, generator=gen) * 3).to(dtype)
    out = ops.softmax(cuda(x))
    assert checks.max_norm_rel(out.cpu(), ref.softmax(x)) < tol(dtype)
    y = cuda(x).clone()
    pointer = y.data_ptr()
    in_place = ops.softmax(y, in_place=True)
    assert in_place.data_ptr() == pointer and torch.equal(bits(in_place), bits(out))


def test_softmax_special_rows(ops) -> None:
    x = torch.randn(6, 300)
    x[0, 5] = float("nan")
    x[1, 7] = float("inf")
    x[2, :] = float("-inf")
    x[3, 9] = float("-inf")
    x[4, :] = 1e30
    out, expect = ops.softmax(cuda(x)).cpu(), torch.softmax(x, -1)
    assert torch.equal(out.isnan(), expect.isnan())
    keep = ~expect.isnan()
    assert (out[keep] - expect[keep]).abs().max() < 1e-6
    assert out[0].isnan().all() and out[1].isnan().all() and out[2].isnan().all()


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(8, 96, 4), (33, 130, 1), (5, 4096, 1), (4, 4100, 1), (6, 768, 12), (2, 40000, 1), (3, 20000, 2),
                                   (2, 16384, 1), (2, 32768, 1), (2, 24584, 1), (2, 65536, 2)])
def test_group_norm(ops, shape, dtype) -> None:
    m, c, groups = shape
    gen = torch.Generator().manual_seed(m + c + groups)
    x = (torch.randn(m, c, generator=gen) * 2 + 0.5).to(dtype)
    w = (1 + 0.1 * torch.randn(c, generator=gen)).to(dtype)
    b = (0.1 * torch.randn(c, generator=gen)).to(dtype)
    out = ops.group_norm(cuda(x), groups, cuda(w), cuda(b), 1e-5)
    expect = ref.group_norm(x, groups, w, b, 1e-5)
    assert checks.max_norm_rel(out.cpu(), expect) < (2e-6 if dtype == F32 else 1e-2)
    if groups == 1:
        torch_ln = F.layer_norm(x.float(), (c,), w.float(), b.float(), 1e-5)
        assert checks.max_norm_rel(ops.layer_norm(cuda(x), cuda(w), cuda(b)).cpu().float(), torch_ln) < (2e-6 if dtype == F32 else 1e-2)
    y = cuda(x).clone()
    assert torch.equal(ops.group_norm(y, groups, cuda(w), cuda(b), 1e-5, in_place=True), out)


def test_group_norm_epilogues(ops) -> None:
    gen = torch.Generator().manual_seed(3)
    x, w, b, extra = (torch.randn(9, 64, generator=gen), torch.randn(64, generator=gen), torch.randn(64, generator=gen),
                      torch.randn(64, generator=gen))
    dx, dw, db, de = cuda(x, w, b, extra)
    for fused, fn in ((ops.mul_extra, torch.mul), (torch.add, torch.add)):
        out = ops.group_norm(dx, 2, dw, db, 1e-5, fused, de)
        assert checks.rel_frobenius(out.cpu(), ref.group_norm(x, 2, w, b, 1e-5, fn, extra)) < 1e-5
    out = ops.group_norm(dx, 2, dw, db, 1e-5, torch.relu)
    assert checks.rel_frobenius(out.cpu(), torch.relu(ref.group_norm(x, 2, w, b, 1e-5))) < 1e-5
    custom = lambda y, e: y * torch.tanh(e)  # noqa: E731
    out = ops.group_norm(dx, 2, dw, db, 1e-5, custom, de)
    assert checks.rel_frobenius(out.cpu(), ref.group_norm(x, 2, w, b, 1e-5, custom, extra)) < 1e-5
    out = ops.group_norm(dx, 4, None, None, 1e-5)
    assert checks.rel_frobenius(out.cpu(), ref.group_norm(x, 4, None, None, 1e-5)) < 1e-5


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(8, 96), (33, 130), (5, 4096), (2, 40000), (3, 16384), (2, 32768), (2, 20008)])
def test_rms_norm(ops, shape, dtype) -> None:
    gen = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=gen) * 2).to(dtype)
    w = (1 + 0.1 * torch.randn(shape[1], generator=gen)).to(dtype)
    out = ops.rms_norm(cuda(x), cuda(w), 1e-5)
    assert checks.max_norm_rel(out.cpu(), ref.rms_norm(x, w, 1e-5)) < (2e-6 if dtype == F32 else 1e-2)
    assert checks.max_norm_rel(ops.rms_norm(cuda(x)).cpu(), ref.rms_norm(x, None, 1e-5)) < (2e-6 if dtype == F32 else 1e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("n", [768, 1000, 1536, 2560, 3072, 5120, 6144, 10240, 11008, 12288, 14336, 16384, 17000, 20000,
                               24000, 25600, 30000, 32000])
def test_row_lengths_that_whole_warps_cover(ops, n, dtype) -> None:
    """Row lengths that no power-of-two number of threads covers run with a number of whole
    warps per row that does (32 threads x 24 values for 768, 192 x 64 for bf16 12288 ...);
    1000, 11008 and 20000 have no such cover: the last vectors of some threads lie beyond
    the row and are filled, not loaded. bf16 rows beyond 16384 values take 512 threads x 40,
    48, 56 or 64 values; with a tail the norms of 56 and 64 keep the row in its 16-bit form
    and widen it again in every pass. More rows than one wave of CTAs holds, a row
    count that leaves the last CTA of two-row CTAs half empty, and the grouped form whose
    parameters depend on the row."""
    rows = 1481
    gen = torch.Generator().manual_seed(n)
    x = (torch.randn(rows, n, generator=gen) * 2 + 0.25).to(dtype)
    w = (1 + 0.1 * torch.randn(n, generator=gen)).to(dtype)
    b = (0.1 * torch.randn(n, generator=gen)).to(dtype)
    dx, dw, db = cuda(x, w, b)
    bound = 2e-6 if dtype == F32 else 1e-2
    assert checks.max_norm_rel(ops.softmax(dx).cpu(), ref.softmax(x)) < tol(dtype)
    assert checks.max_norm_rel(ops.layer_norm(dx, dw, db, 1e-5).cpu(), ref.layer_norm(x, w, b, 1e-5)) < bound
    assert checks.max_norm_rel(ops.rms_norm(dx, dw, 1e-5).cpu(), ref.rms_norm(x, w, 1e-5)) < bound
    groups = 4
    xg = x[:, : n // groups * groups].reshape(rows, -1)[:37]
    wg, bg = w[: xg.shape[1]], b[: xg.shape[1]]
    out = ops.group_norm(cuda(xg), groups, cuda(wg), cuda(bg), 1e-5)
    assert checks.max_norm_rel(out.cpu(), ref.group_norm(xg, groups, wg, bg, 1e-5)) < bound
    # an activation after the norm takes the masked kernel with the same threads per row
    out = ops.group_norm(cuda(xg), groups, cuda(wg), cuda(bg), 1e-5, torch.relu)
    assert checks.max_norm_rel(out.cpu(), torch.relu(ref.group_norm(xg, groups, wg, bg, 1e-5))) < bound


@pytest.mark.parametrize("shape", [(1481, 4096), (1, 4096), (3, 2048), (777, 1024), (4099, 128), (35, 1000), (513, 768),
                                   (129, 3072), (64, 8192), (5, 256)])
def test_bf16_rows_with_f32_parameters(ops, shape) -> None:
    """bf16 activations with f32 weight and bias (mixed-precision modules): layer_norm of rows
    of up to 4096 values runs two rows per group of threads, so odd row counts, one row, a
    tail (1000) and rows that share a warp are all here; rms_norm and wider rows take the
    one-row form with the same operands."""
    rows, n = shape
    gen = torch.Generator().manual_seed(rows * 7 + n)
    x = (torch.randn(rows, n, generator=gen) * 2 + 0.25).to(BF16)
    w = 1 + 0.1 * torch.randn(n, generator=gen)
    b = 0.1 * torch.randn(n, generator=gen)
    dx, dw, db = cuda(x, w, b)
    out = ops.layer_norm(dx, dw, db, 1e-5)
    assert out.dtype == BF16
    assert checks.max_norm_rel(out.cpu(), ref.layer_norm(x, w, b, 1e-5)) < 1e-2
    # f32 parameters that are exact in bf16 against the same parameters given as bf16 (another
    # instantiation, which adds the row up in another order: not the same bits)
    w16, b16 = w.to(BF16), b.to(BF16)
    exact = ops.layer_norm(dx, cuda(w16.float()), cuda(b16.float()), 1e-5)
    assert checks.max_norm_rel(exact.cpu(), ops.layer_norm(dx, cuda(w16), cuda(b16), 1e-5).cpu()) < 1e-2
    assert torch.equal(bits(ops.layer_norm(dx, dw, db, 1e-5)), bits(out))  # and the same bits every run
    y = dx.clone()
    assert torch.equal(bits(ops.layer_norm(y, dw, db, 1e-5, in_place=True)), bits(out))
    assert checks.max_norm_rel(ops.rms_norm(dx, dw, 1e-5).cpu(), ref.rms_norm(x, w, 1e-5)) < 1e-2


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(700, 50304), (301, 32768), (150, 128256), (75, 131072), (300, 65536), (200, 40000),
                                   (40, 262144), (9, 300000)])
def test_rows_longer_than_registers_hold(ops, shape, dtype) -> None:
    """Rows of more values than one CTA's registers hold (16 Ki f32, 32 Ki bf16) take the
    two-pass kernel, one CTA per row: more rows than resident CTAs (so that every CTA walks
    several rows), row lengths of vocabulary sizes, rows with NaN and infinities, in place,
    and the grouped form."""
    rows, n = shape
    gen = torch.Generator().manual_seed(rows + n)
    x = (torch.randn(rows, n, generator=gen) * 2 + 0.25).to(dtype)
    w = (1 + 0.1 * torch.randn(n, generator=gen)).to(dtype)
    b = (0.1 * torch.randn(n, generator=gen)).to(dtype)
    dx, dw, db = cuda(x, w, b)
    bound = 2e-6 if dtype == F32 else 1e-2
    soft = ops.softmax(dx)
    assert checks.max_norm_rel(soft.cpu(), ref.softmax(x)) < tol(dtype)
    assert torch.equal(ops.softmax(dx), soft)  # fixed order over the warps
    assert checks.max_norm_rel(ops.layer_norm(dx, dw, db, 1e-5).cpu(), ref.layer_norm(x, w, b, 1e-5)) < bound
    assert checks.max_norm_rel(ops.rms_norm(dx, dw, 1e-5).cpu(), ref.rms_norm(x, w, 1e-5)) < bound
    y = dx.clone()
    assert torch.equal(ops.softmax(y, in_place=True), soft)
    special = x[:6].clone().float()
    special[0, n - 3] = float("nan")
    special[1, 7] = float("inf")
    special[2, :] = float("-inf")
    special[3, n // 2] = float("-inf")
    special[4, :] = 1e30
    special = special.to(dtype)
    out, expect = ops.softmax(cuda(special)).cpu().float(), torch.softmax(special.float(), -1)
    assert torch.equal(out.isnan(), expect.isnan())
    keep = ~expect.isnan()
    assert (out[keep] - expect[keep]).abs().max() < (1e-6 if dtype == F32 else 1e-2)
    groups = 2  # the grouped form: rows of n / 2 values whose parameters depend on the row
    out = ops.group_norm(dx[:33], groups, dw, db, 1e-5)
    assert checks.max_norm_rel(out.cpu(), ref.group_norm(x[:33], groups, w, b, 1e-5)) < bound


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_c4_configuration(ops, dtype) -> None:
    """x [rows, 4096] ~N(0,2) with 1% of entries at +-30; softmax, layer_norm, rms_norm and the chain."""
    data = inputs.c4_rows(m=512, n=4096, dtype=dtype)
    x, gamma, beta = data["x"], data["gamma"], data["beta"]
    dx, dg, db = cuda(x, gamma, beta)
    bound = 1e-5 if dtype == F32 else 1e-2
    sm = ops.softmax(dx)
    checks.assert_parity(dtype, sm.cpu(), ref.softmax(x), "softmax")
    ln = ops.layer_norm(dx, dg, db, 1e-5)
    checks.assert_parity(dtype, ln.cpu(), ref.layer_norm(x, gamma, beta, 1e-5), "layer_norm")
    rn = ops.rms_norm(dx, dg, 1e-5)
    checks.assert_parity(dtype, rn.cpu(), ref.rms_norm(x, gamma, 1e-5), "rms_norm")
    chain = ops.layer_norm(sm, dg, db, 1e-5)
    # the chain's reference starts from the kernel's own (rounded) softmax
    assert checks.max_norm_rel(chain.cpu(), ref.layer_norm(sm.cpu(), gamma, beta, 1e-5)) < (2e-4 if dtype == F32 else 2e-2)
    # properties that hold at any size
    assert (sm.float().sum(-1) - 1).abs().max() < (1e-5 if dtype == F32 else 2e-2)
    assert torch.equal(ops.softmax(dx), sm)
    shifted = ops.softmax((dx.float() + 3.0).to(dtype)) if dtype == F32 else None
    if shifted is not None:
        assert checks.max_norm_rel(shifted, sm) < 1e-5  # shift invariance
    assert bound > 0


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(33, 65), (16, 520), (1, 1), (7, 4096), (300, 24), (3, 70001), (2000, 8),
                                   # row counts around the four rows a group of threads takes in row_dot on bf16 rows
                                   (1, 4096), (5, 1536), (1026, 64), (4099, 512), (1213, 5120)])
def test_row_and_column_reductions(ops, shape, dtype) -> None:
    m, n = shape
    gen = torch.Generator().manual_seed(m * 7 + n)
    x = torch.randn(m, n, generator=gen).to(dtype)
    v = torch.randn(n, generator=gen)
    dx = cuda(x)
    bound = 1e-5 if dtype == F32 else 1e-2
    assert checks.max_norm_rel(ops.row_sum(dx).cpu(), ref.row_sum(x)) < bound
    assert ops.row_sum(dx).shape == (m, 1) and ops.row_sum(dx).dtype == dtype
    assert checks.max_norm_rel(ops.row_sum(dx, torch.relu).cpu(), ref.row_sum(x, torch.relu)) < bound
    assert checks.max_norm_rel(ops.row_dot(dx, cuda(v)).cpu(), ref.row_dot(x, v)) < bound
    assert torch.equal(bits(ops.row_dot(dx, cuda(v))), bits(ops.row_dot(dx, cuda(v))))
    vec = torch.randn(n, 1, generator=gen).to(dtype)
    assert checks.max_norm_rel(ops.matvec(dx, cuda(vec)).cpu(), ref.matvec(x, vec)) < bound
    col = ops.column_sum(dx)
    assert col.dtype == F32 and col.shape == (n,)
    assert checks.max_norm_rel(col.cpu(), ref.column_sum(x)) < 1e-5
    assert torch.equal(col, ops.column_sum(dx))  # fixed order: same bits
    custom = ops.row_sum(dx, lambda t: t * 0.5 + 1)
    assert checks.max_norm_rel(custom.cpu(), ref.row_sum(x, lambda t: t * 0.5 + 1)) < bound


def test_column_sum_tall(ops) -> None:
    """Many rows: the two-stage path with partial sums in scratch memory."""
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(20000, 96, generator=gen)
    out = ops.column_sum(cuda(x))
    assert checks.max_norm_rel(out.cpu(), ref.column_sum(x)) < 1e-5
    xb = x.bfloat16()
    assert checks.max_norm_rel(ops.column_sum(cuda(xb)).cpu(), ref.column_sum(xb)) < 1e-5


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("shape", [(9, 1030), (1,), (4, 5, 7), (0, 4), (1 << 20,)])
def test_elementwise(ops, shape, dtype) -> None:
    gen = torch.Generator().manual_seed(len(shape))
    x = torch.randn(*shape, generator=gen).to(dtype)
    if x.numel() > 3:
        x.view(-1)[1] = float("nan")
        x.view(-1)[2] = -0.0
    dx = cuda(x)
    assert torch.equal(bits(ops.relu(dx)), bits(torch.relu(x)))
    assert torch.equal(bits(ops.leaky_relu(dx, 0.1)), bits(F.leaky_relu(x, 0.1)))
    assert torch.equal(bits(ops.scalar_mul(dx, 1.7)), bits(x * 1.7))
    assert torch.equal(bits(ops.scalar_mul(dx, torch.tensor(-0.25))), bits(x * -0.25))
    odd = cuda(torch.randn(1025, generator=gen).to(dtype))[1:]  # unaligned base
    assert torch.equal(bits(ops.relu(odd)), bits(torch.relu(odd.cpu())))


def test_seeded_shape_sweep(ops) -> None:
    """Random row counts and lengths (log-uniform up to 70000 columns) through softmax,
    layer_norm and rms_norm in both dtypes: every threads-per-row choice from 4 to 1024,
    masked and whole vectors, and the long-row kernel."""
    import math
    import random

    rng = random.Random(2024)
    gen = torch.Generator().manual_seed(2024)
    for case in range(36):
        n = max(1, int(math.exp(rng.uniform(0.0, math.log(70000.0)))))
        if case % 3 == 0:
            n = max(8, n // 8 * 8)  # whole 16-byte vectors in both dtypes
        m = rng.randint(1, max(1, min(300, 400000 // n)))
        x = torch.randn(m, n, generator=gen) * rng.choice([0.5, 3.0, 20.0])
        w, b = torch.randn(n, generator=gen), torch.randn(n, generator=gen)
        for dtype in (F32, BF16):
            xd, wd, bd = x.to(dtype), w.to(dtype), b.to(dtype)
            dx = cuda(xd)
            what = f"{m}x{n} {dtype}"
            sm = ops.softmax(dx).cpu()
            assert checks.max_norm_rel(sm, ref.softmax(xd)) < tol(dtype), "softmax " + what
            ln = ops.layer_norm(dx, cuda(wd), cuda(bd), 1e-5).cpu()
            checks.assert_parity(dtype, ln, ref.layer_norm(xd, wd, bd, 1e-5).float(), "layer_norm " + what)
            rn = ops.rms_norm(dx, cuda(wd), 1e-5).cpu()
            checks.assert_parity(dtype, rn, ref.rms_norm(xd, wd, 1e-5).float(), "rms_norm " + what)
