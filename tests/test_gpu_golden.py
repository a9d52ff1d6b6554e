"""The CUDA kernels against the fixtures produced by the reference's own operator
code (tests/golden/*.npz): same inputs, through the Python operators and the C ABI."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from helpers import bits
from helpers import cuda
from helpers import load_golden
from oracle import checks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_layouts_bit_exact(ops, tag: str) -> None:
    g = load_golden(f"layouts_{tag}")
    x, w = cuda(g["x"], g["w"])
    x_t = x.T.contiguous()
    assert torch.equal(ops.pad_2d(x, 96, 64).cpu(), g["pad"])
    assert torch.equal(ops.pack_a_blocked(x).cpu(), g["a_blocked"])
    assert torch.equal(ops.pack_a_blocked_t(x_t).cpu(), g["a_blocked_t"])
    assert torch.equal(ops.pack_b_blocked(x).cpu(), g["b_blocked"])
    assert torch.equal(ops.pack_b_blocked_t(x_t).cpu(), g["b_blocked_t"])
    assert torch.equal(ops.pack_b_blocked_vnni(x).cpu(), g["b_vnni"])
    assert torch.equal(ops.pack_b_blocked_vnni_t(x_t).cpu(), g["b_vnni_t"])
    assert torch.equal(ops.pack_b_vnni_t(w, 64).cpu(), g["b_panels64"])
    assert torch.equal(ops.pack_b_vnni_t(w, 32).cpu(), g["b_panels32"])
    if tag == "bf16":
        k_by_n = g["b_vnni"]  # blocks of x read as [K=70, N=45]
        nk = ops.unpack_b_to_nk(cuda(k_by_n)).cpu()
        assert torch.equal(nk[:45, :70], g["x"].T)
        assert nk[45:].abs().sum() == 0 and nk[:, 70:].abs().sum() == 0
        panels = ops.unpack_b_to_nk(cuda(g["b_panels64"])).cpu()
        assert torch.equal(panels[:70, :46], g["w"])


def test_matmul_bf16(ops) -> None:
    g = load_golden("matmul_bf16")
    a, b, bias, scale, shift = cuda(g["a"], g["b"], g["bias"], g["scale"], g["shift"])
    bf16 = torch.bfloat16
    plain = ops.matmul(a, b)
    checks.assert_parity(bf16, plain.cpu(), g["plain"], "plain")
    for name, out in {
        "trans_a": ops.matmul(a.T.contiguous(), b, trans_a=True),
        "trans_b": ops.matmul(a, b.T.contiguous(), trans_b=True),
        "trans_ab": ops.matmul(a.T.contiguous(), b.T.contiguous(), trans_a=True, trans_b=True),
    }.items():
        checks.assert_parity(bf16, out.cpu(), g[name], name)
    checks.assert_parity(bf16, ops.matmul(a, b, bias=bias, epilogue=torch.relu).cpu(), g["bias_relu"], "bias_relu")
    out = ops.matmul(a, b, bias=bias, scale=scale, shift=shift, epilogue=F.gelu)
    checks.assert_parity(bf16, out.cpu(), g["affine_gelu"], "affine_gelu")
    small = load_golden("matmul_bf16_small")
    checks.assert_parity(bf16, ops.matmul(*cuda(small["a"], small["b"])).cpu(), small["plain"], "small")


def test_matmul_f32(ops) -> None:
    f32 = torch.float32
    g = load_golden("matmul_f32_fused")
    a, b = cuda(g["a"], g["b"])
    checks.assert_parity(f32, ops.matmul(a, b).cpu(), g["plain"], "fused")
    out = ops.matmul(a, b.T.contiguous(), trans_b=True, epilogue=torch.relu)
    checks.assert_parity(f32, out.cpu(), g["trans_b_relu"], "fused relu")
    g = load_golden("matmul_f32_blocked")
    a, b, bias, scale, shift = cuda(g["a"], g["b"], g["bias"], g["scale"], g["shift"])
    checks.assert_parity(f32, ops.matmul(a, b).cpu(), g["plain"], "ragged")
    checks.assert_parity(f32, ops.matmul(a, b, bias=bias, epilogue=torch.relu).cpu(), g["bias_relu"], "bias")
    checks.assert_parity(f32, ops.matmul(a, b, bias=bias, scale=scale, shift=shift).cpu(), g["affine"], "affine")
    checks.assert_parity(f32, ops.matmul(a.T.contiguous(), b, trans_a=True).cpu(), g["trans_a"], "trans_a")
    g = load_golden("matmul_f32_split_k")
    a, b = cuda(g["a"], g["b"])
    checks.assert_parity(f32, ops.matmul(a, b, split_k=int(g["splits"])).cpu(), g["plain"], "split-K forced")
    checks.assert_parity(f32, ops.matmul(a, b).cpu(), g["plain"], "split-K auto")


def test_prepacked(ops) -> None:
    g = load_golden("prepacked_vnni")
    x, w, bias, packed = cuda(g["x"], g["w"], g["bias"], g["packed"])
    bf16 = torch.bfloat16
    assert torch.equal(ops.pack_b_vnni_t(w, 64).cpu(), g["packed"])
    checks.assert_parity(bf16, ops.matmul_prepacked_b(x, packed, 100).cpu(), g["plain"], "vnni")
    narrow = ops.matmul_prepacked_b(x, packed, 100, bias, torch.relu)
    checks.assert_parity(bf16, narrow.cpu(), g["bias_relu"], "vnni relu")
    wide = ops.matmul_prepacked_b(x, ops.pack_b_vnni_t(w, 128), 100, bias, torch.relu)
    assert torch.equal(narrow, wide)  # results do not depend on the panel
    call = ops.prepacked_b_call(x, packed, 100, bias, torch.relu)
    checks.assert_parity(bf16, call(x).cpu(), g["bias_relu"], "prepared")
    checks.assert_parity(bf16, call(x[:33].contiguous()).cpu(), g["bias_relu"][:33], "prepared, other shape")
    g = load_golden("prepacked_f32")
    x, w, bias, packed, ps, pb = cuda(g["x"], g["w"], g["bias"], g["packed"], g["post_scale"], g["post_bias"])
    f32 = torch.float32
    assert torch.equal(ops.pack_b_blocked_t(w).cpu(), g["packed"])
    checks.assert_parity(f32, ops.matmul_prepacked_b(x, packed, 40, bias, torch.relu).cpu(), g["rows"], "rows")
    checks.assert_parity(f32, ops.matmul_prepacked_b(x[:50].contiguous(), packed, 40, bias).cpu(), g["ragged_rows"], "ragged")
    out = ops.matmul_prepacked_b_affine(x, packed, 40, bias, ps, pb, torch.relu)
    checks.assert_parity(f32, out.cpu(), g["affine"], "affine")
    with pytest.raises(ValueError, match="is incompatible with"):
        ops.matmul_prepacked_b(x, packed, 70)


def test_bmm_and_linear(ops) -> None:
    g = load_golden("bmm_bf16")
    checks.assert_parity(torch.bfloat16, ops.bmm(*cuda(g["a"], g["b"])).cpu(), g["out"], "bmm bf16")
    g = load_golden("bmm_f32")
    checks.assert_parity(torch.float32, ops.bmm(*cuda(g["a"], g["b"])).cpu(), g["out"], "bmm f32")
    g = load_golden("linear_bf16")
    layer = torch.nn.Linear(96, 80, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        layer.weight.copy_(g["weight"])
        layer.bias.copy_(g["bias"])
    x = cuda(g["x"])
    out, cache = ops.linear(x, layer, F.gelu)
    checks.assert_parity(torch.bfloat16, out.cpu(), g["gelu"], "linear gelu")
    again, cache2 = ops.linear(x, layer, F.gelu, cache)
    assert torch.equal(out, again) and cache2.key == cache.key and cache2.call[2] is cache.call[2]
    affine, _ = ops.linear_affine(x, layer, cuda(g["post"]), None, torch.relu)
    checks.assert_parity(torch.bfloat16, affine.cpu(), g["affine"], "linear affine")
    with torch.no_grad():
        layer.weight.mul_(2)  # in-place: _version changes, the cache is rebuilt
    doubled, cache3 = ops.linear(x, layer, F.gelu, cache2)
    assert cache3.key != cache2.key and not torch.equal(doubled, out)


def test_softmax(ops) -> None:
    g = load_golden("softmax")
    for index in range(5):
        x, y = g[f"x{index}"], g[f"y{index}"]
        error = checks.max_norm_rel(ops.softmax(cuda(x)).cpu(), y)
        assert error < (1e-6 if x.dtype == torch.float32 else 1e-2), (index, error)
    out = ops.softmax(cuda(g["x_one"])).cpu()
    assert torch.equal(out.isnan(), g["y_one"].isnan())
    assert torch.equal(out[~out.isnan()], g["y_one"][~g["y_one"].isnan()])
    assert checks.max_norm_rel(ops.softmax(cuda(g["x_spiky"])).cpu(), g["y_spiky"]) < 1e-6


def test_group_norm(ops) -> None:
    g = load_golden("group_norm")
    x, w, b, extra = cuda(g["x"], g["weight"], g["bias"], g["extra"])
    f32 = torch.float32
    g4 = ops.group_norm(x, 4, w, b, 1e-5)
    checks.assert_parity(f32, g4.cpu(), g["g4"], "G=4")
    checks.assert_parity(f32, ops.group_norm(x, 1, w, b, 1e-5).cpu(), g["g1"], "G=1")
    checks.assert_parity(f32, ops.layer_norm(x, w, b, 1e-5).cpu(), g["g1"], "layer_norm")
    checks.assert_parity(f32, ops.group_norm(x, 3, w, b, 1e-5, torch.add, extra).cpu(), g["g3_add"], "add")
    y = x.clone()
    in_place = ops.group_norm(y, 4, w, b, 1e-5, in_place=True)
    assert in_place.data_ptr() == y.data_ptr() and torch.equal(in_place, g4)
    xb, wb, bb = cuda(g["xb"], g["wb"], g["bb"])
    checks.assert_parity(torch.bfloat16, ops.group_norm(xb, 2, wb, bb, 1e-5).cpu(), g["g2_bf16"], "bf16")


def test_reductions_and_elementwise(ops) -> None:
    g = load_golden("reductions")
    x, xb, v, a, vec = cuda(g["x"], g["xb"], g["v"], g["a"], g["vec"])
    f32, bf16 = torch.float32, torch.bfloat16
    checks.assert_parity(f32, ops.row_sum(x).cpu(), g["row_sum"], "row_sum")
    checks.assert_parity(bf16, ops.row_sum(xb).cpu(), g["row_sum_bf16"], "row_sum bf16")
    checks.assert_parity(bf16, ops.row_dot(xb, v, torch.relu).cpu(), g["row_dot_bf16"], "row_dot")
    checks.assert_parity(f32, ops.column_sum(x).cpu(), g["column_sum"], "column_sum")
    col = ops.column_sum(xb)
    assert col.dtype == torch.float32
    checks.assert_parity(f32, col.cpu(), g["column_sum_bf16"], "column_sum bf16")
    one = ops.column_sum(torch.tensor([[-0.0, 1.5, -2.0]], device="cuda")).cpu()
    assert torch.equal(one, g["column_sum_one_row"]) and not torch.signbit(one[0])
    checks.assert_parity(f32, ops.matvec(a, vec).cpu(), g["matvec"], "matvec")
    g = load_golden("elementwise")
    x, xb = cuda(g["x"], g["xb"])
    assert torch.equal(ops.relu(x).cpu(), g["relu"])
    assert torch.equal(ops.relu(xb).cpu(), g["relu_bf16"])
    assert torch.equal(bits(ops.leaky_relu(x, 0.1)), bits(F.leaky_relu(g["x"], 0.1)))
    assert torch.equal(ops.scalar_mul(x, 1.7).cpu(), g["x"] * 1.7)
    assert torch.equal(ops.scalar_mul(xb, torch.tensor(0.3)).cpu(), g["xb"] * 0.3)
    checks.assert_parity(f32, ops.leaky_relu(x, 0.1).cpu(), g["leaky"], "leaky")
    checks.assert_parity(f32, ops.scalar_mul(x, 1.7).cpu(), g["scaled"], "scaled")
