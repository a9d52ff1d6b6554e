"""The CPU oracle against the fixtures produced by the reference's own operator
code (tests/golden/make_golden.py). Layouts must match bit for bit; arithmetic
within the parity bars (the fixtures themselves come from eager f32/f64 torch
arithmetic in the reference's bodies, so equality of bits is not expected)."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from helpers import load_golden
from oracle import checks
from oracle import ops


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_layouts_bit_exact(tag: str) -> None:
    g = load_golden(f"layouts_{tag}")
    x, w = g["x"], g["w"]
    x_t = x.T.contiguous()
    assert torch.equal(ops.pad_2d(x, 96, 64), g["pad"])
    assert torch.equal(ops.pack_a_blocked(x), g["a_blocked"])
    assert torch.equal(ops.pack_a_blocked_t(x_t), g["a_blocked_t"])
    assert torch.equal(ops.pack_b_blocked(x), g["b_blocked"])
    assert torch.equal(ops.pack_b_blocked_t(x_t), g["b_blocked_t"])
    assert torch.equal(ops.pack_b_blocked_vnni(x), g["b_vnni"])
    assert torch.equal(ops.pack_b_blocked_vnni_t(x_t), g["b_vnni_t"])
    assert torch.equal(ops.pack_b_vnni_t(w, 64), g["b_panels64"])
    assert torch.equal(ops.pack_b_vnni_t(w, 32), g["b_panels32"])
    # the formula of pack_b_blocked_vnni's docstring: out[j,i,r,n,p] = B[32i+2r+p, 32j+n]
    b5 = g["b_vnni"]
    padded = ops.pad_2d(x, 96, 64)
    for j, i, r, n, p in [(0, 0, 0, 0, 0), (1, 2, 7, 5, 1), (0, 1, 15, 31, 1), (1, 0, 3, 12, 0)]:
        assert b5[j, i, r, n, p] == padded[32 * i + 2 * r + p, 32 * j + n]


def test_matmul_bf16() -> None:
    g = load_golden("matmul_bf16")
    a, b, bias, scale, shift = g["a"], g["b"], g["bias"], g["scale"], g["shift"]
    bf16 = torch.bfloat16
    checks.assert_parity(bf16, ops.matmul(a, b), g["plain"], "plain")
    checks.assert_parity(bf16, ops.matmul(a.T.contiguous(), b, trans_a=True), g["trans_a"], "trans_a")
    checks.assert_parity(bf16, ops.matmul(a, b.T.contiguous(), trans_b=True), g["trans_b"], "trans_b")
    checks.assert_parity(
        bf16, ops.matmul(a.T.contiguous(), b.T.contiguous(), trans_a=True, trans_b=True), g["trans_ab"], "trans_ab"
    )
    checks.assert_parity(bf16, ops.matmul(a, b, bias=bias, epilogue=torch.relu), g["bias_relu"], "bias_relu")
    checks.assert_parity(
        bf16, ops.matmul(a, b, bias=bias, scale=scale, shift=shift, epilogue=F.gelu), g["affine_gelu"], "affine_gelu"
    )
    # the four transposes are the same product: the reference gives the same bits
    assert torch.equal(g["plain"], g["trans_a"]) and torch.equal(g["plain"], g["trans_b"])
    small = load_golden("matmul_bf16_small")
    checks.assert_parity(bf16, ops.matmul(small["a"], small["b"]), small["plain"], "small")


def test_matmul_f32() -> None:
    f32 = torch.float32
    g = load_golden("matmul_f32_fused")
    checks.assert_parity(f32, ops.matmul(g["a"], g["b"]), g["plain"], "fused")
    checks.assert_parity(
        f32, ops.matmul(g["a"], g["b"].T.contiguous(), trans_b=True, epilogue=torch.relu), g["trans_b_relu"], "fused relu"
    )
    g = load_golden("matmul_f32_blocked")
    a, b = g["a"], g["b"]
    checks.assert_parity(f32, ops.matmul(a, b), g["plain"], "blocked")
    checks.assert_parity(f32, ops.matmul(a, b, bias=g["bias"], epilogue=torch.relu), g["bias_relu"], "blocked bias")
    checks.assert_parity(
        f32, ops.matmul(a, b, bias=g["bias"], scale=g["scale"], shift=g["shift"]), g["affine"], "blocked affine"
    )
    checks.assert_parity(f32, ops.matmul(a.T.contiguous(), b, trans_a=True), g["trans_a"], "blocked trans_a")
    g = load_golden("matmul_f32_split_k")
    splits = int(g["splits"])
    checks.assert_parity(f32, ops.matmul_split_k(g["a"], g["b"], splits), g["plain"], "split-K")
    checks.assert_parity(f32, ops.matmul(g["a"], g["b"]), g["plain"], "split-K vs unsplit")


def test_prepacked() -> None:
    g = load_golden("prepacked_vnni")
    x, w, bias = g["x"], g["w"], g["bias"]
    assert torch.equal(ops.pack_b_vnni_t(w, 64), g["packed"])
    bf16 = torch.bfloat16
    checks.assert_parity(bf16, ops.matmul_prepacked_b(x, g["packed"], 100), g["plain"], "vnni")
    checks.assert_parity(bf16, ops.matmul_prepacked_b(x, g["packed"], 100, bias, torch.relu), g["bias_relu"], "vnni relu")
    # panel-independence is a reference invariant (tests/test_cpu_utils_prepacked.py:513-566)
    assert torch.equal(g["bias_relu"], g["wide_panel"])
    checks.assert_parity(bf16, ops.linear(x, w, bias, torch.relu), g["bias_relu"], "linear == prepacked")
    g = load_golden("prepacked_f32")
    x, bias = g["x"], g["bias"]
    assert torch.equal(ops.pack_b_blocked_t(g["w"]), g["packed"])
    f32 = torch.float32
    checks.assert_parity(f32, ops.matmul_prepacked_b(x, g["packed"], 40, bias, torch.relu), g["rows"], "rows")
    checks.assert_parity(f32, ops.matmul_prepacked_b(x[:50], g["packed"], 40, bias), g["ragged_rows"], "ragged")
    checks.assert_parity(
        f32,
        ops.matmul_prepacked_b(x, g["packed"], 40, bias, torch.relu, g["post_scale"], g["post_bias"]),
        g["affine"],
        "affine",
    )


def test_bmm_and_linear() -> None:
    g = load_golden("bmm_bf16")
    checks.assert_parity(torch.bfloat16, ops.bmm(g["a"], g["b"]), g["out"], "bmm bf16")
    g = load_golden("bmm_f32")
    checks.assert_parity(torch.float32, ops.bmm(g["a"], g["b"]), g["out"], "bmm f32")
    g = load_golden("linear_bf16")
    checks.assert_parity(torch.bfloat16, ops.linear(g["x"], g["weight"], g["bias"], F.gelu), g["gelu"], "linear gelu")
    checks.assert_parity(
        torch.bfloat16, ops.linear(g["x"], g["weight"], g["bias"], torch.relu, scale=g["post"]), g["affine"], "linear affine"
    )


def test_softmax() -> None:
    g = load_golden("softmax")
    for index in range(5):
        x, y = g[f"x{index}"], g[f"y{index}"]
        error = checks.max_norm_rel(ops.softmax(x), y)
        assert error < (1e-6 if x.dtype == torch.float32 else 1e-2), (index, error)
    x, y = g["x_one"], g["y_one"]
    ref = ops.softmax(x)
    assert torch.equal(ref.isnan(), y.isnan())
    assert torch.equal(ref[~y.isnan()], y[~y.isnan()])
    assert checks.max_norm_rel(ops.softmax(g["x_spiky"]), g["y_spiky"]) < 1e-6


def test_group_norm() -> None:
    g = load_golden("group_norm")
    x, w, b = g["x"], g["weight"], g["bias"]
    f32 = torch.float32
    checks.assert_parity(f32, ops.group_norm(x, 4, w, b, 1e-5), g["g4"], "G=4")
    checks.assert_parity(f32, ops.group_norm(x, 1, w, b, 1e-5), g["g1"], "G=1")
    checks.assert_parity(f32, ops.layer_norm(x, w, b, 1e-5), g["g1"], "layer_norm")
    checks.assert_parity(f32, F.layer_norm(x, (96,), w, b, 1e-5), g["g1"], "torch layer_norm")
    checks.assert_parity(f32, ops.group_norm(x, 3, w, b, 1e-5, torch.add, g["extra"]), g["g3_add"], "G=3 add")
    checks.assert_parity(torch.bfloat16, ops.group_norm(g["xb"], 2, g["wb"], g["bb"], 1e-5), g["g2_bf16"], "bf16")
    assert torch.equal(g["g4"], g["g4_in_place"])  # tests/test_cpu_utils_softmax.py:79-94


def test_reductions_and_elementwise() -> None:
    g = load_golden("reductions")
    f32, bf16 = torch.float32, torch.bfloat16
    checks.assert_parity(f32, ops.row_sum(g["x"]), g["row_sum"], "row_sum")
    checks.assert_parity(bf16, ops.row_sum(g["xb"]), g["row_sum_bf16"], "row_sum bf16")
    checks.assert_parity(bf16, ops.row_dot(g["xb"], g["v"], torch.relu), g["row_dot_bf16"], "row_dot")
    checks.assert_parity(f32, ops.column_sum(g["x"]), g["column_sum"], "column_sum")
    checks.assert_parity(f32, ops.column_sum(g["xb"]), g["column_sum_bf16"], "column_sum bf16")
    assert g["column_sum_bf16"].dtype == torch.float32
    one = g["column_sum_one_row"]
    assert torch.equal(one, torch.tensor([0.0, 1.5, -2.0])) and not torch.signbit(one[0])
    checks.assert_parity(f32, ops.matvec(g["a"], g["vec"]), g["matvec"], "matvec")
    g = load_golden("elementwise")
    assert torch.equal(ops.relu(g["x"]), g["relu"])
    # products: the fixture rounds an f64 product once, torch rounds the f32 scalar first (1 ulp apart)
    checks.assert_parity(f32, ops.leaky_relu(g["x"], 0.1), g["leaky"], "leaky_relu")
    checks.assert_parity(f32, ops.scalar_mul(g["x"], 1.7), g["scaled"], "scalar_mul")
    assert torch.equal(ops.relu(g["xb"]), g["relu_bf16"])
    checks.assert_parity(bf16, ops.scalar_mul(g["xb"], 0.3), g["scaled_bf16"], "scalar_mul bf16")


def test_rms_norm_definition() -> None:
    """No reference body exists (parity unpinned): the oracle must at least be torch's rms_norm."""
    torch.manual_seed(3)
    x, w = torch.randn(9, 40), torch.randn(40)
    assert checks.rel_frobenius(ops.rms_norm(x, w, 1e-5), F.rms_norm(x, (40,), w, 1e-5)) < 1e-6


@pytest.mark.parametrize("tag", ["d64", "d128", "peaky", "f32"])
def test_attention_against_the_reference_body(tag: str) -> None:
    """The two-pass oracle against the reference's online loop run block by block."""
    g = load_golden("attention")
    q, k, v, want = (g[f"{tag}_{name}"] for name in ("q", "k", "v", "out"))
    got = ops.attention(q, k, v, float(g[f"{tag}_scale"]))
    assert got.dtype == want.dtype and got.shape == want.shape
    checks.assert_parity(q.dtype, got, want.double() if q.dtype == torch.float32 else want.float(), f"attention {tag}")
