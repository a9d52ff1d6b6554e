"""Structural recognition of tiled-GEMM kernel bodies: what is recognised, how the
store expression maps to the fused epilogue, and what is refused. The bodies are
parsed, never executed, so the names ``hl`` and ``helion`` need not exist."""

from __future__ import annotations

import torch

from helion_mlir_backend import structure

hl = None  # the bodies below only need to parse


def plain(x, y):
    m, k = x.shape
    _, n = y.shape
    out = torch.empty([m, n], dtype=torch.float32, device=x.device)
    for tile_m, tile_n in hl.tile([m, n]):
        acc = hl.zeros([tile_m, tile_n], dtype=torch.float32)
        for tile_k in hl.tile(k):
            acc = torch.addmm(acc, x[tile_m, tile_k], y[tile_k, tile_n])
        out[tile_m, tile_n] = acc
    return out


def linear_gelu(inp, weight, b):
    """Weight stored [N, K]; bias add, then GELU, rounded to the input type."""
    rows, depth = inp.size()
    cols = weight.size(0)
    result = torch.empty_like(inp)
    for tr, tc in hl.tile([rows, cols]):
        total = hl.zeros([tr, tc], dtype=torch.float32)
        for td in hl.tile(depth):
            total += inp[tr, td] @ weight[tc, td].T
        result[tr, tc] = torch.nn.functional.gelu(total + b[tc], approximate="tanh").to(inp.dtype)
    return result


def affine(x, y, gamma, beta, bias, slope):
    m, k = x.shape
    n = y.shape[1]
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=x.device)
    for tm, tn in hl.tile([m, n]):
        acc = hl.zeros([tm, tn])
        for tk in hl.tile(k):
            acc = acc + torch.matmul(x[tk, tm].t(), y[tk, tn])
        out[tm, tn] = torch.nn.functional.leaky_relu((acc + bias[tn]) * gamma[None, tn] + beta[tn], 0.2)
    return out


def scalar_ops(x, y, alpha):
    m, k = x.shape
    k2, n = y.shape
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    for tm, tn in hl.tile([m, n]):
        acc = hl.zeros([tm, tn], dtype=torch.float32)
        for tk in hl.tile(k):
            acc = hl.dot(x[tm, tk], y[tk, tn], acc=acc)
        out[tm, tn] = torch.sigmoid(alpha * acc - 0.5)
    return out


def row_softmax_after(x, y):  # a reduction in the store: not a fused epilogue
    m, k = x.shape
    k2, n = y.shape
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    for tm, tn in hl.tile([m, n]):
        acc = hl.zeros([tm, tn], dtype=torch.float32)
        for tk in hl.tile(k):
            acc = torch.addmm(acc, x[tm, tk], y[tk, tn])
        out[tm, tn] = torch.softmax(acc, dim=-1)
    return out


def two_products(x, y, z):  # the accumulator appears on both sides
    m, k = x.shape
    k2, n = y.shape
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    for tm, tn in hl.tile([m, n]):
        acc = hl.zeros([tm, tn], dtype=torch.float32)
        for tk in hl.tile(k):
            acc = torch.addmm(acc, x[tm, tk], y[tk, tn])
        out[tm, tn] = acc * acc
    return out


def wrong_index(x, y):  # tiles of the wrong loop variables
    m, k = x.shape
    k2, n = y.shape
    out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    for tm, tn in hl.tile([m, n]):
        acc = hl.zeros([tm, tn], dtype=torch.float32)
        for tk in hl.tile(k):
            acc = torch.addmm(acc, x[tm, tk], y[tn, tk])
        out[tm, tn] = acc
    return out


def test_plain_addmm_loop() -> None:
    body = structure.gemm_body(plain)
    assert body is not None and (body.a, body.b, body.trans_a, body.trans_b) == ("x", "y", False, False)
    assert body.bias is None and body.scale is None and body.shift is None and body.activation is None
    assert body.out_dtype is torch.float32


def test_transposed_weight_bias_gelu() -> None:
    body = structure.gemm_body(linear_gelu)
    assert body is not None and (body.a, body.b, body.trans_a, body.trans_b) == ("inp", "weight", False, True)
    assert body.bias.name == "b" and body.bias.vector and body.activation == "gelu" and body.gelu_tanh
    assert body.out_dtype == "inp"  # the dtype of that parameter


def test_full_affine_chain_and_transposed_a() -> None:
    body = structure.gemm_body(affine)
    assert body is not None and body.trans_a and not body.trans_b
    assert (body.bias.name, body.scale.name, body.shift.name) == ("bias", "gamma", "beta")
    assert body.activation == "leaky_relu" and body.slope == 0.2 and body.out_dtype is torch.bfloat16


def test_scalars_become_scale_and_shift() -> None:
    body = structure.gemm_body(scalar_ops)
    assert body is not None and body.bias is None
    assert body.scale.name == "alpha" and not body.scale.vector
    assert body.shift.value == -0.5 and body.activation == "sigmoid"


def test_unrecognised_bodies_say_why() -> None:
    assert structure.gemm_body(row_softmax_after) is None
    assert "affine" in structure.why_not(row_softmax_after)
    assert structure.gemm_body(two_products) is None
    assert structure.gemm_body(wrong_index) is None
    assert "index" in structure.why_not(wrong_index)
    assert structure.gemm_body(len) is None  # no source
    assert structure.why_not(plain) is None
