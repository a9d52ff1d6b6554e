"""Restatement of the reference's kernel bodies on the CPU (test infrastructure).

Every function names the body it follows by file:line of the reference
(paths inside adam-smnk/helion-mlir-xsmm). Rounding points are the reference's:
bf16/f32 operands as stored, products and sums in a wide type, bias / scale /
shift and the epilogue applied before one rounding to the output type
(``tests/golden/blocked_matmul_bias.txt:16-35``: extf, extf, mulf, addf, ...,
truncf). The reference's tests compute their expectations in f64 from the stored
operands (``tests/test_cpu_utils_softmax.py:32``,
``tests/test_cpu_utils_split_k_bmm.py:50,90``); so do these, except where a
function says it accumulates in f32 (the timed CPU baseline).
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor

BLOCK = 32


def round_up(value: int, block: int) -> int:
    return (value + block - 1) // block * block


def identity(x: Tensor) -> Tensor:
    return x


# --------------------------------------------------------------------------- layouts
# Formulas: tests/test_mlir_execution.py:1963-1981 (pad, reshape, permute).


def pad_2d(x: Tensor, rows: int, cols: int) -> Tensor:
    """helion_mlir_utils/matmul.py:78-89 (_pad_kernel)."""
    out = torch.zeros(rows, cols, dtype=x.dtype)
    out[: x.shape[0], : x.shape[1]] = x
    return out


def _padded(x: Tensor, rows_pad: int | None, cols_pad: int | None) -> Tensor:
    r = round_up(x.shape[0], BLOCK) if rows_pad is None else rows_pad
    c = round_up(x.shape[1], BLOCK) if cols_pad is None else cols_pad
    return pad_2d(x, r, c)


def pack_a_blocked(a: Tensor, m_pad: int | None = None, k_pad: int | None = None) -> Tensor:
    """[M,K] -> [M/32,K/32,32,32]; matmul.py:92-99, 907-913."""
    p = _padded(a, m_pad, k_pad)
    r, c = p.shape
    return p.reshape(r // 32, 32, c // 32, 32).permute(0, 2, 1, 3).contiguous()


def pack_a_blocked_t(a_t: Tensor, m_pad: int | None = None, k_pad: int | None = None) -> Tensor:
    """[K,M] -> [M/32,K/32,32,32]; matmul.py:102-109, 916-924."""
    return pack_a_blocked(a_t.T.contiguous(), m_pad, k_pad)


def pack_b_blocked(b: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """[K,N] -> [N/32,K/32,32(k),32(n)]; matmul.py:112-119, 927-933."""
    p = _padded(b, k_pad, n_pad)
    r, c = p.shape
    return p.reshape(r // 32, 32, c // 32, 32).permute(2, 0, 1, 3).contiguous()


def pack_b_blocked_t(b_t: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """[N,K] -> [N/32,K/32,32,32]; matmul.py:122-129, 936-944."""
    return pack_b_blocked(b_t.T.contiguous(), k_pad, n_pad)


def pack_b_blocked_vnni(b: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """[K,N] -> [N/32,K/32,16,32,2], out[j,i,r,n,p] = B[32i+2r+p, 32j+n]; matmul.py:132-141, 947-958."""
    b4 = pack_b_blocked(b, k_pad, n_pad)
    nb, kb = b4.shape[:2]
    return b4.reshape(nb, kb, 16, 2, 32).transpose(3, 4).contiguous()


def pack_b_blocked_vnni_t(b_t: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """[N,K] -> the layout of pack_b_blocked_vnni(b_t.T); matmul.py:144-153, 961-969."""
    return pack_b_blocked_vnni(b_t.T.contiguous(), k_pad, n_pad)


def pack_b_vnni_t(b_t: Tensor, panel: int = 64) -> Tensor:
    """[N,K] -> [N_pad/P, K_pad/2, P, 2], out[q,c,n,v] = W[qP+n, 2c+v]; N padded to P,
    K to 32; matmul.py:972-983, 1138-1157."""
    n, k = b_t.shape
    if k % 2 or panel % 32:
        raise ValueError("pack_b_vnni_t() needs an even K and a panel of a multiple of 32 columns")
    n_pad, k_pad = round_up(n, panel), round_up(k, 32)
    p = pad_2d(b_t, n_pad, k_pad)
    return p.reshape(n_pad // panel, panel, k_pad // 2, 2).permute(0, 2, 1, 3).contiguous()


def unpack_a_blocked(a4: Tensor) -> Tensor:
    mb, kb = a4.shape[:2]
    return a4.permute(0, 2, 1, 3).reshape(mb * 32, kb * 32)


def unpack_b_blocked(b4: Tensor) -> Tensor:
    """[N/32,K/32,32,32] -> [K_pad, N_pad]."""
    nb, kb = b4.shape[:2]
    return b4.permute(1, 2, 0, 3).reshape(kb * 32, nb * 32)


def unpack_b_blocked_vnni(b5: Tensor) -> Tensor:
    """[N/32,K/32,16,32,2] -> [K_pad, N_pad]."""
    nb, kb = b5.shape[:2]
    b4 = b5.transpose(3, 4).reshape(nb, kb, 32, 32)
    return unpack_b_blocked(b4)


def unpack_b_vnni_panels(b4: Tensor) -> Tensor:
    """[N/P,K/2,P,2] -> [K_pad, N_pad]."""
    panels, pairs, panel, _ = b4.shape
    w = b4.permute(0, 2, 1, 3).reshape(panels * panel, pairs * 2)  # [N_pad, K_pad]
    return w.T


# --------------------------------------------------------------------------- GEMM family


def _affine_epilogue(
    acc: Tensor,
    bias: Tensor | None,
    scale: Tensor | None,
    shift: Tensor | None,
    epilogue: Callable[[Tensor], Tensor],
    out_dtype: torch.dtype,
) -> Tensor:
    """matmul.py:321-327: + bias, * scale, + shift, epilogue, one rounding."""
    if bias is not None:
        acc = acc + bias.to(acc.dtype)
    if scale is not None:
        acc = acc * scale.to(acc.dtype)
    if shift is not None:
        acc = acc + shift.to(acc.dtype)
    return epilogue(acc).to(out_dtype)


def matmul(
    a: Tensor,
    b: Tensor,
    trans_a: bool = False,
    trans_b: bool = False,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    acc_dtype: torch.dtype = torch.float64,
) -> Tensor:
    """``epilogue((op(A) @ op(B) + bias) * scale + shift)``; matmul.py:1446-1570
    (dispatcher), 259-328 (_matmul_fused_pack), 1302-1370 (_matmul_f32_fused_pack),
    156-228 (_matmul_blocked_kernel*)."""
    opa = a.T if trans_a else a
    opb = b.T if trans_b else b
    acc = opa.to(acc_dtype) @ opb.to(acc_dtype)
    return _affine_epilogue(acc, bias, scale, shift, epilogue, a.dtype if out_dtype is None else out_dtype)


def matmul_split_k(a: Tensor, b: Tensor, splits: int, out_dtype: torch.dtype | None = None) -> Tensor:
    """f32 partial products per K chunk, then ``partials.sum(0)`` in ascending s:
    matmul.py:1195-1221 (_split_k_partials, _sum_partials), 1289-1299 (_matmul_split_k).
    Partials are rounded to f32 (the workspace type) before they are added, in f32."""
    m, k = a.shape
    chunk = k // splits
    total = None
    for s in range(splits):
        part = (a[:, s * chunk : (s + 1) * chunk].double() @ b[s * chunk : (s + 1) * chunk].double()).float()
        total = part if total is None else total + part
    return total.to(a.dtype if out_dtype is None else out_dtype)


def matmul_blocked(
    a4: Tensor,
    b4: Tensor,
    m: int,
    n: int,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
) -> Tensor:
    """einsum("akmc,bkcn->abmn") over 32x32 blocks, stored as [M/32,32,N/32,32] =
    row-major [M_pad,N_pad]; matmul.py:156-228, 862-904. ``b4`` may be the 5-D VNNI
    block layout (matmul.py:947-958)."""
    a2 = unpack_a_blocked(a4)
    b2 = unpack_b_blocked_vnni(b4) if b4.dim() == 5 else unpack_b_blocked(b4)
    acc = a2.double() @ b2.double()
    out = _affine_epilogue(acc[:m, :n], bias, scale, shift, epilogue, a4.dtype if out_dtype is None else out_dtype)
    return out


def matmul_prepacked_b(
    a: Tensor,
    b4: Tensor,
    n: int,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
) -> Tensor:
    """matmul.py:1593-1671 (dispatcher), 534-590 (_matmul_prepacked_vnni),
    593-627 (_matmul_prepacked_rows)."""
    if b4.dim() == 4 and b4.shape[-1] == 2:
        b2 = unpack_b_vnni_panels(b4)
    elif b4.dim() == 5:
        b2 = unpack_b_blocked_vnni(b4)
    else:
        b2 = unpack_b_blocked(b4)
    k = a.shape[1]
    acc = a.double() @ b2[:k, :n].double()
    return _affine_epilogue(acc, bias, scale, shift, epilogue, a.dtype)


def bmm(a: Tensor, b: Tensor, split_k: int = 0, out_dtype: torch.dtype | None = None) -> Tensor:
    """matmul.py:1842-1882 (_bmm_direct, _bmm_batched), 1965-2006 (bmm); with
    ``split_k`` the per-batch composition with matmul.py:1195-1221."""
    out_dtype = a.dtype if out_dtype is None else out_dtype
    if split_k and split_k > 1:
        return torch.stack([matmul_split_k(a[i], b[i], split_k, out_dtype) for i in range(a.shape[0])])
    return torch.bmm(a.double(), b.double()).to(out_dtype)


def linear(
    x: Tensor,
    weight: Tensor,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
) -> Tensor:
    """helion_mlir_utils/linear.py:97-180 (linear), 183-261 (linear_affine)."""
    return matmul(x, weight, trans_b=True, bias=bias, epilogue=epilogue, scale=scale, shift=shift)


# --------------------------------------------------------------------------- row-wise ops


def softmax(x: Tensor) -> Tensor:
    """exp(x - rowmax) * (1 / sum); normalization.py:28-87, 138-153."""
    return torch.softmax(x.double(), -1).to(x.dtype)


def group_norm(
    x: Tensor,
    num_groups: int,
    weight: Tensor | None,
    bias: Tensor | None,
    eps: float,
    epilogue: Callable[[Tensor, Tensor], Tensor] | None = None,
    extra: Tensor | None = None,
) -> Tensor:
    """Two-pass mean / biased variance per (row, group); normalization.py:94-123, 156-196."""
    m, c = x.shape
    y = x.double().reshape(m, num_groups, c // num_groups)
    mean = y.mean(-1, keepdim=True)
    centered = y - mean
    var = (centered * centered).mean(-1, keepdim=True)
    y = (centered * torch.rsqrt(var + eps)).reshape(m, c)
    if weight is not None:
        y = y * weight.double().reshape(1, c)
    if bias is not None:
        y = y + bias.double().reshape(1, c)
    if epilogue is not None:
        channel = weight if extra is None else extra
        y = epilogue(y, None if channel is None else channel.double().reshape(1, c))
    return y.to(x.dtype)


def layer_norm(x: Tensor, weight: Tensor | None, bias: Tensor | None, eps: float = 1e-5) -> Tensor:
    """GroupNorm with one group; the body tested at tests/test_dynamic_shapes.py:100-108."""
    return group_norm(x, 1, weight, bias, eps)


def rms_norm(x: Tensor, weight: Tensor | None, eps: float = 1e-5) -> Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight. No reference body: parity unpinned."""
    y = x.double()
    y = y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.double()
    return y.to(x.dtype)


def row_sum(x: Tensor, epilogue: Callable[[Tensor], Tensor] = identity) -> Tensor:
    """reduction.py:79-121."""
    return epilogue(x.double().sum(1, keepdim=True)).to(x.dtype)


def row_dot(x: Tensor, v: Tensor, epilogue: Callable[[Tensor], Tensor] = identity) -> Tensor:
    """reduction.py:166-212."""
    return epilogue(x.double() @ v.double().reshape(-1, 1)).to(x.dtype)


def column_sum(x: Tensor) -> Tensor:
    """reduction.py:124-163: f32 result."""
    return x.double().sum(0).float()


def matvec(a: Tensor, b: Tensor) -> Tensor:
    """reduction.py:24-67."""
    return (a.double() @ b.double()).to(a.dtype)


def relu(x: Tensor) -> Tensor:
    """elementwise.py:14-19."""
    return torch.relu(x)


def leaky_relu(x: Tensor, negative_slope: float = 0.01) -> Tensor:
    """elementwise.py:24-31."""
    return torch.nn.functional.leaky_relu(x, negative_slope)


def attention(q: Tensor, k: Tensor, v: Tensor, scale: float) -> Tensor:
    """softmax(scale * q k^T) v per head of [heads, seq, dim] operands, as the online
    loop of tests/harness.py:263-300 (`_attention`) computes it: scores and sums in
    f32 or wider, the probabilities rounded to q.dtype before the second product
    (`p.to(q.dtype)`, :297), one division at the end (:298). The running-maximum
    rescaling of that loop only changes by which power of e numerator and
    denominator are scaled, so the plain two-pass form below is the same function."""
    scores = torch.einsum("hqd,hkd->hqk", q.double(), k.double()) * scale
    if scores.shape[-1] == 0:
        return torch.zeros_like(q)
    top = scores.amax(-1, keepdim=True)
    p = torch.exp(scores - top)
    total = p.sum(-1, keepdim=True)
    acc = torch.einsum("hqk,hkd->hqd", p.to(q.dtype).double(), v.double())
    return (acc / total).to(q.dtype)


def scalar_mul(a: Tensor, s: float) -> Tensor:
    """elementwise.py:34-39."""
    return a * s
