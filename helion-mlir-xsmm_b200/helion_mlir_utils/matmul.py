"""Matmul on the B200: tensor-core kernels with fused epilogues.

The entry points, argument meaning and error behaviour are those of
``helion_mlir_utils/matmul.py`` of the reference; the implementation is
``b200_gemm`` of ``libb200ops.so``:

* bf16 operands whose rows are 16-byte aligned run the tcgen05/TMEM kernel.
  Row-major ``[M, K]`` / ``[K, N]`` and their transposes are all read in place
  (the tensor cores take K-contiguous and M/N-contiguous tiles alike), so the
  per-tile VNNI packing of the reference's fused kernel (matmul.py:231-328) has
  no counterpart, and ``trans_b`` (``nn.Linear`` weights) needs no packing at all.
* f32 operands, odd pitches and blocked layouts run the exact-f32 FFMA kernel.
* VNNI-packed right-hand sides (``pack_b_vnni_t`` panels, ``pack_b_blocked_vnni``
  blocks) are accepted as the reference lays them out; the tensor-core path
  unpacks them to K-contiguous ``[N, K]`` once per prepared call, or per call
  into scratch memory.

``bias``, ``scale``, ``shift`` and ``epilogue`` are fused into the kernel's
epilogue: ``epilogue((A @ B + bias) * scale + shift)`` in f32, rounded once.
Unsupported operands raise ``ValueError``; nothing falls back to eager PyTorch.
"""

from __future__ import annotations

from collections import OrderedDict
import ctypes
import os
import threading
import weakref
from typing import TYPE_CHECKING
from typing import Callable

import torch
from torch import Tensor

from helion_mlir_backend import native
from helion_mlir_backend import output_pool
from helion_mlir_backend.call_trace import CallExplanation
from helion_mlir_backend.call_trace import trace

from . import epilogues
from . import tuning
from .epilogues import identity_epilogue

if TYPE_CHECKING:
    from collections.abc import Sequence

try:
    from helion_mlir_backend import prepared_call as _prepared_call
except ImportError:  # a backend without prepared calls
    _prepared_call = None

# Block of the blocked (mmt4d-style) layouts: 32 x 32, as the reference packs them.
BLOCK_M = 32
BLOCK_N = 32
BLOCK_K = 32

_SUPPORTED_DTYPES = (torch.bfloat16, torch.float32)
# Columns of a VNNI panel unless the caller chooses (pack_b_vnni_t's default).
_VNNI_PANEL = 64
# K pairs a VNNI panel is padded to (K to a multiple of 32).
_PANEL_PAIRS = 16
# CTA tile of the tensor-core kernel: 128 rows, up to 256 columns, 64-deep K stages.
_TILE_M = 128
_TILE_N = 256
_TILE_K = 64
# A K split must leave every split at least this many K elements.
_SPLIT_K_MIN_CHUNK = 1024
_DEFAULT_SMS = 148


def _round_up(value: int, block: int) -> int:
    return (value + block - 1) // block * block


_SM_COUNTS: dict[int, int] = {}


def _sm_count() -> int:
    """SMs of the current device (148 when there is none to ask); asked once per device."""
    try:
        if torch.cuda.is_available():
            device = torch.cuda.current_device()
            count = _SM_COUNTS.get(device)
            if count is None:
                count = _SM_COUNTS[device] = int(native.module().b200_sm_count()) or _DEFAULT_SMS
            return count
    except (ImportError, OSError):
        pass
    return _DEFAULT_SMS


# --------------------------------------------------------------------------- packs


def _pack(kind: int, src: Tensor, rows_pad: int, cols_pad: int, shape: tuple[int, ...], panel: int = 0) -> Tensor:
    if src.dim() != 2:
        raise ValueError(f"expected a 2-D tensor to pack, got {tuple(src.shape)}")
    device = native.require_cuda(src)
    src = src.contiguous()
    rows, cols = map(int, src.shape)
    out = output_pool.empty(shape, dtype=src.dtype, device=device)
    with native.on_device(device):
        code = native.module().b200_pack(
            kind, native.dtype_code(src.dtype), src.data_ptr(), rows, cols, cols, out.data_ptr(), rows_pad, cols_pad,
            panel, native.stream_ptr(device),
        )
    native.check("b200_pack", code)
    return out


def pad_2d(x: Tensor, rows: int, cols: int) -> Tensor:
    """Contiguous ``x`` zero-padded to ``[rows, cols]``."""
    return _pack(native.PACK_PAD_2D, x, rows, cols, (rows, cols))


def pack_a_blocked(a: Tensor, m_pad: int | None = None, k_pad: int | None = None) -> Tensor:
    """Pack row-major ``[M, K]`` into ``[M/BM, K/BK, BM, BK]`` with optional padding."""
    m, k = int(a.shape[0]), int(a.shape[1])
    mp = _round_up(m, BLOCK_M) if m_pad is None else m_pad
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    return _pack(native.PACK_A_BLOCKED, a, mp, kp, (mp // 32, kp // 32, 32, 32))


def pack_a_blocked_t(a_t: Tensor, m_pad: int | None = None, k_pad: int | None = None) -> Tensor:
    """Pack transposed-layout ``[K, M]`` into ``[M/BM, K/BK, BM, BK]`` with optional padding."""
    k, m = int(a_t.shape[0]), int(a_t.shape[1])
    mp = _round_up(m, BLOCK_M) if m_pad is None else m_pad
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    return _pack(native.PACK_A_BLOCKED_T, a_t, kp, mp, (mp // 32, kp // 32, 32, 32))


def pack_b_blocked(b: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """Pack row-major ``[K, N]`` into ``[N/BN, K/BK, BK, BN]`` with optional padding."""
    k, n = int(b.shape[0]), int(b.shape[1])
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    np_ = _round_up(n, BLOCK_N) if n_pad is None else n_pad
    return _pack(native.PACK_B_BLOCKED, b, kp, np_, (np_ // 32, kp // 32, 32, 32))


def pack_b_blocked_t(b_t: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """Pack transposed-layout ``[N, K]`` into ``[N_pad/BN, K_pad/BK, BK, BN]`` with optional padding."""
    n, k = int(b_t.shape[0]), int(b_t.shape[1])
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    np_ = _round_up(n, BLOCK_N) if n_pad is None else n_pad
    return _pack(native.PACK_B_BLOCKED_T, b_t, np_, kp, (np_ // 32, kp // 32, 32, 32))


def pack_b_blocked_vnni(b: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """Pack row-major ``[K, N]`` into VNNI blocks ``[N/BN, K/BK, BK/2, BN, 2]``:
    ``out[j, i, r, n, p] = B[32i + 2r + p, 32j + n]``."""
    k, n = int(b.shape[0]), int(b.shape[1])
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    np_ = _round_up(n, BLOCK_N) if n_pad is None else n_pad
    return _pack(native.PACK_B_VNNI, b, kp, np_, (np_ // 32, kp // 32, 16, 32, 2))


def pack_b_blocked_vnni_t(b_t: Tensor, k_pad: int | None = None, n_pad: int | None = None) -> Tensor:
    """Pack transposed-layout ``[N, K]`` (e.g. ``nn.Linear`` weights) into the
    layout of :func:`pack_b_blocked_vnni` of ``b_t.T``."""
    n, k = int(b_t.shape[0]), int(b_t.shape[1])
    kp = _round_up(k, BLOCK_K) if k_pad is None else k_pad
    np_ = _round_up(n, BLOCK_N) if n_pad is None else n_pad
    return _pack(native.PACK_B_VNNI_T, b_t, np_, kp, (np_ // 32, kp // 32, 16, 32, 2))


def pack_b_vnni_t(b_t: Tensor, panel: int = _VNNI_PANEL) -> Tensor:
    """Pack transposed-layout ``[N, K]`` (K even) into contiguous column panels of
    the bf16 VNNI layout of ``b_t.T``, ``[N_pad/P, K_pad/2, P, 2]`` with
    ``P = panel`` (a multiple of 32); N is zero-padded to whole panels, K to a
    multiple of 32."""
    n, k = int(b_t.shape[0]), int(b_t.shape[1])
    if k % 2 or panel % BLOCK_N:
        raise ValueError(
            f"pack_b_vnni_t() needs an even K and a panel of a multiple of "
            f"{BLOCK_N} columns, got b_t.shape={(n, k)}, panel={panel}"
        )
    n_pad, k_pad = _round_up(n, panel), _round_up(k, 2 * _PANEL_PAIRS)
    return _pack(native.PACK_B_VNNI_PANELS_T, b_t, n_pad, k_pad, (n_pad // panel, k_pad // 2, panel, 2), panel)


# --------------------------------------------------------------------------- tile hints


def vnni_panel(m: int, n: int, k: int | None = None) -> int:
    """Columns of :func:`pack_b_vnni_t` panels for ``m`` rows.

    On the CPU the panel width is the output tile's width and is chosen from the
    thread count and cache sizes. On the B200 the tile is the kernel's own choice
    and results do not depend on the panel, so the panel only fixes the layout a
    weight is stored in: the widest of 256, 128, 64 that adds no padding columns
    (padding costs weight memory and a strided output view), else 64."""
    for panel in (256, 128, _VNNI_PANEL):
        if n % panel == 0:
            return panel
    return _VNNI_PANEL


def tall_output_tiles(m: int, n: int, k: int) -> tuple[int, int, int] | None:
    """``block_sizes`` of :func:`matmul` for an output of many short rows: tiles
    that span whole output rows, so A is read once. ``None`` (the default choice)
    unless one CTA tile covers the row (``n`` at most 256 columns) and every SM
    gets at least one 128-row tile."""
    if n <= 0 or k <= 0 or n > _TILE_N or n % 16:
        return None
    if m < _TILE_M * _sm_count():
        return None
    return _TILE_M, n, _TILE_K


def whole_row_tiles(m: int, n: int, panel: int | None = None) -> tuple[int, int] | None:
    """``(rows, columns)`` of tiles with which one SM computes whole rows of an
    ``[m, n]`` output. ``None`` unless the rows split evenly into 128-row tiles,
    one at least per SM, and 256, 128 or 64 columns (``panel`` columns, if given)
    divide ``n``."""
    if m % _TILE_M or m // _TILE_M < _sm_count():
        return None
    for columns in (256, 128, 64) if panel is None else (panel,):
        if columns > 0 and n % columns == 0 and columns <= _TILE_N:
            return _TILE_M, columns
    return None


_F32_TENSOR_CORE_MIN_WORK = 1 << 24  # m*n*k from which f32 GEMMs run as widened bf16 products (gemm.cu)


def _split_k(m: int, n: int, k: int, batch: int = 1) -> int:
    """Parallel K splits of a GEMM with fewer output tiles than SMs (0: none): the
    largest power of two that still leaves every SM at most one work item and
    every split ``_SPLIT_K_MIN_CHUNK`` K elements in whole stages."""
    tile_n = min(_TILE_N, _round_up(max(n, 1), 64))
    tiles = -(-m // _TILE_M) * -(-n // tile_n) * batch
    sms = _sm_count()
    splits = 1
    while (
        tiles * splits * 2 <= sms
        and k % (splits * 2 * _TILE_K) == 0
        and k // (splits * 2) >= _SPLIT_K_MIN_CHUNK
    ):
        splits *= 2
    return splits if splits > 1 else 0


# --------------------------------------------------------------------------- launch plans


def supports(a: Tensor, b: Tensor, trans_a: bool = False, trans_b: bool = False) -> bool:
    """Whether :func:`matmul` can handle this pair of operands: 2-D tensors of
    the same dtype (bf16 or f32) on one CUDA device with matching contracted dim."""
    if a.dtype != b.dtype or a.dtype not in _SUPPORTED_DTYPES:
        return False
    if a.device.type != "cuda" or b.device != a.device:
        return False
    if a.dim() != 2 or b.dim() != 2:
        return False
    k_a = a.shape[0] if trans_a else a.shape[1]
    k_b = b.shape[1] if trans_b else b.shape[0]
    return k_a == k_b


def _affine_vector(vector: Tensor | None, n: int, like: Tensor) -> Tensor | None:
    """``vector`` (scalar, ``[1]`` or ``[n]``) as a contiguous 1-D tensor on ``like``'s device."""
    if vector is None:
        return None
    if vector.numel() not in (1, n) or vector.dim() > 1:
        raise ValueError(f"affine vector must be scalar or have shape (1,) or ({n},), got {tuple(vector.shape)}")
    return vector.to(device=like.device).reshape(-1).contiguous()


class GemmPlan:
    """One planned ``b200_gemm`` call: the descriptor with every field but the
    operand pointers filled in. The analogue of the reference's recorded native
    plan (``KernelRun``, ``_compiler/native/call.cpp:501-557``), which holds no
    data pointers either: every call passes its tensors and only pointers are
    swapped in."""

    def __init__(self, desc: native.GemmDesc, device: torch.device, out_shape: tuple[int, ...],
                 out_dtype: torch.dtype, post: Callable[[Tensor], Tensor] | None, final_dtype: torch.dtype,
                 vec_dtype: torch.dtype, parallel_split: bool) -> None:
        self.desc = desc
        self.device = device
        self.out_shape = out_shape
        self.out_dtype = out_dtype
        self.post = post
        self.final_dtype = final_dtype
        self.vec_dtype = vec_dtype
        self.parallel_split = parallel_split
        self.launches = 0
        d = desc
        # packed bf16 operands are unpacked into scratch for the tensor cores
        packed = d.dtype == native.BF16 and (d.a_layout == native.LAYOUT_BLOCKED or d.b_layout >= native.LAYOUT_BLOCKED)
        # f32 operands (plain or 32x32-blocked) run as a widened bf16 GEMM built in scratch
        widened = d.dtype == native.F32 and d.a_layout <= native.LAYOUT_BLOCKED and d.b_layout <= native.LAYOUT_BLOCKED
        self._wants_workspace = packed or widened or (d.split_k > 1 and parallel_split)
        self._workspace_need: int | None = None

    def run(self, a: Tensor, b: Tensor, bias: Tensor | None = None, scale: Tensor | None = None,
            shift: Tensor | None = None, out: Tensor | None = None) -> Tensor:
        desc = native.GemmDesc.from_buffer_copy(self.desc)  # per call: plans are shared between threads
        if out is None:
            out = output_pool.empty(self.out_shape, dtype=self.out_dtype, device=self.device)
        vec = self.vec_dtype
        bias = None if bias is None else bias.to(vec)
        scale = None if scale is None else scale.to(vec)
        shift = None if shift is None else shift.to(vec)
        desc.a, desc.b, desc.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
        desc.bias, desc.scale, desc.shift = native.ptr(bias), native.ptr(scale), native.ptr(shift)
        lib = native.module()
        workspace = None
        desc.workspace, desc.workspace_bytes = None, 0
        fresh_need = False
        if self._wants_workspace:
            need = self._workspace_need
            if need is None:
                # A function of the planned sizes and layouts (and of the device's SM count),
                # but the query also validates this call's pointers and answers 0 for a call
                # it refuses: the figure is only kept once the call it came with has run.
                fresh_need = True
                with native.on_device(self.device):
                    need = int(lib.b200_gemm_workspace_bytes(ctypes.byref(desc)))
            if need:
                workspace = output_pool.empty((need,), dtype=torch.uint8, device=self.device)
                desc.workspace, desc.workspace_bytes = workspace.data_ptr(), need
        with native.on_device(self.device):
            code = lib.b200_gemm(ctypes.byref(desc), native.stream_ptr(self.device))
        native.check("b200_gemm", code)
        if fresh_need:
            self._workspace_need = need
        self.launches += 1
        if self.post is not None:
            out = self.post(out).to(self.final_dtype)
        return out

    def run_host(self, a_host: Tensor, b: Tensor, bias: Tensor | None, scale: Tensor | None, shift: Tensor | None,
                 out_host: Tensor, chunk_rows: int) -> Tensor:
        """The same GEMM with ``a_host`` read from and ``out_host`` written to host
        memory, row chunks streamed through the library's staging ring."""
        desc = native.GemmDesc.from_buffer_copy(self.desc)
        vec = self.vec_dtype
        bias = None if bias is None else bias.to(vec)
        scale = None if scale is None else scale.to(vec)
        shift = None if shift is None else shift.to(vec)
        # Stand-ins for the staged chunks (the library substitutes its ring): only
        # compared with the other operands' address ranges, never dereferenced.
        desc.a, desc.c, desc.b = 1 << 45, 1 << 46, b.data_ptr()
        desc.bias, desc.scale, desc.shift = native.ptr(bias), native.ptr(scale), native.ptr(shift)
        lib = native.module()
        workspace = None
        desc.workspace, desc.workspace_bytes = None, 0
        if self._wants_workspace:
            need = int(lib.b200_gemm_workspace_bytes(ctypes.byref(desc)))
            if need:
                workspace = output_pool.empty((need,), dtype=torch.uint8, device=self.device)
                desc.workspace, desc.workspace_bytes = workspace.data_ptr(), need
        with native.on_device(self.device):
            code = lib.b200_gemm_host_rows(ctypes.byref(desc), a_host.data_ptr(), out_host.data_ptr(), chunk_rows,
                                           native.stream_ptr(self.device))
        native.check("b200_gemm_host_rows", code)
        self.launches += 1
        return out_host

    def explain(self, a: Tensor, b: Tensor) -> CallExplanation:
        desc = native.GemmDesc.from_buffer_copy(self.desc)  # the plan's own descriptor stays as planned
        desc.a, desc.b = a.data_ptr(), b.data_ptr()
        desc.c = 1 << 46  # only compared with the operands' address ranges, never dereferenced
        desc.bias = desc.scale = desc.shift = None
        desc.bias_n = desc.scale_n = desc.shift_n = 0
        desc.workspace, desc.workspace_bytes = (1 << 45 if self._wants_workspace else None), (1 << 40 if self._wants_workspace else 0)
        buf = ctypes.create_string_buffer(256)
        code = native.module().b200_gemm_explain(ctypes.byref(desc), buf, len(buf))
        text = buf.value.decode()
        if self.post is not None:
            text += " + unfused epilogue (f32 result, one elementwise pass)"
        return CallExplanation(code == 0, text, None if code == 0 else text)


def _vector_dtype(vectors: Sequence[Tensor | None], like: Tensor) -> torch.dtype:
    """Bias, scale and shift share one element type in the kernel: bf16 if all
    that are present are bf16, else f32."""
    present = [v for v in vectors if v is not None]
    if not present:
        return like.dtype if like.dtype in _SUPPORTED_DTYPES else torch.float32
    return torch.bfloat16 if all(v.dtype == torch.bfloat16 for v in present) else torch.float32


def _plan_gemm(
    *,
    a: Tensor,
    m: int,
    n: int,
    k: int,
    a_layout: int,
    b_layout: int,
    lda: int,
    ldb: int,
    bias: Tensor | None,
    scale: Tensor | None,
    shift: Tensor | None,
    epilogue: Callable[[Tensor], Tensor],
    out_dtype: torch.dtype | None = None,
    batch: int = 1,
    strides: tuple[int, int, int] = (0, 0, 0),
    split_k: int = 0,
    parallel_split: bool = False,
    tiles: Sequence[int] | None = None,
    b_panel: int = 0,
    out_shape: tuple[int, ...] | None = None,
    ldc: int | None = None,
    force_kernel: int = 0,
    device: torch.device | None = None,
) -> GemmPlan:
    fused = epilogues.resolve(epilogue)
    final_dtype = a.dtype if out_dtype is None else out_dtype
    act, alpha = fused if fused is not None else (native.ACT_IDENTITY, 0.0)
    kernel_out = final_dtype if fused is not None else torch.float32
    vec_dtype = _vector_dtype([bias, scale, shift], a)
    desc = native.GemmDesc()
    desc.dtype = native.dtype_code(a.dtype)
    desc.out_dtype = native.dtype_code(kernel_out)
    desc.a_layout, desc.b_layout, desc.b_panel = a_layout, b_layout, b_panel
    desc.epilogue, desc.alpha = act, alpha
    desc.vec_dtype = native.dtype_code(vec_dtype)
    desc.m, desc.n, desc.k, desc.batch = m, n, k, batch
    desc.lda, desc.ldb, desc.ldc = lda, ldb, n if ldc is None else ldc
    desc.stride_a, desc.stride_b, desc.stride_c = strides
    desc.bias_n = 0 if bias is None else bias.numel()
    desc.scale_n = 0 if scale is None else scale.numel()
    desc.shift_n = 0 if shift is None else shift.numel()
    desc.split_k = split_k
    if tiles is not None:
        hint = [int(t) for t in tiles][:3] + [0, 0, 0]
        desc.tile_m, desc.tile_n, desc.tile_k = hint[0], hint[1], hint[2]
    desc.force_kernel = force_kernel
    shape = (m, n) if out_shape is None else out_shape
    return GemmPlan(desc, a.device if device is None else device, shape, kernel_out,
                    None if fused is not None else epilogue, final_dtype, vec_dtype, parallel_split)


# LRU of launch plans keyed by problem, like the reference's cache of bound
# kernels (matmul.py:332-335, 470-523): epilogues created per call must not pile up.
_PLANS: OrderedDict[tuple[object, ...], GemmPlan] = OrderedDict()
_PLANS_SIZE = 64


_PLANS_LOCK = threading.Lock()


def _cached_plan(key: tuple[object, ...], build: Callable[[], GemmPlan]) -> GemmPlan:
    """Plans are shared between threads: the table is only touched under its lock
    (building a plan, which may consult the tuning table, happens outside it)."""
    with _PLANS_LOCK:
        plan = _PLANS.get(key)
        if plan is not None:
            _PLANS.move_to_end(key)
            return plan
    built = build()
    with _PLANS_LOCK:
        plan = _PLANS.setdefault(key, built)
        _PLANS.move_to_end(key)
        while len(_PLANS) > _PLANS_SIZE:
            _PLANS.popitem(last=False)
    return plan


def _tensor_key(t: Tensor | None) -> tuple[object, ...] | None:
    """What a plan depends on of an operand: its shape and type, never its data."""
    return None if t is None else (tuple(t.shape), t.dtype)


def _matmul_plan(
    a: Tensor,
    b: Tensor,
    trans_a: bool,
    trans_b: bool,
    bias: Tensor | None,
    epilogue: Callable[[Tensor], Tensor],
    block_sizes: Sequence[int] | None,
    scale: Tensor | None,
    shift: Tensor | None,
    out_dtype: torch.dtype | None,
    split_k: int | None,
    choice: tuning.Choice | None = None,
) -> GemmPlan:
    m = int(a.shape[1]) if trans_a else int(a.shape[0])
    n = int(b.shape[0]) if trans_b else int(b.shape[1])
    k = int(a.shape[0]) if trans_a else int(a.shape[1])
    # Everything the plan depends on, as the caller gave it: the heuristics and the
    # tuning table are only consulted when a problem is planned, not on every call.
    key = (
        "matmul", m, n, k, a.dtype, a.device, trans_a, trans_b, _tensor_key(b), _tensor_key(bias), _tensor_key(scale),
        _tensor_key(shift), None if block_sizes is None else tuple(block_sizes), out_dtype, split_k, epilogue, choice,
    )

    def build() -> GemmPlan:
        tiles, splits, picked = block_sizes, split_k, choice
        explicit_split = splits is not None and splits > 1
        plain = bias is None and scale is None and shift is None and epilogue is identity_epilogue
        # A measured choice for this problem on this hardware overrules the heuristics,
        # unless the caller fixed the tiles or the split.
        if picked is None and tiles is None and splits is None and a.dtype == torch.bfloat16:
            picked = tuning.lookup(tune_key(a.dtype, m, n, k, trans_a, trans_b, bias is not None, epilogue), a.device)
        force_kernel = 0
        if picked is not None:
            if picked.tile_n:
                tiles = (_TILE_M, -picked.tile_n, _TILE_K)  # negative: exactly this width, not a hint
            force_kernel = picked.force_kernel()
            if picked.split_k > 1 and plain and splits is None:
                splits = picked.split_k
        if splits is None:
            # f32 problems large enough for the tensor cores (the widened product) spread their
            # K chunks over idle SMs themselves; a split chosen here would keep them on the
            # exact FFMA kernel, which only an explicit split_k asks for.
            widened = a.dtype == torch.float32 and m * n * k >= _F32_TENSOR_CORE_MIN_WORK
            splits = _split_k(m, n, k) if plain and not widened else 0
        return _plan_gemm(
            a=a, m=m, n=n, k=k,
            a_layout=native.LAYOUT_COL if trans_a else native.LAYOUT_ROW,
            b_layout=native.LAYOUT_COL if trans_b else native.LAYOUT_ROW,
            lda=int(a.shape[1]), ldb=int(b.shape[1]),
            bias=bias, scale=scale, shift=shift, epilogue=epilogue, out_dtype=out_dtype,
            split_k=splits, parallel_split=splits > 1 and not explicit_split, tiles=tiles,
            force_kernel=force_kernel,
        )

    return _cached_plan(key, build)


def tune_key(dtype: torch.dtype, m: int, n: int, k: int, trans_a: bool, trans_b: bool, has_bias: bool,
             epilogue: Callable[[Tensor], Tensor]) -> str:
    """The tuning-table key of a :func:`matmul` problem: sizes, layouts and the fused epilogue."""
    fused = epilogues.resolve(epilogue)
    tail = ("bias+" if has_bias else "") + ("unfused" if fused is None else f"act{fused[0]}")
    return tuning.problem_key("matmul", dtype, m, n, k, trans_a, trans_b, 1, tail)


def forget_plans() -> None:
    """Drops the cached launch plans (after the tuning table changed)."""
    with _PLANS_LOCK:
        _PLANS.clear()


def matmul(
    a: Tensor,
    b: Tensor,
    trans_a: bool = False,
    trans_b: bool = False,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
    block_sizes: Sequence[int] | None = None,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    split_k: int | None = None,
    _choice: tuning.Choice | None = None,
) -> Tensor:
    """``epilogue((op(A) @ op(B) + bias) * scale + shift)``, ``op`` transposing
    with ``trans_a``/``trans_b``.

    No pre-packing: operands are read in place in all four transpose
    combinations. ``block_sizes`` (tile rows, columns, K chunk) is a hint: the
    kernel's tile is 128 rows by a multiple of 64 columns up to 256, 64-deep K
    stages. ``bias``, ``scale`` and ``shift`` are ``[N]`` (``scale``/``shift``
    also ``[1]``), broadcast over rows. ``out_dtype`` (an extension) rounds the f32
    accumulator to another type than ``a.dtype``; ``split_k`` forces that many K
    splits, added in ascending order (default: chosen from the SM count for
    plain GEMMs with few output tiles).

    f32 operands with ``m * n * k >= 2**24`` run on the tensor cores as six bf16
    cross products per f32 product (relative Frobenius error about 1e-6, bar 1e-5);
    that path has no representation for values that are not finite or exceed
    bf16's range (|x| > 3.39e38), whose products come out NaN where exact f32
    arithmetic gives an infinity. An explicit ``split_k`` keeps the exact f32 kernel.

    Raises ``ValueError`` if the operands aren't compatible (see
    :func:`supports`) instead of silently falling back to eager PyTorch.
    """
    if not supports(a, b, trans_a=trans_a, trans_b=trans_b):
        raise ValueError(
            f"matmul() does not support these operands (trans_a={trans_a}, "
            f"trans_b={trans_b}): a.shape={tuple(a.shape)} a.dtype={a.dtype} "
            f"a.device={a.device}, b.shape={tuple(b.shape)} b.dtype={b.dtype} "
            f"b.device={b.device}. dtype must be one of {_SUPPORTED_DTYPES}, "
            "both tensors must be 2-D on one cuda device with a matching contracted dim. "
            "Check supports() before calling, or use torch.matmul directly "
            "for unsupported cases."
        )
    a, b = a.contiguous(), b.contiguous()
    n = int(b.shape[0]) if trans_b else int(b.shape[1])
    if bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != n):
        raise ValueError(f"bias must have shape ({n},), got {tuple(bias.shape)}")
    bias = None if bias is None else bias.to(device=a.device).contiguous()
    scale, shift = _affine_vector(scale, n, a), _affine_vector(shift, n, a)
    plan = _matmul_plan(a, b, trans_a, trans_b, bias, epilogue, block_sizes, scale, shift, out_dtype, split_k, _choice)
    trace(f"matmul {tuple(a.shape)} x {tuple(b.shape)}")
    return plan.run(a, b, bias, scale, shift)


def matmul_host(
    a_host: Tensor,
    b: Tensor,
    out_host: Tensor | None = None,
    trans_b: bool = False,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    chunk_rows: int | None = None,
) -> Tensor:
    """:func:`matmul` for activations in host memory (an extension): ``a_host``
    ``[M, K]`` and the result ``[M, N]`` live in pinned host memory, ``b`` and the
    epilogue vectors on the device. Row chunks are copied in, multiplied and copied
    out on three streams at once, so a call costs about the larger of the two PCIe
    transfers. Returns ``out_host`` (allocated pinned when not given) with
    everything enqueued: synchronise the current stream before reading it. The
    epilogue must be one the kernel fuses (see ``epilogues.resolve``).

    ``a_host`` is read by a copy stream of the library that is ordered after
    earlier ``matmul_host`` results (a call may take the ``out_host`` of an earlier
    one as its ``a_host`` without a synchronisation in between) but not after other
    work of the current stream: rows that such work writes asynchronously (a
    non-blocking device-to-host copy, say) must be complete before this call."""
    if a_host.is_cuda or not b.is_cuda:
        raise ValueError("matmul_host() takes a host a_host and a device b")
    if a_host.dim() != 2 or b.dim() != 2 or a_host.dtype != b.dtype or a_host.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"matmul_host() needs 2-D bf16/f32 operands of one dtype, got {tuple(a_host.shape)} "
                         f"{a_host.dtype} and {tuple(b.shape)} {b.dtype}")
    m, k = map(int, a_host.shape)
    n = int(b.shape[0]) if trans_b else int(b.shape[1])
    if int(b.shape[1] if trans_b else b.shape[0]) != k:
        raise ValueError(f"contracted sizes differ: {tuple(a_host.shape)} x {tuple(b.shape)} (trans_b={trans_b})")
    if epilogues.resolve(epilogue) is None:
        raise ValueError("matmul_host() needs an epilogue the kernel fuses; apply others to the host result")
    final = a_host.dtype if out_dtype is None else out_dtype
    if out_host is None:
        out_host = torch.empty((m, n), dtype=final, pin_memory=True)
    if out_host.is_cuda or tuple(out_host.shape) != (m, n) or out_host.dtype != final or not out_host.is_contiguous():
        raise ValueError(f"out_host must be a contiguous host [{m}, {n}] {final} tensor")
    if not a_host.is_contiguous():
        raise ValueError("a_host must be contiguous")
    device = b.device
    b = b.contiguous()
    if bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != n):
        raise ValueError(f"bias must have shape ({n},), got {tuple(bias.shape)}")
    bias = None if bias is None else bias.to(device=device).contiguous()
    scale, shift = _affine_vector(scale, n, b), _affine_vector(shift, n, b)
    if m == 0:
        return out_host
    key = ("matmul_host", m, n, k, a_host.dtype, device, trans_b, _tensor_key(b), _tensor_key(bias),
           _tensor_key(scale), _tensor_key(shift), final, epilogue)

    def build() -> GemmPlan:
        return _plan_gemm(
            a=a_host, m=m, n=n, k=k, a_layout=native.LAYOUT_ROW,
            b_layout=native.LAYOUT_COL if trans_b else native.LAYOUT_ROW, lda=k, ldb=int(b.shape[1]),
            bias=bias, scale=scale, shift=shift, epilogue=epilogue, out_dtype=final, device=device,
        )

    trace(f"matmul_host {tuple(a_host.shape)} x {tuple(b.shape)}")
    return _cached_plan(key, build).run_host(a_host, b, bias, scale, shift, out_host,
                                             0 if chunk_rows is None else int(chunk_rows))


def explain_matmul(a: Tensor, b: Tensor, **kwargs: object) -> CallExplanation:
    """What :func:`matmul` would launch for these operands."""
    trans_a, trans_b = bool(kwargs.get("trans_a", False)), bool(kwargs.get("trans_b", False))
    if not supports(a, b, trans_a=trans_a, trans_b=trans_b):
        return CallExplanation(False, "", "operands not supported (see supports())")
    n = int(b.shape[0]) if trans_b else int(b.shape[1])
    a, b = a.contiguous(), b.contiguous()
    plan = _matmul_plan(
        a, b, trans_a, trans_b, kwargs.get("bias"), kwargs.get("epilogue", identity_epilogue),
        kwargs.get("block_sizes"), _affine_vector(kwargs.get("scale"), n, a), _affine_vector(kwargs.get("shift"), n, a),
        kwargs.get("out_dtype"), kwargs.get("split_k"),
    )
    return plan.explain(a, b)


matmul.explain = explain_matmul  # type: ignore[attr-defined]


# --------------------------------------------------------------------------- prepacked right-hand sides


def _check_bias(bias: Tensor | None, n: int) -> None:
    if bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != n):
        raise ValueError(f"bias must have shape ({n},), got {tuple(bias.shape)}")


def _prepacked_plan(
    a: Tensor,
    b4: Tensor,
    n: int,
    bias: Tensor | None,
    epilogue: Callable[[Tensor], Tensor],
    scale: Tensor | None,
    shift: Tensor | None,
) -> tuple[GemmPlan, int]:
    """Validates a packed right-hand side against ``a`` as the reference does
    (matmul.py:724-754, 1593-1654) and plans the call. Returns the plan and
    the padded output width."""
    m, k = map(int, a.shape)
    if b4.dim() == 2:
        # K-contiguous [N, K]: the form the tensor cores read in place.
        if a.dtype != b4.dtype or int(b4.shape[1]) != k or int(b4.shape[0]) != n:
            raise ValueError(
                f"K-major RHS {tuple(b4.shape)} {b4.dtype} is incompatible with "
                f"a.shape={tuple(a.shape)} {a.dtype} and n={n}"
            )
        n_pad, layout, panel, ldb = n, native.LAYOUT_COL, 0, k
    elif b4.dim() == 4 and b4.shape[-1] == 2:
        panels, pairs_b, panel, vnni = map(int, b4.shape)
        n_pad = panels * panel
        if (
            a.dtype != torch.bfloat16
            or b4.dtype != a.dtype
            or vnni != 2
            or panel % BLOCK_N
            or k % 2
            or 2 * pairs_b != _round_up(k, 2 * _PANEL_PAIRS)
            or _round_up(n, panel) != n_pad
        ):
            raise ValueError(
                f"VNNI-packed RHS {tuple(b4.shape)} {b4.dtype} is incompatible with "
                f"a.shape={tuple(a.shape)} {a.dtype} and n={n}"
            )
        layout, ldb = native.LAYOUT_VNNI_PANELS, 0
    elif b4.dim() == 5:
        blocks_n, blocks_k, half, block_n, vnni = map(int, b4.shape)
        n_pad = blocks_n * BLOCK_N
        if (
            a.dtype != torch.bfloat16
            or b4.dtype != a.dtype
            or (half, block_n, vnni) != (BLOCK_K // 2, BLOCK_N, 2)
            or blocks_k * BLOCK_K != _round_up(k, BLOCK_K)
            or _round_up(n, BLOCK_N) != n_pad
        ):
            raise ValueError(
                f"VNNI-blocked RHS {tuple(b4.shape)} {b4.dtype} is incompatible with "
                f"a.shape={tuple(a.shape)} {a.dtype} and n={n}"
            )
        layout, panel, ldb = native.LAYOUT_BLOCKED_VNNI, 0, 0
    else:
        if a.dim() != 2 or b4.dim() != 4:
            raise ValueError(
                f"matmul_prepacked_b() expects rank-2 a and rank-4 b4, got "
                f"a.shape={tuple(a.shape)} and b4.shape={tuple(b4.shape)}"
            )
        if a.dtype != b4.dtype or a.device != b4.device:
            raise ValueError(
                "matmul_prepacked_b() requires matching dtype and device: "
                f"a=({a.dtype}, {a.device}), b4=({b4.dtype}, {b4.device})"
            )
        blocks_n, blocks_k, block_k, block_n = map(int, b4.shape)
        if block_k != BLOCK_K or block_n != BLOCK_N:
            raise ValueError(
                f"invalid packed RHS block shape {tuple(b4.shape)}; "
                f"expected trailing dimensions ({BLOCK_K}, {BLOCK_N})"
            )
        n_pad = blocks_n * BLOCK_N
        if blocks_k * BLOCK_K != _round_up(k, BLOCK_K) or not 0 < n <= n_pad or _round_up(n, BLOCK_N) != n_pad:
            raise ValueError(
                f"packed RHS shape {tuple(b4.shape)} is incompatible with a.shape={tuple(a.shape)} and n={n}"
            )
        layout, panel, ldb = native.LAYOUT_BLOCKED, 0, 0
    _check_bias(bias, n)
    key = (
        "prepacked", m, n, k, a.dtype, a.device, layout, _tensor_key(b4), _tensor_key(bias), _tensor_key(scale),
        _tensor_key(shift), epilogue,
    )

    def build() -> GemmPlan:
        return _plan_gemm(
            a=a, m=m, n=n, k=k, a_layout=native.LAYOUT_ROW, b_layout=layout, lda=k, ldb=ldb,
            bias=bias, scale=scale, shift=shift, epilogue=epilogue, b_panel=panel if layout == native.LAYOUT_VNNI_PANELS else 0,
        )

    return _cached_plan(key, build), n_pad


def matmul_prepacked_b(
    a: Tensor,
    b4: Tensor,
    n: int,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
) -> Tensor:
    """Multiply row-major ``a`` by a packed right-hand side: 32x32 blocks
    (:func:`pack_b_blocked_t`), bf16 VNNI panels (:func:`pack_b_vnni_t`), bf16
    VNNI blocks (:func:`pack_b_blocked_vnni`), or the K-contiguous ``[N, K]``
    matrix itself (what :func:`~.linear.linear` keeps for bf16 weights on the
    B200); ``scale``/``shift`` as in :func:`matmul`. ``n`` is the output width
    before padding; callers own the lifetime and invalidation of ``b4``."""
    if a.dim() != 2:
        raise ValueError(
            f"matmul_prepacked_b() expects rank-2 a and rank-4 b4, got "
            f"a.shape={tuple(a.shape)} and b4.shape={tuple(b4.shape)}"
        )
    native.require_cuda(a, b4, bias, scale, shift)
    a = a.contiguous()
    scale, shift = _affine_vector(scale, n, a), _affine_vector(shift, n, a)
    b4 = b4.contiguous()
    plan, _ = _prepacked_plan(a, b4, n, bias, epilogue, scale, shift)
    return plan.run(a, b4, bias, scale, shift)


def matmul_prepacked_b_affine(
    a: Tensor,
    b4: Tensor,
    n: int,
    bias: Tensor | None,
    post_scale: Tensor,
    post_bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
) -> Tensor:
    """Prepacked RHS matmul with a per-output affine post-op:
    ``epilogue((a @ b + bias) * post_scale + post_bias)``; the vectors are
    ``[1]`` or ``[n]``."""
    return matmul_prepacked_b(a, b4, n, bias, epilogue, post_scale, post_bias)


def unpack_b_to_nk(b4: Tensor) -> Tensor:
    """A packed bf16 right-hand side (VNNI panels ``[N/P, K/2, P, 2]``, VNNI blocks
    ``[N/32, K/32, 16, 32, 2]`` or plain blocks ``[N/32, K/32, 32, 32]``) as the
    K-contiguous ``[N_pad, K_pad]`` matrix the tensor cores read in place."""
    device = native.require_cuda(b4)
    b4 = b4.contiguous()
    if b4.dtype != torch.bfloat16:
        raise ValueError(f"unpack_b_to_nk() expects bf16, got {b4.dtype}")
    if b4.dim() == 4 and b4.shape[-1] == 2:
        panels, pairs, panel, _ = map(int, b4.shape)
        n_pad, k_pad, kind = panels * panel, 2 * pairs, native.UNPACK_B_VNNI_PANELS_TO_NK
    elif b4.dim() == 5 and tuple(b4.shape[2:]) == (16, 32, 2):
        n_pad, k_pad, kind, panel = int(b4.shape[0]) * 32, int(b4.shape[1]) * 32, native.UNPACK_B_VNNI_TO_NK, 0
    elif b4.dim() == 4 and tuple(b4.shape[2:]) == (BLOCK_K, BLOCK_N):
        n_pad, k_pad, kind, panel = int(b4.shape[0]) * 32, int(b4.shape[1]) * 32, native.UNPACK_B_BLOCKED_TO_NK, 0
    else:
        raise ValueError(f"unpack_b_to_nk() expects a packed right-hand side, got {tuple(b4.shape)}")
    out = output_pool.empty((n_pad, k_pad), dtype=b4.dtype, device=device)
    with native.on_device(device):
        code = native.module().b200_pack(
            kind, native.BF16, b4.data_ptr(), 0, 0, 0, out.data_ptr(), n_pad, k_pad, panel, native.stream_ptr(device)
        )
    native.check("b200_pack", code)
    return out


def prepacked_b_call(
    a: Tensor,
    b4: Tensor,
    n: int,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    tile_m: int | None = None,
) -> Callable[[Tensor], Tensor]:
    """``lambda x: matmul_prepacked_b(x, b4, n, bias, epilogue, scale, shift)``
    with the host work of a call (validation, operand views, the launch plan)
    done once, for activations like ``a``: the same shape and dtype, contiguous;
    others take :func:`matmul_prepacked_b`. ``bias``, ``scale`` and ``shift`` are
    constants of the prepared call, and so is ``b4``: a VNNI-packed ``b4`` is
    unpacked once, here, into the K-contiguous form the tensor cores read.
    ``tile_m`` (a positive multiple of 32) is accepted for compatibility; the
    kernel's tiles are 128 rows."""

    def general(x: Tensor) -> Tensor:
        return matmul_prepacked_b(x, b4, n, bias, epilogue, scale, shift)

    if tile_m is not None and (tile_m <= 0 or tile_m % BLOCK_M):
        raise ValueError(f"tile_m must be a positive multiple of {BLOCK_M}")
    if (
        a.dim() != 2
        or b4.dim() not in (2, 4, 5)
        or a.dtype != b4.dtype
        or a.device != b4.device
        or a.device.type != "cuda"
        or (bias is not None and (bias.dim() != 1 or int(bias.shape[0]) != n or bias.device != a.device))
    ):
        return general
    a = a.contiguous()
    m, k = map(int, a.shape)
    scale_v, shift_v = _affine_vector(scale, n, a), _affine_vector(shift, n, a)
    rhs = b4.contiguous()
    try:
        plan, n_pad = _prepacked_plan(a, rhs, n, bias, epilogue, scale_v, shift_v)
    except ValueError:
        return general
    if plan.desc.b_layout in (native.LAYOUT_BLOCKED_VNNI, native.LAYOUT_VNNI_PANELS) and k % 8 == 0:
        # Unpack once: every later call is a plain tensor-core GEMM on [N_pad, K_pad].
        rhs = unpack_b_to_nk(rhs)
        plan = _plan_gemm(
            a=a, m=m, n=n, k=k, a_layout=native.LAYOUT_ROW, b_layout=native.LAYOUT_COL, lda=k,
            ldb=int(rhs.shape[1]), bias=bias, scale=scale_v, shift=shift_v, epilogue=epilogue,
        )
    shape, dtype, device = a.shape, a.dtype, a.device
    vec = plan.vec_dtype
    bias_c = None if bias is None else bias.to(vec)
    scale_c = None if scale_v is None else scale_v.to(vec)
    shift_c = None if shift_v is None else shift_v.to(vec)

    def run(x: Tensor) -> Tensor:
        return plan.run(x, rhs, bias_c, scale_c, shift_c)

    def call(x: Tensor) -> Tensor:
        if x.shape != shape or x.dtype is not dtype or not x.is_contiguous() or x.device != device:
            return general(x)
        return run(x)

    call.plan = plan  # type: ignore[attr-defined]
    if _prepared_call is None:
        return call
    prepared = _prepared_call(_Preparable(run), (a,), [0], call, views=[tuple(shape)], result_shape=(m, n))
    return call if prepared is None else prepared


class _Preparable:
    """Adapter handing a planned call to :func:`helion_mlir_backend.prepared_call`."""

    def __init__(self, run: Callable[[Tensor], Tensor]) -> None:
        self._run = run

    def prepare(self, args: tuple[object, ...], varying: list[int], views: list[tuple[int, ...] | None],
                result_shape: tuple[int, ...] | None) -> Callable[..., Tensor] | None:
        if varying != [0]:
            return None
        run = self._run
        if result_shape is None:
            return run
        return lambda x: run(x).view(result_shape)


# --------------------------------------------------------------------------- blocked operands


def matmul_blocked(
    a4: Tensor,
    b4: Tensor,
    m: int,
    n: int,
    k: int,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] = identity_epilogue,
    scale: Tensor | None = None,
    shift: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
) -> Tensor:
    """``[M/32, K/32, 32, 32] x packed B -> [M, N]`` row-major, epilogue fused in:
    the blocked kernel of the reference (``_matmul_blocked_kernel[_bias|_affine]``,
    matmul.py:156-228, 862-904) whose output ``[M/32, 32, N/32, 32]`` is a free
    view of row-major ``[M_pad, N_pad]``. ``b4`` is ``[N/32, K/32, 32, 32]``
    (:func:`pack_b_blocked`) or, as an extension, the VNNI blocks
    ``[N/32, K/32, 16, 32, 2]`` of :func:`pack_b_blocked_vnni`. ``m``, ``n``, ``k``
    are the logical sizes (the packed operands are zero beyond them).
    ``out_dtype`` (an extension) selects the type the f32 accumulator is rounded to
    (default ``a4.dtype``)."""
    device = native.require_cuda(a4, b4, bias, scale, shift)
    if a4.dim() != 4 or tuple(a4.shape[2:]) != (BLOCK_M, BLOCK_K):
        raise ValueError(f"matmul_blocked() expects a4 [M/32, K/32, 32, 32], got {tuple(a4.shape)}")
    if a4.dtype != b4.dtype or a4.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"matmul_blocked() requires matching bf16/f32 operands, got {a4.dtype} and {b4.dtype}")
    mb, kb = int(a4.shape[0]), int(a4.shape[1])
    if b4.dim() == 5:
        ok = tuple(b4.shape[2:]) == (16, 32, 2) and a4.dtype == torch.bfloat16
        layout = native.LAYOUT_BLOCKED_VNNI
    else:
        ok = b4.dim() == 4 and tuple(b4.shape[2:]) == (BLOCK_K, BLOCK_N)
        layout = native.LAYOUT_BLOCKED
    if not ok or int(b4.shape[1]) != kb:
        raise ValueError(f"packed RHS shape {tuple(b4.shape)} is incompatible with a4.shape={tuple(a4.shape)}")
    nb = int(b4.shape[0])
    if not (0 < m <= mb * 32 and _round_up(m, 32) == mb * 32 and 0 < n <= nb * 32 and _round_up(n, 32) == nb * 32
            and 0 < k <= kb * 32 and _round_up(k, 32) == kb * 32):
        raise ValueError(f"logical sizes {(m, n, k)} do not match the packed operands {tuple(a4.shape)}, {tuple(b4.shape)}")
    _check_bias(bias, n)
    a4, b4 = a4.contiguous(), b4.contiguous()
    scale_v, shift_v = _affine_vector(scale, n, a4), _affine_vector(shift, n, a4)
    key = ("blocked", m, n, k, a4.dtype, device, layout, _tensor_key(b4), _tensor_key(bias), _tensor_key(scale_v),
           _tensor_key(shift_v), out_dtype, epilogue)

    # A packed bf16 right-hand side is a weight: its K-contiguous form, which the tensor
    # cores read in place, is made once and kept while the packed tensor lives unchanged
    # (the left-hand side is an activation and is read as it comes).
    ldb = 0
    if a4.dtype == torch.bfloat16 and _keep_prepared_weights():
        b4, layout, ldb = _unpacked_rhs(b4), native.LAYOUT_COL, kb * 32
        key = key + ("nk",)

    def build() -> GemmPlan:
        return _plan_gemm(
            a=a4, m=m, n=n, k=k, a_layout=native.LAYOUT_BLOCKED, b_layout=layout, lda=0, ldb=ldb,
            bias=bias, scale=scale_v, shift=shift_v, epilogue=epilogue, out_dtype=out_dtype,
        )

    return _cached_plan(key, build).run(a4, b4, bias, scale_v, shift_v)


# id(packed tensor) -> (weak reference to it, its version when unpacked, the unpacked form).
# Keyed by identity (tensors do not compare as keys); an entry goes when its tensor dies.
_UNPACKED_RHS: dict[int, tuple["weakref.ref[Tensor]", int, Tensor]] = {}
_UNPACKED_RHS_LOCK = threading.Lock()


def _keep_prepared_weights() -> bool:
    """Whether prepared forms of constant weights are kept between calls: the switch of
    ``linear.cache_prepacked_weights`` (``HELION_MLIR_CACHE_PREPACKED_WEIGHTS=0`` prepares
    them on every call; linear.py:25-33 of the reference)."""
    value = os.environ.get("HELION_MLIR_CACHE_PREPACKED_WEIGHTS")
    return value is None or value.strip().lower() not in {"0", "false", "no", "off"}


def _unpacked_rhs(b4: Tensor) -> Tensor:
    """The K-contiguous form of the packed right-hand side ``b4``, remembered per tensor
    object and redone when the tensor was written to (its ``_version`` moved). A change
    through ``.data`` is not seen, as for the weight cache of :func:`linear`."""
    key = id(b4)
    with _UNPACKED_RHS_LOCK:
        hit = _UNPACKED_RHS.get(key)
        if hit is not None and hit[0]() is b4 and hit[1] == b4._version:
            return hit[2]
    unpacked = unpack_b_to_nk(b4)

    def forget(_: object, key: int = key) -> None:
        with _UNPACKED_RHS_LOCK:
            _UNPACKED_RHS.pop(key, None)

    with _UNPACKED_RHS_LOCK:
        _UNPACKED_RHS[key] = (weakref.ref(b4, forget), b4._version, unpacked)
    return unpacked


# --------------------------------------------------------------------------- batched


def _bmm_plan(a: Tensor, b: Tensor, split_k: int | None, out_dtype: torch.dtype | None) -> tuple[GemmPlan, Tensor, Tensor]:
    """Validates the operands of :func:`bmm` and plans the call."""
    if a.dim() != 3:
        raise ValueError(f"bmm() expects 3-D operands, got {tuple(a.shape)}")
    batch, m, k = map(int, a.shape)
    if b.dim() != 3 or b.shape[0] != batch or b.shape[1] != k:
        raise RuntimeError(
            "Expected size for first two dimensions of batch2 tensor to be: "
            f"[{batch}, {k}] but got: {list(b.shape[:2])}."
        )
    if a.dtype != b.dtype or a.dtype not in _SUPPORTED_DTYPES:
        raise ValueError(f"bmm() requires matching bf16/f32 operands, got {a.dtype} and {b.dtype}")
    device = native.require_cuda(a, b)
    n = int(b.shape[2])
    a, b = a.contiguous(), b.contiguous()
    final = a.dtype if out_dtype is None else out_dtype
    splits = 0 if split_k is None or split_k <= 1 else int(split_k)
    # The tensor-core kernel sums the ordered splits on chip; the FFMA kernel keeps
    # them in an f32 output and takes the partial-sum workspace for other types.
    parallel = splits > 1 and a.dtype != torch.bfloat16 and final != torch.float32
    key = ("bmm", batch, m, n, k, a.dtype, device, final, splits, _tensor_key(b))

    def build() -> GemmPlan:
        return _plan_gemm(
            a=a, m=m, n=n, k=k, a_layout=native.LAYOUT_ROW, b_layout=native.LAYOUT_ROW, lda=k, ldb=n,
            bias=None, scale=None, shift=None, epilogue=identity_epilogue, out_dtype=final, batch=batch,
            strides=(m * k, k * n, m * n), split_k=splits, parallel_split=parallel, out_shape=(batch, m, n),
        )

    return _cached_plan(key, build), a, b


def bmm(a: Tensor, b: Tensor, split_k: int | None = None, out_dtype: torch.dtype | None = None) -> Tensor:
    """Batched ``A @ B`` of ``[B, M, K]`` and ``[B, K, N]`` with the batch as a grid
    dimension of one kernel (bf16: tensor cores, operands read in place; f32:
    the widened bf16 product from ``batch * m * n * k >= 2**24``, the exact FFMA kernel below that
    and with ``split_k``). ``split_k`` (an extension): that many K splits per output tile, each
    accumulated from zero in f32 and added in ascending order. ``out_dtype`` (an
    extension): the type the f32 result is rounded to (default ``a.dtype``)."""
    plan, a, b = _bmm_plan(a, b, split_k, out_dtype)
    trace(f"bmm {tuple(a.shape)} x {tuple(b.shape)}")
    return plan.run(a, b)


def explain_bmm(a: Tensor, b: Tensor, split_k: int | None = None, out_dtype: torch.dtype | None = None) -> CallExplanation:
    """What :func:`bmm` would launch for these operands."""
    plan, a, b = _bmm_plan(a, b, split_k, out_dtype)
    return plan.explain(a, b)


bmm.explain = explain_bmm  # type: ignore[attr-defined]
