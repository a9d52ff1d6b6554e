"""Generates tests/golden/*.npz from the reference's own operator code.

Run in the build container, where the reference source tree is mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

The reference's ``helion_mlir_utils`` cannot be imported as is (it needs Helion
and an MLIR toolchain that are not installed). Its kernel *bodies* and host-side
dispatch code are plain Python over torch, though, so this script installs a small
stand-in for the Helion names they use (``helion.kernel``, ``hl.tile``,
``hl.zeros`` ...) that runs a body eagerly, tile by tile, with the semantics the
compiled kernels have:

* a tile past the end of a tensor loads zeros and stores nothing there;
* values loaded from a tensor are widened (to f64) so that products and sums are
  not rounded to bf16 between steps -- the compiled kernels accumulate sub-32-bit
  floats in f32 (``_compiler/mlir/lowering/contraction_ops.py:174-177``) -- and a
  body's explicit ``.to(torch.float32)`` still narrows to f32 as written;
* block sizes are handed to ``hl.register_block_size`` / ``hl.tile`` call sites in
  program order (``README.md:22-25``).

What comes out is what the reference's operators compute on seeded inputs: its
layouts, padding, dispatch, epilogue order and rounding points. The fixtures are
small; ``tests/test_oracle.py`` checks the CPU oracle against them and the GPU
tests check the kernels against the same files.
"""

from __future__ import annotations

import importlib
import itertools
import os
from pathlib import Path
import sys
import threading
import types

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


# --------------------------------------------------------------------------- Helion stand-in


class Tile:
    """One step of ``hl.tile``: ``[begin, end)`` of a loop with block ``block_size``."""

    __slots__ = ("begin", "block_size", "end")

    def __init__(self, begin: int, end: int, block_size: int) -> None:
        self.begin, self.end, self.block_size = begin, end, block_size

    @property
    def id(self) -> int:
        return self.begin // self.block_size

    def __index__(self) -> int:  # hl.zeros([tile, ...]) sizes
        return self.end - self.begin


class ConstExpr:
    def __init__(self, value: object) -> None:
        self.value = value


def _unwrap(value: object) -> object:
    return value.value if isinstance(value, ConstExpr) else value


class DeviceTensor(torch.Tensor):
    """A kernel argument: tile indexing loads with zero fill and widening, stores clip."""

    def _resolve(self, index: object) -> tuple[tuple[object, ...], list[tuple[int, int]], bool]:
        index = index if isinstance(index, tuple) else (index,)
        resolved: list[object] = []
        pads: list[tuple[int, int]] = []  # (result dim, wanted length)
        tiled = False
        src_dim = 0
        out_dim = 0
        for item in index:
            if isinstance(item, Tile):
                tiled = True
                size = self.shape[src_dim]
                stop = min(item.end, size)
                start = min(item.begin, size)
                resolved.append(slice(start, stop))
                pads.append((out_dim, item.end - item.begin))
                src_dim += 1
                out_dim += 1
            elif item is None:
                resolved.append(None)
                out_dim += 1
            elif isinstance(item, slice):
                resolved.append(item)
                src_dim += 1
                out_dim += 1
            else:  # int
                resolved.append(item)
                src_dim += 1
        return tuple(resolved), pads, tiled

    def __getitem__(self, index: object) -> torch.Tensor:
        resolved, pads, tiled = self._resolve(index)
        plain = self.as_subclass(torch.Tensor)
        value = plain[resolved]
        if not tiled:
            return value
        for dim, wanted in pads:
            have = value.shape[dim]
            if have < wanted:
                shape = list(value.shape)
                shape[dim] = wanted - have
                value = torch.cat([value, torch.zeros(shape, dtype=value.dtype)], dim=dim)
        if value.dtype in (torch.bfloat16, torch.float16, torch.float32):
            value = value.to(torch.float64)
        return value

    def __setitem__(self, index: object, value: object) -> None:
        resolved, pads, _ = self._resolve(index)
        plain = self.as_subclass(torch.Tensor)
        target = plain[resolved]
        if isinstance(value, torch.Tensor):
            value = value.as_subclass(torch.Tensor)
            if value.dim() == target.dim():
                clip = tuple(slice(0, size) for size in target.shape)
                value = value[clip]
            value = value.to(target.dtype)
        plain[resolved] = value


class _Context(threading.local):
    def __init__(self) -> None:
        self.stack: list[dict[str, object]] = []


_context = _Context()


def _take_block_size(site: object, count: int) -> list[int]:
    frame = _context.stack[-1]
    sites: dict[object, list[int]] = frame["sites"]  # type: ignore[assignment]
    if site not in sites:
        sizes: list[int] = frame["block_sizes"]  # type: ignore[assignment]
        start: int = frame["next"]  # type: ignore[assignment]
        if start + count > len(sizes):
            raise RuntimeError(f"kernel asks for more block sizes than its config has: {sizes}")
        sites[site] = sizes[start : start + count]
        frame["next"] = start + count
    return sites[site]


def _site() -> object:
    caller = sys._getframe(2)
    return (caller.f_code, caller.f_lineno)


def hl_tile(begin_or_end: object, end_or_none: object = None, block_size: object = None):
    begin_or_end, end_or_none = _unwrap(begin_or_end), _unwrap(end_or_none)
    if isinstance(begin_or_end, (list, tuple, torch.Size)):
        ends = [int(_unwrap(v)) for v in begin_or_end]
        begins = [0] * len(ends) if end_or_none is None else None
        if begins is None:
            begins, ends = ends, [int(_unwrap(v)) for v in end_or_none]  # type: ignore[union-attr]
        if block_size is None:
            blocks = _take_block_size(_site(), len(ends))
        else:
            blocks = [int(b) for b in block_size]  # type: ignore[union-attr]
        ranges = [
            [Tile(s, min(s + bs, e), bs) for s in range(b, e, bs)] for b, e, bs in zip(begins, ends, blocks)
        ]
        return itertools.product(*ranges)
    if end_or_none is None:
        begin, end = 0, int(begin_or_end)  # type: ignore[arg-type]
    else:
        begin, end = int(begin_or_end), int(end_or_none)  # type: ignore[arg-type]
    bs = _take_block_size(_site(), 1)[0] if block_size is None else int(block_size)  # type: ignore[arg-type]
    return iter([Tile(s, min(s + bs, end), bs) for s in range(begin, end, bs)])


def hl_register_block_size(*_bounds: object) -> int:
    return _take_block_size(_site(), 1)[0]


def _sizes(shape: object) -> list[int]:
    return [s.__index__() if isinstance(s, Tile) else int(_unwrap(s)) for s in shape]  # type: ignore[union-attr]


class Accumulator(torch.Tensor):
    """What ``hl.zeros`` / ``hl.full`` return: a register tile of full block width.
    A partial last chunk is narrower than the accumulator it is added to; in a
    compiled kernel its missing lanes are masked loads, i.e. zeros, so an add
    whose operands have the same rank but differ in an extent pads the smaller with zeros
    (a one-row last tile included: same-rank operands of these bodies never broadcast)."""

    _ADDS = (torch.add, torch.Tensor.add, torch.Tensor.__add__, torch.Tensor.__radd__)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in cls._ADDS and len(args) == 2 and all(isinstance(a, torch.Tensor) for a in args):
            a, b = args
            if a.dim() == b.dim() and a.shape != b.shape:
                a, b = a.as_subclass(torch.Tensor), b.as_subclass(torch.Tensor)
                for dim, (sa, sb) in enumerate(zip(a.shape, b.shape)):
                    if sa == sb:
                        continue
                    small, size = (a, sb) if sa < sb else (b, sa)
                    shape = list(small.shape)
                    shape[dim] = size - small.shape[dim]
                    padded = torch.cat([small, torch.zeros(shape, dtype=small.dtype)], dim=dim)
                    a, b = (padded, b) if sa < sb else (a, padded)
                return func(a, b, **kwargs).as_subclass(cls)
        return super().__torch_function__(func, types, args, kwargs)


def hl_zeros(shape: object, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return torch.zeros(_sizes(shape), dtype=dtype).as_subclass(Accumulator)


def hl_full(shape: object, value: float, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return torch.full(_sizes(shape), value, dtype=dtype).as_subclass(Accumulator)


class Config(dict):
    def __init__(self, **kwargs: object) -> None:
        super().__init__(**kwargs)
        self.config = self


class Kernel:
    def __init__(self, fn, config: Config | None = None, **_ignored: object) -> None:
        self.fn = fn
        self.configs = [config] if config is not None else []
        self.name = fn.__name__

    def bind(self, args: tuple[object, ...]) -> "Kernel":
        return self

    def __call__(self, *args: object, **kwargs: object) -> object:
        import inspect

        bound = inspect.signature(self.fn).bind(*args, **kwargs)
        bound.apply_defaults()
        values = {}
        for name, value in bound.arguments.items():
            value = _unwrap(value)
            if isinstance(value, torch.Tensor):
                value = value.as_subclass(DeviceTensor)
            values[name] = value
        block_sizes = list(self.configs[0].get("block_sizes", [])) if self.configs else []
        _context.stack.append({"block_sizes": block_sizes, "next": 0, "sites": {}})
        try:
            result = self.fn(**values)
        finally:
            _context.stack.pop()
        if isinstance(result, torch.Tensor):
            result = result.as_subclass(torch.Tensor)
        return result


def kernel(fn=None, **kwargs: object):
    if fn is None:
        return lambda body: Kernel(body, **kwargs)
    return Kernel(fn, **kwargs)


def install_stand_in() -> None:
    helion = types.ModuleType("helion")
    helion.kernel = kernel
    helion.Config = Config
    helion.Kernel = Kernel
    exc = types.ModuleType("helion.exc")
    exc.TensorOperationInWrapper = type("TensorOperationInWrapper", (Warning,), {})
    helion.exc = exc
    language = types.ModuleType("helion.language")
    language.tile = hl_tile
    language.zeros = hl_zeros
    language.full = hl_full
    language.grid = lambda extent: range(int(_unwrap(extent)))
    language.specialize = lambda value: value
    language.register_block_size = hl_register_block_size
    language.constexpr = ConstExpr
    helion.language = language
    runtime = types.ModuleType("helion.runtime")
    runtime_kernel = types.ModuleType("helion.runtime.kernel")
    runtime_kernel.BoundKernel = Kernel
    runtime.kernel = runtime_kernel
    backend = types.ModuleType("helion_mlir_backend")
    pool = types.ModuleType("helion_mlir_backend.output_pool")
    pool.empty = lambda sizes, *, dtype, device=None: torch.empty(list(sizes), dtype=dtype).as_subclass(DeviceTensor)
    pool.empty_like = lambda x, *, dtype=None: torch.empty_like(
        x.as_subclass(torch.Tensor), dtype=dtype
    ).as_subclass(DeviceTensor)
    backend.output_pool = pool
    for name, module in {
        "helion": helion,
        "helion.exc": exc,
        "helion.language": language,
        "helion.runtime": runtime,
        "helion.runtime.kernel": runtime_kernel,
        "helion_mlir_backend": backend,
        "helion_mlir_backend.output_pool": pool,
    }.items():
        sys.modules[name] = module


# --------------------------------------------------------------------------- cases


def _store(value: torch.Tensor) -> tuple[np.ndarray, str]:
    value = value.detach().contiguous()
    if value.dtype == torch.bfloat16:
        return value.view(torch.int16).numpy().copy(), "bfloat16"
    return value.numpy().copy(), str(value.dtype).replace("torch.", "")


def save(name: str, **tensors: torch.Tensor) -> None:
    arrays: dict[str, np.ndarray] = {}
    for key, value in tensors.items():
        array, dtype = _store(value)
        arrays[key] = array
        arrays[f"{key}__dtype"] = np.array(dtype)
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    print(f"  {name}.npz: " + ", ".join(f"{k}{tuple(v.shape)}" for k, v in tensors.items()))


def randn(generator: torch.Generator, *shape: int, dtype: torch.dtype = torch.float32, scale: float = 1.0):
    return (torch.randn(*shape, generator=generator) * scale).to(dtype)


def load_functions(path: Path, names: list[str], namespace: dict[str, object]) -> dict[str, object]:
    """Executes the named top-level functions and constants of a reference source file
    (and nothing else of it) in ``namespace``: for files whose imports are not installed."""
    import ast

    tree = ast.parse(path.read_text())
    wanted = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            wanted.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in names for t in node.targets):
            wanted.append(node)
    module = ast.Module(body=wanted, type_ignores=[])
    exec(compile(module, str(path), "exec"), namespace)
    return namespace


class _WideningTorch:
    """``torch`` for an executed body, except that ``einsum`` of operands of different
    float types widens them first: the compiled contraction takes a bf16 tile and
    accumulates in f32, eager einsum refuses mixed types."""

    def __getattr__(self, name: str) -> object:
        return getattr(torch, name)

    @staticmethod
    def einsum(equation: str, *operands: torch.Tensor) -> torch.Tensor:
        widest = max((o.dtype for o in operands), key=lambda d: torch.finfo(d).bits)
        return torch.einsum(equation, *[o.to(widest) for o in operands])


def attention_cases(reference: str, g: torch.Generator) -> None:
    """The online-softmax attention body of the reference's tests, run block by block."""
    language = sys.modules["helion.language"]
    namespace = load_functions(
        Path(reference) / "tests" / "harness.py",
        ["_RESCALE_THRESHOLD", "_dot_nt", "_dot_nn", "_attention"],
        {"torch": _WideningTorch(), "hl": language, "__builtins__": __builtins__},
    )
    body = namespace["_attention"]
    bf16 = torch.bfloat16
    cases: dict[str, torch.Tensor] = {}
    for tag, (heads, seq, dim, blocks, dtype, spread) in {
        "d64": (3, 256, 64, [64, 128], bf16, 1.0),
        "d128": (2, 128, 128, [128, 64], bf16, 1.0),
        "peaky": (2, 256, 64, [128, 32], bf16, 6.0),  # maxima that grow past the rescale threshold
        "f32": (2, 96, 32, [32, 32], torch.float32, 1.0),
    }.items():
        q = randn(g, heads, seq, dim, dtype=dtype, scale=spread)
        k = randn(g, heads, seq, dim, dtype=dtype, scale=spread)
        v = randn(g, heads, seq, dim, dtype=dtype)
        scale = dim ** -0.5
        out = Kernel(body, config=Config(block_sizes=blocks))(q, k, v, ConstExpr(scale), ConstExpr(False))
        cases.update({f"{tag}_q": q, f"{tag}_k": k, f"{tag}_v": v, f"{tag}_out": out,
                      f"{tag}_scale": torch.tensor(scale)})
    save("attention", **cases)


def main(reference: str) -> None:
    os.environ["OMP_NUM_THREADS"] = "8"
    os.environ.pop("HELION_MLIR_CACHE_PREPACKED_WEIGHTS", None)
    torch.set_num_threads(8)
    install_stand_in()
    sys.path.insert(0, reference)
    ref = importlib.import_module("helion_mlir_utils")
    ref_matmul = importlib.import_module("helion_mlir_utils.matmul")
    print(f"reference operators imported from {Path(ref.__file__).parent}")
    bf16, f32 = torch.bfloat16, torch.float32
    g = torch.Generator().manual_seed(20240607)

    # --- layouts (bit-exact) -------------------------------------------------
    for dtype, tag in ((f32, "f32"), (bf16, "bf16")):
        x = randn(g, 70, 45, dtype=dtype)
        x_t = x.T.contiguous()
        w = randn(g, 70, 46, dtype=dtype)
        save(
            f"layouts_{tag}",
            x=x,
            w=w,
            pad=ref_matmul.pad_2d(x, 96, 64),
            a_blocked=ref.pack_a_blocked(x),
            a_blocked_t=ref.pack_a_blocked_t(x_t),
            b_blocked=ref.pack_b_blocked(x),
            b_blocked_t=ref.pack_b_blocked_t(x_t),
            b_vnni=ref.pack_b_blocked_vnni(x),
            b_vnni_t=ref.pack_b_blocked_vnni_t(x_t),
            b_panels64=ref.pack_b_vnni_t(w, 64),
            b_panels32=ref.pack_b_vnni_t(w, 32),
        )

    # --- bf16 matmul: ragged, transposes, fused epilogue ----------------------
    a = randn(g, 65, 136, dtype=bf16)
    b = randn(g, 136, 100, dtype=bf16)
    bias = randn(g, 100, dtype=bf16)
    scale = (1.0 + 0.1 * torch.randn(100, generator=g)).to(bf16)
    shift = randn(g, 100, dtype=bf16, scale=0.1)
    save(
        "matmul_bf16",
        a=a,
        b=b,
        bias=bias,
        scale=scale,
        shift=shift,
        plain=ref.matmul(a, b),
        trans_a=ref.matmul(a.T.contiguous(), b, trans_a=True),
        trans_b=ref.matmul(a, b.T.contiguous(), trans_b=True),
        trans_ab=ref.matmul(a.T.contiguous(), b.T.contiguous(), trans_a=True, trans_b=True),
        bias_relu=ref.matmul(a, b, bias=bias, epilogue=torch.relu),
        affine_gelu=ref.matmul(a, b, bias=bias, scale=scale, shift=shift, epilogue=torch.nn.functional.gelu),
    )
    a = randn(g, 20, 47, dtype=bf16)  # smaller than one tile: padded to one (matmul.py:1516-1535)
    b = randn(g, 47, 30, dtype=bf16)
    save("matmul_bf16_small", a=a, b=b, plain=ref.matmul(a, b))

    # --- f32 matmul: fused (whole tiles), blocked (ragged, bias, affine), split-K
    a = randn(g, 128, 64)
    b = randn(g, 64, 192)
    save(
        "matmul_f32_fused",
        a=a,
        b=b,
        plain=ref.matmul(a, b),
        trans_b_relu=ref.matmul(a, b.T.contiguous(), trans_b=True, epilogue=torch.relu),
    )
    a = randn(g, 70, 50)
    b = randn(g, 50, 45)
    bias = randn(g, 45)
    scale = 1.0 + 0.1 * torch.randn(1, generator=g)
    shift = randn(g, 45, scale=0.1)
    save(
        "matmul_f32_blocked",
        a=a,
        b=b,
        bias=bias,
        scale=scale,
        shift=shift,
        plain=ref.matmul(a, b),
        bias_relu=ref.matmul(a, b, bias=bias, epilogue=torch.relu),
        affine=ref.matmul(a, b, bias=bias, scale=scale, shift=shift),
        trans_a=ref.matmul(a.T.contiguous(), b, trans_a=True),
    )
    a = randn(g, 64, 2048)
    b = randn(g, 2048, 128)
    splits = ref_matmul._split_k(64, 128, 2048, False, False, None, None, None, ref.identity_epilogue)
    assert splits == 4, splits  # 1 output tile on 8 threads, K chunks of 512
    save("matmul_f32_split_k", a=a, b=b, splits=torch.tensor(splits), plain=ref.matmul(a, b))

    # --- prepacked right-hand sides ------------------------------------------
    x = randn(g, 70, 90, dtype=bf16)
    w = randn(g, 100, 90, dtype=bf16)  # [N, K]
    bias = randn(g, 100, dtype=bf16)
    packed = ref.pack_b_vnni_t(w, 64)
    save(
        "prepacked_vnni",
        x=x,
        w=w,
        bias=bias,
        packed=packed,
        plain=ref.matmul_prepacked_b(x, packed, 100),
        bias_relu=ref.matmul_prepacked_b(x, packed, 100, bias, torch.relu),
        wide_panel=ref.matmul_prepacked_b(x, ref.pack_b_vnni_t(w, 128), 100, bias, torch.relu),
    )
    x = randn(g, 64, 96)
    w = randn(g, 40, 96)
    bias = randn(g, 40)
    packed = ref.pack_b_blocked_t(w)
    post_scale = 1.0 + 0.1 * torch.randn(40, generator=g)
    post_bias = randn(g, 40, scale=0.1)
    save(
        "prepacked_f32",
        x=x,
        w=w,
        bias=bias,
        packed=packed,
        post_scale=post_scale,
        post_bias=post_bias,
        rows=ref.matmul_prepacked_b(x, packed, 40, bias, torch.relu),
        ragged_rows=ref.matmul_prepacked_b(x[:50].contiguous(), packed, 40, bias),
        affine=ref.matmul_prepacked_b_affine(x, packed, 40, bias, post_scale, post_bias, torch.relu),
    )

    # --- bmm -------------------------------------------------------------------
    a = randn(g, 4, 64, 128, dtype=bf16)
    b = randn(g, 4, 128, 96, dtype=bf16)
    save("bmm_bf16", a=a, b=b, out=ref.bmm(a, b))
    a = randn(g, 3, 64, 32)
    b = randn(g, 3, 32, 64)
    save("bmm_f32", a=a, b=b, out=ref.bmm(a, b))

    # --- linear (cached weight) --------------------------------------------------
    layer = torch.nn.Linear(96, 80, dtype=bf16)
    with torch.no_grad():
        layer.weight.copy_(randn(g, 80, 96, dtype=bf16, scale=0.1))
        layer.bias.copy_(randn(g, 80, dtype=bf16, scale=0.1))
    x = randn(g, 256, 96, dtype=bf16)
    out, cache = ref.linear(x, layer, torch.nn.functional.gelu)
    out2, _ = ref.linear(x, layer, torch.nn.functional.gelu, cache)
    assert torch.equal(out, out2)
    post = (1.0 + 0.1 * torch.randn(80, generator=g)).to(bf16)
    affine, _ = ref.linear_affine(x, layer, post, None, torch.relu)
    save("linear_bf16", x=x, weight=layer.weight.detach(), bias=layer.bias.detach(), post=post, gelu=out, affine=affine)

    # --- row-wise ----------------------------------------------------------------
    cases = {}
    for index, (m, n, dtype, shift_) in enumerate(
        [(130, 515, f32, 0.0), (4, 129, f32, -50.0), (2, 200, bf16, -50.0), (4, 256, f32, -50.0), (3, 47, f32, 0.0)]
    ):
        x = (torch.randn(m, n, generator=g) + shift_).to(dtype)
        cases[f"x{index}"] = x
        cases[f"y{index}"] = ref.softmax(x)
    x = torch.cat([torch.tensor([[0.5], [-3e4], [float("nan")], [float("inf")], [-float("inf")]]), randn(g, 11, 1)])
    cases["x_one"], cases["y_one"] = x, ref.softmax(x)
    spiky = randn(g, 6, 300, scale=1.4)
    spiky[torch.rand(6, 300, generator=g) < 0.02] = 30.0
    cases["x_spiky"], cases["y_spiky"] = spiky, ref.softmax(spiky)
    save("softmax", **cases)

    x = randn(g, 10, 96)
    weight = 1.0 + 0.1 * torch.randn(96, generator=g)
    bias = randn(g, 96, scale=0.1)
    extra = randn(g, 96)
    xb = randn(g, 7, 64, dtype=bf16)
    wb, bb = weight[:64].to(bf16), bias[:64].to(bf16)
    save(
        "group_norm",
        x=x,
        weight=weight,
        bias=bias,
        extra=extra,
        xb=xb,
        wb=wb,
        bb=bb,
        g4=ref.group_norm(x, 4, weight, bias, 1e-5),
        g1=ref.group_norm(x, 1, weight, bias, 1e-5),
        g3_add=ref.group_norm(x, 3, weight, bias, 1e-5, torch.add, extra),
        g2_bf16=ref.group_norm(xb, 2, wb, bb, 1e-5),
        g4_in_place=ref.group_norm(x.clone(), 4, weight, bias, 1e-5, in_place=True),
    )

    x = randn(g, 33, 65)
    xb = randn(g, 16, 520, dtype=bf16)
    v = randn(g, 520)
    a = randn(g, 40, 70)
    vec = randn(g, 70, 1)
    save(
        "reductions",
        x=x,
        xb=xb,
        v=v,
        a=a,
        vec=vec,
        row_sum=ref.row_sum(x),
        row_sum_bf16=ref.row_sum(xb),
        row_dot_bf16=ref.row_dot(xb, v, torch.relu),
        column_sum=ref.column_sum(x),
        column_sum_bf16=ref.column_sum(xb),
        column_sum_one_row=ref.column_sum(torch.tensor([[-0.0, 1.5, -2.0]])),
        matvec=ref.matvec(a, vec),
    )

    x = randn(g, 9, 1030)
    xb = x.to(bf16)
    save(
        "elementwise",
        x=x,
        xb=xb,
        relu=ref.relu(x),
        leaky=ref.leaky_relu(x, 0.1),
        scaled=ref.scalar_mul(x, 1.7),
        relu_bf16=ref.relu(xb),
        scaled_bf16=ref.scalar_mul(xb, torch.tensor(0.3)),
    )
    attention_cases(reference, g)
    print("done")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
