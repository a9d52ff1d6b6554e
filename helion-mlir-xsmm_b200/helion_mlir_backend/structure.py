"""Recognition of tiled-GEMM kernel bodies by structure.

Kernels outside the reference's operator set are not known by name. The common
shape of a hand-written Helion GEMM (``examples/matmul_mlir.py:22-59`` addmm loop,
``examples/fused_ops_mlir.py:22-91`` matmul + relu / + bias) is

    for tile_m, tile_n in hl.tile([m, n]):
        acc = hl.zeros([tile_m, tile_n], dtype=torch.float32)
        for tile_k in hl.tile(k):
            acc = torch.addmm(acc, x[tile_m, tile_k], y[tile_k, tile_n])
        out[tile_m, tile_n] = <elementwise expression of acc and [N] vectors>
    return out

This module parses the body's source (``ast``; the body is never executed),
checks that it is exactly such a loop nest, and turns the store expression into
the fused epilogue of the native GEMM: ``act((acc + bias) * scale + shift)``.
Anything else (other loop nests, reductions in the epilogue, data-dependent
control flow) is not recognised and ``gemm_body`` returns ``None``: the caller
then reports the body as unsupported instead of guessing.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from dataclasses import dataclass, field
from typing import Callable

import torch

_ACTIVATIONS = {
    "relu": "relu",
    "gelu": "gelu",
    "sigmoid": "sigmoid",
    "tanh": "tanh",
    "silu": "silu",
    "leaky_relu": "leaky_relu",
}

_DTYPES = {
    "float32": torch.float32,
    "float": torch.float32,
    "bfloat16": torch.bfloat16,
}


@dataclass
class Operand:
    """A vector parameter indexed by the column tile, or a scalar."""

    name: str | None = None  # parameter name (vector or scalar parameter)
    value: float | None = None  # literal scalar
    vector: bool = False


@dataclass
class GemmBody:
    """What a recognised body computes: ``act((op(a) @ op(b) + bias) * scale + shift)``."""

    params: list[str]
    a: str
    b: str
    trans_a: bool = False
    trans_b: bool = False
    bias: Operand | None = None
    scale: Operand | None = None
    shift: Operand | None = None
    activation: str | None = None
    slope: float = 0.01
    gelu_tanh: bool = False
    out_dtype: torch.dtype | str | None = None  # dtype, or "<param>.dtype" as the parameter's name
    stages: list[str] = field(default_factory=list)  # the affine stages as written, for explain()


class _NotRecognised(Exception):
    pass


def _fail(why: str) -> None:
    raise _NotRecognised(why)


def _dotted(node: ast.AST) -> str:
    """``torch.nn.functional.relu`` -> that string; '' for anything but names/attributes."""
    parts: list[str] = []
    while isinstance(node, ast.Attribute):
        parts.append(node.attr)
        node = node.value
    if isinstance(node, ast.Name):
        parts.append(node.id)
        return ".".join(reversed(parts))
    return ""


def _names(node: ast.AST) -> list[str]:
    if isinstance(node, ast.Name):
        return [node.id]
    if isinstance(node, (ast.Tuple, ast.List)):
        return [n.id for n in node.elts if isinstance(n, ast.Name)]
    return []


def _tile_call(node: ast.AST) -> ast.Call | None:
    if isinstance(node, ast.Call) and _dotted(node.func).split(".")[-1] == "tile" and node.args:
        return node
    return None


def _dtype_of(node: ast.AST | None, params: list[str]) -> torch.dtype | str | None:
    if node is None:
        return None
    text = _dotted(node)
    if text.startswith("torch.") and text[6:] in _DTYPES:
        return _DTYPES[text[6:]]
    if text.endswith(".dtype") and text[:-6] in params:
        return text[:-6]
    _fail(f"output dtype {ast.unparse(node)!r} is not understood")
    return None


class _Parser:
    def __init__(self, fn: Callable[..., object]) -> None:
        try:
            source = textwrap.dedent(inspect.getsource(fn))
        except (OSError, TypeError):
            _fail("source unavailable")
        tree = ast.parse(source)
        defs = [n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef)]
        if not defs:
            _fail("no function definition")
        self.fn = defs[0]
        args = self.fn.args
        if args.vararg or args.kwarg or args.kwonlyargs:
            _fail("variadic parameters")
        self.params = [a.arg for a in args.posonlyargs + args.args]
        self.out: str | None = None
        self.out_dtype: torch.dtype | str | None = None

    # -- statements ---------------------------------------------------------

    def parse(self) -> GemmBody:
        body = [s for s in self.fn.body if not self._skippable(s)]
        loops = [s for s in body if isinstance(s, ast.For)]
        if len(loops) != 1:
            _fail("expected exactly one outer tile loop")
        outer = loops[0]
        position = body.index(outer)
        for stmt in body[:position]:
            self._prologue(stmt)
        rest = body[position + 1:]
        if len(rest) != 1 or not isinstance(rest[0], ast.Return) or _names(rest[0].value or ast.Constant(None)) != [self.out]:
            _fail("the body must end by returning the output tensor")
        return self._outer(outer)

    @staticmethod
    def _skippable(stmt: ast.stmt) -> bool:
        if isinstance(stmt, ast.Assert):
            return True
        if isinstance(stmt, ast.Expr):
            if isinstance(stmt.value, ast.Constant):  # docstring
                return True
            # hl.specialize(...) and friends: hints without effect on the result
            if isinstance(stmt.value, ast.Call) and _dotted(stmt.value.func).split(".")[-1] in ("specialize",):
                return True
        return False

    def _prologue(self, stmt: ast.stmt) -> None:
        if not isinstance(stmt, ast.Assign) or len(stmt.targets) != 1:
            _fail(f"unexpected statement before the loop: {ast.unparse(stmt)}")
        target, value = stmt.targets[0], stmt.value
        if isinstance(value, ast.Call):
            callee = _dotted(value.func)
            last = callee.split(".")[-1]
            if last in ("zeros", "empty", "zeros_like", "empty_like", "new_empty", "new_zeros") and isinstance(target, ast.Name):
                if self.out is not None:
                    _fail("more than one output allocation")
                self.out = target.id
                dtype = next((k.value for k in value.keywords if k.arg == "dtype"), None)
                if dtype is None and last.endswith("_like") and value.args and _dotted(value.args[0]) in self.params:
                    self.out_dtype = _dotted(value.args[0])
                elif dtype is None and last.startswith("new_") and _dotted(value.func)[: -len(last) - 1] in self.params:
                    self.out_dtype = _dotted(value.func)[: -len(last) - 1]
                else:
                    self.out_dtype = _dtype_of(dtype, self.params) if dtype is not None else torch.float32
                return
            if last in ("size",):
                return  # m, k = x.size()
        if isinstance(value, ast.Attribute) and value.attr == "shape":
            return  # m, k = x.shape
        if isinstance(value, ast.Subscript) and isinstance(value.value, ast.Attribute) and value.value.attr == "shape":
            return  # n = y.shape[1]
        _fail(f"unexpected statement before the loop: {ast.unparse(stmt)}")

    def _outer(self, loop: ast.For) -> GemmBody:
        call = _tile_call(loop.iter)
        tiles = _names(loop.target)
        if call is None or len(tiles) != 2 or loop.orelse:
            _fail("the outer loop must be `for tile_m, tile_n in hl.tile([m, n])`")
        tile_m, tile_n = tiles
        stmts = [s for s in loop.body if not self._skippable(s)]
        if len(stmts) != 3:
            _fail("the outer loop must hold: accumulator, K loop, store")
        init, inner, store = stmts
        # acc = hl.zeros([tile_m, tile_n], dtype=torch.float32)
        if not (isinstance(init, ast.Assign) and len(init.targets) == 1 and isinstance(init.targets[0], ast.Name)
                and isinstance(init.value, ast.Call) and _dotted(init.value.func).split(".")[-1] == "zeros"):
            _fail("the accumulator must start as hl.zeros([...])")
        acc = init.targets[0].id
        acc_dtype = next((k.value for k in init.value.keywords if k.arg == "dtype"), None)
        if acc_dtype is not None and _dtype_of(acc_dtype, self.params) is not torch.float32:
            _fail("the accumulator must be f32")
        if not init.value.args or _names(init.value.args[0]) != [tile_m, tile_n]:
            _fail("the accumulator must be a [tile_m, tile_n] tile")
        # for tile_k in hl.tile(k): acc = acc + a_tile @ b_tile
        if not isinstance(inner, ast.For) or _tile_call(inner.iter) is None or inner.orelse:
            _fail("the second statement must be the K loop")
        k_names = _names(inner.target)
        k_body = [s for s in inner.body if not self._skippable(s)]
        if len(k_names) != 1 or len(k_body) != 1:
            _fail("the K loop must hold one accumulation statement")
        a_ref, b_ref = self._accumulation(k_body[0], acc)
        a, trans_a = self._tile_ref(a_ref, (tile_m, k_names[0]))
        b, trans_b = self._tile_ref(b_ref, (k_names[0], tile_n))
        # out[tile_m, tile_n] = expression
        if not (isinstance(store, ast.Assign) and len(store.targets) == 1 and isinstance(store.targets[0], ast.Subscript)):
            _fail("the last statement must store the tile")
        target = store.targets[0]
        if _dotted(target.value) != self.out or _names(target.slice) != [tile_m, tile_n]:
            _fail("the store must be out[tile_m, tile_n] = ...")
        body = GemmBody(params=self.params, a=a, b=b, trans_a=trans_a, trans_b=trans_b, out_dtype=self.out_dtype)
        self._epilogue(store.value, acc, tile_n, body)
        return body

    def _accumulation(self, stmt: ast.stmt, acc: str) -> tuple[ast.AST, ast.AST]:
        """The two tile references of ``acc = acc + a @ b`` in any of its spellings."""
        if isinstance(stmt, ast.AugAssign) and isinstance(stmt.op, ast.Add) and _names(stmt.target) == [acc]:
            return self._product(stmt.value)
        if not (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and _names(stmt.targets[0]) == [acc]):
            _fail("the K loop must assign the accumulator")
        value = stmt.value
        if isinstance(value, ast.Call):
            last = _dotted(value.func).split(".")[-1]
            if last in ("addmm", "baddbmm") and len(value.args) == 3 and _names(value.args[0]) == [acc] and not value.keywords:
                return value.args[1], value.args[2]
            if last == "dot" and len(value.args) >= 2:
                extra = value.args[2:] + [k.value for k in value.keywords if k.arg == "acc"]
                if len(extra) == 1 and _names(extra[0]) == [acc]:
                    return value.args[0], value.args[1]
        if isinstance(value, ast.BinOp) and isinstance(value.op, ast.Add):
            if _names(value.left) == [acc]:
                return self._product(value.right)
            if _names(value.right) == [acc]:
                return self._product(value.left)
        _fail(f"accumulation {ast.unparse(stmt)!r} is not a GEMM update")
        raise AssertionError

    @staticmethod
    def _product(node: ast.AST) -> tuple[ast.AST, ast.AST]:
        if isinstance(node, ast.BinOp) and isinstance(node.op, ast.MatMult):
            return node.left, node.right
        if isinstance(node, ast.Call) and _dotted(node.func).split(".")[-1] in ("matmul", "mm", "dot") and len(node.args) == 2:
            return node.args[0], node.args[1]
        _fail(f"{ast.unparse(node)!r} is not a matrix product")
        raise AssertionError

    def _tile_ref(self, node: ast.AST, plain: tuple[str, str]) -> tuple[str, bool]:
        """``x[tile_r, tile_c]`` -> (x, False); its transposed spellings of ``x[tile_c, tile_r]`` -> (x, True)."""
        transposed = False
        while True:
            if isinstance(node, ast.Attribute) and node.attr in ("T", "mT"):
                transposed, node = not transposed, node.value
            elif (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr in ("t", "transpose")
                  and (node.func.attr == "t" or [getattr(a, "value", None) for a in node.args] in ([0, 1], [1, 0], [-1, -2], [-2, -1]))):
                transposed, node = not transposed, node.func.value
            else:
                break
        if not isinstance(node, ast.Subscript) or _dotted(node.value) not in self.params:
            _fail(f"{ast.unparse(node)!r} is not a tile of a parameter")
        index = tuple(_names(node.slice))
        want = (plain[1], plain[0]) if transposed else plain
        if index != want:
            _fail(f"tile index {index} does not match the loop nest")
        return _dotted(node.value), transposed

    # -- epilogue -----------------------------------------------------------

    def _epilogue(self, node: ast.AST, acc: str, tile_n: str, body: GemmBody) -> None:
        node = self._strip_cast(node, body)
        # one activation, outermost
        if isinstance(node, ast.Call):
            last = _dotted(node.func).split(".")[-1]
            if last in _ACTIVATIONS and node.args:
                body.activation = _ACTIVATIONS[last]
                for kw in node.keywords:
                    if kw.arg == "approximate" and getattr(kw.value, "value", None) == "tanh":
                        body.gelu_tanh = True
                    elif kw.arg == "negative_slope" and isinstance(kw.value, ast.Constant):
                        body.slope = float(kw.value.value)
                    elif kw.arg not in ("approximate", "inplace"):
                        _fail(f"activation argument {kw.arg!r}")
                if last == "leaky_relu" and len(node.args) == 2 and isinstance(node.args[1], ast.Constant):
                    body.slope = float(node.args[1].value)
                elif len(node.args) != 1:
                    _fail("activation with extra operands")
                node = self._strip_cast(node.args[0], body)
        stages: list[tuple[str, Operand]] = []
        self._affine(node, acc, tile_n, stages)
        kinds = "".join("a" if kind == "add" else "m" for kind, _ in stages)
        body.stages = [kind for kind, _ in stages]
        if kinds == "":
            return
        if kinds == "a":
            operand = stages[0][1]
            if operand.vector:
                body.bias = operand
            else:
                body.shift = operand
        elif kinds == "m":
            body.scale = stages[0][1]
        elif kinds == "am":
            if not stages[0][1].vector:
                _fail("a scalar added before a scale has no fused form")
            body.bias, body.scale = stages[0][1], stages[1][1]
        elif kinds == "ma":
            body.scale, body.shift = stages[0][1], stages[1][1]
        elif kinds == "ama":
            if not stages[0][1].vector:
                _fail("a scalar added before a scale has no fused form")
            body.bias, body.scale, body.shift = stages[0][1], stages[1][1], stages[2][1]
        else:
            _fail(f"affine chain {kinds!r} is longer than (acc + bias) * scale + shift")

    def _strip_cast(self, node: ast.AST, body: GemmBody) -> ast.AST:
        while isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr == "to" and len(node.args) == 1:
            _dtype_of(node.args[0], self.params)  # must be a dtype we know; the store rounds to out's dtype anyway
            node = node.func.value
        return node

    def _affine(self, node: ast.AST, acc: str, tile_n: str, stages: list[tuple[str, Operand]]) -> None:
        """Innermost first: appends ('add'|'mul', operand) for each level around ``acc``."""
        if _names(node) == [acc] and isinstance(node, ast.Name):
            return
        if isinstance(node, ast.BinOp) and isinstance(node.op, (ast.Add, ast.Mult, ast.Sub)):
            left_has = self._mentions(node.left, acc)
            right_has = self._mentions(node.right, acc)
            if left_has == right_has:
                _fail(f"{ast.unparse(node)!r} is not affine in the accumulator")
            inner, other = (node.left, node.right) if left_has else (node.right, node.left)
            if isinstance(node.op, ast.Sub):
                if not left_has or not isinstance(other, ast.Constant):
                    _fail("only `expr - constant` subtractions are fused")
                operand = Operand(value=-float(other.value))
                kind = "add"
            else:
                operand = self._operand(other, tile_n)
                kind = "add" if isinstance(node.op, ast.Add) else "mul"
            self._affine(inner, acc, tile_n, stages)
            stages.append((kind, operand))
            return
        _fail(f"{ast.unparse(node)!r} is not an affine expression of the accumulator")

    @staticmethod
    def _mentions(node: ast.AST, name: str) -> bool:
        return any(isinstance(n, ast.Name) and n.id == name for n in ast.walk(node))

    def _operand(self, node: ast.AST, tile_n: str) -> Operand:
        if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)) and not isinstance(node.value, bool):
            return Operand(value=float(node.value))
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub) and isinstance(node.operand, ast.Constant):
            return Operand(value=-float(node.operand.value))
        if isinstance(node, ast.Name) and node.id in self.params:
            return Operand(name=node.id)  # a scalar parameter
        if isinstance(node, ast.Subscript) and _dotted(node.value) in self.params:
            index = node.slice
            names = _names(index)
            # bias[tile_n], or bias[None, tile_n] with the row axis broadcast
            if names == [tile_n] and (isinstance(index, ast.Name) or (
                    isinstance(index, ast.Tuple) and len(index.elts) == 2
                    and isinstance(index.elts[0], ast.Constant) and index.elts[0].value is None)):
                return Operand(name=_dotted(node.value), vector=True)
        _fail(f"epilogue operand {ast.unparse(node)!r} is neither a scalar nor a [N] vector tile")
        raise AssertionError


def gemm_body(fn: Callable[..., object]) -> GemmBody | None:
    """The GEMM a kernel body computes, or ``None`` if it is not a plain tiled GEMM
    with an affine + activation store."""
    try:
        return _Parser(fn).parse()
    except _NotRecognised:
        return None
    except SyntaxError:
        return None


def why_not(fn: Callable[..., object]) -> str | None:
    """Why ``gemm_body`` does not recognise ``fn`` (``None`` if it does)."""
    try:
        _Parser(fn).parse()
    except _NotRecognised as reason:
        return str(reason)
    except SyntaxError as reason:
        return f"source does not parse: {reason}"
    return None


def gemm_adapter(body: GemmBody, block_sizes: tuple[int, ...] | None = None) -> Callable[..., object]:
    """A callable with the kernel body's own parameter list that runs the recognised
    GEMM on the native kernel; ``block_sizes`` (the kernel config's) are tile hints."""
    import torch.nn.functional as F

    import helion_mlir_utils as ops

    epilogue = {
        None: ops.identity_epilogue,
        "relu": torch.relu,
        "gelu": ops.gelu_tanh if body.gelu_tanh else F.gelu,
        "sigmoid": torch.sigmoid,
        "tanh": torch.tanh,
        "silu": F.silu,
        "leaky_relu": ops.leaky_relu_epilogue(body.slope),
    }[body.activation]
    # hl.tile([m, n]) and hl.tile(k) take their block sizes in that order: [m, n, k].
    hint = tuple(block_sizes[:3]) if block_sizes and len(block_sizes) >= 3 else None

    def run(*args: object, **kwargs: object) -> object:
        if len(args) > len(body.params):
            raise TypeError(f"takes {len(body.params)} positional arguments but {len(args)} were given")
        bound = dict(zip(body.params, args))
        for name, value in kwargs.items():
            if name not in body.params or name in bound:
                raise TypeError(f"unexpected or repeated argument {name!r}")
            bound[name] = value
        missing = [p for p in body.params if p not in bound]
        if missing:
            raise TypeError(f"missing arguments: {', '.join(missing)}")
        a, b = bound[body.a], bound[body.b]

        def operand(op: Operand | None) -> torch.Tensor | None:
            if op is None:
                return None
            if op.vector:
                return bound[op.name]  # type: ignore[return-value]
            value = op.value if op.name is None else getattr(bound[op.name], "value", bound[op.name])
            if isinstance(value, torch.Tensor):
                return value.reshape(-1)
            return torch.full((1,), float(value), dtype=torch.float32, device=a.device)  # type: ignore[union-attr, arg-type]

        out_dtype = bound[body.out_dtype].dtype if isinstance(body.out_dtype, str) else body.out_dtype  # type: ignore[union-attr]
        return ops.matmul(
            a, b, trans_a=body.trans_a, trans_b=body.trans_b, bias=operand(body.bias), epilogue=epilogue,
            scale=operand(body.scale), shift=operand(body.shift), out_dtype=out_dtype, block_sizes=hint,
        )

    run.__name__ = "native_gemm_body"
    run.recognised = body  # type: ignore[attr-defined]
    return run
