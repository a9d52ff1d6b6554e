"""Host-side logic that needs no GPU: heuristics, error behaviour, registration
surface, prepared calls, the pool's fall-through rules."""

from __future__ import annotations

import functools
import warnings

import pytest
import torch
import torch.nn.functional as F

import helion_mlir_backend
from helion_mlir_backend import native
from helion_mlir_backend import output_pool
from helion_mlir_backend.driver import PreparedRun
from helion_mlir_backend.driver import prepared_call
from helion_mlir_backend.driver import warn_misspelt_config_keys
from helion_mlir_backend.errors import UnsupportedOperationError
import helion_mlir_utils as ops
from helion_mlir_utils import epilogues
import importlib

mm = importlib.import_module("helion_mlir_utils.matmul")

REFERENCE_NAMES = [
    "CACHE_PREPACKED_WEIGHTS_ENV", "AffineLinearCache", "LinearCache", "bmm", "cache_prepacked_weights",
    "column_sum", "group_norm", "identity_epilogue", "leaky_relu", "linear", "linear_affine", "matmul",
    "matmul_prepacked_b", "matmul_prepacked_b_affine", "matvec", "pack_a_blocked", "pack_a_blocked_t",
    "pack_b_blocked", "pack_b_blocked_t", "pack_b_blocked_vnni", "pack_b_blocked_vnni_t", "pack_b_vnni_t",
    "per_config", "relu", "row_dot", "row_sum", "scalar_mul", "softmax", "supports", "supports_matvec",
    "tall_output_tiles",
]  # helion_mlir_utils/__init__.py:37-69 of the reference


def test_operator_set_has_every_reference_name() -> None:
    for name in REFERENCE_NAMES:
        assert hasattr(ops, name), name
        assert name in ops.__all__
    for name in ("layer_norm", "rms_norm", "matmul_blocked"):
        assert name in ops.__all__


def test_backend_surface() -> None:
    for name in ("install", "output_pool", "prepared_call", "set_native_call", "set_output_pool", "explain",
                 "CallExplanation", "generate_mlir", "compile_mlir", "lower_mlir", "inline_mlir", "InlineMLIRHint"):
        assert hasattr(helion_mlir_backend, name), name
    # Helion is not installed in the build image: registration reports so, as the reference does.
    try:
        import helion  # noqa: F401
    except ImportError:
        assert helion_mlir_backend.install() is False
    with pytest.raises(UnsupportedOperationError, match="no MLIR stage"):
        helion_mlir_backend.generate_mlir(object(), [])
    with pytest.raises(UnsupportedOperationError):
        helion_mlir_backend.lower_mlir(object(), [])
    with pytest.raises(UnsupportedOperationError):
        helion_mlir_backend.inline_mlir("x")


def test_cpu_operands_raise_instead_of_falling_back() -> None:
    a, b = torch.randn(4, 8), torch.randn(8, 4)
    assert not ops.supports(a, b)
    with pytest.raises(ValueError, match=r"matmul\(\) does not support these operands"):
        ops.matmul(a, b)
    with pytest.raises(ValueError, match="CUDA"):
        ops.softmax(a)
    with pytest.raises(ValueError, match=r"softmax\(\) expects a 2-D tensor"):
        ops.softmax(torch.randn(3))
    with pytest.raises(ValueError, match=r"group_norm\(\) expects \[M, C\] with C divisible by 3 groups"):
        ops.group_norm(torch.randn(2, 8), 3, None, None, 1e-5)
    with pytest.raises(ValueError, match=r"row_sum\(\) expects a 2-D tensor"):
        ops.row_sum(torch.randn(3))
    with pytest.raises(ValueError, match=r"row_dot\(\) expects an f32 vector"):
        ops.row_dot(torch.randn(3, 4), torch.randn(4).bfloat16())
    with pytest.raises(ValueError, match=r"column_sum\(\) expects a 2-D tensor"):
        ops.column_sum(torch.randn(3))
    assert not ops.supports_matvec(torch.randn(3, 4), torch.randn(4, 1))
    with pytest.raises(ValueError, match=r"matvec\(\) does not support these operands"):
        ops.matvec(torch.randn(3, 4), torch.randn(4, 1))
    with pytest.raises(RuntimeError, match="Expected size for first two dimensions of batch2 tensor"):
        ops.bmm(torch.randn(2, 3, 4), torch.randn(2, 5, 4))
    with pytest.raises(ValueError, match="even K and a panel of a multiple of 32"):
        ops.pack_b_vnni_t(torch.randn(4, 3))
    with pytest.raises(ValueError, match="tile_m must be a positive multiple of 32"):
        ops.prepacked_b_call(torch.randn(4, 4), torch.randn(1, 1, 32, 32), 4, tile_m=33)


def test_tile_hints_are_pinned(monkeypatch: pytest.MonkeyPatch) -> None:
    monkeypatch.setattr(mm, "_sm_count", lambda: 148)
    assert ops.vnni_panel(8192, 4096, 4096) == 256
    assert ops.vnni_panel(8192, 4224) == 128
    assert ops.vnni_panel(64, 100) == 64
    assert ops.tall_output_tiles(128 * 148, 256, 1024) == (128, 256, 64)
    assert ops.tall_output_tiles(128 * 148 - 1, 256, 1024) is None
    assert ops.tall_output_tiles(1 << 20, 512, 1024) is None
    assert ops.whole_row_tiles(128 * 148, 4096) == (128, 256)
    assert ops.whole_row_tiles(128 * 148, 4096, 64) == (128, 64)
    assert ops.whole_row_tiles(128 * 148 + 32, 4096) is None
    assert ops.whole_row_tiles(128 * 148, 4000) is None
    # split-K: few tiles, deep K
    assert mm._split_k(256, 256, 8192) == 8
    assert mm._split_k(8192, 4096, 4096) == 0
    assert mm._split_k(128, 256, 1 << 16) == 64
    assert mm._split_k(128, 256, 1000) == 0


def test_epilogue_recognition() -> None:
    assert epilogues.resolve(ops.identity_epilogue) == (native.ACT_IDENTITY, 0.0)
    assert epilogues.resolve(torch.relu) == (native.ACT_RELU, 0.0)
    assert epilogues.resolve(F.gelu) == (native.ACT_GELU_ERF, 0.0)
    assert epilogues.resolve(functools.partial(F.gelu, approximate="tanh")) == (native.ACT_GELU_TANH, 0.0)
    assert epilogues.resolve(ops.gelu_tanh) == (native.ACT_GELU_TANH, 0.0)
    assert epilogues.resolve(torch.nn.LeakyReLU(0.2)) == (native.ACT_LEAKY_RELU, pytest.approx(0.2))
    assert epilogues.resolve(ops.leaky_relu_epilogue(0.3)) == (native.ACT_LEAKY_RELU, 0.3)
    assert epilogues.resolve(lambda x: x * 2) is None


def test_per_config_shape() -> None:
    @ops.per_config(backend="mlir")
    def body(x):
        return x

    assert body.body.__name__ == "body"
    k1, k2 = body((32, 64)), body((32, 64))
    assert k1 is k2 and body.cache_info().hits == 1
    assert body((64, 64)) is not k1


def test_misspelt_config_keys_warn_once() -> None:
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        warn_misspelt_config_keys("k", {"block_size": [1], "num_warps": 4, "block_sizes": [2]})
        warn_misspelt_config_keys("k", {"block_size": [1]})
    assert len(seen) == 1 and "block_sizes" in str(seen[0].message)


def test_prepared_call_contract() -> None:
    """tests/test_native_call.py:814-906 of the reference, restated for launch plans."""
    calls = {"native": 0, "fallback": 0}

    class Plan:
        def prepare(self, args, varying, views, result_shape):
            def run(x):
                calls["native"] += 1
                return x + 1

            return run

    def fallback(x):
        calls["fallback"] += 1
        return x + 1

    x = torch.zeros(4, 6)
    prepared = prepared_call(Plan(), (x,), [0], fallback)
    assert isinstance(prepared, PreparedRun)
    prepared(torch.ones(4, 6))
    assert calls == {"native": 1, "fallback": 0}
    prepared(torch.ones(6, 4))  # other shape
    prepared(torch.ones(4, 6, dtype=torch.float64))  # other dtype
    prepared(torch.ones(6, 4).T)  # not contiguous
    assert calls == {"native": 1, "fallback": 3}
    assert prepared.native_calls == 1 and prepared.fallback_calls == 3
    assert prepared_call(object(), (x,), [0], fallback) is None  # no native run: caller keeps its path
    assert prepared_call(Plan(), (x,), [0], fallback, views=[(5, 5)]) is fallback  # numel changes: always fallback
    viewed = prepared_call(Plan(), (x,), [0], fallback, views=[(2, 12)])
    viewed(torch.ones(2, 12))
    assert calls["native"] == 2


def test_pool_falls_through_to_torch_without_cuda() -> None:
    before = output_pool.output_pool_stats()
    t = output_pool.empty((1 << 21,), dtype=torch.float32, device=torch.device("cpu"))
    assert t.device.type == "cpu" and t.numel() == 1 << 21
    like = output_pool.empty_like(torch.zeros(3, 5), dtype=torch.bfloat16)
    assert like.shape == (3, 5) and like.dtype == torch.bfloat16
    meta = output_pool.empty((8, 8), dtype=torch.float32, device="meta")
    assert meta.device.type == "meta"
    with pytest.raises((RuntimeError, TypeError)):
        output_pool.empty((-1,), dtype=torch.float32, device="cpu")
    after = output_pool.output_pool_stats()
    assert (after["hits"], after["misses"]) == (before["hits"], before["misses"])
    assert output_pool.MIN_BYTES == 4 << 20 and output_pool.enabled()


def test_linear_cache_key_tracks_versions() -> None:
    from helion_mlir_utils.linear import _parameter_key

    p = torch.nn.Parameter(torch.zeros(4, 4))
    k0 = _parameter_key(p)
    with torch.no_grad():
        p.add_(1)
    assert _parameter_key(p) != k0  # in-place ops are seen
    k1 = _parameter_key(p)
    p.data.mul_(2)
    assert _parameter_key(p) == k1  # .data changes are not (documented)
    assert ops.cache_prepacked_weights() is True


def test_call_tracing_reports_first_calls_and_summarises(monkeypatch: pytest.MonkeyPatch, capsys: pytest.CaptureFixture[str]) -> None:
    """HELION_MLIR_TRACE_CALLS: one line for the first call of an operator with each kind of
    operands, a line for a call that raises, and per-operator counts in the at-exit summary
    (the reference: _compiler/call_trace.py:220-386). Off, nothing is wrapped."""
    from helion_mlir_backend import call_trace

    def op(x, flag=False):
        if flag:
            raise ValueError("refused on purpose")
        return x

    op.explain = lambda *a, **k: call_trace.CallExplanation(True, "one kernel")
    namespace = {"op": op, "LinearCache": dict}
    monkeypatch.setattr(call_trace, "_trace", False)
    call_trace.install(namespace, ["op", "LinearCache"])
    assert namespace["op"] is op
    monkeypatch.setattr(call_trace, "_trace", True)
    monkeypatch.setattr(call_trace, "_summary_registered", True)  # no atexit hook from a test
    call_trace.install(namespace, ["op", "LinearCache", "missing"])
    traced = namespace["op"]
    assert traced is not op and namespace["LinearCache"] is dict and traced.explain is op.explain
    x32, x16 = torch.zeros(2, 3), torch.zeros(4, dtype=torch.bfloat16)
    traced(x32), traced(x32), traced(x16)
    with pytest.raises(ValueError):
        traced(x32, flag=True)
    err = capsys.readouterr().err.splitlines()
    assert err == [
        "[helion-mlir] op(float32[2d]): native, one kernel",
        "[helion-mlir] op(bfloat16[1d]): native, one kernel",
        "[helion-mlir] op(float32[2d]): raised ValueError: refused on purpose",
    ]
    lines = call_trace.summary_lines()
    assert lines[0] == "at exit: op: 4 calls; raised: 1"
    assert lines[-1].startswith("at exit: library")


def test_environment_turns_the_pool_off_at_import(tmp_path) -> None:
    """tests/test_output_pool.py:333-345: HELION_MLIR_OUTPUT_POOL=0 read at import."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    code = (
        "import sys; sys.path.insert(0, r'%s'); "
        "from helion_mlir_backend import output_pool as p; "
        "print(p.output_pool_stats()['max_bytes'], p.enabled())" % (root / "helion-mlir-xsmm_b200")
    )
    import os

    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                          env={**os.environ, "HELION_MLIR_OUTPUT_POOL": "0"})
    assert done.returncode == 0, done.stderr
    assert done.stdout.split() == ["0", "False"]


def test_pool_falls_back_to_torch_for_what_it_does_not_take() -> None:
    """tests/test_output_pool.py:463-489: other devices, bad sizes, quantized, strided,
    conjugate and subclass tensors give exactly what torch's own functions give."""
    from helion_mlir_backend import output_pool

    before = output_pool.output_pool_stats()
    big, f32, cpu = (256, 256), torch.float32, torch.device("cpu")
    assert output_pool.empty((8, 8), dtype=f32, device=cpu).shape == (8, 8)
    assert output_pool.empty(big, dtype=f32, device=torch.device("meta")).is_meta
    with pytest.raises(RuntimeError):
        output_pool.empty((-1, 256), dtype=f32, device=cpu)
    with pytest.raises(TypeError):
        output_pool.empty(("a", 256), dtype=f32, device=cpu)
    assert output_pool.empty(big, dtype=torch.qint8, device=cpu).is_quantized
    x = torch.randn(256, 256)
    assert output_pool.empty_like(x[::2]).shape == (128, 256)
    assert output_pool.empty_like(x.t()).shape == big
    conjugate = torch.randn(256, 256, dtype=torch.complex64).conj()
    assert output_pool.empty_like(conjugate).is_conj() == torch.empty_like(conjugate).is_conj()

    class Sub(torch.Tensor):
        pass

    assert type(output_pool.empty_like(x.as_subclass(Sub))) is Sub
    after = output_pool.output_pool_stats()
    assert (after["hits"], after["misses"]) == (before["hits"], before["misses"])
