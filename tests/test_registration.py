"""Backend registration against a stand-in for Helion's registry (Helion itself is
not installed in the build image): install() registers a backend named "mlir",
patches BoundKernel.compile_config for kernels on that backend, widens the config
keys, and kernels are recognised by body name and routed to native adapters."""

from __future__ import annotations

import importlib
import sys
import types

import pytest


@pytest.fixture()
def fake_helion(monkeypatch: pytest.MonkeyPatch):
    registry: dict[str, type] = {}

    class Backend:
        pass

    class BoundKernel:
        def __init__(self, fn, backend) -> None:
            self.kernel = types.SimpleNamespace(fn=fn)
            self.env = types.SimpleNamespace(backend=backend)

        def compile_config(self, config=None, *, allow_print: bool = True):
            return "helion-original"

    def register_compiler_backend(cls) -> None:
        registry[cls().name] = cls

    modules = {
        "helion": types.ModuleType("helion"),
        "helion._compiler": types.ModuleType("helion._compiler"),
        "helion._compiler.backend": types.ModuleType("helion._compiler.backend"),
        "helion._compiler.backend_registry": types.ModuleType("helion._compiler.backend_registry"),
        "helion.runtime": types.ModuleType("helion.runtime"),
        "helion.runtime.kernel": types.ModuleType("helion.runtime.kernel"),
        "helion.runtime.config": types.ModuleType("helion.runtime.config"),
    }
    modules["helion._compiler.backend"].Backend = Backend
    modules["helion._compiler.backend_registry"].register_compiler_backend = register_compiler_backend
    modules["helion.runtime.kernel"].BoundKernel = BoundKernel
    modules["helion.runtime.config"].VALID_KEYS = frozenset({"block_sizes", "num_warps"})
    modules["helion.runtime"].config = modules["helion.runtime.config"]
    for name, module in modules.items():
        monkeypatch.setitem(sys.modules, name, module)
    inject = importlib.import_module("helion_mlir_backend.inject")
    monkeypatch.setattr(inject, "_installed", False)
    yield types.SimpleNamespace(registry=registry, BoundKernel=BoundKernel, modules=modules, inject=inject)


def test_install_registers_and_routes(fake_helion) -> None:
    from helion_mlir_backend.errors import UnsupportedOperationError

    inject = fake_helion.inject
    assert inject.install() is True
    backend_class = fake_helion.registry["mlir"]
    backend = backend_class()
    assert backend.name == "mlir" and backend.experimental is True
    assert backend.supports_config_key("block_sizes") and backend.supports_config_key("mlir_pipeline")
    assert not backend.supports_config_key("num_warps")
    assert backend.supports_precompile() is False and backend.pad_factory_tensors_to_power_of_2 is False
    assert backend.classify_autotune_exception(UnsupportedOperationError("x")) == "warn"
    assert backend.classify_autotune_exception(ValueError("x")) is None
    assert "mlir_pipeline" in fake_helion.modules["helion.runtime.config"].VALID_KEYS

    def _softmax_kernel(x, whole, in_place=False):  # the reference's body, by name and parameters
        raise AssertionError("bodies are never executed: the native kernel runs instead")

    def something_else(x):
        return x

    ours = fake_helion.BoundKernel(_softmax_kernel, backend)
    native_op = ours.compile_config({"block_sizes": [128, 8]})
    assert callable(native_op) and native_op != "helion-original"
    with pytest.raises(UnsupportedOperationError, match="matches none of them"):
        fake_helion.BoundKernel(something_else, backend).compile_config({"block_sizes": []})
    # autotune / benchmarking hooks Helion calls on the backend (backend.py:81-113 of the reference)
    ours.kernel.configs = [{"block_sizes": [128, 8]}, {"block_sizes": [64, 8]}]
    assert backend.autotune(ours, (), force=True) == {"block_sizes": [128, 8]}  # hints only: the first config stands
    ours.kernel.configs = []
    ours.config_spec = types.SimpleNamespace(default_config=lambda: {"block_sizes": [1, 1]})
    assert backend.autotune(ours, (), force=False) == {"block_sizes": [1, 1]}
    del ours.config_spec
    with pytest.raises(UnsupportedOperationError, match="no config"):
        backend.autotune(ours, ())
    assert callable(backend.get_do_bench()) and callable(backend.get_interleaved_bench())
    other_backend = types.SimpleNamespace(name="triton")
    assert fake_helion.BoundKernel(_softmax_kernel, other_backend).compile_config({}) == "helion-original"
    assert inject.install() is True  # idempotent


def test_bodies_are_matched_by_name_and_parameters() -> None:
    from helion_mlir_backend import bodies

    def _matmul_fused_pack(a, b, bias, scale, shift, epilogue, k_chunked, k_even, trans_a, trans_b, out=None):
        pass

    def _row_sum_kernel(x, epilogue):
        pass

    assert bodies.adapter_for(_matmul_fused_pack, (128, 256, 64, 64)) is not None
    assert bodies.adapter_for(_row_sum_kernel, None) is not None

    def _row_sum_kernel_wrong(y):  # right name, wrong parameters
        pass

    _row_sum_kernel_wrong.__name__ = "_row_sum_kernel"
    assert bodies.adapter_for(_row_sum_kernel_wrong, None) is None
    assert bodies.adapter_for(lambda x: x, None) is None
    assert len(bodies.KNOWN_BODIES) == 32  # the operator set's 29, the two attention bodies of the tests, the packed-GEMM example
