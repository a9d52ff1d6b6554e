"""Backend registration with Helion.

Counterpart of ``helion_mlir_backend/inject.py`` of the reference:
:func:`install` registers a compiler backend named ``"mlir"`` with Helion's
backend registry and routes ``BoundKernel.compile_config`` of kernels that
select it to this package (inject.py:22-56, 726-748). The reference's backend
compiles the kernel body; this one *recognises* it: a body that is one of the
``helion_mlir_utils`` operator bodies (or the canonical addmm tile loop) is
mapped to its hand-written sm_100a kernel, with ``block_sizes`` passed on as tile
hints, and any other body raises :class:`UnsupportedOperationError`.

Helion is an optional dependency: without it :func:`install` returns ``False``
(as inject.py:27-40 does on ``ImportError``) and the operator set still works
through its own entry points.
"""

from __future__ import annotations

import logging
from typing import Callable
from typing import Sequence

from .driver import CONFIG_KEYS
from .driver import warn_misspelt_config_keys
from .errors import UnsupportedOperationError

log = logging.getLogger(__name__)

BACKEND_NAME = "mlir"
PIPELINE_CONFIG_KEY = "mlir_pipeline"

# body function (by code object) -> factory(block_sizes) -> native callable
_RECOGNISED: dict[object, Callable[[tuple[int, ...] | None], Callable[..., object]]] = {}
_installed = False


def register_body(body: Callable[..., object], factory: Callable[[tuple[int, ...] | None], Callable[..., object]]) -> None:
    """Declare ``factory(block_sizes)`` as the native implementation of a kernel body."""
    _RECOGNISED[body.__code__] = factory


def recognise(fn: Callable[..., object], config: object | None = None) -> Callable[..., object] | None:
    """The native callable for kernel body ``fn`` under ``config``, or ``None``."""
    block_sizes = None
    if config is not None:
        values = getattr(config, "config", config)
        try:
            block_sizes = tuple(int(v) for v in values.get("block_sizes", ()))  # type: ignore[union-attr]
        except AttributeError:
            block_sizes = None
    code = getattr(fn, "__code__", None)
    factory = _RECOGNISED.get(code)
    if factory is not None:
        return factory(block_sizes)
    # The bodies of the reference's operator set, known by name and parameter list.
    from .bodies import adapter_for

    adapter = adapter_for(fn, block_sizes)
    if adapter is not None:
        return adapter
    # Any other body that is a plain tiled GEMM with an affine + activation store.
    from .structure import gemm_adapter, gemm_body

    body = gemm_body(fn)
    return None if body is None else gemm_adapter(body, block_sizes)


def make_backend_class(base: type) -> type:
    """The backend class registered with Helion (cf. ``MLIRBackend``,
    ``_compiler/mlir/backend.py:44-122``): same name, same config keys, no
    precompile, no power-of-two padding of factory tensors."""

    class B200Backend(base):  # type: ignore[misc, valid-type]
        @property
        def name(self) -> str:
            return BACKEND_NAME

        @property
        def experimental(self) -> bool:
            return True

        def supports_config_key(self, key: str) -> bool:
            return key in CONFIG_KEYS

        def supports_precompile(self) -> bool:
            return False

        @property
        def pad_factory_tensors_to_power_of_2(self) -> bool:
            return False

        def classify_autotune_exception(self, err: BaseException) -> str | None:
            return "warn" if isinstance(err, UnsupportedOperationError) else None

        def autotune(self, bound_kernel: object, args: Sequence[object], *, force: bool = True, **kwargs: object) -> object:
            """A config's ``block_sizes`` are tile hints here, so there is no space of
            generated kernels to search (cf. ``MLIRBackend.autotune``,
            ``_compiler/mlir/backend.py:81-103``, which narrows Helion's search to what its
            target compiles). What is measured instead is the launch choice of the
            hand-written GEMM for the operands at hand (tile width, CTA pairs, K splits:
            ``helion_mlir_utils.tuning``), stored per hardware name where later calls
            find it; the config returned is the kernel's first given one, else Helion's
            default for its spec."""
            return autotune_choice(bound_kernel, args, force=force, fallback=getattr(super(), "autotune", None), **kwargs)

        def get_do_bench(self) -> Callable[..., float]:
            """Timing function for Helion's autotuner (``backend.py:105-108`` returns a host
            timer): CUDA events on the current stream, milliseconds per call."""
            return do_bench

        def get_interleaved_bench(self) -> Callable[..., list[float]]:
            return interleaved_bench

    B200Backend.__name__ = "MLIRBackend"
    return B200Backend


def do_bench(fn: Callable[[], object], *_: object, warmup: int = 3, rep: int = 20, **__: object) -> float:
    """Milliseconds per call of ``fn`` (CUDA events on the current stream, after a warm-up)."""
    from helion_mlir_utils import tuning

    return tuning.time_call(fn, iterations=max(1, int(rep)), warmup=max(0, int(warmup))) * 1e-3


def interleaved_bench(fns: Sequence[Callable[[], object]], *_: object, repeat: int = 20, **__: object) -> list[float]:
    """Milliseconds per call of each function, the functions taking turns so that clock
    changes fall on all of them alike."""
    import torch

    fns = list(fns)
    for fn in fns:
        fn()
    totals = [0.0] * len(fns)
    for _ in range(max(1, int(repeat))):
        for i, fn in enumerate(fns):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            stop.synchronize()
            totals[i] += start.elapsed_time(stop)
    return [t / max(1, int(repeat)) for t in totals]


def autotune_choice(bound_kernel: object, args: Sequence[object], *, force: bool = True,
                    fallback: Callable[..., object] | None = None, **kwargs: object) -> object:
    """See ``B200Backend.autotune``. Two bf16 matrices among ``args`` whose inner sizes
    agree are taken as the operands of a recognised GEMM body and tuned; anything else
    leaves the table alone."""
    kernel = getattr(bound_kernel, "kernel", None)
    fn = getattr(kernel, "fn", None)
    configs = list(getattr(kernel, "configs", None) or [])
    if fn is not None and force:
        try:
            import torch

            from helion_mlir_utils import tuning

            mats = [t for t in args if isinstance(t, torch.Tensor) and t.dim() == 2 and t.is_cuda and t.dtype == torch.bfloat16]
            if len(mats) >= 2 and mats[0].shape[1] == mats[1].shape[0] and recognise(fn, configs[0] if configs else None) is not None:
                tuning.tune_matmul(mats[0], mats[1])
        except (RuntimeError, ValueError, ImportError) as exc:
            log.debug("autotune: launch choice not measured: %s", exc)
    if configs:
        return configs[0]
    spec = getattr(bound_kernel, "config_spec", None)
    default = getattr(spec, "default_config", None)
    if callable(default):
        return default()
    if fallback is not None:
        return fallback(bound_kernel, args, force=force, **kwargs)
    raise UnsupportedOperationError("autotune: the kernel has no config and no config spec to take a default from")


def compile_config(bound_kernel: object, config: object, *, allow_print: bool = True) -> Callable[..., object]:
    """What ``BoundKernel.compile_config`` returns for kernels on this backend
    (cf. ``mlir_compile_config``, ``_compiler/mlir/driver.py:75-92``)."""
    kernel = getattr(bound_kernel, "kernel", None)
    fn = getattr(kernel, "fn", None)
    name = getattr(fn, "__name__", "kernel")
    warn_misspelt_config_keys(name, config)
    native_op = recognise(fn, config) if fn is not None else None
    if native_op is None:
        raise UnsupportedOperationError(
            f"{name}: the B200 backend runs hand-written kernels for the helion_mlir_utils operator set; "
            "this kernel body matches none of them"
        )
    return native_op


def install() -> bool:
    """Register the backend with Helion. ``True`` when registration was applied."""
    global _installed
    if _installed:
        return True
    try:
        from helion._compiler.backend import Backend
        from helion._compiler.backend_registry import register_compiler_backend
        from helion.runtime.kernel import BoundKernel
    except ImportError as exc:
        log.debug("Helion backend registration unavailable: %s", exc)
        return False

    backend_class = make_backend_class(Backend)
    register_compiler_backend(backend_class)
    original = BoundKernel.compile_config

    def patched(self, config=None, *, allow_print: bool = True):  # type: ignore[no-untyped-def]
        env = getattr(self, "env", None)
        if getattr(getattr(env, "backend", None), "name", None) == BACKEND_NAME:
            return compile_config(self, config, allow_print=allow_print)
        return original(self, config, allow_print=allow_print)

    BoundKernel.compile_config = patched
    try:  # let Config accept `mlir_pipeline` (accepted and ignored: there is one pipeline)
        from helion.runtime import config as helion_config

        keys = getattr(helion_config, "VALID_KEYS", None)
        if keys is not None and PIPELINE_CONFIG_KEY not in keys:
            helion_config.VALID_KEYS = frozenset(keys) | {PIPELINE_CONFIG_KEY}
    except ImportError:
        pass
    _installed = True
    return True
