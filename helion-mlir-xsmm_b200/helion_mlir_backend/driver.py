"""Per-call host path: prepared calls and config-key checks.

Counterpart of ``helion_mlir_backend/_compiler/mlir/driver.py`` of the
reference, reduced to what a backend without a compiler needs:
:func:`prepared_call` (driver.py:748-788) and the once-per-kernel warning for
misspelt config keys (driver.py:48-72).
"""

from __future__ import annotations

import difflib
from typing import Callable
from typing import Sequence
import warnings

import torch

CONFIG_KEYS = frozenset({"block_sizes", "mlir_pipeline"})
_warned: set[tuple[str, str]] = set()


def warn_misspelt_config_keys(kernel_name: str, config: object) -> None:
    """Unknown config keys are ignored; one that is a near miss of a key this
    backend reads warns once per (kernel, key)."""
    keys = list(getattr(config, "config", config) or ())
    for key in keys:
        if key in CONFIG_KEYS or (kernel_name, key) in _warned:
            continue
        close = difflib.get_close_matches(key, CONFIG_KEYS, n=1, cutoff=0.8)
        if close:
            _warned.add((kernel_name, key))
            warnings.warn(
                f"{kernel_name}: config key {key!r} is ignored by the B200 backend; did you mean {close[0]!r}?",
                stacklevel=3,
            )


class PreparedRun:
    """``lambda *v: run(*args with v at the varying positions)`` with the checks a
    native run makes done up front: the varying tensors must have the recorded
    shape, dtype, device and be contiguous; anything else takes ``fallback``."""

    __slots__ = ("_expected", "_fallback", "_run", "native_calls", "fallback_calls")

    def __init__(
        self,
        run: Callable[..., object],
        expected: Sequence[tuple[tuple[int, ...], torch.dtype, torch.device]],
        fallback: Callable[..., object],
    ) -> None:
        self._run = run
        self._expected = tuple(expected)
        self._fallback = fallback
        self.native_calls = 0
        self.fallback_calls = 0

    def __call__(self, *varying: torch.Tensor) -> object:
        expected = self._expected
        if len(varying) == len(expected):
            for value, (shape, dtype, device) in zip(varying, expected):
                if (
                    type(value) is not torch.Tensor
                    or value.shape != shape
                    or value.dtype is not dtype
                    or value.device != device
                    or not value.is_contiguous()
                ):
                    break
            else:
                self.native_calls += 1
                return self._run(*varying)
        self.fallback_calls += 1
        return self._fallback(*varying)


def prepared_call(
    bound_kernel: object,
    args: Sequence[object],
    varying: Sequence[int],
    fallback: Callable[..., object],
    *,
    views: Sequence[Sequence[int] | None] | None = None,
    result_shape: Sequence[int] | None = None,
) -> Callable[..., object] | None:
    """A call of ``bound_kernel`` with everything but the ``varying`` arguments fixed.

    ``bound_kernel`` is a launch plan of this backend: any object with a
    ``prepare(args, varying, views, result_shape)`` method returning the fast
    callable for the varying tensors (``helion_mlir_utils`` plans have one).
    ``views[k]``: the caller passes a contiguous tensor of that shape standing for
    the kernel's view of the argument. Returns ``None`` if ``bound_kernel`` has no
    such method (the caller then keeps its general path), as the reference does
    for kernels without a native run.
    """
    prepare = getattr(bound_kernel, "prepare", None)
    if prepare is None:
        return None
    varying = list(varying)
    views = [None] * len(varying) if views is None else [None if v is None else tuple(v) for v in views]
    if len(views) != len(varying):
        raise ValueError("views must have one entry per varying argument")
    expected = []
    for position, view in zip(varying, views):
        value = args[position]
        if not isinstance(value, torch.Tensor):
            return None
        shape = tuple(value.shape) if view is None else view
        if view is not None and value.numel() != _numel(view):
            # A view that changes the element count can never match: always the fallback.
            return fallback
        expected.append((torch.Size(shape), value.dtype, value.device))
    run = prepare(tuple(args), varying, views, None if result_shape is None else tuple(result_shape))
    if run is None:
        return None
    return PreparedRun(run, expected, fallback)


def _numel(shape: Sequence[int]) -> int:
    total = 1
    for size in shape:
        total *= size
    return total
