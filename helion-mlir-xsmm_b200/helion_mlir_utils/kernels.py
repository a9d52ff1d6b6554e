"""Kernels of one body that differ by tile config.

Same shape as ``helion_mlir_utils/kernels.py`` of the reference:
``@per_config(backend="mlir")`` on a kernel body makes its name take a hashable
``block_sizes`` and return that config's kernel, cached per config, with the raw
body reachable as ``.body`` and the cache as ``.cache_info()``.

With Helion installed the returned object is a real ``helion.Kernel`` on the
registered backend (which recognises the body and dispatches to the native
kernel). Without Helion it is a :class:`NativeKernel`: the native implementation
registered for the body, carrying the tile hint.
"""

from __future__ import annotations

import functools
from typing import Callable

from helion_mlir_backend import inject
from helion_mlir_backend.errors import UnsupportedOperationError


class NativeKernel:
    """A kernel body bound to one tile config, run by its hand-written kernel."""

    def __init__(self, body: Callable[..., object], block_sizes: tuple[int, ...]) -> None:
        self.fn = body
        self.block_sizes = tuple(block_sizes)
        self.name = body.__name__
        self._native: Callable[..., object] | None = None

    def _resolve(self) -> Callable[..., object]:
        if self._native is None:
            native_op = inject.recognise(self.fn, {"block_sizes": list(self.block_sizes)})
            if native_op is None:
                raise UnsupportedOperationError(f"{self.name}: no hand-written B200 kernel is registered for this body")
            self._native = native_op
        return self._native

    def __call__(self, *args: object, **kwargs: object) -> object:
        return self._resolve()(*args, **kwargs)

    def bind(self, args: tuple[object, ...]) -> Callable[..., object]:
        """Helion's ``Kernel.bind``: the callable for these argument types."""
        return self._resolve()


def per_config(**kernel_args: object) -> Callable[[Callable[..., object]], Callable[[tuple[int, ...]], object]]:
    """A kernel per tile config (see the module docstring)."""

    def wrap(body: Callable[..., object]) -> Callable[[tuple[int, ...]], object]:
        @functools.cache
        def for_config(block_sizes: tuple[int, ...]) -> object:
            try:
                import helion
            except ImportError:
                return NativeKernel(body, tuple(block_sizes))
            return helion.kernel(body, config=helion.Config(block_sizes=list(block_sizes)), **kernel_args)

        for_config.body = body  # type: ignore[attr-defined]
        return for_config

    return wrap
