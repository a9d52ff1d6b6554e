"""Public IR API of the reference (``helion_mlir_backend/api.py``), kept as names.

The reference lowers a Helion kernel to MLIR and JIT-compiles it. This backend
has no IR: each operator is a fixed CUDA kernel family behind a C ABI. The three
functions therefore raise :class:`UnsupportedOperationError` with that
explanation, except ``compile_mlir`` for kernels whose body is one of the
``helion_mlir_utils`` operators, which returns the native callable.
"""

from __future__ import annotations

from typing import Callable

from .errors import UnsupportedOperationError

_NO_IR = (
    "the B200 backend has no MLIR stage: operators run as ahead-of-time compiled sm_100a kernels "
    "(see helion_mlir_backend.explain for what a call launches)"
)


def generate_mlir(kernel: object, args: list[object], *, config: object | None = None, target: str | None = None):
    raise UnsupportedOperationError(f"generate_mlir(): {_NO_IR}")


def lower_mlir(
    kernel: object,
    args: list[object],
    *,
    config: object | None = None,
    target: str | None = None,
    pipeline: str | None = None,
    stop_at: str | None = None,
):
    raise UnsupportedOperationError(f"lower_mlir(): {_NO_IR}")


def compile_mlir(
    kernel: object,
    args: list[object],
    *,
    config: object | None = None,
    target: str | None = None,
    pipeline: str | None = None,
) -> Callable[..., object]:
    """The native callable for a kernel this backend recognises (see
    :func:`helion_mlir_backend.inject.recognise`); others raise."""
    from .inject import recognise

    fn = getattr(kernel, "fn", kernel)
    native_op = recognise(fn, config)
    if native_op is None:
        raise UnsupportedOperationError(f"compile_mlir(): no hand-written B200 kernel matches {fn!r}; {_NO_IR}")
    return native_op
