"""``inline_mlir`` of the reference (``helion_mlir_backend/language.py``) lets a
kernel splice user MLIR into device loops. Without an IR stage there is nothing
to splice into: the names exist so that imports keep working, and use raises."""

from __future__ import annotations

from .errors import UnsupportedOperationError


class InlineMLIRHint:
    def __init__(self, *args: object, **kwargs: object) -> None:
        raise UnsupportedOperationError("InlineMLIRHint: the B200 backend has no MLIR stage")


def inline_mlir(*args: object, **kwargs: object) -> object:
    raise UnsupportedOperationError("inline_mlir(): the B200 backend has no MLIR stage")
