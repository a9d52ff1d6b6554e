"""Exceptions of the backend surface (names kept from
``helion_mlir_backend/_compiler/mlir/support/errors.py`` of the reference)."""

from __future__ import annotations


class MLIRBackendError(RuntimeError):
    """Base class of errors raised by this backend."""


class UnsupportedOperationError(MLIRBackendError):
    """The kernel or operation has no hand-written B200 implementation."""
