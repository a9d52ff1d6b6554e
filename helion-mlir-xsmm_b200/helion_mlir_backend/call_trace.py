"""``explain()``: what a call of an operator would launch.

Counterpart of ``helion_mlir_backend/_compiler/call_trace.py`` of the reference,
whose ``explain`` reports whether a call takes the native path and why not. Here
every call is native; the explanation names the kernel family, tile and grid
(``b200_gemm_explain``) or the refusal.
"""

from __future__ import annotations

import dataclasses
import os
import sys

TRACE_ENV = "HELION_MLIR_TRACE_CALLS"
_trace = os.environ.get(TRACE_ENV, "").strip() not in ("", "0")


@dataclasses.dataclass(frozen=True)
class CallExplanation:
    native: bool
    kernel: str
    reason: str | None = None

    def __str__(self) -> str:
        if self.native:
            return f"native: {self.kernel}"
        return f"refused: {self.reason}"


def explain(op: object, *args: object, **kwargs: object) -> CallExplanation:
    """Explain a call of a ``helion_mlir_utils`` operator without running it.
    Operators that plan their launch expose ``.explain(*args, **kwargs)``; the
    others are single fixed kernels."""
    planner = getattr(op, "explain", None)
    if planner is not None:
        return planner(*args, **kwargs)
    name = getattr(op, "__name__", repr(op))
    return CallExplanation(True, f"{name}: one fixed bandwidth-bound kernel family (see csrc/)")


def trace(message: str) -> None:
    if _trace:
        sys.stderr.write(f"[b200ops] {message}\n")
