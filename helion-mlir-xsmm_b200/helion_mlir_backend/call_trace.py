"""``explain()``: what a call of an operator would launch.

Counterpart of ``helion_mlir_backend/_compiler/call_trace.py`` of the reference,
whose ``explain`` reports whether a call takes the native path and why not. Here
every call is native; the explanation names the kernel family, tile and grid
(``b200_gemm_explain``) or the refusal.
"""

from __future__ import annotations

import atexit
from collections.abc import Callable
import dataclasses
import functools
import os
import sys
import threading

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


# -- HELION_MLIR_TRACE_CALLS ---------------------------------------------------
# The reference prints, with tracing on, one line for the first call of each kernel on
# each path and for each reason (call_trace.py:220-328) and a summary of native calls
# and refusals per compiled kernel at exit (call_trace.py:331-386). Here: one line for
# the first call of each operator with each kind of operands (types and ranks; sizes go
# by uncounted), and at exit the calls per operator beside the library's own counters.
# Off (the default): nothing is wrapped.

_lock = threading.Lock()
_seen: set[tuple[str, str]] = set()
_calls: dict[str, int] = {}
_failures: dict[str, int] = {}
_summary_registered = False


def enabled() -> bool:
    return _trace


def _print(text: str) -> None:
    sys.stderr.write(f"[helion-mlir] {text}\n")


def trace(message: str) -> None:
    """A free-form line (shapes of a planned call), tracing on."""
    if _trace:
        _print(message)


def _kind(args: tuple[object, ...]) -> str:
    parts = []
    for value in args:
        dtype, dim = getattr(value, "dtype", None), getattr(value, "dim", None)
        if dtype is not None and callable(dim):
            parts.append(f"{str(dtype).replace('torch.', '')}[{dim()}d]")
    return ", ".join(parts)


def summary_lines() -> list[str]:
    """The at-exit report: calls (and calls that raised) per operator, then the
    library's counters (kernels launched, C-ABI calls, refusals, CUDA errors)."""
    with _lock:
        lines = [
            f"at exit: {name}: {count} calls" + (f"; raised: {_failures[name]}" if _failures.get(name) else "")
            for name, count in sorted(_calls.items())
        ]
    try:
        from . import native

        c = native.counters()
        lines.append(
            f"at exit: library: {c['calls']} native calls, {c['launches']} kernels launched, "
            f"{c['refusals']} refused" + (f" (last: {native.strerror(c['last_refusal'])})" if c["refusals"] else "")
            + (f", {c['cuda_errors']} CUDA errors" if c["cuda_errors"] else "")
        )
    except Exception as exc:  # noqa: BLE001 - the summary never raises at interpreter exit
        lines.append(f"at exit: library counters unavailable ({type(exc).__name__})")
    return lines


def _summary() -> None:
    for line in summary_lines():
        _print(line)


def traced(name: str, fn: Callable[..., object]) -> Callable[..., object]:
    """``fn`` reporting its calls under ``name``; attributes of ``fn`` (``explain``) are kept."""

    @functools.wraps(fn)
    def wrapper(*args: object, **kwargs: object) -> object:
        event = (name, _kind(args))
        with _lock:
            _calls[name] = _calls.get(name, 0) + 1
            first = event not in _seen
            _seen.add(event)
        try:
            result = fn(*args, **kwargs)
        except Exception as exc:
            with _lock:
                _failures[name] = _failures.get(name, 0) + 1
            _print(f"{name}({event[1]}): raised {type(exc).__name__}: {exc}")
            raise
        if first:
            line = f"{name}({event[1]}): native"
            planner = getattr(fn, "explain", None)
            if planner is not None:
                try:
                    line += f", {planner(*args, **kwargs).kernel}"
                except Exception:  # noqa: BLE001 - an explanation is a courtesy
                    pass
            _print(line)
        return result

    wrapper._helion_mlir_traced = True  # type: ignore[attr-defined]
    return wrapper


def install(namespace: dict[str, object], names: list[str]) -> None:
    """With tracing on, wrap the operators ``names`` of ``namespace`` and register the
    at-exit summary. Off: nothing is wrapped (cf. ``install``, call_trace.py:349-386)."""
    global _summary_registered
    if not _trace:
        return
    for name in names:
        fn = namespace.get(name)
        if callable(fn) and not isinstance(fn, type) and not getattr(fn, "_helion_mlir_traced", False):
            namespace[name] = traced(name, fn)
    if not _summary_registered:
        _summary_registered = True
        atexit.register(_summary)
