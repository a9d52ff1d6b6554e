"""A persisted table of measured launch choices, keyed by the hardware.

The reference picks its tile sizes from ``OMP_NUM_THREADS`` heuristics
(``helion_mlir_utils/matmul.py:400-467, 1057-1135``) and keeps autotuned configs
in a local cache keyed by ``hardware_name()`` (``MLIRAutotuneCache``,
``_compiler/mlir/autotune.py:25-49``). Here the heuristics live in the launcher
(column-tile width from the tile count, CTA pairs from the wave count, K splits
from the SM count); this module lets a measurement overrule them:

* :func:`tune_matmul` times the candidate ``(tile_n, cta_group, split_k)`` choices
  for one problem with CUDA events and records the fastest,
* :func:`lookup` is consulted when a GEMM is planned (once per problem: plans are
  cached), and an entry becomes the plan's tile hint, kernel choice and split,
* the table is one JSON file per hardware name under ``B200_TUNE_DIR`` (default
  ``~/.cache/helion_mlir_b200``), written atomically, ignored when unreadable.

Every candidate computes the same sums in the same order per output element
(a K split changes the order, so split candidates are only tried on request),
so a tuned plan returns the same bits as the untuned one unless ``split_k`` moved.
"""

from __future__ import annotations

import hashlib
import importlib
import json
import os
import tempfile
import threading
from collections.abc import Callable, Iterable
from dataclasses import asdict, dataclass
from pathlib import Path

import torch
from torch import Tensor

TUNE_DIR_ENV = "B200_TUNE_DIR"
TUNE_DISABLE_ENV = "B200_TUNE_DISABLE"
_FORMAT = 1


@dataclass(frozen=True)
class Choice:
    """One launch choice of the bf16 tensor-core GEMM."""

    tile_n: int = 0  # columns of the output tile (0: the launcher's heuristic)
    cta_group: int = 0  # 1: one CTA per 128-row tile, 2: a CTA pair per 256-row tile (0: heuristic)
    split_k: int = 0  # parallel K splits (0: heuristic)

    def force_kernel(self) -> int:
        return {0: 0, 1: 3, 2: 4}[self.cta_group]


def hardware_name(device: torch.device | int | None = None) -> str:
    """The key tables are stored under: device name, compute capability, SM count."""
    if not torch.cuda.is_available():
        return "no-cuda-device"
    props = torch.cuda.get_device_properties(device)
    return f"{props.name} sm_{props.major}{props.minor} {props.multi_processor_count}sm"


def problem_key(kind: str, dtype: torch.dtype, m: int, n: int, k: int, trans_a: bool = False, trans_b: bool = False,
                batch: int = 1, epilogue: str = "") -> str:
    layout = ("t" if trans_a else "n") + ("t" if trans_b else "n")
    return f"{kind}|{str(dtype).removeprefix('torch.')}|{layout}|{batch}x{m}x{n}x{k}|{epilogue}"


class TuneTable:
    """Choices for one hardware name, backed by a JSON file."""

    def __init__(self, hardware: str, directory: str | os.PathLike[str] | None = None) -> None:
        self.hardware = hardware
        base = directory or os.environ.get(TUNE_DIR_ENV) or Path.home() / ".cache" / "helion_mlir_b200"
        digest = hashlib.sha256(hardware.encode()).hexdigest()[:16]
        self.path = Path(base) / f"tune-{digest}.json"
        self._lock = threading.Lock()
        self._entries: dict[str, dict[str, object]] = {}
        self._loaded = False

    def _load(self) -> None:
        if self._loaded:
            return
        self._loaded = True
        try:
            data = json.loads(self.path.read_text())
        except (OSError, ValueError):
            return
        # A table written for other hardware or by another format is not ours to read.
        if not isinstance(data, dict) or data.get("format") != _FORMAT or data.get("hardware") != self.hardware:
            return
        entries = data.get("entries")
        if isinstance(entries, dict):
            self._entries = {str(k): v for k, v in entries.items() if isinstance(v, dict)}

    def get(self, key: str) -> Choice | None:
        with self._lock:
            self._load()
            entry = self._entries.get(key)
        if entry is None:
            return None
        try:
            choice = Choice(int(entry.get("tile_n", 0)), int(entry.get("cta_group", 0)), int(entry.get("split_k", 0)))
        except (TypeError, ValueError):
            return None
        if choice.tile_n < 0 or choice.tile_n > 256 or choice.cta_group not in (0, 1, 2) or not 0 <= choice.split_k <= 1024:
            return None
        return choice

    def put(self, key: str, choice: Choice, microseconds: float | None = None, persist: bool = True) -> None:
        with self._lock:
            self._load()
            entry: dict[str, object] = asdict(choice)
            if microseconds is not None:
                entry["us"] = round(float(microseconds), 3)
            self._entries[key] = entry
            if persist:
                self._save()

    def _save(self) -> None:
        payload = {"format": _FORMAT, "hardware": self.hardware, "entries": self._entries}
        try:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            handle, temp = tempfile.mkstemp(dir=self.path.parent, prefix=self.path.name, suffix=".tmp")
            with os.fdopen(handle, "w") as out:
                json.dump(payload, out, indent=1, sort_keys=True)
            os.replace(temp, self.path)  # readers see the old or the new table, never half of one
        except OSError:
            pass  # a read-only cache directory costs the persistence, not the call

    def __len__(self) -> int:
        with self._lock:
            self._load()
            return len(self._entries)

    def clear(self, persist: bool = True) -> None:
        with self._lock:
            self._entries = {}
            self._loaded = True
            if persist:
                self._save()


_TABLES: dict[tuple[str, str], TuneTable] = {}
_TABLES_LOCK = threading.Lock()


def table(device: torch.device | int | None = None) -> TuneTable:
    """The table of ``device``'s hardware (one object per hardware name and directory)."""
    name = hardware_name(device)
    directory = os.environ.get(TUNE_DIR_ENV, "")
    with _TABLES_LOCK:
        found = _TABLES.get((name, directory))
        if found is None:
            found = _TABLES[(name, directory)] = TuneTable(name, directory or None)
        return found


def lookup(key: str, device: torch.device | int | None = None) -> Choice | None:
    """The recorded choice for ``key`` on ``device``'s hardware (``None``: use the heuristics)."""
    if os.environ.get(TUNE_DISABLE_ENV, "") not in ("", "0"):
        return None
    return table(device).get(key)


def candidates(m: int, n: int, k: int, with_splits: bool = False) -> list[Choice]:
    """The choices worth timing for an ``m x n x k`` bf16 GEMM."""
    widths = [w for w in (64, 128, 192, 256) if w <= max(64, (n + 63) // 64 * 64)]
    out = [Choice()]
    for width in widths:
        out.append(Choice(width, 1, 0))
        if width % 128 == 0 and m > 128:
            out.append(Choice(width, 2, 0))
    if with_splits:
        for splits in (2, 4, 8, 16):
            if k % (splits * 64) == 0 and k // splits >= 512:
                out.append(Choice(0, 0, splits))
    return out


def time_call(call: Callable[[], object], iterations: int = 20, warmup: int = 3) -> float:
    """Microseconds per call of ``call`` on the current stream (CUDA events, after a warm-up)."""
    for _ in range(warmup):
        call()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        call()
    stop.record()
    stop.synchronize()
    return start.elapsed_time(stop) * 1e3 / iterations


def tune_matmul(
    a: Tensor,
    b: Tensor,
    trans_a: bool = False,
    trans_b: bool = False,
    bias: Tensor | None = None,
    epilogue: Callable[[Tensor], Tensor] | None = None,
    choices: Iterable[Choice] | None = None,
    with_splits: bool = False,
    iterations: int = 20,
    persist: bool = True,
) -> tuple[Choice, dict[Choice, float]]:
    """Times ``matmul(a, b, ...)`` under each candidate choice and records the fastest
    in the hardware's table, where later calls of the same problem find it. Returns
    the winner and every candidate's microseconds (refused candidates are left out)."""
    mm = importlib.import_module(__package__ + ".matmul")  # the package attribute of that name is the function

    epilogue = mm.identity_epilogue if epilogue is None else epilogue
    m = int(a.shape[1]) if trans_a else int(a.shape[0])
    k = int(a.shape[0]) if trans_a else int(a.shape[1])
    n = int(b.shape[0]) if trans_b else int(b.shape[1])
    tried = list(choices) if choices is not None else candidates(m, n, k, with_splits)
    timings: dict[Choice, float] = {}
    for choice in tried:
        def call(choice: Choice = choice) -> Tensor:
            return mm.matmul(a, b, trans_a=trans_a, trans_b=trans_b, bias=bias, epilogue=epilogue, _choice=choice)
        try:
            timings[choice] = time_call(call, iterations)
        except (mm.native.NativeCallError, ValueError):
            continue  # a choice the kernels refuse for this problem is no candidate
    if not timings:
        raise RuntimeError("no candidate ran for this problem")
    best = min(timings, key=timings.__getitem__)
    key = mm.tune_key(a.dtype, m, n, k, trans_a, trans_b, bias is not None, epilogue)
    table(a.device).put(key, best, timings[best], persist=persist)
    mm.forget_plans()
    return best, timings
