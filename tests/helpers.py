"""Shared helpers of the tests: golden fixtures and device transfers."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name: str) -> dict[str, torch.Tensor]:
    """A fixture written by tests/golden/make_golden.py as ``{name: tensor}`` (bf16 restored)."""
    out: dict[str, torch.Tensor] = {}
    with np.load(GOLDEN / f"{name}.npz") as data:
        for key in data.files:
            if key.endswith("__dtype"):
                continue
            array = data[key]
            dtype = str(data[f"{key}__dtype"])
            tensor = torch.from_numpy(array.copy())
            if dtype == "bfloat16":
                tensor = tensor.view(torch.bfloat16)
            out[key] = tensor
    return out


def cuda(*tensors: torch.Tensor | None):
    moved = tuple(None if t is None else t.cuda() for t in tensors)
    return moved[0] if len(moved) == 1 else moved


def bits(t: torch.Tensor) -> torch.Tensor:
    """Comparable bit pattern: NaNs compare equal."""
    return t.detach().cpu().to(torch.float64).nan_to_num(7.0, 1e300, -1e300)
