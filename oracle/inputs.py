"""Seeded synthetic inputs of the five benchmark configurations (test infrastructure).

Generated with a CPU ``torch.Generator`` in f32, then cast, so the CPU oracle and
the GPU kernels see identical bits. ``scale`` shrinks the large dimensions for
tests that the oracle must finish in seconds; ``scale=1`` is the full size.

"N(0,1/4096)" and "N(0,2)" are read as variances (sigma 1/64 and sqrt(2));
"N(0,0.02)", "N(1,0.1)", "N(0,0.1)" as standard deviations.
"""

from __future__ import annotations

import math

import torch

SEED_BASE = 1000


def _gen(config: int, extra: int = 0) -> torch.Generator:
    return torch.Generator().manual_seed(SEED_BASE + config + 7919 * extra)


def c1_f32_matmul(size: int = 1024) -> dict[str, torch.Tensor]:
    g = _gen(1)
    return {"a": torch.randn(size, size, generator=g), "b": torch.randn(size, size, generator=g)}


def c2_linear(m: int = 8192, n: int = 4096, k: int = 4096, rank: int = 0) -> dict[str, torch.Tensor]:
    g = _gen(2, rank)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / 64.0).bfloat16()
    b = (torch.randn(n, generator=g) * 0.02).bfloat16()
    return {"x": x, "w": w, "b": b}


def c3_blocked(size: int = 8192) -> dict[str, torch.Tensor]:
    g = _gen(3)
    return {"a": torch.randn(size, size, generator=g).bfloat16(), "b": torch.randn(size, size, generator=g).bfloat16()}


def c4_rows(m: int = 32768, n: int = 4096, dtype: torch.dtype = torch.float32, rank: int = 0) -> dict[str, torch.Tensor]:
    g = _gen(4, rank)
    x = torch.randn(m, n, generator=g) * math.sqrt(2.0)
    spike = torch.rand(m, n, generator=g) < 0.01
    sign = torch.where(torch.rand(m, n, generator=g) < 0.5, -30.0, 30.0)
    x = torch.where(spike, sign, x)
    gamma = 1.0 + 0.1 * torch.randn(n, generator=g)
    beta = 0.1 * torch.randn(n, generator=g)
    return {"x": x.to(dtype), "gamma": gamma.to(dtype), "beta": beta.to(dtype)}


def c5_split_k_bmm(batch: int = 64, m: int = 512, n: int = 512, k: int = 16384, rank: int = 0) -> dict[str, torch.Tensor]:
    g = _gen(5, rank)
    a = (torch.rand(batch, m, k, generator=g) * 2 - 1).bfloat16()
    b = (torch.rand(batch, k, n, generator=g) * 2 - 1).bfloat16()
    return {"a": a, "b": b}
