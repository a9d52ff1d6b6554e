"""Sharding the operator set over the GPUs of one box.

Every operator works on independent units (rows of ``x``, batches, output rows),
so the multi-GPU form is one process per GPU, each running the same operators on
its shard, with **no collective on the data path**. The reference has no
multi-device code at all (its only parallelism is OpenMP threads in one process),
so nothing here has a counterpart there.

The one exchange this module offers is for a linear layer whose *weight* is split
along ``N`` (column sharding): each rank computes ``y[:, shard]`` and the shards
are all-gathered (NCCL over NVLink on GPUs; any ``torch.distributed`` backend
works, which is how the CPU tests exercise it with gloo). Row sharding is the
default and needs no exchange.
"""

from __future__ import annotations

from typing import Callable

import torch
from torch import Tensor
import torch.distributed as dist


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """``[start, stop)`` of ``rank``'s share of ``total`` units: shares differ by at
    most one unit, the larger ones on the lower ranks, and together cover every unit once."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: Tensor, world: int, rank: int, dim: int = 0) -> Tensor:
    """``rank``'s rows (a view)."""
    start, stop = shard_bounds(x.shape[dim], world, rank)
    return x.narrow(dim, start, stop - start)


def gather_rows(local: Tensor, total: int, group: dist.ProcessGroup | None = None, dim: int = 0) -> Tensor:
    """All ranks' shards along ``dim`` put back together (shares as :func:`shard_bounds` gives them)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    sizes = [b - a for a, b in (shard_bounds(total, world, r) for r in range(world))]
    if local.shape[dim] != sizes[rank]:
        raise ValueError(f"rank {rank} holds {local.shape[dim]} units, expected {sizes[rank]}")
    widest = max(sizes)
    moved = local.movedim(dim, 0).contiguous()
    padded = moved
    if sizes[rank] < widest:  # all_gather wants equal shapes
        pad = torch.zeros((widest - sizes[rank], *moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        padded = torch.cat([moved, pad])
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    whole = torch.cat([part[:size] for part, size in zip(parts, sizes)])
    return whole.movedim(0, dim)


def row_sharded(op: Callable[..., Tensor], x: Tensor, *args: object, world: int, rank: int, **kwargs: object) -> Tensor:
    """``op`` on this rank's rows of ``x`` (no communication): the default form."""
    return op(shard_rows(x, world, rank).contiguous(), *args, **kwargs)


def column_sharded_linear(
    x: Tensor,
    weight_shard: Tensor,
    bias_shard: Tensor | None,
    out_features: int,
    epilogue: Callable[[Tensor], Tensor] | None = None,
    group: dist.ProcessGroup | None = None,
    op: Callable[..., Tensor] | None = None,
) -> Tensor:
    """``epilogue(x @ W^T + b)`` with ``W`` ``[N, K]`` split along ``N``: this rank
    holds ``weight_shard`` (its rows of ``W``) and computes its columns of ``y``;
    the column shards are all-gathered into ``[M, N]`` on every rank. ``op`` is the
    matmul to run (default: :func:`helion_mlir_utils.matmul`)."""
    if op is None:
        from .matmul import identity_epilogue
        from .matmul import matmul

        def op(a: Tensor, w: Tensor, bias: Tensor | None) -> Tensor:
            return matmul(a, w, trans_b=True, bias=bias, epilogue=epilogue or identity_epilogue)

    local = op(x, weight_shard, bias_shard)
    return gather_columns(local, out_features, group=group)


def gather_columns(local: Tensor, total: int, group: dist.ProcessGroup | None = None) -> Tensor:
    """The ranks' column shards ``[M, N_r]`` put together as ``[M, N]`` on every rank. Equal
    shards on CUDA devices take one NCCL all-gather into ``[G, M, N/G]`` and one strided copy;
    anything else goes through :func:`gather_rows`."""
    world = dist.get_world_size(group)
    if local.is_cuda and local.dim() == 2 and total % world == 0 and local.shape[1] == total // world:
        local = local.contiguous()
        stacked = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(stacked, local, group=group)
        return stacked.permute(1, 0, 2).reshape(local.shape[0], total)
    return gather_rows(local, total, group=group, dim=1)
