"""The multi-rank host logic on CPU: two gloo ranks shard rows with no exchange,
and the one optional exchange (column-sharded linear + all-gather) reassembles
the full result. The operators themselves are injected as CPU stand-ins here;
on GPUs the same code runs the CUDA operators over NCCL."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helion_mlir_utils import sharding


def test_shard_bounds_partition_every_unit_once() -> None:
    for total in (0, 1, 7, 64, 8192, 8205):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)
        x = torch.randn(37, 24, generator=gen)
        w = torch.randn(10, 24, generator=gen)
        b = torch.randn(10, generator=gen)
        # rows: each rank computes its own rows, nothing is exchanged
        mine = sharding.row_sharded(lambda t: torch.softmax(t, -1), x, world=world, rank=rank)
        start, stop = sharding.shard_bounds(37, world, rank)
        ok_rows = torch.equal(mine, torch.softmax(x[start:stop], -1))
        # the shards put back together are the unsharded result (ragged: 19 + 18 rows)
        whole = sharding.gather_rows(mine, 37)
        ok_gather = torch.equal(whole, torch.softmax(x, -1))
        # column-sharded linear: W split along N, all-gather of the column shards
        n0, n1 = sharding.shard_bounds(10, world, rank)
        y = sharding.column_sharded_linear(
            x, w[n0:n1], b[n0:n1], 10, op=lambda a, ws, bs: torch.relu(a @ ws.T + bs)
        )
        ok_cols = torch.allclose(y, torch.relu(x @ w.T + b), atol=1e-6)
        results.put((rank, ok_rows, ok_gather, ok_cols))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks() -> None:
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    procs = [context.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    seen = sorted(results.get(timeout=10) for _ in range(2))
    assert seen == [(0, True, True, True), (1, True, True, True)]
