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


class _DeviceBlock:
    """Device memory of the library exposed to torch (``__cuda_array_interface__``)."""

    def __init__(self, pointer: int, nbytes: int) -> None:
        self.pointer = pointer
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (pointer, False), "version": 2, "strides": None}


class FusedColumnShardedLinear:
    """The column-sharded linear with the all-gather fused into the GEMM
    (``b200_gemm_to_peers``): every rank computes its columns of ``y`` and its epilogue
    stores them into all ranks' copies of ``y`` over NVLink peer memory while the tensor
    cores work on the next tile; a flag word per rank pair says when a rank's columns have
    landed, and a bounded device-side wait on this rank's flags ends the call. No NCCL call
    and no gather buffer is on the path.

    One object serves one ``[m, n]`` output shape. Construction is collective (every rank
    of ``group`` allocates two copies of ``y`` plus the flag words and maps the other
    ranks' through CUDA IPC handles exchanged with ``all_gather_object``); so is every call.
    Results alternate between the two copies: the tensor a call returns is overwritten by
    the call after the next, and each rank must keep its calls and its uses of the results
    in stream order (that ordering is what keeps a fast rank from storing into a copy a
    slow rank still reads)."""

    WAIT_BUDGET_NS = 2_000_000_000

    def __init__(self, m: int, n: int, k: int, dtype: torch.dtype, device: torch.device,
                 group: dist.ProcessGroup | None = None) -> None:
        import ctypes

        from helion_mlir_backend import native

        if dtype != torch.bfloat16:
            raise ValueError("the fused column-sharded linear runs on the bf16 tensor-core kernel only")
        self.native, self.ctypes = native, ctypes
        self.m, self.n, self.k, self.dtype, self.device, self.group = m, n, k, dtype, device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > native.MAX_PEERS:
            raise ValueError(f"at most {native.MAX_PEERS} ranks")
        if n % self.world:
            raise ValueError(f"{n} columns do not divide over {self.world} ranks")
        self.n0, self.n1 = shard_bounds(n, self.world, self.rank)
        lib = native.module()
        self.y_bytes = m * n * dtype.itemsize
        # per buffer: the copy of y, then `world` flag words, the CTA counter (256-byte slots),
        # and this rank's store descriptors for the copies (128 bytes each)
        self.flag_offset = -(-self.y_bytes // 256) * 256
        self.block_bytes = self.flag_offset + 512 + 128 * native.MAX_PEERS
        self.local: list[int] = []
        handles: list[bytes] = []
        with native.on_device(device):
            for _ in range(2):
                pointer, handle = ctypes.c_void_p(), ctypes.create_string_buffer(native.IPC_HANDLE_BYTES)
                native.check("b200_symm_alloc", lib.b200_symm_alloc(self.block_bytes, ctypes.byref(pointer), handle))
                self.local.append(int(pointer.value))
                handles.append(handle.raw)
        everyone: list[list[bytes]] = [[] for _ in range(self.world)]
        dist.all_gather_object(everyone, handles, group=group)
        self.copies: list[list[int]] = []  # [buffer][rank] -> base address valid on this GPU
        self.opened: list[int] = []
        with native.on_device(device):
            for buffer in range(2):
                row = []
                for r in range(self.world):
                    if r == self.rank:
                        row.append(self.local[buffer])
                        continue
                    pointer = ctypes.c_void_p()
                    native.check("b200_symm_open", lib.b200_symm_open(everyone[r][buffer], ctypes.byref(pointer)))
                    row.append(int(pointer.value))
                    self.opened.append(int(pointer.value))
                self.copies.append(row)
        self.results = [
            torch.as_tensor(_DeviceBlock(self.local[b], self.y_bytes), device=device).view(dtype).view(m, n) for b in range(2)
        ]
        # Destinations in rotated order, this rank's own copy first: at any moment the ranks
        # store to different GPUs instead of all to the same one. Where this rank's columns
        # start in each copy, and the bulk-store descriptors for them, are fixed per buffer.
        item = dtype.itemsize
        self.order = [(self.rank + slot) % self.world for slot in range(self.world)]
        self.targets = [[self.copies[b][r] + self.n0 * item for r in self.order] for b in range(2)]
        self.store_maps = [self.local[b] + self.flag_offset + 512 for b in range(2)]
        with native.on_device(device):
            for b in range(2):
                bases = (ctypes.c_void_p * self.world)(*self.targets[b])
                native.check("b200_peer_store_maps", lib.b200_peer_store_maps(
                    self.store_maps[b], bases, self.world, m, self.n1 - self.n0, n))
        self.epoch = 0
        self._plans: dict[object, object] = {}
        dist.barrier(group=group)  # every rank has mapped every copy before any store

    def __call__(self, x: Tensor, weight_shard: Tensor, bias_shard: Tensor | None,
                 epilogue: Callable[[Tensor], Tensor] | None = None) -> Tensor:
        from . import epilogues
        from .matmul import _plan_gemm
        from .matmul import identity_epilogue

        native, ctypes = self.native, self.ctypes
        epilogue = identity_epilogue if epilogue is None else epilogue
        if epilogues.resolve(epilogue) is None:
            raise ValueError("the fused column-sharded linear needs an epilogue the kernel fuses")
        width = self.n1 - self.n0
        if tuple(x.shape) != (self.m, self.k) or tuple(weight_shard.shape) != (width, self.k) or x.dtype != self.dtype:
            raise ValueError(f"expected x [{self.m}, {self.k}] and a weight shard [{width}, {self.k}] of {self.dtype}")
        x, weight_shard = x.contiguous(), weight_shard.contiguous()
        bias = None if bias_shard is None else bias_shard.to(self.dtype).contiguous()
        key = (epilogue, bias is None)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = _plan_gemm(
                a=x, m=self.m, n=width, k=self.k, a_layout=native.LAYOUT_ROW, b_layout=native.LAYOUT_COL, lda=self.k,
                ldb=self.k, bias=bias, scale=None, shift=None, epilogue=epilogue, ldc=self.n, out_shape=(self.m, self.n),
            )
        self.epoch += 1
        buffer = self.epoch & 1
        item = self.dtype.itemsize
        desc = native.GemmDesc.from_buffer_copy(plan.desc)
        desc.a, desc.b, desc.bias = x.data_ptr(), weight_shard.data_ptr(), native.ptr(bias)
        desc.c = self.targets[buffer][0]
        out = native.PeerOut()
        out.count, out.rank, out.epoch = self.world, 0, self.epoch
        for slot, r in enumerate(self.order):
            out.c[slot] = self.targets[buffer][slot]
            out.flags[slot] = self.copies[buffer][r] + self.flag_offset + 4 * self.rank  # my word on rank r
        out.store_maps = self.store_maps[buffer]
        out.done_counter = self.local[buffer] + self.flag_offset + 256
        lib = native.module()
        stream = native.stream_ptr(self.device)
        with native.on_device(self.device):
            native.check("b200_gemm_to_peers", lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream))
            native.check("b200_peer_wait", lib.b200_peer_wait(self.local[buffer] + self.flag_offset, self.world,
                                                              self.epoch, self.WAIT_BUDGET_NS, stream))
        return self.results[buffer]

    def close(self) -> None:
        """Collective: waits for this rank's work, then unmaps the peers' copies and frees its own."""
        lib = self.native.module()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody stores into a copy that is about to go
        with self.native.on_device(self.device):
            for pointer in self.opened:
                lib.b200_symm_close(pointer)
            self.results = []
            for pointer in self.local:
                lib.b200_symm_free(pointer)
        self.opened, self.local = [], []
