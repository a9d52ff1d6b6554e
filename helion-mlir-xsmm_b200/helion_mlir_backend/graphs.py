"""Replaying operator calls as CUDA graphs.

The reference removes per-call host work with ``prepared_call`` (a recorded native
plan replayed with new pointers, ``_compiler/native/call.cpp:501-557``). On a GPU
the analogue for launch-bound sequences is a CUDA graph: the kernels an operator
(or a chain of operators) enqueues are captured once and replayed with one launch.
Small problems are bound by the host here (a 1024^3 f32 matmul is three kernels
and about 35 microseconds of Python), which a replay takes out of the loop.

    call = graphed(lambda a, b: ops.matmul(a, b), a, b)
    c = call()                # replays on the tensors it captured
    c = call(a2, b2)          # or copies new operands into them first

Everything the kernels need at capture time (tensor maps, plans, scratch) is set
up by a warm-up call before the capture; outputs and scratch come from torch's
capture-aware allocator while capturing, not from the output pool.
"""

from __future__ import annotations

from collections.abc import Callable

import torch
from torch import Tensor


class GraphedCall:
    """``fn(*inputs)`` captured as one CUDA graph. The inputs are held: a replay reads
    whatever they contain at that time, and the result tensor is reused by every replay."""

    def __init__(self, fn: Callable[..., Tensor | tuple[Tensor, ...]], *inputs: Tensor, warmup: int = 2) -> None:
        if not inputs or not all(isinstance(t, Tensor) and t.is_cuda for t in inputs):
            raise ValueError("graphed() needs at least one input, all CUDA tensors")
        device = inputs[0].device
        if any(t.device != device for t in inputs):
            raise ValueError("graphed() inputs must be on one device")
        self.inputs = inputs
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.device(device):
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):  # plans, tensor maps, kernel attributes: all set up eagerly
                    fn(*inputs)
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
            from . import native

            before = native.counters()["launches"]
            with torch.cuda.graph(self.graph):
                self.output = fn(*inputs)
            # kernels of this library in the graph (a replay launches them without passing the C ABI's counters)
            self.kernels = int(native.counters()["launches"] - before)

    def __call__(self, *inputs: Tensor) -> Tensor | tuple[Tensor, ...]:
        if inputs:
            if len(inputs) != len(self.inputs):
                raise TypeError(f"expected {len(self.inputs)} operands, got {len(inputs)}")
            for held, new in zip(self.inputs, inputs):
                if new is not held:
                    if new.shape != held.shape or new.dtype != held.dtype:
                        raise ValueError(f"operand {tuple(new.shape)} {new.dtype} does not match the captured "
                                         f"{tuple(held.shape)} {held.dtype}")
                    held.copy_(new)
        self.graph.replay()
        return self.output


def graphed(fn: Callable[..., Tensor | tuple[Tensor, ...]], *inputs: Tensor, warmup: int = 2) -> GraphedCall:
    """Capture ``fn(*inputs)`` once; see :class:`GraphedCall`."""
    return GraphedCall(fn, *inputs, warmup=warmup)
