"""Operator calls captured as CUDA graphs: same bits as the eager call, replays read the
held operands, new operands are copied in, and capture bypasses the output pool."""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_graphed_calls_replay(built_library) -> None:
    import helion_mlir_utils as ops
    from helion_mlir_backend import graphed

    gen = torch.Generator().manual_seed(17)
    a = torch.randn(512, 384, generator=gen).cuda()
    b = torch.randn(384, 256, generator=gen).cuda()
    call = graphed(lambda x, y: ops.matmul(x, y), a, b)  # f32: two operand splits and the GEMM
    assert torch.equal(call(), ops.matmul(a, b))
    a.mul_(2.0)  # a replay reads what the held operands contain now
    assert torch.equal(call(), ops.matmul(a, b))
    a2, b2 = torch.randn(512, 384, generator=gen).cuda(), torch.randn(384, 256, generator=gen).cuda()
    assert torch.equal(call(a2, b2), ops.matmul(a2, b2))
    with pytest.raises(ValueError, match="does not match"):
        call(a2[:100], b2)

    # a chain of operators, pool-sized intermediates (1024 x 4096 bf16 = 8 MiB)
    x = torch.randn(1024, 1024, generator=gen).bfloat16().cuda()
    w = (torch.randn(4096, 1024, generator=gen) / 32).bfloat16().cuda()
    bias = torch.randn(4096, generator=gen).bfloat16().cuda()

    def chain(x: torch.Tensor) -> torch.Tensor:
        h = ops.matmul(x, w, trans_b=True, bias=bias, epilogue=F.gelu)
        return ops.softmax(ops.layer_norm(h.float(), None, None))

    eager = chain(x)
    graph = graphed(chain, x)
    assert torch.equal(graph(), eager)
    assert torch.equal(graph(), eager)  # replays reuse the captured output
