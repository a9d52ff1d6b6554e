"""The fused column-sharded linear on one GPU: a group of one rank runs the same kernel
(results through the swizzled staging tile and bulk tensor stores into "every" copy of y,
the last CTA raising the flag, the bounded wait) with this GPU's copy as the only
destination. Two and more ranks are covered by tests/test_gpu_multi.py."""

from __future__ import annotations

import socket

import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F

from helpers import cuda
from oracle import checks, inputs
from oracle import ops as ref

pytestmark = pytest.mark.gpu


@pytest.fixture()
def one_rank_group():
    if dist.is_initialized():
        pytest.skip("a process group is already initialised in this process")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        yield
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(1024, 768, 512), (1000, 320, 200), (256, 64, 64)])
def test_fused_linear_with_one_destination_matches_matmul(one_rank_group, shape) -> None:
    import helion_mlir_utils as ops
    from helion_mlir_backend import native
    from helion_mlir_utils import sharding

    m, n, k = shape
    data = inputs.c2_linear(m=m, n=n, k=k)
    x, w, b = cuda(data["x"], data["w"], data["b"])
    whole = ops.matmul(x, w, trans_b=True, bias=b, epilogue=F.gelu)
    fused = sharding.FusedColumnShardedLinear(m, n, k, torch.bfloat16, torch.device("cuda", 0))
    try:
        for call in range(4):  # the two copies of y alternate
            y = fused(x, w, b, F.gelu)
            torch.cuda.synchronize()
            assert torch.equal(y, whole), f"call {call}"
        assert native.kernel_status() == 0
        checks.assert_parity(torch.bfloat16, y.cpu(), ref.linear(data["x"], data["w"], data["b"], F.gelu), "fused, one rank")
        plain = fused(x, w, None, None)
        torch.cuda.synchronize()
        assert torch.equal(plain, ops.matmul(x, w, trans_b=True))
        with pytest.raises(ValueError, match="expected x"):
            fused(x[:, : k // 2].contiguous(), w, b, F.gelu)
    finally:
        fused.close()


def test_peer_gemm_refuses_what_it_cannot_run(one_rank_group) -> None:
    import ctypes

    from helion_mlir_backend import native

    lib = native.module()
    a = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    c = torch.zeros(128, 128, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(64, device="cuda", dtype=torch.int32)
    desc = native.GemmDesc()
    desc.dtype = desc.out_dtype = desc.vec_dtype = native.BF16
    desc.a_layout, desc.b_layout = native.LAYOUT_ROW, native.LAYOUT_COL
    desc.m, desc.n, desc.k, desc.batch = 128, 128, 64, 1
    desc.lda = desc.ldb = 64
    desc.ldc = 128
    desc.a, desc.b, desc.c = a.data_ptr(), a.data_ptr(), c.data_ptr()
    out = native.PeerOut()
    out.count, out.rank, out.epoch = 1, 0, 1
    out.c[0], out.flags[0], out.done_counter = c.data_ptr(), flags.data_ptr(), flags.data_ptr() + 128
    stream = native.stream_ptr(a.device)
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), None, stream) == 6
    out.count = 9
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream) == 7
    out.count = 1
    out.c[0] = c.data_ptr() + 256  # this rank's own copy must be desc->c
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream) == 7
    out.c[0] = c.data_ptr()
    desc.split_k = 2
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream) == 7
    desc.split_k = 0
    desc.dtype = native.F32  # tensor-core path only
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream) != 0
    desc.dtype = native.BF16
    assert lib.b200_gemm_to_peers(ctypes.byref(desc), ctypes.byref(out), stream) == 0  # plain stores (no descriptors)
    assert lib.b200_peer_wait(flags.data_ptr(), 1, 1, 1_000_000_000, stream) == 0
    torch.cuda.synchronize()
    assert native.kernel_status() == 0 and int(flags[0]) == 1 and int(flags[32]) == 0  # flag raised, counter reset
