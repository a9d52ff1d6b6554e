"""The GEMM kernels against the CPU oracle on seeded inputs: the tcgen05 path in
every operand orientation, ragged edges, K tails, fused epilogues, batches, both
forms of split-K, and the five benchmark configurations at reduced size."""

from __future__ import annotations

import ctypes

import pytest
import torch
import torch.nn.functional as F

from helpers import cuda
from oracle import checks
from oracle import inputs
from oracle import ops as ref

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def ops():
    import helion_mlir_utils

    return helion_mlir_utils


@pytest.fixture(autouse=True)
def no_kernel_gave_up():
    """Every bounded wait in the kernels must have been satisfied."""
    yield
    from helion_mlir_backend import native

    torch.cuda.synchronize()
    assert native.kernel_status() == 0


def rand(gen: torch.Generator, *shape: int, dtype=BF16, scale: float = 1.0) -> torch.Tensor:
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def explain(ops, a, b, **kw) -> str:
    return str(ops.matmul.explain(a, b, **kw))


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 192), (200, 328, 136), (1000, 72, 520), (8, 16, 32)])
def test_tensor_core_orientations(ops, shape, trans_a: bool, trans_b: bool) -> None:
    m, n, k = shape
    gen = torch.Generator().manual_seed(m * 31 + n * 7 + k + 2 * trans_a + trans_b)
    a, b = rand(gen, m, k), rand(gen, k, n)
    a_in = a.T.contiguous() if trans_a else a
    b_in = b.T.contiguous() if trans_b else b
    da, db = cuda(a_in, b_in)
    assert "umma_bf16" in explain(ops, da, db, trans_a=trans_a, trans_b=trans_b)
    out = ops.matmul(da, db, trans_a=trans_a, trans_b=trans_b)
    checks.assert_parity(BF16, out.cpu(), ref.matmul(a, b), f"{shape} ta={trans_a} tb={trans_b}")
    assert torch.equal(out, ops.matmul(da, db, trans_a=trans_a, trans_b=trans_b))  # run twice: same bits


def test_tensor_core_matches_ffma_path(ops) -> None:
    """Same operands through both kernels: f32 accumulation either way, one rounding."""
    from helion_mlir_backend import native
    from helion_mlir_utils import matmul as _  # noqa: F401
    import importlib

    mm = importlib.import_module("helion_mlir_utils.matmul")
    gen = torch.Generator().manual_seed(5)
    a, b = cuda(rand(gen, 384, 320), rand(gen, 320, 256))
    fast = ops.matmul(a, b, out_dtype=F32)
    plan = mm._plan_gemm(a=a, m=384, n=256, k=320, a_layout=native.LAYOUT_ROW, b_layout=native.LAYOUT_ROW, lda=320,
                         ldb=256, bias=None, scale=None, shift=None, epilogue=ops.identity_epilogue, out_dtype=F32,
                         force_kernel=2)
    slow = plan.run(a, b)
    assert "simt_ffma" in str(plan.explain(a, b))
    assert checks.rel_frobenius(fast, slow) < 2e-6


@pytest.mark.parametrize("act", ["relu", "gelu", "gelu_tanh", "sigmoid", "tanh", "silu", "leaky", "unfused"])
def test_fused_epilogues(ops, act: str) -> None:
    gen = torch.Generator().manual_seed(11)
    m, n, k = 300, 264, 128
    x, w = rand(gen, m, k), rand(gen, n, k, scale=0.125)
    bias, scale, shift = rand(gen, n, scale=0.5), (1 + 0.1 * torch.randn(n, generator=gen)).to(BF16), rand(gen, 1, scale=0.1)
    fn = {
        "relu": torch.relu, "gelu": F.gelu, "gelu_tanh": ops.gelu_tanh, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
        "silu": F.silu, "leaky": ops.leaky_relu_epilogue(0.2), "unfused": lambda t: t * torch.sigmoid(1.5 * t),
    }[act]
    out = ops.matmul(*cuda(x, w), trans_b=True, bias=cuda(bias), scale=cuda(scale), shift=cuda(shift), epilogue=fn)
    expect = ref.matmul(x, w, trans_b=True, bias=bias, scale=scale, shift=shift, epilogue=fn)
    checks.assert_parity(BF16, out.cpu(), expect, act)
    assert out.dtype == BF16


def test_output_type_and_f32_vectors(ops) -> None:
    gen = torch.Generator().manual_seed(12)
    x, w = rand(gen, 130, 64), rand(gen, 96, 64)
    bias = torch.randn(96, generator=gen)  # f32 bias with bf16 operands
    out = ops.matmul(*cuda(x, w), trans_b=True, bias=cuda(bias), out_dtype=F32)
    assert out.dtype == F32
    assert checks.rel_frobenius(out.cpu(), ref.matmul(x, w, trans_b=True, bias=bias, out_dtype=F32)) < 1e-5


def test_bmm_tail_batches_run_with_half_width_tiles(ops) -> None:
    """More 256x256 tiles than CTA pairs, with a last round less than half full: the batches of
    that round go to a second launch with 128-column tiles. Same results as the oracle, and the
    same bits as each batch computed on its own (no K split: the tile width does not change a sum)."""
    pairs = torch.cuda.get_device_properties(0).multi_processor_count // 2
    batch = pairs + 6
    gen = torch.Generator().manual_seed(29)
    a, b = rand(gen, batch, 256, 192), rand(gen, batch, 192, 256)
    da, db = cuda(a, b)
    text = str(ops.bmm.explain(da, db)) if hasattr(ops.bmm, "explain") else ""
    out = ops.bmm(da, db)
    checks.assert_parity(BF16, out.cpu(), ref.bmm(a, b), "bmm with peeled tail")
    assert torch.equal(out[-1], ops.matmul(da[-1], db[-1]))
    assert torch.equal(out[0], ops.matmul(da[0], db[0]))
    if text:
        assert "tail_batches=6" in text
    split = ops.bmm(da, db, split_k=3, out_dtype=F32)
    assert checks.rel_frobenius(split.cpu(), ref.bmm(a, b, split_k=3, out_dtype=F32)) < 1e-5


def test_bmm_and_split_k(ops) -> None:
    gen = torch.Generator().manual_seed(13)
    a, b = rand(gen, 6, 256, 512), rand(gen, 6, 512, 128)
    da, db = cuda(a, b)
    checks.assert_parity(BF16, ops.bmm(da, db).cpu(), ref.bmm(a, b), "bmm")
    serial = ops.bmm(da, db, split_k=4, out_dtype=F32)
    assert serial.dtype == F32
    assert checks.rel_frobenius(serial.cpu(), ref.bmm(a, b, split_k=4, out_dtype=F32)) < 1e-5
    assert torch.equal(serial, ops.bmm(da, db, split_k=4, out_dtype=F32))  # ordered: same bits every run
    rounded = ops.bmm(da, db, split_k=4)  # bf16 result of the same on-chip ordered sum
    checks.assert_parity(BF16, rounded.cpu(), ref.bmm(a, b, split_k=4), "bmm split bf16")
    assert torch.equal(rounded, serial.to(BF16))
    # parallel split-K chosen automatically: few tiles, deep K
    a2, b2 = rand(gen, 128, 8192), rand(gen, 8192, 128)
    text = explain(ops, *cuda(a2, b2))
    out = ops.matmul(*cuda(a2, b2))
    checks.assert_parity(BF16, out.cpu(), ref.matmul(a2, b2), "auto split " + text)
    with pytest.raises(RuntimeError, match="batch2"):
        ops.bmm(da, db.transpose(1, 2).contiguous())


def test_f32_paths(ops) -> None:
    gen = torch.Generator().manual_seed(14)
    for m, n, k in [(1024 // 4, 1024 // 4, 1024 // 4), (70, 45, 50), (1, 1, 1), (33, 129, 7)]:
        a, b = rand(gen, m, k, dtype=F32), rand(gen, k, n, dtype=F32)
        out = ops.matmul(*cuda(a, b), block_sizes=(64, 64, 64))
        assert checks.rel_frobenius(out.cpu(), ref.matmul(a, b)) < 1e-5
    a, b = rand(gen, 3, 40, 24, dtype=F32), rand(gen, 3, 24, 56, dtype=F32)
    assert checks.rel_frobenius(ops.bmm(*cuda(a, b)).cpu(), ref.bmm(a, b)) < 1e-5
    empty = ops.matmul(torch.zeros(0, 8, device="cuda"), torch.zeros(8, 4, device="cuda"))
    assert empty.shape == (0, 4)
    zero_k = ops.matmul(torch.zeros(5, 0, device="cuda"), torch.zeros(0, 4, device="cuda"))
    assert torch.equal(zero_k.cpu(), torch.zeros(5, 4))


def test_blocked_operands(ops) -> None:
    gen = torch.Generator().manual_seed(15)
    m, n, k = 100, 90, 70
    a, b = rand(gen, m, k), rand(gen, k, n)
    bias = rand(gen, n)
    a4, b4, b5 = ref.pack_a_blocked(a), ref.pack_b_blocked(b), ref.pack_b_blocked_vnni(b)
    expect = ref.matmul(a, b, bias=bias, epilogue=torch.relu, out_dtype=F32)
    for packed in (b4, b5):
        out = ops.matmul_blocked(*cuda(a4, packed), m, n, k, bias=cuda(bias), epilogue=torch.relu, out_dtype=F32)
        assert out.shape == (m, n) and out.dtype == F32
        assert checks.rel_frobenius(out.cpu(), expect) < 1e-5
    out = ops.matmul_blocked(*cuda(a4, b4), m, n, k)
    checks.assert_parity(BF16, out.cpu(), ref.matmul_blocked(a4, b4, m, n), "blocked bf16")


def test_benchmark_configurations_reduced(ops) -> None:
    """C1..C5 of the baseline at sizes the oracle finishes in seconds."""
    c1 = inputs.c1_f32_matmul(256)
    out = ops.matmul(*cuda(c1["a"], c1["b"]), block_sizes=[64, 64, 64])
    assert checks.rel_frobenius(out.cpu(), ref.matmul(c1["a"], c1["b"])) < 1e-5
    c2 = inputs.c2_linear(m=1024, n=512, k=4096)
    out = ops.matmul(*cuda(c2["x"], c2["w"]), trans_b=True, bias=cuda(c2["b"]), epilogue=F.gelu)
    checks.assert_parity(BF16, out.cpu(), ref.linear(c2["x"], c2["w"], c2["b"], F.gelu), "C2")
    c3 = inputs.c3_blocked(512)
    a4, b5 = ref.pack_a_blocked(c3["a"]), ref.pack_b_blocked_vnni(c3["b"])
    out = ops.matmul_blocked(*cuda(a4, b5), 512, 512, 512, out_dtype=F32)
    assert checks.rel_frobenius(out.cpu(), ref.matmul(c3["a"], c3["b"], out_dtype=F32)) < 1e-5
    c5 = inputs.c5_split_k_bmm(batch=4, m=256, n=256, k=4096)
    out = ops.bmm(*cuda(c5["a"], c5["b"]), split_k=8, out_dtype=F32)
    assert checks.rel_frobenius(out.cpu(), ref.bmm(c5["a"], c5["b"], split_k=8, out_dtype=F32)) < 1e-5


def test_full_size_properties(ops) -> None:
    """Size-independent checks at the benchmark's full C2 size: linearity in x and
    agreement of sampled rows with the oracle."""
    c2 = inputs.c2_linear()
    x, w, b = cuda(c2["x"], c2["w"], c2["b"])
    y = ops.matmul(x, w, trans_b=True, bias=b, epilogue=F.gelu)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191])
    expect = ref.linear(c2["x"][rows], c2["w"], c2["b"], F.gelu)
    checks.assert_parity(BF16, y.cpu()[rows], expect, "C2 sampled rows")
    plain = ops.matmul(x, w, trans_b=True, out_dtype=F32)
    doubled = ops.matmul(x * 2, w, trans_b=True, out_dtype=F32)
    assert torch.equal(doubled, plain * 2)  # scaling by 2 is exact in bf16 and f32


def test_c_abi_refuses_what_it_cannot_run(ops) -> None:
    from helion_mlir_backend import native

    lib = native.module()
    a = torch.zeros(64, 64, device="cuda", dtype=BF16)
    desc = native.GemmDesc()
    desc.dtype = desc.out_dtype = desc.vec_dtype = native.BF16
    desc.m = desc.n = desc.k = 64
    desc.batch = 1
    desc.lda = desc.ldb = desc.ldc = 64
    desc.a = desc.b = a.data_ptr()
    desc.c = a.data_ptr()  # output aliases an input
    assert lib.b200_gemm(ctypes.byref(desc), native.stream_ptr(a.device)) == 5
    desc.c = torch.zeros(64, 64, device="cuda", dtype=BF16).data_ptr()
    desc.ldc = 32
    assert lib.b200_gemm(ctypes.byref(desc), native.stream_ptr(a.device)) == 3


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
@pytest.mark.parametrize("shape", [(256, 256, 64), (640, 384, 320), (304, 264, 136), (1024, 512, 1024)])
def test_single_cta_and_cta_pair_tiles_agree(ops, shape, trans_a: bool, trans_b: bool, cta_group: int) -> None:
    """Both tilings of the tcgen05 kernel (one CTA per 128-row tile, a CTA pair per
    256-row tile) against the oracle, with a fused epilogue and ragged edges."""
    import importlib

    from helion_mlir_backend import native

    mm = importlib.import_module("helion_mlir_utils.matmul")
    m, n, k = shape
    gen = torch.Generator().manual_seed(m + 3 * n + 5 * k + trans_a + 2 * trans_b)
    a, b, bias = rand(gen, m, k), rand(gen, k, n, scale=0.25), rand(gen, n)
    a_in = a.T.contiguous() if trans_a else a
    b_in = b.T.contiguous() if trans_b else b
    da, db, dbias = cuda(a_in, b_in, bias)
    plan = mm._plan_gemm(
        a=da, m=m, n=n, k=k, a_layout=native.LAYOUT_COL if trans_a else native.LAYOUT_ROW,
        b_layout=native.LAYOUT_COL if trans_b else native.LAYOUT_ROW, lda=da.shape[1], ldb=db.shape[1],
        bias=dbias, scale=None, shift=None, epilogue=torch.relu, force_kernel=2 + cta_group, tiles=(128, 128, 64),
    )
    text = str(plan.explain(da, db))
    assert f"cta_group={cta_group}" in text, text
    out = plan.run(da, db, dbias)
    checks.assert_parity(BF16, out.cpu(), ref.matmul(a, b, bias=bias, epilogue=torch.relu), text)
    assert torch.equal(out, plan.run(da, db, dbias))


def test_bounded_wait_gives_up_and_reports() -> None:
    """Failure detection without a fault: a wait that nothing satisfies runs out after
    its budget, leaves a code in the device status word, and the context stays usable."""
    import time

    from helion_mlir_backend import native

    lib = native.module()
    torch.cuda.synchronize()
    assert native.kernel_status() == 0
    stream = native.stream_ptr(torch.device("cuda", 0))
    t0 = time.perf_counter()
    assert lib.b200_selftest_wait_timeout(2_000_000, stream) == 0  # 2 ms
    status = native.kernel_status()  # synchronises
    elapsed = time.perf_counter() - t0
    assert status == 16 and elapsed < 1.0
    assert native.kernel_status() == 0  # reading clears the word
    assert lib.b200_selftest_wait_timeout(0, stream) == 7
    x = torch.randn(64, 64, device="cuda")
    assert torch.allclose(torch.softmax(x, -1), __import__("helion_mlir_utils").softmax(x), atol=1e-6)


def test_seeded_shape_sweep(ops) -> None:
    """Forty seeded shapes (multiples of 8, so that the tensor-core path applies) in
    random orientations, with and without a fused epilogue, against the oracle."""
    import random

    rng = random.Random(2024)
    gen = torch.Generator().manual_seed(2024)
    for case in range(40):
        m, n, k = (8 * rng.randint(1, 90) for _ in range(3))
        trans_a, trans_b = rng.random() < 0.5, rng.random() < 0.5
        a, b = rand(gen, m, k), rand(gen, k, n, scale=0.5)
        bias = rand(gen, n) if rng.random() < 0.5 else None
        fn = rng.choice([ops.identity_epilogue, torch.relu, F.gelu])
        a_in = a.T.contiguous() if trans_a else a
        b_in = b.T.contiguous() if trans_b else b
        da, db = cuda(a_in, b_in)
        out = ops.matmul(da, db, trans_a=trans_a, trans_b=trans_b, bias=None if bias is None else cuda(bias), epilogue=fn)
        expect = ref.matmul(a, b, bias=bias, epilogue=fn)
        checks.assert_parity(BF16, out.cpu(), expect, f"case {case}: {(m, n, k)} ta={trans_a} tb={trans_b} {fn.__name__}")


def _explains_tensor_cores(text: str) -> bool:
    return "f32 as 6 bf16 cross products" in text and "umma_bf16" in text


def test_f32_contractions_on_tensor_cores(ops) -> None:
    """f32 GEMMs beyond the plain 2-D case run as the widened bf16 product: batched,
    K above 4096 (more ordered chunks), 32x32-blocked operands and the prepacked-rows
    layout. Relative Frobenius error against the f64 oracle <= 1e-5 (the bar of
    tests/test_cpu_utils_f32_fused.py:58-140 is 1e-6 in max-norm for the exact kernel;
    BASELINE's bar for f32 paths is 1e-5 Frobenius)."""
    gen = torch.Generator().manual_seed(77)
    # batched (bmm, _bmm_direct of the reference: matmul.py:1842-1855)
    a, b = rand(gen, 8, 512, 1024, dtype=F32), rand(gen, 8, 1024, 384, dtype=F32)
    da, db = cuda(a, b)
    assert _explains_tensor_cores(str(ops.bmm.explain(da, db)))
    assert checks.rel_frobenius(ops.bmm(da, db).cpu(), ref.bmm(a, b)) <= 1e-5
    # K above 4096: twelve serial chunks per tile
    a, b = rand(gen, 1024, 8192, dtype=F32), rand(gen, 8192, 768, dtype=F32)
    da, db = cuda(a, b)
    text = str(ops.matmul.explain(da, db))
    assert _explains_tensor_cores(text) and "serial_splits=24" in text, text
    assert checks.rel_frobenius(ops.matmul(da, db).cpu(), ref.matmul(a, b)) <= 1e-5
    # few tiles and K >= 2048: no heuristic split-K keeps it off the tensor cores
    a, b = rand(gen, 512, 4096, dtype=F32), rand(gen, 4096, 512, dtype=F32)
    da, db = cuda(a, b)
    assert _explains_tensor_cores(str(ops.matmul.explain(da, db)))
    assert checks.rel_frobenius(ops.matmul(da, db).cpu(), ref.matmul(a, b)) <= 1e-5
    # an explicit split_k keeps the exact kernel and its partial sums
    assert "simt_ffma" in str(ops.matmul.explain(da, db, split_k=4))
    # 32x32-blocked f32 operands (matmul.py:157-228) and the prepacked-rows layout (matmul.py:594-627)
    m, n, k = 520, 300, 1000
    a, b, bias = rand(gen, m, k, dtype=F32), rand(gen, k, n, dtype=F32), rand(gen, n, dtype=F32)
    a4, b4 = ref.pack_a_blocked(a), ref.pack_b_blocked(b)
    expect = ref.matmul(a, b, bias=bias, epilogue=torch.relu)
    out = ops.matmul_blocked(*cuda(a4, b4), m, n, k, bias=cuda(bias), epilogue=torch.relu)
    assert out.dtype == F32 and checks.rel_frobenius(out.cpu(), expect) <= 1e-5
    rows = ops.matmul_prepacked_b(cuda(a), cuda(ref.pack_b_blocked_t(b.T.contiguous())), n, cuda(bias), torch.relu)
    assert checks.rel_frobenius(rows.cpu(), expect) <= 1e-5
    # all four orientations with ragged sizes (widening along rows for [K, M] / [K, N] operands)
    m, n, k = 264, 520, 300
    a, b = rand(gen, m, k, dtype=F32), rand(gen, k, n, dtype=F32)
    for trans_a in (False, True):
        for trans_b in (False, True):
            a_in = a.T.contiguous() if trans_a else a
            b_in = b.T.contiguous() if trans_b else b
            out = ops.matmul(*cuda(a_in, b_in), trans_a=trans_a, trans_b=trans_b)
            assert checks.rel_frobenius(out.cpu(), ref.matmul(a, b)) <= 1e-5, (trans_a, trans_b)


@pytest.mark.parametrize("positive", [False, True], ids=["zero_mean", "positive_mean"])
def test_f32_widened_product_long_sums(ops, positive: bool) -> None:
    """The widened path at K = 4096 with enough tiles that the chunks run back to back on one
    CTA, on N(0,1) operands and on uniform [0,1) operands (every partial sum of one sign,
    which is where a truncating accumulator's bias adds up)."""
    gen = torch.Generator().manual_seed(78 + positive)
    make = (lambda *s: torch.rand(*s, generator=gen)) if positive else (lambda *s: torch.randn(*s, generator=gen))
    a, b = make(1024, 4096), make(4096, 1024)
    da, db = cuda(a, b)
    text = str(ops.matmul.explain(da, db))
    assert _explains_tensor_cores(text) and "parallel_splits=1" in text, text
    assert checks.rel_frobenius(ops.matmul(da, db).cpu(), ref.matmul(a, b)) <= 1e-5
    a3, b3 = make(1536, 2048), make(2048, 1536)
    assert checks.rel_frobenius(ops.matmul(*cuda(a3, b3)).cpu(), ref.matmul(a3, b3)) <= 1e-5


def test_peer_wait_gives_up_and_reports() -> None:
    """The device-side wait that ends a fused column-sharded linear, on a flag nobody raises:
    it runs out after its budget, leaves bit 32 in the status word, and the context stays
    usable. A flag that is already raised lets it through at once."""
    from helion_mlir_backend import native

    lib = native.module()
    torch.cuda.synchronize()
    assert native.kernel_status() == 0
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    stream = native.stream_ptr(flags.device)
    assert lib.b200_peer_wait(flags.data_ptr(), 2, 1, 2_000_000, stream) == 0  # 2 ms
    assert native.kernel_status() == 32
    flags.fill_(3)
    assert lib.b200_peer_wait(flags.data_ptr(), 8, 3, 2_000_000, stream) == 0
    assert native.kernel_status() == 0
    assert lib.b200_peer_wait(flags.data_ptr(), 9, 1, 2_000_000, stream) == 7
    assert lib.b200_peer_wait(None, 2, 1, 2_000_000, stream) == 6
    assert lib.b200_peer_wait(flags.data_ptr(), 2, 1, 0, stream) == 7


def test_blocked_a_is_read_in_place_also_batched(ops) -> None:
    """A [M/32, K/32, 32, 32] (matmul.py:92-99) reaches the tensor cores through a 5-D tensor
    map: no unpack pass, no scratch, and a batch of blocked operands stays on the same kernel
    (C ABI; ragged M and an odd number of K blocks included)."""
    from helion_mlir_backend import native

    lib = native.module()
    gen = torch.Generator().manual_seed(31)
    batch, m, n, k = 3, 200, 144, 160  # 7 row blocks, 5 K blocks: the last stage is half empty
    a, b = rand(gen, batch, m, k), rand(gen, batch, k, n, scale=0.25)
    a4 = torch.stack([ref.pack_a_blocked(a[i]) for i in range(batch)]).contiguous()
    da, db = cuda(a4, b)
    out = torch.full((batch, m, n), float("nan"), dtype=F32, device="cuda")
    desc = native.GemmDesc()
    desc.dtype, desc.out_dtype, desc.vec_dtype = native.BF16, native.F32, native.BF16
    desc.a_layout, desc.b_layout = native.LAYOUT_BLOCKED, native.LAYOUT_ROW
    desc.m, desc.n, desc.k, desc.batch = m, n, k, batch
    desc.lda, desc.ldb, desc.ldc = 0, n, n
    desc.stride_a, desc.stride_b, desc.stride_c = a4[0].numel(), k * n, m * n
    desc.a, desc.b, desc.c = da.data_ptr(), db.data_ptr(), out.data_ptr()
    buf = ctypes.create_string_buffer(256)
    assert lib.b200_gemm_explain(ctypes.byref(desc), buf, len(buf)) == 0
    text = buf.value.decode()
    assert text.startswith("umma_bf16") and "unpack" not in text, text
    assert lib.b200_gemm_workspace_bytes(ctypes.byref(desc)) == 0
    rc = lib.b200_gemm(ctypes.byref(desc), native.stream_ptr(da.device))
    assert rc == 0, native.strerror(rc)
    expect = torch.stack([ref.matmul(a[i], b[i], out_dtype=F32) for i in range(batch)])
    assert checks.rel_frobenius(out.cpu(), expect) < 1e-5
    # through the operator: the explanation of the blocked call names no unpack of A
    m2, n2, k2 = 300, 200, 96
    a2, b2 = rand(gen, m2, k2), rand(gen, k2, n2)
    out2 = ops.matmul_blocked(*cuda(ref.pack_a_blocked(a2), ref.pack_b_blocked(b2)), m2, n2, k2)
    checks.assert_parity(BF16, out2.cpu(), ref.matmul(a2, b2), "blocked a4 x b4")
