"""The C-ABI library loads without a GPU and exports every symbol include/b200ops.h declares."""

from __future__ import annotations

import ctypes
from pathlib import Path
import re

import pytest

from helion_mlir_backend import native

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200ops.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree() -> None:
    names = declared_functions()
    assert len(names) >= 20
    assert sorted(native.SIGNATURES) == names


def test_library_exports_every_declared_symbol(built_library: Path) -> None:
    lib = ctypes.CDLL(str(built_library))
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_loads_and_answers_without_a_gpu() -> None:
    lib = native.module()
    assert lib.b200_abi_version() == 1
    assert native.strerror(0) == "ok"
    assert "element type" in native.strerror(1)
    assert native.strerror(10) == "native calls are disabled"
    stats = native.PoolStats()
    assert lib.b200_pool_stats(ctypes.byref(stats)) == 0
    assert lib.b200_column_sum_workspace_bytes(1, 100) == 0
    assert lib.b200_column_sum_workspace_bytes(65536, 128) > 0


def test_struct_layout_matches_header() -> None:
    """Field order of the ctypes mirror follows the C struct (names in order)."""
    text = HEADER.read_text()
    body = text[text.index("typedef struct b200_gemm_desc {") : text.index("} b200_gemm_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields: list[str] = []
    for statement in body.split(";"):
        statement = statement.replace("typedef struct b200_gemm_desc {", "").strip()
        if not statement:
            continue
        names = statement.split(",")
        first = names[0].split()[-1].lstrip("*")
        fields.append(first)
        fields.extend(n.strip().lstrip("*") for n in names[1:])
    assert fields == [name for name, _ in native.GemmDesc._fields_]


def test_refusals_are_codes_not_crashes() -> None:
    """Bad arguments come back as refusal codes before any CUDA call is made."""
    lib = native.module()
    assert lib.b200_softmax(7, None, None, 4, 4, 4, None) == 1  # dtype
    assert lib.b200_softmax(native.F32, None, None, 4, 4, 4, None) == 6  # NULL
    assert lib.b200_softmax(native.F32, None, None, 0, 4, 4, None) == 0  # empty: nothing to do
    assert lib.b200_eltwise(9, native.F32, None, None, 4, 0.0, None) == 7
    assert lib.b200_pack(99, native.F32, None, 1, 1, 1, None, 32, 32, 0, None) == 7
    desc = native.GemmDesc()
    desc.dtype = 5
    assert lib.b200_gemm(ctypes.byref(desc), None) == 1
    assert lib.b200_gemm(None, None) == 6
    counters = native.counters()
    assert counters["refusals"] >= 5 and counters["last_refusal"] == 6
    native.set_native_call(False)
    try:
        assert lib.b200_softmax(native.F32, None, None, 4, 4, 4, None) == native.E_DISABLED
    finally:
        native.set_native_call(True)


def test_static_scratch_size_check_refuses_beyond_the_capacity() -> None:
    """The check that keeps b200_column_sum_static inside its fixed array, called with
    capacities other than the array's: under the present launch plan no shape needs more than
    the 2 MiB the array has, so the refusal only shows against a smaller capacity."""
    lib = native.module()
    too_large = 11
    assert "capacity" in native.strerror(too_large)
    limit = 2 << 20
    shapes = [(m, n) for m in (1, 64, 4096, 37888, 1 << 20, 1 << 24) for n in (1, 96, 443, 512, 1024, 4096, 65536, 1 << 20)]
    for m, n in shapes:
        need = int(lib.b200_column_sum_workspace_bytes(m, n))
        assert need <= limit
        assert lib.b200_column_sum_static_fits(m, n, limit) == 0
        if need > 0:
            assert lib.b200_column_sum_static_fits(m, n, need) == 0  # exactly fits
            assert lib.b200_column_sum_static_fits(m, n, need - 1) == too_large
    assert max(int(lib.b200_column_sum_workspace_bytes(m, n)) for m, n in shapes) == limit  # the bound is met, not just respected
