"""Tuning on the device: candidates are timed, the winner is stored and used by the
next plan, results do not depend on the choice."""

from __future__ import annotations

import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tune_matmul_records_and_applies(built_library, tmp_path, monkeypatch) -> None:
    import helion_mlir_utils as ops
    mm = importlib.import_module("helion_mlir_utils.matmul")
    from helion_mlir_utils import tuning

    monkeypatch.setenv(tuning.TUNE_DIR_ENV, str(tmp_path))
    gen = torch.Generator().manual_seed(5)
    a = torch.randn(1024, 512, generator=gen).bfloat16().cuda()
    w = torch.randn(768, 512, generator=gen).bfloat16().cuda()
    baseline = ops.matmul(a, w, trans_b=True)
    # every candidate computes the same bits
    for choice in tuning.candidates(1024, 768, 512):
        assert torch.equal(ops.matmul(a, w, trans_b=True, _choice=choice), baseline), choice
    picked = [tuning.Choice(64, 1, 0), tuning.Choice(128, 2, 0)]
    best, timings = ops.tune_matmul(a, w, trans_b=True, choices=picked, iterations=5)
    assert best in picked and set(timings) == set(picked) and all(t > 0 for t in timings.values())
    key = mm.tune_key(torch.bfloat16, 1024, 768, 512, False, True, False, ops.identity_epilogue)
    assert tuning.table().get(key) == best and tuning.table().path.exists()
    # the next plan of this problem follows the table
    text = str(ops.matmul.explain(a, w, trans_b=True))
    assert f"cta_group={best.cta_group}" in text and f"x{best.tile_n}x" in text
    assert torch.equal(ops.matmul(a, w, trans_b=True), baseline)
    # explicit block_sizes still win over the table
    assert "x256x" in str(ops.matmul.explain(a, w, trans_b=True, block_sizes=(128, 256, 64)))
    mm.forget_plans()
