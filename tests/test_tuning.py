"""The persisted tuning table: keys, round trip through the file, and what is ignored."""

from __future__ import annotations

import json

import torch

from helion_mlir_utils import tuning


def test_round_trip_and_hardware_key(tmp_path) -> None:
    table = tuning.TuneTable("NVIDIA B200 sm_100 148sm", tmp_path)
    key = tuning.problem_key("matmul", torch.bfloat16, 8192, 4096, 4096, False, True, 1, "bias+act2")
    assert key == "matmul|bfloat16|nt|1x8192x4096x4096|bias+act2"
    assert table.get(key) is None and len(table) == 0
    table.put(key, tuning.Choice(256, 2, 0), microseconds=207.25)
    again = tuning.TuneTable("NVIDIA B200 sm_100 148sm", tmp_path)  # a new process reads the file
    assert again.get(key) == tuning.Choice(256, 2, 0) and len(again) == 1
    stored = json.loads(again.path.read_text())
    assert stored["hardware"] == "NVIDIA B200 sm_100 148sm" and stored["entries"][key]["us"] == 207.25
    # another GPU model has its own file and sees nothing of this one
    other = tuning.TuneTable("NVIDIA B200 sm_100 132sm", tmp_path)
    assert other.path != again.path and other.get(key) is None


def test_unreadable_or_foreign_tables_are_ignored(tmp_path) -> None:
    table = tuning.TuneTable("hw", tmp_path)
    table.path.parent.mkdir(parents=True, exist_ok=True)
    table.path.write_text("{ not json")
    assert table.get("k") is None
    table.put("k", tuning.Choice(128, 1, 4))  # and is replaced by a good one
    assert tuning.TuneTable("hw", tmp_path).get("k") == tuning.Choice(128, 1, 4)
    # same file name forged for another hardware string, or with values no kernel has
    table.path.write_text(json.dumps({"format": 1, "hardware": "other", "entries": {"k": {"tile_n": 64}}}))
    assert tuning.TuneTable("hw", tmp_path).get("k") is None
    table.path.write_text(json.dumps({"format": 1, "hardware": "hw", "entries": {
        "wide": {"tile_n": 4096}, "pair": {"cta_group": 7}, "text": {"tile_n": "x"}, "ok": {"tile_n": 192}}}))
    fresh = tuning.TuneTable("hw", tmp_path)
    assert fresh.get("wide") is None and fresh.get("pair") is None and fresh.get("text") is None
    assert fresh.get("ok") == tuning.Choice(192, 0, 0)


def test_candidates_and_choice_codes() -> None:
    cands = tuning.candidates(8192, 4096, 4096)
    assert cands[0] == tuning.Choice() and tuning.Choice(256, 2, 0) in cands and tuning.Choice(192, 2, 0) not in cands
    assert all(c.split_k == 0 for c in cands)
    assert all(c.tile_n <= 64 for c in tuning.candidates(512, 48, 256))
    assert tuning.Choice(0, 0, 8) in tuning.candidates(256, 256, 8192, with_splits=True)
    assert (tuning.Choice(0, 1, 0).force_kernel(), tuning.Choice(0, 2, 0).force_kernel(), tuning.Choice().force_kernel()) == (3, 4, 0)


def test_lookup_can_be_switched_off(tmp_path, monkeypatch) -> None:
    monkeypatch.setenv(tuning.TUNE_DIR_ENV, str(tmp_path))
    tuning.table().put("k", tuning.Choice(64, 1, 0))
    assert tuning.lookup("k") == tuning.Choice(64, 1, 0)
    monkeypatch.setenv(tuning.TUNE_DISABLE_ENV, "1")
    assert tuning.lookup("k") is None
