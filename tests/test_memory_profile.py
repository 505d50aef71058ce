"""Start-up memory options and staged memory profile (no device: the probe is a fake)."""
import json

import pytest

from ironpangu_b200.runtime.memory import MemoryProfile, StartupOptions


def _probe(seq):
    it = iter(seq)
    return lambda: next(it)


def test_options_validation():
    StartupOptions().validate()
    for bad in (dict(max_model_len=0), dict(max_num_seqs=65), dict(max_num_batched_tokens=0),
                dict(gpu_memory_utilization=1.2), dict(profile_only=True)):
        with pytest.raises(ValueError):
            StartupOptions(**bad).validate()
    assert StartupOptions(gpu_memory_utilization=0.5).budget_bytes(1000) == 500


def test_profile_records_stages_and_headroom(tmp_path):
    path = tmp_path / "mem.json"
    total = 1000
    rec = MemoryProfile.start(StartupOptions(memory_profile=str(path), gpu_memory_utilization=0.9),
                              _probe([(990, total), (600, total), (550, total), (540, total)]))
    rec.stage("weights")
    rec.stage("state", note="kv + scratch")
    rec.stage("graphs")
    prof = rec.finish()
    assert rec.summary() == {"weights": 390, "state": 50, "graphs": 10}
    d = json.loads(path.read_text())
    assert d["baseline_used_bytes"] == 10 and d["budget_bytes"] == 900 and d["headroom_bytes"] == 900 - 460
    assert [s["name"] for s in d["stages"]] == ["weights", "state", "graphs"] and d["failed_stage"] is None
    assert prof.stages[1].note == "kv + scratch"


def test_profile_names_the_stage_that_broke_the_budget(tmp_path):
    path = tmp_path / "mem.json"
    rec = MemoryProfile.start(StartupOptions(memory_profile=str(path), gpu_memory_utilization=0.5),
                              _probe([(1000, 1000), (700, 1000), (400, 1000)]))
    rec.stage("weights")
    with pytest.raises(MemoryError, match="state"):
        rec.stage("state")
    d = json.loads(path.read_text())
    assert d["failed_stage"] == "state" and "exceed the budget" in d["failure"]
