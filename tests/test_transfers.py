"""Classified host/device transfers: roles, the guard against implicit copies, the audit documents."""
import pytest
import torch

from ironpangu_b200.runtime.transfers import ImplicitTransfer, TransferAudit, prepared_execution_report, state_copy_report


def test_roles_guard_and_report():
    t = TransferAudit()
    host, dev = torch.arange(6, dtype=torch.int32), torch.zeros(6, dtype=torch.int32)
    with pytest.raises(ImplicitTransfer):           # no role: an implicit copy
        t.h2d(dev, host)
    with t.scope("control_input"):
        t.h2d(dev[:4], host[:4])
        up = t.upload(host, "cpu")
        with pytest.raises(ImplicitTransfer):       # control inputs never come back
            t.d2h(host, dev)
        with t.scope("request_output"):             # scopes nest and restore
            t.d2h(host[:2], dev[:2])
            with pytest.raises(ImplicitTransfer):
                t.h2d(dev, host)
        t.h2d(dev[:1], host[:1])
    assert t.role is None and torch.equal(up, host) and torch.equal(dev[:4], host[:4])
    with t.scope("parameter_preparation"):
        t.h2d(dev, host)
    with pytest.raises(ValueError):
        with t.scope("activation"):
            pass
    r = t.report()
    assert r["format"] == "ifab.transfer-audit.v1" and r["activation_host_transfers"] == 0 and r["rejected"] == 3
    by = {b["role"]: b for b in r["boundaries"]}
    assert by["control_input"] == {"role": "control_input", "h2d_calls": 3, "h2d_bytes": 16 + 24 + 4, "d2h_calls": 0, "d2h_bytes": 0}
    assert by["request_output"]["d2h_bytes"] == 8 and by["request_output"]["h2d_calls"] == 0
    assert by["parameter_preparation"]["h2d_bytes"] == 24
    assert t.totals() == (44 + 24, 8)


def test_engine_reports_have_their_formats():
    class Arena:
        bytes, workspace_bytes, slots, leased, tokens = 1024, 512, {1: (0, 512)}, {1: 100}, 8

    class Dec:
        launches_per_forward, arena, bundle_sha256 = 20, Arena(), "ab" * 32

    class Prefix:
        entries, hits, misses, evicted = {1: 1}, 3, 2, 1

    class Eng:
        dec, _graphs, prefix, allocations_at_ready = Dec(), {1: None, 4: None}, Prefix(), None
        audit_counters = {"prefix_rows_copied": 64, "prefix_rows_published": 32}

    p = prepared_execution_report(Eng())
    assert p["format"] == "ifab.prepared-execution.v1" and p["graph_widths"] == [1, 4] and p["arena"]["planned_rows"] == 8
    assert p["program_sha256"] == "ab" * 32
    s = state_copy_report(Eng())
    assert s == {"format": "ifab.state-copy-audit.v1", "host_bytes": 0, "rows_restored": 64, "rows_published": 32, "snapshots": 1,
                 "hits": 3, "misses": 2, "evicted": 1}


def test_init_plan_loader_stages_through_a_bounded_buffer(tmp_path):
    """Row shards, strided column shards and expert stacks of a two-rank plan: the same bytes whatever the staging size, every
    upload recorded as parameter preparation, a column shard equal to the slice of the checkpoint tensor."""
    import json

    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig
    from ironpangu_b200.runtime.plan_engine import SafetensorsDir, load_parameters

    cfg = MlaMoeConfig.tiny(layers=1)
    src = tmp_path / "m.inferfabric"
    src.write_text(mla_moe_source(cfg, 2, context=64))
    assert compiler.cli("synth-checkpoint", str(src), str(tmp_path / "ck"), "--seed", "1").returncode == 0
    out = compiler.write_bundle(str(src), str(tmp_path / "b"), checkpoint_dir=str(tmp_path / "ck"))
    ck = SafetensorsDir(str(tmp_path / "ck"))
    for rank in (0, 1):
        plan = json.loads((tmp_path / "b" / f"rank-{rank}.init.json").read_text())
        assert any(l["kind"] != "slice" for l in plan["loads"])          # the o_proj / down column shards are strided
        big = load_parameters(plan, ck, "cpu")
        tr = TransferAudit()
        small = load_parameters(plan, ck, "cpu", staging_bytes=4096, transfers=tr)
        total = sum(t.numel() * t.element_size() for t in big.values())
        assert set(big) == set(small) and all(torch.equal(big[k].view(torch.uint8), small[k].view(torch.uint8)) for k in big)
        b = {x["role"]: x for x in tr.report()["boundaries"]}["parameter_preparation"]
        assert b["h2d_calls"] > len(plan["loads"]) and b["d2h_calls"] == 0 and tr.rejected == 0
        assert b["h2d_bytes"] <= total
        mm, off, n, dtype, shape = ck.tensors["model.layers.0.self_attn.o_proj.weight"]
        full = torch.frombuffer(bytearray(mm[off:off + n]), dtype=torch.bfloat16).view(*shape)
        half = shape[1] // 2
        assert torch.equal(big["model.layers.0.self_attn.o_proj"], full[:, rank * half:(rank + 1) * half])
    assert out["instructions"] > 0


def test_step_traces_line_up_across_ranks(tmp_path):
    from ironpangu_b200.runtime.trace import COLUMNS, StepTrace, merge

    counters = [{"rows": 0, "prefill_rows": 0, "launch_groups": 0, "sampled_rows": 0, "h2d_bytes": 0, "d2h_bytes": 0} for _ in range(2)]
    traces = [StepTrace(str(tmp_path), rank=r, use_cuda=False, flush_every=2) for r in range(2)]
    for step in range(5):
        for r, t in enumerate(traces):
            rec = t.begin(counters[r], slices=step + 1)
            counters[r]["rows"] += 3
            counters[r]["prefill_rows"] += 16 if step == 0 else 0
            counters[r]["launch_groups"] += 1
            counters[r]["h2d_bytes"] += 36
            t.end(rec, counters[r])
    for t in traces:
        t.close()
    lines = (tmp_path / "steps-rank1.csv").read_text().splitlines()
    assert lines[0].split(",") == COLUMNS and len(lines) == 6
    first = dict(zip(COLUMNS, lines[1].split(",")))
    assert first["rows"] == "19" and first["prompt_rows"] == "16" and first["slices"] == "1" and first["h2d_bytes"] == "36" and first["device_ms"] == ""
    m = merge(str(tmp_path))
    assert [x["step"] for x in m] == list(range(5)) and all(x["ranks"] == 2 and x["device_ms_max"] is None and x["host_ms_max"] >= 0 for x in m)
    # a rank that recorded fewer steps is reported, not papered over
    (tmp_path / "steps-rank1.csv").write_text("\n".join(lines[:4]) + "\n")
    with pytest.raises(ValueError, match="do not line up"):
        merge(str(tmp_path))
