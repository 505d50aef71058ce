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
