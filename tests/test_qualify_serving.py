"""The serving qualification scenarios, run on CPU: ifab-server in front of the stand-in engine process (the engine-worker socket
protocol with deterministic tokens), every scenario including overload and the death of the engine between two steps."""
import json

from ironpangu_b200.utils import qualify_serving as Q


def test_every_scenario_passes_against_the_stand_in_engine(tmp_path):
    report = tmp_path / "q.json"
    out = Q.main(["--engine", "standin", "--waves", "3", "--wave-requests", "12", "--report", str(report)])
    assert set(out["scenarios"]) == {"repeatability", "cancellation", "prefix_cache", "load_waves", "shutdown", "overload", "engine_failure"}
    bad = {k: v for k, v in out["scenarios"].items() if not v["passed"]}
    assert not bad, bad
    assert json.loads(report.read_text())["passed"] is True
    pc = out["scenarios"]["prefix_cache"]["counters_hits_misses_evicted"]
    assert pc[2][0] > pc[1][0] and pc[4][2] > 0            # the warm prompt hit; the flood evicted
    st = out["scenarios"]["overload"]["statuses"]
    assert set(st) == {"200", "429"}                        # refusals are 429 with a JSON body, never a 5xx or a hang
    ef = out["scenarios"]["engine_failure"]
    assert ef["health_after"] == 503 and ef["request_after"] == 503 and ef["restarted_serves"] == 200


def test_stand_in_engine_follows_the_worker_protocol():
    eng = Q.StandInEngine(residents=2, context=64, vocab=100, budget=16, prefix_slots=2, step_ms=0)
    eng.admit(0, 40)
    p = Q.prompt(1, 32, 100)
    assert eng.step([[0, 0, 16, 0]], p[:16]) == [0]                 # a prompt chunk that does not sample
    t = eng.step([[0, 16, 16, 1]], p[16:])
    assert len(t) == 1 and 0 < t[0] < 100
    assert eng.audit()["prefix_published"] == 1 and eng.audit()["prefix_misses"] == 1
    eng.admit(1, 40)
    assert eng.step([[1, 0, 16, 0]], p[:16]) == [0] and eng.audit()["prefix_hits"] == 1
    assert eng.step([[1, 16, 16, 1]], p[16:]) == t                  # same history, same token
    try:
        eng.step([[1, 40, 1, 1]], [5])
        raise AssertionError("a slice that skips positions must be refused")
    except RuntimeError:
        pass
    try:
        eng.admit(0, 65)
        raise AssertionError("a reservation beyond the context must be refused")
    except OverflowError:
        pass


def test_prefix_snapshot_keys_boundaries_and_salts():
    from ironpangu_b200.runtime.engine_worker import PrefixSnapshots, checkpoint_boundary

    # whole cache blocks and whole prompt slices, and always at least one prompt token left to run
    assert checkpoint_boundary(100, 16, 16) == 96 and checkpoint_boundary(96, 16, 16) == 80 and checkpoint_boundary(16, 16, 16) == 0
    assert checkpoint_boundary(100, 16, 24) == 96 and checkpoint_boundary(95, 16, 24) == 48      # lcm(16, 24) = 48
    assert checkpoint_boundary(1000, 8, 512) == 512 and checkpoint_boundary(0, 8, 8) == 0
    p = PrefixSnapshots(2, block=8, chunk=8, namespace="prod")
    toks = list(range(20))
    p.publish(toks, lambda n: [n], salt="a")
    assert len(p.entries) == 1 and next(iter(p.entries)) == (("prod", "a"), tuple(range(16)))
    assert p.lookup(toks[:8], "a")[0] == tuple(range(16)) and p.lookup(toks[:8], "b") is None and p.lookup(toks[:8]) is None
    assert p.lookup(toks[:17], "a") is None                     # longer than what was stored
    p.publish(toks, lambda n: [n], salt="a")                    # again: refreshed, not duplicated
    p.publish(toks, lambda n: [n], salt="b")
    p.publish(list(range(50, 70)), lambda n: [n], salt="a")     # third entry: the least recently used one goes
    assert p.published == 3 and p.evicted == 1 and p.lookup(toks[:8], "a") is None and p.lookup(toks[:8], "b") is not None
