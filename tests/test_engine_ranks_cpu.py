"""Host-side failure detection of the multi-rank engine worker, on CPU ranks (gloo): every rank executes every request and
the ranks agree on the outcome before rank 0 answers - a rank that fails or samples a different token turns the answer
into a backend error instead of going unnoticed."""
import json
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _session(tmp_path, scenario, requests, mode="strict"):
    path = str(tmp_path / "engine.sock")
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(path)
    srv.listen(1)
    srv.settimeout(120)
    env = dict(os.environ, IFAB_ENGINE_SOCKET=path)
    proc = subprocess.Popen([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                             "--master-port", str(_free_port()), os.path.join(HERE, "gloo_engine_ranks.py"), scenario, mode],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    try:
        conn, _ = srv.accept()
        conn.settimeout(120)
        f = conn.makefile("rwb")
        answers = []
        for req in requests:
            f.write(json.dumps(req).encode() + b"\n")
            f.flush()
            answers.append(json.loads(f.readline()))
        conn.close()
        out, _ = proc.communicate(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()
        srv.close()
        if os.path.exists(path):
            os.unlink(path)
    assert proc.returncode == 0, out[-3000:]
    assert out.count("left the loop") == 2          # both ranks saw the shutdown
    return answers


STEP = {"op": "step", "slices": [[0, 0, 2, 1], [1, 0, 1, 1]], "tokens": [3, 4, 5]}
SCRIPT = [{"op": "info"}, {"op": "admit", "resident": 0, "reserve": 8, "sampling": {}}, STEP, STEP, {"op": "admit", "resident": 1, "reserve": 999},
          {"op": "shutdown"}]


def test_ranks_agree_and_capacity_errors_stay_capacity_errors(tmp_path):
    a = _session(tmp_path, "agree", SCRIPT)
    assert a[0]["ok"] and a[0]["info"]["world"] == 2
    assert a[2] == {"ok": True, "tokens": [12, 13]} and a[3] == a[2]
    assert a[4]["ok"] is False and a[4]["kind"] == "capacity"
    assert a[5]["ok"]


def test_a_rank_that_samples_another_token_is_reported(tmp_path):
    a = _session(tmp_path, "mismatch", SCRIPT)
    assert a[2]["ok"] and a[3]["ok"] is False and a[3]["kind"] == "backend" and "consensus" in a[3]["error"] and "rank 1" in a[3]["error"]


def test_a_rank_that_fails_is_reported_by_rank_zero(tmp_path):
    a = _session(tmp_path, "raise", SCRIPT)
    assert a[2]["ok"] and a[3]["ok"] is False and a[3]["kind"] == "backend" and "rank 1" in a[3]["error"] and "rank-local failure" in a[3]["error"]


def test_deferred_agreement_reports_one_request_later_and_stays_failed(tmp_path):
    """Deferred mode overlaps the comparison of request k with request k + 1: the answer of the step the ranks disagreed on
    has left already, the next answer (and every later one) is the backend error."""
    script = SCRIPT[:4] + [STEP, STEP, {"op": "shutdown"}]
    a = _session(tmp_path, "agree", script, "deferred")
    assert all(x["ok"] for x in a)
    for scenario, needle in (("mismatch", "consensus"), ("raise", "rank-local failure")):
        a = _session(tmp_path, scenario, script, "deferred")
        assert a[2]["ok"] and a[3]["ok"]                       # the second step is the one rank 1 spoils; rank 0 has answered it
        assert a[4]["ok"] is False and a[4]["kind"] == "backend" and "earlier request" in a[4]["error"] and needle in a[4]["error"]
        assert a[5]["ok"] is False and a[5]["error"] == a[4]["error"]


def test_deferred_agreement_reports_at_shutdown_when_no_request_follows(tmp_path):
    """The comparison still in flight when the server says goodbye is waited for: its error rides on the shutdown answer."""
    a = _session(tmp_path, "mismatch", SCRIPT[:4] + [{"op": "shutdown"}], "deferred")
    assert a[2]["ok"] and a[3]["ok"]
    assert a[4]["ok"] is False and "earlier request" in a[4]["error"] and "consensus" in a[4]["error"]
