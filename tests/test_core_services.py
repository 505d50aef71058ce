"""Runs the C++ unit tests of the host runtime services (state pool, prefix index and cache, paging, rank plans,
staged start-up with fault injection, worker group, PD transfer protocol, continuous-batching scheduler, CPU planner)."""
import subprocess

from ironpangu_b200 import _build


def test_core_services_cpp():
    _build.build_core()
    r = subprocess.run([str(_build.TESTS_BIN)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "0 failures" in r.stdout
