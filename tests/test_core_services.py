"""Runs the C++ unit tests of the host runtime services (state pool, prefix index and cache, paging, rank plans,
staged start-up with fault injection, worker group, PD transfer protocol, continuous-batching scheduler, CPU planner)."""
import os
import subprocess

import pytest

from ironpangu_b200 import _build


def test_core_services_cpp():
    import os

    _build.build_core()
    _build.build_plugins()
    env = dict(os.environ, IFAB_PLUGIN_DIR=str(_build.PLUGIN_DIR),
               IFAB_EXAMPLE_MODEL=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "mla_moe_slice_tp1.inferfabric"))
    r = subprocess.run([str(_build.TESTS_BIN)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "0 failures" in r.stdout and "ok   kernel_plugin" in r.stdout and "skip kernel_plugin" not in r.stdout


@pytest.mark.gpu
def test_cuda_kernel_plugin_through_the_loader():
    """The CUDA build of the SwiGLU plugin: dlopen + ABI / contract / target checks + prepare + enqueue on a stream."""
    import ctypes as C
    import json

    import torch

    _build.build_core()
    so = [p for p in _build.build_plugins() if p.name.endswith("swiglu_cuda.so")][0]
    lib = C.CDLL(str(_build.CORE_LIB))
    lib.ifab_core_plugin_swiglu.restype = C.c_void_p
    lib.ifab_core_plugin_swiglu.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_long, C.c_void_p]
    lib.ifab_core_free.argtypes = [C.c_void_p]

    def call(target, x, y):
        raw = lib.ifab_core_plugin_swiglu(str(so).encode(), target, x.data_ptr(), y.data_ptr(), y.shape[0], y.shape[1], x.stride(0),
                                          y.stride(0), torch.cuda.current_stream().cuda_stream)
        out = json.loads(C.string_at(raw).decode())
        lib.ifab_core_free(raw)
        torch.cuda.synchronize()
        return out

    x = torch.randn(37, 2 * 96, device="cuda").to(torch.bfloat16)
    y = torch.zeros(37, 96, dtype=torch.bfloat16, device="cuda")
    assert call(b"cuda-sm100a", x, y)["contract"] == "inferfabric.swiglu.bf16.v1"
    want = torch.nn.functional.silu(x[:, :96].float()) * x[:, 96:].float()
    torch.testing.assert_close(y.float(), want, rtol=1e-2, atol=1e-2)
    assert call(b"cpu", x, y)["error"]["kind"] == "stale"


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_cpp_unit_tests_under_sanitizers(kind):
    """The whole host core (compiler, planner, state pool, scheduler, service threads, HTTP pieces) compiled under
    AddressSanitizer + UBSan, and under ThreadSanitizer: the C++ unit tests must pass without a single report."""
    binary = _build.build_core_tests_sanitized(kind)
    _build.build_plugins()
    env = dict(os.environ, IFAB_PLUGIN_DIR=str(_build.PLUGIN_DIR),
               IFAB_EXAMPLE_MODEL=os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "mla_moe_slice_tp1.inferfabric"),
               ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=0")
    r = subprocess.run([str(binary)], capture_output=True, text=True, timeout=600, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "0 failures" in out and "Sanitizer" not in out and "runtime error" not in out, out[-3000:]
