"""In-tree builds of the native libraries.

Two shared objects are produced next to the sources they come from:

* ``csrc/kernels/libifab_kernels.so`` - every sm_100a CUDA kernel behind a C ABI (``ifab_kernels.h``),
  compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``csrc/core/libifab_core.so`` + ``csrc/cli/ifab`` - the C++20 compiler / planner / runtime services.

The libraries are loaded with ``ctypes``; kernels take raw device pointers (``tensor.data_ptr()``) and
the current CUDA stream, so no torch headers are needed at build time and a build takes seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
KERNEL_DIR = ROOT / "csrc" / "kernels"
CORE_DIR = ROOT / "csrc" / "core"
CLI_DIR = ROOT / "csrc" / "cli"
SERVER_DIR = ROOT / "csrc" / "server"
KERNEL_LIB = KERNEL_DIR / "libifab_kernels.so"
CORE_LIB = CORE_DIR / "libifab_core.so"
CLI_BIN = CLI_DIR / "ifab"
SERVER_BIN = SERVER_DIR / "ifab-server"
DEVICE_DIR = ROOT / "csrc" / "device"
DEVICE_LIB = DEVICE_DIR / "libifab_device.so"
TESTS_DIR = ROOT / "csrc" / "tests"
TESTS_BIN = TESTS_DIR / "core_tests"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]
CXX_FLAGS = ["-std=c++20", "-O2", "-fPIC", "-Wall", "-Wextra", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stale(target: Path, sources, extra: str = "") -> bool:
    stamp = target.with_suffix(target.suffix + ".stamp")
    want = _digest(sources) + extra
    if target.exists() and stamp.exists() and stamp.read_text() == want:
        return False
    return True


def _mark(target: Path, sources, extra: str = "") -> None:
    target.with_suffix(target.suffix + ".stamp").write_text(_digest(sources) + extra)


def _run(cmd, cwd=None):
    r = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``*.cu`` under csrc/kernels for sm_100a into one shared library."""
    cus = sorted(KERNEL_DIR.glob("*.cu"))
    deps = cus + sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    if not force and not _stale(KERNEL_LIB, deps):
        return KERNEL_LIB
    nvcc = _nvcc()
    objdir = KERNEL_DIR / "build"
    objdir.mkdir(exist_ok=True)

    def one(cu: Path):
        obj = objdir / (cu.stem + ".o")
        flags = list(NVCC_FLAGS)
        if verbose:
            flags += ["-Xptxas", "-v"]
        out = _run([nvcc, *flags, "-c", str(cu), "-o", str(obj)], cwd=KERNEL_DIR)
        return obj, out

    with ThreadPoolExecutor(max_workers=min(8, len(cus))) as ex:
        results = list(ex.map(one, cus))
    objs = [str(o) for o, _ in results]
    _run([nvcc, "-shared", "-o", str(KERNEL_LIB), *objs, "-lcudart", "-lcuda"], cwd=KERNEL_DIR)
    _mark(KERNEL_LIB, deps)
    if verbose:
        for _, out in results:
            print(out)
    return KERNEL_LIB


def build_core(force: bool = False) -> Path:
    """Compile the C++20 host libraries and tools (compiler, planner, runtime services, CLI, server)."""
    srcs = sorted(CORE_DIR.glob("*.cpp"))
    deps = srcs + sorted(CORE_DIR.glob("*.h"))
    if srcs and (force or _stale(CORE_LIB, deps)):
        objdir = CORE_DIR / "build"
        objdir.mkdir(exist_ok=True)

        def one(src: Path):
            obj = objdir / (src.stem + ".o")
            _run(["g++", *CXX_FLAGS, "-c", str(src), "-o", str(obj)], cwd=CORE_DIR)
            return str(obj)

        with ThreadPoolExecutor(max_workers=8) as ex:
            objs = list(ex.map(one, srcs))
        _run(["g++", "-shared", "-o", str(CORE_LIB), *objs, "-pthread"], cwd=CORE_DIR)
        _mark(CORE_LIB, deps)
    for bindir, binary in ((CLI_DIR, CLI_BIN), (SERVER_DIR, SERVER_BIN), (TESTS_DIR, TESTS_BIN)):
        bsrcs = sorted(bindir.glob("*.cpp"))
        if not bsrcs:
            continue
        bdeps = bsrcs + sorted(bindir.glob("*.h")) + deps
        if force or _stale(binary, bdeps):
            _run(["g++", *CXX_FLAGS, "-I", str(CORE_DIR), *map(str, bsrcs), "-o", str(binary),
                  "-L", str(CORE_DIR), "-lifab_core", f"-Wl,-rpath,{CORE_DIR}", "-Wl,-rpath,$ORIGIN/../core",
                  "-pthread", "-ldl"], cwd=bindir)
            _mark(binary, bdeps)
    return CORE_LIB


def build_core_tests_sanitized(kind: str, force: bool = False) -> Path:
    """The C++ unit-test binary with the whole host core compiled under a sanitizer: ``"address"`` (AddressSanitizer +
    UndefinedBehaviorSanitizer) or ``"thread"`` (ThreadSanitizer, for the scheduler / state-pool / service threads). One
    statically linked binary per kind under ``csrc/tests/``; the regular libraries are not touched."""
    flags = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "thread": ["-fsanitize=thread"]}[kind]
    out = TESTS_DIR / f"core_tests_{kind}"
    srcs = sorted(CORE_DIR.glob("*.cpp"))
    tsrcs = sorted(TESTS_DIR.glob("*.cpp"))
    deps = srcs + tsrcs + sorted(CORE_DIR.glob("*.h")) + sorted(TESTS_DIR.glob("*.h"))
    if force or _stale(out, deps):
        objdir = CORE_DIR / "build" / kind
        objdir.mkdir(parents=True, exist_ok=True)
        cxx = [f for f in CXX_FLAGS if not f.startswith("-O")] + ["-O1", "-g", "-fno-omit-frame-pointer", *flags]

        def one(src: Path):
            obj = objdir / (src.stem + ".o")
            _run(["g++", *cxx, "-I", str(CORE_DIR), "-c", str(src), "-o", str(obj)], cwd=src.parent)
            return str(obj)

        with ThreadPoolExecutor(max_workers=8) as ex:
            objs = list(ex.map(one, srcs + tsrcs))
        _run(["g++", *flags, "-o", str(out), *objs, "-pthread", "-ldl"], cwd=TESTS_DIR)
        _mark(out, deps)
    return out


PLUGIN_DIR = ROOT / "csrc" / "plugins"


def build_plugins(force: bool = False) -> list:
    """Compile every example kernel plugin (``csrc/plugins/*.cpp`` with g++, ``*.cu`` with nvcc) into its own shared object."""
    out = []
    hdr = [CORE_DIR / "kernel_plugin.h"]
    for src in sorted(PLUGIN_DIR.glob("*.cpp")) + sorted(PLUGIN_DIR.glob("*.cu")):
        so = PLUGIN_DIR / f"libifab_plugin_{src.stem}.so"
        if force or _stale(so, [src] + hdr):
            if src.suffix == ".cu":
                _run([_nvcc(), *NVCC_FLAGS, "-shared", "-Xcompiler", "-fPIC", str(src), "-o", str(so), "-lcudart"], cwd=PLUGIN_DIR)
            else:
                _run(["g++", *CXX_FLAGS, "-shared", str(src), "-o", str(so)], cwd=PLUGIN_DIR)
            _mark(so, [src] + hdr)
        out.append(so)
    return out


def build_device(force: bool = False) -> Path:
    """The native device executor (``csrc/device``): C++ against the CUDA runtime, the kernel library and the host core. The
    server loads it on demand (``ifab-server --program BUNDLE CHECKPOINT --native``), so the server itself needs no CUDA."""
    srcs = sorted(DEVICE_DIR.glob("*.cpp"))
    deps = srcs + sorted(DEVICE_DIR.glob("*.h")) + sorted(CORE_DIR.glob("*.h")) + [KERNEL_DIR / "ifab_kernels.h"]
    if srcs and (force or _stale(DEVICE_LIB, deps)):
        build_kernels()
        build_core()
        cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        _run(["g++", *CXX_FLAGS, "-shared", "-I", str(cuda / "include"), *map(str, srcs), "-o", str(DEVICE_LIB),
              "-L", str(CORE_DIR), "-lifab_core", "-L", str(KERNEL_DIR), "-lifab_kernels", "-L", str(cuda / "lib64"), "-lcudart",
              "-Wl,-rpath,$ORIGIN/../core", "-Wl,-rpath,$ORIGIN/../kernels", f"-Wl,-rpath,{cuda / 'lib64'}"], cwd=DEVICE_DIR)
        _mark(DEVICE_LIB, deps)
    return DEVICE_LIB


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_core(force)
    build_plugins(force)
    build_device(force)


if __name__ == "__main__":
    import sys
    build_kernels(force="--force" in sys.argv, verbose="-v" in sys.argv)
    build_core(force="--force" in sys.argv)
    print("built", KERNEL_LIB, CORE_LIB if CORE_LIB.exists() else "")
