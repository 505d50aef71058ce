"""Python binding of the C++ compiler core (``libifab_core.so``): DSL -> checked graph -> physical
program -> bundle, plus the CPU interpreter. Results come back as parsed JSON; errors raise
:class:`CompileError` with the core's error kind.
"""
from __future__ import annotations

import ctypes as C
import json
import subprocess
from pathlib import Path
from typing import Any, Dict, List, Optional

from .. import _build

_lib = None


class CompileError(RuntimeError):
    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind
        self.message = message


def _load():
    global _lib
    if _lib is None:
        path = _build.build_core()
        lib = C.CDLL(str(path))
        for name, nargs in (("ifab_core_compile", 2), ("ifab_core_write_bundle", 5), ("ifab_core_interpret", 3),
                            ("ifab_core_read_init_plan", 1), ("ifab_core_read_program", 1), ("ifab_core_validate_bundle", 1)):
            fn = getattr(lib, name)
            fn.restype = C.c_void_p
            fn.argtypes = [C.c_char_p] * nargs
        lib.ifab_core_free.argtypes = [C.c_void_p]
        _lib = lib
    return _lib


def _call(name: str, *args: Optional[str]) -> Dict[str, Any]:
    lib = _load()
    raw = getattr(lib, name)(*[None if a is None else a.encode() for a in args])
    try:
        out = json.loads(C.string_at(raw).decode())
    finally:
        lib.ifab_core_free(raw)
    if isinstance(out, dict) and "error" in out:
        raise CompileError(out["error"]["kind"], out["error"]["message"])
    return out


def compile_source(source: str, **options) -> Dict[str, Any]:
    """Compile DSL text. Returns ``{"graph", "program", "program_sha256", "required_tensors"}``."""
    return _call("ifab_core_compile", source, json.dumps(options))


def write_bundle(source_path: str, out_dir: str, checkpoint_dir: Optional[str] = None, **options) -> Dict[str, Any]:
    """Compile ``source_path`` and publish a bundle directory (never overwrites an existing one)."""
    return _call("ifab_core_write_bundle", str(source_path), checkpoint_dir or "", str(out_dir), str(_build.KERNEL_DIR),
                 json.dumps(options))


def interpret(source: str, checkpoint_dir: str, tokens: List[int], steps: int = 0, logits: bool = False,
              all_logits: bool = False, watch: Optional[List[str]] = None) -> Dict[str, Any]:
    """Run the CPU oracle: feed ``tokens`` then decode ``steps`` greedy tokens. ``all_logits`` also returns the
    f32 logits after every fed token (``prompt_logits``); ``watch`` names graph nodes whose values are returned after every
    fed token (``watched``: one ``{name: value}`` object per token)."""
    return _call("ifab_core_interpret", source, str(checkpoint_dir),
                 json.dumps({"tokens": tokens, "steps": steps, "logits": logits, "all_logits": all_logits, "watch": watch or []}))


def read_init_plan(path: str) -> Dict[str, Any]:
    return _call("ifab_core_read_init_plan", str(path))


def validate_bundle(bundle_dir: str) -> Dict[str, Any]:
    """Engine-side contract check of a bundle: kernel contracts of the program, binding contracts of every rank's
    initialization plan. Raises :class:`CompileError` naming the instruction or parameter that breaks a rule."""
    return _call("ifab_core_validate_bundle", str(bundle_dir))


def read_program(path: str) -> Dict[str, Any]:
    return _call("ifab_core_read_program", str(path))


def cli(*args: str) -> subprocess.CompletedProcess:
    """Run the ``ifab`` command line tool."""
    _build.build_core()
    return subprocess.run([str(_build.CLI_BIN), *args], capture_output=True, text=True)
