"""Typed runtime options: one struct, parsed once, recorded with every run.

The model source's ``parallel`` block is the real configuration and the command line carries the serving limits; what is
left are the experimental gates an operator flips per process. They live in one dataclass, ``RuntimeOptions``, filled from
``IFAB_<NAME>`` environment variables and ``--set name=value`` arguments (the latter win), with typed parsing, range checks
and an error for names nobody knows - a misspelt gate must not silently do nothing. ``to_json`` is what engines record in
their audit so that a measurement can be reproduced.
Reference: the environment gates of the native executors (INFERFABRIC_DECODE_GRAPH, ..._EXPERIMENTAL_BULK_COLLECTIVES,
..._TRANSFER_AUDIT_DIR, ... ; native/src/program_engine.cpp:48-62, crates/inferfabric-compiler/src/token.rs:380-381).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from typing import Dict, Iterable, List, Mapping, Optional


@dataclass
class RuntimeOptions:
    decode_graph: bool = True            # replay CUDA graphs for decode launch groups (off: every kernel launched from the host)
    pdl: bool = True                     # programmatic dependent launch between the kernels of a step
    fused_head: Optional[bool] = None    # cluster-per-head attention kernel: None = by context limit, True / False = forced
    kv_int8: bool = False                # packed int8 latent KV cache
    expert_fp8: bool = False             # block-scaled fp8 expert weights
    prefill_chunk: int = 0               # rows per tensor-core prompt call (0 = prompts through the decode kernels)
    prefix_cache_slots: int = 0          # device snapshots kept by the prefix cache
    spin_limit: int = 4_000_000          # polls a kernel waits for a peer before it reports a timeout
    bulk_collectives: bool = True        # fused GEMM + all-reduce for prompt chunks (off: GEMM, then pull all-reduce)
    sequence_parallel: bool = False      # dense prompt chunks keep the residual stream sharded by rows (all-gather GEMM / GEMM + reduce-scatter)
    rank_agreement: str = "deferred"     # ranks of an engine worker compare the outcome of every request: strict (before rank 0 answers), deferred (overlapped with the next request), off
    audit_dir: str = ""                  # where engines write their audit JSON at shutdown ("" = nowhere)
    trace_dir: str = ""                  # where step traces go ("" = off)

    ENV_PREFIX = "IFAB_"

    # -- parsing ---------------------------------------------------------------------------------------------------------
    @classmethod
    def names(cls) -> List[str]:
        return [f.name for f in fields(cls)]

    @staticmethod
    def _parse(name: str, kind, text: str):
        t = text.strip()
        if kind in (bool, Optional[bool], "bool", "Optional[bool]"):
            low = t.lower()
            if low in ("1", "true", "yes", "on"):
                return True
            if low in ("0", "false", "no", "off"):
                return False
            if low in ("", "auto", "none") and kind in (Optional[bool], "Optional[bool]"):
                return None
            raise ValueError(f"option {name}: '{text}' is not a boolean")
        if kind in (int, "int"):
            try:
                return int(t, 0)
            except ValueError:
                raise ValueError(f"option {name}: '{text}' is not an integer") from None
        return t

    def set(self, name: str, text: str) -> None:
        key = name.strip().lower().replace("-", "_")
        for f in fields(self):
            if f.name == key:
                setattr(self, key, self._parse(key, f.type, text))
                return
        raise KeyError(f"unknown runtime option '{name}' (known: {', '.join(self.names())})")

    @classmethod
    def from_env(cls, environ: Mapping[str, str], sets: Iterable[str] = ()) -> "RuntimeOptions":
        """Defaults, then ``IFAB_<NAME>`` variables, then ``name=value`` strings; unknown ``--set`` names are errors, unknown
        ``IFAB_*`` variables that are not options (socket paths and the like) are left alone."""
        o = cls()
        known = {n.upper(): n for n in cls.names()}
        for k, v in environ.items():
            if k.startswith(cls.ENV_PREFIX) and k[len(cls.ENV_PREFIX):] in known:
                o.set(known[k[len(cls.ENV_PREFIX):]], v)
        for item in sets:
            if "=" not in item:
                raise ValueError(f"--set expects name=value, got '{item}'")
            name, value = item.split("=", 1)
            o.set(name, value)
        return o.validate()

    def validate(self) -> "RuntimeOptions":
        if not 0 <= self.prefill_chunk <= 65536:
            raise ValueError("prefill_chunk must be in [0, 65536]")
        if not 0 <= self.prefix_cache_slots <= 4096:
            raise ValueError("prefix_cache_slots must be in [0, 4096]")
        if not 1000 <= self.spin_limit <= 1 << 31:
            raise ValueError("spin_limit must be in [1000, 2^31]")
        mode = {"1": "strict", "true": "strict", "on": "strict", "yes": "strict", "0": "off", "false": "off", "no": "off"}.get(
            str(self.rank_agreement).strip().lower(), str(self.rank_agreement).strip().lower())
        if mode not in ("strict", "deferred", "off"):
            raise ValueError("rank_agreement must be strict, deferred or off")
        self.rank_agreement = mode
        if self.kv_int8 and self.fused_head:
            raise ValueError("fused_head reads bf16 cache rows: it cannot be forced together with kv_int8")
        return self

    # -- recording -------------------------------------------------------------------------------------------------------
    def to_dict(self) -> Dict:
        return asdict(self)

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True)

    def changed(self) -> Dict:
        """Only the options that differ from their defaults (what a report should print)."""
        d, base = self.to_dict(), RuntimeOptions().to_dict()
        return {k: v for k, v in d.items() if v != base[k]}
