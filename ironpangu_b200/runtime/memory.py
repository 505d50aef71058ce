"""Start-up memory options and the staged memory profile of an engine.

``StartupOptions`` validates the serving knobs that size device state (context, sequence slots, step budget, share of
the device the engine may use) and turns them into a byte budget. ``MemoryProfile`` records device-memory snapshots at
named start-up stages (``weights`` / ``state`` / ``workspace`` / ``graphs`` ...) and serialises them as JSON, including
the stage at which a start-up failed, so that an out-of-budget configuration is reported with numbers instead of an
allocator error. The probe is injectable, which keeps the logic testable without a device.
Reference: native memory options and profile (inferfabric-native/src/memory.rs:6-207).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, List, Optional, Tuple


@dataclass
class StartupOptions:
    max_model_len: int = 2048
    max_num_seqs: int = 4
    max_num_batched_tokens: int = 8
    gpu_memory_utilization: float = 0.9
    memory_profile: Optional[str] = None      # path of the JSON profile to write
    profile_only: bool = False                # stop after profiling start-up (no serving)

    def validate(self) -> "StartupOptions":
        if not 1 <= self.max_model_len <= 1 << 20:
            raise ValueError("max_model_len must be in [1, 1048576]")
        if not 1 <= self.max_num_seqs <= 64:
            raise ValueError("max_num_seqs must be in [1, 64]")
        if not 1 <= self.max_num_batched_tokens <= 65536:
            raise ValueError("max_num_batched_tokens must be in [1, 65536]")
        if not 0.05 <= self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in [0.05, 1.0]")
        if self.profile_only and not self.memory_profile:
            raise ValueError("profile_only needs memory_profile (where to write the profile)")
        return self

    def budget_bytes(self, total_bytes: int) -> int:
        return int(total_bytes * self.gpu_memory_utilization)


def cuda_probe() -> Tuple[int, int]:
    """(free, total) bytes of the current CUDA device."""
    import torch

    return torch.cuda.mem_get_info()


@dataclass
class Stage:
    name: str
    used_bytes: int
    delta_bytes: int
    note: str = ""


@dataclass
class MemoryProfile:
    total_bytes: int
    budget_bytes: int
    baseline_used_bytes: int
    stages: List[Stage] = field(default_factory=list)
    failed_stage: Optional[str] = None
    failure: Optional[str] = None

    @staticmethod
    def start(options: StartupOptions, probe: Callable[[], Tuple[int, int]] = cuda_probe) -> "Recorder":
        return Recorder(options, probe)

    def to_json(self) -> str:
        d = asdict(self)
        d["headroom_bytes"] = self.budget_bytes - (self.stages[-1].used_bytes if self.stages else self.baseline_used_bytes)
        return json.dumps(d, indent=1)


class Recorder:
    """Context manager style recorder: ``rec.stage("weights")`` after each start-up step; raises when a stage lands over the
    budget (the profile then names the stage), ``rec.finish()`` writes the JSON when a path was configured."""

    def __init__(self, options: StartupOptions, probe: Callable[[], Tuple[int, int]]):
        self.options, self.probe = options.validate(), probe
        free, total = probe()
        self.profile = MemoryProfile(total, options.budget_bytes(total), total - free)

    def stage(self, name: str, note: str = "") -> Stage:
        free, total = self.probe()
        used = total - free
        prev = self.profile.stages[-1].used_bytes if self.profile.stages else self.profile.baseline_used_bytes
        st = Stage(name, used, used - prev, note)
        self.profile.stages.append(st)
        if used > self.profile.budget_bytes:
            self.fail(name, f"{used} bytes in use after '{name}' exceed the budget of {self.profile.budget_bytes} "
                            f"({self.options.gpu_memory_utilization:.2f} of {total})")
            raise MemoryError(self.profile.failure)
        return st

    def fail(self, stage: str, why: str) -> None:
        self.profile.failed_stage, self.profile.failure = stage, why
        self.finish()

    def finish(self) -> MemoryProfile:
        if self.options.memory_profile:
            with open(self.options.memory_profile, "w") as f:
                f.write(self.profile.to_json())
        return self.profile

    def summary(self) -> Dict[str, int]:
        return {s.name: s.delta_bytes for s in self.profile.stages}
