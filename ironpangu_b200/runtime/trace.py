"""Step traces of an engine: one CSV row per scheduler step and rank, NVTX ranges around the steps for timeline tools, and a
merge of the ranks' files that shows the step time as the slowest rank saw it and the skew between ranks.

``StepTrace(dir, rank)`` is switched on by the runtime option ``trace_dir`` (``IFAB_TRACE_DIR`` / ``--set trace_dir=...``).
Every rank writes ``steps-rank<r>.csv`` with the same step numbers, so the files of a multi-rank job line up without any
communication at run time. Device time comes from a pair of CUDA events per step, read when the trace is flushed (never
inside a step: reading an event synchronises). Columns: step, host_start_ns, host_ms, device_ms, slices, rows, prompt_rows,
launch_groups, sampled_rows, h2d_bytes, d2h_bytes.
Reference: the per-operator profile directory of the native executors (INFERFABRIC_PROFILE_DIR, native/src/execution_profile.h)."""
from __future__ import annotations

import csv
import os
import time
from pathlib import Path
from typing import Dict, List, Optional

import torch

COLUMNS = ["step", "host_start_ns", "host_ms", "device_ms", "slices", "rows", "prompt_rows", "launch_groups", "sampled_rows", "h2d_bytes", "d2h_bytes"]


class StepTrace:
    def __init__(self, directory: str, rank: int = 0, use_cuda: Optional[bool] = None, flush_every: int = 256):
        self.path = Path(directory) / f"steps-rank{rank}.csv"
        os.makedirs(directory, exist_ok=True)
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.flush_every = flush_every
        self.pending: List[Dict] = []
        self.step = 0
        with open(self.path, "w", newline="") as f:
            csv.writer(f).writerow(COLUMNS)

    def begin(self, counters: Dict[str, int], slices: int) -> Dict:
        rec = {"step": self.step, "host_start_ns": time.time_ns(), "t0": time.perf_counter(), "slices": slices, "before": dict(counters)}
        if self.use_cuda:
            torch.cuda.nvtx.range_push(f"ifab.step {self.step}")
            rec["e0"], rec["e1"] = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rec["e0"].record()
        return rec

    def end(self, rec: Dict, counters: Dict[str, int]) -> None:
        if self.use_cuda:
            rec["e1"].record()
            torch.cuda.nvtx.range_pop()
        rec["host_ms"] = (time.perf_counter() - rec.pop("t0")) * 1e3
        before = rec.pop("before")
        d = lambda k: counters.get(k, 0) - before.get(k, 0)
        rec.update(rows=d("rows") + d("prefill_rows"), prompt_rows=d("prefill_rows"), launch_groups=d("launch_groups"), sampled_rows=d("sampled_rows"),
                   h2d_bytes=d("h2d_bytes"), d2h_bytes=d("d2h_bytes"))
        self.pending.append(rec)
        self.step += 1
        if len(self.pending) >= self.flush_every:
            self.flush()

    def flush(self) -> None:
        if not self.pending:
            return
        if self.use_cuda:
            torch.cuda.synchronize()
        with open(self.path, "a", newline="") as f:
            w = csv.writer(f)
            for r in self.pending:
                dev = r["e0"].elapsed_time(r["e1"]) if self.use_cuda else ""
                w.writerow([r["step"], r["host_start_ns"], f"{r['host_ms']:.4f}", f"{dev:.4f}" if dev != "" else "", r["slices"], r["rows"], r["prompt_rows"],
                            r["launch_groups"], r["sampled_rows"], r["h2d_bytes"], r["d2h_bytes"]])
        self.pending = []

    close = flush


def merge(directory: str) -> List[Dict]:
    """One record per step over all ``steps-rank*.csv`` files of ``directory``: the slowest rank's device and host time, the
    skew (slowest minus fastest device time) and the per-rank device times; steps a rank did not record are an error."""
    files = sorted(Path(directory).glob("steps-rank*.csv"), key=lambda p: int(p.stem.split("rank")[1]))
    if not files:
        raise FileNotFoundError(f"no step traces under {directory}")
    per_rank = []
    for f in files:
        with open(f, newline="") as fh:
            per_rank.append({int(r["step"]): r for r in csv.DictReader(fh)})
    steps = sorted(per_rank[0])
    out = []
    for s in steps:
        rows = []
        for i, table in enumerate(per_rank):
            if s not in table:
                raise ValueError(f"{files[i].name} has no step {s}: the ranks' traces do not line up")
            rows.append(table[s])
        dev = [float(r["device_ms"]) for r in rows if r["device_ms"] != ""]
        host = [float(r["host_ms"]) for r in rows]
        out.append({"step": s, "ranks": len(rows), "rows": int(rows[0]["rows"]), "device_ms_max": max(dev) if dev else None,
                    "device_ms_skew": (max(dev) - min(dev)) if dev else None, "host_ms_max": max(host), "device_ms_by_rank": dev})
    return out


if __name__ == "__main__":
    import json
    import sys

    print(json.dumps(merge(sys.argv[1]), indent=1))
