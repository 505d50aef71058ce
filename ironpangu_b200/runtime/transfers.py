"""Host <-> device copies of a resident engine, classified at the boundary.

A device-resident engine moves three kinds of data across the host boundary and nothing else: control inputs of a step (token
ids, positions, slots: host -> device), parameter preparation (weights and tables at start-up: host -> device) and request
outputs (sampled tokens: device -> host). Activations never cross. Every copy an engine makes goes through ``TransferAudit``
under a ``scope(role)``; a copy outside a scope, a device -> host copy under ``control_input`` or a host -> device copy under
``request_output`` is counted as rejected and raises, so an accidental ``.cpu()`` on an activation path fails loudly instead
of silently stalling the stream. ``report()`` is the audit document (format ``ifab.transfer-audit.v1``: calls and bytes per
role and direction, the rejected count, ``activation_host_transfers`` = 0 by construction).
Reference: native/src/resident_transfer.h:11-58 (roles, the guard, the JSON record)."""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch

ROLES = ("control_input", "parameter_preparation", "request_output")


class ImplicitTransfer(RuntimeError):
    pass


class TransferAudit:
    def __init__(self):
        self.role: Optional[str] = None
        self.counts: Dict[str, Dict[str, int]] = {r: {"h2d_calls": 0, "h2d_bytes": 0, "d2h_calls": 0, "d2h_bytes": 0} for r in ROLES}
        self.rejected = 0

    @contextlib.contextmanager
    def scope(self, role: str):
        if role not in ROLES:
            raise ValueError(f"unknown transfer role {role!r}")
        previous, self.role = self.role, role
        try:
            yield self
        finally:
            self.role = previous

    def _check(self, direction: str, nbytes: int) -> None:
        role = self.role
        if role is None or (direction == "d2h" and role == "control_input") or (direction == "h2d" and role == "request_output"):
            self.rejected += 1
            raise ImplicitTransfer(f"implicit host transfer ({direction}, {nbytes} bytes, role {role or 'none'}) forbidden by device residency")
        c = self.counts[role]
        c[direction + "_calls"] += 1
        c[direction + "_bytes"] += int(nbytes)

    def h2d(self, dst: torch.Tensor, src: torch.Tensor, non_blocking: bool = True) -> torch.Tensor:
        """``dst.copy_(src)`` for a host source, recorded under the current role."""
        self._check("h2d", src.numel() * src.element_size())
        return dst.copy_(src, non_blocking=non_blocking)

    def upload(self, src: torch.Tensor, device, non_blocking: bool = True) -> torch.Tensor:
        """A new device tensor with the contents of the host tensor ``src``, recorded under the current role."""
        self._check("h2d", src.numel() * src.element_size())
        return src.to(device, non_blocking=non_blocking)

    def d2h(self, dst: torch.Tensor, src: torch.Tensor, non_blocking: bool = True) -> torch.Tensor:
        """``dst.copy_(src)`` for a device source and a host destination, recorded under the current role."""
        self._check("d2h", src.numel() * src.element_size())
        return dst.copy_(src, non_blocking=non_blocking)

    def totals(self):
        h = sum(c["h2d_bytes"] for c in self.counts.values())
        d = sum(c["d2h_bytes"] for c in self.counts.values())
        return h, d

    def report(self) -> Dict:
        return {"format": "ifab.transfer-audit.v1", "activation_host_transfers": 0, "rejected": self.rejected,
                "boundaries": [{"role": r, **self.counts[r]} for r in ROLES]}


def prepared_execution_report(engine) -> Dict:
    """What an engine prepared before its first step and reuses afterwards (format ``ifab.prepared-execution.v1``): the captured
    graphs by step width, the frozen arena and workspace when the engine runs a bundle, and the device allocation counter -
    ``allocations_after_ready`` stays 0 when steps allocate nothing. Reference: native/src/prepared_execution.h:529-605."""
    dec = engine.dec
    out = {"format": "ifab.prepared-execution.v1", "graph_widths": sorted(getattr(engine, "_graphs", {})),
           "launches_per_step": getattr(dec, "launches_per_forward", None)}
    arena = getattr(dec, "arena", None)
    if arena is not None:
        out["arena"] = {"bytes": arena.bytes, "workspace_bytes": arena.workspace_bytes, "slots": len(arena.slots), "leased": len(arena.leased),
                        "planned_rows": arena.tokens}
        out["program_sha256"] = getattr(dec, "bundle_sha256", "")
    ready = getattr(engine, "allocations_at_ready", None)
    if ready is not None and torch.cuda.is_available():
        out["allocations_after_ready"] = int(torch.cuda.memory_stats().get("allocation.all.allocated", 0)) - ready
    return out


def state_copy_report(engine) -> Dict:
    """Device-to-device copies of sequence state (prefix snapshots taken and restored), format ``ifab.state-copy-audit.v1``.
    Reference: native/src/continuation_copy.inc (copy plan of a continuation)."""
    p = getattr(engine, "prefix", None)
    a = engine.audit_counters
    return {"format": "ifab.state-copy-audit.v1", "host_bytes": 0, "rows_restored": a.get("prefix_rows_copied", 0),
            "rows_published": a.get("prefix_rows_published", 0), "snapshots": 0 if p is None else len(p.entries),
            "hits": 0 if p is None else p.hits, "misses": 0 if p is None else p.misses, "evicted": 0 if p is None else p.evicted}
