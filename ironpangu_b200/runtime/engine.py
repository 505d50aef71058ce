"""Single-sequence generation engine: the public call path a user makes (``prefill`` / ``step`` /
``generate``) on top of a per-rank decoder and its captured CUDA graphs.

Each ``step`` uploads the step's control inputs (token id, position) from pinned host memory, replays
the decode graph and reads the sampled token back - the same host/device contract as the reference's
``set_input_rows`` -> graph replay -> ``emit`` (native/src/token_executor.h:1323-1448). Activations
never cross the host boundary.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .transfers import TransferAudit


class DecodeEngine:
    def __init__(self, decoder, chunk: Optional[int] = None, prefill=None):
        """``prefill``: optional tensor-core prefill object (``models.mla_moe_prefill.MlaMoePrefill``) with
        ``forward(tokens, pos0, slot)`` and ``M`` (rows per chunk); without it prompts go through the decode kernels in
        chunks of ``chunk`` rows."""
        self.dec = decoder
        self.prefill_path = prefill
        self.chunk = chunk or decoder.T
        self.pos = 0
        self._ctl_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._ctl_dev = torch.zeros(2, dtype=torch.int32, device=decoder.tokens.device)
        self._out_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._graph = None
        self._feedback_graph = None
        # decoders whose attention has two forms (one fused launch for short contexts, split-KV kernels for long ones) get one
        # graph per form; the engine knows the position on the host and replays the matching one
        self._graphs = {}
        self._feedback_graphs = {}
        self.transfers = TransferAudit()      # every host <-> device copy of this engine, by role
        self.h2d_bytes_per_step = 8
        self.d2h_bytes_per_step = 4

    # -- graphs ------------------------------------------------------------------------------------
    def _variant(self, last_pos: int):
        d = self.dec
        if getattr(d, "can_fuse_head", False) and getattr(d, "fused_auto", False):
            return last_pos < d.fused_ctx_limit
        return None

    def _select(self, table, variant, capture):
        d = self.dec
        if variant not in table:
            if variant is not None:
                d.fuse_override = variant
            capture()
            table[variant] = self._graph if table is self._graphs else self._feedback_graph
            if variant is not None:
                d.fuse_override = None
        return table[variant]

    def _capture(self):
        d = self.dec
        d.tokens[:1].copy_(self._ctl_dev[0:1])
        d.positions[:1].copy_(self._ctl_dev[1:2])
        d.forward(1)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            d.tokens[:1].copy_(self._ctl_dev[0:1])
            d.positions[:1].copy_(self._ctl_dev[1:2])
            d.forward(1)
        self._graph = g

    def _capture_feedback(self):
        d = self.dec
        d.forward(1)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            if hasattr(d, "forward_feedback"):
                d.forward_feedback(1)
            else:
                d.forward(1)
                d.tokens[:1].copy_(d.next_ids[:1])
                d.positions[:1].add_(1)
        self._feedback_graph = g

    # -- public API --------------------------------------------------------------------------------
    def reset(self) -> None:
        self.pos = 0

    def prefill(self, tokens: List[int]) -> int:
        """Run the prompt through the model in chunks; returns the greedy token after the last prompt token."""
        d = self.dec
        n = len(tokens)
        host = torch.tensor(tokens, dtype=torch.int32).pin_memory()
        last = None
        if self.prefill_path is not None:
            pp = self.prefill_path
            dev_tokens = host.to(d.tokens.device, non_blocking=True)
            for s in range(0, n, pp.M):
                last = pp.forward(dev_tokens[s:s + pp.M], self.pos + s, 0)
            self.pos += n
            self._out_host.copy_(last)
            return int(self._out_host[0])
        for s in range(0, n, self.chunk):
            m = min(self.chunk, n - s)
            d.tokens[:m].copy_(host[s:s + m], non_blocking=True)
            d.positions[:m].copy_(torch.arange(self.pos + s, self.pos + s + m, dtype=torch.int32), non_blocking=False)
            d.slots[:m].zero_()
            d.forward(m)
            last = d.next_ids[m - 1:m]
        self.pos += n
        self._out_host.copy_(last)
        return int(self._out_host[0])

    def step(self, token: int) -> int:
        """One decode step through the captured graph: H2D control inputs, replay, D2H sampled token."""
        self._ctl_host[0] = token
        self._ctl_host[1] = self.pos
        with self.transfers.scope("control_input"):
            self.transfers.h2d(self._ctl_dev, self._ctl_host)
        # a capture's warm-up run executes this very step (same token, same position), never a stale one
        self._graph = self._select(self._graphs, self._variant(self.pos), self._capture)
        self._graph.replay()
        with self.transfers.scope("request_output"):
            self.transfers.d2h(self._out_host, self.dec.next_ids[:1])
        torch.cuda.current_stream().synchronize()
        self.pos += 1
        return int(self._out_host[0])

    def generate(self, prompt: List[int], max_new_tokens: int, eos: int = -1) -> List[int]:
        self.reset()
        tok = self.prefill(prompt)
        out = [tok]
        while len(out) < max_new_tokens and tok != eos:
            tok = self.step(tok)
            out.append(tok)
        return out

    def run_device_loop(self, first_token: Optional[int], steps: int) -> None:
        """Decode ``steps`` tokens with the sampled token fed back on the device (no host round trips)."""
        d = self.dec
        if first_token is not None:
            d.tokens[:1].fill_(first_token)
            d.positions[:1].fill_(self.pos)
            d.slots[:1].zero_()
        # warm-up of a capture = the step about to be replayed (same inputs), so it changes no state
        self._feedback_graph = self._select(self._feedback_graphs, self._variant(self.pos + steps - 1), self._capture_feedback)
        for _ in range(steps):
            self._feedback_graph.replay()
        self.pos += steps
