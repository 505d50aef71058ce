"""Engine worker: the GPU side of ``ifab-server``.

One worker process per GPU (plain ``python -m ...`` for one GPU, under ``torch.distributed.run`` for tensor /
expert parallel models). Rank 0 connects to the Unix socket in ``IFAB_ENGINE_SOCKET`` and answers the server's
newline-delimited JSON requests (``info`` / ``admit`` / ``step`` / ``release`` / ``audit`` / ``shutdown``); every
request is broadcast to the other ranks so that all of them launch the same kernels (the collectives live inside
those kernels). A ``step`` carries slices ``[resident, position, count, sample]`` of several sequences: prompt chunks
and decode rows are packed into launches of up to ``max_tokens`` rows (continuous batching); one token per sampling
slice goes back. Sequence slot ``resident`` owns the pages ``resident * max_pages ...`` of the KV cache.

Besides greedy decoding the engine samples on the device (temperature, top-k <= 64, top-p, min-p, repetition /
frequency / presence penalties, per-request seed) with the vocabulary-sharded sampling kernel, and it keeps a prefix
cache of device snapshots: when a prompt starts with tokens whose KV rows were snapshotted before, the matching
prefill chunks are served by copying those rows into the sequence's pages instead of running the model.

    IFAB_ENGINE_SOCKET=/tmp/e.sock python -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 4

Reference: the ResidentEngine trait and its packed batch path (frontend/src/program_worker.rs:22-61,279-317), the
prefix cache (native/src/prefix_cache.rs), the transfer audit (native/src/resident_transfer.h).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import socket
import sys
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .transfers import TransferAudit, prepared_execution_report, state_copy_report


def checkpoint_boundary(tokens: int, alignment: int, chunk: int) -> int:
    """The longest prefix of a ``tokens``-token prompt that may be published or restored: a whole number of cache blocks
    (``alignment``) AND of prefill chunks (``chunk``) - so a restore lands where an uninterrupted prefill would have a chunk
    boundary - and strictly shorter than the prompt, so at least one prompt token is left to run and produce logits.
    Reference: frontend/src/program_cached.rs:10-15."""
    step = alignment // math.gcd(alignment, chunk) * chunk
    return max(0, tokens - 1) // step * step


class PrefixSnapshots:
    """LRU of device snapshots keyed by (salt, token prefix), prefixes being multiples of ``block`` tokens. A snapshot is the KV
    rows of every layer for positions ``[0, n)``, cloned out of the paged cache, so it survives the release of the slot it came
    from. The salt (the deployment's namespace plus the request's ``cache_salt``) isolates tenants: a prefix is only ever
    found by requests that carry the salt it was published under."""

    def __init__(self, capacity: int, block: int, chunk: int = 0, namespace: str = ""):
        self.capacity, self.block, self.chunk, self.namespace = capacity, block, chunk or block, namespace
        self.entries: "OrderedDict[Tuple, List[torch.Tensor]]" = OrderedDict()
        self.hits = self.misses = self.published = self.evicted = 0

    def lookup(self, tokens: List[int], salt: str = "") -> Optional[Tuple[Tuple[int, ...], List[torch.Tensor]]]:
        """A stored snapshot of the same salt whose tokens start with all of ``tokens``, or None."""
        want, ns = tuple(tokens), (self.namespace, salt)
        for key in reversed(self.entries):
            if key[0] == ns and len(key[1]) >= len(want) and key[1][:len(want)] == want:
                self.entries.move_to_end(key)
                return key[1], self.entries[key]
        return None

    def publish(self, tokens: List[int], rows_of, salt: str = "") -> None:
        """``rows_of(n)`` -> list of per-layer tensors with the first ``n`` KV rows of the sequence."""
        n = checkpoint_boundary(len(tokens), self.block, self.chunk)
        if n == 0 or self.capacity == 0:
            return
        key = ((self.namespace, salt), tuple(tokens[:n]))
        if key in self.entries:
            self.entries.move_to_end(key)
            return
        self.entries[key] = rows_of(n)
        self.published += 1
        while len(self.entries) > self.capacity:
            self.entries.popitem(last=False)
            self.evicted += 1


class BatchEngine:
    """Packs the slices of one scheduler step into decoder launches; greedy or sampled tokens come from the device."""

    TOPK_CAP = 64   # candidates the sampling kernel keeps per row

    def __init__(self, decoder, model_name: str, context: int, vocab: int, eos: int = -1, greedy_only: bool = False,
                 prefix_slots: int = 0, prefill=None, token_budget: int = 0, use_graphs: bool = True, prefix_namespace: str = ""):
        """``prefill``: optional tensor-core chunk executor (``forward(tokens, pos0, slot)``, attribute ``M`` = rows per call);
        prompt slices longer than one decode launch group run through it, and the engine advertises ``M`` as its token budget."""
        self.dec, self.name, self.context, self.eos, self.vocab = decoder, model_name, context, eos, vocab
        self.residents = decoder.num_slots
        self.rows = decoder.T
        self.prefill = prefill
        # one CUDA graph per launch-group width: a decoder step is a few hundred launches, which cost more host time through
        # Python than the kernels take on the device
        self.use_graphs = use_graphs and hasattr(decoder, "capture")
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        # tokens the scheduler may hand over per step: more than one launch group (``rows``) is fine, they run back to back
        self.budget = max(self.rows, prefill.M if prefill is not None else 0, token_budget)
        self.can_sample = getattr(decoder, "logits", None) is not None
        self.greedy_only = greedy_only or not self.can_sample
        dev = decoder.tokens.device
        # one pinned control block per launch group of a step: the copies are asynchronous and a step synchronises once
        self._host = torch.zeros((self.budget + self.rows - 1) // self.rows + 1, 3, self.rows, dtype=torch.int32).pin_memory()
        self._out = torch.zeros(self.rows, dtype=torch.int32).pin_memory()
        self.next_pos = [0] * self.residents
        self.history: List[List[int]] = [[] for _ in range(self.residents)]
        self.sampling: List[Dict] = [{} for _ in range(self.residents)]
        self.prompt_done = [False] * self.residents
        self.salt = [""] * self.residents
        R = self.residents
        if self.can_sample:
            vl = decoder.logits.shape[1]
            self.inv_temp = torch.ones(R, device=dev)
            self.top_p = torch.ones(R, device=dev)
            self.min_p = torch.zeros(R, device=dev)
            self.pen = torch.tensor([[1.0, 0.0, 0.0]] * R, device=dev)
            self.seeds = torch.zeros(R, dtype=torch.int64, device=dev)
            self.counters = torch.zeros(R, dtype=torch.int64, device=dev)
            self.counts = torch.zeros(R, vl, dtype=torch.int16, device=dev)
            self.vocab_offset = decoder.rank * vl
        # snapshots end where the scheduler's prompt slices end (it hands out slices of `budget` tokens): other lengths could
        # never be restored whole
        self.prefix = (PrefixSnapshots(prefix_slots, self.rows, chunk=self.budget, namespace=prefix_namespace)
                       if prefix_slots > 0 and hasattr(decoder, "caches") else None)
        self.transfers = TransferAudit()
        self.trace = None                     # runtime.trace.StepTrace when the runtime option trace_dir is set
        self.allocations_at_ready: Optional[int] = None      # set once the engine has served its first step of every width it will see
        self.audit_counters = {"steps": 0, "launch_groups": 0, "rows": 0, "h2d_bytes": 0, "d2h_bytes": 0, "prefix_rows_copied": 0,
                               "sampled_rows": 0, "prefill_chunks": 0, "prefill_rows": 0}

    # -- contract ------------------------------------------------------------------------------------
    def info(self) -> Dict:
        return {"model": self.name, "residents": self.residents, "token_budget": self.budget, "chunk": self.budget,
                "context": self.context, "vocab": self.vocab, "eos": max(self.eos, 0), "has_eos": self.eos >= 0,
                "world": self.dec.world, "greedy_only": self.greedy_only}

    def audit(self) -> Dict:
        a = {"format": "ifab.engine-audit.v1", **self.audit_counters}
        if self.prefix is not None:
            a.update({"prefix_hits": self.prefix.hits, "prefix_misses": self.prefix.misses, "prefix_published": self.prefix.published,
                      "prefix_evicted": self.prefix.evicted, "prefix_entries": len(self.prefix.entries)})
        a["fabric_status"] = self.dec.fabric.status()
        a["transfers"] = self.transfers.report()
        a["prepared_execution"] = prepared_execution_report(self)
        a["state_copies"] = state_copy_report(self)
        opts = getattr(self, "runtime_options", None)
        if opts is not None:
            a["runtime_options"] = opts.to_dict()
        return a

    def admit(self, resident: int, sampling: Dict, reserve: int) -> None:
        if not 0 <= resident < self.residents:
            raise ValueError("resident out of range")
        if reserve > self.context:
            raise OverflowError("request does not fit the sequence slot")
        temp, top_k = float(sampling.get("temperature", 0.0)), int(sampling.get("top_k", 0))
        greedy = temp <= 0.0 or top_k == 1
        if not greedy and self.greedy_only:
            raise ValueError("this engine samples greedily only")
        if top_k > self.TOPK_CAP:
            raise ValueError(f"top_k above {self.TOPK_CAP} is not supported")
        self.next_pos[resident] = 0
        self.history[resident] = []
        self.prompt_done[resident] = False
        self.sampling[resident] = {"greedy": greedy, "top_k": top_k}
        self.salt[resident] = str(sampling.get("cache_salt", ""))
        if self.can_sample:
            self.inv_temp[resident] = 1.0 / temp if temp > 0 else 1.0
            self.top_p[resident] = float(sampling.get("top_p", 1.0))
            self.min_p[resident] = float(sampling.get("min_p", 0.0))
            self.pen[resident] = torch.tensor([float(sampling.get("repetition_penalty", 1.0)), float(sampling.get("frequency_penalty", 0.0)),
                                               float(sampling.get("presence_penalty", 0.0))], device=self.pen.device)
            seed = sampling.get("seed")
            self.seeds[resident] = int(seed) if seed is not None else (resident + 1) * 0x9E3779B1
            self.counters[resident] = 0
            self.counts[resident].zero_()

    def release(self, resident: int) -> None:
        self.next_pos[resident] = 0
        self.history[resident] = []

    # -- prefix snapshots ----------------------------------------------------------------------------
    def _kv_rows(self, resident: int, lo: int, hi: int) -> torch.Tensor:
        """Flat row indices of positions [lo, hi) of a resident in the paged cache."""
        d = self.dec
        pt = d.caches[0].shape[1]
        pos = torch.arange(lo, hi, device=d.tokens.device)
        pages = d.page_table[resident].long()[pos // pt]
        return pages * pt + pos % pt

    def _snapshot(self, resident: int, n: int) -> List[torch.Tensor]:
        rows = self._kv_rows(resident, 0, n)
        self.audit_counters["prefix_rows_published"] = self.audit_counters.get("prefix_rows_published", 0) + n * len(self.dec.caches)
        return [c.view(-1, c.shape[-1])[rows].clone() for c in self.dec.caches]

    def _restore(self, resident: int, snap: List[torch.Tensor], lo: int, hi: int) -> None:
        rows = self._kv_rows(resident, lo, hi)
        for c, s in zip(self.dec.caches, snap):
            c.view(-1, c.shape[-1])[rows] = s[lo:hi]
        self.audit_counters["prefix_rows_copied"] += (hi - lo) * len(snap)

    # -- one scheduler step ----------------------------------------------------------------------------
    def step(self, slices: List[List[int]], tokens: List[int]) -> List[int]:
        """One scheduler step; with a step trace switched on (runtime option ``trace_dir``) the step is timed and recorded."""
        if self.trace is None:
            return self._step(slices, tokens)
        rec = self.trace.begin(self.audit_counters, len(slices))
        try:
            return self._step(slices, tokens)
        finally:
            self.trace.end(rec, self.audit_counters)

    def _step(self, slices: List[List[int]], tokens: List[int]) -> List[int]:
        d = self.dec
        rows = []                     # (token, position, slot, slice index or -1 when the row does not sample)
        long_slices = []              # prompt slices that go through the matrix-matrix prefill path
        off = 0
        for i, (resident, position, count, sample) in enumerate(slices):
            if position != self.next_pos[resident]:
                raise RuntimeError(f"slice of resident {resident} starts at {position}, expected {self.next_pos[resident]}")
            if position + count > self.context:
                raise RuntimeError("slice runs past the context")
            toks = tokens[off:off + count]
            hist = self.history[resident]
            hist.extend(toks)
            off += count
            self.next_pos[resident] = position + count
            # a whole non-sampling prefill chunk that a snapshot covers is served by a copy
            if self.prefix is not None and not sample and position + count == len(hist):
                hit = self.prefix.lookup(hist, self.salt[resident])
                if hit is not None and len(hit[0]) >= position + count:
                    self._restore(resident, hit[1], position, position + count)
                    self.prefix.hits += 1
                    if self.can_sample:
                        # the restored tokens count towards the penalties exactly as if they had been run
                        local = torch.tensor(toks, dtype=torch.long, device=self.counts.device) - self.vocab_offset
                        ok = (local >= 0) & (local < self.counts.shape[1])
                        self.counts[resident, local[ok]] += 1
                    continue
                self.prefix.misses += 1
            if self.prefill is not None and count > self.rows:
                long_slices.append((i, resident, position, toks, sample))
                continue
            for k in range(count):
                rows.append((toks[k], position + k, resident, i if (sample and k == count - 1) else -1))
        out = [0] * len(slices)
        pending = []                  # (slice indices, device ids) of every launch group, read back once per step
        # prompt chunks: matrix-matrix path, one call per chunk; the row after the chunk's last token is the one that samples
        for i, resident, position, toks, sample in long_slices:
            for c0 in range(0, len(toks), self.prefill.M):
                chunk = toks[c0:c0 + self.prefill.M]
                host = torch.tensor(chunk, dtype=torch.int32).pin_memory()
                with self.transfers.scope("control_input"):
                    dev_toks = self.transfers.upload(host, d.tokens.device)
                self.prefill.forward(dev_toks, position + c0, resident)
                if self.can_sample:
                    local = dev_toks.long() - self.vocab_offset
                    ok = (local >= 0) & (local < self.counts.shape[1])
                    self.counts[resident, local[ok]] += 1
                self.audit_counters["prefill_chunks"] += 1
                self.audit_counters["prefill_rows"] += len(chunk)
                self.audit_counters["h2d_bytes"] += 4 * len(chunk)
            if sample:
                d.slots[:1].fill_(resident)
                pending += self._emit([(toks[-1], position + len(toks) - 1, resident, i)], 1, counted=True)
        batched = (self.prefill is not None and hasattr(self.prefill, "forward_rows") and self.can_sample and
                   len(rows) > getattr(self.prefill, "batch_threshold", self.rows))
        if batched:
            # more rows than one decode launch group: all of them as one matrix-matrix pass per `M` rows
            for r0 in range(0, len(rows), self.prefill.M):
                pending += self._run_rows_batched(rows[r0:r0 + self.prefill.M])
            rows = []
        for r0 in range(0, len(rows), self.rows):
            part = rows[r0:r0 + self.rows]
            n = len(part)
            hb = self._host[(r0 // self.rows) % self._host.shape[0]]
            if r0 // self.rows >= self._host.shape[0]:
                torch.cuda.current_stream().synchronize()     # more groups than control blocks: drain before reuse
            for j, (tok, pos, slot, _) in enumerate(part):
                hb[0, j], hb[1, j], hb[2, j] = tok, pos, slot
            with self.transfers.scope("control_input") as tr:
                tr.h2d(d.tokens[:n], hb[0, :n])
                tr.h2d(d.positions[:n], hb[1, :n])
                tr.h2d(d.slots[:n], hb[2, :n])
            self._run_group(n)
            pending += self._emit(part, n)
            self.audit_counters["launch_groups"] += 1
            self.audit_counters["rows"] += n
            self.audit_counters["h2d_bytes"] += 12 * n
        self._collect(pending, out)
        # publish the prompt of every sequence that just finished its prefill
        if self.prefix is not None:
            for resident, position, count, sample in slices:
                if sample and not self.prompt_done[resident]:      # the first sampling slice of a sequence ends its prompt
                    self.prompt_done[resident] = True
                    self.prefix.publish(list(self.history[resident]), lambda n, r=resident: self._snapshot(r, n), self.salt[resident])
        self.audit_counters["steps"] += 1
        if d.fabric.status() != 0:
            raise RuntimeError(f"kernel status word = {d.fabric.status()}")
        return out

    def _run_rows_batched(self, part):
        """Rows of many sequences (one decode row each, short prompt pieces) through the matrix-matrix path of the prefill
        executor; the sampling rows get their logits from one GEMM and their tokens from the sampling kernel (greedy rows as
        a draw at vanishing temperature). Returns ``[(slice indices, device ids)]`` like :meth:`_emit`."""
        from ..ops import decode as K

        d, n = self.dec, len(part)
        host = torch.tensor([[r[0] for r in part], [r[1] for r in part], [r[2] for r in part]], dtype=torch.int32).pin_memory()
        with self.transfers.scope("control_input"):
            dev = self.transfers.upload(host, d.tokens.device)
        pick = [j for j, r in enumerate(part) if r[3] >= 0]
        sel = torch.tensor(pick or [n - 1], device=dev.device)
        logits = self.prefill.forward_rows(dev[0], dev[1], dev[2], sel)
        slots = dev[2].long()
        local = dev[0].long() - self.vocab_offset
        ok = (local >= 0) & (local < self.counts.shape[1])
        self.counts[slots[ok], local[ok]] += 1
        self.audit_counters["launch_groups"] += 1
        self.audit_counters["rows"] += n
        self.audit_counters["batched_rows"] = self.audit_counters.get("batched_rows", 0) + n
        self.audit_counters["h2d_bytes"] += 12 * n
        if not pick:
            return []
        out = []
        for c0 in range(0, len(pick), 64):            # the sampling kernel takes up to 64 rows a call
            sub = pick[c0:c0 + 64]
            rs = slots[sel[c0:c0 + 64]]
            greedy = torch.tensor([self.sampling[part[j][2]].get("greedy", True) for j in sub], device=dev.device)
            inv_t = torch.where(greedy, torch.full_like(self.inv_temp[rs], 1e4), self.inv_temp[rs]).contiguous()
            top_p = torch.where(greedy, torch.ones_like(self.top_p[rs]), self.top_p[rs]).contiguous()
            min_p = torch.where(greedy, torch.zeros_like(self.min_p[rs]), self.min_p[rs]).contiguous()
            # every row samples with its own request's k (greedy rows: 1), whatever else shares the launch
            k_rows = [1 if self.sampling[part[j][2]].get("greedy", True) else (self.sampling[part[j][2]]["top_k"] or self.TOPK_CAP) for j in sub]
            counters = self.counters[rs].contiguous()
            ids = K.sample_topk(logits[c0:c0 + 64].contiguous(), d.fabric, top_k=max(k_rows), inv_temperature=inv_t, top_p=top_p,
                                top_k_rows=torch.tensor(k_rows, dtype=torch.int32, device=dev.device),
                                min_p=min_p, counts=self.counts[rs].contiguous(), penalties=self.pen[rs].contiguous(),
                                seeds=self.seeds[rs].contiguous(), counters=counters, vocab_offset=self.vocab_offset)
            self.counters[rs] = counters
            self.audit_counters["sampled_rows"] += sum(1 for j in sub if not self.sampling[part[j][2]].get("greedy", True))
            out.append(([part[j][3] for j in sub], ids))
        return out

    def _run_group(self, n: int) -> None:
        """Decoder forward over the ``n`` rows staged in its static input buffers: eager the first time a width is seen
        (that run also warms the capture), a graph replay afterwards."""
        d = self.dec
        if not self.use_graphs:
            d.forward(n)
            return
        g = self._graphs.get(n)
        if g is not None:
            g.replay()
            return
        d.forward(n)                              # the real run of this step
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):                 # capture only records: it does not execute
            d.forward(n)
        self._graphs[n] = g
        self.audit_counters["graphs_captured"] = len(self._graphs)

    def _emit(self, part, n: int, counted: bool = False):
        """Tokens of the sampling rows among the ``n`` rows the decoder just produced (``next_ids`` / ``logits`` rows 0..n-1,
        ``slots`` rows 0..n-1 valid): greedy ids as they are, sampled rows through the sampling kernel. Returns at most one
        ``(slice indices, device ids)`` pair; nothing is copied to the host here."""
        d = self.dec
        ids = d.next_ids[:n]
        if self.can_sample:
            slots = d.slots[:n].long()
            if not counted:
                local = (d.tokens[:n].long() - self.vocab_offset)      # count the fed tokens (repetition / frequency / presence)
                ok = (local >= 0) & (local < self.counts.shape[1])
                self.counts[slots[ok], local[ok]] += 1                  # a token repeated inside one chunk counts once
            hot = [j for j, (_, _, slot, si) in enumerate(part) if si >= 0 and not self.sampling[slot].get("greedy", True)]
            if hot:
                from ..ops import decode as K
                sel = torch.tensor(hot, device=slots.device)
                rs = slots[sel]
                k_rows = [self.sampling[part[j][2]]["top_k"] or self.TOPK_CAP for j in hot]     # each row keeps its own request's k
                counters = self.counters[rs].contiguous()
                sampled = K.sample_topk(d.logits[:n][sel].contiguous(), d.fabric, top_k=max(k_rows), inv_temperature=self.inv_temp[rs].contiguous(),
                                        top_k_rows=torch.tensor(k_rows, dtype=torch.int32, device=slots.device),
                                        top_p=self.top_p[rs].contiguous(), min_p=self.min_p[rs].contiguous(),
                                        counts=self.counts[rs].contiguous(), penalties=self.pen[rs].contiguous(),
                                        seeds=self.seeds[rs].contiguous(), counters=counters, vocab_offset=self.vocab_offset)
                self.counters[rs] = counters
                ids = ids.clone()
                ids[sel] = sampled
                self.audit_counters["sampled_rows"] += len(hot)
        pick = [j for j, (_, _, _, si) in enumerate(part) if si >= 0]
        if not pick:
            return []
        sel_ids = ids[torch.tensor(pick, device=ids.device)] if len(pick) != n else ids.clone()
        return [([part[j][3] for j in pick], sel_ids)]

    def _collect(self, pending, out: List[int]) -> None:
        """One device-to-host copy and one synchronisation for all launch groups of a step."""
        if not pending:
            return
        dev = torch.cat([ids for _, ids in pending])
        if dev.numel() > self._out.numel():
            self._out = torch.zeros(dev.numel(), dtype=torch.int32).pin_memory()
        host = self._out[:dev.numel()]
        with self.transfers.scope("request_output"):
            self.transfers.d2h(host, dev)
        torch.cuda.current_stream().synchronize()
        k = 0
        for slice_ids, ids in pending:
            for si in slice_ids:
                out[si] = int(host[k])
                k += 1
        self.audit_counters["d2h_bytes"] += 4 * dev.numel()


def build_engine(args, rank: int, world: int, rec=None) -> BatchEngine:
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric

    dev = torch.device("cuda", torch.cuda.current_device())
    ro = getattr(args, "runtime_options", None)
    fab = Fabric(rank, world, spin_limit=ro.spin_limit) if ro is not None else Fabric(rank, world)
    mark = (lambda name, note="": rec.stage(name, note)) if rec is not None else (lambda name, note="": None)
    mark("fabric", "symmetric-memory block and peer mappings")
    if args.bundle:
        # a compiled bundle + its checkpoint: the physical program is executed instruction by instruction
        from ironpangu_b200.runtime.plan_engine import PlanEngine

        eng = PlanEngine(args.bundle, args.checkpoint, fab, max_tokens=None, num_slots=args.max_num_seqs)   # rows per step: as planned
        mark("program", "parameters, KV state and workspace of the compiled program")
        head = [i for i in eng.ins if i["op"] == "lm_head"][-1]
        vocab = int(eng._param(head["attrs"]["weight"]).shape[0]) * world
        return BatchEngine(eng, os.path.basename(os.path.normpath(args.bundle)), min(args.max_model_len, eng.max_context), vocab,
                           greedy_only=True)
    if args.model in ("hyper-tiny", "pangu92b", "pangu92b-learned"):
        # the hyper-connected latent-attention + routed-experts family: its generated source compiled for this job's width, random
        # parameters drawn per init-plan load slice (replicated tensors identical on every rank), run by the plan engine
        import tempfile

        from ironpangu_b200 import compiler
        from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source
        from ironpangu_b200.runtime.plan_engine import PlanEngine, random_parameters

        hcfg = {"hyper-tiny": HyperMlaMoeConfig.tiny, "pangu92b": HyperMlaMoeConfig.pangu92b,
                "pangu92b-learned": HyperMlaMoeConfig.pangu92b_learned}[args.model]()
        if args.layers:
            hcfg.layers = args.layers
        work = tempfile.mkdtemp(prefix=f"ifab-worker-r{rank}-")
        src = os.path.join(work, "model.inferfabric")
        with open(src, "w") as f:
            f.write(hyper_mla_moe_source(hcfg, world, context=args.max_model_len))
        compiled = compiler.write_bundle(src, os.path.join(work, "bundle"), prefill_tokens=8)
        with open(os.path.join(compiled["dir"], f"rank-{rank}.init.json")) as f:
            plan = json.load(f)
        params = random_parameters(plan, dev, seed=args.seed)
        mark("weights")
        eng = PlanEngine(compiled["dir"], None, fab, max_tokens=8, num_slots=args.max_num_seqs, parameters=params)
        mark("bundle", f"program {compiled['program_sha256'][:16]}, arena {eng.arena.bytes + eng.arena.workspace_bytes} bytes")
        return BatchEngine(eng, f"ifab-{args.model}", min(args.max_model_len, eng.max_context), hcfg.vocab, greedy_only=True)
    if args.model.startswith("hybrid"):
        # gated delta-rule + gated full-attention family (one GPU): K / V pages, f32 delta state and conv history per sequence slot
        from ironpangu_b200.models import hybrid_delta as H

        if world != 1:
            raise SystemExit("the hybrid decoder runs on one GPU")
        if args.model == "hybrid":
            # a model document + a checkpoint directory: inspected and compiled into the typed plan before any byte is loaded
            if not (args.definition and args.checkpoint):
                raise SystemExit("--model hybrid needs --definition MODEL.inferfabric and --checkpoint DIR")
            hplan = H.typed_plan(args.definition, args.checkpoint)
            hcfg = H.config_of(hplan, args.checkpoint)
            mark("plan", f"typed plan {hplan['key'][:16]}")
            hweights = H.load_weights(hplan, args.checkpoint, dev)
        else:
            hcfg = H.HybridConfig.tiny(args.layers or 1) if args.model == "hybrid-tiny" else H.HybridConfig.text2b()
            if args.model == "hybrid2b" and args.layers:
                hcfg.layers = hcfg.layers[:args.layers]
            hweights = H.random_weights(hcfg, dev, seed=args.seed)
        mark("weights")
        hdec = H.HybridDecoder(hcfg, hweights, fab, max_tokens=8, max_context=args.max_model_len, num_slots=args.max_num_seqs,
                               keep_logits=not args.greedy_only)
        mark("state", "K/V pages, delta state, conv history and step workspace")
        eng = BatchEngine(hdec, f"ifab-{args.model}", args.max_model_len, hcfg.vocab, eos=-1, greedy_only=args.greedy_only,
                          token_budget=args.max_num_batched_tokens, use_graphs=not args.no_graphs)
        mark("sampling", "per-slot sampling state")
        return eng
    if args.model.startswith("dense"):
        # Qwen-style dense GQA decoder (tensor parallel over the fabric): same batch contract, K/V page caches
        from ironpangu_b200.models import dense_gqa as G

        dcfg = G.DenseConfig.tiny(args.layers or 2) if args.model == "dense-tiny" else G.DenseConfig.qwen2b()
        if args.model == "dense2b" and args.layers:
            dcfg.layers = args.layers
        dweights = G.random_rank_weights(dcfg, rank, world, dev, seed=args.seed)
        mark("weights")
        if args.executor == "bundle":
            # the family's .inferfabric source compiled for this job's width, run by the plan engine on the same tensors
            import tempfile

            from ironpangu_b200 import compiler
            from ironpangu_b200.compiler.sources import dense_gqa_source
            from ironpangu_b200.runtime.plan_engine import PlanEngine

            work = tempfile.mkdtemp(prefix=f"ifab-worker-r{rank}-")
            src = os.path.join(work, "model.inferfabric")
            with open(src, "w") as f:
                f.write(dense_gqa_source(dcfg, world, context=args.max_model_len))
            compiled = compiler.write_bundle(src, os.path.join(work, "bundle"), prefill_tokens=8)
            ddec = PlanEngine(compiled["dir"], None, fab, max_tokens=8, num_slots=args.max_num_seqs, keep_logits=not args.greedy_only,
                              parameters=G.bundle_parameters(dcfg, dweights, world))
            mark("bundle", f"program {compiled['program_sha256'][:16]}, arena {ddec.arena.bytes + ddec.arena.workspace_bytes} bytes")
        else:
            ddec = G.DenseDecoder(dcfg, dweights, fab, max_tokens=8, max_context=args.max_model_len, num_slots=args.max_num_seqs,
                                  keep_logits=not args.greedy_only)
        mark("state", "K/V page caches and step workspace")
        dprefill = None
        if args.prefill_chunk > 8:
            from ironpangu_b200.models.dense_prefill import DensePrefill

            dprefill = DensePrefill(ddec, max_rows=args.prefill_chunk)
            dprefill.sequence_parallel = bool(ro is not None and ro.sequence_parallel)
            mark("prefill", "activation buffers of the matrix-matrix prompt path")
        eng = BatchEngine(ddec, f"ifab-{args.model}", args.max_model_len, dcfg.vocab, eos=-1, greedy_only=args.greedy_only, prefill=dprefill,
                          token_budget=args.max_num_batched_tokens, use_graphs=not args.no_graphs)
        mark("sampling", "per-slot sampling state")
        return eng
    cfg = MlaMoeConfig.tiny(args.layers or 2) if args.model == "tiny" else MlaMoeConfig.flagship()
    if args.model != "tiny" and args.layers:
        cfg.layers = args.layers
    weights = random_rank_weights(cfg, rank, world, dev, seed=args.seed)
    mark("weights")
    if args.executor == "bundle" and not args.expert_fp8:
        # the model's .inferfabric source, compiled for this job's width; the plan engine's dispatcher picks the kernels, the
        # activations live in the bundle's frozen arena (a packed int8 cache is declared in the source; fp8 expert storage is not
        # in the language: hand-wired class)
        import tempfile

        from ironpangu_b200 import compiler
        from ironpangu_b200.compiler.sources import mla_moe_source
        from ironpangu_b200.models.mla_moe import bundle_parameters
        from ironpangu_b200.runtime.plan_engine import PlanEngine

        work = tempfile.mkdtemp(prefix=f"ifab-worker-r{rank}-")
        src = os.path.join(work, "model.inferfabric")
        with open(src, "w") as f:
            f.write(mla_moe_source(cfg, world, context=args.max_model_len, kv_int8=args.kv_int8))
        compiled = compiler.write_bundle(src, os.path.join(work, "bundle"), prefill_tokens=8)
        dec = PlanEngine(compiled["dir"], None, fab, max_tokens=8, num_slots=args.max_num_seqs, keep_logits=not args.greedy_only,
                         parameters=bundle_parameters(cfg, weights), fused_head=ro.fused_head if ro is not None else None)
        mark("bundle", f"program {compiled['program_sha256'][:16]}, arena {dec.arena.bytes + dec.arena.workspace_bytes} bytes")
    else:
        dec = MlaMoeDecoder(cfg, weights, fab, max_tokens=8, max_context=args.max_model_len, num_slots=args.max_num_seqs,
                            keep_logits=not args.greedy_only, kv_int8=args.kv_int8, expert_fp8=args.expert_fp8,
                            fused_head=ro.fused_head if ro is not None else None)
    mark("state", "KV cache, recurrent state and step workspace")
    prefill = None
    if args.prefill_chunk > 8:
        # prompt chunks on the tensor cores (fp8 experts are widened one layer at a time; over the int8 cache the attention of a
        # chunk runs in the latent form on the split-KV kernels, everything else as GEMMs)
        from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill

        prefill = MlaMoePrefill(dec, max_rows=args.prefill_chunk)
        mark("prefill", "activation buffers of the matrix-matrix prompt path")
    eng = BatchEngine(dec, f"ifab-{args.model}", args.max_model_len, cfg.vocab, eos=cfg.eos, greedy_only=args.greedy_only,
                      prefix_slots=args.prefix_cache_slots, prefill=prefill, token_budget=args.max_num_batched_tokens,
                      use_graphs=not args.no_graphs, prefix_namespace=args.prefix_cache_namespace)
    mark("sampling", "per-slot sampling state and prefix snapshots")
    return eng


class Agreement:
    """Cross-rank agreement on the outcome of every request. Every rank executes every request; rank 0 answers the server, so
    a rank that failed or sampled a different token must not go unnoticed: any failure, or any difference between the token
    lists of a step, becomes a backend error on rank 0 (which makes the server fail closed).

    The common case costs one small all-reduce over a digest of (ok, tokens); the details (who failed, which tokens) are
    exchanged only when the digests differ. Modes:
      strict    the ranks agree BEFORE rank 0 answers: nothing a rank disagreed on ever reaches a client, and the slowest
                rank's host work plus one CPU all-reduce sit on the critical path of every step;
      deferred  the all-reduce of request k is started asynchronously and checked when request k + 1 has been executed, so
                it overlaps the next step; a disagreement on request k turns the answer to request k + 1 (and every later
                one) into the backend error - at most one answer leaves before the failure is reported."""

    def __init__(self, rank: int, world: int, group, mode: str = "strict"):
        assert mode in ("strict", "deferred")
        self.rank, self.world, self.group, self.mode = rank, world, group, mode
        self.pending = None            # (work, tensor, digest, mine, op, resp) of the request whose all-reduce is in flight
        self.failed: Optional[Dict] = None

    def _start(self, mine, async_op: bool):
        import zlib

        h = zlib.crc32(json.dumps([mine[0], mine[1]]).encode()) if mine[0] else -1 - self.rank
        t = torch.tensor([h, -h], dtype=torch.int64)
        work = dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group, async_op=async_op)
        return work, t, h

    def _verdict(self, t, h, mine, op: str, resp: Dict) -> Dict:
        """``resp`` when all digests were equal, else the error every rank derives from the exchanged details."""
        if mine[0] and int(t[0]) == h and int(t[1]) == -h:
            return resp
        every = [None] * self.world
        dist.all_gather_object(every, mine, group=self.group)
        for r, (ok, _, kind, err) in enumerate(every):
            if not ok:
                if r == self.rank:
                    return resp
                return {"ok": False, "kind": kind or "backend", "error": f"rank {r}: {err}"}
        if op == "step":
            for r, (_, toks, _, _) in enumerate(every):
                if toks != every[0][1]:
                    return {"ok": False, "kind": "backend",
                            "error": f"token consensus mismatch: rank 0 produced {every[0][1]}, rank {r} produced {toks}"}
        return resp

    def check(self, resp: Dict, op: str) -> Dict:
        """The response rank 0 should send for this request."""
        mine = (bool(resp.get("ok")), resp.get("tokens"), resp.get("kind"), resp.get("error"))
        if self.mode == "strict":
            _, t, h = self._start(mine, False)
            return self._verdict(t, h, mine, op, resp)
        if self.failed is not None:                 # every rank reached this state at the same request: no more collectives
            return self.failed
        late = self.finish()
        if late is not None:                        # the digests of the previous request differed: every rank sees that here
            self.failed = late
            return late
        self.pending = self._start(mine, True) + (mine, op, resp)
        return resp

    def finish(self) -> Optional[Dict]:
        """Wait for the all-reduce in flight (deferred mode); returns the error it revealed, if any."""
        if self.pending is None:
            return None
        work, t, h, mine, op, resp = self.pending
        self.pending = None
        work.wait()
        v = self._verdict(t, h, mine, op, resp)
        if v is resp and resp.get("ok"):
            return None
        if v is resp:                               # this rank's own failure: rank 0 already answered with it
            v = {"ok": False, "kind": resp.get("kind") or "backend", "error": f"rank {self.rank}: {resp.get('error')}"}
        return {"ok": False, "kind": v.get("kind") or "backend", "error": "an earlier request: " + str(v.get("error"))}


def serve(engine, rank: int, world: int, sock_path: str, group=None, agreement="strict") -> None:
    """Request loop of one rank. ``group``: process group for the control traffic (request broadcast and agreement); a gloo
    group keeps it off the GPU streams. ``agreement``: "strict", "deferred" or "off" (see :class:`Agreement`)."""
    agreement = {True: "strict", False: "off"}.get(agreement, agreement)
    agreeing = Agreement(rank, world, group, agreement) if world > 1 and agreement != "off" else None
    conn = None
    buf = b""
    if rank == 0:
        conn = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        conn.connect(sock_path)
    while True:
        req = None
        if rank == 0:
            while b"\n" not in buf:
                chunk = conn.recv(1 << 16)
                if not chunk:
                    req = {"op": "shutdown"}
                    break
                buf += chunk
            if req is None:
                line, buf = buf.split(b"\n", 1)
                req = json.loads(line)
        if world > 1:
            box = [req]
            dist.broadcast_object_list(box, src=0, group=group)
            req = box[0]
        op = req.get("op")
        try:
            if op == "info":
                resp = {"ok": True, "info": engine.info()}
            elif op == "admit":
                engine.admit(int(req["resident"]), req.get("sampling", {}), int(req.get("reserve", 0)))
                resp = {"ok": True}
            elif op == "step":
                resp = {"ok": True, "tokens": engine.step(req["slices"], req["tokens"])}
            elif op == "release":
                engine.release(int(req["resident"]))
                resp = {"ok": True}
            elif op == "audit":
                resp = {"ok": True, "audit": engine.audit()}
            elif op == "shutdown":
                resp = {"ok": True}
            else:
                resp = {"ok": False, "kind": "invalid", "error": f"unknown op {op!r}"}
        except OverflowError as e:
            resp = {"ok": False, "kind": "capacity", "error": str(e)}
        except ValueError as e:
            resp = {"ok": False, "kind": "invalid", "error": str(e)}
        except Exception as e:  # noqa: BLE001 - every failure must reach the server as a backend error
            resp = {"ok": False, "kind": "backend", "error": f"{type(e).__name__}: {e}"}
        if agreeing is not None and op in ("info", "admit", "step", "release"):
            resp = agreeing.check(resp, op)
        elif agreeing is not None and op == "shutdown":
            late = agreeing.finish()
            if late is not None:
                resp = late
        if rank == 0 and conn is not None:
            try:
                conn.sendall(json.dumps(resp).encode() + b"\n")
            except OSError:
                op = "shutdown"
        if op == "shutdown":
            break
    if conn is not None:
        conn.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny", choices=["tiny", "flagship", "dense-tiny", "dense2b", "hybrid-tiny", "hybrid2b", "hybrid", "hyper-tiny", "pangu92b", "pangu92b-learned"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--bundle", default="")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--definition", default="", help="model document of --model hybrid (contract qwen35_text_v1)")
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--max-model-len", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=0, help="tokens per scheduler step (0 = one launch group of 8 rows)")
    ap.add_argument("--executor", default="bundle", choices=["bundle", "model"],
                    help="bf16 MLA+MoE models: run the compiled bundle of the model's generated source (plan engine) or the hand-wired decoder class")
    ap.add_argument("--prefix-cache-namespace", default="", help="tenant namespace of the prefix cache: part of every key")
    ap.add_argument("--prefix-cache-slots", type=int, default=0, help="device snapshots kept by the prefix cache (0 = off)")
    ap.add_argument("--kv-int8", action="store_true", help="packed int8 latent KV cache")
    ap.add_argument("--expert-fp8", action="store_true", help="block-scaled fp8 expert weights (1 x 128 scale blocks)")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="rows per tensor-core prefill call (0 = prompts go through the decode kernels)")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel from the host instead of replaying CUDA graphs")
    ap.add_argument("--greedy-only", action="store_true", help="skip the logits buffer; refuse sampled requests")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--memory-profile", default="", help="write the staged start-up memory profile (JSON) here")
    ap.add_argument("--profile-only", action="store_true", help="build the engine, write the memory profile and exit")
    ap.add_argument("--socket", default=os.environ.get("IFAB_ENGINE_SOCKET", ""))
    ap.add_argument("--set", action="append", default=[], metavar="NAME=VALUE",
                    help="runtime option (see runtime/options.py); also read from IFAB_<NAME> environment variables")
    args = ap.parse_args()
    # typed runtime options: environment first, then --set, then the dedicated flags of this command line
    from ironpangu_b200.runtime.options import RuntimeOptions

    ropts = RuntimeOptions.from_env(os.environ, args.set)
    args.kv_int8 = args.kv_int8 or ropts.kv_int8
    args.expert_fp8 = args.expert_fp8 or ropts.expert_fp8
    args.prefill_chunk = args.prefill_chunk or ropts.prefill_chunk
    args.prefix_cache_slots = args.prefix_cache_slots or ropts.prefix_cache_slots
    args.no_graphs = args.no_graphs or not ropts.decode_graph
    ropts.kv_int8, ropts.expert_fp8, ropts.prefill_chunk = args.kv_int8, args.expert_fp8, args.prefill_chunk
    ropts.prefix_cache_slots, ropts.decode_graph = args.prefix_cache_slots, not args.no_graphs
    ropts.validate()
    if not ropts.pdl:
        os.environ["IFAB_PDL"] = "0"           # read by the kernel library when it is loaded
    args.runtime_options = ropts
    if not args.socket and not args.profile_only:
        raise SystemExit("no engine socket: set IFAB_ENGINE_SOCKET or pass --socket")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.runtime.memory import MemoryProfile, StartupOptions

    opts = StartupOptions(args.max_model_len, args.max_num_seqs, max(8, args.max_num_batched_tokens), args.gpu_memory_utilization,
                          (args.memory_profile + (f".rank{rank}" if rank else "")) if args.memory_profile else None, args.profile_only)
    rec = MemoryProfile.start(opts)
    engine = build_engine(args, rank, world, rec)
    engine.runtime_options = ropts
    if ropts.trace_dir:
        from .trace import StepTrace

        engine.trace = StepTrace(ropts.trace_dir, rank)
    rec.finish()
    if args.profile_only:
        torch.cuda.synchronize()
        engine.dec.fabric.close()
        if world > 1:
            dist.destroy_process_group()
        return
    if world > 1:
        os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")              # ranks of one node: no host-name lookup for the CPU group
    ctl = dist.new_group(backend="gloo") if world > 1 else None     # control traffic stays on the CPU
    try:
        serve(engine, rank, world, args.socket, ctl, ropts.rank_agreement)
    finally:
        torch.cuda.synchronize()
        if engine.trace is not None:
            engine.trace.close()
        if ropts.audit_dir:
            # the audit record of this rank (counters, options), for runs that are compared later
            os.makedirs(ropts.audit_dir, exist_ok=True)
            with open(os.path.join(ropts.audit_dir, f"engine-audit-rank{rank}.json"), "w") as f:
                json.dump(engine.audit(), f, indent=1)
        engine.dec.fabric.close()
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
