"""Tensor-core prefill path of the dense GQA decoder (chunks of up to ``max_rows`` prompt tokens).

The decode kernels of ``DenseDecoder`` multiply at most 8 rows per pass on the CUDA cores; measured on a B200 a pass of
8 rows costs about 5 ms for the 2B model, so a 2048-token prompt takes over a second. This path runs a chunk as
matrix-matrix work: the four linears of a layer on the tcgen05 GEMM (gate/up through the grouped kernel's SwiGLU epilogue
with a single "expert", the row-parallel o_proj and down projections through the fused GEMM + all-reduce kernel when the
model is tensor parallel), rotary + cache append through the decode path's kernel, attention through its split-KV kernels
with one query row per token (causality comes from the per-row positions), ``attn_rows`` query rows per launch.
It shares weights, caches and the page table with the decoder, so decode continues from the state it leaves.

Sequence-parallel mode (``sequence_parallel=True``, tensor-parallel models, chunks of a multiple of ``128 * world`` rows): the
residual stream, both norms and the embedding keep only this rank's ``m / world`` rows. The column-parallel linears (qkv,
gate/up) run as all-gather GEMMs that bring the peers' normalised rows over NVLink inside the kernel; the row-parallel ones
(o_proj, down) as GEMM + reduce-scatter, so each rank receives just its rows of the sum. The all-reduce of the plain mode
(reduce-scatter + all-gather of the full activation, then a norm every rank repeats over all rows) becomes the two halves
placed where the data is needed, and norm / residual traffic drops by ``world``.
Reference: batched prompt processing of the Qwen engine (inferfabric-native/src/lib.rs:598-661, consume_batch).
"""
from __future__ import annotations

import math

import torch

from ..ops import decode as K
from ..ops import gemm as G
from ..ops import prefill as P
from .dense_gqa import BF16, DenseDecoder


class DensePrefill:
    # steps with more rows than this go through `forward_rows`: past two rows the CUDA-core GEMV kernels are FMA-bound
    # (4.9 ms per 8-row pass of the 2B model), the GEMM path streams the weights at tensor-core speed whatever the row count
    batch_threshold = 2

    def __init__(self, dec: DenseDecoder, max_rows: int = 512, attn_rows: int = 64):
        self.dec, self.M, self.QC = dec, max_rows, attn_rows
        c, fab, dev = dec.cfg, dec.fabric, dec.fabric.device
        M = max_rows
        Mpad = (M + 127) // 128 * 128          # whole 128-row tiles of the one-expert group are stored
        e = lambda *s, dt=BF16: torch.empty(*s, dtype=dt, device=dev)
        self.tokens = torch.zeros(M, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(M, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(M, dtype=torch.int32, device=dev)
        self.x_sym = fab.symmetric_empty((M, c.hidden)) if fab.world > 1 else None
        self.x = self.x_sym.tensor if self.x_sym is not None else e(M, c.hidden)
        self.h = torch.zeros(Mpad, c.hidden, dtype=BF16, device=dev)
        self.qkv = e(M, (dec.hq + 2 * dec.hk) * c.head_dim)
        self.attn = e(M, dec.hq * c.head_dim)
        self.act = e(Mpad, c.ffn // fab.world)
        self.scratch = e(self.QC * dec.hq * dec.max_splits * (c.head_dim + 2), dt=torch.float32)
        nt = (M + 127) // 128
        st = torch.zeros(nt, 4, dtype=torch.int32)
        for i in range(nt):
            st[i, 1], st[i, 2] = i * 128, 128
        self.tiles = st.to(dev)
        self.ntiles = torch.zeros(1, dtype=torch.int32, device=dev)
        self.launches = 0
        # Prompt attention on the tensor cores for chunks of consecutive positions of one sequence (heads of 128 columns): keys and
        # values of the context are gathered out of their pages (values transposed) and attended by the tcgen05 attention kernel
        # in its grouped-query form, instead of one split-KV pass per 64 query rows.
        self.tc_attention = c.head_dim == 128
        if self.tc_attention:
            cap = (dec.max_context + 127) // 128 * 128
            self.ctx_k = torch.zeros(cap, dec.hk * c.head_dim, dtype=BF16, device=dev)
            self.ctx_vt = torch.zeros(dec.hk * c.head_dim, cap, dtype=BF16, device=dev)
        self._contig = None            # (first position, slot) of the chunk being run, None for rows of many sequences
        # CUDA graphs of the layer stack for small batched steps (one graph per row count): a 64-row decode step is ~250
        # launches, which cost more host time through Python than device time
        self.graph_rows_max = 64
        self._graphs = {}
        self.sequence_parallel = False              # default of `forward` (a serving process sets it once)
        self._sp = {}                               # rows -> sequence-parallel scratch (symmetric shards, gather states)

    def _sym_rows(self, m: int):
        if m == self.M:
            return self.x_sym
        v = object.__new__(type(self.x_sym))
        v.__dict__.update(self.x_sym.__dict__)
        v.tensor = self.x_sym.tensor[:m]
        return v

    def can_sequence_parallel(self, m: int) -> bool:
        w = self.dec.fabric.world
        return w > 1 and m % (128 * w) == 0

    def forward(self, tokens: torch.Tensor, pos0: int, slot: int = 0, sequence_parallel=None) -> torch.Tensor:
        """Run ``tokens`` (int32 ``[m]``, ``m <= max_rows``, on the device) at positions ``pos0 .. pos0+m-1`` of sequence slot
        ``slot``; returns the greedy next token after the last row (device tensor ``[1]``; its logits land in row 0 of the
        decoder's logits buffer when that exists). ``sequence_parallel`` keeps the residual stream sharded by rows where the
        chunk allows it (``can_sequence_parallel``); other chunks take the all-reduce path."""
        d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
        m = tokens.numel()
        assert 1 <= m <= self.M
        self.tokens[:m].copy_(tokens)
        self.positions[:m].copy_(torch.arange(pos0, pos0 + m, dtype=torch.int32, device=tokens.device))
        self.slots[:m].fill_(slot)
        if sequence_parallel is None:
            sequence_parallel = self.sequence_parallel
        self._contig = (pos0, slot)
        try:
            if sequence_parallel and self.can_sequence_parallel(m):
                x = self._layers_sp(m)
            else:
                x = self._layers(m)
        finally:
            self._contig = None
        K.lm_head_argmax(x[m - 1:m], d.w["lm_head"], fab, norm_w=d.w["final_norm"], eps=c.eps, vocab_offset=d.rank * d.vl,
                         partial=d.partial, logits=None if d.logits is None else d.logits[:1], out_ids=d.next_ids[:1],
                         out_vals=d.next_vals[:1])
        self.launches += 1
        return d.next_ids[:1]

    def forward_rows(self, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, select: torch.Tensor) -> torch.Tensor:
        """Batched step over ``m`` independent rows (each with its own position and sequence slot, e.g. one decode row per
        running sequence): the layers run as matrix-matrix work, then the vocabulary shard of the logits of rows ``select``
        (int64 indices) comes from one GEMM. Returns f32 logits ``[len(select), vocab_local]``."""
        d, c = self.dec, self.dec.cfg
        m = tokens.numel()
        assert 1 <= m <= self.M
        self.tokens[:m].copy_(tokens)
        self.positions[:m].copy_(positions)
        self.slots[:m].copy_(slots)
        x = self._layers_graphed(m)
        xs = x.index_select(0, select)
        xn = K.rmsnorm(xs, d.w["final_norm"], c.eps)
        self.launches += 2
        return G.gemm(xn, d.w["lm_head"], out_f32=True, status_ptr=d.fabric.desc.status)

    def _layers_graphed(self, m: int) -> torch.Tensor:
        if m > self.graph_rows_max:
            return self._layers(m)
        g = self._graphs.get(m)
        if g is not None:
            g.replay()
            return self.x[:m]
        x = self._layers(m)                         # the real run of this step (and the warm-up of the capture)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):                   # records only: the caches are not touched a second time
            self._layers(m)
        self._graphs[m] = g
        return x

    def _attention(self, l: int, m: int, qkv: torch.Tensor, pos: torch.Tensor, sl: torch.Tensor, scale: float, st) -> None:
        """Attention of layer ``l`` for the ``m`` rows of ``qkv`` (rotated, keys / values already in the cache) into ``self.attn``."""
        d, c = self.dec, self.dec.cfg
        if self.tc_attention and self._contig is not None:
            pos0, slot = self._contig
            ctx = pos0 + m
            rows = (ctx + 63) // 64 * 64
            P.gqa_ctx_gather(d.k_cache[l], d.v_cache[l], d.page_table, slot, ctx, self.ctx_k[:rows], self.ctx_vt, status_ptr=st)
            P.fa_prefill(qkv[:, :d.hq * c.head_dim], self.ctx_k, self.ctx_vt, self.attn[:m], heads=d.hq, q_head_stride=c.head_dim,
                         k_head_stride=c.head_dim, vt_head_stride=c.head_dim, vt_row0=0, d1=c.head_dim, d2=0, kv_group=d.hq // d.hk, ctx=ctx,
                         pos0=pos0, scale=scale, status_ptr=st)
            return
        for q0 in range(0, m, self.QC):
            q1 = min(m, q0 + self.QC)
            K.gqa_decode_attention(qkv[q0:q1], d.k_cache[l], d.v_cache[l], pos[q0:q1], sl[q0:q1], d.page_table, heads=d.hq,
                                   kv_heads=d.hk, head_dim=c.head_dim, scale=scale, keys_per_split=d.kps, max_splits=d.max_splits,
                                   scratch=self.scratch, out=self.attn[q0:q1], status_ptr=st)

    def _layers(self, m: int) -> torch.Tensor:
        """Embedding + all layers over the ``m`` rows staged in ``tokens / positions / slots``; returns the hidden rows."""
        d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
        w, st = d.w, fab.desc.status
        tok, pos, sl = self.tokens[:m], self.positions[:m], self.slots[:m]
        x, h = self.x[:m], self.h[:m]
        K.embedding(tok, w["embed"], out=x, status_ptr=st)
        self.ntiles.fill_((m + 127) // 128)
        scale = 1.0 / math.sqrt(c.head_dim)
        for l in range(c.layers):
            p = f"layers.{l}."
            K.rmsnorm(x, w[p + "attn_norm"], c.eps, out=h)
            qkv = G.gemm(h, w[p + "qkv"], out=self.qkv[:m], status_ptr=st)
            K.gqa_rope_kv_write(qkv, pos, sl, d.page_table, d.k_cache[l], d.v_cache[l], heads=d.hq, kv_heads=d.hk,
                                head_dim=c.head_dim, theta=c.theta, status_ptr=st)
            self._attention(l, m, qkv, pos, sl, scale, st)
            if fab.world > 1:
                G.gemm_allreduce(self.attn[:m], w[p + "o_proj"], fab, self._sym_rows(m), residual=x)
            else:
                G.gemm(self.attn[:m], w[p + "o_proj"], residual=x, out=x, status_ptr=st)
            K.rmsnorm(x, w[p + "ffn_norm"], c.eps, out=h)
            if m >= 256:
                # whole 256-row tile pairs: the packed gate | up projection and its activation on CTA pairs, one persistent launch
                G.gemm_swiglu(h, w[p + "gate_up"], out=self.act[:m], status_ptr=st)
            else:
                P.grouped_gemm(self.h, w[p + "gate_up"].unsqueeze(0), self.tiles, self.ntiles, self.act[:m], swiglu=True, status_ptr=st)
            if fab.world > 1:
                G.gemm_allreduce(self.act[:m], w[p + "down"], fab, self._sym_rows(m), residual=x)
            else:
                G.gemm(self.act[:m], w[p + "down"], residual=x, out=x, status_ptr=st)
        self.launches = 1 + c.layers * (8 + 2 * ((m + self.QC - 1) // self.QC))
        return x

    # -- sequence parallel ------------------------------------------------------------------------------------------------
    def _sp_state(self, m: int):
        """Scratch of the sequence-parallel path for chunks of ``m`` rows; every rank creates it at the same call (the
        symmetric allocations exchange handles). One gather state per (rows, GEMM): the kernel's tile counters advance by its
        grid width per call, so two GEMMs of different widths cannot share them."""
        st = self._sp.get(m)
        if st is None:
            d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
            rows = m // fab.world
            dev = fab.device
            st = {
                "rows": rows,
                "x": torch.empty(rows, c.hidden, dtype=BF16, device=dev),
                "h_attn": fab.symmetric_empty((rows, c.hidden)),
                "h_ffn": fab.symmetric_empty((rows, c.hidden)),
                "ag_qkv": G.AllGatherGemmState(fab, rows, c.hidden),
                "ag_ffn": G.AllGatherGemmState(fab, rows, c.hidden),
                "gu": torch.empty(m, 2 * (c.ffn // fab.world), dtype=BF16, device=dev),
            }
            self._sp[m] = st
        return st

    def _layers_sp(self, m: int) -> torch.Tensor:
        """The layer stack with the residual stream sharded by rows. Returns the full hidden buffer with only the LAST row
        valid on every rank (what the greedy head needs): the rank that owns the last shard broadcasts it."""
        import torch.distributed as dist

        d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
        w, stt = d.w, fab.desc.status
        sp = self._sp_state(m)
        rows, r = sp["rows"], fab.rank
        tok, pos, sl = self.tokens[:m], self.positions[:m], self.slots[:m]
        xl = sp["x"]
        K.embedding(tok[r * rows:(r + 1) * rows], w["embed"], out=xl, status_ptr=stt)
        scale = 1.0 / math.sqrt(c.head_dim)
        for l in range(c.layers):
            p = f"layers.{l}."
            K.rmsnorm(xl, w[p + "attn_norm"], c.eps, out=sp["h_attn"].tensor)
            qkv = G.allgather_gemm(sp["h_attn"], w[p + "qkv"], sp["ag_qkv"], fab, out=self.qkv[:m])
            K.gqa_rope_kv_write(qkv, pos, sl, d.page_table, d.k_cache[l], d.v_cache[l], heads=d.hq, kv_heads=d.hk,
                                head_dim=c.head_dim, theta=c.theta, status_ptr=stt)
            self._attention(l, m, qkv, pos, sl, scale, stt)
            G.gemm_reduce_scatter(self.attn[:m], w[p + "o_proj"], fab, out=xl, residual=xl)
            K.rmsnorm(xl, w[p + "ffn_norm"], c.eps, out=sp["h_ffn"].tensor)
            gu = G.allgather_gemm(sp["h_ffn"], w[p + "gate_up"], sp["ag_ffn"], fab, out=sp["gu"])
            K.swiglu_rows(gu, out=self.act[:m])
            G.gemm_reduce_scatter(self.act[:m], w[p + "down"], fab, out=xl, residual=xl)
        last = self.x[m - 1:m]
        if r == fab.world - 1:
            last.copy_(xl[rows - 1:rows])
        dist.broadcast(last, src=fab.world - 1, group=fab.group)
        self.launches = 2 + c.layers * (9 + 2 * ((m + self.QC - 1) // self.QC))
        return self.x[:m]
