"""Tensor-core prefill path of the MLA + MoE decoder (chunks of up to ``max_rows`` prompt tokens).

The decode path streams every weight matrix once per step; pushing a long prompt through it 8 tokens at a time
re-reads the whole model 64 times per 512 tokens. This path runs a chunk as matrix-matrix work instead:

* dense linears (qkv_a, q_b, shared expert down) on the tcgen05 GEMM, the row-parallel o_proj on the fused
  GEMM + all-reduce kernel when the model is tensor parallel;
* the absorbed-MLA projections (q_nope @ W_uk, o_lat @ W_uv) as one small GEMM per head;
* attention through the split-KV kernels of the decode path with one query row per token (causality comes from
  the per-row positions), 64 query rows per launch;
* the MoE through a device-side dispatch (routes sorted by expert, 128-row tile table), the grouped expert GEMM
  with the SwiGLU epilogue, the grouped down GEMM and a score-weighted combine; the shared expert rides on the same
  grouped kernel with a single "expert"; across ranks the partial outputs are summed by a pull all-reduce.

It shares the KV cache, the page table and the weights with ``MlaMoeDecoder`` and leaves the cache exactly as
token-by-token decoding would (same normalisation and rotary kernel), so decode continues from it.
Rounding differs from the decode path in one place: expert outputs are stored as bf16 rows before the
combine (the decode kernels keep them in f32), which stays inside the tolerance of the oracle tests.
Reference: the uncaptured 4096-token prefill envelope (native/src/token_executor.h:1449-1587).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import decode as K
from ..ops import gemm as G
from ..ops import prefill as P
from .mla_moe import BF16, MlaMoeDecoder


class MlaMoePrefill:
    # steps with more rows than this go through `forward_rows` (the path launches ~100 kernels per layer, so it only pays
    # beyond one decode launch group)
    batch_threshold = 8

    def __init__(self, dec: MlaMoeDecoder, max_rows: int = 512, attn_rows: int = 64):
        self.dec, self.M, self.QC = dec, max_rows, attn_rows
        c, dev, fab = dec.cfg, dec.fabric.device, dec.fabric
        hl, el, M = dec.hl, dec.el, max_rows
        e = lambda *s, dt=BF16: torch.empty(*s, dtype=dt, device=dev)
        self.tokens = torch.zeros(M, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(M, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(M, dtype=torch.int32, device=dev)
        self.x_sym = fab.symmetric_empty((M, c.hidden)) if fab.world > 1 else None
        self.x = self.x_sym.tensor if self.x_sym is not None else e(M, c.hidden)
        Mpad = (M + 127) // 128 * 128     # whole 128-row tiles of the one-expert group are stored
        self.h = torch.zeros(Mpad, c.hidden, dtype=BF16, device=dev)
        self.qkv = e(M, c.q_lora + c.kv_lora + c.rope)
        self.qn = e(M, c.q_lora)
        self.q = e(M, hl * c.qk_dim)
        self.q_lat = e(M, hl, c.kv_lora + c.rope)
        self.o_lat = e(M, hl, c.kv_lora)
        self.attn = e(M, hl * c.vdim)
        self.scratch = e(self.QC * hl * dec.max_splits * (c.kv_lora + 2), dt=torch.float32)
        self.ids = torch.zeros(M, c.topk, dtype=torch.int32, device=dev)
        self.wts = e(M, c.topk, dt=torch.float32)
        self.route = P.DispatchBuffers(M, c.topk, el, dev)
        R = self.route.max_routes
        self.xp = torch.zeros(R, c.hidden, dtype=BF16, device=dev)
        self.act = e(R, c.expert_ffn)
        self.y = e(R, c.hidden)
        fs = c.shared_ffn // fab.world
        self.sact = e(Mpad, fs)
        self.sd = e(Mpad, c.hidden)
        # the shared expert as a one-expert group over all rows of the chunk (static tile table)
        nt = (M + 127) // 128
        st = torch.zeros(nt, 4, dtype=torch.int32)
        for i in range(nt):
            st[i, 1], st[i, 2] = i * 128, 128
        self.shared_tiles = st.to(dev)
        self.shared_ntiles = torch.zeros(1, dtype=torch.int32, device=dev)
        # block-scaled fp8 experts: the tensor-core kernels take bf16 operands, so one layer's expert matrices are widened into
        # this scratch right before the layer's grouped GEMMs (read 1 byte, write 2 per weight: a fraction of the GEMMs' time
        # for chunks of a few hundred rows and up)
        self.w8 = getattr(dec, "w8", None) if getattr(dec, "expert_fp8", False) else None
        if self.w8 is not None:
            # widening every expert of a layer costs as much as streaming them twice: steps of a few dozen rows of many sequences
            # are cheaper as passes of the eight-row fp8 decode kernels, which read the experts as they are
            self.batch_threshold = 64
            self.wide = {"gate_up": e(el, 2 * c.expert_ffn, c.hidden), "down": e(el, c.hidden, c.expert_ffn),
                         "shared_gate_up": e(2 * fs, c.hidden), "shared_down": e(c.hidden, fs)}
        self.parts = [fab.symmetric_empty((M, c.hidden), torch.float32) for _ in range(2)] if fab.world > 1 else None
        self._calls = 0
        # W_uk^T per head: [hl, latent, nope], the [N, K] operand of the absorb GEMM
        self.w_uk_t = [dec.w[f"layers.{l}.kv_b"][:, :c.nope, :].transpose(1, 2).contiguous() for l in range(c.layers)]
        # Prompt attention on the tensor cores (chunks of consecutive positions of one sequence): the context's latent rows are
        # gathered out of their pages, up-projected for all local heads by two GEMMs (keys as [ctx, heads x 256], values
        # transposed as [heads x 256, ctx]) and attended by the tcgen05 attention kernel in the per-head form - a third of the
        # arithmetic of attention over the 576-wide latent rows, no per-head projection launches, no split / merge passes.
        self.tc_attention = (not dec.kv_int8 and c.kv_lora == 512 and c.rope == 64 and c.nope == 128 and c.vdim == 128)
        if self.tc_attention:
            cap = (dec.max_context + 127) // 128 * 128
            self.ctx_lat = torch.zeros(cap, c.kv_lora, dtype=BF16, device=dev)
            self.ctx_pe = torch.zeros(cap, c.rope, dtype=BF16, device=dev)
            self.kv_up = e(cap, hl * (c.nope + c.vdim))
            self.kvt = e(hl * (c.nope + c.vdim), cap)
        self._contig = None            # (first position, slot) of the chunk being run, None for rows of many sequences
        self.launches = 0
        # CUDA graphs of the layer stack, one per row count (the few most recent): a chunk is ~100 launches per layer and at
        # 4-8 GPUs the host cannot issue them as fast as the devices finish them. The all-reduce staging buffers alternate per
        # layer from host state, so a recorded pass replays correctly only if a pass leaves that state as it found it.
        self.use_graphs = fab.world == 1 or c.layers % 2 == 0
        self._graphs = {}

    def _layers_graphed(self, m: int) -> torch.Tensor:
        if not self.use_graphs:
            return self._layers(m)
        key = (m, self._contig if self.tc_attention else None)       # the tensor-core attention bakes positions into its launches
        g = self._graphs.get(key)
        if g is not None:
            g.replay()
            return self.x[:m]
        x = self._layers(m)                         # the real run of this chunk (and the warm-up of the capture)
        torch.cuda.synchronize()
        calls = self._calls
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):                   # records only: caches and counters are not touched a second time
            self._layers(m)
        self._calls = calls
        if len(self._graphs) >= 4:
            self._graphs.pop(next(iter(self._graphs)))
        self._graphs[key] = g
        return x

    def forward(self, tokens: torch.Tensor, pos0: int, slot: int = 0) -> torch.Tensor:
        """Run ``tokens`` (int32 ``[m]``, ``m <= max_rows``, already on the device) at positions ``pos0 .. pos0+m-1``
        of sequence slot ``slot``; returns the greedy next token after the last row (device tensor ``[1]``)."""
        d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
        w, st, hl = d.w, fab.desc.status, d.hl
        m = tokens.numel()
        assert 1 <= m <= self.M
        self.tokens[:m].copy_(tokens)
        self.positions[:m].copy_(torch.arange(pos0, pos0 + m, dtype=torch.int32, device=tokens.device))
        self.slots[:m].fill_(slot)
        self._contig = (int(pos0), int(slot))
        x = self._layers_graphed(m)
        # greedy token after the last row through the decode head (vocabulary-sharded argmax exchange included)
        K.lm_head_argmax(x[m - 1:m], w["lm_head"], fab, norm_w=w["final_norm"], eps=c.eps, vocab_offset=d.rank * d.vl,
                         partial=d.partial, logits=None if d.logits is None else d.logits[:1], out_ids=d.next_ids[:1],
                         out_vals=d.next_vals[:1])
        self.launches += 1
        return d.next_ids[:1]

    def forward_rows(self, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, select: torch.Tensor) -> torch.Tensor:
        """Batched step over ``m`` independent rows (own position and sequence slot per row, e.g. one decode row per running
        sequence): attention per row over its own cache pages, the experts through the device-side dispatch and the grouped
        GEMM, then the vocabulary shard of the logits of rows ``select`` (int64 indices) from one GEMM (f32 ``[k, vocab_local]``)."""
        d, c = self.dec, self.dec.cfg
        m = tokens.numel()
        assert 1 <= m <= self.M
        self.tokens[:m].copy_(tokens)
        self.positions[:m].copy_(positions)
        self.slots[:m].copy_(slots)
        self._contig = None
        x = self._layers_graphed(m)
        xn = K.rmsnorm(x.index_select(0, select), d.w["final_norm"], c.eps)
        self.launches += 2
        return G.gemm(xn, d.w["lm_head"], out_f32=True, status_ptr=d.fabric.desc.status)

    def _layers(self, m: int) -> torch.Tensor:
        """Embedding + all layers over the ``m`` rows staged in ``tokens / positions / slots``; returns the hidden rows."""
        d, c, fab = self.dec, self.dec.cfg, self.dec.fabric
        w, st, hl = d.w, fab.desc.status, d.hl
        tok, pos, sl = self.tokens[:m], self.positions[:m], self.slots[:m]
        x, h = self.x[:m], self.h[:m]
        n_launch = 0
        K.embedding(tok, w["embed"], out=x, status_ptr=st)
        self.shared_ntiles.fill_((m + 127) // 128)
        for l in range(c.layers):
            p = f"layers.{l}."
            # ---- attention ----
            K.rmsnorm(x, w[p + "attn_norm"], c.eps, out=h)
            qkv = G.gemm(h, w[p + "qkv_a"], out=self.qkv[:m], status_ptr=st)
            if d.kv_int8:
                K.mla_kv_write_q8(qkv[:, c.q_lora:], w[p + "kv_a_norm"], pos, sl, d.page_table, d.caches[l], eps=c.eps, theta=c.theta,
                                  status_ptr=st)
            else:
                K.mla_kv_write(qkv[:, c.q_lora:], w[p + "kv_a_norm"], pos, sl, d.page_table, d.caches[l], latent=c.kv_lora,
                               rope=c.rope, eps=c.eps, theta=c.theta, status_ptr=st)
            K.rmsnorm(qkv[:, :c.q_lora], w[p + "q_a_norm"], c.eps, out=self.qn[:m])
            q = G.gemm(self.qn[:m], w[p + "q_b"], out=self.q[:m], status_ptr=st)
            q_lat, o_lat, attn = self.q_lat[:m], self.o_lat[:m], self.attn[:m]
            if self.tc_attention and self._contig is not None:
                pos0, slot = self._contig
                ctx = pos0 + m
                rows = (ctx + 63) // 64 * 64
                kvb = w[p + "kv_b"].view(hl * (c.nope + c.vdim), c.kv_lora)
                P.mla_ctx_gather(d.caches[l], d.page_table, slot, ctx, self.ctx_lat[:rows], self.ctx_pe[:rows], status_ptr=st)
                G.gemm(self.ctx_lat[:rows], kvb, out=self.kv_up[:rows], status_ptr=st)
                G.gemm(kvb, self.ctx_lat[:rows], out=self.kvt[:, :rows], status_ptr=st)
                P.mla_q_rope_inplace(q, pos, heads=hl, nope=c.nope, rope=c.rope, theta=c.theta)
                P.fa_prefill(q, self.kv_up, self.kvt, attn, heads=hl, q_head_stride=c.qk_dim, k_head_stride=c.nope + c.vdim,
                             vt_head_stride=c.nope + c.vdim, vt_row0=c.nope, d1=c.nope, d2=c.rope, k2=self.ctx_pe, ctx=ctx, pos0=pos0,
                             scale=c.scale, window=c.window, status_ptr=st)
                n_launch += 5 - 2 * hl - 1 - 2 * ((m + self.QC - 1) // self.QC)
            else:
                self._latent_attention(l, m, q, q_lat, o_lat, attn)
            if fab.world > 1:
                G.gemm_allreduce(attn, w[p + "o_proj"], fab, self._sym_rows(m), residual=x)
            else:
                G.gemm(attn, w[p + "o_proj"], residual=x, out=x, status_ptr=st)
            # ---- MoE ----
            P.router_block(x, w[p + "router"], c.topk, self.ids[:m], self.wts[:m], norm_w=w[p + "ffn_norm"], eps=c.eps,
                           scoring=c.scoring, scale=c.route_scale, xn=h)
            P.moe_dispatch(self.ids[:m], d.rank * d.el, d.el, self.route)
            P.moe_gather(h, self.route, self.xp)
            if self.w8 is not None:
                ew = {name: K.dequantize_fp8_block(self.w8[p + name], out=buf) for name, buf in self.wide.items()}
                n_launch += 4
            else:
                ew = {name: w[p + name] for name in ("gate_up", "down", "shared_gate_up", "shared_down")}
            P.grouped_gemm(self.xp, ew["gate_up"], self.route.tiles, self.route.num_tiles, self.act, swiglu=True, status_ptr=st)
            P.grouped_gemm(self.act, ew["down"], self.route.tiles, self.route.num_tiles, self.y, status_ptr=st)
            sgu, sdn = ew["shared_gate_up"], ew["shared_down"]
            if m >= 256 and (sgu.shape[0] // 2) % 32 == 0:
                G.gemm_swiglu(h, sgu, out=self.sact[:m], status_ptr=st)      # the shared expert's gate | up on CTA pairs
            else:
                P.grouped_gemm(h, sgu.unsqueeze(0), self.shared_tiles, self.shared_ntiles, self.sact[:m], swiglu=True, status_ptr=st)
            G.gemm(self.sact[:m], sdn, out=self.sd[:m], status_ptr=st)
            if fab.world > 1:
                part = self.parts[self._calls & 1]
                self._calls += 1
                P.moe_combine(self.y, self.route, self.wts[:m], shared=self.sd[:m], out_f32=part.tensor[:m])
                P.allreduce_rows(part, fab, x, residual=x)
            else:
                P.moe_combine(self.y, self.route, self.wts[:m], shared=self.sd[:m], residual=x, out=x)
            n_launch += 17 + 2 * hl + 2 * ((m + self.QC - 1) // self.QC)
        self.launches = n_launch + 1
        return x

    def _latent_attention(self, l: int, m: int, q, q_lat, o_lat, attn) -> None:
        """Attention of layer ``l`` in the absorbed (latent) form on the split-KV kernels, one query row per token with its own
        position and sequence slot: the form for rows of many sequences, quantised caches and head shapes the tensor-core
        kernel does not take."""
        d, c = self.dec, self.dec.cfg
        w, st, hl = d.w, d.fabric.desc.status, d.hl
        p = f"layers.{l}."
        pos, sl = self.positions[:m], self.slots[:m]
        for hh in range(hl):
            G.gemm(q[:, hh * c.qk_dim: hh * c.qk_dim + c.nope], self.w_uk_t[l][hh], out=q_lat[:, hh, :c.kv_lora], status_ptr=st)
        P.mla_q_rope(q, pos, q_lat, nope=c.nope, rope=c.rope, theta=c.theta)
        for q0 in range(0, m, self.QC):
            q1 = min(m, q0 + self.QC)
            P.mla_split(q_lat[q0:q1], d.caches[l], pos[q0:q1], sl[q0:q1], d.page_table, self.scratch, scale=c.scale,
                        window=c.window, keys_per_split=d.kps, max_splits=d.max_splits, status_ptr=st, packed=d.kv_int8)
            P.mla_merge(self.scratch, pos[q0:q1], o_lat[q0:q1], window=c.window, keys_per_split=d.kps, max_splits=d.max_splits)
        kvb = w[p + "kv_b"]
        for hh in range(hl):
            G.gemm(o_lat[:, hh, :], kvb[hh, c.nope:, :], out=attn[:, hh * c.vdim:(hh + 1) * c.vdim], status_ptr=st)

    def _sym_rows(self, m: int):
        """The symmetric activation buffer restricted to ``m`` rows (same peer pointers, smaller shape)."""
        if m == self.M:
            return self.x_sym
        v = object.__new__(type(self.x_sym))
        v.__dict__.update(self.x_sym.__dict__)
        v.tensor = self.x_sym.tensor[:m]
        return v
