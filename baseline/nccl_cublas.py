"""Library-only baseline of the MLA + MoE decoder: cuBLAS (torch.matmul / bmm) + NCCL all-reduce.

Same model, same per-rank weight shards, same sharding (TP over heads / shared expert / vocabulary,
EP over routed experts) and the same bf16 storage points as ``ironpangu_b200.models.mla_moe``, but
every operator is a stock PyTorch call and every collective is ``torch.distributed.all_reduce``. It
uses none of the package's kernels, so ``bench.py --impl nccl_cublas`` shows what the hand-written
fused kernels buy on the same box. The class exposes the attributes ``DecodeEngine`` drives
(``T``, ``tokens``, ``positions``, ``slots``, ``next_ids``, ``forward``) and is CUDA-graph capturable:
all shapes are static and nothing synchronises with the host.

Design notes (what a careful user of the libraries would write, not a strawman):
  * the KV cache is a dense ``[max_context, latent + rope]`` tensor per layer; attention runs in the
    absorbed MLA form over the whole cache with a position mask, as two batched GEMMs
  * routed experts: the routes of all rows are sorted by local expert and applied with the library's grouped GEMM
    (``torch._grouped_mm``: one call for gate/up, one for down, reading each selected expert's weights once and no
    others); routes owned by other ranks sort behind the last group and contribute zero. Where the installed
    library has no grouped GEMM for this device the selected experts are gathered with ``index_select`` and applied with
    ``torch.bmm`` (the gather triples the expert traffic); ``expert_path`` says which ran
  * RMSNorm is the fused ``torch.nn.functional.rms_norm``
  * one NCCL all-reduce after the attention output projection, one after the MoE, one all-gather-free
    argmax exchange (max of values, then min of the matching index) for the vocabulary-sharded head
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

BF16 = torch.bfloat16


class NcclCublasDecoder:
    def __init__(self, cfg, weights: Dict[str, torch.Tensor], rank: int, world: int, *, max_tokens: int = 8,
                 max_context: int = 1024, keep_logits: bool = False):
        self.cfg, self.w, self.rank, self.world = cfg, weights, rank, world
        c = cfg
        dev = weights["embed"].device
        self.hl, self.el, self.vl = c.heads // world, c.experts // world, c.vocab // world
        self.T, self.max_context = max_tokens, max_context
        T = max_tokens
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_vals = torch.zeros(T, dtype=torch.float32, device=dev)
        self.caches = [torch.zeros(max_context, c.kv_lora + c.rope, dtype=BF16, device=dev) for _ in range(c.layers)]
        self.key_index = torch.arange(max_context, device=dev)
        half = c.rope // 2
        i = torch.arange(half, device=dev, dtype=torch.float32)
        self.inv_freq = torch.exp2(-(2.0 * i / c.rope) * math.log2(c.theta))
        self.logits = torch.empty(T, self.vl, dtype=torch.float32, device=dev) if keep_logits else None
        # library launches per forward, counted from the operator list below (for the bench record only)
        self.launches_per_forward = 0
        self.expert_arange = torch.arange(self.el, device=dev)
        self.expert_path = "grouped_mm" if self._grouped_mm_works() else "index_select+bmm"

    def _grouped_mm_works(self) -> bool:
        """One tiny call decides: the grouped GEMM of the installed library either supports this device and layout or not."""
        if not hasattr(torch, "_grouped_mm"):
            return False
        try:
            dev = self.tokens.device
            a = torch.zeros(8, 64, dtype=BF16, device=dev)
            b = torch.zeros(2, 32, 64, dtype=BF16, device=dev)
            offs = torch.tensor([3, 8], dtype=torch.int32, device=dev)
            torch._grouped_mm(a, b.transpose(1, 2), offs=offs)
            torch.cuda.synchronize()
            return True
        except Exception:
            return False

    # -- helpers -----------------------------------------------------------------------------------
    @staticmethod
    def _norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), w, eps)

    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Half-rotation RoPE, bf16-rounded tables; x [T, ..., d]."""
        ang = pos.float()[:, None] * self.inv_freq[None, :]
        cs, sn = torch.cos(ang).to(BF16).float(), torch.sin(ang).to(BF16).float()
        while cs.dim() < x.dim():
            cs, sn = cs.unsqueeze(1), sn.unsqueeze(1)
        half = x.shape[-1] // 2
        a, b = x[..., :half].float(), x[..., half:].float()
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).to(BF16)

    def _allreduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t)
        return t

    # -- one step ----------------------------------------------------------------------------------
    def forward(self, T: Optional[int] = None) -> torch.Tensor:
        c, w = self.cfg, self.w
        T = self.T if T is None else T
        tok, pos = self.tokens[:T].long(), self.positions[:T].long()
        x = w["embed"][tok]
        # keys visible to row t: index <= position (and inside the sliding window when there is one)
        visible = self.key_index[None, :] <= pos[:, None]
        if c.window > 0:
            visible &= self.key_index[None, :] > (pos[:, None] - c.window)
        for l in range(c.layers):
            p = f"layers.{l}."
            qkv = self._norm(x, w[p + "attn_norm"], c.eps) @ w[p + "qkv_a"].T
            q_a, latent, k_pe = qkv[:, :c.q_lora], qkv[:, c.q_lora:c.q_lora + c.kv_lora], qkv[:, c.q_lora + c.kv_lora:]
            row = torch.cat([self._norm(latent, w[p + "kv_a_norm"], c.eps), self._rope(k_pe, pos)], -1)
            cache = self.caches[l]
            cache.index_copy_(0, pos, row)
            q = (self._norm(q_a, w[p + "q_a_norm"], c.eps) @ w[p + "q_b"].T).view(T, self.hl, c.qk_dim)
            kvb = w[p + "kv_b"]                                                # [hl, nope + v, latent]
            q_lat = torch.bmm(q[..., :c.nope].transpose(0, 1), kvb[:, :c.nope])          # [hl, T, latent]
            q_full = torch.cat([q_lat.transpose(0, 1), self._rope(q[..., c.nope:], pos)], -1)   # [T, hl, latent+rope]
            s = torch.matmul(q_full.reshape(T * self.hl, -1), cache.T).float().view(T, self.hl, -1) * c.scale
            s = s.masked_fill(~visible[:, None, :], float("-inf"))
            pr = torch.softmax(s, -1).to(BF16)
            o_lat = torch.matmul(pr.view(T * self.hl, -1), cache[:, :c.kv_lora]).view(T, self.hl, c.kv_lora)
            attn = torch.bmm(o_lat.transpose(0, 1), kvb[:, c.nope:].transpose(1, 2)).transpose(0, 1).reshape(T, self.hl * c.vdim)
            part = torch.matmul(attn, w[p + "o_proj"].T).float()
            x = (self._allreduce(part).to(BF16).float() + x.float()).to(BF16)

            h2 = self._norm(x, w[p + "ffn_norm"], c.eps)
            scores = h2.float() @ w[p + "router"].T
            if c.scoring == "softmax":
                prob = torch.softmax(scores, -1)
                wts, ids = torch.topk(prob, c.topk, dim=-1)
                wts = wts / wts.sum(-1, keepdim=True)
            else:
                prob = torch.sigmoid(scores)
                wts, ids = torch.topk(prob, c.topk, dim=-1)
                wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
            wts = wts * c.route_scale
            local = ids - self.rank * self.el
            mine = (local >= 0) & (local < self.el)
            local = torch.where(mine, local, torch.zeros_like(local)).reshape(-1)
            wts = torch.where(mine, wts, torch.zeros_like(wts))
            if self.expert_path == "grouped_mm":
                moe = self._experts_grouped(h2, local, mine.reshape(-1), wts.reshape(-1), w[p + "gate_up"], w[p + "down"], T)
            else:
                moe = torch.empty(T, c.hidden, dtype=torch.float32, device=x.device)
                for r0 in range(0, T, 2):                                      # two rows at a time bounds the gather buffers
                    r1 = min(T, r0 + 2)
                    sel = local[r0 * c.topk:r1 * c.topk]
                    gu = w[p + "gate_up"].index_select(0, sel)                 # [rows*topk, 2F, D]
                    dn = w[p + "down"].index_select(0, sel)                    # [rows*topk, D, F]
                    hx = h2[r0:r1].repeat_interleave(c.topk, 0).unsqueeze(2)   # [rows*topk, D, 1]
                    g_u = torch.bmm(gu, hx).squeeze(2)
                    act = (F.silu(g_u[:, :c.expert_ffn].float()) * g_u[:, c.expert_ffn:].float()).to(BF16)
                    y = torch.bmm(dn, act.unsqueeze(2)).squeeze(2).float().view(r1 - r0, c.topk, c.hidden)
                    moe[r0:r1] = (y * wts[r0:r1, :, None]).sum(1)
            sg = h2 @ w[p + "shared_gate_up"].T
            fs = sg.shape[1] // 2
            sact = (F.silu(sg[:, :fs].float()) * sg[:, fs:].float()).to(BF16)
            moe = moe + torch.matmul(sact, w[p + "shared_down"].T).float()
            x = (self._allreduce(moe).to(BF16).float() + x.float()).to(BF16)

        logits = torch.matmul(self._norm(x, w["final_norm"], c.eps), w["lm_head"].T).float()
        if self.logits is not None:
            self.logits[:T].copy_(logits)
        val, idx = logits.max(-1)
        idx = idx + self.rank * self.vl
        if self.world > 1:
            best = val.clone()
            dist.all_reduce(best, op=dist.ReduceOp.MAX)
            idx = torch.where(val == best, idx, torch.full_like(idx, 2 ** 31 - 1))
            dist.all_reduce(idx, op=dist.ReduceOp.MIN)
            val = best
        self.next_ids[:T].copy_(idx.to(torch.int32))
        self.next_vals[:T].copy_(val)
        return self.next_ids[:T]

    def _experts_grouped(self, h2, local, mine, wts, w_gu, w_down, T: int) -> torch.Tensor:
        """Routed experts through the library's grouped GEMM. Routes are sorted by local expert (foreign routes behind the
        last group, outside every offset, never computed); all shapes are static, nothing synchronises with the host."""
        c = self.cfg
        key = torch.where(mine, local, torch.full_like(local, self.el))
        order = torch.argsort(key, stable=True)
        skey = key[order]
        counts = (skey[:, None] == self.expert_arange[None, :]).sum(0)
        offs = torch.cumsum(counts, 0).to(torch.int32)
        token = torch.div(order, c.topk, rounding_mode="floor")
        xs = h2[token]                                                        # [R, D]
        g_u = torch._grouped_mm(xs, w_gu.transpose(1, 2), offs=offs)          # [R, 2F]
        act = (F.silu(g_u[:, :c.expert_ffn].float()) * g_u[:, c.expert_ffn:].float()).to(BF16)
        y = torch._grouped_mm(act, w_down.transpose(1, 2), offs=offs).float()   # [R, D]
        y = torch.where(mine[order][:, None], y * wts[order][:, None], torch.zeros_like(y))
        return torch.zeros(T, c.hidden, dtype=torch.float32, device=h2.device).index_add_(0, token, y)

    def reset(self) -> None:
        for cch in self.caches:
            cch.zero_()
