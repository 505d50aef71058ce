"""Dense GQA decoder (Qwen-style: RMSNorm, RoPE, grouped-query attention, SwiGLU FFN) on the sm_100a
decode kernels, with tensor parallelism over the fused row-parallel GEMV + all-reduce.

Per layer and step: qkv GEMV (norm prologue) -> RoPE + paged KV append -> split-KV GQA attention ->
o_proj GEMV fused with all-reduce + residual -> gate_up GEMV (norm prologue, SwiGLU epilogue) ->
down GEMV fused with all-reduce + residual. 7 launches per layer, no stand-alone collective.
Query rows of different sequences (continuous batching) share every launch: each row carries its
own position and sequence slot. Sampling is greedy (fused with the lm_head) or top-k / top-p on the
device. The reference's dense family runs per-layer composites of vendor ops with an all-gather
after every sharded projection (native/src/inferfabric_acl.cpp:688-755, 1236-1433).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import decode as K
from ..parallel.fabric import Fabric

BF16 = torch.bfloat16


@dataclass
class DenseConfig:
    layers: int = 24
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 4
    head_dim: int = 128
    ffn: int = 6144
    vocab: int = 151936
    theta: float = 1e6
    eps: float = 1e-6
    page_tokens: int = 16

    @staticmethod
    def qwen2b() -> "DenseConfig":
        """Qwen-style 2B: 24 layers, hidden 2048, 16 query / 4 KV heads x 128, SwiGLU 6144, vocab 151936."""
        return DenseConfig()

    @staticmethod
    def tiny(layers: int = 2) -> "DenseConfig":
        return DenseConfig(layers=layers, hidden=256, heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=1024, theta=1e4)

    def param_count(self) -> int:
        c = self
        per = c.hidden * (c.heads + 2 * c.kv_heads) * c.head_dim + c.heads * c.head_dim * c.hidden + 3 * c.hidden * c.ffn + 2 * c.hidden
        return per * c.layers + 2 * c.vocab * c.hidden + c.hidden


def full_weight_shapes(c: DenseConfig) -> Dict[str, tuple]:
    s = {"embed": (c.vocab, c.hidden), "final_norm": (c.hidden,), "lm_head": (c.vocab, c.hidden)}
    for l in range(c.layers):
        p = f"layers.{l}."
        s[p + "attn_norm"] = (c.hidden,)
        s[p + "qkv"] = ((c.heads + 2 * c.kv_heads) * c.head_dim, c.hidden)
        s[p + "o_proj"] = (c.hidden, c.heads * c.head_dim)
        s[p + "ffn_norm"] = (c.hidden,)
        s[p + "gate_up"] = (2 * c.ffn, c.hidden)
        s[p + "down"] = (c.hidden, c.ffn)
    return s


def random_full_weights(c: DenseConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, shape in full_weight_shapes(c).items():
        t = torch.randn(shape, generator=g, dtype=torch.float32) * 0.02
        if name.endswith("norm"):
            t = t + 1.0
        out[name] = t.to(BF16).to(device)
    return out


def shard_weights(c: DenseConfig, full: Dict[str, torch.Tensor], rank: int, world: int, device) -> Dict[str, torch.Tensor]:
    hq, hk, fl, vl, hd = c.heads // world, c.kv_heads // world, c.ffn // world, c.vocab // world, c.head_dim
    out = {}
    for name, t in full.items():
        base = name.split(".")[-1]
        if base == "qkv":
            q, k, v = t[:c.heads * hd], t[c.heads * hd:(c.heads + c.kv_heads) * hd], t[(c.heads + c.kv_heads) * hd:]
            t = torch.cat([q[rank * hq * hd:(rank + 1) * hq * hd], k[rank * hk * hd:(rank + 1) * hk * hd], v[rank * hk * hd:(rank + 1) * hk * hd]], 0)
        elif base == "o_proj":
            t = t[:, rank * hq * hd:(rank + 1) * hq * hd]
        elif base == "gate_up":
            t = torch.cat([t[rank * fl:(rank + 1) * fl], t[c.ffn + rank * fl:c.ffn + (rank + 1) * fl]], 0)
        elif base == "down":
            t = t[:, rank * fl:(rank + 1) * fl]
        elif base == "lm_head":
            t = t[rank * vl:(rank + 1) * vl]
        out[name] = t.contiguous().to(device)
    return out


def random_rank_weights(c: DenseConfig, rank: int, world: int, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init this rank's shard on the device (replicated tensors share a seed across ranks)."""
    hq, hk, fl, vl, hd = c.heads // world, c.kv_heads // world, c.ffn // world, c.vocab // world, c.head_dim
    shapes = {"qkv": ((hq + 2 * hk) * hd, c.hidden), "o_proj": (c.hidden, hq * hd), "gate_up": (2 * fl, c.hidden),
              "down": (c.hidden, fl), "lm_head": (vl, c.hidden)}
    shared = torch.Generator(device=device).manual_seed(seed)
    local = torch.Generator(device=device).manual_seed(seed * 1000 + 17 + rank)
    out = {}
    for name, shape in full_weight_shapes(c).items():
        base = name.split(".")[-1]
        t = torch.empty(shapes.get(base, shape), dtype=BF16, device=device)
        t.normal_(0.0, 0.02, generator=local if base in shapes else shared)
        if base.endswith("norm"):
            t += 1.0
        out[name] = t
    return out


def bundle_parameters(cfg: DenseConfig, weights: Dict[str, torch.Tensor], world: int = 1, prefix: str = "model") -> Dict[str, torch.Tensor]:
    """This module's per-rank weight tensors under the parameter names of a bundle compiled from
    ``compiler.sources.dense_gqa_source`` (``model.layers.N.self_attn.q_proj`` ..., pairs joined by ``|``). The q / k / v
    matrices are row ranges of the packed projection - the same storage, so the bundle's engine finds them back to back and runs
    one packed projection without copying them."""
    c = cfg
    hq, hk, hd = c.heads // world, c.kv_heads // world, c.head_dim
    out = {f"{prefix}.embed_tokens": weights["embed"], f"{prefix}.norm": weights["final_norm"], "lm_head": weights["lm_head"]}
    for l in range(c.layers):
        p, q = f"layers.{l}.", f"{prefix}.layers.{l}."
        a, m = q + "self_attn.", q + "mlp."
        qkv = weights[p + "qkv"]
        out[q + "input_layernorm"], out[q + "post_attention_layernorm"] = weights[p + "attn_norm"], weights[p + "ffn_norm"]
        out[a + "q_proj"], out[a + "k_proj"], out[a + "v_proj"] = qkv[:hq * hd], qkv[hq * hd:(hq + hk) * hd], qkv[(hq + hk) * hd:]
        out[a + "o_proj"] = weights[p + "o_proj"]
        out[m + "gate_proj|" + m + "up_proj"] = weights[p + "gate_up"]
        out[m + "down_proj"] = weights[p + "down"]
    return out


class DenseDecoder:
    """Per-rank executor for up to ``max_tokens`` (<= 8) query rows per launch group; larger batches are
    processed in tiles of 8 rows by :meth:`forward`."""

    def __init__(self, cfg: DenseConfig, weights: Dict[str, torch.Tensor], fabric: Fabric, *, max_tokens: int = 8,
                 max_context: int = 1024, num_slots: int = 1, keys_per_split: int = 64, keep_logits: bool = False,
                 num_pages: Optional[int] = None):
        self.cfg, self.w, self.fabric = cfg, weights, fabric
        self.rank, self.world = fabric.rank, fabric.world
        c, dev = cfg, fabric.device
        assert c.heads % self.world == 0 and c.kv_heads % self.world == 0 and c.ffn % (8 * self.world) == 0 and c.vocab % self.world == 0
        self.hq, self.hk, self.vl = c.heads // self.world, c.kv_heads // self.world, c.vocab // self.world
        self.T = max_tokens
        self.max_context = max_context
        self.max_pages = (max_context + c.page_tokens - 1) // c.page_tokens
        self.num_slots = num_slots
        self.num_pages = num_pages or self.max_pages * num_slots
        self.kps = keys_per_split
        self.max_splits = max(1, min(64, (max_context + keys_per_split - 1) // keys_per_split))
        while self.max_splits * self.kps < max_context:
            self.kps *= 2
        T = self.T
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(T, dtype=torch.int32, device=dev)
        self.page_table = torch.arange(self.max_pages * num_slots, dtype=torch.int32, device=dev).remainder(self.num_pages) \
            .view(num_slots, self.max_pages).contiguous()
        self.k_cache = [torch.zeros(self.num_pages, c.page_tokens, self.hk, c.head_dim, dtype=BF16, device=dev) for _ in range(c.layers)]
        self.v_cache = [torch.zeros_like(self.k_cache[0]) for _ in range(c.layers)]
        e = lambda *s, dt=BF16: torch.empty(*s, dtype=dt, device=dev)
        self.x = e(T, c.hidden)
        self.qkv = e(T, (self.hq + 2 * self.hk) * c.head_dim)
        self.attn = e(T, self.hq * c.head_dim)
        self.act = e(T, c.ffn // self.world)
        self.scratch = e(T * self.hq * self.max_splits * (c.head_dim + 2), dt=torch.float32)
        self.partial = e(((self.vl + 7) // 8) * 8 * 2, dt=torch.float32)
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_vals = torch.zeros(T, dtype=torch.float32, device=dev)
        self.logits = e(T, self.vl, dt=torch.float32) if keep_logits else None
        self.launches_per_forward = 2 + 8 * c.layers
        self._graph = None

    def forward(self, T: Optional[int] = None, sample: bool = True) -> torch.Tensor:
        c, w, fab = self.cfg, self.w, self.fabric
        T = self.T if T is None else T
        tok, pos, slot = self.tokens[:T], self.positions[:T], self.slots[:T]
        x, st = self.x[:T], fab.desc.status
        K.embedding(tok, w["embed"], out=x, status_ptr=st)
        for l in range(c.layers):
            p = f"layers.{l}."
            qkv = self.qkv[:T]
            K.gemv(x, w[p + "qkv"], norm_w=w[p + "attn_norm"], eps=c.eps, out=qkv)
            K.gqa_rope_kv_write(qkv, pos, slot, self.page_table, self.k_cache[l], self.v_cache[l], heads=self.hq,
                                kv_heads=self.hk, head_dim=c.head_dim, theta=c.theta, status_ptr=st)
            K.gqa_decode_attention(qkv, self.k_cache[l], self.v_cache[l], pos, slot, self.page_table, heads=self.hq,
                                   kv_heads=self.hk, head_dim=c.head_dim, scale=1.0 / math.sqrt(c.head_dim),
                                   keys_per_split=self.kps, max_splits=self.max_splits, scratch=self.scratch,
                                   out=self.attn[:T], status_ptr=st)
            K.gemv_allreduce(self.attn[:T], w[p + "o_proj"], fab, residual=x, out=x)
            K.gemv(x, w[p + "gate_up"], norm_w=w[p + "ffn_norm"], eps=c.eps, swiglu=True, out=self.act[:T])
            K.gemv_allreduce(self.act[:T], w[p + "down"], fab, residual=x, out=x)
        if sample:
            K.lm_head_argmax(x, w["lm_head"], fab, norm_w=w["final_norm"], eps=c.eps, vocab_offset=self.rank * self.vl,
                             partial=self.partial, logits=None if self.logits is None else self.logits[:T],
                             out_ids=self.next_ids[:T], out_vals=self.next_vals[:T])
        return self.next_ids[:T]

    def capture(self, T: Optional[int] = None, feedback: bool = False):
        T = self.T if T is None else T
        self.forward(T)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward(T)
            if feedback:
                self.tokens[:T].copy_(self.next_ids[:T])
                self.positions[:T].add_(1)
        self._graph = g
        return g

    def reset(self) -> None:
        for t in self.k_cache + self.v_cache:
            t.zero_()


def forward_ref(c: DenseConfig, W: Dict[str, torch.Tensor], tokens: torch.Tensor, tp: int = 1) -> torch.Tensor:
    """Plain PyTorch fp32 restatement (bf16 rounding where the device stores bf16): logits [T, vocab]."""
    from .mla_moe_ref import _r, rmsnorm_ref, rope_ref

    dev, T = tokens.device, tokens.numel()
    pos = torch.arange(T, device=dev)
    f = lambda n: W[n].to(dev).float()
    x = f("embed")[tokens.long()]
    causal = torch.ones(T, T, dtype=torch.bool, device=dev).tril()
    hd, G = c.head_dim, c.heads // c.kv_heads

    def ksplit(a, w):
        step = a.shape[-1] // tp
        out = torch.zeros(a.shape[0], w.shape[0], device=dev)
        for r in range(tp):
            out = out + a[:, r * step:(r + 1) * step] @ w[:, r * step:(r + 1) * step].T
        return out

    for l in range(c.layers):
        p = f"layers.{l}."
        qkv = _r(rmsnorm_ref(x, f(p + "attn_norm"), c.eps) @ f(p + "qkv").T)
        q = rope_ref(qkv[:, :c.heads * hd].view(T, c.heads, hd), pos, c.theta)
        k = rope_ref(qkv[:, c.heads * hd:(c.heads + c.kv_heads) * hd].view(T, c.kv_heads, hd), pos, c.theta)
        v = qkv[:, (c.heads + c.kv_heads) * hd:].view(T, c.kv_heads, hd)
        kx, vx = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
        s = torch.einsum("thd,shd->hts", q, kx) / math.sqrt(hd)
        s = s.masked_fill(~causal[None], float("-inf"))
        o = _r(torch.einsum("hts,shd->thd", torch.softmax(s, -1), vx)).reshape(T, c.heads * hd)
        x = _r(_r(ksplit(o, f(p + "o_proj"))) + x)
        gu = _r(rmsnorm_ref(x, f(p + "ffn_norm"), c.eps) @ f(p + "gate_up").T)
        a = _r(torch.nn.functional.silu(gu[:, :c.ffn]) * gu[:, c.ffn:])
        x = _r(_r(ksplit(a, f(p + "down"))) + x)
    return rmsnorm_ref(x, f("final_norm"), c.eps) @ f("lm_head").T
