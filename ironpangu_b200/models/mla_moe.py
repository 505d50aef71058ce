"""MLA + MoE decoder (the 92B-class flagship family) on the sm_100a decode kernels.

Layer structure (pre-norm residual blocks)::

    x += o_proj( MLA( norm(x) ) )          q_a|kv_a paired, q_b tp_rows, o_proj tp_columns + all-reduce
    x += MoE( norm(x) ) + Shared( norm(x) ) routed experts owner-local (EP = TP group), shared expert
                                            sharded along its intermediate dim; one fused all-reduce

The reference's OpenPangu module set has the same skeleton (paired q_a/kv_a projection, absorbed
``mla_query``, ``latent_attention``, ``mla_value``, K-sharded ``o_proj`` + ``allreduce``, ``router`` +
``expert_linear``/``expert_swiglu_down``/``expert_reduce`` + ``allreduce``:
examples/openpangu/92b-tp8-ep8.inferfabric:29-75); dims here are attributes of :class:`MlaMoeConfig`,
not constants.

Per decode step and layer this path launches 6 kernels (qkv_a, the cluster-per-head attention kernel, o_proj, router,
expert gate/up, expert down; 10 with the attention steps as separate kernels) and no stand-alone collective: both
all-reduces live inside the o_proj / expert-down kernels, and greedy sampling is fused with the
vocabulary-sharded lm_head.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import decode as K
from ..parallel.fabric import Fabric

BF16 = torch.bfloat16


@dataclass
class MlaMoeConfig:
    layers: int = 46
    hidden: int = 4096
    vocab: int = 153600
    heads: int = 32
    q_lora: int = 1536
    kv_lora: int = 512
    nope: int = 128
    rope: int = 64
    vdim: int = 128
    experts: int = 96
    expert_ffn: int = 1536
    topk: int = 8
    shared_ffn: int = 1536
    theta: float = 6400000.0
    eps: float = 1e-5
    window: int = 0
    scoring: str = "softmax"
    route_scale: float = 1.0
    eos: int = -1
    page_tokens: int = 16

    @staticmethod
    def flagship() -> "MlaMoeConfig":
        """The 92B-class configuration: 46 layers, hidden 4096, 32 heads, 96 experts x 1536, top-8 + 1 shared."""
        return MlaMoeConfig()

    @staticmethod
    def tiny(layers: int = 2) -> "MlaMoeConfig":
        return MlaMoeConfig(layers=layers, hidden=256, vocab=1024, heads=8, q_lora=128, kv_lora=512, nope=32, rope=64,
                            vdim=32, experts=16, expert_ffn=64, topk=4, shared_ffn=64)

    @property
    def qk_dim(self) -> int:
        return self.nope + self.rope

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.qk_dim)

    def param_count(self) -> int:
        c = self
        per = (c.hidden * (c.q_lora + c.kv_lora + c.rope) + c.q_lora * c.heads * c.qk_dim +
               c.heads * (c.nope + c.vdim) * c.kv_lora + c.hidden * c.heads * c.vdim + c.experts * c.hidden +
               c.experts * 3 * c.hidden * c.expert_ffn + 3 * c.hidden * c.shared_ffn + 2 * c.hidden + c.q_lora + c.kv_lora)
        return per * c.layers + 2 * c.vocab * c.hidden + c.hidden


# ---------------------------------------------------------------------------------------------------
# Weights
# ---------------------------------------------------------------------------------------------------
def full_weight_shapes(cfg: MlaMoeConfig) -> Dict[str, tuple]:
    """Names and shapes of the unsharded checkpoint tensors."""
    c = cfg
    s: Dict[str, tuple] = {"embed": (c.vocab, c.hidden), "final_norm": (c.hidden,), "lm_head": (c.vocab, c.hidden)}
    for l in range(c.layers):
        p = f"layers.{l}."
        s[p + "attn_norm"] = (c.hidden,)
        s[p + "qkv_a"] = (c.q_lora + c.kv_lora + c.rope, c.hidden)
        s[p + "q_a_norm"] = (c.q_lora,)
        s[p + "kv_a_norm"] = (c.kv_lora,)
        s[p + "q_b"] = (c.heads * c.qk_dim, c.q_lora)
        s[p + "kv_b"] = (c.heads, c.nope + c.vdim, c.kv_lora)
        s[p + "o_proj"] = (c.hidden, c.heads * c.vdim)
        s[p + "ffn_norm"] = (c.hidden,)
        s[p + "router"] = (c.experts, c.hidden)
        s[p + "gate_up"] = (c.experts, 2 * c.expert_ffn, c.hidden)
        s[p + "down"] = (c.experts, c.hidden, c.expert_ffn)
        s[p + "shared_gate_up"] = (2 * c.shared_ffn, c.hidden)
        s[p + "shared_down"] = (c.hidden, c.shared_ffn)
    return s


def random_full_weights(cfg: MlaMoeConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """N(0, 0.02) weights (norm gains 1 + N(0, 0.02)), bf16 except the f32 router. For small configs / tests."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, shape in full_weight_shapes(cfg).items():
        t = torch.randn(shape, generator=g, dtype=torch.float32) * 0.02
        if name.endswith("norm"):
            t = t + 1.0
        out[name] = (t if name.endswith("router") else t.to(BF16)).to(device)
    return out


def shard_weights(cfg: MlaMoeConfig, full: Dict[str, torch.Tensor], rank: int, world: int, device) -> Dict[str, torch.Tensor]:
    """Slice an unsharded checkpoint for one rank (TP = EP = world)."""
    c = cfg
    hl, el, fs = c.heads // world, c.experts // world, c.shared_ffn // world
    out = {}
    for name, t in full.items():
        base = name.split(".")[-1]
        if base == "q_b":
            t = t.view(c.heads, c.qk_dim, c.q_lora)[rank * hl:(rank + 1) * hl].reshape(hl * c.qk_dim, c.q_lora)
        elif base == "kv_b":
            t = t[rank * hl:(rank + 1) * hl]
        elif base == "o_proj":
            t = t[:, rank * hl * c.vdim:(rank + 1) * hl * c.vdim]
        elif base in ("gate_up", "down"):
            t = t[rank * el:(rank + 1) * el]
        elif base == "shared_gate_up":
            t = torch.cat([t[rank * fs:(rank + 1) * fs], t[c.shared_ffn + rank * fs:c.shared_ffn + (rank + 1) * fs]], 0)
        elif base == "shared_down":
            t = t[:, rank * fs:(rank + 1) * fs]
        elif base == "lm_head":
            vl = c.vocab // world
            t = t[rank * vl:(rank + 1) * vl]
        out[name] = t.contiguous().to(device)
    return out


def random_rank_weights(cfg: MlaMoeConfig, rank: int, world: int, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init this rank's shard directly on the device (benchmarks: no host copy of a 175 GB model).

    Replicated tensors use a seed shared by all ranks so every rank holds identical values."""
    c = cfg
    hl, el, fs, vl = c.heads // world, c.experts // world, c.shared_ffn // world, c.vocab // world
    shapes = {
        "q_b": (hl * c.qk_dim, c.q_lora), "kv_b": (hl, c.nope + c.vdim, c.kv_lora), "o_proj": (c.hidden, hl * c.vdim),
        "gate_up": (el, 2 * c.expert_ffn, c.hidden), "down": (el, c.hidden, c.expert_ffn),
        "shared_gate_up": (2 * fs, c.hidden), "shared_down": (c.hidden, fs), "lm_head": (vl, c.hidden),
    }
    shared_gen = torch.Generator(device=device).manual_seed(seed)
    local_gen = torch.Generator(device=device).manual_seed(seed * 1000 + 17 + rank)
    out = {}
    for name, shape in full_weight_shapes(cfg).items():
        base = name.split(".")[-1]
        sharded = base in shapes
        shp = shapes.get(base, shape)
        gen = local_gen if sharded else shared_gen
        dt = torch.float32 if base == "router" else BF16
        t = torch.empty(shp, dtype=dt, device=device)
        t.normal_(0.0, 0.02, generator=gen)
        if base.endswith("norm"):
            t += 1.0
        out[name] = t
    return out


# ---------------------------------------------------------------------------------------------------
# Decoder
# ---------------------------------------------------------------------------------------------------
class MlaMoeDecoder:
    """Per-rank executor for up to ``max_tokens`` (<= 8) query rows per step.

    State: a paged latent KV cache per layer ``[pages, page_tokens, kv_lora + rope]`` and a page table
    ``[slots, max_pages]``. ``forward`` consumes device-resident ``tokens/positions/slots`` (int32) and
    leaves the greedy next token of every row in ``self.next_ids``; nothing crosses the host boundary.
    """

    def __init__(self, cfg: MlaMoeConfig, weights: Dict[str, torch.Tensor], fabric: Fabric, *, max_tokens: int = 1,
                 max_context: int = 1024, num_slots: int = 1, keys_per_split: int = 64, keep_logits: bool = False,
                 kv_int8: bool = False, expert_fp8: bool = False, drop_bf16_experts: bool = True,
                 fused_head: Optional[bool] = None, shard: Optional[tuple] = None, fused_moe: Optional[bool] = None,
                 l2_prefetch: Optional[bool] = None):
        """``kv_int8``: keep the latent cache as packed int8 rows (656 bytes per token instead of 1152).
        ``expert_fp8``: quantise the routed and shared expert matrices to block-scaled fp8 (1 x 128 scale blocks) at
        construction and decode over them; with ``drop_bf16_experts`` the bf16 originals leave ``weights``.
        ``fused_head``: run cache write, q_b, absorb, attention and value up-projection as one cluster-per-head launch
        (default: on for bf16 caches with contexts up to 2048 keys, and used for steps of one or two rows: measured on a
        B200 it takes 25 us against 38 us per layer at 32 heads and 19 against 29 us at 4 heads with 512 keys, while at 4096
        keys or 8 rows the split-KV kernels, which spread a head over up to 64 CTAs, are faster).
        ``fused_moe``: router, expert gate/up and expert down + all-reduce of a layer as one launch for steps of one or two
        rows (default: off - measured slower than the chain at 1, 2 and 8 GPUs; for bf16 experts up to 1536 wide; bit-identical to the
        three-kernel chain).
        ``shard``: ``(rank, world)`` of the weight shard when it differs from the fabric's (a profiling aid: one GPU runs the
        kernels of rank r of an N-rank job at their real shapes, without the peers; the sums it computes are partial)."""
        assert 1 <= max_tokens <= 8
        # the head kernel can ask for the weights of the layer's next kernels (o_proj, shared expert) while it runs; measured
        # 3.4 % slower at one GPU (the requests compete with the kernel's own loads), so off unless asked for
        self.l2_prefetch = False if l2_prefetch is None else bool(l2_prefetch)
        self.kv_int8 = kv_int8
        self.expert_fp8 = expert_fp8
        can_fuse = (not kv_int8 and cfg.kv_lora == 512 and cfg.rope == 64 and cfg.nope % 32 == 0 and cfg.nope <= 128 and
                    cfg.vdim <= 128 and cfg.q_lora % 8 == 0)
        self.can_fuse_head = can_fuse
        self.fused_ctx_limit = 2048
        self.fused_auto = fused_head is None      # engines that know the position may pick the kernel per step (fuse_override)
        self.fuse_override: Optional[bool] = None
        self.fused_head = (can_fuse and max_context <= self.fused_ctx_limit) if fused_head is None else bool(fused_head)
        self.fused_head_rows = 2 if fused_head is None else 8     # an explicit request fuses every step width
        assert not self.fused_head or can_fuse, "the fused head kernel needs a bf16 cache and 512 + 64 latent rows"
        self.cfg, self.w, self.fabric = cfg, weights, fabric
        if expert_fp8:
            assert cfg.shared_ffn % (16 * (fabric.world if shard is None else int(shard[1]))) == 0 and cfg.expert_ffn % 16 == 0 and cfg.hidden % 16 == 0
            self.w8: Dict[str, tuple] = {}
            for l in range(cfg.layers):
                for name in ("gate_up", "down", "shared_gate_up", "shared_down"):
                    key = f"layers.{l}.{name}"
                    self.w8[key] = K.quantize_fp8_block(weights[key].contiguous())
                    if drop_bf16_experts:
                        del weights[key]
        self.rank, self.world = (fabric.rank, fabric.world) if shard is None else (int(shard[0]), int(shard[1]))
        c, dev = cfg, fabric.device
        assert c.heads % self.world == 0 and c.experts % self.world == 0 and c.vocab % self.world == 0
        assert c.shared_ffn % (8 * self.world) == 0
        self.hl, self.el, self.vl = c.heads // self.world, c.experts // self.world, c.vocab // self.world
        self.T = max_tokens
        self.max_context = max_context
        self.max_pages = (max_context + c.page_tokens - 1) // c.page_tokens
        self.num_slots = num_slots
        self.num_pages = self.max_pages * num_slots
        self.kps = keys_per_split
        self.max_splits = max(1, min(64, (max_context + keys_per_split - 1) // keys_per_split))
        while self.max_splits * self.kps < max_context:
            self.kps *= 2
        T = self.T
        # static inputs (CUDA-graph friendly)
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(T, dtype=torch.int32, device=dev)
        self.page_table = torch.arange(self.num_pages, dtype=torch.int32, device=dev).view(num_slots, self.max_pages).contiguous()
        if kv_int8:
            self.caches = [torch.zeros(self.num_pages, c.page_tokens, 656, dtype=torch.uint8, device=dev) for _ in range(c.layers)]
        else:
            self.caches = [torch.zeros(self.num_pages, c.page_tokens, c.kv_lora + c.rope, dtype=BF16, device=dev)
                           for _ in range(c.layers)]
        # activations
        e = lambda *s, dt=BF16: torch.empty(*s, dtype=dt, device=dev)
        self.x = e(T, c.hidden)
        self.qkv = e(T, c.q_lora + c.kv_lora + c.rope)
        self.q = e(T, self.hl * c.qk_dim)
        self.q_lat = e(T, self.hl, c.kv_lora + c.rope)
        self.attn = e(T, self.hl * c.vdim)
        self.scratch = e(T * self.hl * self.max_splits * (c.kv_lora + 2), dt=torch.float32)
        self.logits_r = e(T, c.experts, dt=torch.float32)
        self.route_ids = e(T, c.topk, dt=torch.int32)
        self.xn = e(T, c.hidden)
        self.route_w = e(T, c.topk, dt=torch.float32)
        self.act = torch.zeros(T, c.topk + 1, c.expert_ffn, dtype=BF16, device=dev)
        self.partial = e(((self.vl + 7) // 8) * 8 * 2, dt=torch.float32)
        can_fuse_moe = (not expert_fp8 and c.expert_ffn <= 1536 and c.expert_ffn % 8 == 0 and (c.shared_ffn // self.world) % 8 == 0
                        and c.experts <= 256 and c.topk <= 16)
        # measured: the one-launch block loses 2-5 % per layer to the three-kernel chain at 1 and 2 GPUs and 1 % at 8 GPUs
        # (3.66 against 3.63 ms per step): its in-grid barrier costs what the two kernel boundaries it replaces cost. Off by default.
        self.fused_moe = False if fused_moe is None else bool(fused_moe)
        assert not self.fused_moe or can_fuse_moe, "the one-launch MoE block needs bf16 experts of at most 1536 columns"
        self.moe_sync = torch.zeros(K.moe_block_sync_words(2, c.experts), dtype=torch.int32, device=dev)
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_vals = torch.zeros(T, dtype=torch.float32, device=dev)
        self.logits = e(T, self.vl, dt=torch.float32) if keep_logits else None
        # embedding + lm_head + per layer: qkv_a, [cache write, q_b, absorb, split, merge+v_up | fused head], o_proj, router, gate_up, down
        self.launches_per_forward = 2 + ((6 if self.fused_head else 10) - (2 if self.fused_moe else 0)) * c.layers
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    def forward_feedback(self, T: Optional[int] = None) -> torch.Tensor:
        """One step whose sampled token and position + 1 become the inputs of the next step (device-side feedback)."""
        T = self.T if T is None else T
        self.forward(T)
        self.tokens[:T].copy_(self.next_ids[:T])
        self.positions[:T].add_(1)
        return self.next_ids[:T]

    # -- one step ----------------------------------------------------------------------------------
    def _ffn(self, l: int, T: int) -> None:
        """o_proj + all-reduce, router, expert FFN + all-reduce of layer ``l`` (consumes ``self.attn``, updates ``self.x``)."""
        c, w, fab = self.cfg, self.w, self.fabric
        p = f"layers.{l}."
        x, attn = self.x[:T], self.attn[:T]
        K.gemv_allreduce(attn, w[p + "o_proj"], fab, residual=x, out=x)
        if self.fused_moe and T <= 2:
            K.moe_block(x, w[p + "router"], w[p + "gate_up"], w[p + "down"], self.rank * self.el, c.topk, fab, sync=self.moe_sync,
                        norm_w=w[p + "ffn_norm"], eps=c.eps, scoring=c.scoring, scale=c.route_scale,
                        w_shared_gu=w[p + "shared_gate_up"], w_shared_down=w[p + "shared_down"], logits=self.logits_r[:T],
                        ids=self.route_ids[:T], wts=self.route_w[:T], act=self.act[:T], out=x)
            return
        K.router_topk(x, w[p + "router"], c.topk, norm_w=w[p + "ffn_norm"], eps=c.eps, scoring=c.scoring,
                      scale=c.route_scale, ticket_ptr=fab.ticket_ptr, logits=self.logits_r[:T],
                      ids=self.route_ids[:T], wts=self.route_w[:T], xn=self.xn[:T])
        xn = self.xn[:T]      # normalised once by the router; the expert kernels skip their own RMSNorm prologue
        if self.expert_fp8:
            w8 = self.w8
            K.moe_gate_up_fp8(xn, self.route_ids[:T], w8[p + "gate_up"], self.rank * self.el,
                              w_shared_gu=w8[p + "shared_gate_up"], act=self.act[:T])
            K.moe_down_allreduce_fp8(self.act[:T], self.route_ids[:T], self.route_w[:T], w8[p + "down"], self.rank * self.el,
                                     fab, w_shared_down=w8[p + "shared_down"], residual=x, out=x)
            return
        K.moe_gate_up(xn, self.route_ids[:T], w[p + "gate_up"], self.rank * self.el, w_shared_gu=w[p + "shared_gate_up"],
                      act=self.act[:T])
        K.moe_down_allreduce(self.act[:T], self.route_ids[:T], self.route_w[:T], w[p + "down"], self.rank * self.el,
                             fab, w_shared_down=w[p + "shared_down"], residual=x, out=x)

    def forward(self, T: Optional[int] = None) -> torch.Tensor:
        c, w, fab = self.cfg, self.w, self.fabric
        T = self.T if T is None else T
        tok, pos, slot = self.tokens[:T], self.positions[:T], self.slots[:T]
        x = self.x[:T]
        st = fab.desc.status
        K.embedding(tok, w["embed"], out=x, status_ptr=st)
        for l in range(c.layers):
            p = f"layers.{l}."
            qkv = self.qkv[:T]
            K.gemv(x, w[p + "qkv_a"], norm_w=w[p + "attn_norm"], eps=c.eps, out=qkv)
            fuse = self.fused_head if self.fuse_override is None else (self.fuse_override and self.can_fuse_head)
            if fuse and T <= self.fused_head_rows:
                K.mla_head_decode(qkv, w[p + "q_a_norm"], w[p + "kv_a_norm"], w[p + "q_b"], w[p + "kv_b"], self.caches[l], pos, slot,
                                  self.page_table, q_lora=c.q_lora, nope=c.nope, scale=c.scale, eps=c.eps, theta=c.theta,
                                  window=c.window, out=self.attn[:T], status_ptr=st,
                                  prefetch=(w[p + "o_proj"], w.get(p + "shared_gate_up"), w.get(p + "shared_down")) if self.l2_prefetch else ())
                self._ffn(l, T)
                continue
            if self.kv_int8:
                K.mla_kv_write_q8(qkv[:, c.q_lora:], w[p + "kv_a_norm"], pos, slot, self.page_table, self.caches[l], eps=c.eps,
                                  theta=c.theta, status_ptr=st)
            else:
                K.mla_kv_write(qkv[:, c.q_lora:], w[p + "kv_a_norm"], pos, slot, self.page_table, self.caches[l],
                               latent=c.kv_lora, rope=c.rope, eps=c.eps, theta=c.theta, status_ptr=st)
            q = self.q[:T]
            K.gemv(qkv[:, :c.q_lora], w[p + "q_b"], norm_w=w[p + "q_a_norm"], eps=c.eps, out=q)
            q_lat = self.q_lat[:T]
            K.mla_q_absorb(q, w[p + "kv_b"], pos, nope=c.nope, rope=c.rope, theta=c.theta, out=q_lat)
            attn = self.attn[:T]
            K.mla_decode_attention(q_lat, self.caches[l], pos, slot, self.page_table, w[p + "kv_b"], nope=c.nope,
                                   scale=c.scale, window=c.window, keys_per_split=self.kps, max_splits=self.max_splits,
                                   scratch=self.scratch, out=attn, status_ptr=st, packed=self.kv_int8)
            self._ffn(l, T)
        K.lm_head_argmax(x, w["lm_head"], fab, norm_w=w["final_norm"], eps=c.eps, vocab_offset=self.rank * self.vl,
                         partial=self.partial, logits=None if self.logits is None else self.logits[:T],
                         out_ids=self.next_ids[:T], out_vals=self.next_vals[:T])
        return self.next_ids[:T]

    # -- CUDA graph ----------------------------------------------------------------------------------
    def capture(self, T: Optional[int] = None, feedback: bool = False) -> torch.cuda.CUDAGraph:
        """Capture one decode step. With ``feedback`` the graph also copies the sampled token into the
        input buffer and advances the positions, so back-to-back replays decode autoregressively with
        no host involvement."""
        T = self.T if T is None else T
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.forward(T)  # warm-up outside capture (module loading, attribute setting)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            if feedback:
                self.forward_feedback(T)
            else:
                self.forward(T)
        self._graph = g
        return g

    def reset(self) -> None:
        for cch in self.caches:
            cch.zero_()


def bundle_parameters(cfg: MlaMoeConfig, weights: Dict[str, torch.Tensor], prefix: str = "model") -> Dict[str, torch.Tensor]:
    """This module's per-rank weight tensors under the parameter names of a bundle compiled from
    ``compiler.sources.mla_moe_source`` (``model.layers.N.self_attn.q_b_proj`` ..., pairs joined by ``|``); the same storage,
    so a bundle's engine and the library baseline can run on one copy of the weights."""
    c = cfg
    out = {f"{prefix}.embed_tokens": weights["embed"], f"{prefix}.norm": weights["final_norm"], "lm_head": weights["lm_head"]}
    for l in range(c.layers):
        p, q = f"layers.{l}.", f"{prefix}.layers.{l}."
        a, m = q + "self_attn.", q + "mlp."
        out[q + "input_layernorm"] = weights[p + "attn_norm"]
        out[a + "q_a_proj|" + a + "kv_a_proj_with_mqa"] = weights[p + "qkv_a"]
        out[a + "q_a_layernorm"], out[a + "kv_a_layernorm"] = weights[p + "q_a_norm"], weights[p + "kv_a_norm"]
        out[a + "q_b_proj"] = weights[p + "q_b"]
        kvb = weights[p + "kv_b"]
        out[a + "kv_b_proj"] = kvb.view(kvb.shape[0] * kvb.shape[1], kvb.shape[2])
        out[a + "o_proj"] = weights[p + "o_proj"]
        out[q + "post_attention_layernorm"] = weights[p + "ffn_norm"]
        out[m + "gate"] = weights[p + "router"]
        e = m + "experts.{expert}."
        out[e + "gate_proj|" + e + "up_proj"] = weights[p + "gate_up"]
        out[e + "down_proj"] = weights[p + "down"]
        out[m + "shared_experts.gate_proj|" + m + "shared_experts.up_proj"] = weights[p + "shared_gate_up"]
        out[m + "shared_experts.down_proj"] = weights[p + "shared_down"]
    return out


def weights_from_checkpoint(cfg: MlaMoeConfig, checkpoint_dir: str, prefix: str = "model") -> Dict[str, torch.Tensor]:
    """Unsharded weights of this module's naming from a safetensors checkpoint that uses the scoped names
    of the DSL examples (``model.layers.N.self_attn.q_a_proj.weight`` ...)."""
    from ..runtime.plan_engine import SafetensorsDir

    st = SafetensorsDir(checkpoint_dir)

    def get(name: str) -> torch.Tensor:
        mm, off, n, dtype, shape = st.tensors[name + ".weight"]
        import numpy as np
        raw = torch.from_numpy(np.frombuffer(mm, dtype=np.uint8, count=n, offset=off).copy())
        t = raw.view(torch.bfloat16 if dtype == "BF16" else torch.float32)
        return t.view(*shape)

    c = cfg
    out = {"embed": get(f"{prefix}.embed_tokens"), "final_norm": get(f"{prefix}.norm"), "lm_head": get("lm_head")}
    for l in range(c.layers):
        p, q = f"layers.{l}.", f"{prefix}.layers.{l}."
        out[p + "attn_norm"] = get(q + "input_layernorm")
        out[p + "qkv_a"] = torch.cat([get(q + "self_attn.q_a_proj"), get(q + "self_attn.kv_a_proj_with_mqa")], 0)
        out[p + "q_a_norm"] = get(q + "self_attn.q_a_layernorm")
        out[p + "kv_a_norm"] = get(q + "self_attn.kv_a_layernorm")
        out[p + "q_b"] = get(q + "self_attn.q_b_proj")
        out[p + "kv_b"] = get(q + "self_attn.kv_b_proj").view(c.heads, c.nope + c.vdim, c.kv_lora)
        out[p + "o_proj"] = get(q + "self_attn.o_proj")
        out[p + "ffn_norm"] = get(q + "post_attention_layernorm")
        out[p + "router"] = get(q + "mlp.gate").float()
        out[p + "gate_up"] = torch.stack([torch.cat([get(q + f"mlp.experts.{e}.gate_proj"), get(q + f"mlp.experts.{e}.up_proj")], 0)
                                          for e in range(c.experts)])
        out[p + "down"] = torch.stack([get(q + f"mlp.experts.{e}.down_proj") for e in range(c.experts)])
        out[p + "shared_gate_up"] = torch.cat([get(q + "mlp.shared_experts.gate_proj"), get(q + "mlp.shared_experts.up_proj")], 0)
        out[p + "shared_down"] = get(q + "mlp.shared_experts.down_proj")
    return out
