"""Hybrid decoder family: gated delta-rule (linear attention) layers interleaved with gated full-attention layers, tied
embedding / output matrix - the model the checkpoint-bound compile path (``csrc/core/hybrid.cpp``, contract
``qwen35_text_v1``) describes as a typed plan. This module executes that plan's mathematics on one GPU:

  full-attention layer   zero-centred RMSNorm -> q_proj (query | output gate per head), k_proj, v_proj -> per-head zero-centred
                         RMSNorm of q and k -> rotary on the first quarter of every head -> paged GQA attention -> * sigmoid(gate)
                         -> o_proj + residual
  delta layer            zero-centred RMSNorm -> in_proj (q | k | v, z, a, b) -> causal conv (width 4) + SiLU over q | k | v with a
                         per-sequence history -> L2-normalised q, k; g = -exp(A_log) * softplus(a + dt_bias); beta = sigmoid(b)
                         -> recurrence  S *= exp(g); r = beta (v - k^T S); S += k (x) r; y = (q / sqrt(d))^T S  (f32 state per
                         sequence and head) -> RMSNorm(y) * w * silu(z) -> out_proj + residual
  both                   zero-centred RMSNorm -> SwiGLU MLP + residual

Linears are the decode GEMV kernels (weights packed so that one launch produces every projection of a layer's input); the row
operators between them are ``ops/hybrid.py``; the recurrence is ``ops/hc.py::delta_rule_decode``; attention is the GQA pair of
``ops/decode.py``. State: K / V pages for the full-attention layers, the f32 delta state and the conv history per sequence slot.
``forward_ref`` is the plain PyTorch fp32 restatement with the same bf16 rounding points.
Reference: crates/inferfabric-compiler/src/bound.rs:520-830 (the typed plan), native/src/qwen_model.cpp (its executor),
crates/inferfabric-cli/src/npu_probe/cpu_model.rs:47-151 (its scalar oracle)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import decode as K
from ..ops import hc as HC
from ..ops import hybrid as HY
from ..parallel.fabric import Fabric

BF16 = torch.bfloat16
PREFIX = "model.language_model."


@dataclass
class HybridConfig:
    hidden: int = 2048
    intermediate: int = 6144
    vocab: int = 248320
    query_heads: int = 8
    kv_heads: int = 2
    head_dim: int = 256
    delta_heads: int = 16
    delta_dim: int = 128
    conv_width: int = 4
    layers: List[str] = field(default_factory=lambda: (["delta"] * 3 + ["full"]) * 6)
    theta: float = 1e7
    eps: float = 1e-6
    page_tokens: int = 16

    @staticmethod
    def text2b() -> "HybridConfig":
        """The 2B-class text model of the contract: 24 layers (three delta layers, then one full-attention layer, six times)."""
        return HybridConfig()

    @staticmethod
    def tiny(groups: int = 1) -> "HybridConfig":
        return HybridConfig(hidden=128, intermediate=256, vocab=512, query_heads=4, kv_heads=2, head_dim=64, delta_heads=4, delta_dim=32,
                            layers=(["delta"] * 3 + ["full"]) * groups, theta=1e4)

    @property
    def rotary_dim(self) -> int:
        return self.head_dim // 4

    @property
    def conv_channels(self) -> int:
        return 3 * self.delta_heads * self.delta_dim


def weight_shapes(c: HybridConfig) -> Dict[str, tuple]:
    """Checkpoint tensor names -> (dtype, shape), as the compile path's schema lists them."""
    s = {PREFIX + "embed_tokens.weight": (BF16, (c.vocab, c.hidden)), PREFIX + "norm.weight": (BF16, (c.hidden,))}
    D = c.delta_heads * c.delta_dim
    for i, kind in enumerate(c.layers):
        l = f"{PREFIX}layers.{i}."
        s[l + "input_layernorm.weight"] = (BF16, (c.hidden,))
        s[l + "post_attention_layernorm.weight"] = (BF16, (c.hidden,))
        s[l + "mlp.gate_proj.weight"] = (BF16, (c.intermediate, c.hidden))
        s[l + "mlp.up_proj.weight"] = (BF16, (c.intermediate, c.hidden))
        s[l + "mlp.down_proj.weight"] = (BF16, (c.hidden, c.intermediate))
        if kind == "full":
            s[l + "self_attn.q_norm.weight"] = (BF16, (c.head_dim,))
            s[l + "self_attn.k_norm.weight"] = (BF16, (c.head_dim,))
            s[l + "self_attn.q_proj.weight"] = (BF16, (2 * c.query_heads * c.head_dim, c.hidden))
            s[l + "self_attn.k_proj.weight"] = (BF16, (c.kv_heads * c.head_dim, c.hidden))
            s[l + "self_attn.v_proj.weight"] = (BF16, (c.kv_heads * c.head_dim, c.hidden))
            s[l + "self_attn.o_proj.weight"] = (BF16, (c.hidden, c.query_heads * c.head_dim))
        else:
            s[l + "linear_attn.A_log"] = (torch.float32, (c.delta_heads,))
            s[l + "linear_attn.norm.weight"] = (torch.float32, (c.delta_dim,))
            s[l + "linear_attn.dt_bias"] = (BF16, (c.delta_heads,))
            s[l + "linear_attn.conv1d.weight"] = (BF16, (c.conv_channels, 1, c.conv_width))
            s[l + "linear_attn.in_proj_a.weight"] = (BF16, (c.delta_heads, c.hidden))
            s[l + "linear_attn.in_proj_b.weight"] = (BF16, (c.delta_heads, c.hidden))
            s[l + "linear_attn.in_proj_qkv.weight"] = (BF16, (c.conv_channels, c.hidden))
            s[l + "linear_attn.in_proj_z.weight"] = (BF16, (D, c.hidden))
            s[l + "linear_attn.out_proj.weight"] = (BF16, (c.hidden, D))
    return s


def random_weights(c: HybridConfig, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init checkpoint tensors: N(0, 0.02) matrices (0.3 for the conv taps), zero-centred gains N(0, 0.02), delta gains
    1 + N(0, 0.02), A_log in [0, 1], dt_bias N(0, 0.5)."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, (dt, shape) in weight_shapes(c).items():
        t = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=g)
        if name.endswith("conv1d.weight"):
            t = t * 15.0
        elif name.endswith("linear_attn.norm.weight"):
            t = t + 1.0
        elif name.endswith("A_log"):
            t = torch.empty(shape, dtype=torch.float32, device=device).uniform_(0.0, 1.0, generator=g)
        elif name.endswith("dt_bias"):
            t = t * 25.0
        out[name] = t.to(dt)
    return out


# ---------------------------------------------------------------------------------------------------------------------------
# checkpoint-bound construction: definition + checkpoint directory -> typed plan (checked by the host core) -> decoder
# ---------------------------------------------------------------------------------------------------------------------------
_ST = {BF16: "BF16", torch.float32: "F32"}


def definition_text(c: HybridConfig, *, label: str = "hybrid", context_buckets=(1024,), batch_buckets=(1, 2, 4, 8), token_budget: int = 64) -> str:
    """The model document (contract ``qwen35_text_v1``) that describes ``c`` on one GPU."""
    return (f"language inferfabric 1;\nmodel Hybrid {{\n    contract = qwen35_text_v1;\n    label = \"{label}\";\n"
            f"    hidden = {c.hidden}; intermediate = {c.intermediate}; vocab = {c.vocab};\n"
            f"    query_heads = {c.query_heads}; kv_heads = {c.kv_heads}; head_dim = {c.head_dim};\n"
            f"    delta_heads = {c.delta_heads}; delta_dim = {c.delta_dim}; conv_width = {c.conv_width};\n"
            f"    layers = [{', '.join(c.layers)}];\n}}\nplan OneGpu for Hybrid {{\n"
            "    prefill = mesh(tp = 1, cp = 1, sp = false);\n    decode = mesh(tp = 1, cp = 1, sp = false);\n"
            f"    page_tokens = {c.page_tokens}; token_budget = {token_budget};\n"
            f"    batch_buckets = [{', '.join(map(str, batch_buckets))}];\n    context_buckets = [{', '.join(map(str, context_buckets))}];\n}}\n")


def save_checkpoint(path, c: HybridConfig, weights: Dict[str, torch.Tensor], *, shards: int = 2, max_position: int = 4096) -> None:
    """Write ``weights`` (this module's checkpoint names) as a sharded safetensors directory with the ``config.json`` and the
    weight index the compile path inspects."""
    import json
    import struct
    from pathlib import Path

    d = Path(path)
    d.mkdir(parents=True, exist_ok=True)
    names = list(weights)
    per = (len(names) + shards - 1) // shards
    parts = [names[i:i + per] for i in range(0, len(names), per)]
    wmap, total = {}, 0
    for i, part in enumerate(parts):
        fname = f"model-{i + 1:05d}-of-{len(parts):05d}.safetensors"
        hdr, blobs, cursor = {}, [], 0
        for n in part:
            t = weights[n].detach().cpu().contiguous()
            raw = t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
            hdr[n] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [cursor, cursor + len(raw)]}
            blobs.append(raw)
            cursor += len(raw)
            wmap[n] = fname
        head = json.dumps(hdr).encode()
        head += b" " * (-len(head) % 8)
        (d / fname).write_bytes(struct.pack("<Q", len(head)) + head + b"".join(blobs))
        total += cursor
    text = {"model_type": "qwen3_5_text", "hidden_size": c.hidden, "intermediate_size": c.intermediate, "vocab_size": c.vocab,
            "num_hidden_layers": len(c.layers), "num_attention_heads": c.query_heads, "num_key_value_heads": c.kv_heads, "head_dim": c.head_dim,
            "linear_num_key_heads": c.delta_heads, "linear_num_value_heads": c.delta_heads, "linear_key_head_dim": c.delta_dim,
            "linear_value_head_dim": c.delta_dim, "linear_conv_kernel_dim": c.conv_width, "attention_bias": False, "attn_output_gate": True,
            "hidden_act": "silu", "rms_norm_eps": c.eps, "tie_word_embeddings": True, "max_position_embeddings": max_position,
            "rope_parameters": {"rope_type": "default", "rope_theta": float(c.theta), "partial_rotary_factor": 0.25},
            "layer_types": ["full_attention" if k == "full" else "linear_attention" for k in c.layers]}
    (d / "config.json").write_text(json.dumps({"model_type": "qwen3_5", "tie_word_embeddings": True, "text_config": text}))
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": wmap}))


def typed_plan(definition_path: str, checkpoint_dir: str) -> dict:
    """The host core's typed plan of (definition, checkpoint): the checkpoint is inspected against the contract (every tensor
    present with its dtype and shape, nothing unexpected, config and definition agree) before anything is loaded."""
    import json

    from .. import compiler

    return json.loads(compiler.cli("compile-checkpoint", str(definition_path), str(checkpoint_dir)).stdout)


def config_of(plan: dict, checkpoint_dir: str) -> HybridConfig:
    """The decoder configuration a typed plan describes (dimensions from the plan, rope base and epsilon from ``config.json``)."""
    import json
    from pathlib import Path

    if plan.get("format") != "inferfabric.typed-plan.v1" or plan.get("contract") != "qwen35_text_v1":
        raise ValueError("not a typed plan of the hybrid decoder contract")
    spec, m = plan["spec"], plan["spec"]["model"]
    if spec["decode"]["tp"] != 1 or spec["decode"]["cp"] != 1:
        raise ValueError("the hybrid decoder executes plans for one GPU (decode mesh tp = 1, cp = 1)")
    text = json.loads((Path(checkpoint_dir) / "config.json").read_text())
    text = text.get("text_config", text)
    return HybridConfig(hidden=m["hidden"], intermediate=m["intermediate"], vocab=m["vocab"], query_heads=m["query_heads"], kv_heads=m["kv_heads"],
                        head_dim=m["head_dim"], delta_heads=m["delta_heads"], delta_dim=m["delta_dim"], conv_width=m["conv_width"],
                        layers=[k.lower() for k in m["layers"]], theta=float(text["rope_parameters"]["rope_theta"]),
                        eps=float(text.get("rms_norm_eps", 1e-6)), page_tokens=spec["page_tokens"])


def load_weights(plan: dict, checkpoint_dir: str, device, *, staging_bytes: int = 64 << 20) -> Dict[str, torch.Tensor]:
    """Every tensor the typed plan binds, read at the (shard, offset, bytes) the plan recorded and uploaded through one bounded
    staging buffer (pinned when the destination is a GPU)."""
    from ..runtime.plan_engine import SafetensorsDir

    dts = {"BF16": BF16, "F32": torch.float32}
    src = SafetensorsDir(checkpoint_dir)
    on_gpu = torch.device(device).type == "cuda"
    stage = torch.empty(max(4096, int(staging_bytes)), dtype=torch.uint8)
    if on_gpu:
        stage = stage.pin_memory()
    out = {}
    for name, info in plan["checkpoint"]["weights"].items():
        dt, n = dts[info["dtype"]], int(info["bytes"])
        host = src.shard_from(info["shard"], int(info["offset"]))[:n]
        if host.size != n:
            raise ValueError(f"{name}: the shard ends before the tensor does")
        dst = torch.empty(n, dtype=torch.uint8, device=device)
        for b in range(0, n, stage.numel()):
            e = min(n, b + stage.numel())
            stage[:e - b].copy_(torch.from_numpy(host[b:e].copy()))
            dst[b:e].copy_(stage[:e - b], non_blocking=False)
        out[name] = dst.view(dt).view(*info["shape"])
    return out


class HybridDecoder:
    """Up to ``max_tokens`` (<= 8) query rows per step on one GPU; rows carry their own position and sequence slot, rows of one
    sequence inside a step must come in position order. Greedy next tokens land in ``next_ids``."""

    def __init__(self, cfg: HybridConfig, weights: Dict[str, torch.Tensor], fabric: Fabric, *, max_tokens: int = 8, max_context: int = 1024,
                 num_slots: int = 1, keys_per_split: int = 64, keep_logits: bool = False):
        assert 1 <= max_tokens <= 8 and fabric.world == 1, "the hybrid decoder runs on one GPU"
        c, dev = cfg, fabric.device
        assert c.head_dim in (64, 128, 256) and c.query_heads % c.kv_heads == 0 and c.delta_dim <= 256 and 2 <= c.conv_width <= 4
        self.cfg, self.fabric, self.rank, self.world = cfg, fabric, 0, 1
        self.T, self.max_context, self.num_slots = max_tokens, max_context, num_slots
        self.max_pages = (max_context + c.page_tokens - 1) // c.page_tokens
        self.num_pages = self.max_pages * num_slots
        self.kps = keys_per_split
        self.max_splits = max(1, min(64, (max_context + keys_per_split - 1) // keys_per_split))
        while self.max_splits * self.kps < max_context:
            self.kps *= 2
        # ---- weights, packed per launch ----
        W = weights
        self.embed, self.final_norm = W[PREFIX + "embed_tokens.weight"], W[PREFIX + "norm.weight"]
        self.layers = []
        for i, kind in enumerate(c.layers):
            l = f"{PREFIX}layers.{i}."
            L = {"kind": kind, "in_norm": W[l + "input_layernorm.weight"], "post_norm": W[l + "post_attention_layernorm.weight"],
                 "gate_up": torch.cat([W[l + "mlp.gate_proj.weight"], W[l + "mlp.up_proj.weight"]], 0).contiguous(),
                 "down": W[l + "mlp.down_proj.weight"]}
            if kind == "full":
                L.update(qkv=torch.cat([W[l + "self_attn.q_proj.weight"], W[l + "self_attn.k_proj.weight"], W[l + "self_attn.v_proj.weight"]], 0).contiguous(),
                         q_norm=W[l + "self_attn.q_norm.weight"], k_norm=W[l + "self_attn.k_norm.weight"], o=W[l + "self_attn.o_proj.weight"],
                         k_cache=torch.zeros(self.num_pages, c.page_tokens, c.kv_heads, c.head_dim, dtype=BF16, device=dev),
                         v_cache=torch.zeros(self.num_pages, c.page_tokens, c.kv_heads, c.head_dim, dtype=BF16, device=dev))
            else:
                L.update(proj=torch.cat([W[l + "linear_attn.in_proj_qkv.weight"], W[l + "linear_attn.in_proj_z.weight"],
                                         W[l + "linear_attn.in_proj_a.weight"], W[l + "linear_attn.in_proj_b.weight"]], 0).contiguous(),
                         conv=W[l + "linear_attn.conv1d.weight"].reshape(c.conv_channels, c.conv_width).contiguous(),
                         a_log=W[l + "linear_attn.A_log"].float().contiguous(), dt_bias=W[l + "linear_attn.dt_bias"].float().contiguous(),
                         gain=W[l + "linear_attn.norm.weight"].float().contiguous(), out=W[l + "linear_attn.out_proj.weight"],
                         state=torch.zeros(num_slots, c.delta_heads, c.delta_dim, c.delta_dim, dtype=torch.float32, device=dev),
                         history=torch.zeros(num_slots, c.conv_channels, c.conv_width - 1, dtype=BF16, device=dev))
            self.layers.append(L)
        # ---- static step buffers ----
        T = self.T
        e = lambda *s, dt=BF16: torch.empty(*s, dtype=dt, device=dev)
        self.tokens = torch.zeros(T, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(T, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(T, dtype=torch.int32, device=dev)
        self.page_table = torch.arange(self.num_pages, dtype=torch.int32, device=dev).view(num_slots, self.max_pages).contiguous()
        D, C, qh, kvh, hd = c.delta_heads * c.delta_dim, c.conv_channels, c.query_heads, c.kv_heads, c.head_dim
        self.x, self.xn = e(T, c.hidden), e(T, c.hidden)
        self.proj_full = e(T, (2 * qh + 2 * kvh) * hd)
        self.qkv, self.gate, self.attn = e(T, (qh + 2 * kvh) * hd), e(T, qh * hd), e(T, qh * hd)
        self.scratch = e(T * qh * self.max_splits * (hd + 2), dt=torch.float32)
        self.proj_delta = e(T, C + D + 2 * c.delta_heads)
        self.conv_out = e(T, C)
        self.dq, self.dk = e(T, c.delta_heads, c.delta_dim), e(T, c.delta_heads, c.delta_dim)
        self.dg, self.dbeta = e(T, c.delta_heads, dt=torch.float32), e(T, c.delta_heads, dt=torch.float32)
        self.dy = e(T, c.delta_heads, c.delta_dim)
        self.mixed = e(T, max(D, qh * hd))
        self.act = e(T, c.intermediate)
        self.partial = e(((c.vocab + 7) // 8) * 8 * 2, dt=torch.float32)
        self.next_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.next_vals = torch.zeros(T, dtype=torch.float32, device=dev)
        self.logits = e(T, c.vocab, dt=torch.float32) if keep_logits else None
        n_full = sum(1 for k in c.layers if k == "full")
        self.launches_per_forward = 3 + n_full * 10 + (len(c.layers) - n_full) * 9      # + one recurrence launch per row and delta layer

    @classmethod
    def from_checkpoint(cls, definition_path: str, checkpoint_dir: str, fabric: Fabric, **kw) -> "HybridDecoder":
        """Definition + checkpoint directory -> decoder: the host core inspects and compiles the pair into the typed plan, the
        plan names the tensors and where their bytes are, and the decoder is built on exactly those. ``self.plan_key`` keeps the
        plan's content key."""
        plan = typed_plan(definition_path, checkpoint_dir)
        dec = cls(config_of(plan, checkpoint_dir), load_weights(plan, checkpoint_dir, fabric.device), fabric, **kw)
        dec.plan_key = plan["key"]
        return dec

    def forward(self, T: Optional[int] = None) -> torch.Tensor:
        c, fab = self.cfg, self.fabric
        T = self.T if T is None else T
        tok, pos, slot = self.tokens[:T], self.positions[:T], self.slots[:T]
        x, xn, st = self.x[:T], self.xn[:T], fab.desc.status
        qh, kvh, hd, dh, dd = c.query_heads, c.kv_heads, c.head_dim, c.delta_heads, c.delta_dim
        D, C = dh * dd, c.conv_channels
        K.embedding(tok, self.embed, out=x, status_ptr=st)
        for L in self.layers:
            HY.zc_rmsnorm(x, L["in_norm"], c.eps, out=xn)
            if L["kind"] == "full":
                proj = K.gemv(xn, L["qkv"], out=self.proj_full[:T])
                HY.qk_prepare(proj[:, :2 * qh * hd], proj[:, 2 * qh * hd:], L["q_norm"], L["k_norm"], c.eps, heads=qh, kv_heads=kvh, head_dim=hd,
                              qkv=self.qkv[:T], gate=self.gate[:T])
                K.gqa_rope_kv_write(self.qkv[:T], pos, slot, self.page_table, L["k_cache"], L["v_cache"], heads=qh, kv_heads=kvh, head_dim=hd,
                                    rotary_dim=c.rotary_dim, theta=c.theta, status_ptr=st)
                K.gqa_decode_attention(self.qkv[:T], L["k_cache"], L["v_cache"], pos, slot, self.page_table, heads=qh, kv_heads=kvh, head_dim=hd,
                                       scale=1.0 / math.sqrt(hd), keys_per_split=self.kps, max_splits=self.max_splits, scratch=self.scratch,
                                       out=self.attn[:T], status_ptr=st)
                mixed = HY.sigmoid_mul(self.attn[:T], self.gate[:T], out=self.mixed[:T, :qh * hd])
                K.gemv_allreduce(mixed, L["o"], fab, residual=x, out=x)
            else:
                proj = K.gemv(xn, L["proj"], out=self.proj_delta[:T])
                HY.conv_silu(proj[:, :C], L["conv"], L["history"], pos, slot, out=self.conv_out[:T])
                HY.delta_prepare(self.conv_out[:T], proj[:, C + D:], L["a_log"], L["dt_bias"], c.eps, heads=dh, dim=dd, q=self.dq[:T], k=self.dk[:T],
                                 g=self.dg[:T], beta=self.dbeta[:T], positions=pos, slots=slot, state=L["state"])
                for t in range(T):      # rows of one sequence must update its state in order: one launch per row
                    vt = self.conv_out[t:t + 1, 2 * D:].view(1, dh, dd)
                    HC.delta_rule_decode(self.dq[t:t + 1], self.dk[t:t + 1], vt, self.dg[t:t + 1], self.dbeta[t:t + 1], L["state"], slot[t:t + 1],
                                         out=self.dy[t:t + 1])
                mixed = HY.gated_rmsnorm(self.dy[:T], proj[:, C:C + D], L["gain"], c.eps, out=self.mixed[:T, :D])
                K.gemv_allreduce(mixed, L["out"], fab, residual=x, out=x)
            HY.zc_rmsnorm(x, L["post_norm"], c.eps, out=xn)
            K.gemv(xn, L["gate_up"], swiglu=True, out=self.act[:T])
            K.gemv_allreduce(self.act[:T], L["down"], fab, residual=x, out=x)
        HY.zc_rmsnorm(x, self.final_norm, c.eps, out=xn)
        K.lm_head_argmax(xn, self.embed, fab, vocab_offset=0, partial=self.partial, logits=None if self.logits is None else self.logits[:T],
                         out_ids=self.next_ids[:T], out_vals=self.next_vals[:T])
        return self.next_ids[:T]

    def forward_feedback(self, T: Optional[int] = None) -> torch.Tensor:
        T = self.T if T is None else T
        self.forward(T)
        self.tokens[:T].copy_(self.next_ids[:T])
        self.positions[:T].add_(1)
        return self.next_ids[:T]

    def capture(self, T: Optional[int] = None, feedback: bool = False) -> torch.cuda.CUDAGraph:
        T = self.T if T is None else T
        self.forward(T)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward_feedback(T) if feedback else self.forward(T)
        return g

    def reset(self) -> None:
        for L in self.layers:
            for name in ("k_cache", "v_cache", "state", "history"):
                if name in L:
                    L[name].zero_()


# ---------------------------------------------------------------------------------------------------------------------------
# fp32 restatement
# ---------------------------------------------------------------------------------------------------------------------------
def _r(t: torch.Tensor) -> torch.Tensor:
    return t.to(BF16).float()


def forward_ref(c: HybridConfig, W: Dict[str, torch.Tensor], tokens: torch.Tensor) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence (positions 0..T-1), fp32 arithmetic with bf16 rounding where the plan's tensors are bf16."""
    dev, T = tokens.device, tokens.numel()
    f = lambda n: W[n].to(dev).float()
    pos = torch.arange(T, device=dev)
    qh, kvh, hd, dh, dd, cw, rot = c.query_heads, c.kv_heads, c.head_dim, c.delta_heads, c.delta_dim, c.conv_width, c.rotary_dim

    def zc(x, w):
        return _r(x * torch.rsqrt((x * x).mean(-1, keepdim=True) + c.eps) * (1.0 + w))

    def rope(x):       # x [T, heads, hd]: half rotation over the first `rot` columns, bf16 cos / sin tables
        i = torch.arange(rot // 2, device=dev, dtype=torch.float32)
        inv = torch.exp2(-(2.0 * i / rot) * math.log2(c.theta))
        ang = pos.float()[:, None] * inv[None]
        cs, sn = _r(torch.cos(ang))[:, None], _r(torch.sin(ang))[:, None]
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        return torch.cat([_r(a * cs - b * sn), _r(b * cs + a * sn), x[..., rot:]], -1)

    x = f(PREFIX + "embed_tokens.weight")[tokens.long()]
    causal = torch.ones(T, T, dtype=torch.bool, device=dev).tril()
    for i, kind in enumerate(c.layers):
        l = f"{PREFIX}layers.{i}."
        n = zc(x, f(l + "input_layernorm.weight"))
        if kind == "full":
            qg = _r(n @ f(l + "self_attn.q_proj.weight").T).view(T, qh, 2 * hd)
            q = rope(zc(qg[..., :hd], f(l + "self_attn.q_norm.weight")))
            gate = qg[..., hd:]
            k = rope(zc(_r(n @ f(l + "self_attn.k_proj.weight").T).view(T, kvh, hd), f(l + "self_attn.k_norm.weight")))
            v = _r(n @ f(l + "self_attn.v_proj.weight").T).view(T, kvh, hd)
            G = qh // kvh
            s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(G, 1)) / math.sqrt(hd)
            s = s.masked_fill(~causal[None], float("-inf"))
            attn = _r(torch.einsum("hts,shd->thd", torch.softmax(s, -1), v.repeat_interleave(G, 1)))
            mixed = _r(attn * _r(torch.sigmoid(gate))).reshape(T, qh * hd)
            x = _r(_r(mixed @ f(l + "self_attn.o_proj.weight").T) + x)
        else:
            D = dh * dd
            qkv = _r(n @ f(l + "linear_attn.in_proj_qkv.weight").T)
            z = _r(n @ f(l + "linear_attn.in_proj_z.weight").T).view(T, dh, dd)
            a = _r(n @ f(l + "linear_attn.in_proj_a.weight").T)
            b = _r(n @ f(l + "linear_attn.in_proj_b.weight").T)
            wc = f(l + "linear_attn.conv1d.weight").reshape(-1, cw)
            padded = torch.cat([torch.zeros(cw - 1, qkv.shape[1], device=dev), qkv], 0)
            conv = sum(padded[j:j + T] * wc[:, j][None] for j in range(cw))
            conv = _r(torch.nn.functional.silu(conv))
            qd, kd, vd = (conv[:, j * D:(j + 1) * D].view(T, dh, dd) for j in range(3))
            l2 = lambda t: _r(t * torch.rsqrt(_r((t * t).sum(-1, keepdim=True)) + c.eps))
            qd, kd = l2(qd), l2(kd)
            g = -torch.exp(f(l + "linear_attn.A_log")) * torch.nn.functional.softplus(a + f(l + "linear_attn.dt_bias"))
            beta = _r(torch.sigmoid(b))
            S = torch.zeros(dh, dd, dd, device=dev)
            ys = []
            for t in range(T):
                S = S * torch.exp(g[t])[:, None, None]
                r = beta[t][:, None] * (vd[t] - torch.einsum("hk,hkv->hv", kd[t], S))
                S = S + kd[t][:, :, None] * r[:, None, :]
                ys.append(_r(torch.einsum("hk,hkv->hv", qd[t] / math.sqrt(dd), S)))
            y = torch.stack(ys)
            y = _r(y * torch.rsqrt((y * y).mean(-1, keepdim=True) + c.eps) * f(l + "linear_attn.norm.weight") * torch.nn.functional.silu(z))
            x = _r(_r(y.reshape(T, D) @ f(l + "linear_attn.out_proj.weight").T) + x)
        n2 = zc(x, f(l + "post_attention_layernorm.weight"))
        gate = _r(n2 @ f(l + "mlp.gate_proj.weight").T)
        up = _r(n2 @ f(l + "mlp.up_proj.weight").T)
        act = _r(torch.nn.functional.silu(gate) * up)
        x = _r(_r(act @ f(l + "mlp.down_proj.weight").T) + x)
    return zc(x, f(PREFIX + "norm.weight")) @ f(PREFIX + "embed_tokens.weight").T
