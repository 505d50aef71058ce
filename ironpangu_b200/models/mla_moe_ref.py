"""Plain PyTorch fp32 restatement of the MLA + MoE decoder (numerical oracle for the CUDA path).

It evaluates a whole sequence at once on unsharded weights, in f32 arithmetic, rounding to bf16 at
the same points where the device plan stores bf16 tensors, so greedy tokens can be compared exactly
and logits tightly. Runs on CPU or GPU; uses no custom kernels.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .mla_moe import MlaMoeConfig


def _r(t: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and come back to f32."""
    return t.to(torch.bfloat16).to(torch.float32)


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float, zero_centered: bool = False) -> torch.Tensor:
    x = x.float()
    g = w.float() + 1.0 if zero_centered else w.float()
    return _r(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g)


def rope_ref(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-rotation RoPE over the last dim with bf16-rounded cos/sin tables. x: [T, ..., d], pos: [T]."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, device=x.device, dtype=torch.float32)
    inv = torch.exp2(-(2.0 * i / d) * torch.log2(torch.tensor(theta, dtype=torch.float32, device=x.device)))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    c, s = _r(torch.cos(ang)), _r(torch.sin(ang))
    while c.dim() < x.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    a, b = x[..., :half].float(), x[..., half:].float()
    return _r(torch.cat([a * c - b * s, b * c + a * s], -1))


def route_ref(logits: torch.Tensor, topk: int, scoring: str = "softmax", bias=None, renorm: bool = True, scale: float = 1.0):
    if scoring == "softmax":
        p = torch.softmax(logits.float(), -1)
        sel = p
    else:
        p = torch.sigmoid(logits.float())
        sel = p + (bias.float() if bias is not None else 0.0)
    # stable: highest score first, ties to the lowest expert id
    order = torch.sort(sel, dim=-1, descending=True, stable=True).indices[..., :topk]
    w = torch.gather(p, -1, order)
    if scoring == "softmax":
        if renorm:
            w = w / w.sum(-1, keepdim=True)
    else:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return order, w * scale


def forward_ref(cfg: MlaMoeConfig, W: Dict[str, torch.Tensor], tokens: torch.Tensor, tp: int = 1) -> torch.Tensor:
    """Logits [T, vocab] (f32) for one sequence ``tokens`` [T] starting at position 0.

    ``tp`` reproduces the partial-sum structure of a tensor-parallel run (K-sharded projections are
    summed per rank first, then across ranks in rank order), which changes f32 rounding only."""
    c = cfg
    dev = tokens.device
    T = tokens.numel()
    pos = torch.arange(T, device=dev)
    f = lambda name: W[name].to(dev).float()
    x = f("embed")[tokens.long()]
    causal = torch.ones(T, T, dtype=torch.bool, device=dev).tril()
    if c.window > 0:
        causal &= ~torch.ones(T, T, dtype=torch.bool, device=dev).tril(-c.window)

    def ksplit_matmul(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a [T,K] @ w[N,K]^T with K split over tp ranks, f32 partials summed in rank order."""
        Kd = a.shape[-1]
        step = Kd // tp
        out = torch.zeros(a.shape[0], w.shape[0], device=dev)
        for r in range(tp):
            out = out + a[:, r * step:(r + 1) * step] @ w[:, r * step:(r + 1) * step].T
        return out

    for l in range(c.layers):
        p = f"layers.{l}."
        h = rmsnorm_ref(x, f(p + "attn_norm"), c.eps)
        qkv = _r(h @ f(p + "qkv_a").T)
        q_a, latent, k_pe = qkv[:, :c.q_lora], qkv[:, c.q_lora:c.q_lora + c.kv_lora], qkv[:, c.q_lora + c.kv_lora:]
        q = _r(rmsnorm_ref(q_a, f(p + "q_a_norm"), c.eps) @ f(p + "q_b").T).view(T, c.heads, c.qk_dim)
        lat_n = rmsnorm_ref(latent, f(p + "kv_a_norm"), c.eps)                 # [T, 512]
        k_r = rope_ref(k_pe, pos, c.theta)                                     # [T, 64]
        kvb = f(p + "kv_b")                                                    # [H, nope+v, 512]
        w_uk, w_uv = kvb[:, :c.nope], kvb[:, c.nope:]
        q_lat = _r(torch.einsum("thd,hdc->thc", q[..., :c.nope], w_uk))        # [T, H, 512]
        q_r = rope_ref(q[..., c.nope:], pos, c.theta)                          # [T, H, 64]
        s = (torch.einsum("thc,sc->hts", q_lat, lat_n) + torch.einsum("thr,sr->hts", q_r, k_r)) * c.scale
        s = s.masked_fill(~causal[None], float("-inf"))
        pr = torch.softmax(s, -1)
        o_lat = _r(torch.einsum("hts,sc->thc", pr, lat_n))
        attn = _r(torch.einsum("thc,hvc->thv", o_lat, w_uv)).reshape(T, c.heads * c.vdim)
        x = _r(_r(ksplit_matmul(attn, f(p + "o_proj"))) + x)

        h2 = rmsnorm_ref(x, f(p + "ffn_norm"), c.eps)
        logits = h2 @ f(p + "router").T
        ids, wts = route_ref(logits, c.topk, c.scoring, None, True, c.route_scale)
        gu, dn = f(p + "gate_up"), f(p + "down")
        el = c.experts // tp
        moe = torch.zeros(T, c.hidden, device=dev)
        for r in range(tp):
            part = torch.zeros(T, c.hidden, device=dev)
            for t in range(T):
                for k in range(c.topk):
                    e = int(ids[t, k])
                    if not (r * el <= e < (r + 1) * el):
                        continue
                    g_u = _r(h2[t] @ gu[e].T)
                    a = _r(torch.nn.functional.silu(g_u[:c.expert_ffn]) * g_u[c.expert_ffn:])
                    part[t] += wts[t, k] * (a @ dn[e].T)
            # tensor-parallel shard of the shared expert
            fs = c.shared_ffn // tp
            sgu, sdn = f(p + "shared_gate_up"), f(p + "shared_down")
            g = _r(h2 @ sgu[r * fs:(r + 1) * fs].T)
            u = _r(h2 @ sgu[c.shared_ffn + r * fs:c.shared_ffn + (r + 1) * fs].T)
            a = _r(torch.nn.functional.silu(g) * u)
            part = part + a @ sdn[:, r * fs:(r + 1) * fs].T
            moe = moe + part
        x = _r(_r(moe) + x)
    hN = rmsnorm_ref(x, f("final_norm"), c.eps)
    return hN @ f("lm_head").T
