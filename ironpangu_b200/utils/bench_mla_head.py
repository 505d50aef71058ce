"""Device time of the attention half of an MLA decode layer: five separate kernels against the cluster-per-head launch.

Builds ``--layers`` independent layers (own q_b / kv_b weights and cache, so every layer streams from HBM), captures each
path over all layers in one CUDA graph and times graph replays with CUDA events. Reported per layer, in microseconds.

    python -m ironpangu_b200.utils.bench_mla_head --heads 32 --context 512        # one GPU's share at tp1
    python -m ironpangu_b200.utils.bench_mla_head --heads 4 --context 512         # one GPU's share at tp8
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from ..ops import decode as K

BF16 = torch.bfloat16


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--layers", type=int, default=46)
    ap.add_argument("--q-lora", type=int, default=1536)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--eager", action="store_true", help="plain launches instead of graph replays (for profilers)")
    a = ap.parse_args()
    dev = torch.device("cuda")
    H, T, L, ql, nope, vdim, pt = a.heads, a.tokens, a.layers, a.q_lora, 128, 128, 16
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g, device=dev) * scale).to(BF16)
    pages = (a.context + pt) // pt + 1
    qkv = rnd(T, ql + 576)
    qn, kn = rnd(ql, scale=0.1) + 1, rnd(512, scale=0.1) + 1
    w_qb = [rnd(H * (nope + 64), ql, scale=0.03) for _ in range(L)]
    w_kvb = [rnd(H, nope + vdim, 512, scale=0.05) for _ in range(L)]
    caches = [rnd(pages * T, pt, 576, scale=0.5) for _ in range(L)]
    table = torch.arange(pages * T, dtype=torch.int32, device=dev).view(T, pages)
    pos = torch.full((T,), a.context - 1, dtype=torch.int32, device=dev)
    slot = torch.arange(T, dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(nope + 64)
    kps = 64
    splits = max(1, min(64, (a.context + kps - 1) // kps))
    q, q_lat = torch.empty(T, H * (nope + 64), dtype=BF16, device=dev), torch.empty(T, H, 576, dtype=BF16, device=dev)
    out = torch.empty(T, H * vdim, dtype=BF16, device=dev)
    scratch = torch.empty(T * H * splits * 514, dtype=torch.float32, device=dev)

    def chain():
        for l in range(L):
            K.mla_kv_write(qkv[:, ql:], kn, pos, slot, table, caches[l], latent=512, rope=64, eps=1e-5, theta=1e4)
            K.gemv(qkv[:, :ql], w_qb[l], norm_w=qn, eps=1e-5, out=q)
            K.mla_q_absorb(q, w_kvb[l], pos, nope=nope, rope=64, theta=1e4, out=q_lat)
            K.mla_decode_attention(q_lat, caches[l], pos, slot, table, w_kvb[l], nope=nope, scale=scale, keys_per_split=kps,
                                   max_splits=splits, scratch=scratch, out=out)

    def fused():
        for l in range(L):
            K.mla_head_decode(qkv, qn, kn, w_qb[l], w_kvb[l], caches[l], pos, slot, table, q_lora=ql, nope=nope, scale=scale,
                              eps=1e-5, theta=1e4, out=out)

    res = {"heads": H, "tokens": T, "context": a.context, "layers": L}
    for name, fn in (("chain_us_per_layer", chain), ("fused_us_per_layer", fused)):
        fn()
        torch.cuda.synchronize()
        if a.eager:
            class _Eager:
                replay = staticmethod(fn)
            graph = _Eager()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        res[name] = round(e0.elapsed_time(e1) * 1e3 / a.iters / L, 3)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
