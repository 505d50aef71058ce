"""Small decode workload for kernel profiling (`ncu`) and per-kernel timing.

Builds the flagship-shaped MLA+MoE decoder with a reduced layer count, marks `--context` cache rows
as present (zero-filled) and runs a few eager single-token decode steps. Kernel names to filter on:
gemv_kernel, gemv_allreduce_kernel, mla_*_kernel, router_topk_kernel, moe_*_kernel,
lm_head_argmax_kernel, embedding_kernel.

    python -m ironpangu_b200.utils.profile_decode --layers 2 --steps 3
    python -m ironpangu_b200.utils.profile_decode --layers 2 --steps 3 --events   # CUDA-event table
"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--events", action="store_true", help="time every op with CUDA events and print a table")
    args = ap.parse_args()

    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    torch.cuda.set_device(0)
    cfg = MlaMoeConfig.flagship()
    cfg.layers = args.layers
    fab = Fabric(0, 1)
    w = random_rank_weights(cfg, 0, 1, torch.device("cuda", 0))
    dec = MlaMoeDecoder(cfg, w, fab, max_tokens=max(1, args.tokens), max_context=args.context + 64)
    T = args.tokens
    dec.tokens[:T].fill_(17)
    dec.slots[:T].zero_()
    for c in dec.caches:
        c.normal_(0, 0.5)
    records = []
    if args.events:
        # wrap every op of the decode module with events
        names = [n for n in dir(K) if not n.startswith("_") and callable(getattr(K, n)) and getattr(getattr(K, n), "__module__", "") == K.__name__]
        orig = {n: getattr(K, n) for n in names}

        def wrap(n):
            def f(*a, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = orig[n](*a, **k)
                e1.record()
                records.append((n, e0, e1))
                return r
            return f

        for n in names:
            setattr(K, n, wrap(n))
    for s in range(args.steps):
        dec.positions[:T].copy_(torch.arange(args.context + s * T, args.context + (s + 1) * T, dtype=torch.int32))
        if s == args.steps - 1:
            records.clear()
        dec.forward(T)
    torch.cuda.synchronize()
    if args.events:
        agg = {}
        for n, e0, e1 in records:
            a = agg.setdefault(n, [0, 0.0])
            a[0] += 1
            a[1] += e0.elapsed_time(e1) * 1e3
        total = sum(v[1] for v in agg.values())
        print(json.dumps({"layers": args.layers, "tokens": T, "total_us": round(total, 1),
                          "ops": {n: {"calls": v[0], "us_per_call": round(v[1] / v[0], 2), "share": round(v[1] / total, 3)}
                                  for n, v in sorted(agg.items(), key=lambda kv: -kv[1][1])}}, indent=1))
    assert fab.status() == 0
    fab.close()


if __name__ == "__main__":
    main()
