"""Time the tcgen05 prompt-attention kernel (``csrc/kernels/fa_prefill.cu``) on one GPU: CUDA events, L2 flushed between runs,
causal FLOPs counted as executed (about half of the dense m x ctx rectangle when m = ctx).

    python -m ironpangu_b200.utils.bench_attention [--cases 4096:32:1:128:64,...] [--library]

A case is ``rows:heads:kv_group:d1:d2`` (query rows = context, positions 0 ..): ``d1`` key columns per head, ``d2`` key columns
shared by all heads (the rotary part of the latent form; 0 for grouped-query attention), values 128 wide.
``--library`` also times torch's scaled-dot-product attention on the equivalent dense tensors (a library kernel, for scale)."""
from __future__ import annotations

import argparse
import json
import math

import torch

BF16 = torch.bfloat16


def time_fn(fn, flush, iters=10):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="4096:32:1:128:64,4096:16:4:128:0,1024:32:1:128:64,512:32:1:128:64")
    ap.add_argument("--library", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    from ironpangu_b200.ops import prefill as P
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(0, 1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    peaks = {}
    try:
        import pathlib
        peaks = json.loads((pathlib.Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    out = []
    for case in args.cases.split(","):
        m, H, group, d1, d2 = (int(x) for x in case.split(":"))
        ctx, Hkv, dq = m, H // group, d1 + d2
        g = torch.Generator(device="cuda").manual_seed(m + H)
        rnd = lambda *s: torch.randn(*s, generator=g, device="cuda").to(BF16)
        q, k, v = rnd(m, H * dq), rnd(ctx, Hkv * d1), rnd(ctx, Hkv, 128)
        k2 = rnd(ctx, d2) if d2 else None
        vt = v.permute(1, 2, 0).reshape(Hkv * 128, ctx).contiguous()
        o = torch.empty(m, H * 128, dtype=BF16, device="cuda")
        scale = 1.0 / math.sqrt(dq)
        run = lambda: P.fa_prefill(q, k, vt, o, heads=H, q_head_stride=dq, k_head_stride=d1, vt_head_stride=128, vt_row0=0, d1=d1, d2=d2, k2=k2,
                                   kv_group=group, ctx=ctx, pos0=0, scale=scale, status_ptr=fab.desc.status)
        ms = time_fn(run, flush, args.iters)
        assert fab.status() == 0
        # executed work: key tiles of 128 up to the diagonal of each 128-row query tile, QK^T (dq) + PV (128) MACs
        tiles = sum((min(ctx, t * 128 + 128) + 127) // 128 for t in range((m + 127) // 128))
        flops = 2.0 * H * tiles * 128 * 128 * (dq + 128)
        rec = {"rows": m, "context": ctx, "heads": H, "kv_group": group, "d1": d1, "d2": d2, "ms": round(ms, 4), "tflops_executed": round(flops / ms / 1e9, 1),
               "tflops_causal_exact": round(2.0 * H * (m * (m + 1) / 2) * (dq + 128) / ms / 1e9, 1)}
        if peaks:
            rec["of_measured_sustained"] = round(rec["tflops_executed"] / peaks["bf16_tflops_sustained"], 3)
        if args.library:
            qq = q.view(m, H, dq).transpose(0, 1).unsqueeze(0)
            kfull = torch.cat([k.view(ctx, Hkv, d1), k2.view(ctx, 1, d2).expand(ctx, Hkv, d2)], -1) if d2 else k.view(ctx, Hkv, d1)
            kk = kfull.repeat_interleave(group, 1).transpose(0, 1).unsqueeze(0).contiguous()
            vv = torch.nn.functional.pad(v, (0, dq - 128)).repeat_interleave(group, 1).transpose(0, 1).unsqueeze(0).contiguous() if dq > 128 else \
                v.repeat_interleave(group, 1).transpose(0, 1).unsqueeze(0).contiguous()
            lib = lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=scale)
            rec["library_sdpa_ms"] = round(time_fn(lib, flush, args.iters), 4)
        out.append(rec)
    print(json.dumps(out, indent=1))
    fab.close()


if __name__ == "__main__":
    main()
