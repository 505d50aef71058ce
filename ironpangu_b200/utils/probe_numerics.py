"""Logit agreement of every execution path of the MLA + MoE decoder with the fp32 oracle, at the flagship layer shapes.

    python -m ironpangu_b200.utils.probe_numerics --layers 24 --tokens 48

Runs one prompt through (a) the native decode kernels one row at a time, (b) eight rows at a time, (c) the tensor-core prompt path,
(d) the cuBLAS + NCCL baseline with ``torch._grouped_mm`` experts and (e) with ``index_select + bmm`` experts, and reports each
path's |logits - oracle| at the last position (the oracle computes in fp32 from the same bf16 weights,
``models/mla_moe_ref.py``). The point of the depth sweep: bf16 rounding noise grows with the layer count for EVERY path alike, so
greedy tokens of two correct implementations differ wherever the oracle's top-2 gap is inside that noise.
One GPU; the oracle needs the layer count to leave room for fp32 copies of one layer's experts (<= 24 layers on 180 GB)."""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=48)
    args = ap.parse_args()
    from baseline.nccl_cublas import NcclCublasDecoder
    from ..models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ..models.mla_moe_prefill import MlaMoePrefill
    from ..models.mla_moe_ref import forward_ref
    from ..parallel.fabric import Fabric

    L, n = args.layers, args.tokens
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfg = MlaMoeConfig.flagship()
    cfg.layers = L
    w = random_rank_weights(cfg, 0, 1, dev)
    fab = Fabric(0, 1)
    prompt = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(0))
    ref = forward_ref(cfg, w, prompt.to(dev))
    gap = ref[-1].topk(2).values
    out = {"layers": L, "tokens": n, "oracle_top2_gap_last": float(gap[0] - gap[1]), "oracle_logit_std": float(ref[-1].std())}

    def report(name, logits_last, tok):
        d = (logits_last.float() - ref[-1]).abs()
        out[name] = {"max_abs": float(d.max()), "mean_abs": float(d.mean()), "rms": float(d.pow(2).mean().sqrt()),
                     "argmax_equal": int(tok) == int(ref[-1].argmax())}

    def rows(decoder, width):
        for s in range(0, n, width):
            m = min(width, n - s)
            decoder.tokens[:m].copy_(prompt[s:s + m].to(torch.int32))
            decoder.positions[:m].copy_(torch.arange(s, s + m, dtype=torch.int32))
            if hasattr(decoder, "slots"):
                decoder.slots[:m].zero_()
            decoder.forward(m)
        return decoder.logits[m - 1], decoder.next_ids[m - 1]

    dec = MlaMoeDecoder(cfg, w, fab, max_tokens=8, max_context=n + 64, keep_logits=True)
    report("native_decode_1row", *rows(dec, 1))
    dec.reset()
    report("native_decode_8rows", *rows(dec, 8))
    dec.reset()
    pre = MlaMoePrefill(dec, max_rows=min(512, n))
    nxt = None
    for s in range(0, n, pre.M):
        nxt = pre.forward(prompt[s:s + pre.M].to(torch.int32).to(dev), s, 0)
    report("native_prompt_path", dec.logits[0], nxt[0])
    b = NcclCublasDecoder(cfg, w, 0, 1, max_tokens=8, max_context=n + 64, keep_logits=True)
    report("library_" + b.expert_path, *rows(b, 8))
    if b.expert_path != "index_select+bmm":
        b.expert_path = "index_select+bmm"
        b.reset()
        report("library_index_select", *rows(b, 8))
    out["fabric_status"] = fab.status()
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
