"""Per-phase time of the single-launch decode step, measured inside the kernel (global timer stamps after every
grid barrier). Flagship shapes with a reduced layer count by default; works under torch.distributed.run too.

    python -m ironpangu_b200.utils.trace_step --layers 8 --context 512
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29544 \
        -m ironpangu_b200.utils.trace_step --layers 8
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--repeat", type=int, default=5)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = MlaMoeConfig.flagship()
    cfg.layers = args.layers
    fab = Fabric(rank, world)
    w = random_rank_weights(cfg, rank, world, dev)
    dec = MlaMoeDecoder(cfg, w, fab, max_tokens=max(1, args.tokens), max_context=args.context + 64, persistent=True)
    T = args.tokens
    dec.tokens[:T].fill_(17)
    dec.slots[:T].zero_()
    dec.positions[:T].copy_(torch.arange(args.context, args.context + T, dtype=torch.int32))
    for c in dec.caches:
        c.normal_(0, 0.5)
    for _ in range(3):
        dec.forward(T)
    runs = [dec.trace_step(T) for _ in range(args.repeat)]
    best = min(runs, key=lambda r: r["total"])
    per_layer = {k: round(v / cfg.layers, 2) for k, v in best.items() if k in dec.PHASES}
    if rank == 0:
        print(json.dumps({"world": world, "layers": cfg.layers, "tokens": T, "context": args.context,
                          "us_per_layer": per_layer, "layer_us": round(sum(per_layer.values()), 2),
                          "embedding_us": round(best["embedding"], 2), "head_us": round(best["head"], 2),
                          "total_us": round(best["total"], 1), "fabric_status": fab.status()}))
    if world > 1:
        dist.barrier()
    fab.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
