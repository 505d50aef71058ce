"""Where a decode step of the MLA + MoE model spends its time, per kernel of the layer chain, at any world size.

Two measurements of the flagship-shaped decoder with a reduced layer count (one query row, ``--context`` keys):

* ``eager``: CUDA events around every kernel launch of one eager step (no overlap between kernels: an upper bound
  per kernel), reported as the maximum over ranks;
* ``graph``: the step as a CUDA graph with the programmatic-dependent-launch chain intact, timed as a whole, and again
  with one kernel of the chain left out at a time - the difference is what that kernel costs inside the chain. (The
  values that flow are wrong once a kernel is left out; the work and the dependencies of the others stay.)

Also reported: per-rank step time and its skew (max - min over ranks), and the routed experts per rank (max / mean).

    python -m ironpangu_b200.utils.profile_chain --layers 4                       # one GPU
    python -m ironpangu_b200.utils.profile_chain --layers 4 --shard-world 8       # rank 0's shard of 8, on one GPU
    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29561 -m ironpangu_b200.utils.profile_chain --layers 4

``--shard-world N`` (one process) runs the kernels of rank ``--shard-rank`` of an N-rank job at their real shapes
without the peers: the compute side of the chain, no NVLink exchange.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

CHAIN = ("gemv", "mla_head_decode", "gemv_allreduce", "router_topk", "moe_gate_up", "moe_down_allreduce", "moe_block")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--shard-world", type=int, default=0)
    ap.add_argument("--shard-rank", type=int, default=0)
    ap.add_argument("--replays", type=int, default=30)
    ap.add_argument("--skip-knockouts", action="store_true")
    ap.add_argument("--fused-moe", type=int, default=0, help="0: router, gate/up and down as three launches")
    args = ap.parse_args()

    import torch.distributed as dist

    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = MlaMoeConfig.flagship()
    cfg.layers = args.layers
    fab = Fabric(rank, world)
    shard = (args.shard_rank, args.shard_world) if args.shard_world else None
    srank, sworld = shard if shard else (rank, world)
    w = random_rank_weights(cfg, srank, sworld, dev)
    dec = MlaMoeDecoder(cfg, w, fab, max_tokens=1, max_context=args.context + 64, shard=shard, fused_moe=bool(args.fused_moe))
    dec.tokens.fill_(17)
    dec.slots.zero_()
    dec.positions.fill_(args.context)
    for c in dec.caches:
        c.normal_(0, 0.5)

    def gather_max(v):
        if world == 1:
            return v, v, v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        return float(hi[0]), float(lo[0]), v

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = {"world": world, "shard": list(shard) if shard else None, "layers": args.layers, "context": args.context}

    # ---- eager, events around every launch -----------------------------------------------------------------------------
    if True:   # eager pass
        names = [n for n in dir(K) if not n.startswith("_") and callable(getattr(K, n)) and
                 getattr(getattr(K, n), "__module__", "") == K.__name__]
        orig = {n: getattr(K, n) for n in names}
        records = []

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
        for s in range(4):
            records.clear()
            sync()
            dec.forward(1)
        torch.cuda.synchronize()
        for n in names:
            setattr(K, n, orig[n])
        agg = {}
        for n, e0, e1 in records:
            a = agg.setdefault(n, [0, 0.0])
            a[0] += 1
            a[1] += e0.elapsed_time(e1) * 1e3
        eager = {}
        for n in sorted(agg):
            hi, lo, _ = gather_max(agg[n][1] / agg[n][0])
            eager[n] = {"calls": agg[n][0], "us_max": round(hi, 2), "us_min": round(lo, 2)}
        out["eager_us_per_call"] = eager
        ids = dec.route_ids[:1].flatten().tolist()
        per_rank = [sum(1 for e in ids if e // dec.el == r) for r in range(sworld)]
        out["routes_last_layer"] = {"per_rank": per_rank, "max": max(per_rank), "mean": sum(per_rank) / len(per_rank)}

    # ---- graph of the whole step, and with one kernel of the chain left out ----------------------------------------------
    def timed_graph():
        sync()
        g = dec.capture(1, feedback=False)
        times = []
        for _ in range(args.replays):
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3)
        med = statistics.median(times)
        hi, lo, mine = gather_max(med)
        return hi, lo

    hi, lo = timed_graph()
    out["graph_step_us"] = {"max": round(hi, 1), "min": round(lo, 1), "skew": round(hi - lo, 1),
                            "per_layer": round(hi / args.layers, 2)}
    # back-to-back replays (what a decode loop does): no host gap between steps
    sync()
    g = dec.capture(1, feedback=False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(args.replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    hi, lo, _ = gather_max(e0.elapsed_time(e1) * 1e3 / args.replays)
    out["graph_back_to_back_us"] = {"max": round(hi, 1), "per_layer": round(hi / args.layers, 2)}
    if not args.skip_knockouts and world == 1:
        # leaving a kernel out is only done in one process: with peers, every rank would have to leave out the same
        # exchange, and the single-process shard run already isolates the compute side
        full = out["graph_step_us"]["max"]
        ko = {}
        for n in CHAIN:
            keep = getattr(K, n)
            setattr(K, n, lambda *a, **k: None)
            try:
                hi, _ = timed_graph()
            finally:
                setattr(K, n, keep)
            ko[n] = {"step_without_us": round(hi, 1), "cost_per_layer_us": round((full - hi) / args.layers, 2)}
        out["knockout"] = ko
    st = fab.status()
    out["fabric_status"] = st
    if rank == 0:
        print(json.dumps(out, indent=1))
    sync()
    fab.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
