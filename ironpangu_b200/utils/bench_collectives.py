"""Latency of the fused decode collectives inside CUDA graphs, against their no-collective and NCCL forms.

Run under ``python -m torch.distributed.run --nproc-per-node N`` (or plainly for one GPU). Every case is
a CUDA graph of ``--calls`` dependent launches; the per-call figure is device time / calls, median of
``--iters`` replays, max over ranks. Cases (flagship decode shapes, one query row):

    gemv              o_proj-shaped GEMV  [4096 x 4096/N], no collective
    gemv_allreduce    the same GEMV fused with the one-shot all-reduce
    nccl_allreduce    torch.distributed.all_reduce of the 4096-element bf16 row
    gemv+nccl         gemv followed by the NCCL all-reduce and the residual add (library composition)
    moe_down_ar       MoE down projection + combine + all-reduce with `topk/N` local routes
    lm_head_argmax    vocabulary-sharded head + greedy sampling exchange

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m ironpangu_b200.utils.bench_collectives --calls 64
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

BF16 = torch.bfloat16


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--calls", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    D, F, E, topk, V = 4096, 1536, 96, 8, 153600
    el, vl = E // world, V // world
    g = torch.Generator(device=dev).manual_seed(rank)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=dev) * 0.02).to(BF16)
    # several weight copies so that consecutive calls stream from HBM, not from L2
    NW = 6
    w_o = [rnd(D, D // world) for _ in range(NW)]
    x_k = rnd(1, D // world)
    x = rnd(1, D)
    res = rnd(1, D)
    y = torch.empty(1, D, dtype=BF16, device=dev)
    w_down = rnd(el, D, F)
    w_sdown = rnd(D, F // world)
    act = rnd(1, topk + 1, F)
    local_routes = max(1, topk // world)
    ids = torch.full((1, topk), -1, dtype=torch.int32, device=dev)
    # `local_routes` routes land on this rank, the others on the next rank's experts
    for k in range(topk):
        owner = rank if k < local_routes else (rank + 1 + (k % max(1, world - 1))) % world
        ids[0, k] = owner * el + (k % el)
    wts = torch.full((1, topk), 1.0 / topk, dtype=torch.float32, device=dev)
    w_head = rnd(vl, D)
    norm = torch.ones(D, dtype=BF16, device=dev)
    partial = torch.empty(((vl + 7) // 8) * 8 * 2, dtype=torch.float32, device=dev)
    out_ids = torch.zeros(1, dtype=torch.int32, device=dev)
    out_vals = torch.zeros(1, dtype=torch.float32, device=dev)
    yf = torch.empty(1, D, dtype=torch.float32, device=dev)

    def nccl(t):
        if world > 1:
            dist.all_reduce(t)

    def gemv_nccl(i):
        K.gemv(x_k, w_o[i % NW], out=yf, out_f32=True)
        nccl(yf)
        torch.add(yf, res, out=yf)

    cases = {
        "gemv": lambda i: K.gemv(x_k, w_o[i % NW], out=y),
        "gemv_allreduce": lambda i: K.gemv_allreduce(x_k, w_o[i % NW], fab, residual=res, out=y),
        "nccl_allreduce": lambda i: nccl(y),
        "gemv+nccl": gemv_nccl,
        "moe_down_ar": lambda i: K.moe_down_allreduce(act, ids, wts, w_down, rank * el, fab, w_shared_down=w_sdown,
                                                      residual=res, out=y),
        "lm_head_argmax": lambda i: K.lm_head_argmax(x, w_head, fab, norm_w=norm, eps=1e-5, vocab_offset=rank * vl,
                                                     partial=partial, out_ids=out_ids, out_vals=out_vals),
    }
    results = {}
    for name, fn in cases.items():
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(args.calls):
                fn(i)
        times = []
        for _ in range(args.iters):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / args.calls)
        t = torch.tensor([statistics.median(times)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[name] = round(float(t), 2)
    if rank == 0:
        print(json.dumps({"world": world, "calls_per_graph": args.calls, "us_per_call": results, "fabric_status": fab.status()}))
    if world > 1:
        dist.barrier()
    fab.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
