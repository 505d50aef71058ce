"""Timings of the fused compute + collective kernels against their library compositions (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29571 \
        -m ironpangu_b200.utils.bench_fused gemm_ar | ag_gemm | ep

* ``gemm_ar``: row-parallel GEMM + all-reduce in one persistent tcgen05 kernel vs cuBLAS + NCCL all-reduce + add, 4096 x 4096 x 4096 / N
* ``ag_gemm``: all-gather fused into the column-parallel GEMM vs NCCL all-gather + cuBLAS
* ``ep``: expert-parallel dispatch + combine exchange of one flagship MoE layer vs NCCL all_to_all_single
Every number is device time per call (CUDA events), the maximum over ranks, with operand sets rotating so that inputs come
from HBM, and is printed with the roofline terms it is compared to (tensor-core time at the measured cuBLAS rate, link time
at the measured peer-copy rate).
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

BF16 = torch.bfloat16


def gemm_ar(rank: int, world: int) -> None:
    from ironpangu_b200.ops.gemm import gemm_allreduce
    from ironpangu_b200.parallel.fabric import Fabric

    # staging: every rank holds world partial copies of the tiles it owns (32 MB per parity half for a 4096 x 4096 output)
    fab = Fabric(rank, world, data_half_bytes=80 << 20, flag_half_words=16384)
    # A single call timed after a host barrier mostly measures how far apart the two processes launch, so
    # each sample times CALLS back-to-back calls that rotate over SETS operand sets (together larger than L2)
    M, N, Kl = 4096, 4096, 4096 // world
    SETS, CALLS = 4, 8
    a = [torch.randn(M, Kl, device="cuda").to(BF16) for _ in range(SETS)]
    b = [torch.randn(N, Kl, device="cuda").to(BF16) for _ in range(SETS)]
    res = [torch.randn(M, N, device="cuda").to(BF16) for _ in range(SETS)]
    out = [torch.empty(M, N, dtype=BF16, device="cuda") for _ in range(SETS)]
    sym = [fab.symmetric_empty((M, N)) for _ in range(SETS)]

    def timed(fn, iters=7):
        for i in range(3):
            fn(i % SETS)
        ts = []
        for _ in range(iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(CALLS):
                fn(i % SETS)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / CALLS], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]

    def baseline(i):
        torch.matmul(a[i], b[i].T, out=out[i])
        dist.all_reduce(out[i])
        out[i].add_(res[i])

    def gemm_only(i):
        torch.matmul(a[i], b[i].T, out=out[i])

    t_f = timed(lambda i: gemm_allreduce(a[i], b[i], fab, sym[i], residual=res[i]))
    t_b = timed(baseline)
    t_g = timed(gemm_only)
    assert fab.status() == 0
    link_bytes = 2 * (world - 1) / world * M * N * 2
    t_link = link_bytes / 770e9 * 1e3
    t_mma = 2.0 * M * N * Kl / 1.6705e15 * 1e3
    if rank == 0:
        print(json.dumps({"shape": f"{M}x{N}x{Kl}*{world}", "calls_per_sample": CALLS, "operand_sets": SETS,
                          "fused_ms": round(t_f, 4), "cublas_nccl_ms": round(t_b, 4), "cublas_gemm_only_ms": round(t_g, 4),
                          "roofline_ms": round(max(t_link, t_mma), 4), "link_ms": round(t_link, 4), "mma_ms": round(t_mma, 4),
                          "fraction_of_roofline": round(max(t_link, t_mma) / t_f, 3)}), flush=True)

    torch.cuda.synchronize()
    dist.barrier()
    fab.close()


def ag_gemm(rank: int, world: int) -> None:
    from ironpangu_b200.ops.gemm import AllGatherGemmState, allgather_gemm
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    rows_local, N, K = 4096 // world * 2, 4096, 4096
    bufs = [fab.symmetric_empty((rows_local, K)) for _ in range(2)]
    state = AllGatherGemmState(fab, rows_local, K)
    for bb in bufs:
        bb.tensor.normal_()
    b = torch.randn(N, K, device="cuda").to(BF16)
    gathered = torch.empty(rows_local * world, K, dtype=BF16, device="cuda")
    out = torch.empty(rows_local * world, N, dtype=BF16, device="cuda")

    def timed(fn, calls=8):
        for i in range(3):
            fn(i)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(calls):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / calls], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def fused(i):
        allgather_gemm(bufs[i & 1], b, state, fab, out=out)

    def baseline(i):
        dist.all_gather_into_tensor(gathered, bufs[i & 1].tensor)
        torch.matmul(gathered, b.T, out=out)

    tf, tb = timed(fused), timed(baseline)
    if rank == 0:
        M = rows_local * world
        print(json.dumps({"shape": f"{M}x{N}x{K}", "world": world, "fused_ms": round(tf, 4), "nccl_cublas_ms": round(tb, 4),
                          "mma_ms_at_measured_peak": round(2.0 * M * N * K / 1.6705e15 * 1e3, 4),
                          "link_ms": round((world - 1) * rows_local * K * 2 / 770e9 * 1e3, 4)}), flush=True)

    torch.cuda.synchronize()
    dist.barrier()
    fab.close()


def ep(rank: int, world: int) -> None:
    """Dispatch and combine exchange of one flagship MoE layer (hidden 4096, top-8 of 96 experts, 512 tokens per rank), device
    time per call, max over ranks, against the same payload through NCCL all_to_all_single with equal splits (routing built
    so that every destination receives the same number of rows, which spares the library path its size exchange)."""
    import json

    from ironpangu_b200.parallel.ep import EpExchange
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    E, topk, D, M = 96, 8, 4096, 512
    el = E // world
    ex = EpExchange(fab, M, topk, D, el)
    g = torch.Generator(device="cuda").manual_seed(3 + rank)
    h = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    # token t picks expert (t + k * E / topk) % E for k = 0..7: uniform over experts, hence over ranks
    ids = ((torch.arange(M, device="cuda")[:, None] + torch.arange(topk, device="cuda")[None, :] * (E // topk)) % E).to(torch.int32).contiguous()
    wts = torch.rand(M, topk, generator=g, device="cuda")
    res = torch.randn(M, D, generator=g, device="cuda").to(BF16)
    out = torch.empty(M, D, dtype=BF16, device="cuda")
    xp = torch.zeros(ex.rows_max, D, dtype=BF16, device="cuda")
    y = torch.zeros(ex.rows_max, D, dtype=BF16, device="cuda")

    def fused_dispatch():
        ex.dispatch(h, ids)
        ex.plan()
        ex.gather(xp)

    def fused_combine():
        ex.send_back(y)
        ex.combine(ids, wts, out, residual=res)

    rows = M * topk
    dest = (ids.view(-1).long() // el)
    order = torch.argsort(dest, stable=True)
    send = torch.empty(rows, D, dtype=BF16, device="cuda")
    recv = torch.empty(rows, D, dtype=BF16, device="cuda")
    back = torch.empty(rows, D, dtype=BF16, device="cuda")
    perm = torch.randperm(rows, device="cuda")
    inv = torch.argsort(order)

    def nccl_dispatch():
        torch.index_select(h, 0, order // topk, out=send)          # rows grouped by destination
        dist.all_to_all_single(recv, send)
        torch.index_select(recv, 0, perm, out=xp[:rows])            # owner: expert-sorted matrix

    def nccl_combine():
        torch.index_select(y[:rows], 0, perm, out=send)
        dist.all_to_all_single(back, send)
        r = torch.index_select(back, 0, inv).view(M, topk, D).float()
        out.copy_(((r * wts[:, :, None]).sum(1).to(BF16).float() + res.float()).to(BF16))

    def timed(pair, iters=10, calls=8):
        # `calls` layers (dispatch + combine) back to back between one pair of events: a single call timed after a host
        # synchronisation mostly measures host launch latency
        for _ in range(3):
            for fn in pair:
                fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(calls):
                for fn in pair:
                    fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / calls)
        ts.sort()
        v = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v[0])

    f = timed([fused_dispatch, fused_combine])
    n = timed([nccl_dispatch, nccl_combine]) if world > 1 else float("nan")
    link_ms = 2 * rows * D * 2 * (world - 1) / world / 770e9 * 1e3
    if rank == 0:
        print(json.dumps({"world": world, "tokens_per_rank": M, "topk": topk, "hidden": D,
                          "bytes_per_rank_both_directions": 2 * rows * D * 2 * (world - 1) // world,
                          "fused_dispatch_plus_combine_ms": round(f, 4), "nccl_dispatch_plus_combine_ms": round(n, 4),
                          "link_ms_at_770GBs": round(link_ms, 4), "fraction_of_link": round(link_ms / f, 3) if world > 1 else None}), flush=True)
    assert fab.status() == 0
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ex.close()
    fab.close()




def main() -> None:
    mode = sys.argv[1] if len(sys.argv) > 1 else ""
    modes = {"gemm_ar": gemm_ar, "ag_gemm": ag_gemm, "ep": ep}
    if mode not in modes:
        raise SystemExit("usage: bench_fused gemm_ar | ag_gemm | ep   (under torch.distributed.run, 2 or more ranks)")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world < 2:
        raise SystemExit("the fused collectives are timed on 2 or more ranks")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    modes[mode](rank, world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
