"""Prompt-chunk time of the tensor-parallel dense decoder: all-reduce layer stack against the sequence-parallel one.

Run under ``python -m torch.distributed.run --nproc-per-node N``. Both paths run the same chunk of ``--rows`` prompt tokens of
the 2B model (random-init weights; every rank streams its ~2 GB shard per call, more than the L2 holds) on the same weights;
the script checks that they pick the same next token, that no kernel reported a timeout, and prints the device time per chunk
(CUDA events, max over ranks).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="0 = the model's own depth")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.models import dense_gqa as G
    from ironpangu_b200.models.dense_prefill import DensePrefill
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = G.DenseConfig.qwen2b()
    if args.layers:
        cfg.layers = args.layers
    m = args.rows
    fab = Fabric(rank, world, data_half_bytes=32 << 20, flag_half_words=8192)
    weights = G.random_rank_weights(cfg, rank, world, "cuda", seed=1)
    mk = lambda: G.DenseDecoder(cfg, weights, fab, max_tokens=8, max_context=m, num_slots=1, keep_logits=False)
    plain, sp = DensePrefill(mk(), max_rows=m), DensePrefill(mk(), max_rows=m)
    assert sp.can_sequence_parallel(m), f"--rows must be a multiple of {128 * world}"
    toks = torch.randint(0, cfg.vocab, (m,), generator=torch.Generator().manual_seed(2)).to(torch.int32).cuda()
    runs = (("all-reduce", lambda: plain.forward(toks, 0, 0)), ("sequence-parallel", lambda: sp.forward(toks, 0, 0, sequence_parallel=True)))
    ids, times = {}, {}
    for name, run in runs:
        for _ in range(args.warmup):
            ids[name] = int(run())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times[name] = float(t)
    status = fab.status()
    if rank == 0:
        for name, _ in runs:
            print(f"dense 2B ({cfg.layers} layers) TP{world}, chunk of {m} rows, {name}: {times[name]:.3f} ms per chunk "
                  f"({m / times[name] * 1e3:.0f} prompt tokens/s), next token {ids[name]}", flush=True)
        print(f"fabric status {status:#x}, same next token: {ids['all-reduce'] == ids['sequence-parallel']}", flush=True)
    fab.close()
    dist.destroy_process_group()
    if status != 0:
        raise SystemExit(3)


if __name__ == "__main__":
    main()
