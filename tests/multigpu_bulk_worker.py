"""Worker for the bulk (prefill-sized) fused kernels: tcgen05 GEMM + two-shot all-reduce over peer memory.
Run under torch.distributed.run. (Timings of the same kernels: ``python -m ironpangu_b200.utils.bench_fused gemm_ar``.)"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BF16 = torch.bfloat16


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.ops.gemm import gemm_allreduce, gemm_reduce_scatter
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world, data_half_bytes=80 << 20, flag_half_words=16384, spin_limit=4_000_000)
    g = torch.Generator(device="cuda").manual_seed(9)
    for M, N, Kl in [(128, 256, 64), (512, 1024, 256), (300, 520, 128), (2048, 4096, 512), (1024, 776, 192)]:
        a = torch.randn(M, Kl * world, generator=g, device="cuda").to(BF16)
        b = (torch.randn(N, Kl * world, generator=g, device="cuda") * 0.05).to(BF16)
        res = torch.randn(M, N, generator=g, device="cuda").to(BF16)
        al, bl = a[:, rank * Kl:(rank + 1) * Kl].contiguous(), b[:, rank * Kl:(rank + 1) * Kl].contiguous()
        ref = torch.zeros(M, N, device="cuda")
        for r in range(world):
            ref += (a[:, r * Kl:(r + 1) * Kl].float() @ b[:, r * Kl:(r + 1) * Kl].float().T).to(BF16).float()
        ref = ref.to(BF16).float() + res.float()
        sym = fab.symmetric_empty((M, N))
        for _ in range(3):   # repeated calls exercise the parity double buffering
            y = gemm_allreduce(al, bl, fab, sym, residual=res)
        torch.cuda.synchronize()
        dist.barrier()
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=3e-2)
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert all(torch.equal(ys[0], t) for t in ys), "ranks hold different results"
        if M % (128 * world) == 0:
            # reduce-scatter form: every rank keeps its own row block (three calls: parity halves and the run-ahead guard)
            rows = M // world
            shard_res = res[rank * rows:(rank + 1) * rows].contiguous()
            for _ in range(3):
                ysh = gemm_reduce_scatter(al, bl, fab, residual=shard_res)
            torch.cuda.synchronize()
            dist.barrier()
            torch.testing.assert_close(ysh.float(), ref[rank * rows:(rank + 1) * rows], rtol=2e-2, atol=3e-2)
            assert torch.equal(ysh, y[rank * rows:(rank + 1) * rows]), "reduce-scatter and all-reduce forms disagree"
            # other fused kernels advance the fabric's call counter between reduce-scatter calls (the head of a decoder
            # does): consecutive reduce-scatters then land on the same staging half or skip one, and the guard against a
            # rank running ahead must still find the previous user of the half (no peer timeout, same result)
            from ironpangu_b200.ops.decode import gemv_allreduce
            xs, ws = torch.randn(2, 64, device="cuda").to(BF16), torch.randn(128, 64, device="cuda").to(BF16)
            for k in (1, 2, 1, 3):
                for _ in range(k):
                    gemv_allreduce(xs, ws, fab)
                ysh2 = gemm_reduce_scatter(al, bl, fab, residual=shard_res)
            torch.cuda.synchronize()
            dist.barrier()
            assert torch.equal(ysh2, ysh) and fab.status() == 0
    assert fab.status() == 0
    print(f"rank {rank}: ok gemm_allreduce bulk", flush=True)

    torch.cuda.synchronize()
    dist.barrier()
    fab.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
