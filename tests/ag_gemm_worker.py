"""All-gather fused into the column-parallel tcgen05 GEMM (remote activation tiles read with TMA from peer memory)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BF16 = torch.bfloat16


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.ops.gemm import AllGatherGemmState, allgather_gemm
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    for rows_local, N, K in [(128, 256, 64), (256, 520, 192), (384, 96, 1024)]:
        bufs = [fab.symmetric_empty((rows_local, K)) for _ in range(2)]
        state = AllGatherGemmState(fab, rows_local, K)
        g = torch.Generator(device="cuda").manual_seed(5)
        b = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(BF16)            # same on all ranks here; any local weight works
        for call in range(3):                                                            # alternate the two shard buffers
            gl = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
            shard = bufs[call & 1]
            shard.tensor.copy_(torch.randn(rows_local, K, generator=gl, device="cuda").to(BF16))
            c = allgather_gemm(shard, b, state, fab)
            torch.cuda.synchronize()
            if world > 1:
                parts = [torch.empty_like(shard.tensor) for _ in range(world)]
                dist.all_gather(parts, shard.tensor)
                full = torch.cat(parts)
            else:
                full = shard.tensor
            ref = full.float() @ b.float().T
            torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-2)
    assert fab.status() == 0
    print(f"rank {rank}: ok allgather gemm", flush=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    fab.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
