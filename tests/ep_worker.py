"""Sharded-token expert parallelism across real GPUs: every rank owns different tokens and different experts.
Run under torch.distributed.run (any world size that divides 16 experts); with world 1 it runs in-process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BF16 = torch.bfloat16


def run(rank: int, world: int) -> None:
    from ironpangu_b200.ops import prefill as P
    from ironpangu_b200.parallel.ep import EpExchange
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    E, topk, D, F, Mmax = 16, 4, 256, 64, 48
    el = E // world
    g = torch.Generator(device="cuda").manual_seed(100)            # same on every rank: full weights, then sliced
    w_gu = (torch.randn(E, 2 * F, D, generator=g, device="cuda") * 0.06).to(BF16)
    w_dn = (torch.randn(E, D, F, generator=g, device="cuda") * 0.06).to(BF16)
    ex = EpExchange(fab, Mmax, topk, D, el)
    xp = torch.zeros(ex.rows_max, D, dtype=BF16, device="cuda")
    act = torch.empty(ex.rows_max, F, dtype=BF16, device="cuda")
    y = torch.empty(ex.rows_max, D, dtype=BF16, device="cuda")
    gl = torch.Generator(device="cuda").manual_seed(7 + rank)       # different tokens per rank
    for layer, M in enumerate([37, 48, 5]):                         # three "layers": buffers and flags are reused
        h = torch.randn(M, D, generator=gl, device="cuda").to(BF16)
        ids = torch.stack([torch.randperm(E, generator=gl, device="cuda")[:topk] for _ in range(M)]).to(torch.int32).contiguous()
        wts = torch.rand(M, topk, generator=gl, device="cuda")
        res = torch.randn(M, D, generator=gl, device="cuda").to(BF16)
        out = torch.empty(M, D, dtype=BF16, device="cuda")
        ex.dispatch(h, ids)
        ex.plan()
        ex.gather(xp)
        P.grouped_gemm(xp, w_gu[rank * el:(rank + 1) * el].contiguous(), ex.tiles, ex.num_tiles, act, swiglu=True)
        P.grouped_gemm(act, w_dn[rank * el:(rank + 1) * el].contiguous(), ex.tiles, ex.num_tiles, y)
        ex.send_back(y)
        ex.combine(ids, wts, out, residual=res)
        torch.cuda.synchronize()
        # reference on this rank's tokens with the full expert bank
        hf = h.float()
        want = torch.zeros(M, D, device="cuda")
        for t in range(M):
            for k in range(topk):
                e = int(ids[t, k])
                gu = (hf[t] @ w_gu[e].float().T).to(BF16).float()
                a = (torch.nn.functional.silu(gu[:F]) * gu[F:]).to(BF16).float()
                want[t] += wts[t, k] * (a @ w_dn[e].float().T).to(BF16).float()
        want = (want.to(BF16).float() + res.float()).to(BF16).float()
        torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-2)
        # bookkeeping: every rank received exactly the routes that name its experts
        mine = torch.tensor([int(((ids >= rank * el) & (ids < (rank + 1) * el)).sum())], device="cuda")
        if world > 1:
            counts = [torch.zeros_like(mine) for _ in range(world)]
            got = torch.tensor([int(ex.total_rows)], device="cuda")
            allids = [torch.empty(48 * topk, dtype=torch.int32, device="cuda") for _ in range(world)]
            pad = torch.full((48 * topk,), -1, dtype=torch.int32, device="cuda")
            pad[:M * topk] = ids.view(-1)
            dist.all_gather(allids, pad)
            expect = sum(int(((a >= rank * el) & (a < (rank + 1) * el)).sum()) for a in allids)
            assert int(got) == expect, (int(got), expect)
        else:
            assert int(ex.total_rows) == int(mine)
    assert fab.status() == 0
    print(f"rank {rank}: ok ep all-to-all world={world}", flush=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ex.close()
    fab.close()


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    run(rank, world)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
