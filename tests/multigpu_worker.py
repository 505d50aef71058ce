"""Worker run under ``torch.distributed.run`` by test_multigpu.py: one rank per GPU, NCCL for plumbing.

Checks, at world size N:
  1. fused row-parallel GEMV + one-shot all-reduce == f32 reference built from all ranks' shards
  2. vocabulary-sharded lm_head + argmax exchange gives every rank the global greedy token
  3. the tiny MLA+MoE decoder (TP = EP = N) reproduces the oracle's logits / greedy tokens, eager and
     under CUDA-graph replay, with a clean status word
Writes ``ok`` lines to stdout; any assertion failure exits non-zero.
"""
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
    from ironpangu_b200.ops import decode as K
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_full_weights, shard_weights
    from ironpangu_b200.models.mla_moe_ref import forward_ref, rmsnorm_ref

    fab = Fabric(rank, world, spin_limit=2_000_000)
    print(f"rank {rank}: nvls {'on' if fab.mc else 'off'}", flush=True)

    # 1. fused GEMV + all-reduce -------------------------------------------------------------------
    g = torch.Generator(device="cuda").manual_seed(5)
    for T, N, Kf in [(1, 4096, 512 * world), (4, 1024, 256 * world), (8, 264, 64 * world)]:
        x = (torch.randn(T, Kf, generator=g, device="cuda")).to(BF16)
        w = (torch.randn(N, Kf, generator=g, device="cuda") * 0.05).to(BF16)
        res = torch.randn(T, N, generator=g, device="cuda").to(BF16)
        kl = Kf // world
        xs, ws = x[:, rank * kl:(rank + 1) * kl].contiguous(), w[:, rank * kl:(rank + 1) * kl].contiguous()
        ref = torch.zeros(T, N, device="cuda")
        for r in range(world):
            ref = ref + x[:, r * kl:(r + 1) * kl].float() @ w[:, r * kl:(r + 1) * kl].float().T
        ref = ref.to(BF16).float() + res.float()
        for it in range(5):  # repeated calls exercise the parity double buffering
            y = K.gemv_allreduce(xs, ws, fab, residual=res)
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
        # every rank must hold bit-identical results (rank-ordered summation)
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert all(torch.equal(ys[0], t) for t in ys)
    assert fab.status() == 0
    print(f"rank {rank}: ok gemv_allreduce", flush=True)

    # 2. sharded lm_head argmax -------------------------------------------------------------------
    T, D, V = 4, 256, 1024 * world
    x = torch.randn(T, D, generator=g, device="cuda").to(BF16)
    nw = (torch.randn(D, generator=g, device="cuda") * 0.1 + 1).to(BF16)
    w = (torch.randn(V, D, generator=g, device="cuda") * 0.05).to(BF16)
    vl = V // world
    ids = K.lm_head_argmax(x, w[rank * vl:(rank + 1) * vl].contiguous(), fab, norm_w=nw, vocab_offset=rank * vl)
    ref = (rmsnorm_ref(x, nw, 1e-5) @ w.float().T).argmax(-1)
    assert torch.equal(ids.long(), ref), (ids, ref)
    print(f"rank {rank}: ok lm_head_argmax", flush=True)

    # 3. tiny model, TP = EP = world ---------------------------------------------------------------
    cfg = MlaMoeConfig.tiny(2)
    full = random_full_weights(cfg, seed=0)
    dec = MlaMoeDecoder(cfg, shard_weights(cfg, full, rank, world, "cuda"), fab, max_tokens=1, max_context=64,
                        keep_logits=True)
    prompt = [5, 77, 300, 12, 999, 41, 8, 650]
    ref = forward_ref(cfg, full, torch.tensor(prompt, device="cuda"), tp=world)
    vl = cfg.vocab // world
    eager_ids = []
    for i, t in enumerate(prompt):
        dec.tokens.fill_(t)
        dec.positions.fill_(i)
        dec.forward(1)
        torch.testing.assert_close(dec.logits[0], ref[i, rank * vl:(rank + 1) * vl], rtol=2e-2, atol=2e-2)
        eager_ids.append(int(dec.next_ids[0]))
        top2 = ref[i].topk(2).values
        if float(top2[0] - top2[1]) > 5e-3:
            assert eager_ids[-1] == int(ref[i].argmax())
    dec.reset()
    dec.capture(1)
    graph_ids = []
    for i, t in enumerate(prompt):
        dec.tokens.fill_(t)
        dec.positions.fill_(i)
        dec._graph.replay()
        graph_ids.append(int(dec.next_ids[0]))
    assert graph_ids == eager_ids, (graph_ids, eager_ids)
    all_ids = [None] * world
    dist.all_gather_object(all_ids, graph_ids)
    assert all(a == all_ids[0] for a in all_ids), "ranks disagree on the sampled tokens"
    assert fab.status() == 0
    # tensor-core prefill path (fused GEMM + all-reduce for o_proj, pull all-reduce after the MoE), then decode on its cache
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    pdec = MlaMoeDecoder(cfg, shard_weights(cfg, full, rank, world, "cuda"), fab, max_tokens=1, max_context=64, keep_logits=True)
    pre = MlaMoePrefill(pdec, max_rows=8, attn_rows=8)
    nxt = pre.forward(torch.tensor(prompt[:7], dtype=torch.int32, device="cuda"), 0)
    torch.testing.assert_close(pdec.logits[0], ref[6, rank * vl:(rank + 1) * vl], rtol=3e-2, atol=3e-2)
    pdec.tokens.fill_(prompt[7])
    pdec.positions.fill_(7)
    pdec.forward(1)
    torch.testing.assert_close(pdec.logits[0], ref[7, rank * vl:(rank + 1) * vl], rtol=3e-2, atol=3e-2)
    # rows with their own positions through the matrix-matrix path (the batched decode step of the serving engine); the
    # second call has the same row count and replays the recorded graph
    ext = prompt + [3, 9, 27, 81]
    ref = forward_ref(cfg, full, torch.tensor(ext, device="cuda"), tp=world)
    for lo in (8, 10):
        rows = torch.tensor(ext[lo:lo + 2], dtype=torch.int32, device="cuda")
        got = pre.forward_rows(rows, torch.tensor([lo, lo + 1], dtype=torch.int32, device="cuda"),
                               torch.zeros(2, dtype=torch.int32, device="cuda"), torch.tensor([0, 1], device="cuda"))
        torch.testing.assert_close(got, ref[lo:lo + 2, rank * vl:(rank + 1) * vl], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    print(f"rank {rank}: ok prefill path tp={world}", flush=True)
    print(f"rank {rank}: ok tiny model tp={world}", flush=True)
    # 4. dense GQA model (TP = world when the tiny model's kv heads divide) + cross-rank top-k sampling
    from ironpangu_b200.models import dense_gqa as D
    dcfg = D.DenseConfig.tiny(2)
    if dcfg.kv_heads % world == 0:
        dfull = D.random_full_weights(dcfg, 0)
        ddec = D.DenseDecoder(dcfg, D.shard_weights(dcfg, dfull, rank, world, "cuda"), fab, max_tokens=8, max_context=64, keep_logits=True)
        dref = D.forward_ref(dcfg, dfull, torch.tensor(prompt, device="cuda"), tp=world)
        n = len(prompt)
        ddec.tokens[:n].copy_(torch.tensor(prompt, dtype=torch.int32))
        ddec.positions[:n].copy_(torch.arange(n, dtype=torch.int32))
        ddec.slots[:n].zero_()
        ddec.forward(n)
        dvl = dcfg.vocab // world
        torch.testing.assert_close(ddec.logits[:n], dref[:, rank * dvl:(rank + 1) * dvl], rtol=2e-2, atol=2e-2)
        seeds = torch.full((n,), 5, dtype=torch.int64, device="cuda")
        counters = torch.zeros(n, dtype=torch.int64, device="cuda")
        invt = torch.full((n,), 1 / 0.7, device="cuda")
        ids = K.sample_topk(ddec.logits[:n], fab, top_k=50, inv_temperature=invt, seeds=seeds, counters=counters, vocab_offset=rank * dvl)
        full_logits = [torch.empty_like(ddec.logits[:n]) for _ in range(world)]
        dist.all_gather(full_logits, ddec.logits[:n].contiguous())
        allowed = torch.cat(full_logits, 1).topk(50, -1).indices
        for t in range(n):
            assert int(ids[t]) in allowed[t].tolist()
        got = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(got, ids)
        assert all(torch.equal(got[0], x) for x in got), "ranks drew different tokens"
        print(f"rank {rank}: ok dense gqa + sampling tp={world}", flush=True)
    assert fab.status() == 0
    torch.cuda.synchronize()
    dist.barrier()
    fab.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
