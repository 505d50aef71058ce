"""Tensor-parallel dense GQA decoder across real GPUs: decode kernels against the PyTorch oracle, and the tensor-core prompt
path / batched-row path (fused GEMM + all-reduce inside) against the decode kernels. Run under torch.distributed.run."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.models import dense_gqa as G
    from ironpangu_b200.models.dense_prefill import DensePrefill
    from ironpangu_b200.parallel.fabric import Fabric

    cfg = G.DenseConfig.tiny(2)
    if world > 2:
        cfg.kv_heads, cfg.heads = world, 2 * world          # every rank needs a KV head
    full = G.random_full_weights(cfg, seed=0)
    fab = Fabric(rank, world, data_half_bytes=32 << 20, flag_half_words=8192)
    mk = lambda slots: G.DenseDecoder(cfg, G.shard_weights(cfg, full, rank, world, "cuda"), fab, max_tokens=8, max_context=256,
                                      num_slots=slots, keep_logits=True)
    a, b = mk(3), mk(3)
    n = 150
    toks = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(5)).to(torch.int32).cuda()
    # decode kernels, 8 rows a time, against the oracle (vocabulary shard of this rank)
    for s in range(0, n, 8):
        k = min(8, n - s)
        b.tokens[:k].copy_(toks[s:s + k])
        b.positions[:k].copy_(torch.arange(s, s + k, dtype=torch.int32))
        b.slots[:k].zero_()
        b.forward(k)
    ref = G.forward_ref(cfg, full, toks.long(), tp=world)
    vl = cfg.vocab // world
    torch.testing.assert_close(b.logits[(n - 1) % 8], ref[n - 1, rank * vl:(rank + 1) * vl], rtol=3e-2, atol=3e-2)
    # tensor-core prompt path in chunks of 64 (row-parallel projections through the fused GEMM + all-reduce)
    pre = DensePrefill(a, max_rows=64, attn_rows=32)
    for s in range(0, n, 64):
        pre.forward(toks[s:s + 64], s, 0)
    torch.cuda.synchronize()
    torch.testing.assert_close(a.logits[0], b.logits[(n - 1) % 8], rtol=3e-2, atol=3e-2)
    for l in range(cfg.layers):
        torch.testing.assert_close(a.k_cache[l].float(), b.k_cache[l].float(), rtol=3e-2, atol=3e-2)
    # one decode row of the sequence plus rows of two fresh sequences as one batched pass
    step = torch.tensor([7, 11, 13], dtype=torch.int32, device="cuda")
    pos = torch.tensor([n, 0, 0], dtype=torch.int32, device="cuda")
    slots = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    got = pre.forward_rows(step, pos, slots, torch.tensor([0, 1, 2], device="cuda"))
    b.tokens[:3].copy_(step)
    b.positions[:3].copy_(pos)
    b.slots[:3].copy_(slots)
    b.forward(3)
    torch.cuda.synchronize()
    torch.testing.assert_close(got, b.logits[:3], rtol=3e-2, atol=3e-2)
    again = pre.forward_rows(step, pos, slots, torch.tensor([0, 1, 2], device="cuda"))      # same rows: replay of the captured graph
    torch.cuda.synchronize()
    assert torch.equal(again, got)
    if world > 1:
        sequence_parallel_check(cfg, full, fab, rank, world)
    assert fab.status() == 0, hex(fab.status())
    print(f"rank {rank}: ok dense tensor parallel", flush=True)
    fab.close()
    if world > 1:
        dist.destroy_process_group()


def sequence_parallel_check(cfg, full, fab, rank, world):
    """One chunk of 128 rows per rank through the sequence-parallel layer stack (all-gather GEMM -> attention -> GEMM +
    reduce-scatter, residual sharded by rows) against the all-reduce path: same next token, logits and caches."""
    from ironpangu_b200.models import dense_gqa as G
    from ironpangu_b200.models.dense_prefill import DensePrefill

    m = 128 * world
    mk = lambda: G.DenseDecoder(cfg, G.shard_weights(cfg, full, rank, world, "cuda"), fab, max_tokens=8, max_context=m,
                                num_slots=1, keep_logits=True)
    c1, c2 = mk(), mk()
    toks = torch.randint(0, cfg.vocab, (m,), generator=torch.Generator().manual_seed(9)).to(torch.int32).cuda()
    p1, p2 = DensePrefill(c1, max_rows=m, attn_rows=32), DensePrefill(c2, max_rows=m, attn_rows=32)
    assert p2.can_sequence_parallel(m) and not p2.can_sequence_parallel(m - 1)
    id1 = p1.forward(toks, 0, 0).clone()
    want = c1.logits[0].clone()
    for _ in range(2):                                  # the second call reuses shards, flags and counters one epoch later
        id2 = p2.forward(toks, 0, 0, sequence_parallel=True).clone()
        torch.cuda.synchronize()
        torch.testing.assert_close(c2.logits[0], want, rtol=3e-2, atol=3e-2)
        assert int(id1) == int(id2)
    for l in range(cfg.layers):
        torch.testing.assert_close(c2.k_cache[l].float(), c1.k_cache[l].float(), rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(c2.v_cache[l].float(), c1.v_cache[l].float(), rtol=3e-2, atol=3e-2)


if __name__ == "__main__":
    main()
