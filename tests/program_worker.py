"""Compiled programs on several GPUs: the hyper-connected latent-attention + routed-experts family and the dense grouped-query
family, each compiled for the job's width and run by the plan engine of every rank against the CPU interpreter of the same
source (all ranks simulated on the host). Run under torch.distributed.run."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_program(text, rank, world, fab, tag, seed, route_aware):
    from ironpangu_b200 import compiler
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    shared = os.path.join(tempfile.gettempdir(), f"ifab-program-worker-{os.environ.get('MASTER_PORT', '0')}-{tag}")
    src = os.path.join(shared, "model.inferfabric")
    if rank == 0:
        os.makedirs(shared, exist_ok=True)
        with open(src, "w") as f:
            f.write(text)
        r = compiler.cli("synth-checkpoint", src, os.path.join(shared, "ck"), "--seed", str(seed))
        assert r.returncode == 0, r.stderr
    dist.barrier()
    bundle = os.path.join(tempfile.mkdtemp(prefix=f"ifab-pw-r{rank}-"), "bundle")
    compiler.write_bundle(src, bundle, checkpoint_dir=os.path.join(shared, "ck"), prefill_tokens=8)
    eng = PlanEngine(bundle, os.path.join(shared, "ck"), fab, max_tokens=8, keep_logits=True)
    vocab = next(int(i["attrs"]["vocab"]) for i in eng.ins if i["op"] == "embedding")
    toks = torch.randint(1, vocab, (29,), generator=torch.Generator().manual_seed(seed)).tolist()
    routers = [k for k, i in enumerate(eng.ins) if i["op"] == "router_topk"]
    oracle = compiler.interpret(text, os.path.join(shared, "ck"), toks, all_logits=True, watch=[eng.ins[k]["name"] for k in routers])
    ref = torch.tensor(oracle["prompt_logits"])
    vl = vocab // world
    picked = {}
    eng.probe = lambda k, T: picked.__setitem__(k, eng.vals[k][0][:T].tolist()) if k in routers else None
    same, tokens = 0, []
    for s in range(0, len(toks), 8):
        n = min(8, len(toks) - s)
        eng.tokens[:n].copy_(torch.tensor(toks[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        torch.cuda.synchronize()
        tokens += eng.next_ids[:n].tolist()
        for i in range(n):
            agree = all(sorted(picked[k][i]) == sorted(oracle["watched"][s + i][eng.ins[k]["name"]]["ids"]) for k in routers)
            same += agree
            if agree or not route_aware:
                torch.testing.assert_close(eng.logits[i].cpu(), ref[s + i, rank * vl:(rank + 1) * vl], rtol=4e-2, atol=4e-2)
    assert same >= len(toks) * 0.8, same
    assert fab.status() == 0
    # every rank samples the same token (sharded argmax across the fabric)
    t = torch.tensor(tokens, dtype=torch.int64, device="cuda")
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi)
    # one-row decode as a CUDA graph with device-side feedback continues the sequence identically on every rank
    eng.probe = None
    eng.tokens[:1].fill_(tokens[-1])
    eng.positions[:1].fill_(len(toks))
    g = eng.capture(1, feedback=True)
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    last = eng.next_ids[:1].to(torch.int64).clone()
    lo, hi = last.clone(), last.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    assert torch.equal(lo, hi) and fab.status() == 0


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, dense_gqa_source, hyper_mla_moe_source
    from ironpangu_b200.models.dense_gqa import DenseConfig
    from ironpangu_b200.parallel.fabric import Fabric

    fab = Fabric(rank, world)
    hc = HyperMlaMoeConfig.tiny(3)
    if world > 4:
        hc.heads = world
    run_program(hyper_mla_moe_source(hc, world, context=128), rank, world, fab, "hyper", 11, True)
    print("ok hyper program", flush=True)
    import dataclasses

    lc = dataclasses.replace(hc, packed_every=2, learned=True, index_heads=8, index_dim=64, index_rotary=32, index_topk=64)
    run_program(hyper_mla_moe_source(lc, world, context=128), rank, world, fab, "learned", 13, True)
    print("ok learned program", flush=True)
    dc = DenseConfig.tiny(2)
    if world > 2:
        dc.kv_heads, dc.heads = world, 2 * world
    run_program(dense_gqa_source(dc, world, context=128), rank, world, fab, "dense", 5, False)
    print("ok dense program", flush=True)
    fab.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
