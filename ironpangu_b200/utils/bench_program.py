"""Decode benchmark of any model program: compile a ``.inferfabric`` source (or one of the built-in generators) for the job's
width, fill the parameters of every rank's initialization plan with random values on the device, run the bundle on the plan
engine, replay the one-row decode step as a CUDA graph with device-side token feedback, and report the time per output token.

    python -m ironpangu_b200.utils.bench_program --model pangu92b --gpus 8 --context 512 --prompt 64 --decode 31

``--model pangu92b`` is the published 92B configuration of the hyper-connected latent-attention family (46 layers, 256 routed
experts, 48 heads, 4 residual streams, 128 sink rows, token convolutions), the model the reference quotes its time per output
token on (TP8 / EP8, context capacity 512, batch one, graph replay, 30 inter-token intervals). One JSON line on rank 0; every
time is measured on the device with CUDA events and is the maximum over ranks.
Reference: docs/validation/2026-10-17-packed-c8/README.md (the published number and its workload)."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="hyper-tiny", help="pangu92b | pangu92b-learned (packed int8 caches + learned sparse attention on every third layer) | hyper-tiny | flagship | tiny | dense2b | dense-tiny")
    ap.add_argument("--source", default="", help="a .inferfabric file instead of a built-in generator (compiled as written)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--decode", type=int, default=31, help="output tokens per run (intervals = decode - 1)")
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--eager", action="store_true", help="launch the step kernel by kernel instead of replaying a graph")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def source_of(args, world: int) -> tuple:
    """(source text, description) of the program to run."""
    from ironpangu_b200.compiler import sources as S

    if args.source:
        return open(args.source).read(), os.path.basename(args.source)
    if args.model in ("pangu92b", "pangu92b-learned", "hyper-tiny"):
        c = {"pangu92b": S.HyperMlaMoeConfig.pangu92b, "pangu92b-learned": S.HyperMlaMoeConfig.pangu92b_learned,
             "hyper-tiny": S.HyperMlaMoeConfig.tiny}[args.model]()
        if args.layers:
            c.layers = args.layers
        return S.hyper_mla_moe_source(c, world, context=args.context), (
            f"{c.layers}L hidden {c.hidden} x {c.streams} streams, {c.heads} heads, q_lora {c.q_lora}, {c.experts} experts x {c.expert_ffn} "
            f"top-{c.topk}, {c.sinks} sinks, vocab {c.vocab}" + (f", packed cache + learned top-{c.index_topk} selection every {c.packed_every} layers" if c.learned else ""))
    if args.model in ("flagship", "tiny"):
        from ironpangu_b200.models.mla_moe import MlaMoeConfig

        c = MlaMoeConfig.flagship() if args.model == "flagship" else MlaMoeConfig.tiny(4)
        if args.layers:
            c.layers = args.layers
        return S.mla_moe_source(c, world, context=args.context), f"{c.layers}L hidden {c.hidden}, {c.heads} heads, {c.experts} experts"
    from ironpangu_b200.models.dense_gqa import DenseConfig

    c = DenseConfig.qwen2b() if args.model == "dense2b" else DenseConfig.tiny(2)
    if args.layers:
        c.layers = args.layers
    return S.dense_gqa_source(c, world, context=args.context), f"{c.layers}L hidden {c.hidden}, {c.heads}/{c.kv_heads} heads x {c.head_dim}"


def main(argv=None) -> int:
    args = parse(argv)
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
                   "--master-port", "29531", "-m", "ironpangu_b200.utils.bench_program"] + (sys.argv[1:] if argv is None else list(argv))
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)      # bootstrap, barriers and the max over ranks; the model's collectives are the fabric's

    from ironpangu_b200 import compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine, random_parameters

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    t0 = time.time()
    text, what = source_of(args, world)
    work = tempfile.mkdtemp(prefix=f"ifab-program-r{rank}-")
    src = os.path.join(work, "model.inferfabric")
    with open(src, "w") as f:
        f.write(text)
    compiled = compiler.write_bundle(src, os.path.join(work, "bundle"), prefill_tokens=8)       # every rank compiles the same bundle
    compile_s = time.time() - t0
    plan = json.loads(open(os.path.join(compiled["dir"], f"rank-{rank}.init.json")).read())
    fab = Fabric(rank, world)
    t0 = time.time()
    params = random_parameters(plan, dev, seed=args.seed)
    torch.cuda.synchronize()
    weight_bytes = sum(t.numel() * t.element_size() for t in params.values())
    eng = PlanEngine(compiled["dir"], None, fab, max_tokens=8, num_slots=1, parameters=params)
    init_s = time.time() - t0
    if args.prompt + args.decode + 1 > eng.max_context:
        raise SystemExit(f"prompt + decode exceeds the program's context ({eng.max_context})")
    vocab = next(int(i["attrs"]["vocab"]) for i in eng.ins if i["op"] == "embedding")
    g = torch.Generator().manual_seed(args.seed)

    def prefill(tokens) -> int:
        """The prompt in launch groups of eight rows through the same kernels; returns the first output token."""
        eng.reset()
        for s in range(0, len(tokens), 8):
            n = min(8, len(tokens) - s)
            eng.tokens[:n].copy_(torch.tensor(tokens[s:s + n], dtype=torch.int32))
            eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
            eng.slots[:n].zero_()
            eng.forward(n)
        return int(eng.next_ids[n - 1])

    # warm-up: one prompt, the graph of the one-row step with feedback, W replays
    first = prefill(torch.randint(0, vocab, (args.prompt,), generator=g).tolist())
    eng.tokens[:1].fill_(first)
    eng.positions[:1].fill_(args.prompt)
    graph = None if args.eager else eng.capture(1, feedback=True)
    for _ in range(max(3, args.warmup)):
        eng.forward_feedback(1) if graph is None else graph.replay()
    barrier()
    runs, tokens_out = [], []
    for r in range(args.runs):
        prompt = torch.randint(0, vocab, (args.prompt,), generator=g).tolist()
        barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        first = prefill(prompt)
        e1.record()
        eng.tokens[:1].fill_(first)
        eng.positions[:1].fill_(args.prompt)
        out = torch.zeros(args.decode, dtype=torch.int32, device=dev)
        out[0] = first
        torch.cuda.synchronize()
        barrier()
        e1.record()
        for i in range(1, args.decode):
            eng.forward_feedback(1) if graph is None else graph.replay()
            out[i:i + 1].copy_(eng.next_ids[:1])
        e2.record()
        barrier()
        runs.append(max_over_ranks(e1.elapsed_time(e2)) / (args.decode - 1))
        tokens_out.append(out.tolist())
    status = int(fab.status())
    if world > 1:
        same = torch.tensor(tokens_out[-1], dtype=torch.int64, device=dev)
        lo, hi = same.clone(), same.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ranks_agree = bool(torch.equal(lo, hi))
    else:
        ranks_agree = True
    if rank == 0:
        runs_sorted = sorted(runs)
        tpot = runs_sorted[len(runs_sorted) // 2]
        print(json.dumps({"metric": "time_per_output_token_ms", "value": round(tpot, 4), "unit": "ms", "higher_is_better": False, "n_gpus": world,
                          "tokens_per_s": round(1000.0 / tpot, 2), "runs_ms": [round(x, 4) for x in runs], "intervals_per_run": args.decode - 1,
                          "model": args.source or args.model, "description": what, "context_capacity": eng.max_context, "prompt": args.prompt,
                          "dtype": "bf16", "data": "synthetic (uniform random prompt ids; N(0,0.02) random-init parameters drawn on the device)",
                          "program_sha256": compiled["program_sha256"], "instructions": compiled["instructions"],
                          "launches_per_step": eng.launches_per_forward, "step": "eager" if graph is None else "cuda graph replay with device-side feedback",
                          "weight_bytes_per_rank": weight_bytes, "arena_bytes": eng.arena.bytes + eng.arena.workspace_bytes,
                          "compile_s": round(compile_s, 2), "init_s": round(init_s, 2), "fabric_status": status, "ranks_agree_on_tokens": ranks_agree,
                          "tokens_head": tokens_out[-1][:8]}))
    fab.close()
    if world > 1:
        dist.destroy_process_group()
    return 0 if status == 0 and ranks_agree else 1


if __name__ == "__main__":
    sys.exit(main())
