"""Headline benchmark: 92B-class MLA+MoE decoder, TP = EP = N GPUs, single sequence, 512-token context,
greedy decode - decode tokens/s for the whole box plus p50 TPOT and TTFT.

    python bench.py --gpus 1 --steps 128 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 128 --warmup 8

A "step" is one decode step (one new token of the sequence). Data are synthetic: uniform random token
ids for the prompt, N(0, 0.02) random-init weights of the named architecture generated on the device.
``--impl nccl_cublas`` runs the same model through cuBLAS linears + NCCL all-reduces (the in-repo
baseline); ``--impl reference`` would run the unmodified reference, which targets Ascend NPUs and has
no CUDA build, so it reports ``unavailable``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# best published decode TPOT of the reference: 17.7293 ms/token on 8x Ascend (graph, bf16 KV) = 56.40 tok/s
BASELINE_TOK_S = 1000.0 / 17.7293


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "nccl_cublas"])
    ap.add_argument("--model", default="flagship", choices=["flagship", "tiny", "dense2b"],
                    help="flagship: the 92B-class MLA+MoE model of the headline metric; dense2b: the Qwen-style 2B dense GQA decoder")
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--prefill", default="gemm", choices=["gemm", "decode"],
                    help="gemm: tensor-core prefill path (native impl only); decode: prompt through the decode kernels, 8 rows a time")
    ap.add_argument("--expert-fp8", action="store_true", help="block-scaled fp8 expert weights (the serving configuration; NOT the bf16 headline)")
    ap.add_argument("--kv-int8", action="store_true", help="packed int8 latent KV cache (the serving configuration; NOT the bf16 headline)")
    ap.add_argument("--layers", type=int, default=0, help="override layer count (marks the run as a reduced config)")
    ap.add_argument("--repeats", type=int, default=5, help="the timed loop of --steps steps runs this many times; the median is reported")
    ap.add_argument("--baseline-steps", type=int, default=16,
                    help="native arm, MLA+MoE models: also run the cuBLAS + NCCL decoder on the same weights in this process - compare "
                         "its first greedy tokens with the native arm's and time this many of its decode steps (0: skip)")
    ap.add_argument("--executor", default="bundle", choices=["bundle", "model"],
                    help="native arm, bf16 MLA+MoE models: 'bundle' compiles the model's .inferfabric source and runs the bundle's "
                         "program (runtime/plan_engine.py); 'model' runs the hand-wired decoder class (models/mla_moe.py)")
    ap.add_argument("--l2-prefetch", type=int, default=-1, help="-1: default (off); 1: the attention kernel requests the layer's next weights (o_proj, shared expert) into L2; 2: o_proj only")
    ap.add_argument("--fused-moe", type=int, default=-1, help="-1: decoder default; 0/1: MoE half of a layer as three launches / one")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def library_arm(cfg, weights, rank, world, max_context, prompt, native_tokens, native_logits, steps, dev, barrier, max_over_ranks):
    """The cuBLAS + NCCL decoder on the same weight tensors.

    (1) Greedy tokens: the library arm reads the same prompt and then the native arm's own tokens (teacher forcing, so that
    one early difference does not end the comparison); after every token its prediction is compared with the native arm's.
    Two correct bf16 implementations differ in summation order, so their logits differ by a measurable noise: eps = RMS over the
    vocabulary of (native logits - library logits) at that step. A differing token counts as agreeing when the library arm
    scores the native arm's token within 4.5 eps of its own best (a top-2 flip inside the noise); ``tokens_match`` is true when
    every compared position agrees in that sense. (2) Its decode step time over ``steps`` graph replays."""
    import torch
    import torch.distributed as dist

    from baseline.nccl_cublas import NcclCublasDecoder
    from ironpangu_b200.runtime.engine import DecodeEngine

    bdec = NcclCublasDecoder(cfg, weights, rank, world, max_tokens=8, max_context=max_context, keep_logits=True)
    beng = DecodeEngine(bdec)
    vl = bdec.vl

    def allreduce(t, op):
        if world > 1:
            dist.all_reduce(t, op=op)
        return t

    def judge(native_tok: int, ln, row: int = 0):
        lb = bdec.logits[row]
        best = allreduce(lb.max().reshape(1).clone(), dist.ReduceOp.MAX)
        local = native_tok - rank * vl
        mine = lb[local].reshape(1).clone() if 0 <= local < vl else torch.full((1,), float("-inf"), device=dev)
        mine = allreduce(mine, dist.ReduceOp.MAX)
        eps = None
        if ln is not None:
            sq = allreduce(((ln.float() - lb) ** 2).sum().reshape(1), dist.ReduceOp.SUM)
            eps = float(torch.sqrt(sq / (vl * world)))
        return float(best - mine), eps

    rows = []
    pred = beng.prefill(prompt)
    last_row = (len(prompt) - 1) % beng.chunk        # the prompt's last token is this row of the library arm's last chunk
    for i, tok in enumerate(native_tokens):
        margin, eps = judge(tok, native_logits[i], last_row if i == 0 else 0)
        rows.append((pred == tok, margin, eps))
        if i + 1 < len(native_tokens):
            pred = beng.step(tok)
    eps_seen = [e for _, _, e in rows if e is not None]
    eps_max = max(eps_seen) if eps_seen else 0.0
    agree = [same or margin <= 4.5 * (eps if eps is not None else eps_max) for same, margin, eps in rows]
    out = {"tokens_match": bool(all(agree)), "tokens_compared": len(rows), "tokens_identical": sum(1 for same, _, _ in rows if same),
           "largest_margin_of_a_differing_token": round(max([m for same, m, _ in rows if not same], default=0.0), 5),
           "logit_noise_rms": round(eps_max, 5), "expert_path": bdec.expert_path,
           # per compared position: identical?, the library arm's margin against the native token, the logit noise there
           "rows": [[int(same), round(margin, 4), None if eps is None else round(eps, 4)] for same, margin, eps in rows]}
    beng.run_device_loop(native_tokens[-1], 3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    beng.run_device_loop(None, steps)
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    out.update({"steps": steps, "ms_per_step": round(ms / steps, 4), "tokens_s": round(steps / (ms / 1e3), 3)})
    del beng, bdec
    torch.cuda.empty_cache()
    return out


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is a Rust + CANN/HCCL stack for Ascend NPUs: no Python package, no CUDA build, "
                          "no Rust toolchain in this image (pip install of the reference tree fails: no setup.py/pyproject)"}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # convenience: re-launch under torch.distributed.run
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29517", __file__] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL carries the bootstrap, the barriers and the max-over-ranks of the timing for the native arm (the model's
        # collectives are the fabric kernels over peer memory) and every collective of the cuBLAS + NCCL arm: library defaults
        dist.init_process_group("nccl", device_id=dev)

    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.engine import DecodeEngine

    dense = args.model == "dense2b"
    if dense:
        from ironpangu_b200.models import dense_gqa as G
        cfg = G.DenseConfig.qwen2b()
    else:
        cfg = MlaMoeConfig.flagship() if args.model == "flagship" else MlaMoeConfig.tiny(4)
    if args.layers:
        cfg.layers = args.layers
    K, W = args.steps, max(args.warmup, 3)
    R = max(1, args.repeats)
    CHECK = 16                                   # greedy tokens compared between the native and the library arm
    max_context = args.context + (R + 2) * K + 2 * W + CHECK + 64
    fab = Fabric(rank, world)
    t0 = time.time()
    bundle_sha = ""
    weights = (G.random_rank_weights if dense else random_rank_weights)(cfg, rank, world, dev, seed=0)
    torch.cuda.synchronize()
    weight_bytes = sum(t.numel() * t.element_size() for t in weights.values())
    if dense:
        if args.impl != "native":
            raise SystemExit("--model dense2b runs on the native path only")
        dec = G.DenseDecoder(cfg, weights, fab, max_tokens=8, max_context=max_context, num_slots=1)
    elif args.impl == "native" and args.executor == "bundle" and not args.expert_fp8:
        # compile the model's source for this tensor-parallel width and run the bundle's program: the dispatcher of the plan
        # engine picks the kernels, the activations live in the bundle's frozen arena, the weights are the tensors above
        import tempfile
        from ironpangu_b200 import compiler
        from ironpangu_b200.compiler.sources import mla_moe_source
        from ironpangu_b200.models.mla_moe import bundle_parameters
        from ironpangu_b200.runtime.plan_engine import PlanEngine
        work = tempfile.mkdtemp(prefix=f"ifab-bench-r{rank}-")
        src = os.path.join(work, "model.inferfabric")
        with open(src, "w") as f:
            f.write(mla_moe_source(cfg, world, context=max_context, kv_int8=args.kv_int8))      # packed int8 cache: declared in the source
        compiled = compiler.write_bundle(src, os.path.join(work, "bundle"), prefill_tokens=8)
        dec = PlanEngine(compiled["dir"], None, fab, max_tokens=8, num_slots=1, parameters=bundle_parameters(cfg, weights),
                         fused_moe=None if args.fused_moe < 0 else bool(args.fused_moe),
                         l2_prefetch=None if args.l2_prefetch < 0 else args.l2_prefetch)
        bundle_sha = compiled["program_sha256"]
    elif args.impl == "native":
        dec = MlaMoeDecoder(cfg, weights, fab, max_tokens=8, max_context=max_context, num_slots=1,
                            expert_fp8=args.expert_fp8, kv_int8=args.kv_int8,
                            fused_moe=None if args.fused_moe < 0 else bool(args.fused_moe))
        # fp8 experts are widened per layer for the prompt's GEMMs; over the int8 cache a prompt chunk attends in the latent form
    else:
        from baseline.nccl_cublas import NcclCublasDecoder
        dec = NcclCublasDecoder(cfg, weights, rank, world, max_tokens=8, max_context=max_context)
    pre = None
    if dense and args.prefill == "gemm":
        from ironpangu_b200.models.dense_prefill import DensePrefill
        pre = DensePrefill(dec, max_rows=min(512, args.context))
    elif args.impl == "native" and args.prefill == "gemm":
        from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
        pre = MlaMoePrefill(dec, max_rows=min(512, args.context))
    eng = DecodeEngine(dec, prefill=pre)
    init_s = time.time() - t0

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

    # ---- TTFT: prefill of the 512-token context (chunked through the same kernels) ------------------
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (args.context,), generator=g).tolist()
    eng.reset()
    warm = torch.randint(0, cfg.vocab, (args.context,), generator=g).tolist()
    eng.prefill(warm)          # warm-up with another prompt of the same length (module loading, graph capture of the chunk shape)
    eng.reset()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    first = eng.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    ttft_ms = max_over_ranks(e0.elapsed_time(e1))

    # ---- greedy tokens of the native arm against the cuBLAS + NCCL decoder on the same weights, and that decoder's step time ----
    native_tokens = [first]
    lib_arm = None
    if args.impl == "native" and not dense and args.baseline_steps > 0 and not (args.expert_fp8 or args.kv_int8):
        from ironpangu_b200.ops import decode as KK
        tok = first
        native_logits = [None]                 # the prompt's last row lives in the prefill path's buffers: no logits kept for it
        for _ in range(CHECK):
            tok = eng.step(tok)
            native_tokens.append(tok)
            # this step's logits of the local vocabulary shard, from the final hidden row (outside the step's own graph)
            native_logits.append(KK.gemv(dec.x[:1], weights["lm_head"], norm_w=weights["final_norm"], eps=cfg.eps, out_f32=True)[0])
        try:
            lib_arm = library_arm(cfg, weights, rank, world, max_context, prompt, native_tokens, native_logits,
                                  args.baseline_steps, dev, barrier, max_over_ranks)
        except Exception as exc:          # e.g. no memory left beside a one-GPU shard of 175 GB: the native numbers still stand
            lib_arm = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            if world > 1:
                raise
        first = native_tokens[-1]

    # ---- device-timed decode: feedback graph, no host round trips; median of R runs of K steps -------
    eng.run_device_loop(first, W)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    runs = []
    for _ in range(R):
        barrier()
        e0.record()
        eng.run_device_loop(None, K)
        e1.record()
        barrier()
        runs.append(max_over_ranks(e0.elapsed_time(e1)))
    dev_ms = statistics.median(runs)

    # ---- per-step TPOT distribution (events around every replay) -----------------------------------
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    d = dec
    evs[0].record()
    for i in range(K):
        eng._feedback_graph.replay()
        evs[i + 1].record()
    eng.pos += K
    torch.cuda.synchronize()
    tpots = [evs[i].elapsed_time(evs[i + 1]) for i in range(K)]
    tpot_p50 = max_over_ranks(statistics.median(tpots))

    # ---- end to end through the public API: H2D control inputs + replay + D2H token every step ------
    tok = first
    for _ in range(W):
        tok = eng.step(tok)
    barrier()
    e0.record()
    for _ in range(K):
        tok = eng.step(tok)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    status = fab.status()

    # launches of this package's kernels in one step, counted at the entry points (one eager step after the timing)
    launches_counted = None
    if args.impl == "native":
        from ironpangu_b200.ops import _lib as native_lib
        n0 = native_lib.launch_count
        dec.forward(1)
        torch.cuda.synchronize()
        launches_counted = native_lib.launch_count - n0
    if rank == 0:
        per_step_launches = launches_counted if launches_counted is not None else getattr(dec, "launches_per_forward", 0)
        value = K / (dev_ms / 1e3)
        line = {
            "metric": "decode_tokens_per_s_per_box", "value": round(value, 3), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None if dense else round(value / BASELINE_TOK_S, 3),
            "dtype": "bf16" + (" activations, fp8 block-scaled experts" if args.expert_fp8 else "") + (", int8 KV" if args.kv_int8 else ""), "impl": args.impl,
            "data": "synthetic (uniform random prompt ids; N(0,0.02) random-init weights generated on device)",
            "config": {"model": ("92B-class MLA+MoE: 46L hidden 4096, 32 heads, q_lora 1536, kv_lora 512, nope 128, rope 64, "
                                 "v 128, 96 experts x 1536 top-8 softmax + 1 shared, vocab 153600") if args.model == "flagship"
                       and not args.layers else ("Qwen-style 2B dense: 24L hidden 2048, 16 q / 4 kv heads x 128, SwiGLU 6144, vocab 151936 "
                                                 "(not the headline model)") if dense and not args.layers
                       else f"{args.model} layers={cfg.layers} (reduced config)",
                       "params_b": round(cfg.param_count() / 1e9, 2), "global_batch": 1, "seq_len": args.context,
                       "decode_tokens": K, "parallelism": f"tp{world}" if dense else f"tp{world}ep{world}", "decode_step": (f"compiled bundle {bundle_sha[:16]}: plan engine, {dec.launches_per_forward} launches" if bundle_sha else "operator chain"),
                       "prefill": args.prefill if args.impl == "native" else "library",
                       "l2": "per-step weight stream (>= 2.5 GB per rank) exceeds the 126 MB L2; no explicit flush",
                       "baseline_ref": "17.7293 ms TPOT on 8x Ascend (docs/validation/2026-10-17-packed-c8/README.md:20-23)",
                       "weight_bytes_per_rank": weight_bytes},
            "tpot_p50_ms": round(tpot_p50, 4), "ttft_ms": round(ttft_ms, 3),
            "e2e": {"value": round(K / (e2e_ms / 1e3), 3), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 4),
                    "h2d_bytes_per_step": eng.h2d_bytes_per_step, "d2h_bytes_per_step": eng.d2h_bytes_per_step},
            "gpu_launches": per_step_launches * K, "launches_per_step": per_step_launches, "clocks": clocks, "fabric_status": status,
            "timed_runs_ms": [round(v, 3) for v in runs], "init_s": round(init_s, 1),
        }
        if args.impl == "native" and not dense:
            line["config"]["moe_block"] = "one launch" if getattr(dec, "fused_moe", False) else "router, gate/up, down"
            line["config"]["nvls"] = bool(getattr(fab, "mc", 0))
        if lib_arm is not None:
            line["tokens_match"] = lib_arm.pop("tokens_match", None)
            line["nccl_cublas"] = lib_arm
        print(json.dumps(line))
    barrier()
    if hasattr(fab, "close"):
        fab.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
