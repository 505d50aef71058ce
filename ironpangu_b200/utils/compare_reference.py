"""Token-level comparison of a serving engine with the CPU oracle, with a divergence analysis of the first differing token.

    # 1. reference cases from the CPU interpreter of the model source (greedy; logits kept for the analysis)
    python -m ironpangu_b200.utils.compare_reference make-reference MODEL.inferfabric CHECKPOINT_DIR cases.json \
        --prompts 4 --prompt-tokens 12 --new-tokens 8 [--seed 0]
    # 2. the engine under test behind ifab-server (any engine: --program, --spawn ...), every case `--repetitions` times
    python -m ironpangu_b200.utils.compare_reference compare cases.json http://127.0.0.1:PORT report.json [--repetitions 3]

The report (format ``ifab.reference-comparison.v1``) has, per case: the reference and the engine's tokens of every repetition,
``exact_all_tokens``, ``exact_through_reference_eos``, ``stable_repetitions`` (an engine must agree with itself before it can
agree with anything else), time to first token and time per output token from the stream, and - where the tokens differ -
``first_difference``: the position, both tokens and the oracle's logit gap between them at equal history. A gap inside bf16
noise (``--noise``, default 1e-2) is a near-tie that two correct implementations may break differently; a larger one is a
defect. Exit code 0 only if every case is exact or differs inside the noise and is stable.
Reference: scripts/compare-program-reference.py:15-57, scripts/analyze-token-divergence.py:14-58."""
from __future__ import annotations

import argparse
import hashlib
import http.client
import json
import random
import statistics
import sys
import time
from pathlib import Path
from typing import Dict, List
from urllib.parse import urlparse


def make_reference(model: str, checkpoint: str, prompts: int, prompt_tokens: int, new_tokens: int, seed: int) -> List[Dict]:
    from .. import compiler

    source = Path(model).read_text()
    info = compiler.compile_source(source)
    vocab = max(int(n["attrs"]["vocab"]) for n in info["graph"]["nodes"] if n["op"] == "embedding") if "graph" in info else 256
    rng = random.Random(seed)
    cases = []
    for c in range(prompts):
        ids = [rng.randrange(1, vocab) for _ in range(prompt_tokens + c)]
        first = compiler.interpret(source, checkpoint, ids, steps=new_tokens)
        out = first["generated"]
        teacher = compiler.interpret(source, checkpoint, ids + out, all_logits=True)["prompt_logits"]
        # logits that chose output token i: the row after position len(ids) - 1 + i
        rows = [teacher[len(ids) - 1 + i] for i in range(len(out))]
        cases.append({"case": f"case-{c}", "input_ids": ids, "output_ids": out, "logits_top": [_top(r, 8) for r in rows]})
    return cases


def _top(row: List[float], k: int) -> Dict[str, float]:
    idx = sorted(range(len(row)), key=lambda i: -row[i])[:k]
    return {str(i): row[i] for i in idx}


def stream_generate(url: str, ids: List[int], n: int):
    u = urlparse(url)
    c = http.client.HTTPConnection(u.hostname, u.port, timeout=600)
    t0 = time.perf_counter()
    c.request("POST", "/inference/v1/generate", json.dumps({"token_ids": ids, "stream": True, "sampling_params": {"max_tokens": n, "temperature": 0, "ignore_eos": True}}),
              {"Content-Type": "application/json"})
    r = c.getresponse()
    if r.status != 200:
        raise RuntimeError(f"engine answered {r.status}: {r.read().decode()[:200]}")
    tokens, stamps, buf = [], [], b""
    while True:
        chunk = r.read1(65536)
        if not chunk:
            break
        buf += chunk
        while b"\n\n" in buf:
            event, buf = buf.split(b"\n\n", 1)
            for line in event.split(b"\n"):
                if line.startswith(b"data: ") and line != b"data: [DONE]":
                    j = json.loads(line[6:])
                    for t in j.get("token_ids", []):
                        tokens.append(int(t))
                        stamps.append(time.perf_counter() - t0)
    c.close()
    return tokens, stamps


def compare(cases: List[Dict], url: str, repetitions: int, eos: int, noise: float) -> List[Dict]:
    if repetitions < 1 or not cases:
        raise ValueError("no cases or no repetitions")
    results = []
    for case in cases:
        want = case["output_ids"]
        if not want or not case["input_ids"]:
            raise ValueError(f"{case.get('case')}: empty reference request")
        runs = [stream_generate(url, case["input_ids"], len(want)) for _ in range(repetitions)]
        outs = [r[0] for r in runs]
        end = want.index(eos) + 1 if eos in want else len(want)
        gaps = [b - a for _, st in runs for a, b in zip(st, st[1:])]
        res = {"case": case.get("case"), "prompt_tokens": len(case["input_ids"]), "reference_output_ids": want,
               "engine_output_ids_by_repetition": outs, "exact_all_tokens": all(o == want for o in outs),
               "exact_through_reference_eos": all(o[:end] == want[:end] for o in outs),
               "stable_repetitions": all(o == outs[0] for o in outs), "repetitions": repetitions,
               "ttft_ms_mean": statistics.mean(st[0] for _, st in runs if st) * 1e3 if all(st for _, st in runs) else None,
               "tpot_ms_median": statistics.median(gaps) * 1e3 if gaps else None, "first_difference": None, "within_noise": True}
        first = next((i for i, (a, b) in enumerate(zip(outs[0], want)) if a != b), None)
        if first is None and len(outs[0]) != len(want):
            first = min(len(outs[0]), len(want))
        if first is not None:
            top = case.get("logits_top", [{}] * len(want))[first] if first < len(want) else {}
            got = outs[0][first] if first < len(outs[0]) else None
            gap = top[str(want[first])] - top[str(got)] if first < len(want) and str(got) in top else None
            res["first_difference"] = {"output_index": first, "position": len(case["input_ids"]) - 1 + first,
                                       "expected_token": want[first] if first < len(want) else None, "engine_token": got,
                                       "matching_prefix_tokens": first, "oracle_logit_gap": gap, "oracle_top": top}
            res["within_noise"] = gap is not None and gap <= noise
        results.append(res)
    return results


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="verb", required=True)
    m = sub.add_parser("make-reference")
    m.add_argument("model"); m.add_argument("checkpoint"); m.add_argument("output")
    m.add_argument("--prompts", type=int, default=4); m.add_argument("--prompt-tokens", type=int, default=12)
    m.add_argument("--new-tokens", type=int, default=8); m.add_argument("--seed", type=int, default=0)
    c = sub.add_parser("compare")
    c.add_argument("reference"); c.add_argument("url"); c.add_argument("output")
    c.add_argument("--repetitions", type=int, default=3); c.add_argument("--eos", type=int, default=-1)
    c.add_argument("--noise", type=float, default=1e-2)
    args = ap.parse_args(argv)
    if args.verb == "make-reference":
        cases = make_reference(args.model, args.checkpoint, args.prompts, args.prompt_tokens, args.new_tokens, args.seed)
        Path(args.output).write_text(json.dumps(cases, indent=1) + "\n")
        print(f"{len(cases)} cases -> {args.output}")
        return 0
    raw = Path(args.reference).read_bytes()
    results = compare(json.loads(raw), args.url, args.repetitions, args.eos, args.noise)
    report = {"format": "ifab.reference-comparison.v1", "reference_sha256": hashlib.sha256(raw).hexdigest(), "engine": args.url,
              "timing_scope": "client-side stream timestamps; concurrent load on the engine is included", "cases": results,
              "passed": all((r["exact_all_tokens"] or r["within_noise"]) and r["stable_repetitions"] for r in results)}
    Path(args.output).write_text(json.dumps(report, indent=1) + "\n")
    print(json.dumps({"passed": report["passed"], "cases": len(results), "exact": sum(r["exact_all_tokens"] for r in results)}))
    return 0 if report["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
