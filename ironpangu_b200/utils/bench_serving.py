"""Load generator for the OpenAI-compatible server: continuous-batching throughput, TTFT and TPOT over HTTP/SSE.

Starts ``ifab-server`` in the requested mode (or talks to ``--url`` of a running one), opens ``--requests`` streaming
completions with Poisson arrivals at ``--rate`` requests/s (0 = all at once, the saturation case), prompts of uniform
random token ids with lengths uniform in ``--prompt-len lo,hi`` and ``max_tokens`` uniform in ``--output-len lo,hi``,
and reports one JSON line: request and token throughput, p50/p95 time to first token, p50/p95 time per output token,
error counts and the server's own counters (``/metrics``, ``/load``). Timing is wall clock at the client, the number a
user of the HTTP API sees; engine-side device timings are the business of ``bench.py``.

    python -m ironpangu_b200.utils.bench_serving --mode mock --requests 64
    python -m ironpangu_b200.utils.bench_serving --mode worker --gpus 2 --model dense2b --requests 64 \\
        --prompt-len 128,2048 --output-len 64,512 --top-k 50 --temperature 0.7

Reference: HTTP qualification of the program engine (scripts/qualify-program-http.py) and the native TPOT benchmark
(scripts/benchmark-native-tpot.py).
"""
from __future__ import annotations

import argparse
import http.client
import json
import os
import random
import signal
import subprocess
import sys
import threading
import time
from typing import Dict, List, Optional, Tuple
from urllib.parse import urlparse

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def percentile(xs: List[float], q: float) -> Optional[float]:
    if not xs:
        return None
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


class Launched:
    """``ifab-server`` child process; the port is read from its ``listening on`` line."""

    def __init__(self, args: List[str], timeout: float = 600.0):
        from ironpangu_b200 import _build

        _build.build_core()
        env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen([str(_build.SERVER_BIN), "--port", "0", *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                     text=True, cwd=ROOT, env=env)
        self.port = None
        self.log: List[str] = []
        ready = threading.Event()

        def reader() -> None:
            for line in self.proc.stdout:
                self.log.append(line)
                if self.port is None and line.startswith("listening on"):
                    self.port = int(line.rsplit(":", 1)[1])
                    ready.set()
            ready.set()                     # the server exited

        threading.Thread(target=reader, daemon=True).start()
        ready.wait(timeout)
        if not self.port:
            self.close()
            raise RuntimeError("server did not come up:\n" + "".join(self.log[-40:]))

    def close(self) -> int:
        if self.proc.poll() is None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait()
        return self.proc.returncode


def one_request(host: str, port: int, body: Dict, timeout: float) -> Dict:
    """Stream one completion; returns send time, arrival time of every content event and the final status."""
    out = {"ok": False, "status": 0, "times": [], "tokens": 0, "error": ""}
    t_send = time.perf_counter()
    out["t_send"] = t_send
    try:
        c = http.client.HTTPConnection(host, port, timeout=timeout)
        c.request("POST", "/v1/completions", json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        out["status"] = r.status
        if r.status != 200:
            out["error"] = r.read().decode()[:200]
            c.close()
            return out
        buf = b""
        done = False
        while not done:
            chunk = r.read1(65536)
            if not chunk:
                break
            now = time.perf_counter()
            buf += chunk
            while b"\n\n" in buf:
                ev, buf = buf.split(b"\n\n", 1)
                if not ev.startswith(b"data: "):
                    continue
                payload = ev[6:]
                if payload == b"[DONE]":
                    done = True
                    break
                d = json.loads(payload)
                if "error" in d:
                    out["error"] = str(d["error"])[:200]
                    continue
                ch = d.get("choices") or [{}]
                if ch[0].get("text", "") != "" or ch[0].get("finish_reason") is None:
                    out["times"].append(now)
                usage = d.get("usage")
                if usage:
                    out["tokens"] = usage.get("completion_tokens", out["tokens"])
        c.close()
        out["ok"] = done and not out["error"]
        if not out["tokens"]:
            out["tokens"] = len(out["times"])
    except Exception as e:  # noqa: BLE001 - a failed request is a data point
        out["error"] = f"{type(e).__name__}: {e}"
    out["t_end"] = time.perf_counter()
    return out


def run_load(host: str, port: int, n: int, rate: float, prompt_len: Tuple[int, int], output_len: Tuple[int, int], vocab: int, seed: int,
             sampling: Dict, timeout: float) -> Dict:
    rng = random.Random(seed)
    plans = []
    t = 0.0
    for i in range(n):
        if rate > 0:
            t += rng.expovariate(rate)
        plans.append((t, [rng.randrange(vocab) for _ in range(rng.randint(*prompt_len))], rng.randint(*output_len)))
    results: List[Optional[Dict]] = [None] * n
    t0 = time.perf_counter()

    def worker(i: int) -> None:
        at, prompt, max_tokens = plans[i]
        delay = t0 + at - time.perf_counter()
        if delay > 0:
            time.sleep(delay)
        body = dict(model="default", prompt=prompt, max_tokens=max_tokens, stream=True, ignore_eos=True, **sampling)
        results[i] = one_request(host, port, body, timeout)
        results[i]["prompt_tokens"] = len(prompt)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(n)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if r and r["ok"]]
    ttft = [r["times"][0] - r["t_send"] for r in ok if r["times"]]
    tpot = [(r["times"][-1] - r["times"][0]) / (len(r["times"]) - 1) for r in ok if len(r["times"]) > 1]
    out_tokens = sum(r["tokens"] for r in ok)
    statuses: Dict[str, int] = {}
    for r in results:
        key = str(r["status"]) if r else "none"
        statuses[key] = statuses.get(key, 0) + 1
    return {
        "requests": n, "completed": len(ok), "statuses": statuses, "wall_s": round(wall, 4),
        "requests_per_s": round(len(ok) / wall, 3) if wall > 0 else None,
        "output_tokens": out_tokens, "output_tokens_per_s": round(out_tokens / wall, 2) if wall > 0 else None,
        "prompt_tokens": sum(r["prompt_tokens"] for r in ok),
        "ttft_ms": {"p50": _ms(percentile(ttft, 0.5)), "p95": _ms(percentile(ttft, 0.95))},
        "tpot_ms": {"p50": _ms(percentile(tpot, 0.5)), "p95": _ms(percentile(tpot, 0.95))},
        "errors": [r["error"] for r in results if r and r["error"]][:5],
    }


def _ms(v: Optional[float]) -> Optional[float]:
    return None if v is None else round(v * 1e3, 3)


def get_json(host: str, port: int, path: str) -> Optional[Dict]:
    try:
        c = http.client.HTTPConnection(host, port, timeout=10)
        c.request("GET", path)
        r = c.getresponse()
        data = r.read().decode()
        c.close()
        return json.loads(data) if r.status == 200 else None
    except Exception:  # noqa: BLE001
        return None


def server_args(a) -> List[str]:
    common = ["--max-num-seqs", str(a.max_num_seqs), "--max-num-batched-tokens", str(a.max_num_batched_tokens), "--max-model-len",
              str(a.max_model_len), "--max-queue", str(max(64, 2 * a.requests))]
    if a.mode == "mock":
        return ["--mock", "--vocab", str(a.vocab), "--step-micros", str(a.step_micros), *common]
    if a.mode == "worker":
        worker = (f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model {a.model} --max-num-seqs {a.max_num_seqs} "
                  f"--max-model-len {a.max_model_len} --max-num-batched-tokens {a.max_num_batched_tokens}")
        if a.layers:
            worker += f" --layers {a.layers}"
        if a.prefill_chunk:
            worker += f" --prefill-chunk {a.prefill_chunk}"
        if a.gpu_memory_utilization != 0.9:
            worker += f" --gpu-memory-utilization {a.gpu_memory_utilization}"
        if a.kv_int8:
            worker += " --kv-int8"
        if a.expert_fp8:
            worker += " --expert-fp8"
        if a.prefix_cache_slots:
            worker += f" --prefix-cache-slots {a.prefix_cache_slots}"
        if a.gpus > 1:
            worker = (f"{sys.executable} -m torch.distributed.run --nnodes=1 --nproc-per-node {a.gpus} --master-addr 127.0.0.1 "
                      f"--master-port {a.master_port} -m ironpangu_b200.runtime.engine_worker" + worker.split("engine_worker", 1)[1])
        return ["--spawn", worker, "--accept-seconds", "900", *common]
    if a.mode == "program":
        return ["--program", a.bundle, a.checkpoint, *(["--cpu"] if a.cpu else ["--gpus", str(a.gpus)]), *common]
    raise SystemExit(f"unknown mode {a.mode}")


def main(argv: Optional[List[str]] = None) -> Dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--url", default="", help="talk to a running server instead of launching one")
    ap.add_argument("--mode", default="mock", choices=["mock", "worker", "program"])
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--bundle", default="")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--master-port", type=int, default=29611)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--kv-int8", action="store_true")
    ap.add_argument("--expert-fp8", action="store_true")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="rows per tensor-core prefill call of the worker (0 = decode kernels)")
    ap.add_argument("--prefix-cache-slots", type=int, default=0)
    ap.add_argument("--max-num-seqs", type=int, default=8)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--step-micros", type=int, default=200)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=0.0, help="Poisson arrival rate in requests/s; 0 = all at once")
    ap.add_argument("--prompt-len", default="16,64")
    ap.add_argument("--output-len", default="8,32")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args(argv)
    lo_hi = lambda s: tuple(int(v) for v in s.split(","))  # noqa: E731
    sampling: Dict = {"temperature": a.temperature}
    if a.top_k:
        sampling["top_k"] = a.top_k
    if a.top_p < 1.0:
        sampling["top_p"] = a.top_p
    server = None
    if a.url:
        u = urlparse(a.url)
        host, port = u.hostname or "127.0.0.1", u.port or 80
    else:
        server = Launched(server_args(a), timeout=a.timeout)
        host, port = "127.0.0.1", server.port
    try:
        models = get_json(host, port, "/v1/models") or {}
        vocab = a.vocab
        load0 = get_json(host, port, "/load") or {}
        vocab = int(load0.get("vocab", vocab)) if isinstance(load0, dict) else vocab
        res = run_load(host, port, a.requests, a.rate, lo_hi(a.prompt_len), lo_hi(a.output_len), vocab, a.seed, sampling, a.timeout)
        res["server"] = {"mode": a.mode if not a.url else "url", "gpus": a.gpus, "max_num_seqs": a.max_num_seqs,
                         "models": [m.get("id") for m in models.get("data", [])], "load": get_json(host, port, "/load")}
        res["workload"] = {"rate": a.rate, "prompt_len": a.prompt_len, "output_len": a.output_len, "sampling": sampling, "seed": a.seed}
    finally:
        rc = server.close() if server else 0
    res["server_exit"] = rc
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
