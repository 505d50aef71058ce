"""Serving qualification: drives ``ifab-server`` over HTTP through the scenarios a deployment has to survive and writes a JSON
report (exit code 0 only when every scenario passes).

    python -m ironpangu_b200.utils.qualify_serving --engine standin                 # CPU: the server with a stand-in engine process
    python -m ironpangu_b200.utils.qualify_serving --engine worker --model tiny     # GPU: the real engine worker behind the server
    python -m ironpangu_b200.utils.qualify_serving --engine worker --model dense2b --gpus 2 --report out.json

Scenarios (each reports ``passed`` and what it measured):

* ``repeatability``     the same greedy request twice gives the same tokens; a request alone equals the same request among peers
* ``cancellation``      a streamed request is abandoned in the middle while peers run: the peers finish, the cancellation is counted,
                        the slot is reused
* ``prefix_cache``      cold prompt (misses) -> same prompt again (hits, same tokens) -> same prompt under another ``cache_salt``
                        (misses: tenants share nothing) -> a prompt that shares only the first blocks
                        (partial reuse) -> enough distinct prompts to evict the first -> the first again (misses again: LRU)
* ``overload``          a burst larger than the admission queue: the excess is refused with 429 and a JSON error, nothing hangs,
                        and a request after the burst succeeds (recovery)
* ``load_waves``        repeated waves of concurrent requests; resident memory, open descriptors and threads of the server (and of its
                        engine process) after the last wave stay within a bound of what they were after the first
* ``engine_failure``    the engine process dies between steps (host-side: it exits): running requests end with an error, /health
                        turns 503, new requests get 503 (fail closed, nothing hangs); a restarted server serves again

The stand-in engine is a CPU process that speaks the engine-worker socket protocol (info / admit / step / release / audit /
shutdown) with deterministic tokens (a hash of the sequence so far), block-keyed prefix snapshots with LRU eviction and an optional
"exit after N steps". It exists so that every scenario, the failure one included, runs without a GPU.
Reference scenarios: scripts/qualify-program-http.py:184-202, scripts/qualify-program-engine.py:89-102.
"""
from __future__ import annotations

import argparse
import hashlib
import http.client
import json
import math
import os
import signal
import socket
import subprocess
import sys
import threading
import time
from collections import OrderedDict
from pathlib import Path
from typing import Dict, List, Optional

ROOT = Path(__file__).resolve().parents[2]


# ---------------------------------------------------------------------------------------------------------------------------
# stand-in engine (CPU): `python -m ironpangu_b200.utils.qualify_serving --serve-standin SOCKET ...`
# ---------------------------------------------------------------------------------------------------------------------------
class StandInEngine:
    BLOCK = 16

    def __init__(self, residents: int, context: int, vocab: int, budget: int, prefix_slots: int, step_ms: float):
        self.residents, self.context, self.vocab, self.budget = residents, context, vocab, budget
        self.history: List[List[int]] = [[] for _ in range(residents)]
        self.prompt_done = [False] * residents
        self.salt = [""] * residents
        self.prefix: "OrderedDict[tuple, int]" = OrderedDict()
        self.prefix_slots = prefix_slots
        self.counters = {"steps": 0, "rows": 0, "prefix_hits": 0, "prefix_misses": 0, "prefix_published": 0, "prefix_evicted": 0}
        self.step_ms = step_ms

    def info(self) -> Dict:
        return {"model": "standin", "residents": self.residents, "token_budget": self.budget, "chunk": self.budget, "context": self.context,
                "vocab": self.vocab, "eos": 0, "has_eos": False, "world": 1, "greedy_only": True}

    def admit(self, resident: int, reserve: int, salt: str = "") -> None:
        if not 0 <= resident < self.residents:
            raise ValueError("resident out of range")
        if reserve > self.context:
            raise OverflowError("request does not fit the sequence slot")
        self.history[resident] = []
        self.prompt_done[resident] = False
        self.salt[resident] = salt

    def _token(self, hist: List[int]) -> int:
        h = hashlib.blake2b(repr(hist).encode(), digest_size=8).digest()
        return 1 + int.from_bytes(h, "little") % (self.vocab - 1)

    def step(self, slices, tokens) -> List[int]:
        """One token per slice (0 where the slice does not sample). Prefix traffic follows the engine worker: a whole
        non-sampling prompt chunk that a stored prompt covers is a hit, else a miss; a prompt is published (its whole blocks)
        when its first sampling slice ends it."""
        if self.step_ms > 0:
            time.sleep(self.step_ms / 1e3)
        out, off = [0] * len(slices), 0
        self.counters["steps"] += 1
        for i, (resident, position, count, sample) in enumerate(slices):
            hist = self.history[resident]
            if position != len(hist):
                raise RuntimeError(f"slice of resident {resident} starts at {position}, expected {len(hist)}")
            hist.extend(tokens[off:off + count])
            off += count
            self.counters["rows"] += count
            if self.prefix_slots and not sample:
                want, salt = tuple(hist), self.salt[resident]
                hit = next((k for k in reversed(self.prefix) if k[0] == salt and len(k[1]) >= len(want) and k[1][:len(want)] == want), None)
                if hit is not None:
                    self.prefix.move_to_end(hit)
                    self.counters["prefix_hits"] += 1
                else:
                    self.counters["prefix_misses"] += 1
            if sample:
                out[i] = self._token(hist)
                if self.prefix_slots and not self.prompt_done[resident]:
                    self.prompt_done[resident] = True
                    step = self.BLOCK // math.gcd(self.BLOCK, self.budget) * self.budget
                    n = (len(hist) - 1) // step * step       # whole blocks and whole prompt slices, one prompt token left over
                    key = (self.salt[resident], tuple(hist[:n]))
                    if n and key in self.prefix:
                        self.prefix.move_to_end(key)
                    elif n:
                        self.prefix[key] = n
                        self.counters["prefix_published"] += 1
                        while len(self.prefix) > self.prefix_slots:
                            self.prefix.popitem(last=False)
                            self.counters["prefix_evicted"] += 1
        return out

    def audit(self) -> Dict:
        return {"format": "ifab.engine-audit.v1", **self.counters, "prefix_entries": len(self.prefix), "fabric_status": 0}


def serve_standin(sock_path: str, args) -> None:
    eng = StandInEngine(args.max_num_seqs, args.max_model_len, args.vocab, args.max_num_batched_tokens, args.prefix_cache_slots, args.step_ms)
    conn = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    conn.connect(sock_path)
    buf, steps = b"", 0
    while True:
        while b"\n" not in buf:
            chunk = conn.recv(1 << 16)
            if not chunk:
                return
            buf += chunk
        line, buf = buf.split(b"\n", 1)
        req = json.loads(line)
        op = req.get("op")
        try:
            if op == "info":
                resp = {"ok": True, "info": eng.info()}
            elif op == "admit":
                eng.admit(int(req["resident"]), int(req.get("reserve", 0)), str(req.get("sampling", {}).get("cache_salt", "")))
                resp = {"ok": True}
            elif op == "step":
                steps += 1
                if args.die_after_steps and steps > args.die_after_steps:
                    os._exit(17)             # the induced failure: the engine process is gone between two steps
                resp = {"ok": True, "tokens": eng.step(req["slices"], req["tokens"])}
            elif op == "release":
                resp = {"ok": True}
            elif op == "audit":
                resp = {"ok": True, "audit": eng.audit()}
            elif op == "shutdown":
                conn.sendall(b'{"ok": true}\n')
                return
            else:
                resp = {"ok": False, "kind": "invalid", "error": f"unknown op {op!r}"}
        except OverflowError as e:
            resp = {"ok": False, "kind": "capacity", "error": str(e)}
        except ValueError as e:
            resp = {"ok": False, "kind": "invalid", "error": str(e)}
        except Exception as e:  # noqa: BLE001
            resp = {"ok": False, "kind": "backend", "error": f"{type(e).__name__}: {e}"}
        conn.sendall(json.dumps(resp).encode() + b"\n")


# ---------------------------------------------------------------------------------------------------------------------------
# the server under test
# ---------------------------------------------------------------------------------------------------------------------------
class ServerUnderTest:
    def __init__(self, args, extra_engine_flags: str = "", max_queue: Optional[int] = None):
        from ironpangu_b200 import _build

        _build.build_core()
        common = f"--max-num-seqs {args.max_num_seqs} --max-model-len {args.max_model_len}"
        if args.engine == "standin":
            spawn = (f"{sys.executable} -m ironpangu_b200.utils.qualify_serving --serve-standin \"$IFAB_ENGINE_SOCKET\" {common} --vocab {args.vocab} "
                     f"--max-num-batched-tokens {args.max_num_batched_tokens} --prefix-cache-slots {args.prefix_cache_slots} "
                     f"--step-ms {args.step_ms} {extra_engine_flags}")
        else:
            worker = (f"-m ironpangu_b200.runtime.engine_worker --model {args.model} {common} --prefix-cache-slots {args.prefix_cache_slots} "
                      f"--greedy-only {args.worker_flags}")
            spawn = (f"{sys.executable} -m torch.distributed.run --nnodes=1 --nproc-per-node {args.gpus} --master-addr 127.0.0.1 "
                     f"--master-port 29588 {worker}" if args.gpus > 1 else f"{sys.executable} {worker}")
        cmd = [str(_build.SERVER_BIN), "--port", "0", "--spawn", spawn, "--accept-seconds", "600"]
        if max_queue is not None:
            cmd += ["--max-queue", str(max_queue)]
        env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(ROOT), env=env)
        self.port = None
        self.lines: List[str] = []
        t0 = time.time()
        while time.time() - t0 < 900:
            line = self.proc.stdout.readline()
            if not line:
                break
            self.lines.append(line)
            if line.startswith("listening on"):
                self.port = int(line.rsplit(":", 1)[1])
                break
        if not self.port:
            raise RuntimeError("server did not come up:\n" + "".join(self.lines[-20:]))
        threading.Thread(target=self._drain, daemon=True).start()

    def _drain(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line)

    def request(self, method: str, path: str, body=None, timeout: float = 120):
        c = http.client.HTTPConnection("127.0.0.1", self.port, timeout=timeout)
        c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        data = r.read().decode()
        c.close()
        return r.status, data

    def generate(self, ids: List[int], n: int, timeout: float = 300, salt: str = ""):
        sp = {"max_tokens": n, "temperature": 0}
        if salt:
            sp["cache_salt"] = salt
        st, data = self.request("POST", "/inference/v1/generate", {"token_ids": ids, "sampling_params": sp}, timeout)
        try:
            return st, json.loads(data)
        except ValueError:
            return st, {"raw": data}

    def audit(self) -> Dict:
        st, data = self.request("GET", "/audit")
        return json.loads(data) if st == 200 else {}

    def metrics(self) -> Dict[str, float]:
        out = {}
        for l in self.request("GET", "/metrics")[1].splitlines():
            if l and not l.startswith("#"):
                k, v = l.rsplit(" ", 1)
                out[k] = float(v)
        return out

    def family(self) -> List[int]:
        """pids of the server and of everything below it (the engine processes)"""
        pids, frontier = [self.proc.pid], [self.proc.pid]
        while frontier:
            p = frontier.pop()
            try:
                for t in os.listdir(f"/proc/{p}/task"):
                    kids = Path(f"/proc/{p}/task/{t}/children").read_text().split()
                    for k in map(int, kids):
                        if k not in pids:
                            pids.append(k)
                            frontier.append(k)
            except OSError:
                pass
        return pids

    def resources(self) -> Dict[str, int]:
        rss = fds = threads = 0
        for p in self.family():
            try:
                for l in Path(f"/proc/{p}/status").read_text().splitlines():
                    if l.startswith("VmRSS:"):
                        rss += int(l.split()[1]) * 1024
                    elif l.startswith("Threads:"):
                        threads += int(l.split()[1])
                fds += len(os.listdir(f"/proc/{p}/fd"))
            except OSError:
                pass
        return {"rss_bytes": rss, "open_fds": fds, "threads": threads}

    def close(self) -> int:
        if self.proc.poll() is None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait()
        return self.proc.returncode


def parallel(calls):
    out = [None] * len(calls)

    def run(i, f):
        try:
            out[i] = f()
        except Exception as e:  # noqa: BLE001
            out[i] = ("exception", repr(e))

    ts = [threading.Thread(target=run, args=(i, f)) for i, f in enumerate(calls)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return out


# ---------------------------------------------------------------------------------------------------------------------------
# scenarios
# ---------------------------------------------------------------------------------------------------------------------------
def prompt(seed: int, n: int, vocab: int) -> List[int]:
    return [1 + (seed * 7919 + i * 104729) % (vocab - 1) for i in range(n)]


def scenario_repeatability(s: ServerUnderTest, args) -> Dict:
    p = prompt(1, 24, args.vocab)
    a = s.generate(p, 12)
    b = s.generate(p, 12)
    peers = parallel([lambda i=i: s.generate(prompt(10 + i, 8 + i, args.vocab), 10) for i in range(args.max_num_seqs)] + [lambda: s.generate(p, 12)])
    ok = a[0] == 200 and a[1].get("token_ids") == b[1].get("token_ids") == peers[-1][1].get("token_ids") and len(a[1]["token_ids"]) == 12
    return {"passed": bool(ok), "tokens": a[1].get("token_ids"), "peer_statuses": [x[0] for x in peers]}


def scenario_cancellation(s: ServerUnderTest, args) -> Dict:
    before = s.metrics().get("ifab_requests_cancelled_total", 0)
    c = http.client.HTTPConnection("127.0.0.1", s.port, timeout=30)
    c.request("POST", "/inference/v1/generate", json.dumps({"token_ids": prompt(3, 6, args.vocab), "stream": True,
                                                            "sampling_params": {"max_tokens": min(200, args.max_model_len - 16), "temperature": 0}}))
    r = c.getresponse()
    r.read(16)
    peers = [threading.Thread(target=lambda i=i: results.__setitem__(i, s.generate(prompt(30 + i, 5, args.vocab), 16))) for i in range(max(1, args.max_num_seqs - 1))]
    results: Dict[int, tuple] = {}
    [t.start() for t in peers]
    c.close()                                    # walk away in the middle of the stream
    [t.join() for t in peers]
    cancelled = before
    for _ in range(200):
        cancelled = s.metrics().get("ifab_requests_cancelled_total", 0)
        if cancelled > before:
            break
        time.sleep(0.05)
    after = s.generate(prompt(4, 5, args.vocab), 4)
    ok = cancelled > before and all(v[0] == 200 and len(v[1]["token_ids"]) == 16 for v in results.values()) and after[0] == 200
    return {"passed": bool(ok), "cancelled_total": cancelled, "peers_ok": len(results)}


def scenario_prefix_cache(s: ServerUnderTest, args) -> Dict:
    if not args.prefix_cache_slots:
        return {"passed": True, "skipped": "prefix cache off (--prefix-cache-slots 0)"}
    n = min(96, args.max_model_len - 16)
    base = prompt(5, n, args.vocab)

    def hits():
        a = s.audit().get("engine", s.audit())
        return a.get("prefix_hits", 0), a.get("prefix_misses", 0), a.get("prefix_evicted", 0)

    h0 = hits()
    cold = s.generate(base, 6)
    h1 = hits()
    warm = s.generate(base, 6)
    h2 = hits()
    salted = s.generate(base, 6, salt="tenant-b")          # the same prompt under another salt shares nothing
    hs = hits()
    branch = s.generate(base[:n // 2] + prompt(6, n - n // 2, args.vocab), 6)
    h3 = hits()
    for i in range(args.prefix_cache_slots + 2):        # distinct prompts until the first one's snapshots are evicted
        s.generate(prompt(100 + i, n, args.vocab), 2)
    h4 = hits()
    again = s.generate(base, 6)
    h5 = hits()
    ok = (cold[0] == warm[0] == branch[0] == again[0] == 200 and cold[1]["token_ids"] == warm[1]["token_ids"] == again[1]["token_ids"]
          and h1[0] == h0[0] and h1[1] > h0[1]            # cold: only misses
          and h2[0] > h1[0]                              # warm: hits
          and salted[0] == 200 and salted[1]["token_ids"] == cold[1]["token_ids"] and hs[0] == h2[0] and hs[1] > h2[1]   # salt isolation
          and h3[0] > hs[0] and h3[1] > hs[1]            # shared first half hits, the new second half misses
          and h4[2] > h3[2]                              # the flood evicted something
          and h5[1] > h4[1])                             # the first prompt misses again: least recently used went first
    return {"passed": bool(ok), "counters_hits_misses_evicted": [h0, h1, h2, h3, h4, h5], "after_salted_request": hs}


def scenario_overload(args) -> Dict:
    q = 4
    s = ServerUnderTest(args, max_queue=q)
    try:
        n = q + args.max_num_seqs + 8
        res = parallel([lambda i=i: s.generate(prompt(200 + i, 6, args.vocab), 24) for i in range(n)])
        statuses = [r[0] for r in res]
        refused = [r for r in res if r[0] == 429]
        shaped = all(isinstance(r[1], dict) and r[1].get("error", {}).get("type") == "overloaded" for r in refused)
        after = s.generate(prompt(7, 6, args.vocab), 4)
        ok = statuses.count(200) >= args.max_num_seqs and len(refused) >= 1 and shaped and set(statuses) <= {200, 429} and after[0] == 200
        return {"passed": bool(ok), "burst": n, "statuses": {str(k): statuses.count(k) for k in set(statuses)}, "after_burst": after[0]}
    finally:
        s.close()


def scenario_load_waves(s: ServerUnderTest, args) -> Dict:
    samples = []
    for w in range(args.waves):
        res = parallel([lambda i=i: s.generate(prompt(300 + w * 50 + i, 4 + i % 9, args.vocab), 6 + i % 5) for i in range(args.wave_requests)])
        if any(r[0] != 200 for r in res):
            return {"passed": False, "wave": w, "statuses": [r[0] for r in res]}
        time.sleep(0.2)
        samples.append(s.resources())
    first, last = samples[min(1, len(samples) - 1)], samples[-1]
    ok = (last["rss_bytes"] <= first["rss_bytes"] * 1.25 + (64 << 20) and last["open_fds"] <= first["open_fds"] + 8 and
          last["threads"] <= first["threads"] + 8)
    return {"passed": bool(ok), "waves": args.waves, "requests_per_wave": args.wave_requests, "after_warm_up_wave": first, "after_last_wave": last}


def scenario_engine_failure(args) -> Dict:
    if args.engine != "standin":
        # the real worker is taken down the same way a crash would: its process group gets SIGKILL between two requests
        s = ServerUnderTest(args)
        try:
            ok0 = s.generate(prompt(8, 6, args.vocab), 4)[0] == 200
            for p in s.family()[1:]:
                try:
                    os.kill(p, signal.SIGKILL)
                except OSError:
                    pass
            return _after_failure(s, args, ok0)
        finally:
            s.close()
    s = ServerUnderTest(args, extra_engine_flags="--die-after-steps 12")
    try:
        ok0 = s.generate(prompt(8, 6, args.vocab), 4)[0] == 200          # a few steps: fine
        return _after_failure(s, args, ok0, trigger=lambda: s.generate(prompt(9, 6, args.vocab), 40, timeout=60))
    finally:
        s.close()


def _after_failure(s: ServerUnderTest, args, ok0: bool, trigger=None) -> Dict:
    t0 = time.time()
    broke = trigger() if trigger else None
    health = 200
    for _ in range(200):
        health = s.request("GET", "/health", timeout=10)[0]
        if health == 503:
            break
        time.sleep(0.05)
    refused = s.generate(prompt(10, 4, args.vocab), 4, timeout=30)
    took = time.time() - t0
    rc = s.close()
    fresh = ServerUnderTest(args)
    try:
        again = fresh.generate(prompt(8, 6, args.vocab), 4)
    finally:
        fresh.close()
    ok = ok0 and health == 503 and refused[0] == 503 and took < 60 and again[0] == 200 and (broke is None or broke[0] != 200 or len(broke[1].get("token_ids", [])) < 40)
    return {"passed": bool(ok), "health_after": health, "request_after": refused[0], "seconds_to_fail_closed": round(took, 2), "server_exit": rc,
            "restarted_serves": again[0]}


def main(argv=None) -> Dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("--engine", default="standin", choices=["standin", "worker"])
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--worker-flags", default="", help="extra flags for the engine worker")
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--max-model-len", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--prefix-cache-slots", type=int, default=6)
    ap.add_argument("--step-ms", type=float, default=0.5, help="stand-in engine: time per step")
    ap.add_argument("--waves", type=int, default=5)
    ap.add_argument("--wave-requests", type=int, default=16)
    ap.add_argument("--only", default="", help="comma-separated scenario names")
    ap.add_argument("--report", default="")
    ap.add_argument("--serve-standin", default="", help=argparse.SUPPRESS)
    ap.add_argument("--die-after-steps", type=int, default=0, help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.serve_standin:
        serve_standin(args.serve_standin, args)
        return {}
    only = set(filter(None, args.only.split(",")))
    want = lambda name: not only or name in only
    report: Dict[str, Dict] = {}
    shared = [n for n in ("repeatability", "cancellation", "prefix_cache", "load_waves") if want(n)]
    if shared:
        s = ServerUnderTest(args)
        try:
            for name in shared:
                t0 = time.time()
                try:
                    report[name] = globals()["scenario_" + name](s, args)
                except Exception as e:  # noqa: BLE001
                    report[name] = {"passed": False, "exception": repr(e), "server_tail": s.lines[-5:]}
                report[name]["seconds"] = round(time.time() - t0, 2)
            report["shutdown"] = {"passed": s.close() == 0}
        finally:
            s.close()
    for name in ("overload", "engine_failure"):
        if want(name):
            t0 = time.time()
            try:
                report[name] = globals()["scenario_" + name](args)
            except Exception as e:  # noqa: BLE001
                report[name] = {"passed": False, "exception": repr(e)}
            report[name]["seconds"] = round(time.time() - t0, 2)
    out = {"format": "ifab.serving-qualification.v1", "engine": args.engine, "model": args.model if args.engine == "worker" else "standin",
           "passed": all(v.get("passed") for v in report.values()), "scenarios": report}
    text = json.dumps(out, indent=1)
    if args.report:
        Path(args.report).write_text(text)
    print(text)
    return out


if __name__ == "__main__":
    sys.exit(0 if main().get("passed", True) else 1)
