"""ifab-server over real HTTP: the mock engine on CPU, the engine worker (tiny MLA + MoE model) on a GPU."""
import http.client
import json
import os
import signal
import subprocess
import sys
import threading
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Server:
    def __init__(self, *args, timeout=120):
        from ironpangu_b200 import _build

        _build.build_core()
        env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen([str(_build.SERVER_BIN), "--port", "0", *args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                     text=True, cwd=ROOT, env=env)
        self.lines = []
        self.port = None
        t0 = time.time()
        while time.time() - t0 < timeout:
            line = self.proc.stdout.readline()
            if not line:
                break
            self.lines.append(line)
            if line.startswith("listening on"):
                self.port = int(line.rsplit(":", 1)[1])
                break
        assert self.port, "server did not come up:\n" + "".join(self.lines)

    def request(self, method, path, body=None, timeout=60):
        c = http.client.HTTPConnection("127.0.0.1", self.port, timeout=timeout)
        c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        data = r.read().decode()
        c.close()
        return r.status, data

    def post(self, path, body, **kw):
        status, data = self.request("POST", path, body, **kw)
        return status, json.loads(data)

    def sse(self, path, body, timeout=60):
        c = http.client.HTTPConnection("127.0.0.1", self.port, timeout=timeout)
        c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        assert r.status == 200 and r.getheader("Content-Type").startswith("text/event-stream")
        events = [l[6:] for l in r.read().decode().split("\n") if l.startswith("data: ")]
        c.close()
        assert events[-1] == "[DONE]"
        return [json.loads(e) for e in events[:-1]]

    def close(self):
        if self.proc.poll() is None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                self.proc.kill()


@pytest.fixture
def mock_server():
    s = Server("--mock", "--max-num-seqs", "3", "--max-num-batched-tokens", "6", "--vocab", "300", "--max-model-len", "96", "--step-micros", "300")
    yield s
    s.close()
    assert s.proc.returncode == 0


def test_routes_and_openai_shapes(mock_server):
    s = mock_server
    assert s.request("GET", "/health")[0] == 200
    assert s.request("GET", "/nope")[0] == 404
    assert s.request("GET", "/v1/completions")[0] == 405
    st, models = s.request("GET", "/v1/models")
    assert json.loads(models)["data"][0]["max_model_len"] == 96
    st, tk = s.post("/tokenize", {"prompt": "hé"})
    assert tk["tokens"] == [3 + 0x68, 3 + 0xC3, 3 + 0xA9] and tk["count"] == 3
    st, dt = s.post("/detokenize", {"tokens": tk["tokens"]})
    assert dt["prompt"] == "hé"
    st, c = s.post("/v1/completions", {"prompt": "hello", "max_tokens": 5})
    assert st == 200 and c["object"] == "text_completion" and c["choices"][0]["finish_reason"] == "length"
    assert c["usage"] == {"prompt_tokens": 5, "completion_tokens": 5, "total_tokens": 10}
    # token-in / token-out, streamed and not, agree; generation is deterministic
    st, g = s.post("/inference/v1/generate", {"token_ids": [5, 6, 7], "sampling_params": {"max_tokens": 6}})
    ev = s.sse("/inference/v1/generate", {"token_ids": [5, 6, 7], "sampling_params": {"max_tokens": 6}, "stream": True})
    assert [t for e in ev for t in e["token_ids"]] == g["token_ids"] and ev[-1]["finish_reason"] == "length" and len(g["token_ids"]) == 6
    # the same prompt as text ids through /v1/completions yields the same continuation (stop token honoured)
    st, c2 = s.post("/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 6, "stop_token_ids": [g["token_ids"][2]]})
    assert c2["choices"][0]["finish_reason"] == "stop" and c2["usage"]["completion_tokens"] == 3
    ch = s.sse("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True})
    assert ch[0]["choices"][0]["delta"]["role"] == "assistant" and ch[-1]["choices"][0]["finish_reason"] == "length"
    assert all(e["object"] == "chat.completion.chunk" for e in ch)


def test_audit_route_reports_engine_and_service_counters(mock_server):
    st, _ = mock_server.post("/v1/completions", {"prompt": "abc", "max_tokens": 4})
    assert st == 200
    st, body = mock_server.request("GET", "/audit")
    a = json.loads(body)
    assert st == 200 and a["service"]["requests_finished"] == 1 and a["engine"]["steps"] >= 4 and a["engine"]["rows"] >= 6


def test_chat_route_accepts_tools_and_returns_a_parsed_message():
    mock_server = Server("--mock", "--max-num-seqs", "2", "--max-num-batched-tokens", "64", "--vocab", "300", "--max-model-len", "2048")
    try:
        _chat_tools_checks(mock_server)
    finally:
        mock_server.close()


def _chat_tools_checks(mock_server):
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    st, r = mock_server.post("/v1/chat/completions", {"messages": [{"role": "user", "content": "weather?"}], "tools": tools, "max_tokens": 6})
    assert st == 200
    msg = r["choices"][0]["message"]
    assert msg["role"] == "assistant" and "content" in msg and r["usage"]["prompt_tokens"] > 200     # the tool block is part of the prompt
    st, r = mock_server.post("/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "tools": [{"type": "retrieval"}]})
    assert st == 400 and "function" in r["error"]["message"]


def test_errors_are_openai_errors(mock_server):
    s = mock_server
    for body, needle in [({"prompt": "x", "max_tokens": 5000}, "exceeds the context"), ({"prompt": "x", "n": 2}, "'n'"),
                         ({"prompt": "x", "temperature": 1000}, "temperature"), ({"prompt": [1, 99999]}, "vocabulary"),
                         ({"prompt": "x", "logprobs": 3}, "logprobs"), ({"max_tokens": 3}, "prompt")]:
        st, e = s.post("/v1/completions", body)
        assert st == 400 and e["error"]["type"] == "invalid_request_error" and needle in e["error"]["message"], (body, e)
    st, raw = s.request("POST", "/v1/completions", None)
    assert st == 400
    # request fields the engine does not implement are refused (501), not silently dropped
    for path, body in [("/v1/completions", {"prompt": "x", "logit_bias": {"5": 1.0}}),
                       ("/inference/v1/generate", {"token_ids": [5], "sampling_params": {"allowed_token_ids": [1, 2]}})]:
        st, e = s.post(path, body)
        assert st == 501 and e["error"]["type"] == "unsupported", (body, e)


def test_continuous_batching_many_clients_and_metrics(mock_server):
    s = mock_server
    results, errors = {}, []

    def client(i):
        try:
            st, g = s.post("/inference/v1/generate", {"token_ids": [10 + i, 20 + i, 30 + i][: 1 + i % 3], "sampling_params": {"max_tokens": 8 + i % 5}})
            results[i] = (st, g)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=client, args=(i,)) for i in range(12)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors and len(results) == 12
    for i, (st, g) in results.items():
        assert st == 200 and len(g["token_ids"]) == 8 + i % 5
    # a sequence generated alone equals the one generated among eleven others
    st, alone = s.post("/inference/v1/generate", {"token_ids": [10, 20, 30][:1], "sampling_params": {"max_tokens": 8}})
    assert alone["token_ids"] == results[0][1]["token_ids"]
    metrics = dict(l.split(" ") for l in s.request("GET", "/metrics")[1].splitlines() if l and not l.startswith("#"))
    assert float(metrics["ifab_requests_finished_total"]) == 13
    assert float(metrics["ifab_engine_rows_total"]) > float(metrics["ifab_engine_steps_total"])   # rows shared steps
    assert float(metrics["ifab_healthy"]) == 1
    # latency histograms: one first-token observation per finished request, one inter-token observation per later token
    assert float(metrics["ifab_time_to_first_token_seconds_count"]) == 13
    assert float(metrics["ifab_inter_token_latency_seconds_count"]) == float(metrics["ifab_generation_tokens_total"]) - 13
    assert float(metrics['ifab_time_to_first_token_seconds_bucket{le="+Inf"}']) == 13
    assert float(metrics["ifab_time_to_first_token_seconds_sum"]) > 0


def test_disconnect_cancels_and_server_keeps_serving(mock_server):
    s = mock_server
    c = http.client.HTTPConnection("127.0.0.1", s.port, timeout=10)
    c.request("POST", "/inference/v1/generate", json.dumps({"token_ids": [1, 2], "sampling_params": {"max_tokens": 90}, "stream": True}))
    r = c.getresponse()
    r.read(20)
    c.close()      # walk away in the middle of the stream
    for _ in range(100):
        metrics = dict(l.split(" ") for l in s.request("GET", "/metrics")[1].splitlines() if l and not l.startswith("#"))
        if float(metrics["ifab_requests_cancelled_total"]) >= 1:
            break
        time.sleep(0.05)
    assert float(metrics["ifab_requests_cancelled_total"]) >= 1
    st, g = s.post("/inference/v1/generate", {"token_ids": [3], "sampling_params": {"max_tokens": 3}})
    assert st == 200 and len(g["token_ids"]) == 3


@pytest.mark.gpu
def test_gpu_engine_worker_serves_the_tiny_model():
    """Server -> Unix socket -> engine worker -> CUDA decode kernels, three sequences batched; tokens equal the
    single-sequence engine on the same weights."""
    import torch

    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.engine import DecodeEngine

    s = Server("--spawn", f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 3 --max-model-len 128 --greedy-only",
               "--accept-seconds", "300", timeout=400)
    try:
        prompts = [[5, 77, 300, 12, 999, 41, 8, 650, 3, 17, 256], [9], [100, 200, 300]]
        out = {}

        def client(i):
            out[i] = s.post("/inference/v1/generate", {"token_ids": prompts[i], "sampling_params": {"max_tokens": 6}}, timeout=120)

        threads = [threading.Thread(target=client, args=(i,)) for i in range(3)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        cfg = MlaMoeConfig.tiny(2)
        fab = Fabric(0, 1)
        dec = MlaMoeDecoder(cfg, random_rank_weights(cfg, 0, 1, torch.device("cuda", 0), seed=0), fab, max_tokens=8, max_context=128)
        for i, p in enumerate(prompts):
            st, g = out[i]
            assert st == 200, g
            dec.reset()
            assert g["token_ids"] == DecodeEngine(dec).generate(p, 6)
        st, e = s.post("/v1/completions", {"prompt": "x", "temperature": 0.7})
        assert st == 400 and "greedy" in e["error"]["message"]
        fab.close()
    finally:
        s.close()


@pytest.mark.gpu
def test_gpu_engine_worker_serves_the_hyper_connected_family():
    """The worker compiles the generated hyper-connected source (residual streams, sink rows, token convolution, routed experts),
    draws its parameters from the init plan and serves it through the plan engine: three sequences batched into one step
    generate the tokens each of them generates alone (sequence slots reused: the convolution history and the caches of a
    slot's previous sequence are never read)."""
    s = Server("--spawn", f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model hyper-tiny --layers 3 --max-num-seqs 3 "
               "--max-model-len 128 --greedy-only", "--accept-seconds", "300", timeout=400)
    try:
        prompts = [[5, 77, 300, 12, 99, 41, 8, 65, 3, 17, 256], [9], [100, 200, 300]]
        out = {}

        def client(i):
            out[i] = s.post("/inference/v1/generate", {"token_ids": prompts[i], "sampling_params": {"max_tokens": 6}}, timeout=120)

        threads = [threading.Thread(target=client, args=(i,)) for i in range(3)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        for i in range(3):
            st, g = out[i]
            assert st == 200, g
            assert len(g["token_ids"]) == 6 and all(0 <= t < 512 for t in g["token_ids"])
        for i in (2, 0, 1):                          # other slots than the first time
            st, g = s.post("/inference/v1/generate", {"token_ids": prompts[i], "sampling_params": {"max_tokens": 6}}, timeout=120)
            assert st == 200, g
            assert g["token_ids"] == out[i][1]["token_ids"]
    finally:
        s.close()


def test_program_engine_abi_and_cpu_server(tmp_path):
    """A compiled bundle + synthetic checkpoint served on the host: the program-engine C ABI and `--program ... --cpu` agree
    with the interpreter, token for token."""
    import ctypes as C

    from ironpangu_b200 import _build, compiler

    src = os.path.join(ROOT, "examples", "mla_moe_slice_tp1.inferfabric")
    ckpt, bundle = tmp_path / "ckpt", tmp_path / "bundle"
    r = compiler.cli("synth-checkpoint", src, str(ckpt))
    assert r.returncode == 0, r.stderr
    r = compiler.cli("compile-token", src, str(ckpt), str(bundle), "--resident-sequences", "2", "--prefill-tokens", "8")
    assert r.returncode == 0, r.stderr
    prompt = [5, 77, 300, 12, 9]
    want = compiler.interpret(open(src).read(), str(ckpt), prompt, steps=4)["generated"]
    lib = C.CDLL(str(_build.build_core()))
    lib.ifab_program_error.restype = C.c_char_p
    h = C.c_void_p()
    assert lib.ifab_program_open(str(bundle).encode(), str(ckpt).encode(), 0, C.byref(h)) == 0, lib.ifab_program_error()
    assert lib.ifab_program_abi_version() == 1
    ctx, vocab, eos, cap = C.c_uint32(), C.c_uint32(), C.c_uint32(), C.c_uint32()
    assert lib.ifab_program_info(h, C.byref(ctx), C.byref(vocab), C.byref(eos)) == 0 and vocab.value > 300
    assert lib.ifab_program_resident_capacity(h, C.byref(cap)) == 0 and cap.value == 2
    out = C.c_uint32()
    arr = (C.c_uint32 * len(prompt))(*prompt)
    assert lib.ifab_program_select_resident(h, 1) == 0
    assert lib.ifab_program_prefill(h, arr, len(prompt), 0, 1, C.byref(out)) == 0, lib.ifab_program_error()
    got = [out.value]
    for i in range(3):
        assert lib.ifab_program_token(h, got[-1], len(prompt) + i, 1, C.byref(out)) == 0
        got.append(out.value)
    assert got == want
    # wrong position, unknown slot, copy rules
    assert lib.ifab_program_token(h, 1, 3, 1, C.byref(out)) != 0 and b"stands at position" in lib.ifab_program_error()
    assert lib.ifab_program_select_resident(h, 7) != 0
    assert lib.ifab_program_copy_resident(h, 1, 0, len(prompt) + 3) == 0
    assert lib.ifab_program_copy_resident(h, 1, 0, len(prompt) + 3) != 0                 # destination no longer reset
    # batch: resident 0 continues the copied sequence, resident 1 too; both produce the same next token
    Seq = C.c_uint32 * 4
    seqs = (Seq * 2)(Seq(0, len(prompt) + 3, 1, 1), Seq(1, len(prompt) + 3, 1, 1))
    toks = (C.c_uint32 * 2)(got[-1], got[-1])
    outs, n = (C.c_uint32 * 2)(), C.c_uint32()
    assert lib.ifab_program_batch(h, seqs, 2, toks, 2, outs, 2, C.byref(n)) == 0, lib.ifab_program_error()
    assert n.value == 2 and outs[0] == outs[1]
    assert lib.ifab_program_close(h) == 0
    s = Server("--program", str(bundle), str(ckpt), "--cpu")
    try:
        st, g = s.post("/inference/v1/generate", {"token_ids": prompt, "sampling_params": {"max_tokens": 4}}, timeout=120)
        assert st == 200 and g["token_ids"] == want
        st, e = s.post("/v1/completions", {"prompt": "x", "temperature": 0.9})
        assert st == 400 and "greedy" in e["error"]["message"]
    finally:
        s.close()


@pytest.mark.gpu
def test_gpu_engine_sampling_prefix_cache_and_int8_kv():
    """The engine worker with device sampling, the prefix cache of device snapshots and the packed int8 KV cache."""
    s = Server("--spawn", f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 2 --max-model-len 128 "
               "--prefix-cache-slots 4", "--accept-seconds", "300", timeout=400)
    try:
        prompt = list(range(10, 10 + 27))
        body = {"token_ids": prompt, "sampling_params": {"max_tokens": 8}}
        st, first = s.post("/inference/v1/generate", body, timeout=120)
        st, again = s.post("/inference/v1/generate", body, timeout=120)          # 24 of the 27 prompt rows come from the snapshot
        assert st == 200 and again["token_ids"] == first["token_ids"]
        st, longer = s.post("/inference/v1/generate", {"token_ids": prompt + [5, 6], "sampling_params": {"max_tokens": 4}}, timeout=120)
        assert st == 200 and len(longer["token_ids"]) == 4
        # seeded sampling is reproducible, different seeds diverge, temperature 0 equals greedy
        samp = lambda seed: s.post("/inference/v1/generate", {"token_ids": prompt, "sampling_params": {
            "max_tokens": 12, "temperature": 1.5, "top_k": 40, "top_p": 0.95, "seed": seed, "presence_penalty": 0.5}}, timeout=120)[1]["token_ids"]
        a, b, c = samp(1), samp(1), samp(2)
        assert a == b and a != c and a != first["token_ids"][:12]
        st, bad = s.post("/inference/v1/generate", {"token_ids": prompt, "sampling_params": {"temperature": 1.0, "top_k": 500}}, timeout=60)
        assert st == 503 or st == 400
    finally:
        s.close()
    s = Server("--spawn", f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 2 --max-model-len 128 --kv-int8",
               "--accept-seconds", "300", timeout=400)
    try:
        st, q8 = s.post("/inference/v1/generate", {"token_ids": list(range(10, 37)), "sampling_params": {"max_tokens": 8}}, timeout=120)
        assert st == 200 and len(q8["token_ids"]) == 8
    finally:
        s.close()


@pytest.mark.gpu
def test_gpu_engine_worker_profile_only_writes_the_memory_profile(tmp_path):
    import json
    import subprocess

    path = tmp_path / "mem.json"
    r = subprocess.run([sys.executable, "-m", "ironpangu_b200.runtime.engine_worker", "--model", "tiny", "--max-num-seqs", "2",
                        "--max-model-len", "128", "--memory-profile", str(path), "--profile-only"],
                       capture_output=True, text=True, timeout=300, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads(path.read_text())
    assert [s["name"] for s in d["stages"]] == ["fabric", "weights", "bundle", "state", "sampling"]
    assert d["failed_stage"] is None and d["headroom_bytes"] > 0 and d["stages"][1]["delta_bytes"] > 0


def test_serving_load_generator_against_the_mock_server():
    from ironpangu_b200.utils import bench_serving

    res = bench_serving.main(["--mode", "mock", "--requests", "12", "--rate", "400", "--max-model-len", "128", "--vocab", "300",
                              "--prompt-len", "4,20", "--output-len", "3,9", "--max-num-seqs", "3"])
    assert res["completed"] == 12 and res["statuses"] == {"200": 12} and res["server_exit"] == 0
    assert res["output_tokens"] >= 36 and res["ttft_ms"]["p50"] > 0 and res["tpot_ms"]["p50"] > 0


@pytest.mark.gpu
def test_gpu_engine_prefills_long_prompts_on_the_tensor_cores():
    """With --prefill-chunk the worker advertises a larger token budget and runs prompt slices through the matrix-matrix path;
    the first generated token equals the one of the decode-kernel prefill."""
    cmd = f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model tiny --max-num-seqs 2 --max-model-len 256 --greedy-only"
    prompt = [(7 * i + 3) % 1000 for i in range(150)]
    outs = []
    for extra in ("", " --prefill-chunk 64"):
        s = Server("--spawn", cmd + extra, "--accept-seconds", "300", timeout=400)
        try:
            st, r = s.post("/inference/v1/generate", {"token_ids": prompt, "sampling_params": {"max_tokens": 6}}, timeout=120)
            assert st == 200 and len(r["token_ids"]) == 6
            outs.append(r["token_ids"])
        finally:
            s.close()
    assert outs[0][0] == outs[1][0]


@pytest.mark.gpu
def test_gpu_dense_worker_batches_decode_rows_on_the_tensor_cores():
    """Dense model behind the server with a tensor-core prompt path: many concurrent sampled requests complete, and the
    decode rows of a step run as one matrix-matrix pass (audit counter)."""
    from ironpangu_b200.utils import bench_serving

    res = bench_serving.main(["--mode", "worker", "--model", "dense-tiny", "--requests", "12", "--max-model-len", "256", "--vocab", "1024",
                              "--prompt-len", "20,90", "--output-len", "6,14", "--max-num-seqs", "12", "--max-num-batched-tokens", "96",
                              "--prefill-chunk", "64", "--temperature", "0.8", "--top-k", "20", "--timeout", "300"])
    assert res["completed"] == 12 and res["server_exit"] == 0, res
    assert res["output_tokens"] >= 72

    cmd = (f"{sys.executable} -m ironpangu_b200.runtime.engine_worker --model dense-tiny --max-num-seqs 4 --max-model-len 256 "
           "--max-num-batched-tokens 64 --set prefill_chunk=32 --set spin_limit=2000000")
    s = Server("--spawn", cmd, "--accept-seconds", "300", timeout=400)
    try:
        prompt = [(5 * i + 1) % 1000 for i in range(70)]
        outs = [None] * 3
        def go(i):
            outs[i] = s.post("/inference/v1/generate", {"token_ids": prompt[: 40 + 10 * i], "sampling_params": {"max_tokens": 8}}, timeout=120)
        ths = [threading.Thread(target=go, args=(i,)) for i in range(3)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        assert all(o[0] == 200 and len(o[1]["token_ids"]) == 8 for o in outs)
        st, body = s.request("GET", "/audit")
        a = json.loads(body)["engine"]
        assert st == 200 and a["prefill_chunks"] >= 3 and a["fabric_status"] == 0
        assert a["runtime_options"]["prefill_chunk"] == 32 and a["runtime_options"]["spin_limit"] == 2000000
    finally:
        s.close()


def test_server_fails_fast_when_the_spawned_engine_dies():
    """A worker that exits before connecting ends the wait at once instead of after the whole accept window."""
    from ironpangu_b200 import _build

    _build.build_core()
    t0 = time.time()
    r = subprocess.run([str(_build.SERVER_BIN), "--port", "0", "--spawn", "exit 3", "--accept-seconds", "120"], capture_output=True, text=True,
                       timeout=60)
    assert r.returncode != 0 and time.time() - t0 < 20
    assert "exited before connecting" in (r.stdout + r.stderr)
