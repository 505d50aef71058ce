"""The native device executor (csrc/device): a compiled bundle run on the GPU from C++ - through its C ABI and as the engine of
`ifab-server --program ... --native` - against the CPU interpreter of the same program and against the Python plan engine."""
import ctypes as C
import json
import os
import signal
import subprocess
import http.client
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
SLICE = ROOT / "examples" / "mla_moe_slice_tp1.inferfabric"


def _bundle(tmp_path, residents=2):
    from ironpangu_b200 import compiler

    ck, bundle = tmp_path / "ck", tmp_path / "bundle"
    assert compiler.cli("synth-checkpoint", str(SLICE), str(ck), "--seed", "3").returncode == 0
    r = compiler.cli("compile-token", str(SLICE), str(ck), str(bundle), "--resident-sequences", str(residents), "--prefill-tokens", "8")
    assert r.returncode == 0, r.stderr
    return ck, bundle


def test_c_abi_matches_the_interpreter_and_the_plan_engine(tmp_path):
    from ironpangu_b200 import _build, compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    ck, bundle = _bundle(tmp_path)
    lib = C.CDLL(str(_build.build_device()))
    lib.ifab_device_program_error.restype = C.c_char_p
    h = C.c_void_p()
    assert lib.ifab_device_program_open(str(bundle).encode(), str(ck).encode(), 0, 2, C.byref(h)) == 0, lib.ifab_device_program_error()
    ctx, vocab, eos, res, rows = (C.c_uint32() for _ in range(5))
    assert lib.ifab_device_program_info(h, C.byref(ctx), C.byref(vocab), C.byref(eos), C.byref(res), C.byref(rows)) == 0
    assert (vocab.value, res.value, rows.value) == (1024, 2, 8) and ctx.value >= 64

    def run(tokens, positions, slots):
        n = len(tokens)
        arr = lambda v: (C.c_int32 * n)(*v)
        out = (C.c_int32 * n)()
        assert lib.ifab_device_program_rows(h, arr(tokens), arr(positions), arr(slots), n, out) == 0, lib.ifab_device_program_error()
        return list(out)

    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1024, (16,), generator=g).tolist()
    first = compiler.interpret(SLICE.read_text(), str(ck), prompt, steps=8)
    oracle = compiler.interpret(SLICE.read_text(), str(ck), prompt + first["generated"], all_logits=True)
    ref = torch.tensor(oracle["prompt_logits"])
    seq = prompt + first["generated"]
    # teacher-forced on the oracle's tokens, eight rows per launch group, in resident slot 1
    got = []
    for s in range(0, len(seq), 8):
        got += run(seq[s:s + 8], list(range(s, min(len(seq), s + 8))), [1] * len(seq[s:s + 8]))
    for i, t in enumerate(got):
        top2 = ref[i].topk(2).values
        if float(top2[0] - top2[1]) > 1e-2:
            assert t == int(ref[i].argmax()), (i, t)
    # the Python plan engine runs the same kernels on the same bundle: identical tokens, row for row
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, num_slots=2)
    same = []
    for s in range(0, len(seq), 8):
        n = len(seq[s:s + 8])
        eng.tokens[:n].copy_(torch.tensor(seq[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].fill_(1)
        eng.forward(n)
        same += eng.next_ids[:n].tolist()
    assert got == same
    fab.close()
    # single-row decode in the other slot replays a graph; the two residents do not disturb each other
    tok, dec = prompt[0], []
    for i in range(12):
        tok = run([tok], [i], [0])[0]
        dec.append(tok)
    again = run(seq[:8], list(range(8)), [1] * 8)
    assert again == got[:8]
    buf = C.create_string_buffer(1 << 16)
    assert lib.ifab_device_program_audit(h, buf, len(buf)) == 0
    audit = json.loads(buf.value)
    assert audit["format"] == "ifab.device-program-audit.v1" and audit["graph_widths"] == [1, 8] and audit["steps"] == 3 + 12 + 1
    assert audit["arena"]["planned_rows"] == 8 and audit["parameter_bytes_uploaded"] > 0
    assert audit["device_allocations_after_ready"] == 0                     # a step allocates nothing
    # misuse is refused with a message, the engine stays usable
    assert lib.ifab_device_program_rows(h, (C.c_int32 * 1)(5000), (C.c_int32 * 1)(0), (C.c_int32 * 1)(0), 1, (C.c_int32 * 1)()) != 0
    assert b"vocabulary" in lib.ifab_device_program_error()
    assert lib.ifab_device_program_rows(h, (C.c_int32 * 1)(5), (C.c_int32 * 1)(0), (C.c_int32 * 1)(7), 1, (C.c_int32 * 1)()) != 0
    assert run([prompt[0]], [0], [0])[0] == dec[0]
    assert lib.ifab_device_program_close(h) == 0


def test_server_runs_the_bundle_natively(tmp_path):
    from ironpangu_b200 import _build, compiler

    ck, bundle = _bundle(tmp_path)
    _build.build_device()
    prompt = [5, 77, 300, 12, 9, 41, 8, 100, 3, 250, 17]
    want = compiler.interpret(SLICE.read_text(), str(ck), prompt, steps=6)["generated"]
    proc = subprocess.Popen([str(_build.SERVER_BIN), "--port", "0", "--program", str(bundle), str(ck), "--native"], stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True)
    try:
        port, lines = None, []
        for line in proc.stdout:
            lines.append(line)
            if line.startswith("listening on"):
                port = int(line.rsplit(":", 1)[1])
                break
        assert port, "".join(lines)

        def post(path, body):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
            r = c.getresponse()
            data = r.read().decode()
            c.close()
            return r.status, json.loads(data)

        st, g = post("/inference/v1/generate", {"token_ids": prompt, "sampling_params": {"max_tokens": 6}})
        assert st == 200 and len(g["token_ids"]) == 6
        oracle = compiler.interpret(SLICE.read_text(), str(ck), prompt + want, all_logits=True)["prompt_logits"]
        for i, (a, b) in enumerate(zip(g["token_ids"], want)):
            if a != b:
                top2 = torch.tensor(oracle[len(prompt) - 1 + i]).topk(2).values
                assert float(top2[0] - top2[1]) < 1e-2
                break
        # two requests at once share the engine's launch groups
        import threading
        out = {}
        ts = [threading.Thread(target=lambda i=i: out.__setitem__(i, post("/inference/v1/generate", {"token_ids": prompt[:4 + i], "sampling_params": {"max_tokens": 5}})))
              for i in range(2)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert all(v[0] == 200 and len(v[1]["token_ids"]) == 5 for v in out.values())
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
        c.request("GET", "/audit")
        audit = json.loads(c.getresponse().read())
        assert audit["engine"]["format"] == "ifab.device-program-audit.v1" and audit["engine"]["fused_head"] is True
        st, e = post("/v1/completions", {"prompt": "x", "temperature": 0.9})
        assert st == 400 and "greedy" in e["error"]["message"]
    finally:
        proc.send_signal(signal.SIGTERM)
        proc.wait(timeout=60)
    assert proc.returncode == 0


def test_dense_bundle_runs_natively_like_the_plan_engine(tmp_path):
    """A grouped-query-attention program: the native executor packs q | k | v, rotates and appends, attends - tokens equal the
    CPU interpreter's where its logits are decisive, and the Python plan engine's row for row."""
    from ironpangu_b200 import _build, compiler
    from ironpangu_b200.compiler.sources import dense_gqa_source
    from ironpangu_b200.models.dense_gqa import DenseConfig
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = DenseConfig.tiny(2)
    src, ck, bundle = tmp_path / "dense.inferfabric", tmp_path / "ck", tmp_path / "bundle"
    src.write_text(dense_gqa_source(cfg, 1, 128))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "4").returncode == 0
    r = compiler.cli("compile-token", str(src), str(ck), str(bundle), "--resident-sequences", "2", "--prefill-tokens", "8")
    assert r.returncode == 0, r.stderr
    lib = C.CDLL(str(_build.build_device()))
    lib.ifab_device_program_error.restype = C.c_char_p
    h = C.c_void_p()
    assert lib.ifab_device_program_open(str(bundle).encode(), str(ck).encode(), 0, 2, C.byref(h)) == 0, lib.ifab_device_program_error()

    def run(tokens, positions, slots):
        n = len(tokens)
        arr = lambda v: (C.c_int32 * n)(*v)
        out = (C.c_int32 * n)()
        assert lib.ifab_device_program_rows(h, arr(tokens), arr(positions), arr(slots), n, out) == 0, lib.ifab_device_program_error()
        return list(out)

    seq = torch.randint(0, cfg.vocab, (27,), generator=torch.Generator().manual_seed(9)).tolist()
    ref = torch.tensor(compiler.interpret(src.read_text(), str(ck), seq, all_logits=True)["prompt_logits"])
    got = []
    for s in range(0, len(seq), 8):
        got += run(seq[s:s + 8], list(range(s, min(len(seq), s + 8))), [1] * len(seq[s:s + 8]))
    decisive = 0
    for i, t in enumerate(got):
        top2 = ref[i].topk(2).values
        if float(top2[0] - top2[1]) > 2e-2:
            decisive += 1
            assert t == int(ref[i].argmax()), (i, t)
    assert decisive >= len(seq) // 2
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, num_slots=2)
    same = []
    for s in range(0, len(seq), 8):
        n = len(seq[s:s + 8])
        eng.tokens[:n].copy_(torch.tensor(seq[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].fill_(1)
        eng.forward(n)
        same += eng.next_ids[:n].tolist()
    assert got == same
    fab.close()
    one = [run([seq[i]], [i], [0])[0] for i in range(10)]            # single rows in the other slot, graph replay after the first
    assert all(a == b for i, (a, b) in enumerate(zip(one, got)) if float(ref[i].topk(2).values[0] - ref[i].topk(2).values[1]) > 2e-2)
    buf = C.create_string_buffer(1 << 16)
    assert lib.ifab_device_program_audit(h, buf, len(buf)) == 0
    audit = json.loads(buf.value)
    assert audit["device_allocations_after_ready"] == 0 and audit["launches_per_step"] == 1 + cfg.layers * 7 + 1
    assert lib.ifab_device_program_close(h) == 0


def test_hyper_connected_bundle_runs_natively_like_the_plan_engine(tmp_path):
    """Residual streams mixed by mHC modules, token convolutions with per-resident history, sink rows, a folded branch norm and
    an optional norm the checkpoint lacks: the native executor gives the plan engine's tokens row for row, and the CPU
    interpreter's wherever its logits are decisive; the two residents keep separate histories."""
    import sys

    sys.path.insert(0, str(ROOT / "tests"))
    from hyper_source import source

    from ironpangu_b200 import _build, compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    src, ck, bundle = tmp_path / "hyper.inferfabric", tmp_path / "ck", tmp_path / "bundle"
    src.write_text(source(layers=2))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "7").returncode == 0
    r = compiler.cli("compile-token", str(src), str(ck), str(bundle), "--resident-sequences", "2", "--prefill-tokens", "8")
    assert r.returncode == 0, r.stderr
    lib = C.CDLL(str(_build.build_device()))
    lib.ifab_device_program_error.restype = C.c_char_p
    h = C.c_void_p()
    assert lib.ifab_device_program_open(str(bundle).encode(), str(ck).encode(), 0, 2, C.byref(h)) == 0, lib.ifab_device_program_error()

    def run(tokens, positions, slots):
        n = len(tokens)
        arr = lambda v: (C.c_int32 * n)(*v)
        out = (C.c_int32 * n)()
        assert lib.ifab_device_program_rows(h, arr(tokens), arr(positions), arr(slots), n, out) == 0, lib.ifab_device_program_error()
        return list(out)

    seq = torch.randint(1, 512, (21,), generator=torch.Generator().manual_seed(4)).tolist()
    other = torch.randint(1, 512, (9,), generator=torch.Generator().manual_seed(5)).tolist()
    ref = torch.tensor(compiler.interpret(src.read_text(), str(ck), seq, all_logits=True)["prompt_logits"])
    got = run(seq[:8], list(range(8)), [0] * 8)
    run(other[:8], list(range(8)), [1] * 8)                        # another resident in between: its history and pages are its own
    got += run(seq[8:16], list(range(8, 16)), [0] * 8)
    got += [run([seq[i]], [i], [0])[0] for i in range(16, 21)]     # single rows: a graph per width
    decisive = 0
    for i, t in enumerate(got):
        top2 = ref[i].topk(2).values
        if float(top2[0] - top2[1]) > 2e-2:
            decisive += 1
            assert t == int(ref[i].argmax()), (i, t)
    assert decisive >= len(seq) // 2
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, num_slots=2)
    same = []
    for s in (0, 8):
        eng.tokens[:8].copy_(torch.tensor(seq[s:s + 8], dtype=torch.int32))
        eng.positions[:8].copy_(torch.arange(s, s + 8, dtype=torch.int32))
        eng.slots[:8].zero_()
        eng.forward(8)
        same += eng.next_ids[:8].tolist()
    for i in range(16, 21):
        eng.tokens[:1].fill_(seq[i])
        eng.positions[:1].fill_(i)
        eng.slots[:1].zero_()
        eng.forward(1)
        same.append(int(eng.next_ids[0]))
    assert got == same
    fab.close()
    assert lib.ifab_device_program_reset(h) == 0
    assert run(seq[:8], list(range(8)), [0] * 8) == got[:8]       # after a reset the histories are empty again
    buf = C.create_string_buffer(1 << 16)
    assert lib.ifab_device_program_audit(h, buf, len(buf)) == 0
    assert json.loads(buf.value)["device_allocations_after_ready"] == 0
    assert lib.ifab_device_program_close(h) == 0


def test_learned_selection_bundle_runs_natively_like_the_plan_engine(tmp_path):
    """Packed int8 latent caches, an int8 index cache, the selector and attention over its selection (one layer computing it, a
    later one reusing it): the native executor's tokens equal the plan engine's."""
    import dataclasses

    from ironpangu_b200 import _build, compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = dataclasses.replace(HyperMlaMoeConfig.tiny(3), packed_every=2, learned=True, index_heads=8, index_dim=64, index_rotary=32, index_topk=6)
    src, ck, bundle = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "bundle"
    src.write_text(hyper_mla_moe_source(cfg, 1, context=128))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "13").returncode == 0
    r = compiler.cli("compile-token", str(src), str(ck), str(bundle), "--resident-sequences", "2", "--prefill-tokens", "8")
    assert r.returncode == 0, r.stderr
    lib = C.CDLL(str(_build.build_device()))
    lib.ifab_device_program_error.restype = C.c_char_p
    h = C.c_void_p()
    assert lib.ifab_device_program_open(str(bundle).encode(), str(ck).encode(), 0, 2, C.byref(h)) == 0, lib.ifab_device_program_error()

    def run(tokens, positions, slots):
        n = len(tokens)
        arr = lambda v: (C.c_int32 * n)(*v)
        out = (C.c_int32 * n)()
        assert lib.ifab_device_program_rows(h, arr(tokens), arr(positions), arr(slots), n, out) == 0, lib.ifab_device_program_error()
        return list(out)

    seq = torch.randint(1, 512, (26,), generator=torch.Generator().manual_seed(9)).tolist()
    got = []
    for s in range(0, 24, 8):
        got += run(seq[s:s + 8], list(range(s, s + 8)), [1] * 8)
    got += [run([seq[i]], [i], [1])[0] for i in (24, 25)]
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, num_slots=2)
    same = []
    for s in range(0, 24, 8):
        eng.tokens[:8].copy_(torch.tensor(seq[s:s + 8], dtype=torch.int32))
        eng.positions[:8].copy_(torch.arange(s, s + 8, dtype=torch.int32))
        eng.slots[:8].fill_(1)
        eng.forward(8)
        same += eng.next_ids[:8].tolist()
    for i in (24, 25):
        eng.tokens[:1].fill_(seq[i])
        eng.positions[:1].fill_(i)
        eng.slots[:1].fill_(1)
        eng.forward(1)
        same.append(int(eng.next_ids[0]))
    assert got == same
    fab.close()
    assert lib.ifab_device_program_reset(h) == 0
    assert run(seq[:8], list(range(8)), [1] * 8) == got[:8]
    assert lib.ifab_device_program_close(h) == 0
