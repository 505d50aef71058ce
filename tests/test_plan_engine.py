"""Compiled bundle -> device execution: the plan-driven engine against the CPU interpreter of the same plan."""
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
SLICE = ROOT / "examples" / "mla_moe_slice_tp1.inferfabric"


def test_bundle_executes_token_exact_against_cpu_interpreter(tmp_path):
    from ironpangu_b200 import compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.engine import DecodeEngine
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    ck, bundle = tmp_path / "ck", tmp_path / "bundle"
    assert compiler.cli("synth-checkpoint", str(SLICE), str(ck), "--seed", "3").returncode == 0
    compiler.write_bundle(SLICE, bundle, checkpoint_dir=str(ck))
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1024, (16,), generator=g).tolist()
    first = compiler.interpret(SLICE.read_text(), str(ck), prompt, steps=8)
    seq = prompt + first["generated"]
    oracle = compiler.interpret(SLICE.read_text(), str(ck), seq, all_logits=True)
    ref = torch.tensor(oracle["prompt_logits"])

    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, keep_logits=True)
    drv = DecodeEngine(eng)
    # teacher-forced on the oracle's tokens; logits must agree everywhere, tokens wherever the oracle has no near-tie
    for s in range(0, len(seq), 8):
        chunk = seq[s:s + 8]
        n = len(chunk)
        eng.tokens[:n].copy_(torch.tensor(chunk, dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        got, logits = eng.next_ids[:n].tolist(), eng.logits[:n].cpu()
        torch.testing.assert_close(logits, ref[s:s + n], rtol=2e-2, atol=1e-2)
        for i in range(n):
            top2 = ref[s + i].topk(2).values
            if float(top2[0] - top2[1]) > 1e-2:
                assert got[i] == int(ref[s + i].argmax()), (s + i, got[i])
            assert got[i] == int(logits[i].argmax())
    # engine API: greedy generation through prefill chunks + captured decode graph
    eng.reset()
    out = drv.generate(prompt, 8)
    assert len(out) == 8 and all(0 <= t < 1024 for t in out)
    if all(float(ref[15 + i].topk(2).values.diff().abs()) > 1e-2 for i in range(8)):
        assert out == first["generated"]
    assert fab.status() == 0
    fab.close()
