"""Kernel / loader fixtures: round trip of the file format, shard shapes of a two-rank plan, the MoE partials of both ranks sum
to the unsharded result."""
import json

import torch

from ironpangu_b200.utils import export_fixture as X


def test_fixtures_of_a_two_rank_bundle(tmp_path):
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig

    cfg = MlaMoeConfig.tiny(layers=1)
    src, ck, b = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "b"
    src.write_text(mla_moe_source(cfg, 2, context=64))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "2").returncode == 0
    compiler.write_bundle(str(src), str(b), checkpoint_dir=str(ck))
    assert X.main(["tensor", str(ck), "model.layers.0.self_attn.o_proj", str(tmp_path / "t.bin")]) == 0
    full = X.read_fixture(str(tmp_path / "t.bin"))["model.layers.0.self_attn.o_proj.weight"]
    assert full.shape == (cfg.hidden, cfg.heads * cfg.vdim) and full.dtype == torch.bfloat16
    assert X.main(["load-plan", str(b), "1", str(tmp_path / "lp.json")]) == 0
    lp = json.loads((tmp_path / "lp.json").read_text())
    assert lp["format"] == "ifab.load-plan-fixture.v1" and all("parameter" in l and "shard" in l for l in lp["loads"])
    for rank in (0, 1):
        assert X.main(["linear", str(b), str(ck), str(rank), "model.layers.0.self_attn.o_proj", str(tmp_path / f"l{rank}.bin"), "--rows", "3"]) == 0
    l0, l1 = X.read_fixture(str(tmp_path / "l0.bin")), X.read_fixture(str(tmp_path / "l1.bin"))
    assert torch.equal(torch.cat([l0["weight"], l1["weight"]], 1), full)                     # the column shards of the two ranks
    assert l0["expected"].shape == (3, cfg.hidden)
    torch.testing.assert_close(l0["expected"].float(), l0["input"].float() @ l0["weight"].float().T, rtol=1e-2, atol=1e-2)
    for rank in (0, 1):
        assert X.main(["moe", str(b), str(ck), str(rank), "0", str(tmp_path / f"m{rank}.bin"), "--rows", "2", "--seed", "4"]) == 0
    m0, m1 = X.read_fixture(str(tmp_path / "m0.bin")), X.read_fixture(str(tmp_path / "m1.bin"))
    assert torch.equal(m0["input"], m1["input"]) and torch.equal(m0["route_ids"], m1["route_ids"])
    assert m0["gate_up"].shape == (cfg.experts // 2, 2 * cfg.expert_ffn, cfg.hidden)
    # every route is owned by exactly one rank: the partials add up to the unsharded mixture
    gu, dn = torch.cat([m0["gate_up"], m1["gate_up"]]), torch.cat([m0["down"], m1["down"]])
    want = torch.zeros(2, cfg.hidden)
    for t in range(2):
        for k in range(cfg.topk):
            e = int(m0["route_ids"][t, k])
            h = m0["input"][t].float() @ gu[e].float().T
            a = (torch.nn.functional.silu(h[:cfg.expert_ffn]) * h[cfg.expert_ffn:]).to(torch.bfloat16).float()
            want[t] += m0["route_weights"][t, k] * (a @ dn[e].float().T)
    torch.testing.assert_close(m0["expected_partial"] + m1["expected_partial"], want, rtol=1e-4, atol=1e-5)
