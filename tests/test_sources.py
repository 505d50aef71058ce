"""Generated .inferfabric sources: they compile for every tensor-parallel width, and the init plans they produce name exactly the
tensors (shape, dtype) that ``bundle_parameters`` hands to the plan engine."""
import json
from pathlib import Path

import pytest
import torch


@pytest.mark.parametrize("tp", [1, 2, 8])
def test_generated_source_matches_the_decoders_weights(tmp_path, tp):
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, bundle_parameters, random_rank_weights

    cfg = MlaMoeConfig.tiny(layers=3)
    src = tmp_path / "m.inferfabric"
    src.write_text(mla_moe_source(cfg, tp, context=256))
    out = compiler.write_bundle(str(src), str(tmp_path / "b"), prefill_tokens=8)
    assert out["collectives_per_token"] == 2 * cfg.layers + 1
    weights = random_rank_weights(cfg, tp - 1, tp, "cpu")
    given = bundle_parameters(cfg, weights)
    plan = json.loads((Path(out["dir"]) / f"rank-{tp - 1}.init.json").read_text())
    names = {p["name"] for p in plan["parameters"]}
    assert names == set(given), (names ^ set(given))
    for p in plan["parameters"]:
        t = given[p["name"]]
        assert list(t.shape) == p["dims"], p["name"]
        assert {"bf16": torch.bfloat16, "f32": torch.float32}[p["dtype"]] == t.dtype, p["name"]


def test_flagship_example_is_the_generated_source_at_tp8(tmp_path):
    """The checked-in example and the generator describe the same program (same instruction stream and parameters)."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig

    root = Path(__file__).resolve().parents[1]
    cfg = MlaMoeConfig.flagship()
    cfg.eos = 2
    gen = tmp_path / "g.inferfabric"
    gen.write_text(mla_moe_source(cfg, 8, context=1024, name="MlaMoe92B"))
    a = compiler.write_bundle(str(gen), str(tmp_path / "a"))
    b = compiler.write_bundle(str(root / "examples" / "mla_moe_92b_tp8.inferfabric"), str(tmp_path / "b"))
    pa = json.loads((Path(a["dir"]) / "device-program.json").read_text())["instructions"]
    pb = json.loads((Path(b["dir"]) / "device-program.json").read_text())["instructions"]
    assert len(pa) == len(pb) == 554
    strip = lambda i: (i["op"], i["width"], i["dtype"], i["inputs"], {k: (float(v) if k in ("norm_eps", "eps", "scale", "theta") else v)
                                                                      for k, v in i["attrs"].items()})
    assert [strip(i) for i in pa] == [strip(i) for i in pb]


def test_hyper_and_dense_examples_are_the_generated_sources(tmp_path):
    """`examples/hyper_mla_moe_92b_tp8.inferfabric` (46 layers, 4 residual streams, 256 experts, 128 sinks) and
    `examples/dense_gqa_2b_tp2.inferfabric` are what the generators write; the 92B program needs 35,085 checkpoint tensors."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, dense_gqa_source, hyper_mla_moe_source
    from ironpangu_b200.models.dense_gqa import DenseConfig

    root = Path(__file__).resolve().parents[1] / "examples"
    assert (root / "hyper_mla_moe_92b_tp8.inferfabric").read_text() == hyper_mla_moe_source(HyperMlaMoeConfig.pangu92b(), 8, context=512,
                                                                                             name="HyperMlaMoe92B")
    assert (root / "dense_gqa_2b_tp2.inferfabric").read_text() == dense_gqa_source(DenseConfig.qwen2b(), 2, context=2048, name="DenseGqa2B")
    r = compiler.cli("explain", str(root / "hyper_mla_moe_92b_tp8.inferfabric"))
    assert r.returncode == 0, r.stderr
    e = json.loads(r.stdout)
    assert e["checkpoint_tensors"] == 35085 and e["checkpoint_bytes"] == 183188067132 and e["parallel"]["tp"] == 8
    ops = e["physical_ops"]
    assert ops["mhc_pre"] == 92 and ops["mhc_post"] == 92 and ops["mome"] == 138 and ops["sink_normalize"] == 46 and ops["moe_down_allreduce"] == 44
    assert "norm" not in ops          # every norm is folded: into a projection, the router, or the return of a hyper-connection
    out = compiler.write_bundle(str(root / "hyper_mla_moe_92b_tp8.inferfabric"), str(tmp_path / "b"))
    assert compiler.validate_bundle(out["dir"])["ranks"] == 8
    # the variant with packed int8 caches and learned sparse attention on every third layer (eight of those sixteen layers run the indexer)
    assert (root / "hyper_mla_moe_92b_learned_tp8.inferfabric").read_text() == hyper_mla_moe_source(HyperMlaMoeConfig.pangu92b_learned(), 8,
                                                                                                     context=512, name="HyperMlaMoe92BLearned")
    r = compiler.cli("explain", str(root / "hyper_mla_moe_92b_learned_tp8.inferfabric"))
    assert r.returncode == 0, r.stderr
    e = json.loads(r.stdout)
    assert e["checkpoint_tensors"] == 35117 and e["checkpoint_bytes"] == 183244626748
    assert e["physical_ops"]["sparse_index"] == 8 and e["physical_ops"]["index_cache_append"] == 8
    d = compiler.cli("explain", str(root / "dense_gqa_2b_tp2.inferfabric"))
    assert d.returncode == 0 and json.loads(d.stdout)["physical_ops"]["paged_attention"] == 24


def test_packed_cache_source_quantises_in_the_oracle(tmp_path):
    """`kv_int8=True` declares packed int8 latent caches; the CPU oracle then reads back quantised latent rows: logits move by
    the quantisation noise (not zero, not large) and the cache instructions carry the packed dtype."""
    import dataclasses

    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig

    cfg = dataclasses.replace(MlaMoeConfig.tiny(2), eos=2)
    plain, packed = tmp_path / "plain.inferfabric", tmp_path / "packed.inferfabric"
    plain.write_text(mla_moe_source(cfg, 1, context=64))
    packed.write_text(mla_moe_source(cfg, 1, context=64, kv_int8=True))
    assert compiler.cli("synth-checkpoint", str(plain), str(tmp_path / "ck"), "--seed", "2").returncode == 0
    out = compiler.write_bundle(str(packed), str(tmp_path / "b"), checkpoint_dir=str(tmp_path / "ck"))
    ins = json.loads((Path(out["dir"]) / "device-program.json").read_text())["instructions"]
    assert [i["dtype"] for i in ins if i["op"] == "mla_kv_write"] == ["int8_ds_mla"] * cfg.layers
    toks = [5, 17, 99, 3, 64, 120, 8, 41]
    a = torch.tensor(compiler.interpret(plain.read_text(), str(tmp_path / "ck"), toks, all_logits=True)["prompt_logits"])
    b = torch.tensor(compiler.interpret(packed.read_text(), str(tmp_path / "ck"), toks, all_logits=True)["prompt_logits"])
    diff = float((a - b).abs().max())
    assert 0.0 < diff < 0.1, diff


def test_random_parameters_follow_the_init_plan(tmp_path):
    """Random init without a checkpoint: every parameter of a rank's plan is filled with its planned shape and dtype, replicated
    tensors come out identical on every rank, the shards of a split tensor differ, gains of norms are near one, and the same seed
    gives the same values."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source
    from ironpangu_b200.runtime.plan_engine import random_parameters

    src = tmp_path / "m.inferfabric"
    src.write_text(hyper_mla_moe_source(HyperMlaMoeConfig.tiny(3), 2, context=64))
    out = compiler.write_bundle(str(src), str(tmp_path / "b"), prefill_tokens=8)
    plans = [json.loads((Path(out["dir"]) / f"rank-{r}.init.json").read_text()) for r in range(2)]
    P = [random_parameters(pl, "cpu", seed=4) for pl in plans]
    for pl, params in zip(plans, P):
        assert set(params) == {p["name"] for p in pl["parameters"]}
        for p in pl["parameters"]:
            t = params[p["name"]]
            assert list(t.shape) == p["dims"] and t.dtype == {"bf16": torch.bfloat16, "f32": torch.float32}[p["dtype"]], p["name"]
    router, q_b, norm = "model.layers.1.mlp.gate", "model.layers.0.self_attn.q_b_proj", "model.layers.0.input_layernorm"
    assert torch.equal(P[0][router], P[1][router]) and torch.equal(P[0][norm], P[1][norm])            # replicated
    assert not torch.equal(P[0][q_b], P[1][q_b])                                                      # row shards of one tensor
    experts = "model.layers.1.mlp.experts.{expert}.down_proj"
    assert not torch.equal(P[0][experts], P[1][experts])                                              # different experts per rank
    assert abs(float(P[0][norm].float().mean()) - 1.0) < 0.02 and abs(float(P[0][q_b].float().std()) - 0.02) < 0.004
    again = random_parameters(plans[0], "cpu", seed=4)
    assert all(torch.equal(again[k], v) for k, v in P[0].items())
    other = random_parameters(plans[0], "cpu", seed=5)
    assert not torch.equal(other[q_b], P[0][q_b])


@pytest.mark.parametrize("args", [["tiny", "--tp", "2", "--kv-int8"], ["dense-tiny", "--tp", "2"], ["hyper-tiny", "--learned"],
                                  ["hyper-tiny", "--kv-int8", "--layers", "2"], ["pangu92b", "--tp", "8", "--learned"]])
def test_source_printer_writes_programs_that_compile(tmp_path, args):
    import subprocess
    import sys

    from ironpangu_b200 import compiler

    r = subprocess.run([sys.executable, "-m", "ironpangu_b200.compiler.sources", *args], capture_output=True, text=True,
                       cwd=str(Path(__file__).resolve().parents[1]))
    assert r.returncode == 0 and r.stdout.startswith("language inferfabric 1;"), r.stderr
    src = tmp_path / "m.inferfabric"
    src.write_text(r.stdout)
    e = compiler.cli("explain", str(src))
    assert e.returncode == 0, e.stderr
    tp = int(args[args.index("--tp") + 1]) if "--tp" in args else 1
    assert json.loads(e.stdout)["parallel"]["tp"] == tp
