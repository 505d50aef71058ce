"""CPU-only tests of the offline toolchain: DSL -> checked graph -> physical program -> init plans -> bundle,
and the CPU interpreter against the PyTorch oracle."""
import json
import os
import re
import shutil
import struct
from pathlib import Path

import pytest
import torch

from ironpangu_b200 import compiler

ROOT = Path(__file__).resolve().parents[1]
FLAGSHIP = ROOT / "examples" / "mla_moe_92b_tp8.inferfabric"
SLICE = ROOT / "examples" / "mla_moe_slice_tp1.inferfabric"


@pytest.fixture(scope="module")
def flagship():
    return compiler.compile_source(FLAGSHIP.read_text())


def test_flagship_expands_to_checked_plan(flagship):
    g, p = flagship["graph"], flagship["program"]
    assert len(g["nodes"]) == 1154
    ops = [n["op"] for n in g["nodes"]]
    assert ops.count("allreduce") == 92 and ops.count("gather") == 1 and ops.count("router") == 46
    assert g["max_context"] == 1024 and g["parallel"]["tp"] == 8 and g["parallel"]["devices"] == list(range(8))
    # hygienic instance paths and expansion frames survive
    n = next(n for n in g["nodes"] if n["name"] == "hidden[3]/block/attention/cache")
    assert n["op"] == "cache_norm_rope_append" and n["attrs"]["weight"] == "model.layers.3.self_attn.kv_a_layernorm"
    assert [f["what"] for f in n["frames"]] == ["fold i=3", "module DecoderBlock", "module MLAAttention"]
    # fused lowering: one kernel per fused group, every all-reduce lives inside a compute kernel
    pops = [i["op"] for i in p["instructions"]]
    assert pops.count("linear_allreduce") == 46 and pops.count("moe_down_allreduce") == 46 and pops.count("lm_head") == 1
    assert "allreduce" not in pops and "norm" not in pops and "add" not in pops
    assert p["launches_per_token"] == 416 and p["collectives_per_token"] == 93
    assert p["magic"] == "IFTOKN02"
    down = next(i for i in p["instructions"] if i["op"] == "moe_down_allreduce")
    assert down["attrs"]["residual"] == "input2" and "shared_weight" in down["attrs"]
    head = p["instructions"][p["output"]]
    assert head["op"] == "lm_head" and head["attrs"]["norm_weight"] == "model.norm" and head["width"] == 153600


def test_required_tensors_cover_the_92b_checkpoint(flagship):
    need = flagship["required_tensors"]
    total = sum(int(torch.tensor(t["shape"]).prod()) * (4 if t["dtype"] == "f32" else 2) for t in need.values())
    assert len(need) == 13849
    assert abs(total - 174.6e9) < 0.3e9
    assert need["model.layers.7.mlp.experts.95.down_proj.weight"]["shape"] == [4096, 1536]
    assert need["model.layers.0.self_attn.kv_b_proj.weight"]["shape"] == [32 * 256, 512]


def test_bundle_files_init_plans_and_no_overwrite(tmp_path):
    out = tmp_path / "bundle"
    s = compiler.write_bundle(FLAGSHIP, out)
    assert s["logical_nodes"] == 1154 and s["instructions"] == 554
    names = {p.name for p in out.iterdir()}
    for f in ["execution.bin", "logical.bin", "execution.json", "execution.dot", "execution.html", "device-program.json",
              "physical.json", "serving.json", "plan.json", "arena.json"] + [f"rank-{r}.bin" for r in range(8)] + \
             [f"rank-{r}.init.json" for r in range(8)] + [f"arena-rank-{r}.txt" for r in range(8)]:
        assert f in names, f
    assert json.loads((out / "plan.json").read_text())["format"] == "inferfabric.token-bundle.v1"
    assert (out / "execution.bin").read_bytes()[:8] == b"IFTOKN02"
    # expert stacks and packed pairs take several loads per parameter: the extended container, not the reference's form
    assert (out / "rank-3.bin").read_bytes()[:8] == b"IFINIT02"
    plan = json.loads((out / "rank-3.init.json").read_text())
    by = {p["name"]: p for p in plan["parameters"]}
    loads = {}
    for l in plan["loads"]:
        loads.setdefault(l["dest"], []).append(l)
    # K-sharded o_proj: strided source rows, 512 local columns of 4096
    o = by["model.layers.0.self_attn.o_proj"]
    assert o["dims"] == [4096, 512]
    (l,) = loads[o["id"]]
    assert l["kind"] == "strided_rows" and l["row_bytes"] == 1024 and l["stride_bytes"] == 8192
    assert l["shard"] == "model.safetensors" and (l["offset"] - 3 * 1024) % 2 == 0
    base_o = l["offset"] - 3 * 1024            # file offset of the tensor: every rank's slice starts rank * 1024 bytes in
    assert json.loads((out / "rank-5.init.json").read_text())["loads"][plan["loads"].index(l)]["offset"] == base_o + 5 * 1024
    # row-sharded q_b: one contiguous slice at rank * rows
    qb = by["model.layers.0.self_attn.q_b_proj"]
    (l,) = loads[qb["id"]]
    assert qb["dims"] == [768, 1536] and l["kind"] == "slice" and l["bytes"] == 768 * 1536 * 2
    l0 = json.loads((out / "rank-0.init.json").read_text())["loads"][plan["loads"].index(l)]
    assert l["offset"] - l0["offset"] == 3 * 768 * 1536 * 2
    # local experts 36..47 of 96, gate and up packed per expert
    gu = by["model.layers.5.mlp.experts.{expert}.gate_proj|model.layers.5.mlp.experts.{expert}.up_proj"]
    assert gu["dims"] == [12, 3072, 4096]
    ts = [l["tensor"] for l in loads[gu["id"]]]
    assert ts[0] == "model.layers.5.mlp.experts.36.gate_proj.weight" and ts[1] == "model.layers.5.mlp.experts.36.up_proj.weight"
    assert ts[-1] == "model.layers.5.mlp.experts.47.up_proj.weight" and len(ts) == 24
    # router weights are widened bf16 -> f32 only if the checkpoint stores bf16; here the synthetic metadata is f32
    assert by["model.layers.0.mlp.gate"]["dtype"] == "f32"
    # the physical inspection plan: one step per instruction, the selected kernel first among its candidates, every
    # all-reduce / gather / argmax exchange numbered in order, a complete analytical cost, nothing executable claimed
    phys = json.loads((out / "physical.json").read_text())
    sched = phys["schedules"][0]
    assert phys["format"] == "inferfabric.physical.v1" and phys["executable"] is False and len(phys["ranks"]) == 8
    assert len(sched["steps"]) == s["instructions"] and sched["cost_complete"] and sched["estimated_serial_ns"] > 500_000
    colls = [st["operation"]["collective"] for st in sched["steps"] if st["operation"]["collective"]]
    assert [c["sequence"] for c in colls] == list(range(len(colls))) and len(colls) == s["collectives_per_token"]
    lin = next(st for st in sched["steps"] if st["operation"]["candidates"][0]["id"] == "ifab_gemv_allreduce_bf16")
    assert lin["selected"] == 0 and lin["operation"]["candidates"][1]["eligible"] is False and "9 or more rows" in lin["operation"]["candidates"][1]["rejection"]
    man = json.loads((out / "serving.json").read_text())
    assert len(man["states"]) == 46 and man["states"][0]["storage"] == {"kind": "pages", "page_tokens": 16, "row_bytes": 1152}
    arena = (out / "arena-rank-0.txt").read_text().split("\n")[0].split()
    assert arena[0] == "IFARENA2" and int(arena[3]) % 512 == 0
    with pytest.raises(compiler.CompileError, match="refusing to overwrite"):
        compiler.write_bundle(FLAGSHIP, out)
    assert not [p for p in tmp_path.iterdir() if "staging" in p.name]


def test_program_variants_select_the_container_version():
    src = SLICE.read_text()
    assert compiler.compile_source(src, resident_sequences=4)["program"]["magic"] == "IFTOKN03"
    assert compiler.compile_source(src, prefill_variants=[2, 4, 8])["program"]["magic"] == "IFTOKN06"
    p = compiler.compile_source(src, prefill_tokens=4096, uncaptured_prefill=True, output_rows=True)["program"]
    assert p["magic"] == "IFTOKN08" and p["options"]["prefill_tokens"] == 4096
    with pytest.raises(compiler.CompileError):
        compiler.compile_source(src, prefill_variants=[8, 4])


@pytest.mark.parametrize("mutate,needle", [
    (lambda s: s.replace("language inferfabric 1;", "language inferfabric 2;"), "language version"),
    (lambda s: s.replace("experts = 16, topk = 4", "experts = 2, topk = 4"), "topk exceeds experts"),
    (lambda s: s.replace("start = 640, width = 64", "start = 700, width = 64"), "slice exceeds"),
    (lambda s: s.replace('placement = "replicated"', 'placement = "diagonal"'), "placement must be"),
    (lambda s: s.replace("eps = 1e-5, theta = 6400000);", "eps = 1e-5, theta = 6400000, bogus = 1);"), "unknown attribute"),
    (lambda s: s.replace("yield logits;", "let dead = add(embedded, embedded);\n    yield logits;"), "does not contribute"),
    (lambda s: s.replace("tp = 1;", "tp = 3;").replace("ep = 1;", "ep = 3;"), "tp must be"),
    (lambda s: s.replace("let h = add(x, attention);", "let h = add(x, DecoderBlock(x, w, window));"), "recursive module"),
    (lambda s: s.replace("range(0, 2)", "range(0, 5000)"), "4096"),
    (lambda s: s.replace("expert.gate_proj, paired", "w.shared_experts.gate_proj, paired"), "must contain {expert}"),
    (lambda s: s.replace("max_model_len = 128", "max_model_len = 256"), "max_model_len"),
])
def test_malformed_sources_are_rejected(mutate, needle):
    with pytest.raises(compiler.CompileError, match=re.escape(needle)):
        compiler.compile_source(mutate(SLICE.read_text()))


def test_cli_roundtrip_and_inspect(tmp_path):
    r = compiler.cli("compile-token", str(SLICE), "-", str(tmp_path / "b"), "--resident-sequences", "2", "--prefill-variants", "2,4,8")
    assert r.returncode == 0, r.stderr
    r = compiler.cli("inspect", str(tmp_path / "b" / "execution.bin"))
    prog = json.loads(r.stdout)
    assert prog["magic"] == "IFTOKN06" and prog["options"]["prefill_variants"] == [2, 4, 8]
    assert json.loads(compiler.cli("inspect", str(tmp_path / "b" / "rank-0.bin")).stdout)["rank"] == 0
    r = compiler.cli("compile-token", str(SLICE), "-", str(tmp_path / "b"))
    assert r.returncode == 1 and "refusing to overwrite" in r.stderr
    assert compiler.cli("demo").returncode == 0


def test_interpreter_matches_pytorch_oracle(tmp_path):
    """Config-1 smoke: the 2-layer hidden-256 slice on a 16-token prompt, C++ interpreter vs the PyTorch restatement."""
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, weights_from_checkpoint
    from ironpangu_b200.models.mla_moe_ref import forward_ref

    ck = tmp_path / "ck"
    assert compiler.cli("synth-checkpoint", str(SLICE), str(ck), "--seed", "0").returncode == 0
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 1024, (16,), generator=g).tolist()
    out = compiler.interpret(SLICE.read_text(), str(ck), prompt, steps=4, logits=True)
    cfg = MlaMoeConfig.tiny(2)
    full = weights_from_checkpoint(cfg, str(ck))
    seq = prompt + out["generated"]          # the oracle is teacher-forced on the interpreter's own tokens
    ref = forward_ref(cfg, full, torch.tensor(seq))
    ref_ids = ref.argmax(-1).tolist()
    got = out["prompt_argmax"][:15] + out["generated"]
    for i, (a, b) in enumerate(zip(got, ref_ids[:19])):
        if a != b:  # only a near-tie may flip
            top2 = ref[i].topk(2).values
            assert float(top2[0] - top2[1]) < 2e-3, (i, a, b)
    torch.testing.assert_close(torch.tensor(out["logits_last"]), ref[19], rtol=2e-2, atol=5e-3)


def test_cli_checkpoint_metadata_verbs(tmp_path):
    """inspect-checkpoint / bind-checkpoint / plan-placement: metadata audits that read no tensor data."""
    ck = tmp_path / "ck"
    assert compiler.cli("synth-checkpoint", str(SLICE), str(ck), "--seed", "0").returncode == 0
    r = compiler.cli("inspect-checkpoint", str(ck), str(tmp_path / "audit.json"))
    assert r.returncode == 0, r.stderr
    audit = json.loads((tmp_path / "audit.json").read_text())
    assert audit["layers"] == 2 and audit["tensors"] == len(audit["tensor_list"]) and audit["bytes"] == sum(t["bytes"] for t in audit["tensor_list"])
    r = compiler.cli("bind-checkpoint", str(SLICE), str(ck))
    bound = json.loads(r.stdout)
    assert r.returncode == 0 and bound["complete"] and bound["bound"] == audit["tensors"] and bound["excluded"] == []
    # a checkpoint that lacks a tensor binds incompletely and says which one
    victim = next(p for p in ck.iterdir() if p.suffix == ".safetensors")
    other = tmp_path / "ck2"
    other.mkdir()
    for p in ck.iterdir():
        if p != victim:
            (other / p.name).write_bytes(p.read_bytes())
    if any(other.iterdir()):
        r = compiler.cli("bind-checkpoint", str(SLICE), str(other))
        assert r.returncode == 1 and json.loads(r.stdout)["missing"]
    place = json.loads(compiler.cli("plan-placement", str(ROOT / "examples" / "mla_moe_92b_tp8.inferfabric"), "-").stdout)
    assert len(place["ranks"]) == 8 and place["executable"] is False
    assert len({r["device_bytes"] for r in place["ranks"]}) == 1 and place["ranks"][0]["strided_slices"] > 0


def test_bundles_pass_the_engine_side_contract_check(tmp_path):
    """validate-bundle / compiler.validate_bundle: kernel contracts of execution.bin and binding contracts of every rank-N.bin;
    a bundle whose program was altered after compilation is refused with the instruction named."""
    out = tmp_path / "b"
    assert compiler.cli("compile-token", str(SLICE), "-", str(out)).returncode == 0
    ok = compiler.validate_bundle(str(out))
    assert ok["valid"] and ok["ranks"] == 1 and ok["instructions"] > 10
    r = compiler.cli("validate-bundle", str(out))
    assert r.returncode == 0 and json.loads(r.stdout)["valid"]
    big = tmp_path / "b8"
    assert compiler.cli("compile-token", str(ROOT / "examples" / "mla_moe_92b_tp8.inferfabric"), "-", str(big)).returncode == 0
    assert compiler.validate_bundle(str(big))["ranks"] == 8
    # swap a kernel name for another of the same length inside the serialized program
    raw = (out / "execution.bin").read_bytes()
    assert b"ifab_router_topk" in raw
    (out / "execution.bin").write_bytes(raw.replace(b"ifab_router_topk", b"ifab_router_topX", 1))
    with pytest.raises(compiler.CompileError, match="router"):
        compiler.validate_bundle(str(out))
    r = compiler.cli("validate-bundle", str(out))
    assert r.returncode == 1 and "kernel contract" in r.stderr
