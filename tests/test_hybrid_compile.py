"""Checkpoint-bound compile path of the hybrid (gated-delta + full-attention) decoder family, on a small synthetic checkpoint."""
import json
import struct
from pathlib import Path

import pytest

from ironpangu_b200 import compiler

LAYERS = ["delta", "delta", "delta", "full"] * 2
DOC = """language inferfabric 1;
model Small {
    contract = qwen35_text_v1;
    label = "hybrid-small";
    hidden = 64; intermediate = 96; vocab = 320;
    query_heads = 4; kv_heads = 2; head_dim = 32;
    delta_heads = 4; delta_dim = 16; conv_width = 4;
    layers = [%s];
}
plan Local for Small {
    prefill = mesh(tp = %d, cp = 1, sp = false);
    decode = mesh(tp = %d, cp = 1, sp = false);
    page_tokens = 16; token_budget = 64;
    batch_buckets = [1, 2, 4];
    context_buckets = [128, 512];
}
"""


def schema():
    H, I, V, qh, kvh, hd, dh, dd, cw = 64, 96, 320, 4, 2, 32, 4, 16, 4
    s = {"embed_tokens.weight": ("BF16", [V, H]), "norm.weight": ("BF16", [H])}
    for i, kind in enumerate(LAYERS):
        p = f"layers.{i}."
        s[p + "input_layernorm.weight"] = ("BF16", [H])
        s[p + "post_attention_layernorm.weight"] = ("BF16", [H])
        s[p + "mlp.gate_proj.weight"] = ("BF16", [I, H])
        s[p + "mlp.up_proj.weight"] = ("BF16", [I, H])
        s[p + "mlp.down_proj.weight"] = ("BF16", [H, I])
        if kind == "full":
            s[p + "self_attn.q_norm.weight"] = ("BF16", [hd])
            s[p + "self_attn.k_norm.weight"] = ("BF16", [hd])
            s[p + "self_attn.q_proj.weight"] = ("BF16", [2 * qh * hd, H])
            s[p + "self_attn.k_proj.weight"] = ("BF16", [kvh * hd, H])
            s[p + "self_attn.v_proj.weight"] = ("BF16", [kvh * hd, H])
            s[p + "self_attn.o_proj.weight"] = ("BF16", [H, qh * hd])
        else:
            s[p + "linear_attn.A_log"] = ("F32", [dh])
            s[p + "linear_attn.norm.weight"] = ("F32", [dd])
            s[p + "linear_attn.dt_bias"] = ("BF16", [dh])
            s[p + "linear_attn.conv1d.weight"] = ("BF16", [3 * dh * dd, 1, cw])
            s[p + "linear_attn.in_proj_a.weight"] = ("BF16", [dh, H])
            s[p + "linear_attn.in_proj_b.weight"] = ("BF16", [dh, H])
            s[p + "linear_attn.in_proj_qkv.weight"] = ("BF16", [3 * dh * dd, H])
            s[p + "linear_attn.in_proj_z.weight"] = ("BF16", [dh * dd, H])
            s[p + "linear_attn.out_proj.weight"] = ("BF16", [H, dh * dd])
    return {"model.language_model." + k: v for k, v in s.items()}


def write_shard(path: Path, tensors: dict, gap: int = 0, trailing: int = 0):
    hdr, cursor = {}, 0
    for name, (dt, shape) in tensors.items():
        n = (2 if dt == "BF16" else 4)
        for d in shape:
            n *= d
        hdr[name] = {"dtype": dt, "shape": shape, "data_offsets": [cursor + gap, cursor + gap + n]}
        cursor += n + gap
        gap = 0
    blob = json.dumps(hdr).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + bytes(cursor + trailing))
    return cursor


def config(**over):
    t = {"model_type": "qwen3_5_text", "hidden_size": 64, "intermediate_size": 96, "vocab_size": 320, "num_hidden_layers": 8,
         "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 32, "linear_num_key_heads": 4, "linear_num_value_heads": 4,
         "linear_key_head_dim": 16, "linear_value_head_dim": 16, "linear_conv_kernel_dim": 4, "attention_bias": False,
         "attn_output_gate": True, "hidden_act": "silu", "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
         "max_position_embeddings": 4096, "rope_parameters": {"rope_type": "default", "rope_theta": 10000000.0, "partial_rotary_factor": 0.25},
         "layer_types": ["full_attention" if k == "full" else "linear_attention" for k in LAYERS]}
    t.update(over)
    return {"model_type": "qwen3_5", "tie_word_embeddings": True, "text_config": t}


def make_checkpoint(d: Path, *, extra=None, cfg=None, drop=None, two_shards=True, **shard_kw):
    d.mkdir()
    tensors = schema()
    if drop:
        tensors.pop("model.language_model." + drop)
    if extra:
        tensors.update(extra)
    names = list(tensors)
    parts = [names[: len(names) // 2], names[len(names) // 2:]] if two_shards else [names]
    wmap, total = {}, 0
    for i, part in enumerate(parts):
        fname = f"model-{i + 1:05d}-of-{len(parts):05d}.safetensors"
        total += write_shard(d / fname, {n: tensors[n] for n in part}, **(shard_kw if i == 0 else {}))
        wmap.update({n: fname for n in part})
    (d / "config.json").write_text(json.dumps(cfg or config()))
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": wmap}))
    return d


def doc(tmp_path, tp=1, layers=LAYERS):
    f = tmp_path / f"small-tp{tp}.inferfabric"
    f.write_text(DOC % (", ".join(layers), tp, tp))
    return str(f)


def test_inspect_compile_lower(tmp_path):
    ck = make_checkpoint(tmp_path / "ck", extra={"model.visual.patch.weight": ("BF16", [8, 8]), "mtp.head.weight": ("BF16", [4])})
    r = compiler.cli("inspect-hybrid-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 0, r.stderr
    meta = json.loads(r.stdout)
    assert len(meta["weights"]) == len(schema()) and meta["excluded"] == {"mtp": 1, "vision": 1} and len(meta["shards"]) == 2
    w = meta["weights"]["model.language_model.layers.3.self_attn.q_proj.weight"]
    assert w["shape"] == [256, 64] and w["bytes"] == 256 * 64 * 2 and w["offset"] > 8          # absolute file offsets, header included
    r = compiler.cli("compile-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 0, r.stderr
    plan = json.loads(r.stdout)
    assert plan["format"] == "inferfabric.typed-plan.v1" and plan["executable"] is False and len(plan["key"]) == 64
    ops = {}
    for n in plan["nodes"]:
        ops[n["op"]] = ops.get(n["op"], 0) + 1
    # 6 delta layers and 2 full-attention layers, each with its MLP; one embedding, one frontier select, the tied head
    assert ops["DeltaRecurrence"] == 6 and ops["CausalConvSilu"] == 6 and ops["GatedRms"] == 6 and ops["PagedAttention"] == 2
    assert ops["TextRope"] == 4 and ops["Embedding"] == 1 and ops["SelectFrontier"] == 1 and ops["Add"] == 16
    assert ops["Linear"] == 6 * 5 + 2 * 4 + 8 * 3 + 1
    kinds = [s["kind"] for s in plan["states"]]
    assert kinds.count("delta_key_value") == 6 and kinds.count("conv_previous_inputs") == 6 and kinds.count("paged_keys") == 2
    assert all(s["initially_zero"] == (s["kind"] in ("delta_key_value", "conv_previous_inputs")) for s in plan["states"])
    rope = next(n for n in plan["nodes"] if n["op"] == "TextRope")["attrs"]
    assert rope["rotary_dim"] == "8" and rope["interleaved_sections"] == "2,2,0"
    assert plan["recurrent_and_conv_bytes_per_request"] == 6 * (4 * 16 * 16 * 4 + 192 * 3 * 2)
    assert plan["kv_bytes_per_page"] == 2 * 2 * 16 * 2 * 32 * 2
    assert plan["inputs"][4]["shape"] == ["requests", 32]                                        # 512 / 16 pages per request
    # the same inputs give the same key; another context bucket list gives another
    assert json.loads(compiler.cli("compile-checkpoint", doc(tmp_path), str(ck)).stdout)["key"] == plan["key"]
    r = compiler.cli("lower-checkpoint", doc(tmp_path), str(ck), "512", "4")
    assert r.returncode == 0, r.stderr
    prog = json.loads(r.stdout)
    assert prog["batch"] == 4 and prog["context"] == 512 and prog["source_key"] == plan["key"] and len(prog["blocks"]) == 8
    b3 = {b["name"].split("layers.3.")[1]: b["transform"] for b in prog["blocks"][3]["bindings"]}
    assert prog["blocks"][3]["kind"] == "full" and b3["self_attn.q_norm.weight"] == "one_plus_fp32" and b3["self_attn.q_proj.weight"] == "identity"
    b0 = {b["name"].split("layers.0.")[1]: b["transform"] for b in prog["blocks"][0]["bindings"]}
    assert b0["input_layernorm.weight"] == "one_plus_fp32" and b0["linear_attn.norm.weight"] == "identity" and len(b0) == 14
    assert prog["final_norm"]["transform"] == "one_plus_fp32"
    assert compiler.cli("lower-checkpoint", doc(tmp_path), str(ck), "300").returncode == 1      # not a declared bucket
    assert compiler.cli("lower-checkpoint", doc(tmp_path), str(ck), "512", "65").returncode == 1


@pytest.mark.parametrize("how,message", [
    (dict(drop="layers.2.linear_attn.A_log"), "lacks model.language_model.layers.2.linear_attn.A_log"),
    (dict(extra={"model.language_model.layers.0.mlp.bias": ("BF16", [4])}), "does not know"),
    (dict(cfg=config(hidden_size=128)), "hidden_size disagrees"),
    (dict(cfg=config(attn_output_gate=False)), "attn_output_gate"),
    (dict(cfg=config(layer_types=["full_attention"] * 8)), "layer_types[0]"),
    (dict(gap=16), "overlap or leave a gap"),
    (dict(trailing=8), "not described by the header"),
])
def test_checkpoint_metadata_is_checked(tmp_path, how, message):
    ck = make_checkpoint(tmp_path / "ck", **how)
    r = compiler.cli("inspect-hybrid-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 1 and message in r.stderr, r.stderr


def test_index_and_files_are_checked(tmp_path):
    ck = make_checkpoint(tmp_path / "a")
    idx = json.loads((ck / "model.safetensors.index.json").read_text())
    idx["metadata"]["total_size"] += 2
    (ck / "model.safetensors.index.json").write_text(json.dumps(idx))
    r = compiler.cli("inspect-hybrid-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 1 and "total_size" in r.stderr
    ck = make_checkpoint(tmp_path / "b")
    idx = json.loads((ck / "model.safetensors.index.json").read_text())
    first = next(iter(idx["weight_map"]))
    idx["weight_map"][first] = "../b/model-00002-of-00002.safetensors"
    (ck / "model.safetensors.index.json").write_text(json.dumps(idx))
    r = compiler.cli("inspect-hybrid-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 1 and "not a plain name" in r.stderr
    ck = make_checkpoint(tmp_path / "c")
    idx = json.loads((ck / "model.safetensors.index.json").read_text())
    names = list(idx["weight_map"])
    idx["weight_map"][names[0]], idx["weight_map"][names[-1]] = idx["weight_map"][names[-1]], idx["weight_map"][names[0]]
    (ck / "model.safetensors.index.json").write_text(json.dumps(idx))
    r = compiler.cli("inspect-hybrid-checkpoint", doc(tmp_path), str(ck))
    assert r.returncode == 1 and "index says otherwise" in r.stderr


def test_contract_and_parallel_limits(tmp_path):
    ck = make_checkpoint(tmp_path / "ck")
    assert compiler.cli("compile-checkpoint", doc(tmp_path, tp=2), str(ck)).returncode == 0
    r = compiler.cli("compile-checkpoint", doc(tmp_path, tp=4), str(ck))
    assert r.returncode == 1 and "TP 1 or 2" in r.stderr
    structural = tmp_path / "s.inferfabric"
    structural.write_text((DOC % (", ".join(LAYERS), 1, 1)).replace("qwen35_text_v1", "qwen_structure_v1"))
    r = compiler.cli("compile-checkpoint", str(structural), str(ck))
    assert r.returncode == 1 and "qwen35_text_v1" in r.stderr
    # another layer schedule in the document than in the checkpoint's config
    r = compiler.cli("compile-checkpoint", doc(tmp_path, layers=["full"] * 8), str(ck))
    assert r.returncode == 1


def test_typed_plan_viewer(tmp_path):
    """`explain-model PLAN.json --html OUT.html`: one table per layer, every operator and state of the plan on the page."""
    ck = make_checkpoint(tmp_path / "ck")
    plan_path, page = tmp_path / "plan.json", tmp_path / "model.html"
    assert compiler.cli("compile-checkpoint", doc(tmp_path), str(ck), str(plan_path)).returncode == 0
    r = compiler.cli("explain-model", str(plan_path), "--html", str(page))
    assert r.returncode == 0, r.stderr
    plan = json.loads(plan_path.read_text())
    assert f"{len(plan['nodes'])} operators" in r.stdout and "8 layers" in r.stdout
    html = page.read_text()
    assert html.startswith("<!doctype html>") and html.count('<table class="layer">') == 9          # the input + 8 layers
    for op in ("DeltaRecurrence", "PagedAttention", "GatedRms", "CausalConvSilu", "SelectFrontier"):
        assert html.count(f"<td>{op}</td>") == sum(1 for n in plan["nodes"] if n["op"] == op)
    assert "layer.3.keys" in html and "S *= exp(g)" in html and "&lt;" not in plan["key"]
    # a document of another format is refused
    other = tmp_path / "other.json"
    other.write_text(json.dumps({"format": "something.else"}))
    r = compiler.cli("explain-model", str(other), "--html", str(tmp_path / "x.html"))
    assert r.returncode != 0 and "not a typed plan" in r.stderr
