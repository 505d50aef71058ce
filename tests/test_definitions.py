"""Model definitions: contract documents, the CPU graph target, token graphs and the JSON model artifact."""
import json
import os
from pathlib import Path

import pytest

from ironpangu_b200 import compiler

ROOT = Path(__file__).resolve().parents[1]
SLICE = ROOT / "examples" / "mla_moe_slice_tp1.inferfabric"
# the upstream project's own example documents, when a checkout sits next to this repository (or where the variable points)
REFERENCE_EXAMPLES = Path(os.environ.get("IFAB_REFERENCE_EXAMPLES", ROOT.parent / "reference" / "examples"))

HYBRID = """language inferfabric 1;
model Hybrid {
    contract = %s;
    label = "hybrid-2b";
    hidden = 2048; intermediate = 6144; vocab = 248320;
    query_heads = 8; kv_heads = 2; head_dim = 256;
    delta_heads = 16; delta_dim = 128; conv_width = 4;
    layers = [delta, delta, delta, full, delta, delta, delta, full];
}
plan Local for Hybrid {
    prefill = mesh(tp = 2, cp = %d, sp = %s);
    decode = mesh(tp = 2, cp = 1, sp = false);
    page_tokens = 128; token_budget = 1024;
    batch_buckets = [1, 2, 4, 8];
    context_buckets = [128, 512, 2048];
}
"""


def explain(tmp_path, text, name="m.inferfabric"):
    f = tmp_path / name
    f.write_text(text)
    r = compiler.cli("explain", str(f))
    return r, (json.loads(r.stdout) if r.returncode == 0 else None)


def test_contract_documents_become_specs(tmp_path):
    r, j = explain(tmp_path, HYBRID % ("qwen35_text_v1", 1, "false"))
    assert r.returncode == 0, r.stderr
    assert j == {"kind": "qwen", "checkpoint": True, "model": "hybrid-2b", "layers": 8, "full_attention_layers": 2, "delta_layers": 6,
                 "prefill_ranks": 2, "decode_ranks": 2, "max_context": 2048}
    r, j = explain(tmp_path, HYBRID % ("qwen_structure_v1", 2, "true"))
    assert r.returncode == 0 and j["checkpoint"] is False and j["prefill_ranks"] == 4
    # a structural document compiles straight to per-rank plans: SP gathers / scatters and the CP ring are in them
    f = tmp_path / "d.inferfabric"
    f.write_text(HYBRID % ("qwen_structure_v1", 2, "true"))
    r = compiler.cli("compile", str(f), str(tmp_path / "plans.bin"))
    assert r.returncode == 0, r.stderr
    art = json.loads(r.stdout)
    names = {i["name"] for p in art["plans"] for i in p["instructions"] if i["kind"] == "communication"}
    assert {"all_gather", "reduce_scatter", "send", "receive"} <= names
    assert (tmp_path / "plans.bin").read_bytes()[:8] == b"PANGU\0\0\x01"


@pytest.mark.parametrize("mutate,message", [
    (lambda s: s.replace("qwen35_text_v1", "llama_v9"), "contract llama_v9"),
    (lambda s: s.replace("hidden = 2048;", "hidden = 2048; hidden = 4096;"), "given twice"),
    (lambda s: s.replace("conv_width = 4;", "conv_width = 4; rope_theta = 10;"), "does not know: rope_theta"),
    (lambda s: s.replace("vocab = 248320;", ""), "vocab is missing"),
    (lambda s: s.replace("[delta, delta, delta, full, delta, delta, delta, full]", "[delta, sliding]"), "`full` or `delta`"),
    (lambda s: s.replace("sp = false);\n    decode", "sp = maybe);\n    decode"), "sp is true or false"),
    (lambda s: s.replace("label = \"hybrid-2b\";", "label = \"hybrid-2b\"; let x = add(a, b);"), "fields only"),
    (lambda s: s.replace("query_heads = 8", "query_heads = 7"), "KV groups"),
    (lambda s: s.replace("batch_buckets = [1, 2, 4, 8]", "batch_buckets = [4, 2]"), "ascending"),
])
def test_contract_documents_are_checked(tmp_path, mutate, message):
    r, _ = explain(tmp_path, mutate(HYBRID % ("qwen35_text_v1", 1, "false")))
    assert r.returncode == 1 and message in r.stderr, r.stderr


def test_parallel_only_contract(tmp_path):
    text = """language inferfabric 1;
model Big { contract = openpangu_v2_tp_ep_v1; }
plan Box for Big { tp = 8; ep = 8; devices = [0,1,2,3,4,5,6,7]; max_num_seqs = 4; max_num_batched_tokens = 4096; max_model_len = 65536; }
"""
    r, j = explain(tmp_path, text)
    assert r.returncode == 0, r.stderr
    assert j["kind"] == "open_pangu" and j["parallel"]["tp"] == 8 and j["parallel"]["devices"] == list(range(8))
    r, _ = explain(tmp_path, text.replace("ep = 8", "ep = 4"))
    assert r.returncode == 1
    r, _ = explain(tmp_path, text.replace("[0,1,2,3,4,5,6,7]", "[0,1,2,3,4,5,6,6]"))
    assert r.returncode == 1


def test_model_artifact_round_trip_for_every_kind(tmp_path):
    cpu_graph = """language inferfabric 1;
model Residual { input x: tensor<f32>[2, 2]; const w: tensor<f32>[2, 2] = [1, 0, 0, 1];
  let p = matmul(x, w); let s = add(p, x); let y = relu(s); yield y; }
plan Cpu for Residual { target = cpu_f32_v1; }
"""
    sources = {"qwen": HYBRID % ("qwen35_text_v1", 1, "false"), "graph": cpu_graph, "execution": SLICE.read_text()}
    for kind, text in sources.items():
        src = tmp_path / f"{kind}.inferfabric"
        src.write_text(text)
        art = tmp_path / f"{kind}.json"
        r = compiler.cli("compile-model", str(src), str(art))
        assert r.returncode == 0, r.stderr
        doc = json.loads(art.read_text())
        assert doc["format"] == "inferfabric.model" and doc["version"] == 1 and doc["definition"]["kind"] == kind
        # the artifact is accepted wherever a document is, and means the same
        a, b = compiler.cli("explain", str(src)), compiler.cli("explain", str(art))
        assert a.returncode == 0 and b.returncode == 0 and json.loads(a.stdout) == json.loads(b.stdout), b.stderr
        # and it is stable: compiling the artifact gives the artifact
        again = compiler.cli("compile-model", str(art))
        assert again.returncode == 0 and json.loads(again.stdout) == doc


def test_model_artifact_is_not_trusted(tmp_path):
    src = tmp_path / "q.inferfabric"
    src.write_text(HYBRID % ("qwen_structure_v1", 1, "false"))
    doc = json.loads(compiler.cli("compile-model", str(src)).stdout)

    def refused(d, text=None):
        f = tmp_path / "bad.json"
        f.write_text(text if text is not None else json.dumps(d))
        r = compiler.cli("explain", str(f))
        assert r.returncode == 1, r.stdout
        return r.stderr

    assert "version 1" in refused({**doc, "version": 2})
    assert "version 1" in refused({**doc, "format": "inferfabric.modle"})
    assert "unknown field" in refused({**doc, "extra": 1})
    bad = json.loads(json.dumps(doc))
    bad["definition"]["spec"]["decode"]["cp"] = 2              # decode runs with CP = 1: validation applies to artifacts too
    assert "CP = 1" in refused(bad)
    bad = json.loads(json.dumps(doc))
    bad["definition"]["kind"] = "transformer"
    assert "unknown definition kind" in refused(bad)
    bad = json.loads(json.dumps(doc))
    bad["definition"]["hook"] = "os.system"
    assert "unknown field hook" in refused(bad)
    assert "larger than the limit" in refused(None, "{" + " " * (17 << 20) + "}")       # the 16 MiB bound of an artifact
    # a token-graph artifact whose node list was edited is re-checked by the type checker
    ex = tmp_path / "s.json"
    assert compiler.cli("compile-model", str(SLICE), str(ex)).returncode == 0
    g = json.loads(ex.read_text())
    g["definition"]["graph"]["nodes"][3]["inputs"] = [9999]
    assert "not defined earlier" in refused(g)


@pytest.mark.skipif(not REFERENCE_EXAMPLES.is_dir(), reason="no checkout of the upstream examples next to this repository")
def test_upstream_example_documents_compile_unchanged(tmp_path):
    """Every `.inferfabric` document the upstream project ships compiles here unchanged, with the structure its own tests pin."""
    docs = sorted(REFERENCE_EXAMPLES.rglob("*.inferfabric"))
    assert len(docs) >= 9
    facts = {}
    for d in docs:
        r = compiler.cli("explain", str(d))
        assert r.returncode == 0, (d.name, r.stderr)
        facts[d.name] = json.loads(r.stdout)
    for name in ("92b-tp8-ep8.inferfabric", "92b-tp8-ep8-c8.inferfabric"):
        f = facts[name]
        assert f["logical_nodes"] == 1701 and f["logical_ops"]["allreduce"] == 92 and f["parallel"]["tp"] == 8 and f["parallel"]["ep"] == 8
    for name in ("92b-tp8-ep8-c8-learned.inferfabric", "92b-tp8-ep8-c8-serving.inferfabric"):
        f = facts[name]
        assert f["logical_ops"]["allreduce"] == 92 and f["logical_ops"]["sparse_index"] == 8 and f["logical_ops"]["index_cache_append"] == 8
    assert facts["qwen35-2b-tp2.inferfabric"] == {"kind": "qwen", "checkpoint": True, "model": "Qwen3.5-2B-text", "layers": 24,
                                                  "full_attention_layers": 6, "delta_layers": 18, "prefill_ranks": 2, "decode_ranks": 2,
                                                  "max_context": 8192}
    assert facts["qwen35-2b-distributed.inferfabric"]["prefill_ranks"] == 4 and facts["residual.inferfabric"]["kind"] == "graph"
    # the 92B document as a bundle: 8 rank plans, K-sharded weights as strided source rows (stride = 8 x row), 46 x 4 serving states
    out = tmp_path / "bundle"
    r = compiler.cli("compile-token", str(REFERENCE_EXAMPLES / "openpangu" / "92b-tp8-ep8.inferfabric"), "-", str(out))
    assert r.returncode == 0, r.stderr
    assert len(list(out.glob("rank-*.bin"))) == 8
    plan = json.loads((out / "rank-3.init.json").read_text())
    strided = [l for l in plan["loads"] if l["kind"] == "strided_rows"]
    assert strided and all(l["stride_bytes"] == 8 * l["row_bytes"] for l in strided)
    man = json.loads((out / "serving.json").read_text())
    assert len(man["states"]) == 46 * 4
    with pytest.raises(Exception):
        compiler.write_bundle(REFERENCE_EXAMPLES / "openpangu" / "92b-tp8-ep8.inferfabric", out)     # refuses to overwrite
