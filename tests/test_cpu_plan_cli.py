"""CPU f32 planner verbs: stage dumps, kernel overrides (`tune-plan`), the HTML view of a plan."""
import json

from ironpangu_b200 import compiler

GRAPH = {
    "version": 1,
    "name": "mlp",
    "inputs": [{"name": "x", "shape": [4, 64]}],
    "constants": [{"name": "w1", "shape": [64, 64], "data": [0.01 * ((i * 7) % 13 - 6) for i in range(64 * 64)]},
                  {"name": "a", "shape": [2, 2], "data": [1, 2, 3, 4]}, {"name": "b", "shape": [2, 2], "data": [1, 1, 1, 1]}],
    "states": [],
    "nodes": [{"name": "h", "op": "matmul", "inputs": ["x", "w1"]}, {"name": "r", "op": "relu", "inputs": ["h"]},
              {"name": "y", "op": "add", "inputs": ["r", "x"]}, {"name": "folded", "op": "add", "inputs": ["a", "b"]},
              {"name": "dead", "op": "relu", "inputs": ["x"]}],
    "outputs": ["y", "folded"],
    "updates": {},
}


def test_stage_dumps_tuning_and_html(tmp_path):
    g, plan, ir = tmp_path / "g.json", tmp_path / "p.ifplan", tmp_path / "ir"
    g.write_text(json.dumps(GRAPH))
    r = compiler.cli("plan", str(g), str(plan), "--dump-ir", str(ir))
    assert r.returncode == 0, r.stderr
    assert sorted(p.name for p in ir.iterdir()) == ["00-logical.json", "01-typed.json", "02-optimized.json", "03-physical.json", "04-bundle-manifest.json"]
    typed, opt, phys = (json.loads((ir / n).read_text()) for n in ("01-typed.json", "02-optimized.json", "03-physical.json"))
    assert [n["name"] for n in typed["nodes"]] == ["h", "r", "y", "folded", "dead"]
    assert {v["name"]: v["shape"] for v in typed["values"]}["h"] == [4, 64]
    assert [n["name"] for n in opt["nodes"]] == ["h", "r", "y"] and opt["folded_constants"] == 1 and opt["eliminated_nodes"] == 1
    assert [s["name"] for s in phys["steps"]] == ["h", "r", "y"] and phys["steps"][0]["kernel"] == "MatmulBlockedF32V1"
    assert json.loads((ir / "04-bundle-manifest.json").read_text())["body_bytes"] > 0
    # tune: the matmul forced to the naive kernel; same results from both plans
    over, tuned = tmp_path / "o.json", tmp_path / "t.ifplan"
    over.write_text(json.dumps({"h": "MatmulNaiveF32V1"}))
    r = compiler.cli("tune-plan", str(plan), str(over), str(tuned))
    assert r.returncode == 0, r.stderr
    t = json.loads(r.stdout)
    assert t["steps"][0]["kernel"] == "MatmulNaiveF32V1" and t["steps"][0]["selection_reason"] == "forced by override"
    assert [b.get("offset") for b in t["buffers"]] == [b.get("offset") for b in phys["buffers"]]
    over.write_text(json.dumps({"h": "AddF32V1"}))
    r = compiler.cli("tune-plan", str(plan), str(over), str(tmp_path / "bad.ifplan"))
    assert r.returncode != 0 and "does not implement" in r.stderr
    over.write_text(json.dumps({"nope": "AddF32V1"}))
    assert "no step named" in compiler.cli("tune-plan", str(plan), str(over), str(tmp_path / "bad.ifplan")).stderr
    # the HTML view of the encoded plan
    page = tmp_path / "p.html"
    r = compiler.cli("explain-plan", str(tuned), "--html", str(page))
    assert r.returncode == 0, r.stderr
    html = page.read_text()
    assert html.startswith("<!doctype html>") and "MatmulNaiveF32V1" in html and "forced by override" in html
    assert html.count("<tr><td>") == len(t["steps"]) + len(t["buffers"])
