"""Reference comparison: cases from the CPU oracle, the engine under test behind ifab-server (here the program engine on the
host), exact agreement; a doctored reference shows up as a first difference with the oracle's logit gap."""
import json
import os
import subprocess

from ironpangu_b200.utils import compare_reference as CR

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_program_engine_matches_the_oracle_and_differences_are_analysed(tmp_path):
    from ironpangu_b200 import _build, compiler

    src = os.path.join(ROOT, "examples", "mla_moe_slice_tp1.inferfabric")
    ckpt, bundle, cases, report = tmp_path / "ckpt", tmp_path / "bundle", tmp_path / "cases.json", tmp_path / "report.json"
    assert compiler.cli("synth-checkpoint", src, str(ckpt)).returncode == 0
    assert compiler.cli("compile-token", src, str(ckpt), str(bundle), "--resident-sequences", "2", "--prefill-tokens", "8").returncode == 0
    assert CR.main(["make-reference", src, str(ckpt), str(cases), "--prompts", "2", "--prompt-tokens", "6", "--new-tokens", "4"]) == 0
    ref = json.loads(cases.read_text())
    assert len(ref) == 2 and all(len(c["output_ids"]) == 4 and len(c["logits_top"]) == 4 for c in ref)
    assert all(str(c["output_ids"][i]) == max(c["logits_top"][i], key=c["logits_top"][i].get) for c in ref for i in range(4))
    _build.build_core()
    proc = subprocess.Popen([str(_build.SERVER_BIN), "--port", "0", "--program", str(bundle), str(ckpt), "--cpu"], stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True)
    try:
        port = None
        for line in proc.stdout:
            if line.startswith("listening on"):
                port = int(line.rsplit(":", 1)[1])
                break
        assert port
        url = f"http://127.0.0.1:{port}"
        assert CR.main(["compare", str(cases), url, str(report), "--repetitions", "2"]) == 0
        rep = json.loads(report.read_text())
        assert rep["format"] == "ifab.reference-comparison.v1" and rep["passed"]
        assert all(c["exact_all_tokens"] and c["stable_repetitions"] and c["first_difference"] is None and c["ttft_ms_mean"] > 0 for c in rep["cases"])
        # a reference whose third token is the oracle's runner-up: reported as a difference with the (positive) logit gap
        top = ref[0]["logits_top"][2]
        runner_up = sorted(top, key=top.get)[-2]
        ref[0]["output_ids"][2] = int(runner_up)
        cases.write_text(json.dumps(ref))
        rc = CR.main(["compare", str(cases), url, str(tmp_path / "r2.json"), "--repetitions", "1", "--noise", "0"])
        d = json.loads((tmp_path / "r2.json").read_text())["cases"][0]["first_difference"]
        assert d["output_index"] == 2 and d["expected_token"] == int(runner_up) and d["matching_prefix_tokens"] == 2
        assert d["oracle_logit_gap"] < 0 and rc == 0       # the engine's token scores HIGHER than the doctored one: within any noise
    finally:
        proc.terminate()
        proc.wait(timeout=30)
