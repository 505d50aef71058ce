"""Host-core path of a hyper-connected model (mHC modules, token convolutions, attention sinks): the parameters of those operators
are planned from the checkpoint, the bundle passes its contracts, and the lowering keeps the mixed streams alive until the branch
returns."""
import json

import pytest

from hyper_source import source
from ironpangu_b200 import compiler


def _compiled(tmp_path, **kw):
    src, ck, bundle = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "b"
    src.write_text(source(**kw))
    r = compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "3")
    assert r.returncode == 0, r.stderr
    compiler.write_bundle(str(src), str(bundle), checkpoint_dir=str(ck), prefill_tokens=8)
    return src, ck, bundle


@pytest.mark.parametrize("tp", [1, 2])
def test_parameters_of_hyper_connection_convolution_and_sinks_are_planned(tmp_path, tp):
    src, ck, bundle = _compiled(tmp_path, layers=1, tp=tp)
    assert compiler.validate_bundle(str(bundle))["valid"]
    for rank in range(tp):
        plan = json.loads((bundle / f"rank-{rank}.init.json").read_text())
        P = {p["name"]: p for p in plan["parameters"]}
        m = "model.layers.0."
        assert P[m + "attn_mhc.phi"]["dims"] == [24, 1024] and P[m + "attn_mhc.phi"]["dtype"] == "f32"
        assert P[m + "attn_mhc.gamma"]["dims"] == [1024] and P[m + "attn_mhc.alpha"]["dims"] == [3] and P[m + "attn_mhc.beta"]["dims"] == [24]
        assert P["model.merge_mhc.phi"]["dims"] == [24, 1024]
        # depthwise taps load as [channels, taps]; a rank that convolves its own channel range still holds every channel's taps
        assert P[m + "attn.qa_conv"]["dims"] == [384, 3] and P[m + "attn.kv_conv"]["dims"] == [512, 3] and P[m + "attn.o_conv"]["dims"] == [512, 3]
        assert P[m + "attn.qa_conv"]["dtype"] == "f32"
        assert P[m + "attn.param_sink_compressed_kv"]["dims"] == [5, 512] and P[m + "attn.param_sink_k_pe"]["dims"] == [5, 64]
        assert m + "block_norm" not in P                    # optional, absent from the checkpoint


def test_lowering_keeps_the_mixed_streams_alive_for_the_return_of_the_branch(tmp_path):
    src, ck, bundle = _compiled(tmp_path, layers=2)
    prog = json.loads((bundle / "device-program.json").read_text())
    ins = prog["instructions"]
    posts = [i for i in ins if i["op"] == "mhc_post"]
    assert len(posts) == 4
    for p in posts:
        hc, branch, streams = p["inputs"]
        assert ins[hc]["op"] == "mhc_pre" and ins[hc]["inputs"] == [streams] and ins[streams]["width"] == p["width"]
    # the arena therefore never hands the streams' slot to an instruction between the module and its return
    arena = (bundle / "arena-rank-0.txt").read_text().split("\n")
    n = int(arena[0].split()[4])
    slots = {}
    for i in range(n):
        off, size = (int(x) for x in arena[1 + i].split())
        owner, first, last = (int(x) for x in arena[2 + n + i].split())
        slots[owner] = (off, size, first, last)
    for k, p in enumerate(ins):
        if p["op"] != "mhc_post":
            continue
        streams = p["inputs"][2]
        while streams not in slots and ins[streams]["op"] == "optional_norm":
            streams = ins[streams]["inputs"][0]       # a norm the checkpoint lacks hands its source's slot on
        s_off, s_size, _, s_last = slots[streams]
        assert s_last >= k
        for owner, (off, size, first, last) in slots.items():
            if owner != streams and p["inputs"][0] <= owner < k:
                assert off + size <= s_off or s_off + s_size <= off, (owner, k)


def test_an_optional_norm_the_checkpoint_lacks_gets_no_slot_and_keeps_its_source_alive(tmp_path):
    src, ck, bundle = _compiled(tmp_path, layers=2)
    ins = json.loads((bundle / "device-program.json").read_text())["instructions"]
    arena = (bundle / "arena-rank-0.txt").read_text().split("\n")
    n = int(arena[0].split()[4])
    live = {int(l.split()[0]): (int(l.split()[1]), int(l.split()[2])) for l in arena[2 + n:2 + 2 * n]}
    users = {}
    for k, i in enumerate(ins):
        for j in i["inputs"]:
            users.setdefault(j, []).append(k)
    optional = [k for k, i in enumerate(ins) if i["op"] == "optional_norm"]
    assert len(optional) == 2
    for k in optional:
        assert k not in live
        assert live[ins[k]["inputs"][0]][1] >= max(users[k])


def test_sink_rows_must_come_from_a_sink_normalize(tmp_path):
    text = source(layers=1).replace("cache_norm_rope_append(kc, kr, sinks,", "cache_norm_rope_append(kc, kr, kc,")
    src = tmp_path / "bad.inferfabric"
    src.write_text(text)
    with pytest.raises(compiler.CompileError):
        compiler.write_bundle(str(src), str(tmp_path / "b"))


def test_interpreter_runs_the_model_and_sinks_and_history_matter(tmp_path):
    src, ck, _ = _compiled(tmp_path, layers=1)
    toks = [5, 17, 99, 3, 64]
    a = compiler.interpret(src.read_text(), str(ck), toks, all_logits=True)["prompt_logits"]
    assert len(a) == 5 and all(abs(v) < 50 for row in a for v in row)
    # the same token at two positions sees a different convolution history and a longer context
    b = compiler.interpret(src.read_text(), str(ck), [5, 5, 5], all_logits=True)["prompt_logits"]
    assert max(abs(x - y) for x, y in zip(b[0], b[2])) > 1e-3
    # without sinks the first position attends to itself only; with sinks it does not
    no_sinks = tmp_path / "nosinks.inferfabric"
    text = source(layers=1).replace("cache_norm_rope_append(kc, kr, sinks,", "cache_norm_rope_append(kc, kr,")
    no_sinks.write_text("\n".join(l for l in text.split("\n") if "sink_normalize" not in l))        # an unused node is an error
    c = compiler.interpret(no_sinks.read_text(), str(ck), toks[:1], all_logits=True)["prompt_logits"]
    assert max(abs(x - y) for x, y in zip(a[0], c[0])) > 1e-4
