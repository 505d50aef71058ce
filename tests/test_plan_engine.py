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
    compiler.write_bundle(SLICE, bundle, checkpoint_dir=str(ck), prefill_tokens=8)      # the arena is planned for 8 query rows
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1024, (16,), generator=g).tolist()
    first = compiler.interpret(SLICE.read_text(), str(ck), prompt, steps=8)
    seq = prompt + first["generated"]
    oracle = compiler.interpret(SLICE.read_text(), str(ck), seq, all_logits=True)
    ref = torch.tensor(oracle["prompt_logits"])

    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, keep_logits=True)
    drv = DecodeEngine(eng)
    # activations live in the bundle's frozen arena: one block of the planned size, every result a view at its planned offset
    assert eng.arena.tokens == 8 and eng.arena.block.numel() == eng.arena.bytes + eng.arena.workspace_bytes
    base, end = eng.arena.block.data_ptr(), eng.arena.block.data_ptr() + eng.arena.block.numel()
    for k, v in enumerate(eng.vals):
        for t in (v if isinstance(v, tuple) else (v,)):
            if isinstance(t, torch.Tensor) and t is not eng.next_ids:
                assert base <= t.data_ptr() < end and (t.data_ptr() - base) % 4 == 0, k
    assert base + eng.arena.bytes <= eng.scratch.data_ptr() < end
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
    # engine API: greedy generation through prefill chunks + captured decode graph; once the graph exists a step allocates nothing
    eng.reset()
    out = drv.generate(prompt, 8)
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    tok = out[-1]
    for _ in range(4):
        tok = drv.step(tok)
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    assert len(out) == 8 and all(0 <= t < 1024 for t in out)
    if all(float(ref[15 + i].topk(2).values.diff().abs()) > 1e-2 for i in range(8)):
        assert out == first["generated"]
    assert fab.status() == 0
    fab.close()


def test_arena_is_enforced(tmp_path):
    """A bundle whose arena was planned for fewer rows than the engine runs, or whose arena file belongs to another program, is
    refused before anything runs; a lease larger than its slot is refused too."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import FrozenArena, PlanEngine

    ck, small, other = tmp_path / "ck", tmp_path / "small", tmp_path / "other"
    assert compiler.cli("synth-checkpoint", str(SLICE), str(ck), "--seed", "3").returncode == 0
    compiler.write_bundle(SLICE, small, checkpoint_dir=str(ck))                     # one query row
    fab = Fabric(0, 1)
    with pytest.raises(ValueError, match="planned for 1 query rows"):
        PlanEngine(str(small), str(ck), fab, max_tokens=8)
    eng = PlanEngine(str(small), str(ck), fab, max_tokens=1)
    with pytest.raises(RuntimeError, match="leased its arena slot twice"):
        eng.arena.lease(next(iter(eng.arena.leased)), 16)
    free = [k for k in eng.arena.slots if k not in eng.arena.leased]
    if free:
        with pytest.raises(RuntimeError, match="arena slot holds"):
            eng.arena.lease(free[0], eng.arena.slots[free[0]][1] + 512)
    with pytest.raises(RuntimeError, match="workspace"):
        eng.arena.workspace(eng.arena.workspace_bytes + 1)
    compiler.write_bundle(SLICE, other, checkpoint_dir=str(ck), resident_sequences=2)   # another program variant
    (small / "arena-rank-0.txt").write_text((other / "arena-rank-0.txt").read_text())
    with pytest.raises(ValueError, match="another program"):
        FrozenArena(small, 0, 1, "cuda")
    fab.close()


@pytest.mark.parametrize("fused_head,fused_moe", [(None, None), (False, False), (True, True)])
def test_bundle_engine_equals_the_hand_wired_decoder(tmp_path, fused_head, fused_moe):
    """The generated source, compiled, run by the plan engine on adopted weights: bit-identical logits and tokens to the
    decoder class that wires the same kernels by hand, for every dispatcher choice; the prompt executor and the single-sequence
    engine run on the bundle's engine through its decoder attributes."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, bundle_parameters, random_rank_weights
    from ironpangu_b200.models.mla_moe_prefill import MlaMoePrefill
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.engine import DecodeEngine
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = MlaMoeConfig.tiny(layers=3)
    dev = torch.device("cuda", 0)
    weights = random_rank_weights(cfg, 0, 1, dev, seed=5)
    src = tmp_path / "m.inferfabric"
    src.write_text(mla_moe_source(cfg, 1, context=256))
    out = compiler.write_bundle(str(src), str(tmp_path / "b"), prefill_tokens=8)
    fab = Fabric(0, 1)
    eng = PlanEngine(out["dir"], None, fab, max_tokens=8, keep_logits=True, parameters=bundle_parameters(cfg, weights),
                     fused_head=fused_head, fused_moe=fused_moe)
    ref = MlaMoeDecoder(cfg, weights, fab, max_tokens=8, max_context=256, keep_logits=True, fused_head=fused_head, fused_moe=fused_moe)
    import dataclasses
    assert eng.cfg == dataclasses.replace(cfg, eos=2) and eng.hl == ref.hl and eng.el == ref.el and len(eng.caches) == cfg.layers
    assert eng.launches_per_forward == ref.launches_per_forward
    assert eng.fused_head == ref.fused_head and eng.fused_moe == ref.fused_moe
    g = torch.Generator().manual_seed(11)
    seq = torch.randint(0, cfg.vocab, (40,), generator=g).to(torch.int32)
    for width in (8, 1, 2):
        eng.reset(); ref.reset()
        for s in range(0, len(seq), width):
            n = min(width, len(seq) - s)
            for d in (eng, ref):
                d.tokens[:n].copy_(seq[s:s + n])
                d.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
                d.slots[:n].zero_()
                d.forward(n)
            assert torch.equal(eng.logits[:n], ref.logits[:n]), (width, s)
            assert torch.equal(eng.next_ids[:n], ref.next_ids[:n])
        for a, b in zip(eng.caches, ref.caches):
            assert torch.equal(a, b)
    # prompt executor + single-sequence engine over the bundle's engine
    eng.reset(); ref.reset()
    prompt = seq[:33].tolist()
    got = DecodeEngine(eng, prefill=MlaMoePrefill(eng, max_rows=32)).generate(prompt, 6)
    want = DecodeEngine(ref, prefill=MlaMoePrefill(ref, max_rows=32)).generate(prompt, 6)
    assert got == want
    # a parameter with the wrong shape, or a missing one, is refused before anything runs
    bad = dict(bundle_parameters(cfg, weights))
    bad["lm_head"] = bad["lm_head"][:-1]
    with pytest.raises(ValueError, match="lm_head"):
        PlanEngine(out["dir"], None, fab, parameters=bad)
    del bad["lm_head"]
    with pytest.raises(KeyError, match="lm_head"):
        PlanEngine(out["dir"], None, fab, parameters=bad)
    assert fab.status() == 0
    fab.close()


@pytest.mark.parametrize("topk,window,index_dtype", [(5, 0, "bf16"), (64, 0, "bf16"), (6, 12, "bf16"), (5, 0, "int8"), (6, 12, "int8")])
def test_sparse_indexer_program_on_the_device_matches_the_interpreter(tmp_path, topk, window, index_dtype):
    """A program with an index cache, the weighted-ReLU selector and attention over the learned selection: the plan engine binds
    rotary_prefix, index_cache_append, sparse_index, add and the indexed split-KV attention; selections equal the CPU oracle's
    and logits agree within bf16 noise."""
    from indexer_source import source

    from ironpangu_b200 import compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    src, ck, bundle = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "b"
    src.write_text(source(topk, True, window, index_dtype))       # int8: keys and query heads quantised row-wise, as in the oracle
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "5").returncode == 0
    compiler.write_bundle(str(src), str(bundle), checkpoint_dir=str(ck), prefill_tokens=8)
    toks = torch.randint(1, 512, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    oracle = compiler.interpret(src.read_text(), str(ck), toks, all_logits=True, watch=["picked"])
    ref = torch.tensor(oracle["prompt_logits"])
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, keep_logits=True)
    picked_at = next(k for k, i in enumerate(eng.ins) if i["op"] == "sparse_index")
    for s in range(0, len(toks), 8):
        n = min(8, len(toks) - s)
        eng.tokens[:n].copy_(torch.tensor(toks[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        sel = eng.vals[picked_at][:n].tolist()
        for i in range(n):
            want = oracle["watched"][s + i]["picked"]["ids"]
            got = [p for p in sel[i] if p >= 0]
            if got != want:
                # near-ties of the score may be broken differently by bf16 arithmetic: at most one position differs then
                assert len(got) == len(want) and len(set(got) ^ set(want)) <= 2, (s + i, got, want)
        torch.testing.assert_close(eng.logits[:n].cpu(), ref[s:s + n], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    fab.close()


@pytest.mark.gpu
@pytest.mark.parametrize("width", [8, 1, 3])
def test_hyper_connected_program_on_the_device_matches_the_interpreter(tmp_path, width):
    """Residual streams mixed by mHC modules, token convolutions with per-sequence history on the low-rank query, the latent and
    the attention value, attention sinks, stand-alone post-norms, an optional norm the checkpoint lacks: the plan engine binds
    repeat, mhc_pre / mhc_input / mhc_post / mhc_merge, mome, sink_normalize and the cache write with sink rows; logits agree
    with the CPU oracle at every step width, and a second sequence slot does not disturb the first."""
    from hyper_source import source

    from ironpangu_b200 import compiler
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    src, ck, bundle = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "b"
    src.write_text(source(layers=2))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "7").returncode == 0
    compiler.write_bundle(str(src), str(bundle), checkpoint_dir=str(ck), prefill_tokens=8, resident_sequences=2)
    toks = torch.randint(1, 512, (21,), generator=torch.Generator().manual_seed(4)).tolist()
    other = torch.randint(1, 512, (9,), generator=torch.Generator().manual_seed(5)).tolist()
    ref = torch.tensor(compiler.interpret(src.read_text(), str(ck), toks, all_logits=True)["prompt_logits"])
    ref_other = torch.tensor(compiler.interpret(src.read_text(), str(ck), other, all_logits=True)["prompt_logits"])
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, num_slots=2, keep_logits=True)
    ops = {i["op"] for i in eng.ins}
    assert {"repeat", "mhc_pre", "mhc_input", "mhc_post", "mhc_merge", "mome", "sink_normalize", "optional_norm"} <= ops

    def run(seq, slot, want, step):
        for s in range(0, len(seq), step):
            n = min(step, len(seq) - s)
            eng.tokens[:n].copy_(torch.tensor(seq[s:s + n], dtype=torch.int32))
            eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
            eng.slots[:n].fill_(slot)
            eng.forward(n)
            torch.testing.assert_close(eng.logits[:n].cpu(), want[s:s + n], rtol=3e-2, atol=3e-2)

    run(toks[:10], 0, ref, width)
    run(other, 1, ref_other, 8)              # another sequence in between: its convolution history and pages are its own
    # continue the first sequence where it stopped
    for s in range(10, len(toks), width):
        n = min(width, len(toks) - s)
        eng.tokens[:n].copy_(torch.tensor(toks[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        torch.testing.assert_close(eng.logits[:n].cpu(), ref[s:s + n], rtol=3e-2, atol=3e-2)
    assert fab.status() == 0
    eng.reset()
    run(toks[:8], 0, ref, 8)                 # after a reset the histories are empty again
    fab.close()


@pytest.mark.gpu
def test_generated_hyper_mla_moe_program_matches_the_interpreter(tmp_path):
    """The family generator (dense first layer, routed experts with sigmoid scoring and a sharded shared expert, windows that
    alternate by layer, sinks, convolutions, hyper-connections) at its tiny size: device logits equal the CPU oracle's."""
    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    src, ck, bundle = tmp_path / "m.inferfabric", tmp_path / "ck", tmp_path / "b"
    src.write_text(hyper_mla_moe_source(HyperMlaMoeConfig.tiny(3), 1, context=128))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "11").returncode == 0
    compiler.write_bundle(str(src), str(bundle), checkpoint_dir=str(ck), prefill_tokens=8)
    toks = torch.randint(1, 512, (37,), generator=torch.Generator().manual_seed(6)).tolist()     # longer than the short window (16)
    fab = Fabric(0, 1)
    eng = PlanEngine(str(bundle), str(ck), fab, max_tokens=8, keep_logits=True)
    routers = [k for k, i in enumerate(eng.ins) if i["op"] == "router_topk"]
    assert len(routers) == 2
    oracle = compiler.interpret(src.read_text(), str(ck), toks, all_logits=True, watch=[eng.ins[k]["name"] for k in routers])
    ref = torch.tensor(oracle["prompt_logits"])
    picked = {}
    eng.probe = lambda k, T: picked.__setitem__(k, eng.vals[k][0][:T].tolist()) if k in routers else None
    same_routes = 0
    for s in range(0, len(toks), 8):
        n = min(8, len(toks) - s)
        eng.tokens[:n].copy_(torch.tensor(toks[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        torch.cuda.synchronize()
        for i in range(n):
            # two experts whose scores are a bf16 rounding apart may swap; such a row is compared on its routes only
            agree = all(sorted(picked[k][i]) == sorted(oracle["watched"][s + i][eng.ins[k]["name"]]["ids"]) for k in routers)
            same_routes += agree
            if agree:
                torch.testing.assert_close(eng.logits[i].cpu(), ref[s + i], rtol=4e-2, atol=4e-2)
    assert same_routes >= len(toks) * 0.8, same_routes
    assert fab.status() == 0
    fab.close()


@pytest.mark.gpu
def test_packed_int8_caches_in_compiled_programs(tmp_path):
    """`cache_dtype = int8_ds_mla` in the source: the plan engine keeps 656-byte packed rows, writes them with per-128 scales and
    attends over them; the CPU oracle simulates the same quantisation. Once for the latent-attention + routed-experts family
    (every layer packed; equal to the hand-wired decoder with an int8 cache), once for the hyper-connected family with a
    packed cache on every second layer (convolved latent: the split cache write)."""
    import dataclasses

    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source, mla_moe_source
    from ironpangu_b200.models.mla_moe import MlaMoeConfig, MlaMoeDecoder, bundle_parameters, random_rank_weights
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    fab = Fabric(0, 1)
    dev = torch.device("cuda", 0)
    # ---- latent attention + routed experts, every layer packed ----
    cfg = dataclasses.replace(MlaMoeConfig.tiny(2), eos=2)
    src = tmp_path / "a.inferfabric"
    src.write_text(mla_moe_source(cfg, 1, context=128, kv_int8=True))
    out = compiler.write_bundle(str(src), str(tmp_path / "a"), prefill_tokens=8)
    W = random_rank_weights(cfg, 0, 1, dev, seed=0)
    eng = PlanEngine(out["dir"], None, fab, max_tokens=8, keep_logits=True, parameters=bundle_parameters(cfg, W))
    assert eng.kv_int8 and all(c.dtype == torch.uint8 and c.shape[-1] == 656 for c in eng.caches) and not eng.fused_head
    ref = MlaMoeDecoder(cfg, W, fab, max_tokens=8, max_context=128, keep_logits=True, kv_int8=True)
    toks = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(8)).to(torch.int32)
    for s in range(0, 24, 8):
        for d in (eng, ref):
            d.tokens[:8].copy_(toks[s:s + 8])
            d.positions[:8].copy_(torch.arange(s, s + 8, dtype=torch.int32))
            d.slots[:8].zero_()
            d.forward(8)
        torch.cuda.synchronize()
        assert torch.equal(eng.logits[:8], ref.logits[:8]) and torch.equal(eng.next_ids[:8], ref.next_ids[:8])
    for a, b in zip(eng.caches, ref.caches):
        assert torch.equal(a, b)
    # ---- hyper-connected family, packed cache on layers 0 and 2 ----
    hc = dataclasses.replace(HyperMlaMoeConfig.tiny(3), packed_every=2)
    hsrc, ck = tmp_path / "h.inferfabric", tmp_path / "ck"
    hsrc.write_text(hyper_mla_moe_source(hc, 1, context=128))
    assert compiler.cli("synth-checkpoint", str(hsrc), str(ck), "--seed", "11").returncode == 0
    compiler.write_bundle(str(hsrc), str(tmp_path / "h"), checkpoint_dir=str(ck), prefill_tokens=8)
    heng = PlanEngine(str(tmp_path / "h"), str(ck), fab, max_tokens=8, keep_logits=True)
    assert [c.dtype for c in heng.caches] == [torch.uint8, torch.bfloat16, torch.uint8]
    seq = torch.randint(1, 512, (21,), generator=torch.Generator().manual_seed(6)).tolist()
    routers = [k for k, i in enumerate(heng.ins) if i["op"] == "router_topk"]
    oracle = compiler.interpret(hsrc.read_text(), str(ck), seq, all_logits=True, watch=[heng.ins[k]["name"] for k in routers])
    want = torch.tensor(oracle["prompt_logits"])
    picked = {}
    heng.probe = lambda k, T: picked.__setitem__(k, heng.vals[k][0][:T].tolist()) if k in routers else None
    agree = 0
    for s in range(0, len(seq), 8):
        n = min(8, len(seq) - s)
        heng.tokens[:n].copy_(torch.tensor(seq[s:s + n], dtype=torch.int32))
        heng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        heng.slots[:n].zero_()
        heng.forward(n)
        torch.cuda.synchronize()
        for i in range(n):
            same = all(sorted(picked[k][i]) == sorted(oracle["watched"][s + i][heng.ins[k]["name"]]["ids"]) for k in routers)
            agree += same
            if same:
                torch.testing.assert_close(heng.logits[i].cpu(), want[s + i], rtol=5e-2, atol=5e-2)
    assert agree >= len(seq) * 0.8 and fab.status() == 0
    fab.close()


@pytest.mark.gpu
def test_learned_selection_variant_of_the_hyper_family_matches_the_interpreter(tmp_path):
    """The family's variant with packed int8 caches and learned sparse attention on every second layer: the first packed layer
    runs its indexer (int8 index keys), the next one reuses the carried selection; with a top-k that covers the whole context
    the selection is every causal position and logits follow the oracle."""
    import dataclasses

    from ironpangu_b200 import compiler
    from ironpangu_b200.compiler.sources import HyperMlaMoeConfig, hyper_mla_moe_source
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = dataclasses.replace(HyperMlaMoeConfig.tiny(3), packed_every=2, learned=True, index_heads=8, index_dim=64, index_rotary=32, index_topk=64)
    src, ck = tmp_path / "m.inferfabric", tmp_path / "ck"
    src.write_text(hyper_mla_moe_source(cfg, 1, context=128))
    assert compiler.cli("synth-checkpoint", str(src), str(ck), "--seed", "13").returncode == 0
    compiler.write_bundle(str(src), str(tmp_path / "b"), checkpoint_dir=str(ck), prefill_tokens=8)
    fab = Fabric(0, 1)
    eng = PlanEngine(str(tmp_path / "b"), str(ck), fab, max_tokens=8, keep_logits=True)
    att = [i for i in eng.ins if i["op"] == "mla_attention"]
    sel = [k for k, i in enumerate(eng.ins) if i["op"] == "sparse_index"]
    assert len(sel) == 1 and [len(a["inputs"]) for a in att] == [3, 2, 3] and att[0]["inputs"][2] == att[2]["inputs"][2] == sel[0]
    seq = torch.randint(1, 512, (21,), generator=torch.Generator().manual_seed(9)).tolist()
    routers = [k for k, i in enumerate(eng.ins) if i["op"] == "router_topk"]
    oracle = compiler.interpret(src.read_text(), str(ck), seq, all_logits=True, watch=[eng.ins[k]["name"] for k in routers + sel])
    want = torch.tensor(oracle["prompt_logits"])
    seen = {}
    eng.probe = lambda k, T: seen.__setitem__(k, (eng.vals[k][0] if k in routers else eng.vals[k])[:T].tolist()) if k in routers or k in sel else None
    agree = 0
    for s in range(0, len(seq), 8):
        n = min(8, len(seq) - s)
        eng.tokens[:n].copy_(torch.tensor(seq[s:s + n], dtype=torch.int32))
        eng.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
        eng.slots[:n].zero_()
        eng.forward(n)
        torch.cuda.synchronize()
        for i in range(n):
            assert [p for p in seen[sel[0]][i] if p >= 0] == oracle["watched"][s + i][eng.ins[sel[0]]["name"]]["ids"] == list(range(s + i + 1))
            same = all(sorted(seen[k][i]) == sorted(oracle["watched"][s + i][eng.ins[k]["name"]]["ids"]) for k in routers)
            agree += same
            if same:
                torch.testing.assert_close(eng.logits[i].cpu(), want[s + i], rtol=5e-2, atol=5e-2)
    assert agree >= len(seq) * 0.8 and fab.status() == 0
    fab.close()
