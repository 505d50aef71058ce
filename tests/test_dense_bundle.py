"""The dense grouped-query-attention decoder written in the model language: the source compiles, the host interpreter agrees with
the plain PyTorch restatement of the model, and the bundle's engine on the GPU agrees with the hand-wired decoder."""
import dataclasses
import json

import pytest
import torch

from ironpangu_b200 import compiler
from ironpangu_b200.compiler.sources import dense_gqa_source
from ironpangu_b200.models import dense_gqa as G


def _bundle(tmp_path, cfg, tp=1, context=128, **options):
    src = tmp_path / "dense.inferfabric"
    src.write_text(dense_gqa_source(cfg, tp, context))
    return compiler.write_bundle(src, tmp_path / "bundle", **options)


def test_dense_source_compiles_to_grouped_query_instructions(tmp_path):
    cfg = G.DenseConfig.tiny(2)
    out = _bundle(tmp_path, cfg)
    prog = json.loads((tmp_path / "bundle" / "device-program.json").read_text())
    ops = [i["op"] for i in prog["instructions"]]
    assert ops.count("paged_attention") == cfg.layers and ops.count("kv_cache_append") == cfg.layers and ops.count("rotary_prefix") == 2 * cfg.layers
    assert ops.count("linear_allreduce") == 2 * cfg.layers and ops[-1] == "lm_head" and "norm" not in ops        # norms folded, residuals absorbed
    assert all(i["kernel"] != "unsupported" for i in prog["instructions"])
    assert out["instructions"] == len(ops)


@pytest.mark.parametrize("tp", [1, 2])
def test_interpreter_of_the_dense_source_matches_the_restatement(tmp_path, tp):
    import numpy as np

    from ironpangu_b200.runtime.plan_engine import SafetensorsDir

    cfg = dataclasses.replace(G.DenseConfig.tiny(2), hidden=64, heads=4, kv_heads=2, head_dim=16, ffn=96, vocab=128)
    src = tmp_path / "dense.inferfabric"
    src.write_text(dense_gqa_source(cfg, tp, 64))
    r = compiler.cli("synth-checkpoint", str(src), str(tmp_path / "ck"), "--seed", "5")
    assert r.returncode == 0, r.stderr
    st = SafetensorsDir(str(tmp_path / "ck"))

    def get(name):
        mm, off, n, dtype, shape = st.tensors[name + ".weight"]
        assert dtype == "BF16"
        return torch.from_numpy(np.frombuffer(mm, dtype=np.uint8, count=n, offset=off).copy()).view(torch.bfloat16).view(*shape)

    full = {"embed": get("model.embed_tokens"), "final_norm": get("model.norm"), "lm_head": get("lm_head")}
    for l in range(cfg.layers):
        p, q = f"layers.{l}.", f"model.layers.{l}."
        full[p + "attn_norm"], full[p + "ffn_norm"] = get(q + "input_layernorm"), get(q + "post_attention_layernorm")
        full[p + "qkv"] = torch.cat([get(q + "self_attn.q_proj"), get(q + "self_attn.k_proj"), get(q + "self_attn.v_proj")], 0)
        full[p + "o_proj"], full[p + "down"] = get(q + "self_attn.o_proj"), get(q + "mlp.down_proj")
        full[p + "gate_up"] = torch.cat([get(q + "mlp.gate_proj"), get(q + "mlp.up_proj")], 0)
    tokens = [5, 17, 99, 2, 64, 31, 7]
    got = compiler.interpret(src.read_text(), str(tmp_path / "ck"), tokens, all_logits=True)
    ref = G.forward_ref(cfg, full, torch.tensor(tokens), tp=tp)
    got = torch.tensor(got["prompt_logits"]).view(len(tokens), -1)
    torch.testing.assert_close(got, ref, rtol=3e-2, atol=3e-2)
    gap = ref.topk(2, -1).values
    clear = (gap[:, 0] - gap[:, 1]) > 0.05
    assert torch.equal(got.argmax(-1)[clear], ref.argmax(-1)[clear])


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])
def test_gpu_bundle_engine_equals_the_hand_wired_dense_decoder(tmp_path, fused):
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = G.DenseConfig.tiny(2)
    dev = torch.device("cuda", 0)
    out = _bundle(tmp_path, cfg, context=128, prefill_tokens=8, resident_sequences=2)
    fab = Fabric(0, 1)
    W = G.random_rank_weights(cfg, 0, 1, dev, seed=1)
    dec = G.DenseDecoder(cfg, W, fab, max_tokens=8, max_context=128, num_slots=2, keep_logits=True)
    eng = PlanEngine(out["dir"], None, fab, max_tokens=8, num_slots=2, keep_logits=True, parameters=G.bundle_parameters(cfg, W), fused_gqa=fused)
    assert len(eng.gqa_groups) == cfg.layers and eng.fused_gqa == fused
    if fused:
        assert all(eng._gqa_packed[k].data_ptr() == W[f"layers.{l}.qkv"].data_ptr() for l, k in enumerate(sorted(eng.gqa_groups)))   # no copy
    seq = torch.randint(0, cfg.vocab, (21,), generator=torch.Generator().manual_seed(3)).to(torch.int32)
    for width, slot in ((8, 0), (1, 1), (3, 0)):
        for d in (dec, eng):
            d.reset()
        for s in range(0, len(seq), width):
            n = min(width, len(seq) - s)
            for d in (dec, eng):
                d.tokens[:n].copy_(seq[s:s + n])
                d.positions[:n].copy_(torch.arange(s, s + n, dtype=torch.int32))
                d.slots[:n].fill_(slot)
                d.forward(n)
            torch.cuda.synchronize()
            if fused:
                assert torch.equal(eng.logits[:n], dec.logits[:n]), (width, s)
            else:
                torch.testing.assert_close(eng.logits[:n], dec.logits[:n], rtol=2e-2, atol=2e-2)
            assert fused is False or torch.equal(eng.next_ids[:n], dec.next_ids[:n])
    assert int(fab.status()) == 0 if hasattr(fab, "status") else True
    fab.close()


@pytest.mark.gpu
def test_gpu_prompt_executor_runs_on_the_bundle_engine(tmp_path):
    """The dense prompt path (matrix-matrix kernels, chunks of 64 rows) reads a bundle's engine through its decoder facade: it
    leaves the same K / V pages and the same first token as on the hand-wired decoder, and decode continues from them."""
    from ironpangu_b200.models.dense_prefill import DensePrefill
    from ironpangu_b200.parallel.fabric import Fabric
    from ironpangu_b200.runtime.plan_engine import PlanEngine

    cfg = G.DenseConfig.tiny(2)
    dev = torch.device("cuda", 0)
    out = _bundle(tmp_path, cfg, context=256, prefill_tokens=8)
    fab = Fabric(0, 1)
    W = G.random_rank_weights(cfg, 0, 1, dev, seed=2)
    dec = G.DenseDecoder(cfg, W, fab, max_tokens=8, max_context=256, keep_logits=True)
    eng = PlanEngine(out["dir"], None, fab, max_tokens=8, keep_logits=True, parameters=G.bundle_parameters(cfg, W))
    assert dataclasses.asdict(eng.cfg) == dataclasses.asdict(cfg) and (eng.hq, eng.hk, eng.vl) == (dec.hq, dec.hk, dec.vl)
    toks = torch.randint(0, cfg.vocab, (150,), generator=torch.Generator().manual_seed(5)).to(torch.int32).cuda()
    firsts = []
    for d in (dec, eng):
        pre = DensePrefill(d, max_rows=64, attn_rows=32)
        for s in range(0, 150, 64):
            nxt = pre.forward(toks[s:s + 64], s, 0)
        firsts.append(int(nxt[0]) if nxt.numel() else int(d.next_ids[0]))
    torch.cuda.synchronize()
    assert firsts[0] == firsts[1]
    for l in range(cfg.layers):
        assert torch.equal(dec.k_cache[l], eng.k_cache[l]) and torch.equal(dec.v_cache[l], eng.v_cache[l])
    gen = [[], []]
    for j, d in enumerate((dec, eng)):
        t = firsts[j]
        for step in range(6):
            d.tokens[:1].fill_(t)
            d.positions[:1].fill_(150 + step)
            d.slots[:1].zero_()
            d.forward(1)
            t = int(d.next_ids[0])
            gen[j].append(t)
    assert gen[0] == gen[1]
    fab.close()
