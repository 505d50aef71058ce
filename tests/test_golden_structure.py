"""Structural facts of the two 92B example programs at eight ranks, read back from the published bundle (no GPU, no weights)."""
import collections
import json
import os
import struct

import pytest

from ironpangu_b200 import compiler

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bundle(tmp_path, name):
    out = compiler.write_bundle(os.path.join(ROOT, "examples", name), str(tmp_path / "b"), prefill_tokens=8)
    with open(os.path.join(out["dir"], "device-program.json")) as f:
        return out, json.load(f)


def _count(ins):
    return collections.Counter(i["op"] for i in ins)


def test_learned_92b_program_has_two_attention_windows_and_eight_shared_selectors(tmp_path):
    out, prog = _bundle(tmp_path, "hyper_mla_moe_92b_learned_tp8.inferfabric")
    ins = prog["instructions"]
    ops = _count(ins)
    # 46 layers, the first two with a dense feed-forward: one cache write, one attention, one sink state per layer
    assert ops["mla_attention"] == ops["mla_kv_write"] == ops["sink_normalize"] == 46
    assert ops["router_topk"] == ops["moe_gate_up"] == ops["moe_down_allreduce"] == 44
    assert ops["mhc_pre"] == ops["mhc_post"] == 92 and ops["mhc_merge"] == 1 and ops["repeat"] == 1      # 4 streams in, 1 out
    assert ops["mome"] == 3 * 46                                                                  # q, latent and rope-key convolutions
    attn = [i for i in ins if i["op"] == "mla_attention"]
    kinds = collections.Counter((int(i["attrs"]["window"]), i["attrs"]["selection"]) for i in attn)
    assert kinds == {(512, "all_causal_within_window"): 30, (2048, "learned_indices"): 16}
    # a selection is computed on every sixth layer and used by that layer and the long-window layer three later
    selectors = [k for k, i in enumerate(ins) if i["op"] == "sparse_index"]
    assert len(selectors) == 8 and ops["index_cache_append"] == 8
    users = collections.Counter(x for i in attn for x in i["inputs"] if x in selectors)
    assert sorted(users) == selectors and set(users.values()) == {2}
    for k in selectors:
        assert ins[k]["attrs"] == {"head_dim": "128", "heads": "24", "scoring": "weighted_relu", "topk": "2048"}
    # the sixteen long-window layers keep the packed int8 cache, the other thirty plain bf16 rows
    dtypes = collections.Counter(i["attrs"].get("cache_dtype", "bf16") for i in ins if i["op"] == "mla_kv_write")
    assert dtypes == {"bf16": 30, "int8_ds_mla": 16}
    for i in attn:
        writer = next(ins[x] for x in i["inputs"] if ins[x]["op"] == "mla_kv_write")
        assert (writer["attrs"].get("cache_dtype") == "int8_ds_mla") == (i["attrs"]["selection"] == "learned_indices")
    # per token: one collective per o_proj, per feed-forward and for the vocabulary head
    assert prog["collectives_per_token"] == 46 + 46 + 1 and prog["launches_per_token"] < len(ins)
    assert prog["parallel"]["tp"] == prog["parallel"]["ep"] == 8 and prog["parallel"]["devices"] == list(range(8))


def test_bf16_92b_program_windows_and_header(tmp_path):
    out, prog = _bundle(tmp_path, "hyper_mla_moe_92b_tp8.inferfabric")
    ins = prog["instructions"]
    ops = _count(ins)
    assert ops["sparse_index"] == 0 and ops["index_cache_append"] == 0
    kinds = collections.Counter((int(i["attrs"]["window"]), i["attrs"]["selection"]) for i in ins if i["op"] == "mla_attention")
    assert kinds == {(512, "all_causal_within_window"): 30, (2048, "all_causal_within_window"): 16}
    assert all("cache_dtype" not in i["attrs"] for i in ins if i["op"] == "mla_kv_write")
    # binary program header: magic, context, end-of-sequence id, output value, instruction count, ..., ranks at bytes 28..32
    with open(os.path.join(out["dir"], "execution.bin"), "rb") as f:
        head = f.read(32)
    assert head[:8] == prog["magic"].encode() == b"IFTOKN04"
    context, eos, output, count = struct.unpack_from("<4I", head, 8)
    assert (context, eos, output, count) == (prog["max_context"], prog["eos"], prog["output"], len(ins))
    assert struct.unpack_from("<I", head, 28)[0] == 8
    # every rank's init plan binds the same number of tensors; the arena report exists per rank
    sizes = set()
    for r in range(8):
        with open(os.path.join(out["dir"], f"rank-{r}.init.json")) as f:
            sizes.add(len(json.load(f)["loads"]))
        assert os.path.exists(os.path.join(out["dir"], f"arena-rank-{r}.txt"))
    assert len(sizes) == 1
