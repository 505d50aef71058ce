"""CPU oracle: index cache, sparse indexer and attention over learned selections, checked against a NumPy restatement of the
selector (from the watched node values) and against the dense-attention model where the selection covers everything."""
import numpy as np
import pytest


def source(topk: int, learned: bool, cache_dtype: str = "bf16") -> str:
    sel = ('latent_attention(query, cache, picked, scale_dim = 32, window = 0, selection = "learned_indices")' if learned else
           'latent_attention(query, cache, scale_dim = 32, window = 0, selection = "all_causal_within_window")')
    indexer = f"""
    let iq = rotary_prefix(linear(xn, weight = w.iq, width = 48, placement = "replicated"), heads = 3, head_dim = 16, rotary_dim = 8, theta = 10000);
    let ik = rotary_prefix(linear(xn, weight = w.ik, width = 16, placement = "replicated"), heads = 1, head_dim = 16, rotary_dim = 8, theta = 10000);
    let iw = linear(xn, weight = w.iw, width = 3, placement = "replicated");
    let icache = index_cache_append(ik, width = 16, page_tokens = 16, cache_dtype = "{cache_dtype}");
    let picked = sparse_index(iq, iw, icache, heads = 3, head_dim = 16, topk = {topk}, scoring = "weighted_relu");""" if learned else ""
    return f"""language inferfabric 1;
model Indexed {{
    context = 64;
    eos = 2;
    let w = weights("model");
    let x = embedding(weight = w.embed, width = 64, vocab = 128);
    let xn = norm(x, weight = w.ln, eps = 1e-5);
    let q = linear(xn, weight = w.q, width = 64, placement = "replicated");
    let latent = linear(xn, weight = w.kv, width = 32, placement = "replicated");
    let kr = linear(xn, weight = w.kr, width = 16, placement = "replicated");
    let cache = cache_norm_rope_append(latent, kr, weight = w.kv_ln, eps = 1e-5, theta = 10000);{indexer}
    let query = mla_query(q, weight = w.kvb, theta = 10000, heads = 2, nope = 16, rope = 16, latent = 32, value = 16, input_layout = "rank_local");
    let attended = {sel};
    let value = mla_value(attended, weight = w.kvb, heads = 2, latent = 32, value = 16, nope = 16);
    let h = add(x, linear(value, weight = w.o, width = 64, placement = "replicated"));
    let logits = linear(norm(h, weight = w.fln, eps = 1e-5), weight = weights("lm_head"), width = 128, placement = "replicated");
    yield logits;
}}
plan P for Indexed {{
    target = b200_token_v1;
    tp = 1;
    ep = 1;
    devices = [0];
    max_num_seqs = 1;
    max_num_batched_tokens = 1;
    max_model_len = 64;
}}
"""


@pytest.mark.parametrize("cache_dtype", ["bf16", "int8"])
def test_sparse_indexer_and_learned_selection(tmp_path, cache_dtype):
    from ironpangu_b200 import compiler

    dense, full, few = (tmp_path / n for n in ("dense.inferfabric", "full.inferfabric", "few.inferfabric"))
    dense.write_text(source(64, False, cache_dtype))
    full.write_text(source(64, True, cache_dtype))
    few.write_text(source(3, True, cache_dtype))
    ck = tmp_path / "ck"
    r = compiler.cli("synth-checkpoint", str(full), str(ck), "--seed", "5")
    assert r.returncode == 0, r.stderr
    toks = [5, 17, 99, 3, 64, 120, 8, 41, 77, 12]
    a = compiler.interpret(dense.read_text(), str(ck), toks, all_logits=True)
    b = compiler.interpret(full.read_text(), str(ck), toks, all_logits=True, watch=["picked"])
    # a selection that may take every position is dense attention
    assert np.array_equal(np.array(a["prompt_logits"]), np.array(b["prompt_logits"]))
    assert [w["picked"]["ids"] for w in b["watched"]] == [list(range(i + 1)) for i in range(len(toks))]
    c = compiler.interpret(few.read_text(), str(ck), toks, all_logits=True, watch=["picked", "iq", "ik", "iw", "icache"])
    keys = []
    for i, w in enumerate(c["watched"]):
        q, wt = np.array(w["iq"]["ranks"][0], dtype=np.float32).reshape(3, 16), np.array(w["iw"]["ranks"][0], dtype=np.float32)
        key = np.array(w["icache"]["last_row"], dtype=np.float32)
        assert w["icache"]["cache_rows"] == i + 1
        if cache_dtype == "int8":
            # rows hold rint(x / s) * s with s = max|x| / 127 (half-precision scale): at most 255 distinct levels, the largest kept
            raw = np.array(w["ik"]["ranks"][0], dtype=np.float32)
            s = float(np.float16(np.abs(raw).max() / 127))
            assert np.allclose(key, np.clip(np.rint(raw / s), -127, 127) * s, rtol=0, atol=1e-7)
            sq = np.float16(np.abs(q).max(1) / 127).astype(np.float32)[:, None]
            q = np.clip(np.rint(q / sq), -127, 127) * sq
        else:
            assert np.array_equal(key, np.array(w["ik"]["ranks"][0], dtype=np.float32))
        keys.append(key)
        score = (np.maximum(q @ np.stack(keys).T, 0) * wt[:, None]).sum(0)
        order = sorted(range(i + 1), key=lambda p: (-score[p], p))[:3]
        assert w["picked"]["ids"] == sorted(order), (i, score)
    # with three of up to ten positions the output differs from dense attention once more than three keys exist
    la, lc = np.array(a["prompt_logits"]), np.array(c["prompt_logits"])
    assert np.array_equal(la[:3], lc[:3]) and not np.array_equal(la[5:], lc[5:])
