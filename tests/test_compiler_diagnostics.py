"""Diagnostics of the model-language checker on a latent-attention model with a sparse indexer and on a hyper-connected model:
every malformed variant is refused with a message that names the offending binding (scoped through folds and modules)."""
import re
import sys
import os

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import hyper_source  # noqa: E402
import indexer_source  # noqa: E402

from ironpangu_b200 import compiler  # noqa: E402

CASES = [
    ("sparse_index(iq, iw, icache, heads = 8", "sparse_index(iq, iw, icache, heads = 4", "sparse_index 'picked': index query/weight/cache widths are inconsistent"),
    ("head_dim = 64, topk", "head_dim = 32, topk", "sparse_index 'picked': index query/weight/cache widths are inconsistent"),
    ("weight = w.iw, width = 8", "weight = w.iw, width = 4", "sparse_index 'picked': index query/weight/cache widths are inconsistent"),
    ('"weighted_relu"', '"softmax"', "scoring must be weighted_relu"),
    ('cache_dtype = "bf16"', 'cache_dtype = "fp4"', "index_cache_append 'icache': index cache_dtype must be int8 or bf16"),
    ("page_tokens = 16", "page_tokens = 0", "index_cache_append 'icache': page_tokens out of range"),
    ('"learned_indices"', '"random"', "selection must be all_causal_within_window or learned_indices"),
    ("latent_attention(query, cache, picked,", "latent_attention(query, cache,", "learned_indices needs (only) an index input"),
    ("window = 0", "window = -4", "window must be >= 0"),
    ("heads = 1, head_dim = 64, rotary_dim = 32", "heads = 1, head_dim = 64, rotary_dim = 96", "rotary_prefix 'ik': rotary_dim must be even and <= head_dim"),
    ("heads = 1, head_dim = 64, rotary_dim = 32", "heads = 1, head_dim = 64, rotary_dim = 31", "rotary_prefix 'ik': rotary_dim must be even and <= head_dim"),
    ("heads = 2, nope = 128, rope = 64, latent = 512, value = 128, input", "heads = 3, nope = 128, rope = 64, latent = 512, value = 128, input",
     "mla_query 'query': input width 384 != 576"),
    ("start = 384, width = 512", "start = 384, width = 256", "query width must be a multiple of the cache row width"),
    ("div(512, 1)", "div(512, 0)", "division by zero"),
    ("devices = [0];", "devices = [0, 0];", "devices must list exactly tp entries"),
    ("yield logits;", "", "model does not yield an output"),
    ("let logits = gather(local_logits);", "let logits = gather(local_logits);\n    let logits = gather(local_logits);", "duplicate binding logits"),
    ("gather(local_logits)", "scatter(local_logits)", "unknown function or module scatter"),
]


@pytest.mark.parametrize("old,new,needle", CASES, ids=[f"{k:02d}" for k in range(len(CASES))])
def test_malformed_indexer_sources_are_refused(old, new, needle):
    good = indexer_source.source(16)
    assert old in good
    with pytest.raises(compiler.CompileError, match=re.escape(needle)):
        compiler.compile_source(good.replace(old, new))


def test_the_unmutated_source_compiles_and_a_selection_wider_than_the_context_is_clamped_not_refused():
    assert compiler.compile_source(indexer_source.source(16))["program"]["instructions"]
    assert compiler.compile_source(indexer_source.source(4096))["program"]["instructions"]     # the 92B plans ask for 2048 of a 512-row context


HYPER_CASES = [
    ("let attn_hc = mhc_pre(x, weight = w.attn_mhc, streams = 4", "let attn_hc = mhc_pre(x, weight = w.attn_mhc, streams = 3",
     "mhc_pre 'hidden[0]/block/attn_hc': input width must be a multiple of streams"),
    ("repeat(embedded, count = 4)", "repeat(embedded, count = 2)", "mhc_post 'hidden[0]/block/residual': branch width differs from the hyper-connection width"),
    ("weight = w.qa_conv, taps = 3", "weight = w.qa_conv, taps = 0", "mome 'hidden[0]/block/attention/qc': taps out of range"),
    ("weight = w.qa_conv, taps = 3", "weight = w.qa_conv, taps = 64", "mome 'hidden[0]/block/attention/qc': taps out of range"),
    ('taps = 3, placement = "tp_channels"', 'taps = 3, placement = "tp_rows"', "mome 'hidden[0]/block/attention/oc': placement must be replicated or tp_channels"),
    ("count = 5, latent = 512", "count = 5, latent = 256", "sink rows must be a multiple of latent+rope"),
    ("count = 5, latent", "count = 0, latent", "sink_normalize 'hidden[0]/block/attention/sinks': count out of range"),
    ("cache_norm_rope_append(kc, kr, sinks,", "cache_norm_rope_append(kc, kr, kc,", "sink rows must be a multiple of latent+rope"),
    ("w.mlp_mhc, streams = 4, sinkhorn = 20", "w.mlp_mhc, streams = 4, sinkhorn = -1", "mhc_pre 'hidden[0]/block/ffn_hc': sinkhorn out of range"),
    ("mhc_post(attn_hc, norm(attention", "mhc_post(x, norm(attention", "mhc_post 'hidden[0]/block/residual': input 0 must be hyper_connection, got tensor"),
    ("norm(mhc_input(attn_hc)", "norm(mhc_input(x)", "input 0 must be hyper_connection, got tensor"),
    ("mhc_post(ffn_hc, norm(ffn, weight = w.norm4, eps = 1e-5))", "mhc_post(ffn_hc, attn_hc)", "mhc_post 'hidden[0]/block/post': input 1 must be tensor, got hyper_connection"),
]


@pytest.mark.parametrize("old,new,needle", HYPER_CASES, ids=[f"{k:02d}" for k in range(len(HYPER_CASES))])
def test_malformed_hyper_connected_sources_are_refused(old, new, needle):
    good = hyper_source.source()
    assert old in good
    with pytest.raises(compiler.CompileError, match=re.escape(needle)):
        compiler.compile_source(good.replace(old, new))
