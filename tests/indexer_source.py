"""The .inferfabric source of a one-layer latent-attention model with a sparse indexer, at dimensions the device kernels take."""
def source(topk, learned=True, window=0, index_dtype="bf16"):
    sel = ('latent_attention(query, cache, picked, scale_dim = 192, window = %d, selection = "learned_indices")' % window if learned else
           'latent_attention(query, cache, scale_dim = 192, window = %d, selection = "all_causal_within_window")' % window)
    indexer = f"""
    let iq = rotary_prefix(linear(xn, weight = w.iq, width = 512, placement = "replicated"), heads = 8, head_dim = 64, rotary_dim = 32, theta = 10000);
    let ik = rotary_prefix(linear(xn, weight = w.ik, width = 64, placement = "replicated"), heads = 1, head_dim = 64, rotary_dim = 32, theta = 10000);
    let iw = linear(xn, weight = w.iw, width = 8, placement = "replicated");
    let icache = index_cache_append(ik, width = 64, page_tokens = 16, cache_dtype = "{index_dtype}");
    let picked = sparse_index(iq, iw, icache, heads = 8, head_dim = 64, topk = {topk}, scoring = "weighted_relu");""" if learned else ""
    return f"""language inferfabric 1;
model Indexed {{
    context = 128;
    eos = 2;
    let w = weights("model");
    let x = embedding(weight = w.embed, width = 256, vocab = 512);
    let xn = norm(x, weight = w.ln, eps = 1e-5);
    let qkv = linear(xn, weight = w.q, paired_weight = w.kva, width = 384, paired_width = 576, placement = "replicated");
    let q = slice(qkv, start = 0, width = 384);
    let latent = slice(qkv, start = 384, width = 512);
    let kr = slice(qkv, start = 896, width = 64);
    let cache = cache_norm_rope_append(latent, kr, weight = w.kv_ln, eps = 1e-5, theta = 10000);{indexer}
    let query = mla_query(q, weight = w.kvb, theta = 10000, heads = 2, nope = 128, rope = 64, latent = 512, value = 128, input_layout = "rank_local");
    let attended = {sel};
    let value = mla_value(attended, weight = w.kvb, heads = 2, latent = 512, value = 128, nope = 128);
    let h = add(x, linear(value, weight = w.o, width = 256, placement = "replicated"));
    let local_logits = linear(norm(h, weight = w.fln, eps = 1e-5), weight = weights("lm_head"), width = div(512, 1), placement = "tp_rows");
    let logits = gather(local_logits);
    yield logits;
}}
plan P for Indexed {{
    target = b200_token_v1;
    tp = 1;
    ep = 1;
    devices = [0];
    max_num_seqs = 1;
    max_num_batched_tokens = 1;
    max_model_len = 128;
}}
"""
