"""The .inferfabric source of a small hyper-connected latent-attention model (residual streams mixed by mHC modules, causal
token convolutions on the low-rank query, the latent and the attention value, attention sinks, post-norms), at dimensions the
device kernels take."""


def source(layers=2, streams=4, sinks=5, tp=1, context=128):
    devices = ", ".join(str(i) for i in range(tp))
    return f"""language inferfabric 1;

module Attention(x, w) {{
    let qkv = linear(x, weight = w.q_a, paired_weight = w.kv_a, width = 384, paired_width = 576, placement = "replicated");
    let qa = slice(qkv, start = 0, width = 384);
    let qc = mome(qa, weight = w.qa_conv, taps = 3);
    let q = linear(norm(qc, weight = w.q_norm, eps = 1e-5), weight = w.q_b, width = div(768, {tp}), placement = "tp_rows");
    let latent = slice(qkv, start = 384, width = 512);
    let kr = slice(qkv, start = 896, width = 64);
    let kc = mome(latent, weight = w.kv_conv, taps = 3);
    let sinks = sink_normalize(weight = w, norm = w.kv_norm, count = {sinks}, latent = 512, rope = 64, eps = 1e-5);
    let cache = cache_norm_rope_append(kc, kr, sinks, weight = w.kv_norm, eps = 1e-5, theta = 10000);
    let query = mla_query(q, weight = w.kv_b, theta = 10000, heads = 4, nope = 128, rope = 64, latent = 512, value = 128, input_layout = "rank_local");
    let attended = latent_attention(query, cache, scale_dim = 192, window = 0, selection = "all_causal_within_window");
    let value = mla_value(attended, weight = w.kv_b, heads = 4, latent = 512, value = 128, nope = 128);
    let oc = mome(value, weight = w.o_conv, taps = 3, placement = "tp_channels");
    let output = allreduce(linear(oc, weight = w.o, width = 256, placement = "tp_columns"));
    yield output;
}}

module Mlp(x, w) {{
    let act = swiglu(linear(x, weight = w.gate, paired_weight = w.up, width = div(512, {tp}), paired_width = div(512, {tp}), placement = "tp_rows"));
    let output = allreduce(linear(act, weight = w.down, width = 256, placement = "tp_columns"));
    yield output;
}}

module Block(x, w) {{
    let attn_hc = mhc_pre(x, weight = w.attn_mhc, streams = {streams}, sinkhorn = 20, eps = 1e-6);
    let attention = Attention(norm(mhc_input(attn_hc), weight = w.norm1, eps = 1e-5), w.attn);
    let residual = mhc_post(attn_hc, norm(attention, weight = w.norm2, eps = 1e-5));
    let ffn_hc = mhc_pre(residual, weight = w.mlp_mhc, streams = {streams}, sinkhorn = 20, eps = 1e-6);
    let ffn = Mlp(norm(mhc_input(ffn_hc), weight = w.norm3, eps = 1e-5), w.mlp);
    let post = mhc_post(ffn_hc, norm(ffn, weight = w.norm4, eps = 1e-5));
    let output = optional_norm(post, weight = w.block_norm, eps = 1e-5);
    yield output;
}}

model Hyper {{
    context = {context};
    eos = 2;
    let w = weights("model");
    let embedded = embedding(weight = w.embed, width = 256, vocab = 512);
    let hidden = fold i in range(0, {layers}) carry(x = repeat(embedded, count = {streams})) {{
        let block = Block(x, child(w.layers, i));
        yield block;
    }};
    let merged = mhc_input(mhc_merge(hidden, weight = w.merge_mhc, streams = {streams}, sinkhorn = 20, eps = 1e-6));
    let local_logits = linear(norm(merged, weight = w.norm, eps = 1e-5), weight = weights("lm_head"), width = div(512, {tp}), placement = "tp_rows");
    let logits = gather(local_logits);
    yield logits;
}}

plan P for Hyper {{
    target = b200_token_v1;
    tp = {tp};
    ep = {tp};
    devices = [{devices}];
    max_num_seqs = 1;
    max_num_batched_tokens = 1;
    max_model_len = {context};
}}
"""
