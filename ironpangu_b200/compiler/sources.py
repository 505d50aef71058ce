""".inferfabric sources of the built-in model families, written out for a configuration and a tensor-parallel width.

The engines do not wire kernels to a configuration by hand: they compile one of these sources (``write_bundle``) and run
the bundle's program (``runtime/plan_engine.py``). ``examples/mla_moe_92b_tp8.inferfabric`` is ``mla_moe_source`` of the
flagship configuration at tp = 8, kept as a file.
Reference: examples/openpangu/92b-tp8-ep8.inferfabric (the same structure in the reference's vocabulary)."""
from __future__ import annotations


def _num(x: float) -> str:
    return repr(int(x)) if float(x) == int(x) else repr(float(x))


def mla_moe_source(cfg, tp: int, context: int = 1024, name: str = "MlaMoe") -> str:
    """DSL source of the multi-head-latent-attention + routed-experts decoder ``cfg`` (``models.mla_moe.MlaMoeConfig``)."""
    c = cfg
    if c.heads % tp or c.experts % tp or c.vocab % tp or c.shared_ffn % tp:
        raise ValueError(f"tp={tp} does not divide heads / experts / vocab / shared width of the model")
    qw, lat, theta, eps = c.q_lora, c.kv_lora, _num(c.theta), repr(c.eps)
    devices = ", ".join(str(i) for i in range(tp))
    eos = f"    eos = {c.eos if c.eos >= 0 else 2};\n"      # the language wants one; engines stop on it only when told to
    return f"""language inferfabric 1;

// {c.layers} layers, hidden {c.hidden}, vocab {c.vocab}; MLA: {c.heads} heads, q_lora {qw}, kv_lora {lat}, nope {c.nope}, rope {c.rope}, v {c.vdim};
// MoE: {c.experts} routed experts (FFN {c.expert_ffn}), top-{c.topk} {c.scoring} routing, 1 shared expert (FFN {c.shared_ffn}); tp = ep = {tp}.

module MLAAttention(x, w, window) {{
    let qkv = linear(x, weight = w.q_a_proj, paired_weight = w.kv_a_proj_with_mqa,
                     width = {qw}, paired_width = {lat + c.rope}, placement = "replicated");
    let qa = slice(qkv, start = 0, width = {qw});
    let qn = norm(qa, weight = w.q_a_layernorm, eps = {eps});
    let q = linear(qn, weight = w.q_b_proj, width = div({c.heads * c.qk_dim}, {tp}), placement = "tp_rows");

    let latent = slice(qkv, start = {qw}, width = {lat});
    let kr = slice(qkv, start = {qw + lat}, width = {c.rope});
    let cache = cache_norm_rope_append(latent, kr, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta});

    let query = mla_query(q, weight = w.kv_b_proj, theta = {theta}, heads = {c.heads}, nope = {c.nope}, rope = {c.rope},
                          latent = {lat}, value = {c.vdim}, input_layout = "rank_local");
    let attended = latent_attention(query, cache, scale_dim = {c.qk_dim}, window = window,
                                    selection = "all_causal_within_window");
    let value = mla_value(attended, weight = w.kv_b_proj, heads = {c.heads}, latent = {lat}, value = {c.vdim}, nope = {c.nope});
    let partial = linear(value, weight = w.o_proj, width = {c.hidden}, placement = "tp_columns");
    let output = allreduce(partial);
    yield output;
}}

module RoutedMoE(x, w) {{
    let routes = router(x, weight = w.gate, experts = {c.experts}, topk = {c.topk}, scoring = "{c.scoring}", scale = {_num(c.route_scale) if float(c.route_scale) != int(c.route_scale) else repr(float(c.route_scale))});
    let expert = child(w.experts, "{{expert}}");
    let gate_up = expert_linear(x, routes, weight = expert.gate_proj, paired_weight = expert.up_proj, width = {c.expert_ffn});
    let down = expert_swiglu_down(gate_up, routes, weight = expert.down_proj, width = {c.hidden});
    let local = expert_reduce(down, routes);
    let shared_act = swiglu(linear(x, weight = w.shared_experts.gate_proj, paired_weight = w.shared_experts.up_proj,
                                   width = div({c.shared_ffn}, {tp}), paired_width = div({c.shared_ffn}, {tp}), placement = "tp_rows"));
    let shared_partial = linear(shared_act, weight = w.shared_experts.down_proj, width = {c.hidden}, placement = "tp_columns");
    let output = allreduce(add(local, shared_partial));
    yield output;
}}

module DecoderBlock(x, w, window) {{
    let attention = MLAAttention(norm(x, weight = w.input_layernorm, eps = {eps}), w.self_attn, window);
    let h = add(x, attention);
    let ffn = RoutedMoE(norm(h, weight = w.post_attention_layernorm, eps = {eps}), w.mlp);
    let output = add(h, ffn);
    yield output;
}}

model {name} {{
    context = {context};
{eos}    let w = weights("model");
    let embedded = embedding(weight = w.embed_tokens, width = {c.hidden}, vocab = {c.vocab});

    let hidden = fold i in range(0, {c.layers}) carry(x = embedded) {{
        let block = DecoderBlock(x, child(w.layers, i), {c.window});
        yield block;
    }};

    let normalized = norm(hidden, weight = w.norm, eps = {eps});
    let local_logits = linear(normalized, weight = weights("lm_head"), width = div({c.vocab}, {tp}), placement = "tp_rows");
    let logits = gather(local_logits);
    yield logits;
}}

plan TP{tp}EP{tp} for {name} {{
    target = b200_token_v1;
    tp = {tp};
    ep = {tp};
    devices = [{devices}];
    max_num_seqs = 1;
    max_num_batched_tokens = 1;
    max_model_len = {context};
}}
"""


def dense_gqa_source(cfg, tp: int, context: int = 1024, name: str = "DenseGqa", eos: int = 2) -> str:
    """DSL source of the dense grouped-query-attention decoder ``cfg`` (``models.dense_gqa.DenseConfig``): per layer
    RMSNorm -> q / k / v projections -> rotary on q and k -> K / V page append -> paged attention -> output projection
    (all-reduced) + residual; RMSNorm -> SwiGLU MLP (all-reduced) + residual."""
    c = cfg
    if c.heads % tp or c.kv_heads % tp or c.ffn % tp or c.vocab % tp:
        raise ValueError(f"tp={tp} does not divide heads / kv heads / FFN / vocab of the model")
    hd, theta, eps = c.head_dim, _num(c.theta), repr(c.eps)
    devices = ", ".join(str(i) for i in range(tp))
    return f"""language inferfabric 1;

// {c.layers} layers, hidden {c.hidden}, vocab {c.vocab}; GQA: {c.heads} query / {c.kv_heads} KV heads x {hd}; SwiGLU {c.ffn}; tp = {tp}.

module GQAAttention(x, w) {{
    let q = rotary_prefix(linear(x, weight = w.q_proj, width = div({c.heads * hd}, {tp}), placement = "tp_rows"),
                          heads = div({c.heads}, {tp}), head_dim = {hd}, rotary_dim = {hd}, theta = {theta});
    let k = rotary_prefix(linear(x, weight = w.k_proj, width = div({c.kv_heads * hd}, {tp}), placement = "tp_rows"),
                          heads = div({c.kv_heads}, {tp}), head_dim = {hd}, rotary_dim = {hd}, theta = {theta});
    let v = linear(x, weight = w.v_proj, width = div({c.kv_heads * hd}, {tp}), placement = "tp_rows");
    let cache = kv_cache_append(k, v, kv_heads = {c.kv_heads}, head_dim = {hd});
    let attended = paged_attention(q, cache, heads = {c.heads}, kv_heads = {c.kv_heads}, head_dim = {hd}, scale = {repr(1.0 / (hd ** 0.5))});
    let partial = linear(attended, weight = w.o_proj, width = {c.hidden}, placement = "tp_columns");
    let output = allreduce(partial);
    yield output;
}}

module SwiGLU(x, w) {{
    let act = swiglu(linear(x, weight = w.gate_proj, paired_weight = w.up_proj, width = div({c.ffn}, {tp}),
                            paired_width = div({c.ffn}, {tp}), placement = "tp_rows"));
    let partial = linear(act, weight = w.down_proj, width = {c.hidden}, placement = "tp_columns");
    let output = allreduce(partial);
    yield output;
}}

module DecoderBlock(x, w) {{
    let attention = GQAAttention(norm(x, weight = w.input_layernorm, eps = {eps}), w.self_attn);
    let h = add(x, attention);
    let ffn = SwiGLU(norm(h, weight = w.post_attention_layernorm, eps = {eps}), w.mlp);
    let output = add(h, ffn);
    yield output;
}}

model {name} {{
    context = {context};
    eos = {eos};
    let w = weights("model");
    let embedded = embedding(weight = w.embed_tokens, width = {c.hidden}, vocab = {c.vocab});

    let hidden = fold i in range(0, {c.layers}) carry(x = embedded) {{
        let block = DecoderBlock(x, child(w.layers, i));
        yield block;
    }};

    let normalized = norm(hidden, weight = w.norm, eps = {eps});
    let local_logits = linear(normalized, weight = weights("lm_head"), width = div({c.vocab}, {tp}), placement = "tp_rows");
    let logits = gather(local_logits);
    yield logits;
}}

plan TP{tp} for {name} {{
    target = b200_token_v1;
    tp = {tp};
    ep = {tp};
    devices = [{devices}];
    max_num_seqs = 1;
    max_num_batched_tokens = 1;
    max_model_len = {context};
}}
"""
