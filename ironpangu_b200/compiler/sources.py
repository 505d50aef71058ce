""".inferfabric sources of the built-in model families, written out for a configuration and a tensor-parallel width.

The engines do not wire kernels to a configuration by hand: they compile one of these sources (``write_bundle``) and run
the bundle's program (``runtime/plan_engine.py``). ``examples/mla_moe_92b_tp8.inferfabric`` is ``mla_moe_source`` of the
flagship configuration at tp = 8, kept as a file.
Reference: examples/openpangu/92b-tp8-ep8.inferfabric (the same structure in the reference's vocabulary)."""
from __future__ import annotations

from dataclasses import dataclass


def _num(x: float) -> str:
    return repr(int(x)) if float(x) == int(x) else repr(float(x))


_PACKED_CACHE = ', cache_dtype = int8_ds_mla, cache_scale_dtype = f32, cache_quantization = pertile128, cache_rope_dtype = bf16'


def mla_moe_source(cfg, tp: int, context: int = 1024, name: str = "MlaMoe", kv_int8: bool = False) -> str:
    """DSL source of the multi-head-latent-attention + routed-experts decoder ``cfg`` (``models.mla_moe.MlaMoeConfig``).
    ``kv_int8``: every layer keeps its latent cache as packed int8 rows (one f32 scale per 128 columns, rotary columns in bf16)."""
    c = cfg
    packed = _PACKED_CACHE if kv_int8 else ""
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
    let cache = cache_norm_rope_append(latent, kr, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta}{packed});

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


@dataclass
class HyperMlaMoeConfig:
    """A latent-attention + routed-experts decoder whose residual is ``streams`` parallel streams mixed by hyper-connection
    modules, with causal token convolutions (``taps`` wide) on the low-rank query, the latent and the attention value,
    ``sinks`` learned sink rows per attention layer, norms before and after every branch, ``first_dense`` leading layers with
    a dense FFN, and a long window on every ``long_every``-th layer."""
    layers: int = 46
    hidden: int = 2560
    vocab: int = 151552
    heads: int = 48
    q_lora: int = 1024
    kv_lora: int = 512
    nope: int = 128
    rope: int = 64
    vdim: int = 128
    experts: int = 256
    topk: int = 8
    expert_ffn: int = 1024
    shared_ffn: int = 1024
    dense_ffn: int = 9216
    first_dense: int = 2
    streams: int = 4
    sinkhorn: int = 20
    taps: int = 3
    sinks: int = 128
    long_every: int = 3
    long_window: int = 2048
    short_window: int = 512
    theta: float = 6.4e6
    eps: float = 1e-5
    route_scale: float = 2.5
    scoring: str = "sigmoid_bias_group_topk"
    eos: int = 2
    packed_every: int = 0          # > 0: layers whose index is a multiple of it keep a packed int8 latent cache (the long-window layers at 3)
    learned: bool = False          # those layers also attend over a learned selection: a sparse indexer (int8 index cache) picks
                                   # `index_topk` positions on every second one of them, the other ones reuse the previous selection
    index_heads: int = 24
    index_dim: int = 128
    index_rotary: int = 64
    index_topk: int = 2048

    @staticmethod
    def pangu92b() -> "HyperMlaMoeConfig":
        """The published 92B configuration of this family (46 layers, 256 experts of 1024, 48 heads, 4 streams, 128 sinks)."""
        return HyperMlaMoeConfig()

    @staticmethod
    def pangu92b_learned() -> "HyperMlaMoeConfig":
        """The same with packed int8 caches and learned sparse attention on the long-window layers (every third layer)."""
        return HyperMlaMoeConfig(packed_every=3, learned=True)

    @staticmethod
    def tiny(layers: int = 3) -> "HyperMlaMoeConfig":
        return HyperMlaMoeConfig(layers=layers, hidden=256, vocab=512, heads=4, q_lora=384, experts=8, topk=2, expert_ffn=128, shared_ffn=128,
                                 dense_ffn=512, first_dense=1, sinks=5, long_window=64, short_window=16, theta=1e4)

    @property
    def qk_dim(self) -> int:
        return self.nope + self.rope


def hyper_mla_moe_source(cfg: HyperMlaMoeConfig, tp: int, context: int = 512, name: str = "HyperMlaMoe") -> str:
    """DSL source of ``cfg`` at tensor / expert parallel width ``tp``. Dense and shared-expert projections are sharded over the
    ranks and packed (gate | up) so that the lowering fuses them with their activation and their all-reduce."""
    c = cfg
    if c.heads % tp or c.experts % tp or c.vocab % tp or c.shared_ffn % tp or c.dense_ffn % tp:
        raise ValueError(f"tp={tp} does not divide heads / experts / vocab / FFN widths of the model")
    qw, lat, theta, eps = c.q_lora, c.kv_lora, _num(c.theta), repr(c.eps)
    H, S = c.hidden, c.streams
    mhc = f"streams = {S}, sinkhorn = {c.sinkhorn}, eps = 1e-6"
    packed_expr = f"eq(mod(index, {c.packed_every}), 0)" if c.packed_every > 0 else "lt(index, 0)"
    if c.learned and c.packed_every <= 0:
        raise ValueError("learned selection runs on the packed layers: set packed_every")
    if c.learned:
        return _hyper_learned_source(c, tp, context, name, mhc, packed_expr, ", ".join(str(i) for i in range(tp)))
    devices = ", ".join(str(i) for i in range(tp))
    return f"""language inferfabric 1;

// {c.layers} layers ({c.first_dense} with a dense FFN), hidden {H} x {S} residual streams, vocab {c.vocab};
// MLA: {c.heads} heads, q_lora {qw}, kv_lora {lat}, nope {c.nope}, rope {c.rope}, v {c.vdim}, {c.sinks} sink rows, token convolutions of {c.taps} taps;
// MoE: {c.experts} routed experts (FFN {c.expert_ffn}), top-{c.topk} {c.scoring}, shared expert (FFN {c.shared_ffn}); tp = ep = {tp}.

module Attention(x, w, window, packed) {{
    let qkv = linear(x, weight = w.q_a_proj, paired_weight = w.kv_a_proj_with_mqa, width = {qw}, paired_width = {lat + c.rope}, placement = "replicated");
    let qc = mome(slice(qkv, start = 0, width = {qw}), weight = w.qa_conv, taps = {c.taps});
    let q = linear(norm(qc, weight = w.q_a_layernorm, eps = {eps}), weight = w.q_b_proj, width = div({c.heads * c.qk_dim}, {tp}), placement = "tp_rows");
    let kc = mome(slice(qkv, start = {qw}, width = {lat}), weight = w.compresskv_conv, taps = {c.taps});
    let kr = slice(qkv, start = {qw + lat}, width = {c.rope});
    let sinks = sink_normalize(weight = w, norm = w.kv_a_layernorm, count = {c.sinks}, latent = {lat}, rope = {c.rope}, eps = {eps});
    let cache = choose(packed,
        cache_norm_rope_append(kc, kr, sinks, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta}{_PACKED_CACHE}),
        cache_norm_rope_append(kc, kr, sinks, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta}));
    let query = mla_query(q, weight = w.kv_b_proj, theta = {theta}, heads = {c.heads}, nope = {c.nope}, rope = {c.rope}, latent = {lat},
                          value = {c.vdim}, input_layout = "rank_local");
    let attended = latent_attention(query, cache, scale_dim = {c.qk_dim}, window = window, selection = "all_causal_within_window");
    let value = mla_value(attended, weight = w.kv_b_proj, heads = {c.heads}, latent = {lat}, value = {c.vdim}, nope = {c.nope});
    let oc = mome(value, weight = w.o_conv, taps = {c.taps}, placement = "tp_channels");
    let output = allreduce(linear(oc, weight = w.o_proj, width = {H}, placement = "tp_columns"));
    yield output;
}}

module DenseFFN(x, w) {{
    let act = swiglu(linear(x, weight = w.gate_proj, paired_weight = w.up_proj, width = div({c.dense_ffn}, {tp}),
                            paired_width = div({c.dense_ffn}, {tp}), placement = "tp_rows"));
    let output = allreduce(linear(act, weight = w.down_proj, width = {H}, placement = "tp_columns"));
    yield output;
}}

module RoutedMoE(x, w) {{
    let routes = router(x, weight = w.gate, experts = {c.experts}, topk = {c.topk}, scoring = "{c.scoring}", scale = {repr(float(c.route_scale))});
    let expert = child(w.experts, "{{expert}}");
    let gate_up = expert_linear(x, routes, weight = expert.gate_proj, paired_weight = expert.up_proj, width = {c.expert_ffn});
    let down = expert_swiglu_down(gate_up, routes, weight = expert.down_proj, width = {H});
    let local = expert_reduce(down, routes);
    let shared_act = swiglu(linear(x, weight = w.shared_experts.gate_proj, paired_weight = w.shared_experts.up_proj,
                                   width = div({c.shared_ffn}, {tp}), paired_width = div({c.shared_ffn}, {tp}), placement = "tp_rows"));
    let shared_partial = linear(shared_act, weight = w.shared_experts.down_proj, width = {H}, placement = "tp_columns");
    let output = allreduce(add(local, shared_partial));
    yield output;
}}

module Block(x, w, index, window) {{
    let attn_hc = mhc_pre(x, weight = w.attn_mhc_module, {mhc});
    let attention = Attention(norm(mhc_input(attn_hc), weight = w.input_layernorm, eps = {eps}), w.self_attn, window, {packed_expr});
    let residual = mhc_post(attn_hc, norm(attention, weight = w.post_attention_layernorm, eps = {eps}));
    let ffn_hc = mhc_pre(residual, weight = w.mlp_mhc_module, {mhc});
    let ffn_in = norm(mhc_input(ffn_hc), weight = w.pre_mlp_layernorm, eps = {eps});
    let ffn = choose(lt(index, {c.first_dense}), DenseFFN(ffn_in, w.mlp), RoutedMoE(ffn_in, w.mlp));
    let mixed = mhc_post(ffn_hc, norm(ffn, weight = w.post_mlp_layernorm, eps = {eps}));
    let output = optional_norm(mixed, weight = w.block_post_layernorm, eps = {eps});
    yield output;
}}

model {name} {{
    context = {context};
    eos = {c.eos};
    let w = weights("model");
    let embedded = embedding(weight = w.embed_tokens, width = {H}, vocab = {c.vocab});

    let hidden = fold i in range(0, {c.layers}) carry(x = repeat(embedded, count = {S})) {{
        let window = choose(eq(mod(i, {c.long_every}), 0), {c.long_window}, {c.short_window});
        let block = Block(x, child(w.layers, i), i, window);
        yield block;
    }};

    let merged = mhc_input(mhc_merge(hidden, weight = w.merge_mhc_module, {mhc}));
    let local_logits = linear(norm(merged, weight = w.norm, eps = {eps}), weight = weights("lm_head"), width = div({c.vocab}, {tp}), placement = "tp_rows");
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


def _hyper_learned_source(c: HyperMlaMoeConfig, tp: int, context: int, name: str, mhc: str, packed_expr: str, devices: str) -> str:
    """The variant with a sparse indexer: the fold carries a record (residual streams, last selection); a packed layer attends
    over the selection - computed by its own indexer when its index is a multiple of ``2 * packed_every``, else the one carried
    from the previous packed layer."""
    qw, lat, theta, eps = c.q_lora, c.kv_lora, _num(c.theta), repr(c.eps)
    H, S = c.hidden, c.streams
    iw = c.index_heads * c.index_dim
    fresh_expr = f"eq(mod(index, {2 * c.packed_every}), 0)"
    return f"""language inferfabric 1;

// {c.layers} layers ({c.first_dense} with a dense FFN), hidden {H} x {S} residual streams, vocab {c.vocab};
// MLA: {c.heads} heads, q_lora {qw}, kv_lora {lat}, nope {c.nope}, rope {c.rope}, v {c.vdim}, {c.sinks} sink rows, token convolutions of {c.taps} taps;
// every {c.packed_every}th layer: packed int8 latent cache + attention over a learned selection ({c.index_heads} index heads x {c.index_dim},
// top-{c.index_topk}, int8 index keys), recomputed on every second one of them;
// MoE: {c.experts} routed experts (FFN {c.expert_ffn}), top-{c.topk} {c.scoring}, shared expert (FFN {c.shared_ffn}); tp = ep = {tp}.

module Selector(x, qr, w) {{
    let iq = rotary_prefix(linear(qr, weight = w.wq_b, width = {iw}, placement = "replicated"),
                           heads = {c.index_heads}, head_dim = {c.index_dim}, rotary_dim = {c.index_rotary}, theta = {theta});
    let ik = rotary_prefix(norm(linear(x, weight = w.wk, width = {c.index_dim}, placement = "replicated"), weight = w.k_norm, eps = {eps}),
                           heads = 1, head_dim = {c.index_dim}, rotary_dim = {c.index_rotary}, theta = {theta});
    let gains = linear(x, weight = w.weights_proj, width = {c.index_heads}, placement = "replicated");
    let keys = index_cache_append(ik, width = {c.index_dim}, page_tokens = 16, cache_dtype = "int8");
    let picked = sparse_index(iq, gains, keys, heads = {c.index_heads}, head_dim = {c.index_dim}, topk = {c.index_topk}, scoring = "weighted_relu");
    yield picked;
}}

module Attention(x, w, window, packed, fresh, carried) {{
    let qkv = linear(x, weight = w.q_a_proj, paired_weight = w.kv_a_proj_with_mqa, width = {qw}, paired_width = {lat + c.rope}, placement = "replicated");
    let qc = mome(slice(qkv, start = 0, width = {qw}), weight = w.qa_conv, taps = {c.taps});
    let qn = norm(qc, weight = w.q_a_layernorm, eps = {eps});
    let q = linear(qn, weight = w.q_b_proj, width = div({c.heads * c.qk_dim}, {tp}), placement = "tp_rows");
    let kc = mome(slice(qkv, start = {qw}, width = {lat}), weight = w.compresskv_conv, taps = {c.taps});
    let kr = slice(qkv, start = {qw + lat}, width = {c.rope});
    let sinks = sink_normalize(weight = w, norm = w.kv_a_layernorm, count = {c.sinks}, latent = {lat}, rope = {c.rope}, eps = {eps});
    let cache = choose(packed,
        cache_norm_rope_append(kc, kr, sinks, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta}{_PACKED_CACHE}),
        cache_norm_rope_append(kc, kr, sinks, weight = w.kv_a_layernorm, eps = {eps}, theta = {theta}));
    let query = mla_query(q, weight = w.kv_b_proj, theta = {theta}, heads = {c.heads}, nope = {c.nope}, rope = {c.rope}, latent = {lat},
                          value = {c.vdim}, input_layout = "rank_local");
    let selection = choose(packed, choose(fresh, Selector(x, qn, w.indexer), carried), carried);
    let attended = choose(packed,
        latent_attention(query, cache, selection, scale_dim = {c.qk_dim}, window = window, selection = "learned_indices"),
        latent_attention(query, cache, scale_dim = {c.qk_dim}, window = window, selection = "all_causal_within_window"));
    let value = mla_value(attended, weight = w.kv_b_proj, heads = {c.heads}, latent = {lat}, value = {c.vdim}, nope = {c.nope});
    let oc = mome(value, weight = w.o_conv, taps = {c.taps}, placement = "tp_channels");
    let output = allreduce(linear(oc, weight = w.o_proj, width = {H}, placement = "tp_columns"));
    let result = record(hidden = output, selection = selection);
    yield result;
}}

module DenseFFN(x, w) {{
    let act = swiglu(linear(x, weight = w.gate_proj, paired_weight = w.up_proj, width = div({c.dense_ffn}, {tp}),
                            paired_width = div({c.dense_ffn}, {tp}), placement = "tp_rows"));
    let output = allreduce(linear(act, weight = w.down_proj, width = {H}, placement = "tp_columns"));
    yield output;
}}

module RoutedMoE(x, w) {{
    let routes = router(x, weight = w.gate, experts = {c.experts}, topk = {c.topk}, scoring = "{c.scoring}", scale = {repr(float(c.route_scale))});
    let expert = child(w.experts, "{{expert}}");
    let gate_up = expert_linear(x, routes, weight = expert.gate_proj, paired_weight = expert.up_proj, width = {c.expert_ffn});
    let down = expert_swiglu_down(gate_up, routes, weight = expert.down_proj, width = {H});
    let local = expert_reduce(down, routes);
    let shared_act = swiglu(linear(x, weight = w.shared_experts.gate_proj, paired_weight = w.shared_experts.up_proj,
                                   width = div({c.shared_ffn}, {tp}), paired_width = div({c.shared_ffn}, {tp}), placement = "tp_rows"));
    let shared_partial = linear(shared_act, weight = w.shared_experts.down_proj, width = {H}, placement = "tp_columns");
    let output = allreduce(add(local, shared_partial));
    yield output;
}}

module Block(x, w, index, window) {{
    let attn_hc = mhc_pre(x.hidden, weight = w.attn_mhc_module, {mhc});
    let attention = Attention(norm(mhc_input(attn_hc), weight = w.input_layernorm, eps = {eps}), w.self_attn, window, {packed_expr}, {fresh_expr}, x.selection);
    let residual = mhc_post(attn_hc, norm(attention.hidden, weight = w.post_attention_layernorm, eps = {eps}));
    let ffn_hc = mhc_pre(residual, weight = w.mlp_mhc_module, {mhc});
    let ffn_in = norm(mhc_input(ffn_hc), weight = w.pre_mlp_layernorm, eps = {eps});
    let ffn = choose(lt(index, {c.first_dense}), DenseFFN(ffn_in, w.mlp), RoutedMoE(ffn_in, w.mlp));
    let mixed = mhc_post(ffn_hc, norm(ffn, weight = w.post_mlp_layernorm, eps = {eps}));
    let output = optional_norm(mixed, weight = w.block_post_layernorm, eps = {eps});
    let result = record(hidden = output, selection = attention.selection);
    yield result;
}}

model {name} {{
    context = {context};
    eos = {c.eos};
    let w = weights("model");
    let embedded = embedding(weight = w.embed_tokens, width = {H}, vocab = {c.vocab});

    // the first layer computes its own selection, so the carried one only needs a value to start from
    let hidden = fold i in range(0, {c.layers}) carry(x = record(hidden = repeat(embedded, count = {S}), selection = embedded)) {{
        let window = choose(eq(mod(i, {c.long_every}), 0), {c.long_window}, {c.short_window});
        let block = Block(x, child(w.layers, i), i, window);
        yield block;
    }};

    let merged = mhc_input(mhc_merge(hidden.hidden, weight = w.merge_mhc_module, {mhc}));
    let local_logits = linear(norm(merged, weight = w.norm, eps = {eps}), weight = weights("lm_head"), width = div({c.vocab}, {tp}), placement = "tp_rows");
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


def main(argv=None) -> int:
    """``python -m ironpangu_b200.compiler.sources FAMILY [--tp N] [--context N] [--layers N] [--kv-int8] [--learned]`` prints the
    ``.inferfabric`` source of a built-in family at a built-in size: ``flagship`` / ``tiny`` (latent attention + routed experts),
    ``dense2b`` / ``dense-tiny`` (grouped-query attention), ``pangu92b`` / ``hyper-tiny`` (hyper-connected latent attention +
    routed experts; ``--learned``: packed caches and learned sparse attention on every third layer)."""
    import argparse
    import sys

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("family", choices=["flagship", "tiny", "dense2b", "dense-tiny", "pangu92b", "hyper-tiny"])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--kv-int8", action="store_true")
    ap.add_argument("--learned", action="store_true")
    a = ap.parse_args(argv)
    if a.family in ("flagship", "tiny"):
        from ..models.mla_moe import MlaMoeConfig

        c = MlaMoeConfig.flagship() if a.family == "flagship" else MlaMoeConfig.tiny(2)
        if a.layers:
            c.layers = a.layers
        text = mla_moe_source(c, a.tp, context=a.context, kv_int8=a.kv_int8)
    elif a.family in ("dense2b", "dense-tiny"):
        from ..models.dense_gqa import DenseConfig

        c = DenseConfig.qwen2b() if a.family == "dense2b" else DenseConfig.tiny(2)
        if a.layers:
            c.layers = a.layers
        text = dense_gqa_source(c, a.tp, context=a.context)
    else:
        if a.family == "pangu92b":
            c = HyperMlaMoeConfig.pangu92b_learned() if a.learned else HyperMlaMoeConfig.pangu92b()
        else:
            c = HyperMlaMoeConfig.tiny()
            if a.learned:
                c.packed_every, c.learned, c.index_heads, c.index_dim, c.index_rotary, c.index_topk = 2, True, 8, 64, 32, 64
        if a.layers:
            c.layers = a.layers
        if a.kv_int8 and not c.packed_every:
            c.packed_every = 1
        text = hyper_mla_moe_source(c, a.tp, context=a.context)
    sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
