#include "config_audit.h"

#include <map>
#include <set>

namespace ifab::config_audit {
namespace {

struct Fields {
  const Json& c;
  uint64_t count(const char* key, bool required, uint64_t fallback = 0, bool positive = false) const {
    const Json* v = c.find(key);
    if (!v || v->is_null()) {
      if (required) invalid(std::string("config: ") + key + " is missing");
      return fallback;
    }
    if (!v->is_int() || v->as_int() < 0) invalid(std::string("config: ") + key + " must be a non-negative integer");
    if (positive && v->as_int() == 0) invalid(std::string("config: ") + key + " must be positive");
    return (uint64_t)v->as_int();
  }
  bool flag(const char* key, bool fallback) const {
    const Json* v = c.find(key);
    if (!v || v->is_null()) return fallback;
    if (!v->is_bool()) invalid(std::string("config: ") + key + " must be true or false");
    return v->as_bool();
  }
  // a list of distinct layer indices below `bound`
  std::vector<uint64_t> layer_list(const char* key, uint64_t bound) const {
    std::vector<uint64_t> out;
    const Json* v = c.find(key);
    if (!v || v->is_null()) return out;
    if (!v->is_array()) invalid(std::string("config: ") + key + " must be a list");
    std::set<uint64_t> seen;
    for (auto& e : v->as_array()) {
      if (!e.is_int() || e.as_int() < 0 || (uint64_t)e.as_int() >= bound) invalid(std::string("config: ") + key + " names a layer outside the model");
      if (!seen.insert((uint64_t)e.as_int()).second) invalid(std::string("config: ") + key + " names layer " + std::to_string(e.as_int()) + " twice");
      out.push_back((uint64_t)e.as_int());
    }
    return out;
  }
};

struct OpRow {
  const char* operation;
  const char* kernel;     // entry point of libifab_kernels that implements it ("" = none)
};

// The one weight-quantisation scheme the family ships: compressed-tensors, int8 weights with one static symmetric scale per
// output channel, int8 activations with one dynamic symmetric scale per token, applied to Linear modules except those named
// (exactly, no patterns) under `ignore`. Anything else - groups, block structures, activation ordering, quantised outputs
// or caches, several groups - is refused: a different scheme needs its own kernels.
Json quantization_map(const Json& c) {
  Json out = Json::object();
  const Json* q = c.find("quantization_config");
  if (!q || q->is_null()) {
    out.set("declared", false);
    return out;
  }
  if (!q->is_object()) invalid("config: quantization_config must be an object");
  auto want = [](const Json& o, const char* key, const Json& value, const char* where) {
    const Json* v = o.find(key);
    if (!v || v->dump() != value.dump()) invalid(std::string("config: quantization ") + where + key + " must be " + value.dump());
  };
  want(*q, "quant_method", Json("compressed-tensors"), "");
  want(*q, "quantize", Json("w8a8_dynamic"), "");
  want(*q, "format", Json("int-quantized"), "");
  want(*q, "quantization_status", Json("compressed"), "");
  const Json* groups = q->find("config_groups");
  if (!groups || !groups->is_object() || groups->size() != 1) invalid("config: quantization needs exactly one config group (W8A8 over Linear)");
  const Json& g = groups->as_object().front().second;
  Json linear = Json::array();
  linear.push("Linear");
  want(g, "targets", linear, "group ");
  for (const char* side : {"weights", "input_activations"}) {
    const Json* o = g.find(side);
    if (!o || !o->is_object()) invalid(std::string("config: quantization group lacks ") + side);
    const std::string where = std::string(side) + ".";
    want(*o, "num_bits", Json((int64_t)8), where.c_str());
    want(*o, "type", Json("int"), where.c_str());
    want(*o, "symmetric", Json(true), where.c_str());
    for (const char* key : {"actorder", "group_size", "block_structure"})
      if (const Json* v = o->find(key); v && !v->is_null()) invalid(std::string("config: quantization ") + where + key + " is not supported");
  }
  want(g.at("weights"), "strategy", Json("channel"), "weights.");
  want(g.at("weights"), "dynamic", Json(false), "weights.");
  want(g.at("input_activations"), "strategy", Json("token"), "input_activations.");
  want(g.at("input_activations"), "dynamic", Json(true), "input_activations.");
  if (const Json* v = g.find("output_activations"); v && !v->is_null()) invalid("config: quantised output activations need their own contract");
  if (const Json* v = q->find("kv_cache_scheme"); v && !v->is_null()) invalid("config: a quantised cache scheme needs its own contract");
  Json ignore = Json::array();
  if (const Json* ig = q->find("ignore"); ig && !ig->is_null()) {
    if (!ig->is_array()) invalid("config: quantization ignore must be a list of module names");
    std::set<std::string> seen;
    for (auto& e : ig->as_array()) {
      if (!e.is_string() || e.as_string().empty() || e.as_string().find_first_of("*?[") != std::string::npos)
        invalid("config: quantization ignore entries must be exact module names (no patterns)");
      if (seen.insert(e.as_string()).second) ignore.push(e.as_string());
    }
  }
  out.set("declared", true);
  out.set("scheme", "w8a8_dynamic");
  out.set("weights", "int8, symmetric, one static scale per output channel (<module>.weight_scale)");
  out.set("activations", "int8, symmetric, one dynamic scale per token");
  out.set("applies_to", "every Linear module not listed under ignore");
  out.set("ignore", ignore);
  return out;
}

}  // namespace

Json audit(std::string_view bytes) {
  if (bytes.size() > kMaxConfigBytes) fail(ErrorKind::Capacity, "config: larger than 1 MiB");
  const Json c = Json::parse(bytes, kMaxConfigBytes);
  if (!c.is_object()) invalid("config: not a JSON object");
  const Json* type = c.find("model_type");
  if (!type || !type->is_string() || (type->as_string() != "pangu_v2_moe" && type->as_string() != "openpangu_v2"))
    invalid("config: model_type must be pangu_v2_moe or openpangu_v2 (other families have their own contracts)");
  const Fields f{c};
  for (const char* key : {"hidden_size", "intermediate_size", "vocab_size", "num_attention_heads", "kv_lora_rank", "qk_nope_head_dim",
                          "qk_rope_head_dim", "v_head_dim", "max_position_embeddings"})
    f.count(key, true, 0, true);
  const uint64_t layers = f.count("num_hidden_layers", true, 0, true), mtp = f.count("num_nextn_predict_layers", false, 0);
  if (layers > 4096 || mtp > 256) fail(ErrorKind::Capacity, "config: more layers than the audit handles (4096 + 256)");
  const uint64_t total = layers + mtp, dense = f.count("first_k_dense_replace", false, layers);
  if (dense > layers) invalid("config: first_k_dense_replace exceeds the layer count");
  const bool moe = dense < layers;
  if (moe) {
    const uint64_t experts = f.count("n_routed_experts", true, 0, true), topk = f.count("num_experts_per_tok", true, 0, true);
    f.count("moe_intermediate_size", true, 0, true);
    f.count("n_shared_experts", true);
    f.flag("norm_topk_prob", false);
    if (topk > experts) invalid("config: num_experts_per_tok exceeds n_routed_experts");
  }
  // sliding windows: one window per listed layer
  const std::vector<uint64_t> swa = f.layer_list("swa_layers", total);
  std::map<uint64_t, uint64_t> window_of;
  {
    const Json* w = c.find("sliding_window_list");
    const size_t n = w && !w->is_null() ? (w->is_array() ? w->size() : SIZE_MAX) : 0;
    if (n != swa.size()) invalid("config: sliding_window_list must have one window per entry of swa_layers");
    for (size_t i = 0; i < swa.size(); ++i) {
      const Json& e = w->as_array()[i];
      if (!e.is_int() || e.as_int() <= 0) invalid("config: sliding windows must be positive integers");
      window_of[swa[i]] = (uint64_t)e.as_int();
    }
  }
  f.layer_list("dsa_layers", layers);
  f.layer_list("block_post_layernorm_idx", layers);
  const uint64_t index_topk = f.count("index_topk", false, 0);
  if (index_topk) {
    f.count("index_n_heads", true, 0, true);
    f.count("index_head_dim", true, 0, true);
    f.count("q_lora_rank", true, 0, true);
  }
  const bool mome = f.flag("use_mome", false);
  if (mome) {
    f.count("router_sliding_window", true, 0, true);
    f.count("q_lora_rank", true, 0, true);
  }
  const uint64_t streams = f.count("mhc_num_stream", false, 1);
  if (streams == 0 || streams > 1024) invalid("config: mhc_num_stream must be between 1 and 1024");
  const bool mhc = streams > 1;
  Json warnings = Json::array();
  if (c.find("use_mhc") && f.flag("use_mhc", false) != mhc)
    warnings.push("use_mhc disagrees with mhc_num_stream; the stream count decides (more than one stream = hyper-connections): settle this before compiling");
  if (mhc) {
    f.count("mhc_recur_norm", true, 0, true);
    if (!f.flag("mhc_use_gamma", false)) invalid("config: hyper-connections need mhc_use_gamma");
  }
  // cross-layer cache reuse: {"reuse": source} or [[reuse, source], ...]
  std::map<uint64_t, uint64_t> reuse_of;
  if (const Json* m = c.find("cla_explicit_mapping"); m && !m->is_null()) {
    std::vector<std::pair<uint64_t, uint64_t>> pairs;
    if (m->is_object()) {
      for (auto& kv : m->as_object()) {
        if (kv.first.empty() || kv.first.find_first_not_of("0123456789") != std::string::npos || !kv.second.is_int() || kv.second.as_int() < 0)
          invalid("config: cla_explicit_mapping must map layer numbers to layer numbers");
        pairs.emplace_back(std::stoull(kv.first), (uint64_t)kv.second.as_int());
      }
    } else if (m->is_array()) {
      for (auto& e : m->as_array()) {
        if (!e.is_array() || e.size() != 2 || !e.as_array()[0].is_int() || !e.as_array()[1].is_int() || e.as_array()[0].as_int() < 0 || e.as_array()[1].as_int() < 0)
          invalid("config: cla_explicit_mapping entries must be [reuse layer, source layer] pairs");
        pairs.emplace_back((uint64_t)e.as_array()[0].as_int(), (uint64_t)e.as_array()[1].as_int());
      }
    } else {
      invalid("config: cla_explicit_mapping must be an object or a list of pairs");
    }
    for (auto& p : pairs)
      if (p.first >= layers || p.second >= p.first || !reuse_of.emplace(p.first, p.second).second)
        invalid("config: a cache-reuse layer must lie inside the model, come after its source and appear once");
  }
  std::vector<std::string> modes;
  if (const Json* m = c.find("indexer_types"); m && !m->is_null()) {
    if (!m->is_array()) invalid("config: indexer_types must be a list of strings");
    for (auto& e : m->as_array()) {
      if (!e.is_string() || e.as_string().empty()) invalid("config: indexer_types must be a list of non-empty strings");
      modes.push_back(e.as_string());
    }
    if (modes.size() < layers || modes.size() > total) invalid("config: indexer_types must cover every layer (and at most the prediction layers beyond)");
  }
  const bool sinks = f.count("param_sink_number", false, 0) > 0;
  bool index_sharing = false;
  for (auto& m : modes) index_sharing |= m == "shared";

  Json summary = Json::array();
  for (uint64_t i = 0; i < layers; ++i) {
    Json l = Json::object();
    l.set("index", i);
    auto w = window_of.find(i);
    l.set("attention", w != window_of.end() ? "sliding_window_mla" : index_topk ? "sparse_mla" : "full_mla");
    l.set("sliding_window", w != window_of.end() ? Json((int64_t)w->second) : Json(nullptr));
    l.set("feed_forward", i < dense ? "dense" : "moe");
    auto r = reuse_of.find(i);
    l.set("cache_source_layer", r != reuse_of.end() ? Json((int64_t)r->second) : Json(nullptr));
    l.set("indexer_mode", i < modes.size() ? Json(modes[i]) : Json(nullptr));
    summary.push(std::move(l));
  }
  Json features = Json::object();
  features.set("cross_layer_cache_reuse_declared", !reuse_of.empty());
  features.set("index_sharing_declared", index_sharing);
  features.set("learned_sinks", sinks);
  features.set("mhc", mhc);
  features.set("moe", moe);
  features.set("mome", mome);
  features.set("mtp_declared", mtp > 0);
  const Json* q = c.find("quantization_config");
  features.set("quantization_declared", q != nullptr && !q->is_null());
  features.set("sparse_indexer", index_topk > 0);

  std::vector<OpRow> ops = {{"embedding", "ifab_embedding_bf16"},       {"rms_norm", "ifab_rmsnorm_bf16"},
                            {"linear", "ifab_gemv_bf16 / ifab_gemm_bf16"}, {"rotary", "ifab_mla_q_absorb (query) / ifab_mla_kv_write (key)"},
                            {"mla_cache_append", "ifab_mla_kv_write"},  {"mla_attention", "ifab_mla_head_decode / ifab_mla_decode_attention / ifab_fa_prefill_bf16"},
                            {"gated_ffn", "ifab_gemv_bf16 (SwiGLU epilogue)"}, {"residual", "fused into ifab_gemv_allreduce_bf16"},
                            {"logits", "ifab_lm_head_argmax"},          {"sampling", "ifab_sample_topk"}};
  if (!reuse_of.empty()) ops.push_back({"shared_layer_cache_views", ""});
  if (index_sharing) ops.push_back({"shared_sparse_indices", ""});
  if (moe)
    for (OpRow r : {OpRow{"sigmoid_router", "ifab_router_topk (scoring sigmoid_bias_group_topk)"}, OpRow{"routing_bias_topk", "ifab_router_topk"},
                    OpRow{"expert_permutation", "ifab_moe_dispatch"}, OpRow{"grouped_matmul", "ifab_grouped_gemm_bf16 / ifab_moe_gate_up"},
                    OpRow{"weighted_combine", "ifab_moe_down_allreduce / ifab_moe_combine"}, OpRow{"shared_experts", "ifab_moe_gate_up (shared slot)"}})
      ops.push_back(r);
  if (mome)
    for (OpRow r : {OpRow{"causal_channel_convolution", "ifab_mome"}, OpRow{"history_gather_update", "ifab_mome (state update)"}}) ops.push_back(r);
  if (mhc)
    for (OpRow r : {OpRow{"mhc_pre", "ifab_mhc_pre"}, OpRow{"sinkhorn", "ifab_mhc_pre (Sinkhorn iterations)"}, OpRow{"mhc_post", "ifab_mhc_post"}}) ops.push_back(r);
  if (index_topk)
    for (OpRow r : {OpRow{"indexer_cache_append", ""}, OpRow{"sparse_topk", "ifab_sparse_index"}, OpRow{"sparse_attention", ""}}) ops.push_back(r);
  if (sinks) ops.push_back({"attention_sinks", "ifab_mla_decode_attention (sink rows)"});
  if (!swa.empty()) ops.push_back({"sliding_window_attention", "ifab_mla_decode_attention (window)"});
  Json required = Json::array(), gaps = Json::array();
  for (auto& r : ops) {
    Json o = Json::object();
    o.set("operation", r.operation);
    o.set("kernel", r.kernel);
    required.push(std::move(o));
    if (!*r.kernel) gaps.push(r.operation);
  }
  warnings.push("attention form per layer follows the default selection: a sliding window first, then a positive index_topk, else full attention; dsa_layers is kept in the raw config but selects nothing here");
  warnings.push("the raw config is preserved with its unknown fields; this audit does not establish model semantics, index sharing, cache reuse, quantisation or multi-token prediction");
  Json unresolved = Json::array();
  for (const char* u : {"exact tensor binding, shapes and payload integrity of the checkpoint (ifab bind-checkpoint)",
                        "tokenizer, chat template and generation defaults", "rank placement, replicated / transformed weights and load staging (ifab plan-placement)",
                        "cache, indexer and convolution state, activation / workspace / communication memory", "numerical and serving qualification on the full checkpoint"})
    unresolved.push(u);
  Json out = Json::object();
  out.set("format", "ifab.config-audit.v1");
  out.set("executable", false);
  out.set("hardware_qualified", false);
  out.set("config_sha256", Sha256::of(bytes));
  out.set("config", c);
  out.set("layers", summary);
  out.set("features", features);
  out.set("quantization", quantization_map(c));
  out.set("required_operations", required);
  out.set("operations_without_a_kernel", gaps);
  out.set("warnings", warnings);
  out.set("unresolved", unresolved);
  return out;
}

}  // namespace ifab::config_audit
