#include "graph.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <set>

namespace ifab::graph {

const char* kind_name(Kind k) {
  switch (k) {
    case Kind::Tensor: return "tensor";
    case Kind::HyperConnection: return "hyper_connection";
    case Kind::Routes: return "routes";
    case Kind::Experts: return "experts";
    case Kind::Cache: return "cache";
    case Kind::Quantized: return "quantized";
    case Kind::IndexCache: return "index_cache";
    case Kind::Indices: return "indices";
  }
  return "?";
}

const std::string* Node::attr(std::string_view key) const {
  for (auto& kv : attrs)
    if (kv.first == key) return &kv.second;
  return nullptr;
}
const std::string& Node::need(std::string_view key) const {
  if (auto p = attr(key)) return *p;
  invalid("byte " + std::to_string(byte) + ": " + op + " '" + name + "' is missing attribute " + std::string(key));
}
int64_t Node::int_attr(std::string_view key) const {
  const std::string& s = need(key);
  char* end = nullptr;
  long long v = strtoll(s.c_str(), &end, 10);
  if (!end || *end || s.empty()) invalid("byte " + std::to_string(byte) + ": attribute " + std::string(key) + " of '" + name + "' must be an integer");
  return v;
}
double Node::num_attr(std::string_view key) const {
  const std::string& s = need(key);
  char* end = nullptr;
  double v = strtod(s.c_str(), &end);
  if (!end || *end || s.empty() || !std::isfinite(v)) invalid("byte " + std::to_string(byte) + ": attribute " + std::string(key) + " of '" + name + "' must be a number");
  return v;
}

void Parallel::validate() const {
  if (tp != ep) invalid("plan: tp and ep must be equal (expert parallelism shares the tensor-parallel group)");
  if (tp != 1 && tp != 2 && tp != 4 && tp != 8) invalid("plan: tp must be 1, 2, 4 or 8");
  if (devices.size() != tp) invalid("plan: devices must list exactly tp entries");
  std::set<uint32_t> seen(devices.begin(), devices.end());
  if (seen.size() != devices.size()) invalid("plan: devices must be distinct");
  if (max_num_seqs == 0 || max_num_batched_tokens == 0 || max_model_len == 0) invalid("plan: limits must be positive");
  if (max_num_seqs > 1024) fail(ErrorKind::Capacity, "plan: max_num_seqs above 1024");
}
Json Parallel::to_json() const {
  Json j = Json::object();
  j.set("target", target);
  j.set("tp", tp);
  j.set("ep", ep);
  Json d = Json::array();
  for (auto x : devices) d.push((int64_t)x);
  j.set("devices", d);
  j.set("max_num_seqs", max_num_seqs);
  j.set("max_num_batched_tokens", max_num_batched_tokens);
  j.set("max_model_len", max_model_len);
  return j;
}

// ---------------------------------------------------------------------------------------------
namespace {

[[noreturn]] void bad(const Node& n, const std::string& m) { invalid("byte " + std::to_string(n.byte) + ": " + n.op + " '" + n.name + "': " + m); }

void attrs_exact(const Node& n, std::initializer_list<const char*> required, std::initializer_list<const char*> optional = {}) {
  for (auto r : required)
    if (!n.has(r)) bad(n, std::string("missing attribute ") + r);
  for (auto& kv : n.attrs) {
    bool ok = false;
    for (auto r : required) ok |= kv.first == r;
    for (auto o : optional) ok |= kv.first == o;
    if (!ok) bad(n, "unknown attribute " + kv.first);
  }
}
void arity(const Node& n, const std::vector<Type>& in, size_t lo, size_t hi) {
  if (in.size() < lo || in.size() > hi) bad(n, "expects " + std::to_string(lo) + (hi != lo ? ".." + std::to_string(hi) : "") + " inputs, got " + std::to_string(in.size()));
}
void want(const Node& n, const std::vector<Type>& in, size_t i, Kind k) {
  if (in[i].kind != k) bad(n, "input " + std::to_string(i) + " must be " + kind_name(k) + ", got " + kind_name(in[i].kind));
}
void weight_name(const Node& n, const char* key, bool expert = false) {
  const std::string& w = n.need(key);
  if (w.empty() || w.size() > 1024) bad(n, "bad weight name");
  for (unsigned char c : w)
    if (!(isalnum(c) || c == '.' || c == '_' || c == '{' || c == '}')) bad(n, "weight name may only contain [A-Za-z0-9._{}]");
  if (w.find("..") != std::string::npos) bad(n, "weight name contains '..'");
  if (expert && w.find("{expert}") == std::string::npos) bad(n, "expert weight name must contain {expert}");
}
uint32_t pos_int(const Node& n, const char* key, int64_t lo = 1, int64_t hi = 1 << 30) {
  int64_t v = n.int_attr(key);
  if (v < lo || v > hi) bad(n, std::string(key) + " out of range");
  return (uint32_t)v;
}
Type tensor(uint32_t w) { return Type{Kind::Tensor, w, 0}; }

const std::set<std::string> kCacheDtypes = {"bf16", "int8", "int4", "int8_ds_mla"};
void cache_attrs(const Node& n) {
  if (auto d = n.attr("cache_dtype")) {
    if (!kCacheDtypes.count(*d)) bad(n, "cache_dtype must be bf16, int8, int4 or int8_ds_mla");
    if (*d == "bf16" && (n.has("cache_quantization") || n.has("cache_scale_dtype"))) bad(n, "bf16 cache takes no quantization attributes");
    if (*d != "bf16") {
      const std::string& q = n.need("cache_quantization");
      if (q != "per_token_head_symmetric" && q != "pertile128") bad(n, "cache_quantization must be per_token_head_symmetric or pertile128");
      if (*d == "int8_ds_mla" && q != "pertile128") bad(n, "int8_ds_mla uses pertile128 scales");
    }
  } else if (n.has("cache_quantization") || n.has("cache_scale_dtype") || n.has("cache_rope_dtype")) {
    bad(n, "cache quantization attributes need cache_dtype");
  }
}

}  // namespace

Type infer(const Node& n, const std::vector<Type>& in, const Parallel& par) {
  const std::string& op = n.op;
  const uint32_t tp = par.tp;
  if (op == "embedding") {
    arity(n, in, 0, 0);
    attrs_exact(n, {"weight", "width", "vocab"});
    weight_name(n, "weight");
    pos_int(n, "vocab");
    return tensor(pos_int(n, "width"));
  }
  if (op == "cast") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"dtype"});
    if (n.need("dtype") != "bf16" && n.need("dtype") != "f32") bad(n, "dtype must be bf16 or f32");
    return in[0];
  }
  if (op == "quantize") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"dtype", "scheme", "scale_dtype"});
    const std::string& d = n.need("dtype");
    if (d != "int8" && d != "fp8_e4m3") bad(n, "dtype must be int8 or fp8_e4m3");
    if (n.need("scheme") != "per_token_symmetric" && n.need("scheme") != "block128") bad(n, "scheme must be per_token_symmetric or block128");
    if (n.need("scale_dtype") != "f32") bad(n, "scale_dtype must be f32");
    return Type{Kind::Quantized, in[0].width, 0};
  }
  if (op == "repeat") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"count"});
    return tensor(in[0].width * pos_int(n, "count", 1, 16));
  }
  if (op == "mhc_pre" || op == "mhc_merge") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "streams", "sinkhorn", "eps"});
    weight_name(n, "weight");
    uint32_t s = pos_int(n, "streams", 1, 16);
    pos_int(n, "sinkhorn", 1, 64);
    if (n.num_attr("eps") <= 0) bad(n, "eps must be positive");
    if (in[0].width % s) bad(n, "input width must be a multiple of streams");
    return Type{Kind::HyperConnection, in[0].width / s, s};
  }
  if (op == "mhc_input") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::HyperConnection);
    attrs_exact(n, {});
    return tensor(in[0].width);
  }
  if (op == "mhc_post") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::HyperConnection);
    want(n, in, 1, Kind::Tensor);
    attrs_exact(n, {});
    if (in[1].width != in[0].width) bad(n, "branch width differs from the hyper-connection width");
    return tensor(in[0].width * in[0].aux);
  }
  if (op == "norm" || op == "optional_norm") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "eps"}, {"zero_centered"});
    weight_name(n, "weight");
    if (n.num_attr("eps") <= 0) bad(n, "eps must be positive");
    return in[0];
  }
  if (op == "linear") {
    arity(n, in, 1, 1);
    if (in[0].kind != Kind::Tensor && in[0].kind != Kind::Quantized) bad(n, "input must be a tensor or a quantized tensor");
    attrs_exact(n, {"weight", "width", "placement"}, {"paired_weight", "paired_width", "weight_dtype"});
    weight_name(n, "weight");
    const std::string& pl = n.need("placement");
    if (pl != "tp_rows" && pl != "tp_columns" && pl != "replicated") bad(n, "placement must be tp_rows, tp_columns or replicated");
    uint32_t w = pos_int(n, "width");
    if (n.has("paired_weight") != n.has("paired_width")) bad(n, "paired_weight and paired_width go together");
    if (n.has("paired_weight")) {
      weight_name(n, "paired_weight");
      if (pl == "tp_columns") bad(n, "paired projections cannot be K-sharded");
      if (in[0].kind != Kind::Tensor) bad(n, "paired projections take a bf16 input");
      w += pos_int(n, "paired_width");
    }
    return tensor(w);
  }
  if (op == "gather") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {});
    return tensor(in[0].width * tp);
  }
  if (op == "allreduce") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {}, {"dtype"});
    if (auto d = n.attr("dtype"))
      if (*d != "f32" && *d != "bf16") bad(n, "dtype must be f32 or bf16");
    return in[0];
  }
  if (op == "mome") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "taps"}, {"placement"});
    weight_name(n, "weight");
    pos_int(n, "taps", 2, 8);
    if (auto p = n.attr("placement"))
      if (*p != "replicated" && *p != "tp_channels") bad(n, "placement must be replicated or tp_channels");
    return in[0];
  }
  if (op == "slice") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"start", "width"});
    int64_t s = n.int_attr("start");
    uint32_t w = pos_int(n, "width");
    if (s < 0 || (uint64_t)s + w > in[0].width) bad(n, "slice exceeds the input width");
    return tensor(w);
  }
  if (op == "rotary_prefix") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"heads", "head_dim", "rotary_dim", "theta"});
    uint32_t h = pos_int(n, "heads"), d = pos_int(n, "head_dim"), r = pos_int(n, "rotary_dim");
    if (r > d || r % 2) bad(n, "rotary_dim must be even and <= head_dim");
    if (in[0].width != h * d) bad(n, "input width must equal heads*head_dim");
    if (n.num_attr("theta") <= 1) bad(n, "theta must be > 1");
    return in[0];
  }
  if (op == "rope") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"theta"});
    if (in[0].width % 2) bad(n, "rope width must be even");
    if (n.num_attr("theta") <= 1) bad(n, "theta must be > 1");
    return in[0];
  }
  if (op == "concat") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Tensor);
    attrs_exact(n, {});
    return tensor(in[0].width + in[1].width);
  }
  if (op == "mla_query") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "theta", "heads", "nope", "rope", "latent"}, {"input_layout", "rotary_dtype", "value"});
    weight_name(n, "weight");
    uint32_t h = pos_int(n, "heads"), np = pos_int(n, "nope"), rp = pos_int(n, "rope"), lat = pos_int(n, "latent");
    if (h % tp) bad(n, "heads must be divisible by tp");
    if (rp % 2) bad(n, "rope must be even");
    std::string layout = n.attr("input_layout") ? *n.attr("input_layout") : "replicated";
    if (layout != "rank_local" && layout != "replicated") bad(n, "input_layout must be rank_local or replicated");
    uint32_t expect = (layout == "rank_local" ? h / tp : h) * (np + rp);
    if (in[0].width != expect) bad(n, "input width " + std::to_string(in[0].width) + " != " + std::to_string(expect) + " for layout " + layout);
    return tensor((h / tp) * (lat + rp));
  }
  if (op == "sink_normalize") {
    arity(n, in, 0, 0);
    attrs_exact(n, {"weight", "norm", "count", "latent", "rope", "eps"});
    weight_name(n, "weight");
    weight_name(n, "norm");
    return tensor(pos_int(n, "count", 1, 4096) * (pos_int(n, "latent") + pos_int(n, "rope")));
  }
  if (op == "cache_append") {
    arity(n, in, 1, 2);
    want(n, in, 0, Kind::Tensor);
    if (in.size() == 2) want(n, in, 1, Kind::Tensor);
    attrs_exact(n, {}, {"cache_dtype", "cache_scale_dtype", "cache_quantization", "cache_rope_dtype", "rope"});
    cache_attrs(n);
    uint32_t rp = n.has("rope") ? pos_int(n, "rope") : 64;
    if (rp >= in[0].width) bad(n, "rope columns exceed the row width");
    if (in.size() == 2 && in[1].width % in[0].width) bad(n, "sink rows must be a multiple of the cache row width");
    return Type{Kind::Cache, in[0].width, rp};
  }
  if (op == "cache_norm_rope_append") {
    arity(n, in, 2, 3);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Tensor);
    if (in.size() == 3) want(n, in, 2, Kind::Tensor);
    attrs_exact(n, {"weight", "eps", "theta"}, {"cache_dtype", "cache_scale_dtype", "cache_quantization", "cache_rope_dtype"});
    weight_name(n, "weight");
    cache_attrs(n);
    if (in[1].width % 2) bad(n, "rope input width must be even");
    if (in.size() == 3 && in[2].width % (in[0].width + in[1].width)) bad(n, "sink rows must be a multiple of latent+rope");
    if (auto d = n.attr("cache_dtype"))
      if (*d == "int8_ds_mla" && in[0].width % 128) bad(n, "pertile128 needs a latent width divisible by 128");
    return Type{Kind::Cache, in[0].width + in[1].width, in[1].width};
  }
  if (op == "index_cache_append") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"width", "page_tokens"}, {"cache_dtype"});
    if (pos_int(n, "width") != in[0].width) bad(n, "width attribute differs from the input width");
    pos_int(n, "page_tokens", 1, 1024);
    if (auto d = n.attr("cache_dtype"))
      if (*d != "int8" && *d != "bf16") bad(n, "index cache_dtype must be int8 or bf16");
    return Type{Kind::IndexCache, in[0].width, 0};
  }
  if (op == "sparse_index") {
    arity(n, in, 3, 3);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Tensor);
    want(n, in, 2, Kind::IndexCache);
    attrs_exact(n, {"heads", "head_dim", "topk", "scoring"});
    uint32_t h = pos_int(n, "heads"), d = pos_int(n, "head_dim");
    if (n.need("scoring") != "weighted_relu") bad(n, "scoring must be weighted_relu");
    if (in[0].width != h * d || in[1].width != h || in[2].width != d) bad(n, "index query/weight/cache widths are inconsistent");
    return Type{Kind::Indices, pos_int(n, "topk", 1, 65536), 0};
  }
  if (op == "latent_attention") {
    arity(n, in, 2, 3);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Cache);
    attrs_exact(n, {"scale_dim", "window", "selection"});
    pos_int(n, "scale_dim");
    int64_t win = n.int_attr("window");
    if (win < 0) bad(n, "window must be >= 0 (0 = full causal)");
    const std::string& sel = n.need("selection");
    if (sel != "all_causal_within_window" && sel != "learned_indices") bad(n, "selection must be all_causal_within_window or learned_indices");
    if ((sel == "learned_indices") != (in.size() == 3)) bad(n, "learned_indices needs (only) an index input");
    if (in.size() == 3) want(n, in, 2, Kind::Indices);
    if (in[0].width % in[1].width) bad(n, "query width must be a multiple of the cache row width");
    return tensor(in[0].width / in[1].width * (in[1].width - in[1].aux));
  }
  if (op == "mla_value") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "heads", "latent", "value"}, {"nope"});
    weight_name(n, "weight");
    uint32_t h = pos_int(n, "heads"), lat = pos_int(n, "latent"), v = pos_int(n, "value");
    if (h % tp) bad(n, "heads must be divisible by tp");
    if (in[0].width != (h / tp) * lat) bad(n, "input width must equal local heads * latent");
    return tensor((h / tp) * v);
  }
  if (op == "swiglu") {
    arity(n, in, 1, 2);
    attrs_exact(n, {});
    want(n, in, 0, Kind::Tensor);
    if (in.size() == 1) {
      if (in[0].width % 2) bad(n, "packed swiglu input must have an even width");
      return tensor(in[0].width / 2);
    }
    want(n, in, 1, Kind::Tensor);
    if (in[0].width != in[1].width) bad(n, "gate and up widths differ");
    return in[0];
  }
  if (op == "router") {
    arity(n, in, 1, 1);
    want(n, in, 0, Kind::Tensor);
    attrs_exact(n, {"weight", "experts", "topk", "scoring", "scale"}, {"renorm"});
    weight_name(n, "weight");
    uint32_t e = pos_int(n, "experts", 1, 256), k = pos_int(n, "topk", 1, 16);
    if (k > e) bad(n, "topk exceeds experts");
    if (e % par.ep) bad(n, "experts must be divisible by ep");
    const std::string& sc = n.need("scoring");
    if (sc != "softmax" && sc != "sigmoid_bias_group_topk") bad(n, "scoring must be softmax or sigmoid_bias_group_topk");
    if (n.num_attr("scale") <= 0) bad(n, "scale must be positive");
    return Type{Kind::Routes, k, e};
  }
  if (op == "expert_linear") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Routes);
    attrs_exact(n, {"weight", "width"}, {"paired_weight", "weight_dtype"});
    weight_name(n, "weight", true);
    uint32_t w = pos_int(n, "width");
    if (n.has("paired_weight")) {
      weight_name(n, "paired_weight", true);
      w *= 2;
    }
    return Type{Kind::Experts, w, 0};
  }
  if (op == "expert_swiglu_down") {
    arity(n, in, 2, 3);
    attrs_exact(n, {"weight", "width"}, {"weight_dtype"});
    weight_name(n, "weight", true);
    want(n, in, 0, Kind::Experts);
    if (in.size() == 3) {
      want(n, in, 1, Kind::Experts);
      want(n, in, 2, Kind::Routes);
      if (in[0].width != in[1].width) bad(n, "gate and up expert widths differ");
    } else {
      want(n, in, 1, Kind::Routes);
      if (in[0].width % 2) bad(n, "packed gate_up width must be even");
    }
    return Type{Kind::Experts, pos_int(n, "width"), 0};
  }
  if (op == "expert_reduce") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Experts);
    want(n, in, 1, Kind::Routes);
    attrs_exact(n, {});
    return tensor(in[0].width);
  }
  if (op == "add") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Tensor);
    attrs_exact(n, {});
    if (in[0].width != in[1].width) bad(n, "operand widths differ");
    return in[0];
  }
  if (op == "kv_cache_append") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Tensor);
    attrs_exact(n, {"kv_heads", "head_dim"}, {"cache_dtype"});
    uint32_t kvh = pos_int(n, "kv_heads"), hd = pos_int(n, "head_dim");
    if (kvh % tp && tp % kvh) bad(n, "kv_heads and tp must divide one another");
    uint32_t local = std::max(1u, kvh / tp);
    if (in[0].width != local * hd || in[1].width != local * hd) bad(n, "k/v width must equal local kv heads * head_dim");
    return Type{Kind::Cache, 2 * local * hd, local};
  }
  if (op == "paged_attention") {
    arity(n, in, 2, 2);
    want(n, in, 0, Kind::Tensor);
    want(n, in, 1, Kind::Cache);
    attrs_exact(n, {"heads", "kv_heads", "head_dim", "scale"}, {"window"});
    uint32_t h = pos_int(n, "heads"), hd = pos_int(n, "head_dim");
    if (h % tp) bad(n, "heads must be divisible by tp");
    if (in[0].width != (h / tp) * hd) bad(n, "query width must equal local heads * head_dim");
    if (n.num_attr("scale") <= 0) bad(n, "scale must be positive");
    return tensor(in[0].width);
  }
  bad(n, "unknown primitive");
}

// ---------------------------------------------------------------------------------------------
namespace {
std::vector<uint32_t> parse_uint_list(const std::string& s, const char* what) {
  if (s.size() < 2 || s.front() != '[' || s.back() != ']') invalid(std::string("plan: ") + what + " must be a list");
  std::vector<uint32_t> out;
  size_t b = 1;
  while (b < s.size() - 1) {
    size_t e = s.find(',', b);
    if (e == std::string::npos || e > s.size() - 1) e = s.size() - 1;
    std::string t = s.substr(b, e - b);
    char* end = nullptr;
    long long v = strtoll(t.c_str(), &end, 10);
    if (t.empty() || !end || *end || v < 0) invalid(std::string("plan: bad entry in ") + what);
    out.push_back((uint32_t)v);
    b = e + 1;
  }
  return out;
}
uint32_t parse_u32(const std::string& s, const char* what) {
  char* end = nullptr;
  long long v = strtoll(s.c_str(), &end, 10);
  if (s.empty() || !end || *end || v < 0 || v > 0x7fffffff) invalid(std::string(what) + " must be a nonnegative integer");
  return (uint32_t)v;
}
}  // namespace

Graph elaborate(const lang::Expanded& ex) {
  Graph g;
  g.name = ex.model_name;
  // plan
  std::set<std::string> known = {"target", "tp", "ep", "devices", "max_num_seqs", "max_num_batched_tokens", "max_model_len"};
  for (auto& kv : ex.plan)
    if (!known.count(kv.first)) invalid("plan: unknown field " + kv.first);
  auto field = [&](const char* k) -> const std::string* {
    auto it = ex.plan.find(k);
    return it == ex.plan.end() ? nullptr : &it->second;
  };
  if (auto t = field("target")) g.parallel.target = *t;
  if (g.parallel.target != "b200_token_v1" && g.parallel.target != "ascend_token_v1") invalid("plan: unsupported token target " + g.parallel.target);
  if (auto v = field("tp")) g.parallel.tp = parse_u32(*v, "plan: tp");
  g.parallel.ep = g.parallel.tp;
  if (auto v = field("ep")) g.parallel.ep = parse_u32(*v, "plan: ep");
  if (auto v = field("devices")) g.parallel.devices = parse_uint_list(*v, "devices");
  else {
    g.parallel.devices.clear();
    for (uint32_t i = 0; i < g.parallel.tp; ++i) g.parallel.devices.push_back(i);
  }
  if (auto v = field("max_num_seqs")) g.parallel.max_num_seqs = parse_u32(*v, "plan: max_num_seqs");
  if (auto v = field("max_num_batched_tokens")) g.parallel.max_num_batched_tokens = parse_u32(*v, "plan: max_num_batched_tokens");
  // model fields
  for (auto& kv : ex.fields)
    if (kv.first != "context" && kv.first != "eos") invalid("model: unknown field " + kv.first);
  auto ctx = ex.fields.find("context");
  if (ctx == ex.fields.end()) invalid("model: missing field context");
  g.max_context = parse_u32(ctx->second, "model: context");
  auto eos = ex.fields.find("eos");
  if (eos == ex.fields.end()) invalid("model: missing field eos");
  g.eos = parse_u32(eos->second, "model: eos");
  g.parallel.max_model_len = g.max_context;
  if (auto v = field("max_model_len")) g.parallel.max_model_len = parse_u32(*v, "plan: max_model_len");
  if (g.parallel.max_model_len != g.max_context) invalid("plan: max_model_len must equal the model context");
  g.parallel.validate();

  std::map<std::string, uint32_t> index;
  std::vector<Type> types;
  for (auto& fn : ex.nodes) {
    Node n;
    n.name = fn.name;
    n.op = fn.op;
    n.attrs = fn.attrs;
    n.byte = fn.byte;
    n.frames = fn.frames;
    std::vector<Type> in;
    for (auto& s : fn.inputs) {
      auto it = index.find(s);
      if (it == index.end()) invalid("byte " + std::to_string(fn.byte) + ": input " + s + " of " + fn.name + " is not defined earlier");
      n.inputs.push_back(it->second);
      in.push_back(types[it->second]);
    }
    n.type = infer(n, in, g.parallel);
    index[n.name] = (uint32_t)g.nodes.size();
    types.push_back(n.type);
    g.nodes.push_back(std::move(n));
  }
  auto out = index.find(ex.output);
  if (out == index.end()) invalid("model output is not a graph node");
  g.output = out->second;
  g.validate();
  return g;
}

Graph compile_source(std::string_view source) { return elaborate(lang::expand(lang::parse(source))); }

void Graph::validate() const {
  if (nodes.empty()) invalid("graph has no nodes");
  if (nodes.size() > 10000) fail(ErrorKind::Capacity, "graph exceeds 10000 nodes");
  if (max_context < 1 || max_context > 65536 * 2) invalid("context must be 1..131072");
  if (output >= nodes.size()) invalid("output index out of range");
  std::set<std::string> names;
  std::vector<std::vector<uint32_t>> users(nodes.size());
  for (uint32_t i = 0; i < nodes.size(); ++i) {
    if (!names.insert(nodes[i].name).second) invalid("duplicate node name " + nodes[i].name);
    for (uint32_t in : nodes[i].inputs) {
      if (in >= i) invalid("node " + nodes[i].name + " uses a later node (graph is not topologically ordered)");
      users[in].push_back(i);
    }
  }
  const Node& out = nodes[output];
  if (out.type.kind != Kind::Tensor) invalid("model output must be a logits tensor");
  // route provenance: every consumer of Routes in one expert pipeline traces to the same router
  auto router_of = [&](uint32_t id) {
    std::set<uint32_t> routers;
    std::vector<uint32_t> stack{id};
    std::set<uint32_t> seen;
    while (!stack.empty()) {
      uint32_t c = stack.back();
      stack.pop_back();
      if (!seen.insert(c).second) continue;
      if (nodes[c].op == "router") { routers.insert(c); continue; }
      if (nodes[c].type.kind == Kind::Routes || nodes[c].type.kind == Kind::Experts)
        for (uint32_t in : nodes[c].inputs)
          if (nodes[in].type.kind == Kind::Routes || nodes[in].type.kind == Kind::Experts) stack.push_back(in);
    }
    return routers;
  };
  for (uint32_t i = 0; i < nodes.size(); ++i) {
    const Node& n = nodes[i];
    if (n.op == "expert_linear" || n.op == "expert_swiglu_down" || n.op == "expert_reduce") {
      std::set<uint32_t> all;
      for (uint32_t in : n.inputs) {
        if (nodes[in].type.kind != Kind::Routes && nodes[in].type.kind != Kind::Experts) continue;
        auto r = router_of(in);
        all.insert(r.begin(), r.end());
      }
      if (all.size() != 1) invalid("byte " + std::to_string(n.byte) + ": " + n.name + " mixes routes of different routers");
    }
    // restricted consumers
    if (n.type.kind == Kind::Cache) {
      if (users[i].empty()) invalid("byte " + std::to_string(n.byte) + ": cache " + n.name + " is never attended");
      for (uint32_t u : users[i])
        if (nodes[u].op != "latent_attention" && nodes[u].op != "paged_attention") invalid("cache " + n.name + " may only feed attention");
    }
    if (n.type.kind == Kind::HyperConnection) {
      bool has_input = false, has_post = false;
      for (uint32_t u : users[i]) {
        if (nodes[u].op == "mhc_input") has_input = true;
        else if (nodes[u].op == "mhc_post") has_post = true;
        else invalid("hyper-connection " + n.name + " may only feed mhc_input / mhc_post");
      }
      if (!has_input) invalid("hyper-connection " + n.name + " has no mhc_input");
      (void)has_post;
    }
  }
  // liveness: everything must reach the output
  std::vector<char> live(nodes.size(), 0);
  std::vector<uint32_t> stack{output};
  while (!stack.empty()) {
    uint32_t c = stack.back();
    stack.pop_back();
    if (live[c]) continue;
    live[c] = 1;
    for (uint32_t in : nodes[c].inputs) stack.push_back(in);
  }
  for (uint32_t i = 0; i < nodes.size(); ++i)
    if (!live[i]) invalid("byte " + std::to_string(nodes[i].byte) + ": node " + nodes[i].name + " does not contribute to the output");
}

std::string Graph::encode() const {
  ByteWriter w;
  w.raw("IFTOKN01");
  w.u32(max_context);
  w.u32(eos);
  w.u32(output);
  w.u32((uint32_t)nodes.size());
  for (auto& n : nodes) {
    w.u32((uint32_t)n.type.kind);
    w.u32(n.type.width);
    w.str(n.name);
    w.str(n.op);
    w.u32((uint32_t)n.inputs.size());
    for (auto i : n.inputs) w.u32(i);
    w.u32((uint32_t)n.attrs.size());
    for (auto& kv : n.attrs) {
      w.str(kv.first);
      w.str(kv.second);
    }
  }
  return w.take();
}

Graph Graph::decode(std::string_view bytes) {
  ByteReader r(bytes);
  if (r.raw(8) != "IFTOKN01") invalid("not an IFTOKN01 graph");
  Graph g;
  g.max_context = r.u32();
  g.eos = r.u32();
  g.output = r.u32();
  uint32_t n = r.u32();
  if (n > 10000) fail(ErrorKind::Capacity, "graph exceeds 10000 nodes");
  for (uint32_t i = 0; i < n; ++i) {
    Node nd;
    uint32_t tag = r.u32();
    if (tag > 7) invalid("unknown value kind tag");
    nd.type.kind = (Kind)tag;
    nd.type.width = r.u32();
    nd.name = r.str(4096);
    nd.op = r.str(64);
    uint32_t ni = r.u32();
    if (ni > 8) invalid("too many inputs");
    for (uint32_t k = 0; k < ni; ++k) {
      uint32_t id = r.u32();
      if (id >= i) invalid("input refers to a later node");
      nd.inputs.push_back(id);
    }
    uint32_t na = r.u32();
    if (na > 32) invalid("too many attributes");
    for (uint32_t k = 0; k < na; ++k) {
      std::string key = r.str(64), val = r.str(4096);
      nd.attrs.emplace_back(std::move(key), std::move(val));
    }
    g.nodes.push_back(std::move(nd));
  }
  if (!r.done()) invalid("trailing bytes after the graph");
  if (g.output >= g.nodes.size()) invalid("output index out of range");
  return g;
}

std::string Graph::dot() const {
  std::string s = "digraph \"" + json_escape(name) + "\" {\n  rankdir=TB;\n  node [shape=box, fontname=\"monospace\", fontsize=9];\n";
  for (uint32_t i = 0; i < nodes.size(); ++i) {
    const Node& n = nodes[i];
    s += "  n" + std::to_string(i) + " [label=\"" + json_escape(n.op) + "\\n" + json_escape(n.name) + "\\n" + kind_name(n.type.kind) + "(" + std::to_string(n.type.width) + ")\"";
    if (n.op == "allreduce" || n.op == "gather") s += ", style=filled, fillcolor=\"#ffd9a8\"";
    if (i == output) s += ", peripheries=2";
    s += "];\n";
    for (uint32_t in : n.inputs) s += "  n" + std::to_string(in) + " -> n" + std::to_string(i) + ";\n";
  }
  return s + "}\n";
}

Json Graph::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.token-graph.v1");
  j.set("name", name);
  j.set("max_context", max_context);
  j.set("eos", eos);
  j.set("output", output);
  j.set("parallel", parallel.to_json());
  Json arr = Json::array();
  for (auto& n : nodes) {
    Json o = Json::object();
    o.set("name", n.name);
    o.set("op", n.op);
    Json in = Json::array();
    for (auto i : n.inputs) in.push((int64_t)i);
    o.set("inputs", in);
    Json at = Json::object();
    for (auto& kv : n.attrs) at.set(kv.first, kv.second);
    o.set("attrs", at);
    o.set("kind", kind_name(n.type.kind));
    o.set("width", n.type.width);
    o.set("byte", (int64_t)n.byte);
    if (!n.frames.empty()) {
      Json fr = Json::array();
      for (auto& f : n.frames) {
        Json fo = Json::object();
        fo.set("what", f.what);
        fo.set("byte", (int64_t)f.byte);
        fr.push(fo);
      }
      o.set("frames", fr);
    }
    arr.push(o);
  }
  j.set("nodes", arr);
  return j;
}

Graph Graph::from_json(const Json& j) {
  if (j.at("format").as_string() != "inferfabric.token-graph.v1") invalid("not a token graph (inferfabric.token-graph.v1)");
  Graph g;
  g.name = j.at("name").as_string();
  g.max_context = (uint32_t)j.at("max_context").as_int();
  g.eos = (uint32_t)j.at("eos").as_int();
  const Json& par = j.at("parallel");
  g.parallel.target = par.at("target").as_string();
  g.parallel.tp = (uint32_t)par.at("tp").as_int();
  g.parallel.ep = (uint32_t)par.at("ep").as_int();
  g.parallel.devices.clear();
  for (auto& d : par.at("devices").as_array()) g.parallel.devices.push_back((uint32_t)d.as_int());
  g.parallel.max_num_seqs = (uint32_t)par.at("max_num_seqs").as_int();
  g.parallel.max_num_batched_tokens = (uint32_t)par.at("max_num_batched_tokens").as_int();
  g.parallel.max_model_len = (uint32_t)par.at("max_model_len").as_int();
  g.parallel.validate();
  const JsonArray& nodes = j.at("nodes").as_array();
  if (nodes.size() > 10000) fail(ErrorKind::Capacity, "graph exceeds 10000 nodes");
  std::vector<Type> types;
  for (auto& o : nodes) {
    Node n;
    n.name = o.at("name").as_string();
    n.op = o.at("op").as_string();
    if (!lang::primitives().count(n.op)) invalid("node " + n.name + ": unknown operator " + n.op);
    std::vector<Type> in;
    for (auto& i : o.at("inputs").as_array()) {
      const int64_t k = i.as_int();
      if (k < 0 || (size_t)k >= g.nodes.size()) invalid("node " + n.name + " reads a node that is not defined earlier");
      n.inputs.push_back((uint32_t)k);
      in.push_back(types[(size_t)k]);
    }
    for (auto& kv : o.at("attrs").as_object()) n.attrs.emplace_back(kv.first, kv.second.as_string());
    std::sort(n.attrs.begin(), n.attrs.end());
    if (auto b = o.find("byte")) n.byte = (size_t)b->as_int();
    if (auto fr = o.find("frames"))
      for (auto& f : fr->as_array()) n.frames.push_back({f.at("what").as_string(), (size_t)f.at("byte").as_int()});
    n.type = infer(n, in, g.parallel);
    types.push_back(n.type);
    g.nodes.push_back(std::move(n));
  }
  const int64_t out = j.at("output").as_int();
  if (out < 0 || (size_t)out >= g.nodes.size()) invalid("output index out of range");
  g.output = (uint32_t)out;
  g.validate();
  return g;
}

std::map<std::string, size_t> Graph::op_histogram() const {
  std::map<std::string, size_t> h;
  for (auto& n : nodes) ++h[n.op];
  return h;
}

}  // namespace ifab::graph
