#include "hybrid.h"

#include <cstring>

#include <algorithm>
#include <cmath>
#include <filesystem>
#include <fstream>
#include <set>

namespace ifab::hybrid {

namespace fs = std::filesystem;
using rankplan::Layer;

namespace {

constexpr uint64_t kMaxJson = (uint64_t)16 << 20;

const char* dtype_text(init::DType d) { return d == init::DType::F32 ? "F32" : "BF16"; }

// A checkpoint file is named by a plain file name and must resolve to a file directly inside the directory.
fs::path local_file(const fs::path& root, const std::string& name) {
  if (name.empty() || name == "." || name == ".." || name.find_first_of("/\\:") != std::string::npos) invalid("checkpoint file name " + name + " is not a plain name");
  std::error_code ec;
  fs::path p = fs::canonical(root / name, ec);
  if (ec) fail(ErrorKind::Io, "cannot open " + (root / name).string());
  if (p.parent_path() != root) invalid("checkpoint file " + name + " leaves the directory (symlink)");
  return p;
}

uint64_t u64_of(const Json& j, const char* what) {
  if (!j.is_int() || j.as_int() < 0) invalid(std::string(what) + " must be a non-negative integer");
  return (uint64_t)j.as_int();
}

// One safetensors header: name -> Weight with absolute offsets; the ranges must tile [base, file_size) exactly.
std::map<std::string, Weight> parse_header(std::string_view text, const std::string& shard, uint64_t base, uint64_t file_size) {
  const Json hdr = Json::parse(text, kMaxJson);
  if (!hdr.is_object()) invalid(shard + ": the header is not a JSON object");
  std::map<std::string, Weight> out;
  std::vector<std::pair<uint64_t, uint64_t>> ranges;
  for (auto& kv : hdr.as_object()) {
    if (kv.first == "__metadata__") continue;
    Weight w;
    w.shard = shard;
    const std::string& dt = kv.second.at("dtype").as_string();
    if (dt == "BF16") w.dtype = init::DType::Bf16;
    else if (dt == "F32") w.dtype = init::DType::F32;
    else invalid(shard + ": tensor " + kv.first + " has unsupported dtype " + dt);
    uint64_t count = init::dtype_bytes(w.dtype);
    for (auto& d : kv.second.at("shape").as_array()) {
      const uint64_t v = u64_of(d, "a dimension");
      if (v != 0 && count > UINT64_MAX / v) invalid(shard + ": tensor " + kv.first + " overflows 64 bits");
      count *= v;
      w.shape.push_back(v);
    }
    const JsonArray& off = kv.second.at("data_offsets").as_array();
    if (off.size() != 2) invalid(shard + ": tensor " + kv.first + " needs two data offsets");
    const uint64_t b = u64_of(off[0], "an offset"), e = u64_of(off[1], "an offset");
    if (e < b || e - b != count || e > file_size - base) invalid(shard + ": tensor " + kv.first + " has a byte range that does not fit its shape or the file");
    w.offset = base + b;
    w.bytes = count;
    ranges.emplace_back(b, e);
    out.emplace(kv.first, std::move(w));
  }
  std::sort(ranges.begin(), ranges.end());
  uint64_t cursor = 0;
  for (auto& r : ranges) {
    if (r.first != cursor) invalid(shard + ": tensor ranges overlap or leave a gap");
    cursor = r.second;
  }
  if (base + cursor != file_size) invalid(shard + ": bytes after the last tensor are not described by the header");
  return out;
}

std::vector<uint64_t> rope_sections(uint64_t rotary_dim) {
  // three interleaved position axes share the rotary_dim / 2 frequency pairs as evenly as possible (32 -> 11, 11, 10)
  const uint64_t pairs = rotary_dim / 2, a = (pairs + 2) / 3;
  return {a, a, pairs - 2 * a};
}

std::string eps_text() { return "1e-6"; }

}  // namespace

// ---------------------------------------------------------------------------------------------
Schema schema(const rankplan::Model& m) {
  Schema s;
  const uint64_t H = m.hidden, I = m.intermediate, qh = m.query_heads, kvh = m.kv_heads, hd = m.head_dim, dh = m.delta_heads, dd = m.delta_dim;
  auto add = [&](const std::string& name, init::DType dt, std::vector<uint64_t> shape) { s[kPrefix + name] = {dt, std::move(shape)}; };
  const auto bf = init::DType::Bf16, f32 = init::DType::F32;
  add("embed_tokens.weight", bf, {m.vocab, H});
  add("norm.weight", bf, {H});
  for (size_t i = 0; i < m.layers.size(); ++i) {
    const std::string l = "layers." + std::to_string(i) + ".";
    add(l + "input_layernorm.weight", bf, {H});
    add(l + "post_attention_layernorm.weight", bf, {H});
    add(l + "mlp.gate_proj.weight", bf, {I, H});
    add(l + "mlp.up_proj.weight", bf, {I, H});
    add(l + "mlp.down_proj.weight", bf, {H, I});
    if (m.layers[i] == Layer::Full) {
      add(l + "self_attn.q_norm.weight", bf, {hd});
      add(l + "self_attn.k_norm.weight", bf, {hd});
      add(l + "self_attn.q_proj.weight", bf, {2 * qh * hd, H});      // query rows and output-gate rows per head
      add(l + "self_attn.k_proj.weight", bf, {kvh * hd, H});
      add(l + "self_attn.v_proj.weight", bf, {kvh * hd, H});
      add(l + "self_attn.o_proj.weight", bf, {H, qh * hd});
    } else {
      add(l + "linear_attn.A_log", f32, {dh});
      add(l + "linear_attn.norm.weight", f32, {dd});
      add(l + "linear_attn.dt_bias", bf, {dh});
      add(l + "linear_attn.conv1d.weight", bf, {3 * dh * dd, 1, m.conv_width});
      add(l + "linear_attn.in_proj_a.weight", bf, {dh, H});
      add(l + "linear_attn.in_proj_b.weight", bf, {dh, H});
      add(l + "linear_attn.in_proj_qkv.weight", bf, {3 * dh * dd, H});
      add(l + "linear_attn.in_proj_z.weight", bf, {dh * dd, H});
      add(l + "linear_attn.out_proj.weight", bf, {H, dh * dd});
    }
  }
  return s;
}

void validate_config(const Json& c, const rankplan::Model& m) {
  if (!c.is_object()) invalid("config.json is not an object");
  auto want_bool = [&](const Json& o, const char* k, bool v, const char* where) {
    const Json* x = o.find(k);
    if (!x || !x->is_bool() || x->as_bool() != v) invalid(std::string("config: ") + where + k + " must be " + (v ? "true" : "false"));
  };
  want_bool(c, "tie_word_embeddings", true, "");
  const Json& t = c.at("text_config");
  auto want_int = [&](const char* k, uint64_t v) {
    const Json* x = t.find(k);
    if (!x || !x->is_int() || (uint64_t)x->as_int() != v) invalid(std::string("config: text_config.") + k + " disagrees with the model document (expected " + std::to_string(v) + ")");
  };
  want_int("hidden_size", m.hidden);
  want_int("intermediate_size", m.intermediate);
  want_int("vocab_size", m.vocab);
  want_int("num_hidden_layers", m.layers.size());
  want_int("num_attention_heads", m.query_heads);
  want_int("num_key_value_heads", m.kv_heads);
  want_int("head_dim", m.head_dim);
  want_int("linear_num_key_heads", m.delta_heads);
  want_int("linear_num_value_heads", m.delta_heads);
  want_int("linear_key_head_dim", m.delta_dim);
  want_int("linear_value_head_dim", m.delta_dim);
  want_int("linear_conv_kernel_dim", m.conv_width);
  want_bool(t, "attention_bias", false, "text_config.");
  want_bool(t, "attn_output_gate", true, "text_config.");
  want_bool(t, "tie_word_embeddings", true, "text_config.");
  const Json* act = t.find("hidden_act");
  if (!act || !act->is_string() || act->as_string() != "silu") invalid("config: text_config.hidden_act must be silu");
  const Json* eps = t.find("rms_norm_eps");
  if (!eps || !eps->is_number() || std::fabs(eps->as_double() - 1e-6) > 1e-12) invalid("config: text_config.rms_norm_eps must be 1e-6");
  const Json* pos = t.find("max_position_embeddings");
  if (!pos || !pos->is_int() || pos->as_int() < 1 || (uint64_t)pos->as_int() > kMaxModelLen) invalid("config: text_config.max_position_embeddings is missing or above 262144");
  const Json& rope = t.at("rope_parameters");
  const Json* prf = rope.find("partial_rotary_factor");
  if (!prf || !prf->is_number() || std::fabs(prf->as_double() - 0.25) > 1e-9) invalid("config: rope partial_rotary_factor must be 0.25");
  const Json* theta = rope.find("rope_theta");
  if (!theta || !theta->is_number() || theta->as_double() < 1.0) invalid("config: rope_theta is missing");
  const JsonArray& kinds = t.at("layer_types").as_array();
  if (kinds.size() != m.layers.size()) invalid("config: layer_types has a different length than the model document");
  for (size_t i = 0; i < kinds.size(); ++i) {
    const std::string& k = kinds[i].as_string();
    if (k != (m.layers[i] == Layer::Full ? "full_attention" : "linear_attention")) invalid("config: layer_types[" + std::to_string(i) + "] disagrees with the model document");
  }
}

Checkpoint inspect(const std::string& directory, const rankplan::Model& m) {
  std::error_code ec;
  const fs::path root = fs::canonical(directory, ec);
  if (ec) fail(ErrorKind::Io, "cannot open checkpoint directory " + directory);
  const std::string config = read_file(local_file(root, "config.json").string(), kMaxJson);
  validate_config(Json::parse(config, kMaxJson), m);
  const std::string index_bytes = read_file(local_file(root, "model.safetensors.index.json").string(), kMaxJson);
  const Json index = Json::parse(index_bytes, kMaxJson);
  std::map<std::string, std::string> map;
  for (auto& kv : index.at("weight_map").as_object()) map[kv.first] = kv.second.as_string();
  if (map.empty()) invalid("the index maps no tensors");
  Checkpoint ck;
  std::map<std::string, Weight> all;
  uint64_t total = 0;
  for (auto& kv : map) {
    const std::string& name = kv.second;
    if (ck.shards.count(name)) continue;
    const fs::path path = local_file(root, name);
    std::ifstream f(path, std::ios::binary);
    if (!f) fail(ErrorKind::Io, "cannot open " + path.string());
    const uint64_t file_size = (uint64_t)fs::file_size(path);
    unsigned char prefix[8];
    f.read((char*)prefix, 8);
    if (!f) invalid(name + ": shorter than a safetensors prefix");
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | prefix[i];
    if (n == 0 || n > kMaxJson || n > file_size - 8) invalid(name + ": header size out of range");
    std::string hdr(n, '\0');
    f.read(hdr.data(), (std::streamsize)n);
    if (!f) invalid(name + ": truncated header");
    for (auto& t : parse_header(hdr, name, 8 + n, file_size)) {
      auto it = map.find(t.first);
      if (it == map.end() || it->second != name) invalid("tensor " + t.first + " is in " + name + " but the index says otherwise");
      if (!all.emplace(t.first, t.second).second) invalid("tensor " + t.first + " appears twice");
    }
    total += file_size - 8 - n;
    ck.shards[name] = {file_size, Sha256::of(hdr)};
  }
  if (all.size() != map.size()) invalid("the index lists tensors that no shard holds");
  const Json* meta = index.find("metadata");
  const Json* ts = meta ? meta->find("total_size") : nullptr;
  if (!ts || !ts->is_int() || (uint64_t)ts->as_int() != total) invalid("index metadata.total_size does not match the shards");
  const Schema want = schema(m);
  for (auto& kv : want) {
    auto it = all.find(kv.first);
    if (it == all.end()) invalid("checkpoint lacks " + kv.first);
    if (it->second.dtype != kv.second.first || it->second.shape != kv.second.second) invalid("tensor " + kv.first + " has another dtype or shape than the model document implies");
  }
  for (auto& kv : all) {
    if (want.count(kv.first)) ck.weights.emplace(kv.first, kv.second);
    else if (kv.first.rfind("model.visual.", 0) == 0) ++ck.excluded["vision"];
    else if (kv.first.rfind("mtp.", 0) == 0) ++ck.excluded["mtp"];
    else invalid("checkpoint holds a tensor this contract does not know: " + kv.first);
  }
  ck.config_sha256 = Sha256::of(config);
  ck.index_sha256 = Sha256::of(index_bytes);
  ck.metadata_sha256 = Sha256::of(ck.to_json().dump());
  return ck;
}

Json Checkpoint::to_json() const {
  Json j = Json::object();
  j.set("config_sha256", config_sha256);
  j.set("index_sha256", index_sha256);
  Json sh = Json::object();
  for (auto& kv : shards) {
    Json o = Json::object();
    o.set("bytes", kv.second.bytes);
    o.set("header_sha256", kv.second.header_sha256);
    sh.set(kv.first, o);
  }
  j.set("shards", sh);
  Json ws = Json::object();
  for (auto& kv : weights) {
    Json o = Json::object();
    o.set("shard", kv.second.shard);
    o.set("dtype", dtype_text(kv.second.dtype));
    Json shp = Json::array();
    for (auto d : kv.second.shape) shp.push((int64_t)d);
    o.set("shape", shp);
    o.set("offset", kv.second.offset);
    o.set("bytes", kv.second.bytes);
    ws.set(kv.first, o);
  }
  j.set("weights", ws);
  Json ex = Json::object();
  for (auto& kv : excluded) ex.set(kv.first, kv.second);
  j.set("excluded", ex);
  j.set("metadata_sha256", metadata_sha256);
  return j;
}

// ---------------------------------------------------------------------------------------------
const char* op_name(Op op) {
  static const char* names[] = {"Embedding", "Linear", "ZeroCenteredRms", "Reshape", "Split", "TextRope", "PagedAttention", "Sigmoid", "Silu",
                                "Multiply", "Add", "CausalConvSilu", "L2Norm", "DeltaDecay", "DeltaRecurrence", "GatedRms", "SelectFrontier"};
  return names[(int)op];
}

namespace {

class Builder {
 public:
  std::vector<Node> nodes;
  std::vector<State> states;

  static std::vector<Dim> per_token(std::initializer_list<uint64_t> fixed) {
    std::vector<Dim> s{{Dim::Kind::Tokens, 0}};
    for (auto v : fixed) s.push_back(Dim::fixed(v));
    return s;
  }
  std::vector<std::string> emit(Op op, std::vector<std::string> inputs, std::vector<std::pair<std::vector<Dim>, Scalar>> outs,
                                std::map<std::string, std::string> attrs = {}) {
    Node n;
    n.op = op;
    n.inputs = std::move(inputs);
    n.attrs = std::move(attrs);
    std::vector<std::string> names;
    for (auto& o : outs) {
      Tensor t{"t" + std::to_string(serial_++), std::move(o.first), o.second};
      names.push_back(t.name);
      n.outputs.push_back(std::move(t));
    }
    nodes.push_back(std::move(n));
    return names;
  }
  std::string one(Op op, std::vector<std::string> inputs, std::initializer_list<uint64_t> fixed, Scalar dt = Scalar::Bf16,
                  std::map<std::string, std::string> attrs = {}) {
    return emit(op, std::move(inputs), {{per_token(fixed), dt}}, std::move(attrs))[0];
  }
  std::string linear(const std::string& x, const std::string& weight, uint64_t width) { return one(Op::Linear, {x}, {width}, Scalar::Bf16, {{"weight", weight}}); }
  std::string rms(const std::string& x, const std::string& weight, std::initializer_list<uint64_t> shape) {
    return one(Op::ZeroCenteredRms, {x}, shape, Scalar::Bf16, {{"weight", weight}, {"epsilon", eps_text()}, {"gain", "1 + w, f32"}});
  }
  std::string state(const std::string& name, std::vector<Dim> shape, Scalar dt, StateKind kind) {
    states.push_back({Tensor{name, std::move(shape), dt}, kind, kind == StateKind::DeltaKeyValue || kind == StateKind::ConvPreviousInputs});
    return name;
  }

 private:
  size_t serial_ = 0;
};

Json dim_json(const Dim& d) {
  switch (d.kind) {
    case Dim::Kind::Tokens: return Json("tokens");
    case Dim::Kind::Requests: return Json("requests");
    case Dim::Kind::RequestBoundaries: return Json("request_boundaries");
    case Dim::Kind::Pages: return Json("pages");
    case Dim::Kind::Fixed: return Json((int64_t)d.n);
  }
  return Json();
}
Json tensor_json(const Tensor& t) {
  Json o = Json::object();
  o.set("name", t.name);
  Json s = Json::array();
  for (auto& d : t.shape) s.push(dim_json(d));
  o.set("shape", s);
  o.set("dtype", t.dtype == Scalar::Bf16 ? "bf16" : t.dtype == Scalar::Fp32 ? "fp32" : "i64");
  return o;
}

}  // namespace

Json Plan::to_json() const {
  Json j = Json::object();
  j.set("format", format);
  j.set("executable", executable);
  j.set("contract", contract);
  j.set("key", key);
  j.set("spec", spec.to_json());
  j.set("checkpoint", checkpoint.to_json());
  Json in = Json::array();
  for (auto& t : inputs) in.push(tensor_json(t));
  j.set("inputs", in);
  Json st = Json::array();
  static const char* kinds[] = {"paged_keys", "paged_values", "delta_key_value", "conv_previous_inputs"};
  for (auto& s : states) {
    Json o = tensor_json(s.tensor);
    o.set("kind", kinds[(int)s.kind]);
    o.set("initially_zero", s.initially_zero);
    st.push(o);
  }
  j.set("states", st);
  Json ns = Json::array();
  for (auto& n : nodes) {
    Json o = Json::object();
    o.set("op", op_name(n.op));
    Json ins = Json::array();
    for (auto& i : n.inputs) ins.push(i);
    o.set("inputs", ins);
    Json outs = Json::array();
    for (auto& t : n.outputs) outs.push(tensor_json(t));
    o.set("outputs", outs);
    if (!n.attrs.empty()) {
      Json a = Json::object();
      for (auto& kv : n.attrs) a.set(kv.first, kv.second);
      o.set("attrs", a);
    }
    ns.push(o);
  }
  j.set("nodes", ns);
  j.set("output", output);
  j.set("text_weight_bytes", text_weight_bytes);
  j.set("recurrent_and_conv_bytes_per_request", recurrent_and_conv_bytes_per_request);
  j.set("kv_bytes_per_page", kv_bytes_per_page);
  return j;
}

Plan compile(const rankplan::Spec& spec, const Checkpoint& checkpoint) {
  spec.validate();
  const rankplan::Model& m = spec.model;
  for (const rankplan::Mesh* mesh : {&spec.prefill, &spec.decode})
    if ((mesh->tp != 1 && mesh->tp != 2) || mesh->cp != 1 || mesh->sp) invalid("a checkpoint-bound plan runs with TP 1 or 2, CP = 1 and without SP");
  if (spec.prefill.tp != spec.decode.tp) invalid("prefill and decode must use the same TP width");
  if (spec.max_context() > kMaxModelLen) invalid("context exceeds the checkpoint's position limit");
  if (m.head_dim % 8) invalid("head_dim must be a multiple of 8 (a quarter of it rotates, in pairs)");
  const Schema want = schema(m);
  if (checkpoint.weights.size() != want.size()) invalid("the checkpoint's tensor set is not the one this model calls for");
  for (auto& kv : want) {
    auto it = checkpoint.weights.find(kv.first);
    if (it == checkpoint.weights.end() || it->second.dtype != kv.second.first || it->second.shape != kv.second.second)
      invalid("checkpoint tensor " + kv.first + " is missing or has another dtype / shape");
  }
  const uint64_t H = m.hidden, I = m.intermediate, qh = m.query_heads, kvh = m.kv_heads, hd = m.head_dim, dh = m.delta_heads, dd = m.delta_dim,
                 cw = m.conv_width, C = 3 * dh * dd, rotary = hd / 4;
  const std::vector<uint64_t> sections = rope_sections(rotary);
  Plan plan;
  plan.spec = spec;
  plan.checkpoint = checkpoint;
  const uint64_t max_pages = (spec.max_context() + spec.page_tokens - 1) / spec.page_tokens;
  plan.inputs = {
      {"token_ids", {{Dim::Kind::Tokens, 0}}, Scalar::I64},
      {"positions", {{Dim::Kind::Tokens, 0}}, Scalar::I64},
      {"request_offsets", {{Dim::Kind::RequestBoundaries, 0}}, Scalar::I64},     // CSR boundaries: requests + 1 entries
      {"request_slots", {{Dim::Kind::Requests, 0}}, Scalar::I64},
      {"page_table", {{Dim::Kind::Requests, 0}, Dim::fixed(max_pages)}, Scalar::I64},
  };
  Builder b;
  const std::string embedding = std::string(kPrefix) + "embed_tokens.weight";
  std::string x = b.one(Op::Embedding, {"token_ids"}, {H}, Scalar::Bf16, {{"weight", embedding}});
  size_t n_full = 0, n_delta = 0;
  for (size_t i = 0; i < m.layers.size(); ++i) {
    auto w = [&](const char* name) { return std::string(kPrefix) + "layers." + std::to_string(i) + "." + name; };
    const std::string norm = b.rms(x, w("input_layernorm.weight"), {H});
    std::string mixed;
    if (m.layers[i] == Layer::Full) {
      ++n_full;
      std::string qg = b.linear(norm, w("self_attn.q_proj.weight"), 2 * qh * hd);
      qg = b.one(Op::Reshape, {qg}, {qh, 2 * hd});
      auto halves = b.emit(Op::Split, {qg}, {{Builder::per_token({qh, hd}), Scalar::Bf16}, {Builder::per_token({qh, hd}), Scalar::Bf16}},
                           {{"axis", "2"}, {"lengths", std::to_string(hd) + "," + std::to_string(hd)}});
      std::string q = b.rms(halves[0], w("self_attn.q_norm.weight"), {qh, hd});
      std::string k = b.linear(norm, w("self_attn.k_proj.weight"), kvh * hd);
      k = b.one(Op::Reshape, {k}, {kvh, hd});
      k = b.rms(k, w("self_attn.k_norm.weight"), {kvh, hd});
      std::string v = b.linear(norm, w("self_attn.v_proj.weight"), kvh * hd);
      v = b.one(Op::Reshape, {v}, {kvh, hd});
      const std::map<std::string, std::string> rope = {{"rotary_dim", std::to_string(rotary)},
                                                       {"rotation", "half"},
                                                       {"position_axes", "text: all three equal the absolute position"},
                                                       {"interleaved_sections", std::to_string(sections[0]) + "," + std::to_string(sections[1]) + "," + std::to_string(sections[2])}};
      q = b.one(Op::TextRope, {q, "positions"}, {qh, hd}, Scalar::Bf16, rope);
      k = b.one(Op::TextRope, {k, "positions"}, {kvh, hd}, Scalar::Bf16, rope);
      const std::vector<Dim> pages = {{Dim::Kind::Pages, 0}, Dim::fixed(spec.page_tokens), Dim::fixed(kvh), Dim::fixed(hd)};
      const std::string keys = b.state("layer." + std::to_string(i) + ".keys", pages, Scalar::Bf16, StateKind::PagedKeys);
      const std::string values = b.state("layer." + std::to_string(i) + ".values", pages, Scalar::Bf16, StateKind::PagedValues);
      const std::string attn = b.one(Op::PagedAttention, {q, k, v, "positions", "request_offsets", "request_slots", "page_table"}, {qh, hd}, Scalar::Bf16,
                                     {{"keys", keys}, {"values", values}, {"scale", "1/sqrt(" + std::to_string(hd) + ")"}, {"causal", "true"}});
      const std::string gate = b.one(Op::Sigmoid, {halves[1]}, {qh, hd});
      const std::string gated = b.one(Op::Multiply, {attn, gate}, {qh, hd});
      const std::string flat = b.one(Op::Reshape, {gated}, {qh * hd});
      mixed = b.linear(flat, w("self_attn.o_proj.weight"), H);
    } else {
      ++n_delta;
      const std::string qkv = b.linear(norm, w("linear_attn.in_proj_qkv.weight"), C);
      std::string z = b.linear(norm, w("linear_attn.in_proj_z.weight"), dh * dd);
      z = b.one(Op::Reshape, {z}, {dh, dd});
      const std::string a = b.linear(norm, w("linear_attn.in_proj_a.weight"), dh);
      std::string beta = b.linear(norm, w("linear_attn.in_proj_b.weight"), dh);
      beta = b.one(Op::Sigmoid, {beta}, {dh});
      const std::string decay = b.one(Op::DeltaDecay, {a}, {dh}, Scalar::Fp32,
                                      {{"a_log", w("linear_attn.A_log")}, {"dt_bias", w("linear_attn.dt_bias")}, {"clamp", "false"},
                                       {"formula", "g = -exp(A_log) * softplus(a + dt_bias), f32"}});
      const std::string history = b.state("layer." + std::to_string(i) + ".conv", {{Dim::Kind::Requests, 0}, Dim::fixed(C), Dim::fixed(cw - 1)}, Scalar::Bf16,
                                          StateKind::ConvPreviousInputs);
      const std::string conv = b.one(Op::CausalConvSilu, {qkv, "request_offsets", "request_slots"}, {C}, Scalar::Bf16,
                                     {{"weight", w("linear_attn.conv1d.weight")}, {"history", history}, {"kernel_width", std::to_string(cw)},
                                      {"history_order", "oldest first"}});
      auto parts = b.emit(Op::Split, {conv},
                          {{Builder::per_token({dh * dd}), Scalar::Bf16}, {Builder::per_token({dh * dd}), Scalar::Bf16}, {Builder::per_token({dh * dd}), Scalar::Bf16}},
                          {{"axis", "1"}, {"lengths", std::to_string(dh * dd) + "," + std::to_string(dh * dd) + "," + std::to_string(dh * dd)}});
      std::vector<std::string> heads;
      for (auto& p : parts) heads.push_back(b.one(Op::Reshape, {p}, {dh, dd}));
      const std::map<std::string, std::string> l2 = {{"epsilon", eps_text()}, {"rounding", "bf16 before epsilon is added"}};
      const std::string q = b.one(Op::L2Norm, {heads[0]}, {dh, dd}, Scalar::Bf16, l2);
      const std::string k = b.one(Op::L2Norm, {heads[1]}, {dh, dd}, Scalar::Bf16, l2);
      const std::string st = b.state("layer." + std::to_string(i) + ".delta", {{Dim::Kind::Requests, 0}, Dim::fixed(dh), Dim::fixed(dd), Dim::fixed(dd)}, Scalar::Fp32,
                                     StateKind::DeltaKeyValue);
      const std::string delta = b.one(Op::DeltaRecurrence, {q, k, heads[2], decay, beta, "request_offsets", "request_slots"}, {dh, dd}, Scalar::Bf16,
                                      {{"state", st}, {"q_scale", "1/sqrt(" + std::to_string(dd) + ")"}, {"state_layout", "request,head,key,value"},
                                       {"recurrence", "S *= exp(g); r = beta * (v - k^T S); S += k outer r; y = (q * q_scale)^T S; f32 state"}});
      const std::string gated = b.one(Op::GatedRms, {delta, z}, {dh, dd}, Scalar::Bf16,
                                      {{"weight", w("linear_attn.norm.weight")}, {"epsilon", eps_text()}, {"normalize_before_gate", "true"}, {"gain", "w, f32 (no 1 + w)"}});
      const std::string flat = b.one(Op::Reshape, {gated}, {dh * dd});
      mixed = b.linear(flat, w("linear_attn.out_proj.weight"), H);
    }
    x = b.one(Op::Add, {x, mixed}, {H});
    const std::string n2 = b.rms(x, w("post_attention_layernorm.weight"), {H});
    std::string gate = b.linear(n2, w("mlp.gate_proj.weight"), I);
    const std::string up = b.linear(n2, w("mlp.up_proj.weight"), I);
    gate = b.one(Op::Silu, {gate}, {I});
    const std::string act = b.one(Op::Multiply, {gate, up}, {I});
    const std::string down = b.linear(act, w("mlp.down_proj.weight"), H);
    x = b.one(Op::Add, {x, down}, {H});
  }
  x = b.rms(x, std::string(kPrefix) + "norm.weight", {H});
  const std::string frontier = b.emit(Op::SelectFrontier, {x, "request_offsets"}, {{{{Dim::Kind::Requests, 0}, Dim::fixed(H)}, Scalar::Bf16}})[0];
  plan.output = b.emit(Op::Linear, {frontier}, {{{{Dim::Kind::Requests, 0}, Dim::fixed(m.vocab)}, Scalar::Bf16}}, {{"weight", embedding}})[0];
  plan.nodes = std::move(b.nodes);
  plan.states = std::move(b.states);
  for (auto& kv : checkpoint.weights) plan.text_weight_bytes += kv.second.bytes;
  plan.recurrent_and_conv_bytes_per_request = n_delta * (dh * dd * dd * 4 + C * (cw - 1) * 2);
  plan.kv_bytes_per_page = n_full * 2 * spec.page_tokens * kvh * hd * 2;
  validate(plan);
  plan.key = Sha256::of(plan.to_json().dump());
  return plan;
}

std::string html_view(const Json& doc) {
  if (!doc.is_object() || !doc.find("format") || doc.at("format").as_string() != "inferfabric.typed-plan.v1") invalid("explain-model: not a typed plan document");
  auto esc = [](const std::string& t) {
    std::string o;
    for (char c : t) {
      if (c == '<') o += "&lt;";
      else if (c == '>') o += "&gt;";
      else if (c == '&') o += "&amp;";
      else if (c == '"') o += "&quot;";
      else o += c;
    }
    return o;
  };
  auto tensor = [&](const Json& t) {
    std::string s = esc(t.at("name").as_string()) + " : " + t.at("dtype").as_string() + "[";
    bool first = true;
    for (auto& d : t.at("shape").as_array()) {
      s += std::string(first ? "" : ", ") + (d.is_string() ? d.as_string() : std::to_string(d.as_int()));
      first = false;
    }
    return s + "]";
  };
  // the layer an operator belongs to: the number after "layers." in any of its weight / state attributes
  auto layer_of = [](const Json& n) -> int64_t {
    const Json* a = n.find("attrs");
    if (!a) return -1;
    for (auto& kv : a->as_object()) {
      if (!kv.second.is_string()) continue;
      const std::string& v = kv.second.as_string();
      for (const char* tag : {"layers.", "layer."}) {
        const size_t p = v.find(tag);
        if (p != std::string::npos) return std::atoll(v.c_str() + p + std::strlen(tag));
      }
    }
    return -1;
  };
  const Json& model = doc.at("spec").at("model");
  const auto& nodes = doc.at("nodes").as_array();
  std::string h = "<!doctype html><html><head><meta charset=\"utf-8\"><title>typed plan</title><style>body{font:13px monospace;margin:1.5em}"
                  "table{border-collapse:collapse;margin:.5em 0 1.5em}td,th{border:1px solid #999;padding:2px 8px;text-align:left;vertical-align:top}"
                  "th{background:#eee}h3{margin:.2em 0}.attr{color:#555}</style></head><body>";
  h += "<h1>" + esc(model.find("name") && model.at("name").is_string() ? model.at("name").as_string() : std::string("model")) + "</h1>";
  h += "<p>contract " + esc(doc.at("contract").as_string()) + ", key " + esc(doc.at("key").as_string()).substr(0, 16) + ", " + std::to_string(nodes.size()) +
       " operators, " + std::to_string(doc.at("states").size()) + " state tensors, " + std::to_string(doc.at("checkpoint").at("weights").size()) +
       " weights (" + std::to_string(doc.at("text_weight_bytes").as_int()) + " bytes); state per request " +
       std::to_string(doc.at("recurrent_and_conv_bytes_per_request").as_int()) + " bytes, KV per page " + std::to_string(doc.at("kv_bytes_per_page").as_int()) + " bytes</p>";
  h += "<h2>States</h2><table id=\"states\"><tr><th>tensor</th><th>kind</th><th>starts at zero</th></tr>";
  for (auto& s : doc.at("states").as_array())
    h += "<tr><td>" + tensor(s) + "</td><td>" + esc(s.at("kind").as_string()) + "</td><td>" + (s.at("initially_zero").as_bool() ? "yes" : "") + "</td></tr>";
  h += "</table><h2>Operators</h2>";
  int64_t current = -2;
  bool open = false;
  for (auto& n : nodes) {
    int64_t layer = layer_of(n);
    if (layer < 0) layer = current < 0 ? -1 : current;      // glue operators stay with the layer around them
    if (layer != current) {
      if (open) h += "</table>";
      h += layer < 0 ? "<h3>input</h3>" : "<h3>layer " + std::to_string(layer) + "</h3>";
      h += "<table class=\"layer\"><tr><th>operator</th><th>inputs</th><th>outputs</th><th>attributes</th></tr>";
      current = layer;
      open = true;
    }
    std::string in, out, attrs;
    for (auto& i : n.at("inputs").as_array()) in += (in.empty() ? "" : ", ") + esc(i.as_string());
    for (auto& o : n.at("outputs").as_array()) out += (out.empty() ? "" : "<br>") + tensor(o);
    if (const Json* a = n.find("attrs"))
      for (auto& kv : a->as_object()) attrs += (attrs.empty() ? "" : "<br>") + esc(kv.first) + " = " + esc(kv.second.is_string() ? kv.second.as_string() : kv.second.dump());
    h += "<tr><td>" + esc(n.at("op").as_string()) + "</td><td>" + in + "</td><td>" + out + "</td><td class=\"attr\">" + attrs + "</td></tr>";
  }
  if (open) h += "</table>";
  h += "<p>output: " + esc(doc.at("output").as_string()) + "</p></body></html>\n";
  return h;
}

void validate(const Plan& plan) {
  const rankplan::Model& m = plan.spec.model;
  std::map<std::string, const Tensor*> defined;
  for (auto& t : plan.inputs)
    if (!defined.emplace(t.name, &t).second) invalid("typed plan: input " + t.name + " is declared twice");
  std::map<std::string, const State*> states;
  for (auto& s : plan.states)
    if (!states.emplace(s.tensor.name, &s).second) invalid("typed plan: state " + s.tensor.name + " is declared twice");
  std::set<std::string> bound;
  auto weight = [&](const Node& n, const char* key) -> const Weight& {
    auto a = n.attrs.find(key);
    if (a == n.attrs.end()) invalid(std::string("typed plan: ") + op_name(n.op) + " lacks attribute " + key);
    auto it = plan.checkpoint.weights.find(a->second);
    if (it == plan.checkpoint.weights.end()) invalid("typed plan: " + a->second + " is not in the checkpoint");
    bound.insert(a->second);
    return it->second;
  };
  auto state_of = [&](const Node& n, const char* key, StateKind kind) -> const State& {
    auto a = n.attrs.find(key);
    if (a == n.attrs.end() || !states.count(a->second)) invalid(std::string("typed plan: ") + op_name(n.op) + " names no declared state in " + key);
    const State& s = *states[a->second];
    if (s.kind != kind) invalid("typed plan: state " + a->second + " has the wrong kind for " + op_name(n.op));
    return s;
  };
  auto fixed_tail = [](const Tensor& t) { return t.shape.empty() || t.shape.back().kind != Dim::Kind::Fixed ? (uint64_t)0 : t.shape.back().n; };
  auto elements = [](const Tensor& t) {
    uint64_t n = 1;
    for (size_t i = 1; i < t.shape.size(); ++i) n *= t.shape[i].kind == Dim::Kind::Fixed ? t.shape[i].n : 0;
    return n;
  };
  for (auto& n : plan.nodes) {
    std::vector<const Tensor*> in;
    for (auto& name : n.inputs) {
      auto it = defined.find(name);
      if (it == defined.end()) invalid("typed plan: " + std::string(op_name(n.op)) + " uses " + name + " before it is defined");
      in.push_back(it->second);
    }
    if (in.empty() || n.outputs.empty()) invalid(std::string("typed plan: ") + op_name(n.op) + " needs inputs and outputs");
    const Tensor& x = *in[0];
    const Tensor& y = n.outputs[0];
    auto same = [&](const Tensor& a, const Tensor& b2) { return a.shape == b2.shape && a.dtype == b2.dtype; };
    auto bad = [&](const char* why) { invalid(std::string("typed plan: ") + op_name(n.op) + " -> " + y.name + ": " + why); };
    switch (n.op) {
      case Op::Embedding: {
        const Weight& w = weight(n, "weight");
        if (x.dtype != Scalar::I64 || in.size() != 1) bad("token ids are one i64 tensor");
        if (w.shape.size() != 2 || fixed_tail(y) != w.shape[1] || y.dtype != Scalar::Bf16) bad("output width is the table's row width");
        break;
      }
      case Op::Linear: {
        const Weight& w = weight(n, "weight");
        if (in.size() != 1 || x.dtype != Scalar::Bf16 || w.shape.size() != 2 || fixed_tail(x) != w.shape[1]) bad("input width must equal the weight's columns");
        if (fixed_tail(y) != w.shape[0] || y.shape.size() != x.shape.size() || y.dtype != Scalar::Bf16) bad("output width must equal the weight's rows");
        break;
      }
      case Op::ZeroCenteredRms:
      case Op::GatedRms: {
        const Weight& w = weight(n, "weight");
        auto e = n.attrs.find("epsilon");
        if (w.shape.size() != 1 || fixed_tail(x) != w.shape[0] || x.dtype != Scalar::Bf16 || e == n.attrs.end() || e->second != eps_text()) bad("norm contract (1-D gain over the last axis, epsilon 1e-6)");
        if (in.size() != (n.op == Op::GatedRms ? 2u : 1u) || !same(x, y)) bad("wrong operand count or output shape");
        if (n.op == Op::GatedRms && (!same(*in[1], x) || w.dtype != init::DType::F32)) bad("gate and value shapes differ, or the gain is not f32");
        break;
      }
      case Op::Reshape:
        if (in.size() != 1 || x.shape.empty() || y.shape.empty() || !(x.shape[0] == y.shape[0]) || elements(x) != elements(y) || elements(x) == 0 || x.dtype != y.dtype)
          bad("reshape keeps the leading axis, the element count and the dtype");
        break;
      case Op::Split: {
        uint64_t sum = 0;
        for (auto& o : n.outputs) {
          if (o.shape.size() != x.shape.size() || o.dtype != x.dtype) bad("split outputs keep rank and dtype");
          sum += fixed_tail(o);
        }
        if (in.size() != 1 || sum != fixed_tail(x)) bad("split lengths must add up to the last axis");
        break;
      }
      case Op::TextRope: {
        auto r = n.attrs.find("rotary_dim");
        if (in.size() != 2 || in[1]->dtype != Scalar::I64 || !same(x, y) || r == n.attrs.end() || std::stoull(r->second) > fixed_tail(x) || std::stoull(r->second) % 2) bad("rope takes (x, positions) and rotates an even prefix of the last axis");
        break;
      }
      case Op::PagedAttention: {
        const State& ks = state_of(n, "keys", StateKind::PagedKeys);
        const State& vs = state_of(n, "values", StateKind::PagedValues);
        if (in.size() != 7 || !same(*in[1], *in[2]) || in[1]->shape.size() != 3 || x.shape.size() != 3 || fixed_tail(x) != fixed_tail(*in[1])) bad("q [tokens, heads, d], k and v [tokens, kv heads, d]");
        if (x.shape[1].n % in[1]->shape[1].n) bad("query heads must divide into key / value groups");
        if (ks.tensor.shape != vs.tensor.shape || ks.tensor.shape.size() != 4 || ks.tensor.shape[2].n != in[1]->shape[1].n || ks.tensor.shape[3].n != fixed_tail(x)) bad("page shape [pages, page_tokens, kv heads, d]");
        if (!same(x, y)) bad("output has the query's shape");
        break;
      }
      case Op::Sigmoid:
      case Op::Silu:
        if (in.size() != 1 || !same(x, y)) bad("elementwise, one operand");
        break;
      case Op::Multiply:
      case Op::Add:
        if (in.size() != 2 || !same(x, *in[1]) || !same(x, y)) bad("elementwise, two operands of one shape");
        break;
      case Op::CausalConvSilu: {
        const Weight& w = weight(n, "weight");
        const State& h = state_of(n, "history", StateKind::ConvPreviousInputs);
        if (in.size() != 3 || w.shape.size() != 3 || w.shape[0] != fixed_tail(x) || w.shape[1] != 1 || !same(x, y)) bad("depthwise weight [channels, 1, width]");
        if (h.tensor.shape.size() != 3 || h.tensor.shape[1].n != w.shape[0] || h.tensor.shape[2].n + 1 != w.shape[2]) bad("history holds width - 1 earlier inputs per channel");
        break;
      }
      case Op::L2Norm:
        if (in.size() != 1 || !same(x, y) || n.attrs.count("epsilon") == 0) bad("one operand, epsilon given");
        break;
      case Op::DeltaDecay: {
        const Weight& a = weight(n, "a_log");
        const Weight& dt = weight(n, "dt_bias");
        auto c = n.attrs.find("clamp");
        if (in.size() != 1 || a.shape != dt.shape || a.shape.size() != 1 || a.shape[0] != fixed_tail(x) || y.dtype != Scalar::Fp32 || y.shape != x.shape) bad("per-head decay in f32");
        if (c == n.attrs.end() || c->second != "false") bad("the decay is never clamped");
        break;
      }
      case Op::DeltaRecurrence: {
        const State& s = state_of(n, "state", StateKind::DeltaKeyValue);
        if (in.size() != 7 || !same(x, *in[1]) || !same(x, *in[2]) || !same(x, y) || in[3]->dtype != Scalar::Fp32) bad("q, k, v of one shape; f32 decay");
        if (s.tensor.dtype != Scalar::Fp32 || s.tensor.shape.size() != 4 || s.tensor.shape[1].n != x.shape[1].n || s.tensor.shape[2].n != fixed_tail(x) || s.tensor.shape[3].n != fixed_tail(x)) bad("state [requests, heads, key, value] in f32");
        break;
      }
      case Op::SelectFrontier:
        if (in.size() != 2 || y.shape.size() != 2 || y.shape[0].kind != Dim::Kind::Requests || fixed_tail(y) != fixed_tail(x) || y.dtype != x.dtype) bad("one row per request");
        break;
    }
    for (auto& t : n.outputs)
      if (!defined.emplace(t.name, &t).second) invalid("typed plan: " + t.name + " is assigned twice");
  }
  if (!defined.count(plan.output)) invalid("typed plan: the output is not produced by any node");
  if (bound.size() != plan.checkpoint.weights.size()) invalid("typed plan: " + std::to_string(plan.checkpoint.weights.size() - bound.size()) + " checkpoint tensors are bound by no node");
  // the mixed-precision exception of the family survives: exactly two f32 tensors per delta layer
  size_t f32 = 0, delta = 0;
  for (auto& kv : plan.checkpoint.weights) f32 += kv.second.dtype == init::DType::F32;
  for (auto l : m.layers) delta += l == Layer::Delta;
  if (f32 != 2 * delta) invalid("typed plan: unexpected f32 tensors in the checkpoint");
}

// ---------------------------------------------------------------------------------------------
Json Program::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.hybrid-program.v1");
  j.set("key", key);
  j.set("source_key", source_key);
  auto bind = [](const Binding& b) {
    Json o = Json::object();
    o.set("name", b.name);
    o.set("transform", b.transform == Transform::Identity ? "identity" : "one_plus_fp32");
    return o;
  };
  Json bs = Json::array();
  for (auto& b : blocks) {
    Json o = Json::object();
    o.set("layer", b.layer);
    o.set("kind", b.kind == Layer::Full ? "full" : "delta");
    Json arr = Json::array();
    for (auto& x : b.bindings) arr.push(bind(x));
    o.set("bindings", arr);
    bs.push(o);
  }
  j.set("blocks", bs);
  j.set("embedding", embedding);
  j.set("final_norm", bind(final_norm));
  j.set("batch", batch);
  j.set("context", context);
  j.set("page_tokens", page_tokens);
  return j;
}

namespace {
void require_canonical(const Plan& plan, const char* what) {
  Plan again = compile(plan.spec, plan.checkpoint);
  if (again.to_json().dump() != plan.to_json().dump()) invalid(std::string(what) + " takes the canonical plan of its spec and checkpoint, not an edited one");
}
}  // namespace

Program lower_batch(const Plan& plan, uint32_t context, uint32_t batch) {
  if (batch == 0 || batch > 64) invalid("the lane count of a lowered program is 1..64");
  require_canonical(plan, "lowering");
  const auto& buckets = plan.spec.context_buckets;
  if (std::find(buckets.begin(), buckets.end(), context) == buckets.end()) invalid("the context of a lowered program must be one of the declared buckets");
  Program p;
  p.source_key = plan.key;
  p.batch = batch;
  p.context = context;
  p.page_tokens = plan.spec.page_tokens;
  p.embedding = std::string(kPrefix) + "embed_tokens.weight";
  p.final_norm = {std::string(kPrefix) + "norm.weight", Transform::OnePlusFp32};
  const auto& layers = plan.spec.model.layers;
  for (size_t i = 0; i < layers.size(); ++i) {
    Block b;
    b.layer = (uint32_t)i;
    b.kind = layers[i];
    auto bind = [&](const char* name, Transform t) { b.bindings.push_back({std::string(kPrefix) + "layers." + std::to_string(i) + "." + name, t}); };
    bind("input_layernorm.weight", Transform::OnePlusFp32);
    bind("post_attention_layernorm.weight", Transform::OnePlusFp32);
    for (auto n : {"mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"}) bind(n, Transform::Identity);
    if (layers[i] == Layer::Delta) {
      for (auto n : {"linear_attn.in_proj_qkv.weight", "linear_attn.in_proj_z.weight", "linear_attn.in_proj_a.weight", "linear_attn.in_proj_b.weight",
                     "linear_attn.conv1d.weight", "linear_attn.A_log", "linear_attn.dt_bias", "linear_attn.norm.weight", "linear_attn.out_proj.weight"})
        bind(n, Transform::Identity);
    } else {
      for (auto n : {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight"}) bind(n, Transform::Identity);
      bind("self_attn.q_norm.weight", Transform::OnePlusFp32);
      bind("self_attn.k_norm.weight", Transform::OnePlusFp32);
    }
    p.blocks.push_back(std::move(b));
  }
  p.key = Sha256::of(p.to_json().dump());
  return p;
}

Plan specialize_context(const Plan& plan, uint32_t context) {
  if (context == 0 || context > kMaxModelLen) invalid("context exceeds the checkpoint's position limit");
  require_canonical(plan, "context specialisation");
  rankplan::Spec spec = plan.spec;
  spec.context_buckets = {context};
  return compile(spec, plan.checkpoint);
}

}  // namespace ifab::hybrid
