#include "definition.h"

#include <algorithm>

namespace ifab::definition {

const char* kind_name(Kind k) {
  switch (k) {
    case Kind::Qwen: return "qwen";
    case Kind::OpenPangu: return "open_pangu";
    case Kind::Graph: return "graph";
    case Kind::Execution: return "execution";
  }
  return "?";
}

namespace {

// The `key = value;` members of a contract block, each consumed exactly once.
class FieldSet {
 public:
  FieldSet(const std::vector<lang::Member>& members, const char* where) : where_(where) {
    for (auto& m : members) {
      if (m.kind != lang::Member::Kind::Field)
        invalid("byte " + std::to_string(m.start) + ": a contract " + where_ + " block holds `key = value;` fields only");
      if (!fields_.emplace(m.name, m.expr).second) invalid("byte " + std::to_string(m.start) + ": field " + m.name + " is given twice");
    }
  }
  lang::ExprPtr take(const std::string& key) {
    auto it = fields_.find(key);
    if (it == fields_.end()) invalid(where_ + ": field " + key + " is missing");
    lang::ExprPtr e = it->second;
    fields_.erase(it);
    return e;
  }
  std::string word(const std::string& key) {
    lang::ExprPtr e = take(key);
    if (e->kind != lang::Expr::Kind::Name && e->kind != lang::Expr::Kind::String) invalid(where_ + ": " + key + " takes a name or a string");
    return e->text;
  }
  uint32_t number(const std::string& key) { return to_u32(*take(key), key); }
  std::vector<uint32_t> numbers(const std::string& key) {
    lang::ExprPtr e = take(key);
    if (e->kind != lang::Expr::Kind::List) invalid(where_ + ": " + key + " takes a list of integers");
    std::vector<uint32_t> out;
    for (auto& a : e->args) out.push_back(to_u32(*a.second, key));
    return out;
  }
  rankplan::Mesh mesh(const std::string& key) {
    lang::ExprPtr e = take(key);
    if (e->kind != lang::Expr::Kind::Call || e->text != "mesh") invalid(where_ + ": " + key + " takes mesh(tp = .., cp = .., sp = ..)");
    rankplan::Mesh m;
    bool tp = false, cp = false, sp = false;
    for (auto& a : e->args) {
      if (a.first == "tp" && !tp) { m.tp = to_u32(*a.second, "tp"); tp = true; }
      else if (a.first == "cp" && !cp) { m.cp = to_u32(*a.second, "cp"); cp = true; }
      else if (a.first == "sp" && !sp) {
        if (a.second->kind != lang::Expr::Kind::Name || (a.second->text != "true" && a.second->text != "false")) invalid("mesh: sp is true or false");
        m.sp = a.second->text == "true";
        sp = true;
      } else {
        invalid("mesh: unexpected or repeated argument" + (a.first.empty() ? std::string(" (arguments are named)") : " " + a.first));
      }
    }
    if (!tp || !cp || !sp) invalid("mesh needs tp, cp and sp");
    return m;
  }
  void done() const {
    if (fields_.empty()) return;
    std::string names;
    for (auto& kv : fields_) names += (names.empty() ? "" : ", ") + kv.first;
    invalid(where_ + ": fields this contract does not know: " + names);
  }

 private:
  uint32_t to_u32(const lang::Expr& e, const std::string& key) const {
    if (e.kind != lang::Expr::Kind::Number) invalid(where_ + ": " + key + " takes an integer");
    char* end = nullptr;
    const unsigned long long v = strtoull(e.text.c_str(), &end, 10);
    if (!end || *end || e.text.empty() || e.text[0] == '-' || v > 0xffffffffull) invalid(where_ + ": " + key + " is not an unsigned 32-bit integer");
    return (uint32_t)v;
  }
  std::string where_;
  std::map<std::string, lang::ExprPtr> fields_;
};

const lang::Member* field_named(const std::vector<lang::Member>& members, const char* key) {
  for (auto& m : members)
    if (m.kind == lang::Member::Kind::Field && m.name == key) return &m;
  return nullptr;
}

graph::Parallel parallel_from(FieldSet& plan, const char* target) {
  graph::Parallel p;
  p.target = target;
  p.tp = plan.number("tp");
  p.ep = plan.number("ep");
  p.devices = plan.numbers("devices");
  p.max_num_seqs = plan.number("max_num_seqs");
  p.max_num_batched_tokens = plan.number("max_num_batched_tokens");
  p.max_model_len = plan.number("max_model_len");
  return p;
}

graph::Parallel parallel_from_json(const Json& j) {
  static const char* known[] = {"target", "tp", "ep", "devices", "max_num_seqs", "max_num_batched_tokens", "max_model_len"};
  for (auto& kv : j.as_object())
    if (std::none_of(std::begin(known), std::end(known), [&](const char* k) { return kv.first == k; })) invalid("parallel: unknown field " + kv.first);
  graph::Parallel p;
  if (auto t = j.find("target")) p.target = t->as_string();
  p.tp = (uint32_t)j.at("tp").as_int();
  p.ep = (uint32_t)j.at("ep").as_int();
  p.devices.clear();
  for (auto& d : j.at("devices").as_array()) p.devices.push_back((uint32_t)d.as_int());
  p.max_num_seqs = (uint32_t)j.at("max_num_seqs").as_int();
  p.max_num_batched_tokens = (uint32_t)j.at("max_num_batched_tokens").as_int();
  p.max_model_len = (uint32_t)j.at("max_model_len").as_int();
  return p;
}

}  // namespace

void ModelDefinition::validate() const {
  switch (kind) {
    case Kind::Qwen: spec.validate(); break;
    case Kind::OpenPangu: parallel.validate(); break;
    case Kind::Execution:
      parallel.validate();
      execution.validate();
      if (parallel.max_model_len != execution.max_context) invalid("the plan's max_model_len and the graph's context disagree");
      break;
    case Kind::Graph: cpu::verify(cpu::compile(logical)); break;
  }
}

Json ModelDefinition::to_json() const {
  Json j = Json::object();
  j.set("kind", kind_name(kind));
  switch (kind) {
    case Kind::Qwen:
      j.set("checkpoint", checkpoint);
      j.set("spec", spec.to_json());
      break;
    case Kind::OpenPangu: j.set("parallel", parallel.to_json()); break;
    case Kind::Graph: j.set("graph", logical.to_json()); break;
    case Kind::Execution:
      j.set("parallel", parallel.to_json());
      j.set("graph", execution.to_json());
      break;
  }
  return j;
}

ModelDefinition ModelDefinition::from_json(const Json& j) {
  ModelDefinition d;
  const std::string& k = j.at("kind").as_string();
  auto only = [&](std::initializer_list<const char*> allowed) {
    for (auto& kv : j.as_object())
      if (kv.first != "kind" && std::none_of(allowed.begin(), allowed.end(), [&](const char* a) { return kv.first == a; }))
        invalid("definition of kind " + k + ": unknown field " + kv.first);
  };
  if (k == "qwen") {
    only({"checkpoint", "spec"});
    d.kind = Kind::Qwen;
    d.checkpoint = j.at("checkpoint").as_bool();
    d.spec = rankplan::Spec::from_json(j.at("spec"));
  } else if (k == "open_pangu") {
    only({"parallel"});
    d.kind = Kind::OpenPangu;
    d.parallel = parallel_from_json(j.at("parallel"));
  } else if (k == "graph") {
    only({"graph"});
    d.kind = Kind::Graph;
    d.logical = cpu::LogicalGraph::from_json(j.at("graph"));
  } else if (k == "execution") {
    only({"parallel", "graph"});
    d.kind = Kind::Execution;
    d.parallel = parallel_from_json(j.at("parallel"));
    d.execution = graph::Graph::from_json(j.at("graph"));
  } else {
    invalid("unknown definition kind " + k);
  }
  return d;
}

ModelDefinition elaborate(const lang::Document& doc) {
  ModelDefinition d;
  const lang::Member* target = field_named(doc.plan, "target");
  const std::string tname = target && target->expr && target->expr->kind == lang::Expr::Kind::Name ? target->expr->text : "";
  if (tname == "b200_token_v1" || tname == "ascend_token_v1") {
    d.kind = Kind::Execution;
    d.execution = graph::elaborate(lang::expand(doc));
    d.parallel = d.execution.parallel;
    d.validate();
    return d;
  }
  if (!doc.modules.empty()) invalid("modules need a token target (b200_token_v1)");
  const lang::Member* contract = field_named(doc.model, "contract");
  if (contract) {
    FieldSet model(doc.model, "model"), plan(doc.plan, "plan");
    const std::string c = model.word("contract");
    if (c == "openpangu_v2_tp_ep_v1") {
      model.done();
      d.kind = Kind::OpenPangu;
      d.parallel = parallel_from(plan, "b200_token_v1");
      plan.done();
    } else if (c == "qwen_structure_v1" || c == "qwen35_text_v1") {
      d.kind = Kind::Qwen;
      d.checkpoint = c == "qwen35_text_v1";
      rankplan::Model& m = d.spec.model;
      m.name = model.word("label");
      m.hidden = model.number("hidden");
      m.intermediate = model.number("intermediate");
      m.vocab = model.number("vocab");
      m.query_heads = model.number("query_heads");
      m.kv_heads = model.number("kv_heads");
      m.head_dim = model.number("head_dim");
      m.delta_heads = model.number("delta_heads");
      m.delta_dim = model.number("delta_dim");
      m.conv_width = model.number("conv_width");
      lang::ExprPtr layers = model.take("layers");
      if (layers->kind != lang::Expr::Kind::List) invalid("model: layers takes a list of `full` / `delta`");
      for (auto& a : layers->args) {
        const lang::Expr& e = *a.second;
        if (e.kind == lang::Expr::Kind::Name && e.text == "full") m.layers.push_back(rankplan::Layer::Full);
        else if (e.kind == lang::Expr::Kind::Name && e.text == "delta") m.layers.push_back(rankplan::Layer::Delta);
        else invalid("model: a layer is `full` or `delta`");
      }
      d.spec.prefill = plan.mesh("prefill");
      d.spec.decode = plan.mesh("decode");
      d.spec.page_tokens = plan.number("page_tokens");
      d.spec.token_budget = plan.number("token_budget");
      d.spec.batch_buckets = plan.numbers("batch_buckets");
      d.spec.context_buckets = plan.numbers("context_buckets");
      model.done();
      plan.done();
    } else {
      invalid("model contract " + c + " is not one this compiler knows");
    }
    d.validate();
    return d;
  }
  if (tname != "cpu_f32_v1") invalid(tname.empty() ? "the plan names no target and the model no contract" : "plan target " + tname + " is not implemented");
  d.kind = Kind::Graph;
  d.logical = cpu::from_expanded(lang::expand(doc));
  d.validate();
  return d;
}

ModelDefinition definition(std::string_view source) {
  size_t i = 0;
  while (i < source.size() && isspace((unsigned char)source[i])) ++i;
  if (i < source.size() && source[i] == '{') return decode(source);
  return elaborate(lang::parse(source));
}

std::string encode(const ModelDefinition& d) {
  d.validate();
  Json a = Json::object();
  a.set("format", "inferfabric.model");
  a.set("version", 1);
  a.set("definition", d.to_json());
  return a.dump(1);
}

ModelDefinition decode(std::string_view bytes) {
  if (bytes.size() > kMaxArtifactBytes) fail(ErrorKind::Capacity, "model artifact exceeds 16 MiB");
  const Json a = Json::parse(bytes, kMaxArtifactBytes);
  for (auto& kv : a.as_object())
    if (kv.first != "format" && kv.first != "version" && kv.first != "definition") invalid("model artifact: unknown field " + kv.first);
  if (a.at("format").as_string() != "inferfabric.model" || a.at("version").as_int() != 1) invalid("not an inferfabric.model artifact of version 1");
  ModelDefinition d = ModelDefinition::from_json(a.at("definition"));
  d.validate();
  return d;
}

rankplan::Spec parse_spec(std::string_view source) {
  ModelDefinition d = definition(source);
  if (d.kind != Kind::Qwen) invalid("the document does not define a hybrid-decoder (qwen) model");
  return d.spec;
}

rankplan::Spec parse_checkpoint_spec(std::string_view source) {
  ModelDefinition d = definition(source);
  if (d.kind != Kind::Qwen || !d.checkpoint) invalid("a checkpoint compile needs the qwen35_text_v1 contract");
  return d.spec;
}

}  // namespace ifab::definition
