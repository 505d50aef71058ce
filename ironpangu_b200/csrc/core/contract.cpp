#include "contract.h"

#include <filesystem>
#include <set>

namespace ifab::contract {
namespace {

using program::Instruction;
using program::Program;
constexpr uint32_t kTensor = 0, kRoutes = 2, kExperts = 3, kCache = 4, kView = program::kKindView;
constexpr uint32_t kAny = 0xffffffffu;

struct OpRule {
  std::vector<std::string> kernels;        // any of these entry points (a '|'-joined pair in the file must be a subset)
  std::vector<uint32_t> inputs;            // kinds of the inputs (kAny: not checked); empty + variadic = any count
  bool variadic = false;
  std::vector<std::string> attrs;          // attributes the kernel reads
  uint32_t kind = kAny;                    // kind of the result
};

// entry points per fused operation of the device program; operations that are not listed are checked against the
// lowering's own recipe table only (name -> kernel)
const std::map<std::string, OpRule>& rules() {
  static const std::map<std::string, OpRule> r = {
      {"embedding", {{"ifab_embedding_bf16"}, {}, false, {"vocab", "weight", "width"}, kTensor}},
      {"linear", {{"ifab_gemv_bf16", "ifab_gemm_bf16"}, {kTensor}, false, {"weight", "width"}, kTensor}},
      {"view", {{"view"}, {kAny}, false, {"start", "width"}, kView}},
      // a third input holds the attention-sink rows that every query of the cache also attends to
      {"mla_kv_write", {{"ifab_mla_kv_write", "ifab_mla_kv_write_q8"}, {kAny, kAny}, true, {"eps", "theta", "weight"}, kCache}},
      {"mla_q_absorb", {{"ifab_mla_q_absorb"}, {kTensor}, false, {"heads", "latent", "nope", "rope", "theta", "weight"}, kTensor}},
      // a third input is the sparse indexer's selection (selection = learned_indices)
      {"mla_attention", {{"ifab_mla_decode_attention", "ifab_mla_prefill_attention"}, {kTensor, kCache}, true, {"heads", "latent", "weight"}, kTensor}},
      {"linear_allreduce", {{"ifab_gemv_allreduce_bf16", "ifab_gemm_reduce_scatter_bf16", "ifab_gemm_allreduce_bf16"}, {kTensor}, true, {"weight", "width"}, kTensor}},
      {"router_topk", {{"ifab_router_topk"}, {kTensor}, false, {"experts", "topk", "weight"}, kRoutes}},
      {"moe_gate_up", {{"ifab_moe_gate_up_decode", "ifab_grouped_gemm_bf16", "ifab_moe_gate_up_decode_fp8"}, {kTensor, kRoutes}, false, {"weight", "width"}, kExperts}},
      {"moe_down_allreduce", {{"ifab_moe_down_allreduce_decode", "ifab_moe_combine", "ifab_moe_down_allreduce_decode_fp8"}, {kExperts, kRoutes}, true, {"weight", "width"}, kTensor}},
      {"lm_head", {{"ifab_lm_head_argmax"}, {kTensor}, false, {"weight", "width"}, kTensor}},
  };
  return r;
}

[[noreturn]] void bad(const Instruction& i, const std::string& why) {
  invalid("invalid kernel contract: " + i.name + " (" + i.op + "): " + why);
}

std::vector<std::string> split_alternatives(const std::string& s) {
  std::vector<std::string> out;
  size_t b = 0;
  while (b <= s.size()) {
    size_t e = s.find('|', b);
    if (e == std::string::npos) e = s.size();
    out.push_back(s.substr(b, e - b));
    b = e + 1;
  }
  return out;
}

uint64_t number(const Instruction& i, const char* key, uint64_t lo, uint64_t hi) {
  const std::string* v = i.attr(key);
  if (!v) bad(i, std::string("missing attribute ") + key);
  uint64_t n = 0;
  if (v->empty() || v->size() > 12) bad(i, std::string("attribute ") + key + " is not a number");
  for (char c : *v) {
    if (c < '0' || c > '9') bad(i, std::string("attribute ") + key + " is not a number");
    n = n * 10 + (uint64_t)(c - '0');
  }
  if (n < lo || n > hi) bad(i, std::string("attribute ") + key + " out of range");
  return n;
}

// root buffer and element range an instruction's result occupies (views resolve to their origin)
struct Region { uint32_t root; uint64_t start, width; };
Region region_of(const Program& p, uint32_t id) {
  uint64_t start = 0;
  const uint64_t width = p.instructions[id].width;
  for (size_t depth = 0; depth <= p.instructions.size(); ++depth) {
    const Instruction& n = p.instructions[id];
    if (n.op != "view") return Region{id, start, width};
    const std::string* s = n.attr("start");
    start += s ? std::stoull(*s) : 0;
    id = n.inputs.at(0);
  }
  invalid("invalid kernel contract: view chain does not terminate");
}

}  // namespace

void validate_kernels(const Program& p) {
  p.validate();
  const auto& recipe = program::recipes();
  for (uint32_t idx = 0; idx < p.instructions.size(); ++idx) {
    const Instruction& i = p.instructions[idx];
    if (i.kernel == "unsupported") bad(i, "no kernel implements this operation");
    const auto alts = split_alternatives(i.kernel);
    auto rit = rules().find(i.op);
    if (rit == rules().end()) {
      // not a fused device operation: the entry point must be the one the recipe table registers for the name
      auto it = recipe.find(i.op);
      if (it == recipe.end()) bad(i, "unknown operation");
      if (i.kernel != it->second && i.kernel != "view" && i.kernel != "none") bad(i, "kernel " + i.kernel + " is not registered for the operation");
      continue;
    }
    const OpRule& r = rit->second;
    for (const auto& k : alts)
      if (std::find(r.kernels.begin(), r.kernels.end(), k) == r.kernels.end()) bad(i, "kernel " + k + " is not registered for the operation");
    if (r.variadic ? i.inputs.size() < r.inputs.size() : i.inputs.size() != r.inputs.size()) bad(i, "wrong number of inputs");
    for (size_t k = 0; k < r.inputs.size(); ++k) {
      if (r.inputs[k] == kAny) continue;
      // a view of a tensor is a tensor
      uint32_t src = i.inputs[k];
      uint32_t kind = p.instructions[src].kind;
      if (kind == kView) kind = p.instructions[region_of(p, src).root].kind;
      if (kind != r.inputs[k]) bad(i, "input " + std::to_string(k) + " has the wrong kind");
    }
    if (i.op == "mla_kv_write" && (i.inputs.size() > 3 || (i.inputs.size() == 3 && p.instructions[i.inputs[2]].op != "sink_normalize")))
      bad(i, "the third input must be the sink rows of a sink_normalize");
    if (r.kind != kAny && i.kind != r.kind) bad(i, "result has the wrong kind");
    for (const auto& a : r.attrs)
      if (!i.attr(a)) bad(i, "missing attribute " + a);
    if (i.op == "view") {
      const uint64_t start = number(i, "start", 0, 1u << 24), width = number(i, "width", 1, 1u << 24);
      const Instruction& src = p.instructions[i.inputs[0]];
      if (width != i.width) bad(i, "width attribute differs from the result width");
      if (src.width && start + width > src.width) bad(i, "view leaves its input");
      continue;
    }
    if (i.attr("width")) {
      const uint64_t w = number(i, "width", 1, 1u << 24);
      if (i.op != "lm_head" && i.op != "embedding" && w % 8 != 0) bad(i, "width is not a multiple of 8 elements");
    }
    if (i.op == "mla_attention") {
      const std::string* sel = i.attr("selection");
      const bool learned = sel && *sel == "learned_indices";
      if (i.inputs.size() != (learned ? 3u : 2u)) bad(i, "attention takes (query, cache) or, with learned_indices, (query, cache, selection)");
      if (learned && p.instructions[i.inputs[2]].op != "sparse_index") bad(i, "the selection must come from a sparse_index instruction");
    }
    if (i.op == "router_topk") {
      const uint64_t e = number(i, "experts", 1, 4096), k = number(i, "topk", 1, 16);
      if (k > e) bad(i, "topk exceeds the expert count");
    }
    if (i.op == "mla_q_absorb" || i.op == "mla_attention") {
      if (number(i, "latent", 8, 1024) != 512) bad(i, "the latent cache kernels are built for 512 latent columns");
      number(i, "heads", 1, 1024);
    }
    if (i.op == "linear_allreduce" || i.op == "moe_down_allreduce") {
      // the fused all-reduce writes its result into the residual stream it also reads: no other live value may share
      // the buffer of its first input (the kernel stages that operand while peers still write the output)
      const Region a = region_of(p, i.inputs[0]);
      for (uint32_t j = idx + 1; j < p.instructions.size(); ++j) {
        if (p.instructions[j].op == "view") continue;
        for (uint32_t in : p.instructions[j].inputs) {
          const Region b = region_of(p, in);
          if (b.root == a.root && b.start < a.start + a.width && a.start < b.start + b.width && in != i.inputs[0] && p.instructions[in].op != "view")
            bad(i, "operand of a fused all-reduce is aliased by a later reader");
        }
      }
    }
  }
}

void validate_bindings(const Program& p, const init::Plan& plan) {
  std::map<std::string, const init::Parameter*> params;
  for (const auto& q : plan.parameters) {
    if (!params.emplace(q.name, &q).second) invalid("invalid binding contract: parameter " + q.name + " appears twice");
    if (q.dims.empty() || q.bytes() == 0) invalid("invalid binding contract: parameter " + q.name + " is empty");
  }
  std::set<std::string> used;
  for (const Instruction& i : p.instructions) {
    // a projection fused with its pair is one parameter named "weight|paired_weight"
    auto joined = [&](const char* key, const char* pair_key) -> std::string {
      const std::string* name = i.attr(key);
      if (!name || name->empty()) return "";
      const std::string* pair = i.attr(pair_key);
      return (pair && !pair->empty()) ? *name + "|" + *pair : *name;
    };
    std::string names[3] = {joined("weight", "paired_weight"), joined("shared_weight", "shared_paired_weight"),
                            i.attr("norm_weight") ? *i.attr("norm_weight") : std::string()};
    // operators whose `weight` names a scope: their parameters are the tensors under it
    std::vector<std::string> scoped;
    if (i.op == "mhc_pre" || i.op == "mhc_merge") {
      for (const char* part : {".phi", ".gamma", ".alpha", ".beta"}) scoped.push_back(names[0] + part);
      names[0].clear();
    } else if (i.op == "sink_normalize") {
      scoped = {names[0] + ".param_sink_compressed_kv", names[0] + ".param_sink_k_pe", i.attr("norm") ? *i.attr("norm") : std::string()};
      names[0].clear();
    }
    for (const auto& nm : scoped) {
      if (nm.empty() || !params.count(nm)) invalid("invalid binding contract: " + i.name + " reads " + nm + ", which rank " + std::to_string(plan.rank) + " does not load");
      used.insert(nm);
    }
    for (int k = 0; k < 3; ++k) {
      if (names[k].empty()) continue;
      if (!params.count(names[k])) {
        // optional norms may be absent from a checkpoint; everything else must be bound
        if ((k == 2 && i.attr("norm_optional")) || (k == 0 && i.op == "optional_norm")) continue;
        invalid("invalid binding contract: " + i.name + " reads " + names[k] + ", which rank " + std::to_string(plan.rank) + " does not load");
      }
      used.insert(names[k]);
    }
    // the leading dimension of a linear weight is the instruction's own output width plus the paired projection's
    if ((i.op == "linear" || i.op == "lm_head") && !names[0].empty() && i.attr("width")) {
      const init::Parameter& q = *params[names[0]];
      uint64_t rows = std::stoull(*i.attr("width"));
      const std::string* pw = i.attr("paired_width");
      const std::string* pn = i.attr("paired_weight");
      if (pw && !pw->empty() && pn && !pn->empty()) rows += std::stoull(*pw);
      if (q.dims[0] != rows)
        invalid("invalid binding contract: " + names[0] + " has " + std::to_string(q.dims[0]) + " rows, " + i.name + " needs " + std::to_string(rows));
    }
  }
  for (const auto& q : plan.parameters)
    if (!used.count(q.name)) invalid("invalid binding contract: parameter " + q.name + " is loaded but never read");
  // load slices must target parameters of the plan and stay inside them
  std::vector<uint64_t> filled(plan.parameters.size(), 0);
  for (const auto& l : plan.loads) {
    if (l.dest >= plan.parameters.size()) invalid("invalid binding contract: load slice targets parameter " + std::to_string(l.dest));
    const uint64_t grow = l.bytes / init::dtype_bytes(l.src_dtype) * init::dtype_bytes(plan.parameters[l.dest].dtype);
    filled[l.dest] += grow;
  }
  for (size_t k = 0; k < filled.size(); ++k)
    if (filled[k] != plan.parameters[k].bytes())
      invalid("invalid binding contract: parameter " + plan.parameters[k].name + " receives " + std::to_string(filled[k]) + " of " +
              std::to_string(plan.parameters[k].bytes()) + " bytes");
}

Json validate_bundle(const std::string& dir) {
  namespace fs = std::filesystem;
  Program p = Program::decode(read_file(dir + "/execution.bin"));
  validate_kernels(p);
  Json j = Json::object();
  j.set("program", p.name);
  j.set("instructions", (int64_t)p.instructions.size());
  int64_t ranks = 0;
  for (uint32_t r = 0;; ++r) {
    const std::string path = dir + "/rank-" + std::to_string(r) + ".bin";
    if (!fs::exists(path)) break;
    validate_bindings(p, init::Plan::decode(read_file(path)));
    ++ranks;
  }
  if (ranks == 0) invalid("bundle has no rank-N.bin initialization plan");
  j.set("ranks", ranks);
  j.set("valid", true);
  return j;
}

}  // namespace ifab::contract
