#include "program.h"

#include <algorithm>
#include <functional>
#include <set>

namespace ifab::program {

using graph::Graph;
using graph::Kind;
using graph::Node;

const std::string* Instruction::attr(std::string_view key) const {
  for (auto& kv : attrs)
    if (kv.first == key) return &kv.second;
  return nullptr;
}

const std::map<std::string, std::string>& recipes() {
  static const std::map<std::string, std::string> r = {
      {"embedding", "ifab_embedding_bf16"},
      {"norm", "ifab_rmsnorm_bf16"},
      {"linear", "ifab_gemv_bf16|ifab_gemm_bf16"},
      {"linear_allreduce", "ifab_gemv_allreduce_bf16|ifab_gemm_reduce_scatter_bf16"},
      {"view", "view"},
      {"mla_kv_write", "ifab_mla_kv_write"},
      {"mla_q_absorb", "ifab_mla_q_absorb"},
      {"mla_attention", "ifab_mla_decode_attention|ifab_mla_prefill_attention"},
      {"router_topk", "ifab_router_topk"},
      {"moe_gate_up", "ifab_moe_gate_up_decode|ifab_grouped_gemm_bf16"},
      {"moe_down_allreduce", "ifab_moe_down_allreduce_decode|ifab_moe_combine"},
      {"lm_head", "ifab_lm_head_argmax"},
      {"rotary_prefix", "ifab_gqa_rope_kv_write"},
      {"kv_cache_append", "ifab_gqa_rope_kv_write"},
      {"paged_attention", "ifab_gqa_decode_attention"},
      {"allreduce", "ifab_allreduce_f32"},
      {"gather", "ifab_allgather_bf16"},
      {"add", "ifab_add_bf16"},
      {"swiglu", "ifab_swiglu_bf16"},
      {"cast", "ifab_cast"},
      {"concat", "ifab_concat_bf16"},
      {"repeat", "ifab_repeat_bf16"},
      {"rope", "ifab_rope_bf16"},
      {"mome", "ifab_causal_conv"},
      {"mhc_pre", "ifab_mhc_pre"},
      {"mhc_merge", "ifab_mhc_pre"},
      {"mhc_input", "view"},
      {"mhc_post", "ifab_mhc_post"},
      {"quantize", "ifab_quantize_rows"},
      {"sink_normalize", "ifab_rmsnorm_bf16"},
      {"cache_append", "ifab_cache_append"},
      {"index_cache_append", "ifab_index_cache_append"},
      {"sparse_index", "ifab_sparse_index_topk"},
      {"latent_attention", "ifab_mla_decode_attention"},
      {"mla_value", "ifab_gemv_bf16"},
      {"mla_query", "ifab_mla_q_absorb"},
      {"router", "ifab_router_topk"},
      {"expert_linear", "ifab_grouped_gemm_bf16"},
      {"expert_swiglu_down", "ifab_grouped_gemm_bf16"},
      {"expert_reduce", "ifab_moe_combine"},
      {"optional_norm", "ifab_rmsnorm_bf16"},
      {"cache_norm_rope_append", "ifab_mla_kv_write"},
  };
  return r;
}

namespace {

struct Lowering {
  const Graph& g;
  const Options& opt;
  Program p;
  std::vector<std::vector<uint32_t>> users;
  std::vector<int64_t> val;          // logical node -> instruction id (-1: folded away)
  std::vector<char> skip;            // member of a fused group, emitted at the group's anchor
  std::map<uint32_t, std::function<void()>> anchors;  // logical node -> group emitter
  std::vector<int64_t> folded_norm;  // logical norm node folded into its consumers -> 1
  std::map<std::pair<uint32_t, std::string>, uint32_t> cast_cse;

  Lowering(const Graph& graph, const Options& o) : g(graph), opt(o) {
    users.resize(g.nodes.size());
    for (uint32_t i = 0; i < g.nodes.size(); ++i)
      for (uint32_t in : g.nodes[i].inputs) users[in].push_back(i);
    val.assign(g.nodes.size(), -1);
    skip.assign(g.nodes.size(), 0);
    folded_norm.assign(g.nodes.size(), 0);
  }

  bool sole_user(uint32_t n, uint32_t u) const { return users[n].size() == 1 && users[n][0] == u; }
  const Node& N(uint32_t i) const { return g.nodes[i]; }

  uint32_t emit(Instruction ins) {
    auto it = recipes().find(ins.op);
    if (ins.kernel.empty()) ins.kernel = it == recipes().end() ? "unsupported" : it->second;
    std::sort(ins.attrs.begin(), ins.attrs.end());
    p.instructions.push_back(std::move(ins));
    return (uint32_t)p.instructions.size() - 1;
  }
  uint32_t value_of(uint32_t logical) {
    if (val[logical] < 0) invalid("lowering: value of " + N(logical).name + " was folded away but is still needed");
    return (uint32_t)val[logical];
  }
  // ensure `ins` has dtype `want`, inserting (and re-using) an explicit cast
  uint32_t with_dtype(uint32_t ins, const std::string& want, uint32_t logical) {
    if (p.instructions[ins].dtype == want) return ins;
    auto key = std::make_pair(ins, want);
    auto it = cast_cse.find(key);
    if (it != cast_cse.end()) return it->second;
    Instruction c;
    c.kind = p.instructions[ins].kind;
    c.width = p.instructions[ins].width;
    c.name = p.instructions[ins].name + ".as_" + want;
    c.op = "cast";
    c.inputs = {ins};
    c.attrs = {{"dtype", want}};
    c.dtype = want;
    c.logical_node = logical;
    uint32_t id = emit(std::move(c));
    cast_cse[key] = id;
    return id;
  }

  // activation source of a consumer: resolves a folded norm into (source value, norm attrs)
  struct Src {
    uint32_t value;
    std::vector<std::pair<std::string, std::string>> norm;
  };
  Src source(uint32_t logical_in) {
    if (folded_norm[logical_in]) {
      const Node& nn = N(logical_in);
      Src s{with_dtype(value_of(nn.inputs[0]), "bf16", logical_in), {}};
      s.norm.emplace_back("norm_weight", nn.need("weight"));
      s.norm.emplace_back("norm_eps", nn.need("eps"));
      if (nn.has("zero_centered")) s.norm.emplace_back("norm_zero_centered", *nn.attr("zero_centered"));
      if (nn.op == "optional_norm") s.norm.emplace_back("norm_optional", "true");
      return s;
    }
    return Src{with_dtype(value_of(logical_in), "bf16", logical_in), {}};
  }

  bool norm_foldable(uint32_t i) const {
    if (users[i].empty()) return false;
    for (uint32_t u : users[i]) {
      const Node& c = N(u);
      // the branch that returns into a hyper-connection: its norm runs inside the mixing kernel
      if (c.op == "mhc_post" && c.inputs.size() == 2 && c.inputs[1] == i && c.inputs[0] != i && N(i).op == "norm" && !N(i).has("zero_centered")) continue;
      if (c.inputs[0] != i) return false;
      if (c.op != "linear" && c.op != "router" && c.op != "expert_linear") return false;
    }
    return true;
  }

  // -- group recognition -------------------------------------------------------------------------
  void recognise() {
    for (uint32_t a = 0; a < g.nodes.size(); ++a) {
      const Node& A = N(a);
      if (A.op == "allreduce") recognise_allreduce(a);
      if (A.op == "mla_value" && N(A.inputs[0]).op == "latent_attention" && sole_user(A.inputs[0], a)) {
        uint32_t att = A.inputs[0];
        skip[att] = 1;
        anchors[a] = [this, a, att] { emit_attention(att, a); };
      }
      if (A.op == "swiglu" && A.inputs.size() == 1 && !skip[a]) {
        uint32_t l = A.inputs[0];
        if (N(l).op == "linear" && N(l).has("paired_weight") && sole_user(l, a) && !skip[l]) {
          skip[l] = 1;
          anchors[a] = [this, a, l] { emit_swiglu_linear(l, a); };
        }
      }
      if (A.op == "gather" && a == g.output) {
        uint32_t l = A.inputs[0];
        if (N(l).op == "linear" && *N(l).attr("placement") == "tp_rows" && sole_user(l, a)) {
          skip[l] = 1;
          anchors[a] = [this, a, l] { emit_head(l, a); };
        }
      }
    }
    // a swiglu pair swallowed by an MoE group must not keep its own anchor
    for (auto it = anchors.begin(); it != anchors.end();)
      it = skip[it->first] ? anchors.erase(it) : std::next(it);
  }

  // residual add absorbed by a fused all-reduce: allreduce -> add(other, allreduce) with `other` computed earlier
  int64_t absorbable_residual(uint32_t a, uint32_t* add_node) const {
    if (users[a].size() != 1) return -1;
    uint32_t k = users[a][0];
    const Node& K = N(k);
    if (K.op != "add") return -1;
    uint32_t other = K.inputs[0] == a ? K.inputs[1] : K.inputs[0];
    if (other >= a) return -1;
    *add_node = k;
    return other;
  }

  void recognise_allreduce(uint32_t a) {
    const Node& A = N(a);
    uint32_t j = A.inputs[0];
    const Node& J = N(j);
    if (J.op == "linear" && *J.attr("placement") == "tp_columns" && sole_user(j, a)) {
      skip[j] = 1;
      uint32_t add_node = 0;
      int64_t res = absorbable_residual(a, &add_node);
      if (res >= 0) skip[a] = 1;
      uint32_t anchor = res >= 0 ? add_node : a;
      anchors[anchor] = [this, a, j, res, anchor] { emit_linear_allreduce(j, a, res, anchor); };
      return;
    }
    // MoE: allreduce(expert_reduce) or allreduce(add(expert_reduce, shared K-sharded linear))
    uint32_t red = j, addn = UINT32_MAX, l2 = UINT32_MAX;
    if (J.op == "add" && sole_user(j, a)) {
      for (int side = 0; side < 2; ++side) {
        uint32_t x = J.inputs[side], y = J.inputs[1 - side];
        if (N(x).op == "expert_reduce" && N(y).op == "linear" && *N(y).attr("placement") == "tp_columns" &&
            sole_user(x, j) && sole_user(y, j)) {
          red = x;
          l2 = y;
          addn = j;
        }
      }
      if (addn == UINT32_MAX) return;
    }
    if (N(red).op != "expert_reduce") return;
    if (addn == UINT32_MAX && !sole_user(red, a)) return;
    uint32_t d = N(red).inputs[0];
    if (N(d).op != "expert_swiglu_down" || N(d).inputs.size() != 2 || !sole_user(d, red)) return;
    uint32_t gu = N(d).inputs[0];
    if (N(gu).op != "expert_linear" || !N(gu).has("paired_weight") || !sole_user(gu, d)) return;
    uint32_t routes = N(gu).inputs[1];
    if (N(d).inputs[1] != routes || N(red).inputs[1] != routes) return;
    uint32_t sw = UINT32_MAX, l1 = UINT32_MAX;
    if (l2 != UINT32_MAX) {
      sw = N(l2).inputs[0];
      if (N(sw).op != "swiglu" || N(sw).inputs.size() != 1 || !sole_user(sw, l2)) return;
      l1 = N(sw).inputs[0];
      if (N(l1).op != "linear" || !N(l1).has("paired_weight") || *N(l1).attr("placement") != "tp_rows" || !sole_user(l1, sw)) return;
      if (N(l1).inputs[0] != N(gu).inputs[0]) return;  // shared expert must read the same activations
    }
    for (uint32_t m : {gu, d, red}) skip[m] = 1;
    if (l2 != UINT32_MAX)
      for (uint32_t m : {l1, sw, l2, addn}) skip[m] = 1;
    uint32_t add_node = 0;
    int64_t res = absorbable_residual(a, &add_node);
    if (res >= 0) skip[a] = 1;
    uint32_t anchor = res >= 0 ? add_node : a;
    anchors[anchor] = [this, a, gu, d, l1, l2, res, anchor, routes] { emit_moe(gu, d, l1, l2, a, routes, res, anchor); };
  }

  // -- group emitters -----------------------------------------------------------------------------
  void emit_linear_allreduce(uint32_t lin, uint32_t ar, int64_t residual, uint32_t anchor) {
    const Node& L = N(lin);
    Src s = source(L.inputs[0]);
    Instruction ins;
    ins.kind = (uint32_t)Kind::Tensor;
    ins.width = L.type.width;
    ins.name = N(anchor).name;
    ins.op = "linear_allreduce";
    ins.inputs = {s.value};
    ins.attrs = {{"weight", L.need("weight")}, {"width", L.need("width")}, {"placement", "tp_columns"}};
    if (opt.bulk_collectives) ins.attrs.emplace_back("bulk", "reduce_scatter_all_gather");
    for (auto& kv : s.norm) ins.attrs.push_back(kv);
    if (residual >= 0) {
      ins.inputs.push_back(with_dtype(value_of((uint32_t)residual), "bf16", anchor));
      ins.attrs.emplace_back("residual", "input1");
    }
    ins.dtype = "bf16";
    ins.logical_node = ar;
    uint32_t id = emit(std::move(ins));
    val[ar] = id;
    val[anchor] = id;
  }

  void emit_attention(uint32_t att, uint32_t mv) {
    const Node& A = N(att);
    const Node& V = N(mv);
    Instruction ins;
    ins.kind = (uint32_t)Kind::Tensor;
    ins.width = V.type.width;
    ins.name = V.name;
    ins.op = "mla_attention";
    ins.inputs = {with_dtype(value_of(A.inputs[0]), "bf16", att), value_of(A.inputs[1])};
    if (A.inputs.size() == 3) ins.inputs.push_back(value_of(A.inputs[2]));
    ins.attrs = {{"scale_dim", A.need("scale_dim")}, {"window", A.need("window")}, {"selection", A.need("selection")},
                 {"weight", V.need("weight")}, {"heads", V.need("heads")}, {"latent", V.need("latent")}, {"value", V.need("value")}};
    ins.dtype = "bf16";
    ins.logical_node = mv;
    val[mv] = emit(std::move(ins));
  }

  void emit_swiglu_linear(uint32_t lin, uint32_t sw) {
    const Node& L = N(lin);
    Src s = source(L.inputs[0]);
    Instruction ins;
    ins.kind = (uint32_t)Kind::Tensor;
    ins.width = N(sw).type.width;
    ins.name = N(sw).name;
    ins.op = "linear";
    ins.inputs = {s.value};
    ins.attrs = {{"weight", L.need("weight")}, {"paired_weight", L.need("paired_weight")}, {"width", L.need("width")},
                 {"placement", L.need("placement")}, {"activation", "swiglu"}};
    // the parameter holds both halves: gate rows, then the paired (up) rows
    ins.attrs.emplace_back("paired_width", L.has("paired_width") ? *L.attr("paired_width") : L.need("width"));
    for (auto& kv : s.norm) ins.attrs.push_back(kv);
    ins.dtype = "bf16";
    ins.logical_node = sw;
    val[sw] = emit(std::move(ins));
  }

  void emit_head(uint32_t lin, uint32_t gather) {
    const Node& L = N(lin);
    Src s = source(L.inputs[0]);
    Instruction ins;
    ins.kind = (uint32_t)Kind::Tensor;
    ins.width = N(gather).type.width;
    ins.name = N(gather).name;
    ins.op = "lm_head";
    ins.inputs = {s.value};
    ins.attrs = {{"weight", L.need("weight")}, {"width", L.need("width")}, {"placement", "tp_rows"}, {"sample", "greedy_sharded_argmax"}};
    for (auto& kv : s.norm) ins.attrs.push_back(kv);
    ins.dtype = "f32";
    ins.logical_node = gather;
    val[gather] = emit(std::move(ins));
  }

  void emit_moe(uint32_t gu, uint32_t d, uint32_t l1, uint32_t l2, uint32_t ar, uint32_t routes, int64_t residual, uint32_t anchor) {
    const Node& G = N(gu);
    const Node& D = N(d);
    Src s = source(G.inputs[0]);
    Instruction a;
    a.kind = (uint32_t)Kind::Experts;
    a.width = G.type.width / 2;
    a.name = G.name;
    a.op = "moe_gate_up";
    a.inputs = {s.value, value_of(routes)};
    a.attrs = {{"weight", G.need("weight")}, {"paired_weight", G.need("paired_weight")}, {"width", G.need("width")}, {"activation", "swiglu"}};
    for (auto& kv : s.norm) a.attrs.push_back(kv);
    if (G.has("weight_dtype")) a.attrs.emplace_back("weight_dtype", *G.attr("weight_dtype"));
    if (l1 != UINT32_MAX) {
      const Node& L1 = N(l1);
      a.attrs.emplace_back("shared_weight", L1.need("weight"));
      a.attrs.emplace_back("shared_paired_weight", L1.need("paired_weight"));
      a.attrs.emplace_back("shared_width", L1.need("width"));
    }
    a.dtype = "bf16";
    a.logical_node = gu;
    uint32_t act = emit(std::move(a));
    Instruction b;
    b.kind = (uint32_t)Kind::Tensor;
    b.width = D.type.width;
    b.name = N(anchor).name;
    b.op = "moe_down_allreduce";
    b.inputs = {act, value_of(routes)};
    b.attrs = {{"weight", D.need("weight")}, {"width", D.need("width")}};
    if (D.has("weight_dtype")) b.attrs.emplace_back("weight_dtype", *D.attr("weight_dtype"));
    if (l2 != UINT32_MAX) b.attrs.emplace_back("shared_weight", N(l2).need("weight"));
    if (opt.bulk_collectives) b.attrs.emplace_back("bulk", "dispatch_combine");
    if (residual >= 0) {
      b.inputs.push_back(with_dtype(value_of((uint32_t)residual), "bf16", anchor));
      b.attrs.emplace_back("residual", "input2");
    }
    b.dtype = "bf16";
    b.logical_node = ar;
    uint32_t id = emit(std::move(b));
    val[ar] = id;
    val[anchor] = id;
  }

  // -- main pass ------------------------------------------------------------------------------------
  std::string dtype_of(const Node& n, const std::vector<uint32_t>& ins) const {
    if (n.op == "cast") return n.need("dtype");
    if (n.op == "allreduce") return n.has("dtype") ? *n.attr("dtype") : "f32";
    if (n.op == "quantize") return n.need("dtype") == "int8" ? "int8" : "fp8";
    if (n.op == "router") return "f32";
    if (n.op == "sparse_index") return "i32";
    if (n.op == "expert_reduce") return "f32";
    if (n.op == "add") {
      for (uint32_t i : ins)
        if (p.instructions[i].dtype == "f32") return "f32";
      return "bf16";
    }
    return "bf16";
  }

  void run() {
    p.name = g.name;
    p.max_context = g.max_context;
    p.eos = g.eos;
    p.parallel = g.parallel;
    p.options = opt;
    recognise();
    for (uint32_t i = 0; i < g.nodes.size(); ++i) {
      auto an = anchors.find(i);
      if (an != anchors.end()) {
        an->second();
        continue;
      }
      if (skip[i]) continue;
      const Node& n = N(i);
      if ((n.op == "norm" || n.op == "optional_norm") && norm_foldable(i)) {
        folded_norm[i] = 1;
        continue;
      }
      Instruction ins;
      ins.kind = (uint32_t)n.type.kind;
      ins.width = n.type.width;
      ins.name = n.name;
      ins.op = n.op;
      ins.attrs = n.attrs;
      ins.logical_node = i;
      if (n.op == "slice") {
        ins.op = "view";
        ins.kind = kKindView;
        ins.inputs = {value_of(n.inputs[0])};
        ins.dtype = p.instructions[ins.inputs[0]].dtype;
      } else if (n.op == "linear" || n.op == "router" || n.op == "expert_linear") {
        Src s = source(n.inputs[0]);
        ins.inputs = {s.value};
        for (size_t k = 1; k < n.inputs.size(); ++k) ins.inputs.push_back(value_of(n.inputs[k]));
        for (auto& kv : s.norm) ins.attrs.push_back(kv);
        if (n.op == "router") ins.op = "router_topk";
        ins.dtype = dtype_of(n, ins.inputs);
      } else {
        if (n.op == "mhc_post" && folded_norm[n.inputs[1]]) {
          Src s = source(n.inputs[1]);
          ins.inputs = {value_of(n.inputs[0]), s.value};
          for (auto& kv : s.norm) ins.attrs.push_back(kv);
        } else {
          for (uint32_t in : n.inputs) ins.inputs.push_back(value_of(in));
        }
        // the streams a hyper-connection mixed are read again when its branch returns: name them, so that they stay alive
        if (n.op == "mhc_post") ins.inputs.push_back(value_of(N(n.inputs[0]).inputs[0]));
        if (n.op == "cache_norm_rope_append") ins.op = "mla_kv_write";
        if (n.op == "mla_query") ins.op = "mla_q_absorb";
        if (n.op == "add") {
          // f32 + bf16 mixes are made explicit: both operands are brought to the result dtype
          std::string dt = dtype_of(n, ins.inputs);
          for (auto& in : ins.inputs) in = with_dtype(in, dt, i);
          ins.dtype = dt;
        } else {
          ins.dtype = dtype_of(n, ins.inputs);
          if (n.op != "cast" && n.op != "allreduce" && n.op != "mhc_post" && n.op != "mhc_input")
            for (auto& in : ins.inputs)
              if (p.instructions[in].kind == (uint32_t)Kind::Tensor && p.instructions[in].dtype == "f32") in = with_dtype(in, "bf16", i);
        }
      }
      if (ins.kind == (uint32_t)Kind::Cache || ins.kind == (uint32_t)Kind::IndexCache) ins.dtype = n.has("cache_dtype") ? *n.attr("cache_dtype") : "bf16";
      val[i] = emit(std::move(ins));
    }
    p.output = value_of(g.output);
    if (opt.output_rows) {
      // instructions that only feed the output through row-wise ops may run on sampled rows only
      static const std::set<std::string> rowwise = {"norm", "linear", "lm_head", "gather", "cast", "view"};
      std::vector<std::vector<uint32_t>> iu(p.instructions.size());
      for (uint32_t k = 0; k < p.instructions.size(); ++k)
        for (uint32_t in : p.instructions[k].inputs) iu[in].push_back(k);
      uint32_t cur = p.output;
      while (rowwise.count(p.instructions[cur].op)) {
        p.output_suffix.push_back(cur);
        if (p.instructions[cur].inputs.empty()) break;
        uint32_t prev = p.instructions[cur].inputs[0];
        if (iu[prev].size() != 1) break;
        cur = prev;
      }
      std::reverse(p.output_suffix.begin(), p.output_suffix.end());
    }
    p.validate();
  }
};

}  // namespace

Program lower(const Graph& g, const Options& opt) {
  if (opt.resident_sequences == 0 || opt.resident_sequences > 1024) invalid("resident_sequences must be 1..1024");
  if (opt.prefill_tokens == 0 || opt.prefill_tokens > 65536) invalid("prefill_tokens must be 1..65536");
  for (size_t i = 0; i < opt.prefill_variants.size(); ++i) {
    if (opt.prefill_variants[i] < 2) invalid("prefill variants must be >= 2");
    if (i && opt.prefill_variants[i] <= opt.prefill_variants[i - 1]) invalid("prefill variants must be strictly ascending");
  }
  if (!opt.prefill_variants.empty() && opt.uncaptured_prefill) invalid("captured prefill variants and the uncaptured envelope are exclusive");
  Lowering l(g, opt);
  l.run();
  return std::move(l.p);
}

void Program::validate() const {
  if (instructions.empty()) invalid("program has no instructions");
  if (output >= instructions.size()) invalid("program output out of range");
  std::set<std::string> names;
  for (uint32_t i = 0; i < instructions.size(); ++i) {
    const Instruction& ins = instructions[i];
    if (ins.kind > kKindNone) invalid("instruction " + ins.name + ": bad kind");
    for (uint32_t in : ins.inputs)
      if (in >= i) invalid("instruction " + ins.name + " reads a later instruction");
    if (ins.op == "view" && ins.inputs.size() != 1) invalid("view takes one input");
    if (ins.kernel.empty()) invalid("instruction " + ins.name + " has no kernel");
    if (ins.op == "linear_allreduce" || ins.op == "moe_down_allreduce") {
      if (ins.dtype != "bf16") invalid(ins.name + ": fused all-reduce emits bf16");
    }
    if (ins.op == "cast" && (ins.inputs.size() != 1 || !ins.attr("dtype"))) invalid("malformed cast");
  }
  if (instructions[output].kind != (uint32_t)Kind::Tensor) invalid("program output must be a tensor");
  if (max_context == 0) invalid("program context is zero");
}

std::string Program::magic() const {
  if (options.bulk_collectives) return "IFTOKN09";
  if (options.output_rows) return "IFTOKN08";
  if (options.uncaptured_prefill) return "IFTOKN07";
  if (!options.prefill_variants.empty()) return "IFTOKN06";
  if (options.shared_pages) return "IFTOKN05";
  if (options.prefill_tokens > 1) return "IFTOKN04";
  if (options.resident_sequences > 1) return "IFTOKN03";
  return "IFTOKN02";
}

std::string Program::encode() const {
  ByteWriter w;
  std::string m = magic();
  w.raw(m);
  w.u32(max_context);
  w.u32(eos);
  w.u32(output);
  w.u32((uint32_t)instructions.size());
  int level = m[7] - '0';
  if (level >= 3) w.u32(options.resident_sequences);
  if (level >= 4) w.u32(options.prefill_tokens);
  if (level >= 5) w.u32(options.shared_pages ? 1 : 0);
  if (level >= 6) {
    w.u32((uint32_t)options.prefill_variants.size());
    for (auto v : options.prefill_variants) w.u32(v);
  }
  if (level >= 7) w.u32(options.uncaptured_prefill ? 1 : 0);
  if (level >= 8) {
    w.u32((uint32_t)output_suffix.size());
    for (auto v : output_suffix) w.u32(v);
  }
  if (level >= 9) w.u32(options.bulk_collectives ? 1 : 0);
  for (auto& ins : instructions) {
    w.u32(ins.kind);
    w.u32(ins.width);
    w.str(ins.name);
    w.str(ins.op);
    w.u32((uint32_t)ins.inputs.size());
    for (auto i : ins.inputs) w.u32(i);
    w.u32((uint32_t)ins.attrs.size());
    for (auto& kv : ins.attrs) {
      w.str(kv.first);
      w.str(kv.second);
    }
    w.str(ins.dtype);
    w.str(ins.kernel);
    w.u32(ins.logical_node);
  }
  return w.take();
}

Program Program::decode(std::string_view bytes) {
  ByteReader r(bytes);
  std::string m(r.raw(8));
  if (m.compare(0, 7, "IFTOKN0") != 0 || m[7] < '2' || m[7] > '9') invalid("not an IFTOKN02..09 program");
  int level = m[7] - '0';
  Program p;
  p.max_context = r.u32();
  p.eos = r.u32();
  p.output = r.u32();
  uint32_t n = r.u32();
  if (n == 0 || n > 20000) fail(ErrorKind::Capacity, "instruction count out of range");
  if (level >= 3) p.options.resident_sequences = r.u32();
  if (level >= 4) p.options.prefill_tokens = r.u32();
  if (level >= 5) p.options.shared_pages = r.u32() != 0;
  if (level >= 6) {
    uint32_t k = r.u32();
    if (k > 16) invalid("too many prefill variants");
    for (uint32_t i = 0; i < k; ++i) p.options.prefill_variants.push_back(r.u32());
  }
  if (level >= 7) p.options.uncaptured_prefill = r.u32() != 0;
  if (level >= 8) {
    uint32_t k = r.u32();
    if (k > n) invalid("output suffix longer than the program");
    for (uint32_t i = 0; i < k; ++i) p.output_suffix.push_back(r.u32());
    p.options.output_rows = true;
  }
  if (level >= 9) p.options.bulk_collectives = r.u32() != 0;
  for (uint32_t i = 0; i < n; ++i) {
    Instruction ins;
    ins.kind = r.u32();
    ins.width = r.u32();
    ins.name = r.str(4096);
    ins.op = r.str(64);
    uint32_t ni = r.u32();
    if (ni > 8) invalid("too many inputs");
    for (uint32_t k = 0; k < ni; ++k) ins.inputs.push_back(r.u32());
    uint32_t na = r.u32();
    if (na > 48) invalid("too many attributes");
    for (uint32_t k = 0; k < na; ++k) {
      std::string key = r.str(64), v = r.str(4096);
      ins.attrs.emplace_back(std::move(key), std::move(v));
    }
    ins.dtype = r.str(16);
    ins.kernel = r.str(128);
    ins.logical_node = r.u32();
    p.instructions.push_back(std::move(ins));
  }
  if (!r.done()) invalid("trailing bytes after the program");
  p.validate();
  return p;
}

Json Program::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.device-program.v1");
  j.set("magic", magic());
  j.set("name", name);
  j.set("max_context", max_context);
  j.set("eos", eos);
  j.set("output", output);
  j.set("parallel", parallel.to_json());
  Json o = Json::object();
  o.set("resident_sequences", options.resident_sequences);
  o.set("prefill_tokens", options.prefill_tokens);
  Json pv = Json::array();
  for (auto v : options.prefill_variants) pv.push((int64_t)v);
  o.set("prefill_variants", pv);
  o.set("uncaptured_prefill", options.uncaptured_prefill);
  o.set("shared_pages", options.shared_pages);
  o.set("output_rows", options.output_rows);
  o.set("bulk_collectives", options.bulk_collectives);
  j.set("options", o);
  j.set("launches_per_token", (int64_t)launches_per_token());
  j.set("collectives_per_token", (int64_t)collectives_per_token());
  Json arr = Json::array();
  for (auto& ins : instructions) {
    Json q = Json::object();
    q.set("name", ins.name);
    q.set("op", ins.op);
    q.set("kernel", ins.kernel);
    q.set("dtype", ins.dtype);
    q.set("kind", ins.kind);
    q.set("width", ins.width);
    Json in = Json::array();
    for (auto i : ins.inputs) in.push((int64_t)i);
    q.set("inputs", in);
    Json at = Json::object();
    for (auto& kv : ins.attrs) at.set(kv.first, kv.second);
    q.set("attrs", at);
    q.set("logical_node", ins.logical_node);
    arr.push(q);
  }
  j.set("instructions", arr);
  Json rec = Json::object();
  for (auto& kv : recipes()) rec.set(kv.first, kv.second);
  j.set("recipes", rec);
  return j;
}

std::map<std::string, size_t> Program::op_histogram() const {
  std::map<std::string, size_t> h;
  for (auto& i : instructions) ++h[i.op];
  return h;
}
size_t Program::launches_per_token() const {
  size_t n = 0;
  for (auto& i : instructions)
    if (i.kernel != "view" && i.kernel != "none") ++n;
  return n;
}
size_t Program::collectives_per_token() const {
  size_t n = 0;
  for (auto& i : instructions)
    if (i.op == "linear_allreduce" || i.op == "moe_down_allreduce" || i.op == "allreduce" || i.op == "gather" || i.op == "lm_head") ++n;
  return n;
}

}  // namespace ifab::program
