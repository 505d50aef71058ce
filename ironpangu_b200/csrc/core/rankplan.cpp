#include "rankplan.h"

#include <algorithm>

namespace ifab::rankplan {

const char* role_name(Role r) { return r == Role::Prefill ? "prefill" : "decode"; }
const char* comm_name(CommKind k) {
  switch (k) {
    case CommKind::AllReduce: return "all_reduce";
    case CommKind::AllGather: return "all_gather";
    case CommKind::ReduceScatter: return "reduce_scatter";
    case CommKind::Send: return "send";
    case CommKind::Receive: return "receive";
  }
  return "?";
}
static CommKind parse_comm(const std::string& s) {
  for (CommKind k : {CommKind::AllReduce, CommKind::AllGather, CommKind::ReduceScatter, CommKind::Send, CommKind::Receive})
    if (s == comm_name(k)) return k;
  invalid("unknown collective " + s);
}

void Spec::validate() const {
  const Model& m = model;
  const uint32_t dims[] = {m.hidden, m.intermediate, m.vocab, m.query_heads, m.kv_heads, m.head_dim, page_tokens, token_budget};
  if (m.name.empty() || m.layers.empty()) invalid("names, layers and dimensions must be nonzero");
  for (uint32_t d : dims) {
    if (d == 0) invalid("names, layers and dimensions must be nonzero");
    if (d > 16777216) invalid("dimension exceeds metadata limit");
  }
  const bool has_delta = std::find(m.layers.begin(), m.layers.end(), Layer::Delta) != m.layers.end();
  if (has_delta && (m.delta_heads == 0 || m.delta_dim == 0 || m.conv_width == 0)) invalid("delta layers need delta_heads, delta_dim and conv_width");
  if (m.query_heads % m.kv_heads) invalid("Q heads must divide into KV groups");
  for (const Mesh* mesh : {&prefill, &decode}) {
    auto pow2 = [](uint32_t v) { return v == 1 || v == 2 || v == 4 || v == 8; };
    if (!pow2(mesh->tp) || !pow2(mesh->cp)) invalid("TP and CP must be 1, 2, 4 or 8");
    if (mesh->tp * mesh->cp > 8) invalid("a mesh spans at most 8 ranks (one NVSwitch domain)");
    for (uint32_t d : {m.hidden, m.intermediate, m.query_heads})
      if (d % mesh->tp) invalid("non-divisible TP shard");
    if (m.kv_heads % mesh->tp && mesh->tp % m.kv_heads) invalid("TP width breaks the GQA grouping");
    if (has_delta && m.delta_heads % mesh->tp) invalid("non-divisible TP shard of the delta heads");
    if (mesh->sp && mesh->tp == 1) invalid("SP requires TP > 1");
  }
  if (decode.cp != 1 || decode.sp) invalid("decode runs with CP = 1 and without SP");
  if (prefill.tp != decode.tp) invalid("prefill and decode must use the same TP width (pages are not resharded)");
  for (const auto* b : {&batch_buckets, &context_buckets}) {
    if (b->empty() || (*b)[0] == 0) invalid("buckets must be positive, ascending and unique");
    for (size_t i = 1; i < b->size(); ++i)
      if ((*b)[i] <= (*b)[i - 1]) invalid("buckets must be positive, ascending and unique");
    if (b->size() > 64) invalid("metadata exceeds limits");
  }
  if (m.layers.size() > 4096) invalid("metadata exceeds limits");
}

static Json mesh_json(const Mesh& m) {
  Json j = Json::object();
  j.set("tp", m.tp);
  j.set("cp", m.cp);
  j.set("sp", m.sp);
  return j;
}
static Mesh mesh_of(const Json& j) {
  for (auto& kv : j.as_object())
    if (kv.first != "tp" && kv.first != "cp" && kv.first != "sp") invalid("mesh: unknown field " + kv.first);
  return Mesh{(uint32_t)j.at("tp").as_int(), (uint32_t)j.at("cp").as_int(), j.at("sp").as_bool()};
}

Json Spec::to_json() const {
  Json j = Json::object(), m = Json::object();
  m.set("name", model.name);
  m.set("hidden", model.hidden);
  m.set("intermediate", model.intermediate);
  m.set("vocab", model.vocab);
  m.set("query_heads", model.query_heads);
  m.set("kv_heads", model.kv_heads);
  m.set("head_dim", model.head_dim);
  m.set("delta_heads", model.delta_heads);
  m.set("delta_dim", model.delta_dim);
  m.set("conv_width", model.conv_width);
  Json ls = Json::array();
  for (auto l : model.layers) ls.push(l == Layer::Full ? "Full" : "Delta");
  m.set("layers", ls);
  j.set("model", m);
  j.set("prefill", mesh_json(prefill));
  j.set("decode", mesh_json(decode));
  j.set("page_tokens", page_tokens);
  j.set("token_budget", token_budget);
  Json bb = Json::array(), cb = Json::array();
  for (auto b : batch_buckets) bb.push((int64_t)b);
  for (auto c : context_buckets) cb.push((int64_t)c);
  j.set("batch_buckets", bb);
  j.set("context_buckets", cb);
  return j;
}

Spec Spec::from_json(const Json& j) {
  static const char* known[] = {"model", "prefill", "decode", "page_tokens", "token_budget", "batch_buckets", "context_buckets"};
  for (auto& kv : j.as_object()) {
    bool ok = false;
    for (auto k : known) ok |= kv.first == k;
    if (!ok) invalid("spec: unknown field " + kv.first);
  }
  Spec s;
  const Json& m = j.at("model");
  s.model.name = m.at("name").as_string();
  auto u = [&](const char* k) { return (uint32_t)m.at(k).as_int(); };
  s.model.hidden = u("hidden");
  s.model.intermediate = u("intermediate");
  s.model.vocab = u("vocab");
  s.model.query_heads = u("query_heads");
  s.model.kv_heads = u("kv_heads");
  s.model.head_dim = u("head_dim");
  s.model.delta_heads = m.find("delta_heads") ? u("delta_heads") : 0;
  s.model.delta_dim = m.find("delta_dim") ? u("delta_dim") : 0;
  s.model.conv_width = m.find("conv_width") ? u("conv_width") : 0;
  for (auto& l : m.at("layers").as_array()) {
    const std::string& t = l.as_string();
    if (t == "Full" || t == "full") s.model.layers.push_back(Layer::Full);
    else if (t == "Delta" || t == "delta") s.model.layers.push_back(Layer::Delta);
    else invalid("unknown layer kind " + t);
  }
  s.prefill = mesh_of(j.at("prefill"));
  s.decode = mesh_of(j.at("decode"));
  s.page_tokens = (uint32_t)j.at("page_tokens").as_int();
  s.token_budget = (uint32_t)j.at("token_budget").as_int();
  s.batch_buckets.clear();
  s.context_buckets.clear();
  for (auto& b : j.at("batch_buckets").as_array()) s.batch_buckets.push_back((uint32_t)b.as_int());
  for (auto& c : j.at("context_buckets").as_array()) s.context_buckets.push_back((uint32_t)c.as_int());
  s.validate();
  return s;
}

std::string content_key(const Spec& spec, const std::string& target) {
  return Sha256::of("inferfabric.rankplan.v1\n" + target + "\n" + spec.to_json().dump()).substr(0, 32);
}

// ---------------------------------------------------------------------------------------------
static Instruction kernel(const std::string& name, uint32_t layer) {
  Instruction i;
  i.kind = Instruction::Kind::Kernel;
  i.name = name;
  i.layer = layer;
  return i;
}
static Instruction comm(CommKind k, const std::string& group, uint32_t layer, uint64_t elements, uint32_t peer = 0) {
  Instruction i;
  i.kind = Instruction::Kind::Communication;
  i.name = comm_name(k);
  i.comm = k;
  i.group = group;
  i.layer = layer;
  i.elements = elements;
  i.peer = peer;
  return i;
}
static Instruction fence(const std::string& label, uint32_t layer) {
  Instruction i;
  i.kind = Instruction::Kind::Fence;
  i.name = label;
  i.layer = layer;
  return i;
}

Artifact compile(const Spec& spec, const std::string& target) {
  spec.validate();
  Artifact a;
  a.key = content_key(spec, target);
  a.target = target;
  a.spec = spec;
  for (uint32_t b : spec.batch_buckets)
    for (uint32_t c : spec.context_buckets) a.buckets.push_back({b, c});
  const Model& m = spec.model;
  for (Role role : {Role::Prefill, Role::Decode}) {
    const Mesh& mesh = role == Role::Prefill ? spec.prefill : spec.decode;
    for (uint32_t rank = 0; rank < mesh.ranks(); ++rank) {
      RankPlan p;
      p.role = role;
      p.rank = rank;
      p.tp_rank = rank % mesh.tp;
      p.cp_rank = rank / mesh.tp;
      auto& out = p.instructions;
      out.push_back(kernel("embedding", 0));
      for (uint32_t l = 0; l < m.layers.size(); ++l) {
        const bool full = m.layers[l] == Layer::Full;
        out.push_back(kernel("rmsnorm", l));
        if (mesh.sp) out.push_back(comm(CommKind::AllGather, "tp", l, m.hidden));   // tokens were sequence-sharded
        if (full) {
          out.push_back(kernel("qkv_projection_column_parallel", l));
          out.push_back(kernel("rope_kv_append", l));
          p.states.emplace_back(StateKind::Kv, l);
          if (mesh.cp > 1) {
            // causal ring: pass the local KV shard around, merging partial attention with online softmax
            const uint32_t nxt = ((p.cp_rank + 1) % mesh.cp) * mesh.tp + p.tp_rank;
            const uint32_t prv = ((p.cp_rank + mesh.cp - 1) % mesh.cp) * mesh.tp + p.tp_rank;
            out.push_back(kernel("causal_attention_local_shard", l));
            for (uint32_t step = 1; step < mesh.cp; ++step) {
              out.push_back(comm(CommKind::Send, "cp", l, (uint64_t)2 * m.kv_heads / mesh.tp * m.head_dim, nxt));
              out.push_back(comm(CommKind::Receive, "cp", l, (uint64_t)2 * m.kv_heads / mesh.tp * m.head_dim, prv));
              out.push_back(kernel("causal_attention_online_softmax_merge_" + std::to_string(step), l));
            }
          } else {
            out.push_back(kernel("paged_attention", l));
          }
          out.push_back(kernel("o_projection_row_parallel", l));
        } else {
          out.push_back(kernel("delta_in_projection_column_parallel", l));
          out.push_back(kernel("causal_conv_silu", l));
          p.states.emplace_back(StateKind::Conv, l);
          if (mesh.cp > 1) {
            // the recurrent state flows through the context ranks in order
            if (p.cp_rank > 0) out.push_back(comm(CommKind::Receive, "cp", l, (uint64_t)m.delta_heads / mesh.tp * m.delta_dim * m.delta_dim, (p.cp_rank - 1) * mesh.tp + p.tp_rank));
            out.push_back(kernel("gated_delta_recurrence", l));
            if (p.cp_rank + 1 < mesh.cp) out.push_back(comm(CommKind::Send, "cp", l, (uint64_t)m.delta_heads / mesh.tp * m.delta_dim * m.delta_dim, (p.cp_rank + 1) * mesh.tp + p.tp_rank));
          } else {
            out.push_back(kernel("gated_delta_recurrence", l));
          }
          p.states.emplace_back(StateKind::Recurrent, l);
          out.push_back(kernel("gated_rmsnorm", l));
          out.push_back(kernel("delta_out_projection_row_parallel", l));
        }
        if (mesh.tp > 1) out.push_back(comm(mesh.sp ? CommKind::ReduceScatter : CommKind::AllReduce, "tp", l, m.hidden));
        out.push_back(kernel("residual_rmsnorm", l));
        if (mesh.sp) out.push_back(comm(CommKind::AllGather, "tp", l, m.hidden));
        out.push_back(kernel("gate_up_projection_column_parallel_swiglu", l));
        out.push_back(kernel("down_projection_row_parallel", l));
        if (mesh.tp > 1) out.push_back(comm(mesh.sp ? CommKind::ReduceScatter : CommKind::AllReduce, "tp", l, m.hidden));
        out.push_back(kernel("residual_add", l));
      }
      const uint32_t last = (uint32_t)m.layers.size();
      if (mesh.sp) out.push_back(comm(CommKind::AllGather, "tp", last, m.hidden));
      out.push_back(kernel("final_rmsnorm", last));
      out.push_back(kernel("lm_head_column_parallel", last));
      if (mesh.tp > 1) out.push_back(comm(CommKind::AllGather, "tp", last, m.vocab / mesh.tp));
      out.push_back(kernel("select_frontier", last));
      if (role == Role::Prefill) {
        out.push_back(fence("prefill_complete", last));
        // hand the pages of this TP shard to the decode rank with the same tp index
        out.push_back(comm(CommKind::Send, "pd", last, (uint64_t)spec.page_tokens, p.tp_rank));
      } else {
        out.push_back(fence("step_complete", last));
      }
      a.plans.push_back(std::move(p));
    }
  }
  return a;
}

// ---------------------------------------------------------------------------------------------
Json Artifact::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.rank-plans.v1");
  j.set("key", key);
  j.set("target", target);
  j.set("spec", spec.to_json());
  Json bs = Json::array();
  for (auto& b : buckets) {
    Json o = Json::object();
    o.set("batch", b.batch);
    o.set("context", b.context);
    bs.push(o);
  }
  j.set("buckets", bs);
  Json ps = Json::array();
  for (auto& p : plans) {
    Json o = Json::object();
    o.set("role", role_name(p.role));
    o.set("rank", p.rank);
    o.set("tp_rank", p.tp_rank);
    o.set("cp_rank", p.cp_rank);
    Json is = Json::array();
    for (auto& i : p.instructions) {
      Json q = Json::object();
      q.set("kind", i.kind == Instruction::Kind::Kernel ? "kernel" : i.kind == Instruction::Kind::Fence ? "fence" : "communication");
      q.set("name", i.name);
      q.set("layer", i.layer);
      if (i.kind == Instruction::Kind::Communication) {
        q.set("group", i.group);
        q.set("elements", i.elements);
        if (i.comm == CommKind::Send || i.comm == CommKind::Receive) q.set("peer", i.peer);
      }
      is.push(q);
    }
    o.set("instructions", is);
    Json st = Json::array();
    for (auto& s : p.states) {
      Json q = Json::object();
      q.set("kind", s.first == StateKind::Kv ? "kv" : s.first == StateKind::Recurrent ? "recurrent" : "conv");
      q.set("layer", s.second);
      st.push(q);
    }
    o.set("states", st);
    ps.push(o);
  }
  j.set("plans", ps);
  return j;
}

Artifact Artifact::from_json(const Json& j) {
  if (j.at("format").as_string() != "inferfabric.rank-plans.v1") invalid("not a rank-plan artifact");
  Artifact a;
  a.key = j.at("key").as_string();
  a.target = j.at("target").as_string();
  a.spec = Spec::from_json(j.at("spec"));
  for (auto& b : j.at("buckets").as_array()) a.buckets.push_back({(uint32_t)b.at("batch").as_int(), (uint32_t)b.at("context").as_int()});
  for (auto& p : j.at("plans").as_array()) {
    RankPlan r;
    r.role = p.at("role").as_string() == "prefill" ? Role::Prefill : Role::Decode;
    r.rank = (uint32_t)p.at("rank").as_int();
    r.tp_rank = (uint32_t)p.at("tp_rank").as_int();
    r.cp_rank = (uint32_t)p.at("cp_rank").as_int();
    for (auto& q : p.at("instructions").as_array()) {
      Instruction i;
      const std::string& k = q.at("kind").as_string();
      i.kind = k == "kernel" ? Instruction::Kind::Kernel : k == "fence" ? Instruction::Kind::Fence : Instruction::Kind::Communication;
      i.name = q.at("name").as_string();
      i.layer = (uint32_t)q.at("layer").as_int();
      if (i.kind == Instruction::Kind::Communication) {
        i.comm = parse_comm(i.name);
        i.group = q.at("group").as_string();
        i.elements = (uint64_t)q.at("elements").as_int();
        if (auto pr = q.find("peer")) i.peer = (uint32_t)pr->as_int();
      }
      r.instructions.push_back(std::move(i));
    }
    for (auto& s : p.at("states").as_array()) {
      const std::string& k = s.at("kind").as_string();
      r.states.emplace_back(k == "kv" ? StateKind::Kv : k == "recurrent" ? StateKind::Recurrent : StateKind::Conv, (uint32_t)s.at("layer").as_int());
    }
    a.plans.push_back(std::move(r));
  }
  return a;
}

std::string encode(const Artifact& a) {
  std::string body = a.to_json().dump();
  std::string out("PANGU\0\0\x01", 8);
  out += Sha256::of(body);
  out += body;
  return out;
}
Artifact decode(std::string_view bytes) {
  if (bytes.size() < 72 || bytes.substr(0, 8) != std::string_view("PANGU\0\0\x01", 8)) invalid("not a rank-plan artifact");
  std::string_view sha = bytes.substr(8, 64), body = bytes.substr(72);
  if (Sha256::of(body) != sha) fail(ErrorKind::Stale, "rank-plan artifact: integrity hash mismatch");
  return Artifact::from_json(Json::parse(body));
}

Artifact cached(const Spec& spec, const std::string& target, const std::string& cache_dir, bool* hit) {
  const std::string key = content_key(spec, target);
  const std::string path = cache_dir + "/" + key + ".inferfabric-bin";
  if (hit) *hit = false;
  if (path_exists(path)) {
    try {
      Artifact a = decode(read_file(path));
      if (a.key == key) {
        if (hit) *hit = true;
        return a;
      }
    } catch (const Error&) {
      // a damaged cache entry is recompiled and replaced
    }
  }
  Artifact a = compile(spec, target);
  make_dirs(cache_dir);
  write_file_atomic(path, encode(a));
  return a;
}

}  // namespace ifab::rankplan
