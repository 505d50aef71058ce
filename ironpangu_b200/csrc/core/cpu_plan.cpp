#include "cpu_plan.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <set>

#include "lang.h"

namespace ifab::cpu {

const char* op_name(Op op) {
  switch (op) {
    case Op::Add: return "add";
    case Op::Mul: return "mul";
    case Op::Relu: return "relu";
    case Op::Matmul: return "matmul";
  }
  return "?";
}
static Op parse_op(const std::string& s) {
  if (s == "add") return Op::Add;
  if (s == "mul") return Op::Mul;
  if (s == "relu") return Op::Relu;
  if (s == "matmul") return Op::Matmul;
  invalid("unsupported cpu op " + s);
}
const char* kernel_name(Kernel k) {
  switch (k) {
    case Kernel::AddF32V1: return "AddF32V1";
    case Kernel::MulF32V1: return "MulF32V1";
    case Kernel::ReluF32V1: return "ReluF32V1";
    case Kernel::MatmulNaiveF32V1: return "MatmulNaiveF32V1";
    case Kernel::MatmulBlockedF32V1: return "MatmulBlockedF32V1";
  }
  return "?";
}
static Kernel parse_kernel(const std::string& s) {
  for (Kernel k : {Kernel::AddF32V1, Kernel::MulF32V1, Kernel::ReluF32V1, Kernel::MatmulNaiveF32V1, Kernel::MatmulBlockedF32V1})
    if (s == kernel_name(k)) return k;
  invalid("unknown kernel " + s);
}
Op kernel_op(Kernel k) {
  switch (k) {
    case Kernel::AddF32V1: return Op::Add;
    case Kernel::MulF32V1: return Op::Mul;
    case Kernel::ReluF32V1: return Op::Relu;
    default: return Op::Matmul;
  }
}
static const char* storage_name(Storage s) {
  switch (s) {
    case Storage::Input: return "input";
    case Storage::Constant: return "constant";
    case Storage::State: return "state";
    case Storage::Temporary: return "temporary";
  }
  return "?";
}
static Storage parse_storage(const std::string& s) {
  if (s == "input") return Storage::Input;
  if (s == "constant") return Storage::Constant;
  if (s == "state") return Storage::State;
  if (s == "temporary") return Storage::Temporary;
  invalid("unknown storage " + s);
}
size_t Buffer::elements() const {
  size_t n = 1;
  for (auto d : shape) n *= d;
  return n;
}

// ---------------------------------------------------------------------------------------------
static std::vector<size_t> shape_of(const Json& j) {
  std::vector<size_t> s;
  for (auto& d : j.as_array()) {
    int64_t v = d.as_int();
    if (v <= 0 || v > (1 << 20)) invalid("bad dimension");
    s.push_back((size_t)v);
  }
  if (s.empty() || s.size() > 4) invalid("tensor rank must be 1..4");
  return s;
}
static Json shape_json(const std::vector<size_t>& s) {
  Json a = Json::array();
  for (auto d : s) a.push((int64_t)d);
  return a;
}
static Json floats_json(const std::vector<float>& v) {
  Json a = Json::array();
  for (float x : v) a.push((double)x);
  return a;
}
static std::vector<float> floats_of(const Json& j) {
  std::vector<float> v;
  for (auto& x : j.as_array()) v.push_back((float)x.as_double());
  return v;
}

LogicalGraph LogicalGraph::from_json(const Json& j) {
  LogicalGraph g;
  g.version = (uint32_t)j.at("version").as_int();
  if (g.version != 1) invalid("unsupported logical graph version");
  g.name = j.at("name").as_string();
  for (auto& t : j.at("inputs").as_array()) g.inputs.push_back({t.at("name").as_string(), shape_of(t.at("shape"))});
  auto consts = [&](const char* key, std::vector<ConstantDecl>& out) {
    if (auto arr = j.find(key))
      for (auto& t : arr->as_array()) {
        ConstantDecl c{t.at("name").as_string(), shape_of(t.at("shape")), floats_of(t.at("data"))};
        size_t n = 1;
        for (auto d : c.shape) n *= d;
        if (n != c.data.size()) invalid(c.name + ": data length does not match shape");
        out.push_back(std::move(c));
      }
  };
  consts("constants", g.constants);
  consts("states", g.states);
  for (auto& n : j.at("nodes").as_array()) {
    LogicalNode x{n.at("name").as_string(), parse_op(n.at("op").as_string()), {}};
    for (auto& i : n.at("inputs").as_array()) x.inputs.push_back(i.as_string());
    g.nodes.push_back(std::move(x));
  }
  for (auto& o : j.at("outputs").as_array()) g.outputs.push_back(o.as_string());
  if (auto u = j.find("updates"))
    for (auto& kv : u->as_object()) g.updates[kv.first] = kv.second.as_string();
  return g;
}

Json LogicalGraph::to_json() const {
  Json j = Json::object();
  j.set("version", version);
  j.set("name", name);
  Json in = Json::array();
  for (auto& t : inputs) {
    Json o = Json::object();
    o.set("name", t.name);
    o.set("shape", shape_json(t.shape));
    in.push(o);
  }
  j.set("inputs", in);
  auto consts = [&](const char* key, const std::vector<ConstantDecl>& v) {
    Json a = Json::array();
    for (auto& c : v) {
      Json o = Json::object();
      o.set("name", c.name);
      o.set("shape", shape_json(c.shape));
      o.set("data", floats_json(c.data));
      a.push(o);
    }
    j.set(key, a);
  };
  consts("constants", constants);
  consts("states", states);
  Json ns = Json::array();
  for (auto& n : nodes) {
    Json o = Json::object();
    o.set("name", n.name);
    o.set("op", op_name(n.op));
    Json i = Json::array();
    for (auto& s : n.inputs) i.push(s);
    o.set("inputs", i);
    ns.push(o);
  }
  j.set("nodes", ns);
  Json outs = Json::array();
  for (auto& o : outputs) outs.push(o);
  j.set("outputs", outs);
  Json up = Json::object();
  for (auto& kv : updates) up.set(kv.first, kv.second);
  j.set("updates", up);
  return j;
}

static std::vector<size_t> parse_dims(const std::string& s) {
  std::vector<size_t> d;
  size_t b = 1;
  while (b < s.size() - 1) {
    size_t e = s.find(',', b);
    if (e == std::string::npos) e = s.size() - 1;
    d.push_back((size_t)std::stoul(s.substr(b, e - b)));
    b = e + 1;
  }
  return d;
}
static std::vector<float> parse_floats(const std::string& s) {
  std::vector<float> d;
  size_t b = 1;
  while (b < s.size() - 1) {
    size_t e = s.find(',', b);
    if (e == std::string::npos) e = s.size() - 1;
    d.push_back(std::stof(s.substr(b, e - b)));
    b = e + 1;
  }
  return d;
}

LogicalGraph from_dsl(std::string_view source) { return from_expanded(lang::expand(lang::parse(source))); }

LogicalGraph from_expanded(const lang::Expanded& ex) {
  auto t = ex.plan.find("target");
  if (t == ex.plan.end() || t->second != "cpu_f32_v1") invalid("plan target must be cpu_f32_v1");
  LogicalGraph g;
  g.name = ex.model_name;
  for (auto& n : ex.nodes) {
    auto attr = [&](const char* k) -> const std::string& {
      for (auto& kv : n.attrs)
        if (kv.first == k) return kv.second;
      invalid("node " + n.name + " lacks " + k);
    };
    if (n.op == "input") g.inputs.push_back({n.name, parse_dims(attr("shape"))});
    else if (n.op == "const") g.constants.push_back({n.name, parse_dims(attr("shape")), parse_floats(attr("data"))});
    else if (n.op == "state") g.states.push_back({n.name, parse_dims(attr("shape")), parse_floats(attr("data"))});
    else {
      if (!n.attrs.empty()) invalid("cpu op " + n.op + " takes no attributes");
      g.nodes.push_back({n.name, parse_op(n.op), n.inputs});
    }
  }
  g.outputs.push_back(ex.output);
  for (auto& kv : ex.fields)
    if (kv.first.rfind("update.", 0) == 0) g.updates[kv.first.substr(7)] = kv.second;
    else invalid("cpu model: unknown field " + kv.first);
  return g;
}

// ---------------------------------------------------------------------------------------------
namespace {

void eval_kernel(Kernel k, const std::vector<const float*>& in, const std::vector<std::vector<size_t>>& shapes, float* out) {
  auto count = [](const std::vector<size_t>& s) {
    size_t n = 1;
    for (auto d : s) n *= d;
    return n;
  };
  switch (k) {
    case Kernel::AddF32V1: {
      size_t n = count(shapes[0]);
      for (size_t i = 0; i < n; ++i) out[i] = in[0][i] + in[1][i];
      break;
    }
    case Kernel::MulF32V1: {
      size_t n = count(shapes[0]);
      for (size_t i = 0; i < n; ++i) out[i] = in[0][i] * in[1][i];
      break;
    }
    case Kernel::ReluF32V1: {
      size_t n = count(shapes[0]);
      for (size_t i = 0; i < n; ++i) out[i] = in[0][i] > 0.f ? in[0][i] : 0.f;
      break;
    }
    case Kernel::MatmulNaiveF32V1:
    case Kernel::MatmulBlockedF32V1: {
      const size_t M = shapes[0][0], K = shapes[0][1], N = shapes[1][1];
      if (k == Kernel::MatmulNaiveF32V1) {
        for (size_t m = 0; m < M; ++m)
          for (size_t n = 0; n < N; ++n) {
            float s = 0.f;
            for (size_t kk = 0; kk < K; ++kk) s += in[0][m * K + kk] * in[1][kk * N + n];
            out[m * N + n] = s;
          }
      } else {
        // same summation order per output element as the naive kernel (k ascending), tiled over m/n
        constexpr size_t B = 32;
        for (size_t m0 = 0; m0 < M; m0 += B)
          for (size_t n0 = 0; n0 < N; n0 += B)
            for (size_t m = m0; m < std::min(M, m0 + B); ++m)
              for (size_t n = n0; n < std::min(N, n0 + B); ++n) {
                float s = 0.f;
                for (size_t kk = 0; kk < K; ++kk) s += in[0][m * K + kk] * in[1][kk * N + n];
                out[m * N + n] = s;
              }
      }
      break;
    }
  }
}

std::vector<size_t> infer_shape(Op op, const std::vector<std::vector<size_t>>& in, const std::string& name) {
  switch (op) {
    case Op::Add:
    case Op::Mul:
      if (in.size() != 2) invalid(name + ": expects two inputs");
      if (in[0] != in[1]) invalid(name + ": operand shapes differ");
      return in[0];
    case Op::Relu:
      if (in.size() != 1) invalid(name + ": expects one input");
      return in[0];
    case Op::Matmul:
      if (in.size() != 2 || in[0].size() != 2 || in[1].size() != 2) invalid(name + ": matmul takes two rank-2 tensors");
      if (in[0][1] != in[1][0]) invalid(name + ": inner dimensions differ");
      return {in[0][0], in[1][1]};
  }
  return {};
}

size_t work_of(Op op, const std::vector<std::vector<size_t>>& in) {
  if (op == Op::Matmul) return in[0][0] * in[0][1] * in[1][1];
  size_t n = 1;
  for (auto d : in[0]) n *= d;
  return n;
}

}  // namespace

PhysicalPlan compile(const LogicalGraph& g, const Options& opt, Stages* stages) {
  struct V { std::string name; std::vector<size_t> shape; Storage st; std::vector<float> data; bool is_const = false; };
  std::vector<V> values;
  std::map<std::string, size_t> index;
  auto add_value = [&](V v) {
    if (!index.emplace(v.name, values.size()).second) invalid("duplicate value name " + v.name);
    values.push_back(std::move(v));
  };
  for (auto& t : g.inputs) add_value({t.name, t.shape, Storage::Input, {}, false});
  for (auto& c : g.constants) add_value({c.name, c.shape, Storage::Constant, c.data, true});
  for (auto& s : g.states) add_value({s.name, s.shape, Storage::State, s.data, false});
  struct TN { std::string name; Op op; std::vector<size_t> in; size_t out; };
  std::vector<TN> nodes;
  for (auto& n : g.nodes) {
    TN t{n.name, n.op, {}, 0};
    std::vector<std::vector<size_t>> shapes;
    for (auto& s : n.inputs) {
      auto it = index.find(s);
      if (it == index.end()) invalid("node " + n.name + " uses undefined value " + s + " (graph must be topologically ordered)");
      t.in.push_back(it->second);
      shapes.push_back(values[it->second].shape);
    }
    t.out = values.size();
    add_value({n.name, infer_shape(n.op, shapes, n.name), Storage::Temporary, {}, false});
    nodes.push_back(std::move(t));
  }
  std::vector<size_t> outs;
  for (auto& o : g.outputs) {
    auto it = index.find(o);
    if (it == index.end()) invalid("unknown output " + o);
    outs.push_back(it->second);
  }
  if (outs.empty()) invalid("graph has no outputs");
  auto dump_nodes = [&](const std::vector<TN>& list) {
    Json vals = Json::array(), ns = Json::array();
    for (auto& v : values) {
      Json j = Json::object(), shp = Json::array();
      for (size_t d : v.shape) shp.push((int64_t)d);
      j.set("name", v.name);
      j.set("shape", shp);
      j.set("storage", v.st == Storage::Input ? "input" : v.st == Storage::Constant ? "constant" : v.st == Storage::State ? "state" : "temporary");
      vals.push(std::move(j));
    }
    for (auto& n : list) {
      Json j = Json::object(), in = Json::array();
      for (size_t i : n.in) in.push(values[i].name);
      j.set("name", n.name);
      j.set("op", op_name(n.op));
      j.set("inputs", in);
      ns.push(std::move(j));
    }
    Json out = Json::object();
    out.set("values", vals);
    out.set("nodes", ns);
    return out;
  };
  if (stages) stages->typed = dump_nodes(nodes);
  std::map<size_t, size_t> updates;
  for (auto& kv : g.updates) {
    auto s = index.find(kv.first), v = index.find(kv.second);
    if (s == index.end() || values[s->second].st != Storage::State) invalid("update of unknown state " + kv.first);
    if (v == index.end()) invalid("update from unknown value " + kv.second);
    if (values[s->second].shape != values[v->second].shape) invalid("update of " + kv.first + " changes its shape");
    updates[s->second] = v->second;
  }
  // dead-code elimination
  std::vector<char> live(values.size(), 0);
  std::vector<size_t> stack(outs.begin(), outs.end());
  for (auto& kv : updates) stack.push_back(kv.second);
  std::map<size_t, size_t> producer;
  for (size_t i = 0; i < nodes.size(); ++i) producer[nodes[i].out] = i;
  while (!stack.empty()) {
    size_t v = stack.back();
    stack.pop_back();
    if (live[v]) continue;
    live[v] = 1;
    auto p = producer.find(v);
    if (p != producer.end())
      for (size_t in : nodes[p->second].in) stack.push_back(in);
  }
  PhysicalPlan plan;
  plan.name = g.name;
  size_t eliminated = 0;
  // constant folding (bounded total work)
  size_t budget = opt.fold_work_limit;
  std::vector<TN> kept;
  for (auto& n : nodes) {
    if (!live[n.out]) { ++eliminated; continue; }
    bool all_const = true;
    std::vector<std::vector<size_t>> shapes;
    for (size_t in : n.in) {
      all_const &= values[in].is_const;
      shapes.push_back(values[in].shape);
    }
    size_t work = work_of(n.op, shapes);
    if (all_const && work <= budget && !opt.override_kernels.count(n.name)) {
      budget -= work;
      std::vector<const float*> ptrs;
      for (size_t in : n.in) ptrs.push_back(values[in].data.data());
      V& o = values[n.out];
      size_t cnt = 1;
      for (auto d : o.shape) cnt *= d;
      o.data.assign(cnt, 0.f);
      Kernel k = n.op == Op::Add ? Kernel::AddF32V1 : n.op == Op::Mul ? Kernel::MulF32V1 : n.op == Op::Relu ? Kernel::ReluF32V1 : Kernel::MatmulNaiveF32V1;
      eval_kernel(k, ptrs, shapes, o.data.data());
      o.is_const = true;
      o.st = Storage::Constant;
      ++plan.folded_constants;
      continue;
    }
    kept.push_back(n);
  }
  if (stages) {
    stages->optimized = dump_nodes(kept);
    stages->optimized.set("folded_constants", (int64_t)plan.folded_constants);
    stages->optimized.set("eliminated_nodes", (int64_t)eliminated);
  }
  // constants that only fed folded nodes may now be dead: recompute liveness over kept nodes
  std::fill(live.begin(), live.end(), 0);
  for (size_t o : outs) live[o] = 1;
  for (auto& kv : updates) live[kv.second] = live[kv.first] = 1;
  for (auto it = kept.rbegin(); it != kept.rend(); ++it)
    if (live[it->out])
      for (size_t in : it->in) live[in] = 1;
  for (size_t i = 0; i < values.size(); ++i)
    if (values[i].st == Storage::Input || values[i].st == Storage::State) live[i] = 1;  // interface values stay
  // value compaction
  std::vector<size_t> remap(values.size(), SIZE_MAX);
  for (size_t i = 0; i < values.size(); ++i) {
    if (!live[i]) continue;
    remap[i] = plan.buffers.size();
    Buffer b;
    b.name = values[i].name;
    b.shape = values[i].shape;
    b.storage = values[i].st;
    if (values[i].st == Storage::Constant || values[i].st == Storage::State) b.initial = values[i].data;
    plan.buffers.push_back(std::move(b));
  }
  plan.eliminated_nodes = eliminated;
  // steps + lifetimes
  for (size_t si = 0; si < kept.size(); ++si) {
    const TN& n = kept[si];
    Step s;
    s.name = n.name;
    std::vector<std::vector<size_t>> shapes;
    for (size_t in : n.in) {
      s.inputs.push_back(remap[in]);
      shapes.push_back(values[in].shape);
    }
    s.output = remap[n.out];
    auto ov = opt.override_kernels.find(n.name);
    if (ov != opt.override_kernels.end()) {
      if (kernel_op(ov->second) != n.op) invalid("override for " + n.name + " does not implement " + op_name(n.op));
      s.kernel = ov->second;
      s.selection_reason = "forced by override";
    } else if (n.op == Op::Matmul) {
      size_t macs = work_of(n.op, shapes);
      s.kernel = macs >= 4096 ? Kernel::MatmulBlockedF32V1 : Kernel::MatmulNaiveF32V1;
      s.selection_reason = std::to_string(macs) + " MACs " + (macs >= 4096 ? ">= 4096: blocked tiles" : "< 4096: naive loop");
    } else {
      s.kernel = n.op == Op::Add ? Kernel::AddF32V1 : n.op == Op::Mul ? Kernel::MulF32V1 : Kernel::ReluF32V1;
      s.selection_reason = "only candidate";
    }
    plan.steps.push_back(std::move(s));
  }
  const size_t nsteps = plan.steps.size();
  for (size_t si = 0; si < nsteps; ++si) {
    Buffer& o = plan.buffers[plan.steps[si].output];
    o.has_lifetime = true;
    o.first = o.last = si;
  }
  for (size_t si = 0; si < nsteps; ++si)
    for (size_t in : plan.steps[si].inputs) {
      Buffer& b = plan.buffers[in];
      if (b.storage == Storage::Temporary && b.has_lifetime) b.last = std::max(b.last, si);
    }
  for (size_t o : outs) {
    plan.outputs.push_back(remap[o]);
    Buffer& b = plan.buffers[remap[o]];
    if (b.storage == Storage::Temporary) b.last = nsteps;   // outputs outlive the run
  }
  for (auto& kv : updates) {
    plan.updates[remap[kv.first]] = remap[kv.second];
    Buffer& b = plan.buffers[remap[kv.second]];
    if (b.storage == Storage::Temporary) b.last = nsteps;
  }
  // first-fit offsets in step order, 64-byte lines
  struct Live { size_t off, bytes, last, buf; };
  std::vector<Live> livev;
  for (size_t si = 0; si < nsteps; ++si) {
    Step& s = plan.steps[si];
    Buffer& o = plan.buffers[s.output];
    const size_t need = (o.bytes() + 63) / 64 * 64;
    // bytes freed before this step may be reused; the reuse dependency is the last reader
    std::vector<Live> still;
    std::vector<Live> freed;
    for (auto& l : livev) (l.last < si ? freed : still).push_back(l);
    livev = still;
    std::sort(livev.begin(), livev.end(), [](const Live& a, const Live& b) { return a.off < b.off; });
    size_t off = 0;
    for (auto& l : livev) {
      if (off + need <= l.off) break;
      off = std::max(off, l.off + l.bytes);
    }
    o.has_offset = true;
    o.offset = off;
    plan.arena_bytes = std::max(plan.arena_bytes, off + need);
    livev.push_back({off, need, o.last, s.output});
    for (size_t in : s.inputs) {
      const Buffer& b = plan.buffers[in];
      if (b.storage == Storage::Temporary)
        for (size_t k = 0; k < si; ++k)
          if (plan.steps[k].output == in) s.dependencies.push_back(k);
    }
  }
  // reuse dependencies: for every earlier buffer whose bytes overlap, the steps that read it last
  for (size_t si = 0; si < nsteps; ++si) {
    Step& s = plan.steps[si];
    const Buffer& o = plan.buffers[s.output];
    std::set<size_t> deps;
    for (size_t k = 0; k < si; ++k) {
      const Buffer& e = plan.buffers[plan.steps[k].output];
      const size_t eb = (e.bytes() + 63) / 64 * 64, ob = (o.bytes() + 63) / 64 * 64;
      if (e.offset + eb <= o.offset || o.offset + ob <= e.offset) continue;
      // e's bytes are overwritten by s: every reader of e (and its producer) must have finished
      deps.insert(k);
      for (size_t r = k + 1; r < si; ++r)
        for (size_t in : plan.steps[r].inputs)
          if (in == plan.steps[k].output) deps.insert(r);
    }
    for (size_t d : s.dependencies) deps.erase(d);
    s.reuse_dependencies.assign(deps.begin(), deps.end());
  }
  return plan;
}

void verify(const PhysicalPlan& p) {
  const size_t n = p.steps.size();
  for (auto& b : p.buffers) {
    if (b.storage == Storage::Temporary) {
      if (!b.has_offset || !b.has_lifetime) invalid("verify: temporary " + b.name + " has no placement");
      if (b.offset % 64) invalid("verify: " + b.name + " is not 64-byte aligned");
      if (b.offset + b.bytes() > p.arena_bytes) invalid("verify: " + b.name + " exceeds the arena");
    } else if ((b.storage == Storage::Constant || b.storage == Storage::State) && b.initial.size() != b.elements()) {
      invalid("verify: " + b.name + " initial data does not match its shape");
    }
  }
  for (size_t si = 0; si < n; ++si) {
    const Step& s = p.steps[si];
    if (s.output >= p.buffers.size()) invalid("verify: step output out of range");
    const Buffer& o = p.buffers[s.output];
    if (o.storage != Storage::Temporary) invalid("verify: step " + s.name + " writes a non-temporary buffer");
    if (o.first != si) invalid("verify: lifetime of " + o.name + " does not start at its producer");
    for (size_t in : s.inputs) {
      if (in >= p.buffers.size()) invalid("verify: step input out of range");
      const Buffer& b = p.buffers[in];
      if (b.storage == Storage::Temporary) {
        if (!(b.first < si && si <= b.last)) invalid("verify: step " + s.name + " reads " + b.name + " outside its lifetime");
        if (in == s.output) invalid("verify: step " + s.name + " aliases its own input");
        bool dep = false;
        for (size_t d : s.dependencies) dep |= p.steps.at(d).output == in;
        if (!dep) invalid("verify: step " + s.name + " lacks a dependency on the producer of " + b.name);
      }
    }
    for (size_t d : s.dependencies)
      if (d >= si) invalid("verify: dependency on a later step");
    // aliasing: two temporaries that are live together must not share bytes
    for (size_t k = 0; k < si; ++k) {
      const Buffer& e = p.buffers[p.steps[k].output];
      const bool space = !(e.offset + e.bytes() <= o.offset || o.offset + o.bytes() <= e.offset);
      if (!space) continue;
      if (e.last >= si) invalid("verify: " + o.name + " overwrites " + e.name + " while it is live");
      // all readers of e must be ordered before s through dependencies or reuse dependencies
      std::set<size_t> need{k};
      for (size_t r = k + 1; r < si; ++r)
        for (size_t in : p.steps[r].inputs)
          if (in == p.steps[k].output) need.insert(r);
      for (size_t r : need) {
        bool ok = std::find(s.dependencies.begin(), s.dependencies.end(), r) != s.dependencies.end() ||
                  std::find(s.reuse_dependencies.begin(), s.reuse_dependencies.end(), r) != s.reuse_dependencies.end();
        if (!ok) invalid("verify: step " + s.name + " reuses bytes of " + e.name + " without a reuse dependency on step " + p.steps[r].name);
      }
    }
  }
  for (size_t o : p.outputs)
    if (o >= p.buffers.size()) invalid("verify: output out of range");
  for (auto& kv : p.updates) {
    if (kv.first >= p.buffers.size() || kv.second >= p.buffers.size()) invalid("verify: update out of range");
    if (p.buffers[kv.first].storage != Storage::State) invalid("verify: update target is not a state");
    if (p.buffers[kv.first].shape != p.buffers[kv.second].shape) invalid("verify: update changes the state's shape");
  }
}

// ---------------------------------------------------------------------------------------------
Json PhysicalPlan::to_json() const {
  Json j = Json::object();
  j.set("version", version);
  j.set("name", name);
  j.set("target", target);
  j.set("policy", policy);
  j.set("arena_bytes", (int64_t)arena_bytes);
  j.set("folded_constants", (int64_t)folded_constants);
  j.set("eliminated_nodes", (int64_t)eliminated_nodes);
  Json bs = Json::array();
  for (auto& b : buffers) {
    Json o = Json::object();
    o.set("name", b.name);
    o.set("shape", shape_json(b.shape));
    o.set("storage", storage_name(b.storage));
    if (!b.initial.empty()) o.set("initial", floats_json(b.initial));
    if (b.has_offset) o.set("offset", (int64_t)b.offset);
    if (b.has_lifetime) {
      Json l = Json::array();
      l.push((int64_t)b.first);
      l.push((int64_t)b.last);
      o.set("lifetime", l);
    }
    bs.push(o);
  }
  j.set("buffers", bs);
  Json ss = Json::array();
  for (auto& s : steps) {
    Json o = Json::object();
    o.set("name", s.name);
    o.set("kernel", kernel_name(s.kernel));
    auto list = [](const std::vector<size_t>& v) {
      Json a = Json::array();
      for (auto x : v) a.push((int64_t)x);
      return a;
    };
    o.set("inputs", list(s.inputs));
    o.set("output", (int64_t)s.output);
    o.set("rank", (int64_t)s.rank);
    o.set("stream", (int64_t)s.stream);
    o.set("dependencies", list(s.dependencies));
    o.set("reuse_dependencies", list(s.reuse_dependencies));
    o.set("selection_reason", s.selection_reason);
    ss.push(o);
  }
  j.set("steps", ss);
  Json outs = Json::array();
  for (auto o : outputs) outs.push((int64_t)o);
  j.set("outputs", outs);
  Json up = Json::object();
  for (auto& kv : updates) up.set(std::to_string(kv.first), (int64_t)kv.second);
  j.set("updates", up);
  return j;
}

PhysicalPlan PhysicalPlan::from_json(const Json& j) {
  PhysicalPlan p;
  p.version = (uint32_t)j.at("version").as_int();
  p.name = j.at("name").as_string();
  p.target = j.at("target").as_string();
  p.policy = j.at("policy").as_string();
  p.arena_bytes = (size_t)j.at("arena_bytes").as_int();
  if (auto v = j.find("folded_constants")) p.folded_constants = (size_t)v->as_int();
  if (auto v = j.find("eliminated_nodes")) p.eliminated_nodes = (size_t)v->as_int();
  for (auto& b : j.at("buffers").as_array()) {
    Buffer x;
    x.name = b.at("name").as_string();
    x.shape = shape_of(b.at("shape"));
    x.storage = parse_storage(b.at("storage").as_string());
    if (auto i = b.find("initial")) x.initial = floats_of(*i);
    if (auto o = b.find("offset")) { x.has_offset = true; x.offset = (size_t)o->as_int(); }
    if (auto l = b.find("lifetime")) { x.has_lifetime = true; x.first = (size_t)l->as_array().at(0).as_int(); x.last = (size_t)l->as_array().at(1).as_int(); }
    p.buffers.push_back(std::move(x));
  }
  for (auto& s : j.at("steps").as_array()) {
    Step x;
    x.name = s.at("name").as_string();
    x.kernel = parse_kernel(s.at("kernel").as_string());
    auto list = [](const Json& a) {
      std::vector<size_t> v;
      for (auto& e : a.as_array()) v.push_back((size_t)e.as_int());
      return v;
    };
    x.inputs = list(s.at("inputs"));
    x.output = (size_t)s.at("output").as_int();
    x.rank = (size_t)s.at("rank").as_int();
    x.stream = (size_t)s.at("stream").as_int();
    x.dependencies = list(s.at("dependencies"));
    x.reuse_dependencies = list(s.at("reuse_dependencies"));
    x.selection_reason = s.at("selection_reason").as_string();
    p.steps.push_back(std::move(x));
  }
  for (auto& o : j.at("outputs").as_array()) p.outputs.push_back((size_t)o.as_int());
  for (auto& kv : j.at("updates").as_object()) p.updates[(size_t)std::stoul(kv.first)] = (size_t)kv.second.as_int();
  return p;
}

PhysicalPlan tune(const PhysicalPlan& plan, const std::map<std::string, std::string>& overrides) {
  PhysicalPlan out = plan;
  std::map<std::string, size_t> by_name;
  for (size_t i = 0; i < out.steps.size(); ++i) by_name[out.steps[i].name] = i;
  static const Kernel kAll[] = {Kernel::AddF32V1, Kernel::MulF32V1, Kernel::ReluF32V1, Kernel::MatmulNaiveF32V1, Kernel::MatmulBlockedF32V1};
  for (auto& kv : overrides) {
    auto it = by_name.find(kv.first);
    if (it == by_name.end()) invalid("tune: the plan has no step named " + kv.first);
    const Kernel* chosen = nullptr;
    for (const Kernel& k : kAll)
      if (kv.second == kernel_name(k)) chosen = &k;
    if (!chosen) invalid("tune: unknown kernel " + kv.second);
    Step& s = out.steps[it->second];
    if (kernel_op(*chosen) != kernel_op(s.kernel))
      invalid("tune: " + kv.second + " does not implement the operation of step " + kv.first + " (" + op_name(kernel_op(s.kernel)) + ")");
    s.kernel = *chosen;
    s.selection_reason = "forced by override";
  }
  verify(out);
  return out;
}

std::string html_view(const PhysicalPlan& plan) {
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
  auto shape = [](const std::vector<size_t>& s) {
    std::string o = "[";
    for (size_t i = 0; i < s.size(); ++i) o += (i ? ", " : "") + std::to_string(s[i]);
    return o + "]";
  };
  std::string h = "<!doctype html><html><head><meta charset=\"utf-8\"><title>" + esc(plan.name) + " - " + esc(plan.target) +
                  "</title><style>body{font:13px monospace;margin:1.5em}table{border-collapse:collapse;margin:1em 0}td,th{border:1px solid #999;"
                  "padding:2px 8px;text-align:left}th{background:#eee}.bar{background:#48a;height:10px;display:inline-block}</style></head><body>";
  h += "<h1>" + esc(plan.name) + "</h1><p>target " + esc(plan.target) + ", policy " + esc(plan.policy) + ", " + std::to_string(plan.steps.size()) +
       " steps, arena " + std::to_string(plan.arena_bytes) + " bytes, " + std::to_string(plan.folded_constants) + " constants folded, " +
       std::to_string(plan.eliminated_nodes) + " nodes eliminated</p>";
  h += "<h2>Steps</h2><table id=\"steps\"><tr><th>#</th><th>name</th><th>kernel</th><th>inputs</th><th>output</th><th>depends on</th><th>reuse after</th><th>why</th></tr>";
  for (size_t i = 0; i < plan.steps.size(); ++i) {
    const Step& s = plan.steps[i];
    std::string in, dep, reuse;
    for (size_t b : s.inputs) in += (in.empty() ? "" : ", ") + esc(plan.buffers[b].name);
    for (size_t d : s.dependencies) dep += (dep.empty() ? "" : ", ") + std::to_string(d);
    for (size_t d : s.reuse_dependencies) reuse += (reuse.empty() ? "" : ", ") + std::to_string(d);
    h += "<tr><td>" + std::to_string(i) + "</td><td>" + esc(s.name) + "</td><td>" + kernel_name(s.kernel) + "</td><td>" + in + "</td><td>" +
         esc(plan.buffers[s.output].name) + "</td><td>" + dep + "</td><td>" + reuse + "</td><td>" + esc(s.selection_reason) + "</td></tr>";
  }
  h += "</table><h2>Buffers</h2><table id=\"buffers\"><tr><th>name</th><th>shape</th><th>storage</th><th>bytes</th><th>arena offset</th><th>live steps</th><th></th></tr>";
  const size_t n = std::max<size_t>(1, plan.steps.size());
  for (auto& b : plan.buffers) {
    const char* st = b.storage == Storage::Input ? "input" : b.storage == Storage::Constant ? "constant" : b.storage == Storage::State ? "state" : "temporary";
    std::string life, bar;
    if (b.has_lifetime) {
      life = std::to_string(b.first) + " - " + std::to_string(b.last);
      bar = "<span style=\"display:inline-block;width:" + std::to_string(200 * b.first / n) + "px\"></span><span class=\"bar\" style=\"width:" +
            std::to_string(std::max<size_t>(2, 200 * (std::min(b.last, n) - b.first + 1) / n)) + "px\"></span>";
    }
    h += "<tr><td>" + esc(b.name) + "</td><td>" + shape(b.shape) + "</td><td>" + st + "</td><td>" + std::to_string(b.bytes()) + "</td><td>" +
         (b.has_offset ? std::to_string(b.offset) : "") + "</td><td>" + life + "</td><td>" + bar + "</td></tr>";
  }
  h += "</table></body></html>\n";
  return h;
}

std::string encode_plan(const PhysicalPlan& p) {
  std::string body = p.to_json().dump();
  ByteWriter w;
  w.raw("IFPLAN01");
  w.u64(body.size());
  w.raw(Sha256::of(body));
  w.raw(body);
  return w.take();
}
PhysicalPlan decode_plan(std::string_view bytes) {
  ByteReader r(bytes);
  if (r.raw(8) != "IFPLAN01") invalid("not an IFPLAN01 file");
  uint64_t len = r.u64();
  std::string sha(r.raw(64));
  if (len != r.remaining()) invalid("IFPLAN01: length field does not match the file");
  std::string_view body = r.raw(len);
  if (Sha256::of(body) != sha) fail(ErrorKind::Stale, "IFPLAN01: integrity hash mismatch");
  PhysicalPlan p = PhysicalPlan::from_json(Json::parse(body));
  verify(p);
  return p;
}
Json manifest(std::string_view bytes) {
  ByteReader r(bytes);
  if (r.raw(8) != "IFPLAN01") invalid("not an IFPLAN01 file");
  Json j = Json::object();
  j.set("format", "IFPLAN01");
  j.set("body_bytes", r.u64());
  j.set("sha256", std::string(r.raw(64)));
  return j;
}

// ---------------------------------------------------------------------------------------------
Json RunReport::to_json() const {
  Json j = Json::object();
  Json o = Json::object();
  for (auto& kv : outputs) o.set(kv.first, floats_json(kv.second));
  j.set("outputs", o);
  j.set("steps", (int64_t)steps);
  j.set("arena_bytes", (int64_t)arena_bytes);
  Json k = Json::array();
  for (auto& s : kernels) k.push(s);
  j.set("kernels", k);
  return j;
}

Executor::Executor(PhysicalPlan plan) : plan_(std::move(plan)) {
  verify(plan_);
  arena_.assign((plan_.arena_bytes + 63) / 64 * 16, 0.f);
  for (size_t i = 0; i < plan_.buffers.size(); ++i) {
    const Buffer& b = plan_.buffers[i];
    if (b.storage == Storage::Constant || b.storage == Storage::State) resident_[i] = b.initial;
  }
}
void Executor::bind(const std::string& step_name, CompiledKernel k) {
  bool found = false;
  for (auto& s : plan_.steps) found |= s.name == step_name;
  if (!found) invalid("bind: no step named " + step_name);
  bound_[step_name] = std::move(k);
}
const std::vector<float>& Executor::state(const std::string& name) const {
  for (size_t i = 0; i < plan_.buffers.size(); ++i)
    if (plan_.buffers[i].name == name && plan_.buffers[i].storage == Storage::State) return resident_.at(i);
  invalid("no state named " + name);
}

RunReport Executor::run(const std::map<std::string, std::vector<float>>& inputs) {
  std::map<size_t, const std::vector<float>*> in_ptr;
  for (size_t i = 0; i < plan_.buffers.size(); ++i) {
    const Buffer& b = plan_.buffers[i];
    if (b.storage != Storage::Input) continue;
    auto it = inputs.find(b.name);
    if (it == inputs.end()) invalid("missing input " + b.name);
    if (it->second.size() != b.elements()) invalid("input " + b.name + " has the wrong number of elements");
    in_ptr[i] = &it->second;
  }
  for (auto& kv : inputs) {
    bool known = false;
    for (auto& b : plan_.buffers) known |= b.storage == Storage::Input && b.name == kv.first;
    if (!known) invalid("unknown input " + kv.first);
  }
  auto ptr = [&](size_t i) -> const float* {
    const Buffer& b = plan_.buffers[i];
    if (b.storage == Storage::Input) return in_ptr.at(i)->data();
    if (b.storage == Storage::Temporary) return arena_.data() + b.offset / 4;
    return resident_.at(i).data();
  };
  RunReport rep;
  for (auto& s : plan_.steps) {
    std::vector<const float*> ins;
    std::vector<std::vector<size_t>> shapes;
    for (size_t in : s.inputs) {
      ins.push_back(ptr(in));
      shapes.push_back(plan_.buffers[in].shape);
    }
    float* out = arena_.data() + plan_.buffers[s.output].offset / 4;
    auto b = bound_.find(s.name);
    if (b != bound_.end()) b->second(ins, shapes, out);
    else eval_kernel(s.kernel, ins, shapes, out);
    const size_t n = plan_.buffers[s.output].elements();
    for (size_t i = 0; i < n; ++i)
      if (!std::isfinite(out[i])) fail(ErrorKind::Backend, "step " + s.name + " produced a non-finite value");
    rep.kernels.push_back(kernel_name(s.kernel));
  }
  for (size_t o : plan_.outputs) {
    const Buffer& b = plan_.buffers[o];
    const float* p = ptr(o);
    rep.outputs[b.name] = std::vector<float>(p, p + b.elements());
  }
  // simultaneous state commit: read every new value before any state changes
  std::map<size_t, std::vector<float>> staged;
  for (auto& kv : plan_.updates) {
    const float* p = ptr(kv.second);
    staged[kv.first] = std::vector<float>(p, p + plan_.buffers[kv.second].elements());
  }
  for (auto& kv : staged) resident_[kv.first] = std::move(kv.second);
  rep.steps = plan_.steps.size();
  rep.arena_bytes = plan_.arena_bytes;
  return rep;
}

}  // namespace ifab::cpu
