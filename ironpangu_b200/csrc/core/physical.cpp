#include "physical.h"

#include <algorithm>
#include <set>

namespace ifab::physical {

namespace {

const char* kReasonCost = "cheapest conservative bound among the eligible candidates; ties go to the lower id";
const char* kReasonBaseline = "lowest id among the eligible candidates: some cost is unknown, so no latency is compared";

void check_cost(const Cost& c) {
  if (c.source == CostSource::Unknown) {
    if (c.estimate_ns || c.upper_ns) invalid("a cost of unknown source carries numbers");
    return;
  }
  if (!c.estimate_ns || !c.upper_ns || c.evidence.empty() || *c.upper_ns < *c.estimate_ns) invalid("a cost needs an estimate, a bound not below it, and its evidence");
}

uint64_t host_peak(const std::vector<Value>& values, size_t n) {
  // values are defined in step order; sum the host-resident payloads that are alive after every definition
  std::vector<uint64_t> ends(n + 1, 0);
  uint64_t alive = 0, peak = 0;
  for (size_t i = 0; i < values.size(); ++i) {
    const uint64_t bytes = values[i].location == Location::Host ? values[i].payload_bytes.value_or(0) : 0;
    if (alive > UINT64_MAX - bytes) invalid("host payload overflows");
    alive += bytes;
    peak = std::max(peak, alive);
    ends[values[i].last] += bytes;
    if (ends[i] > alive) invalid("host payload lifetimes are inconsistent");
    alive -= ends[i];
  }
  return peak;
}

uint64_t unit_bytes(const std::string& dtype) {
  if (dtype == "i8" || dtype == "u8" || dtype == "fp8_e4m3") return 1;
  if (dtype == "bf16" || dtype == "f16") return 2;
  if (dtype == "f32" || dtype == "i32") return 4;
  if (dtype == "f64" || dtype == "i64") return 8;
  invalid("a value with a known payload needs a concrete dtype (got '" + dtype + "')");
}

std::optional<uint64_t> add_cost(std::optional<uint64_t> sum, std::optional<uint64_t> x) {
  if (!sum || !x) return std::nullopt;
  if (*sum > UINT64_MAX - *x) invalid("schedule cost overflows");
  return *sum + *x;
}

std::vector<size_t> previous_step(size_t i) { return i > 0 ? std::vector<size_t>{i - 1} : std::vector<size_t>{}; }

template <typename E>
const char* name_of(E e, std::initializer_list<const char*> names) { return *(names.begin() + (int)e); }
#define COST_NAMES {"unknown", "analytical", "measured", "interpolated"}
#define LOC_NAMES {"host", "device", "opaque"}
#define BOUNDARY_NAMES {"host_to_device", "device_to_host", "control_upload", "parameter_upload", "parameter_readback", "request_output", "synchronize", "dynamic_allocation", "internal_launches", "persistent_state"}

template <typename E>
E parse_enum(const std::string& s, std::initializer_list<const char*> names, const char* what) {
  int i = 0;
  for (auto n : names) {
    if (s == n) return (E)i;
    ++i;
  }
  invalid(std::string("unknown ") + what + " '" + s + "'");
}

Json opt_json(const std::optional<uint64_t>& v) { return v ? Json(*v) : Json(); }
std::optional<uint64_t> opt_of(const Json* j) {
  if (!j || j->is_null()) return std::nullopt;
  if (!j->is_int() || j->as_int() < 0) invalid("expected a non-negative integer or null");
  return (uint64_t)j->as_int();
}
Json sizes_json(const std::vector<size_t>& v) {
  Json a = Json::array();
  for (auto x : v) a.push((int64_t)x);
  return a;
}
std::vector<size_t> sizes_of(const Json& j) {
  std::vector<size_t> v;
  for (auto& x : j.as_array()) {
    if (!x.is_int() || x.as_int() < 0) invalid("expected an index");
    v.push_back((size_t)x.as_int());
  }
  return v;
}
void only_fields(const Json& o, std::initializer_list<const char*> known, const char* what) {
  for (auto& kv : o.as_object())
    if (std::none_of(known.begin(), known.end(), [&](const char* k) { return kv.first == k; })) invalid(std::string(what) + ": unknown field " + kv.first);
}

}  // namespace

Choice choose(const std::vector<Candidate>& candidates) {
  if (candidates.empty()) invalid("an operation needs at least one implementation candidate");
  std::set<std::string> ids;
  for (auto& c : candidates) {
    // residency is an admission rule, applied before any cost: not even a rejected host implementation may be listed
    bool crosses = c.location != Location::Device;
    for (auto& b : c.boundaries) crosses |= b.kind == BoundaryKind::HostToDevice || b.kind == BoundaryKind::DeviceToHost;
    if (crosses) invalid("candidate " + c.id + " leaves the device: activations never fall back to the host");
    check_cost(c.cost);
    if (c.id.empty() || !ids.insert(c.id).second || c.contract_revision.empty() || c.numerical_contract.empty()) invalid("a candidate needs a unique id, a contract revision and a numerical contract");
    if (c.eligible != c.rejection.empty()) invalid("candidate " + c.id + ": an ineligible candidate says why, an eligible one says nothing");
  }
  std::vector<size_t> legal;
  for (size_t i = 0; i < candidates.size(); ++i)
    if (candidates[i].eligible) legal.push_back(i);
  if (legal.empty()) invalid("no candidate is eligible");
  bool complete = true;
  for (size_t i : legal) {
    if (candidates[i].numerical_contract != candidates[legal[0]].numerical_contract) invalid("candidates of one operation differ in their numerical contract");
    complete &= candidates[i].cost.upper_ns.has_value();
  }
  std::sort(legal.begin(), legal.end(), [&](size_t a, size_t b) {
    const Candidate &x = candidates[a], &y = candidates[b];
    if (complete && *x.cost.upper_ns != *y.cost.upper_ns) return *x.cost.upper_ns < *y.cost.upper_ns;
    return x.id < y.id;
  });
  return {legal[0], complete ? kReasonCost : kReasonBaseline};
}

Plan serial_plan(std::string name, std::string target, std::string logical_digest, const std::vector<uint32_t>& devices,
                 std::vector<Operation> operations, std::vector<Value> values, std::vector<size_t> outputs) {
  const size_t n = operations.size();
  if (n == 0 || n > 10000 || values.size() != n || devices.empty() || devices.size() > 256 || outputs.empty()) invalid("physical graph out of bounds (1..10000 operations, one value each, 1..256 devices, at least one output)");
  for (auto o : outputs)
    if (o >= n) invalid("an output names no operation");
  for (size_t i = 0; i < n; ++i) {
    if (values[i].location != Location::Device) invalid("every value of a device-resident plan lives on the device");
    values[i].first = values[i].last = i;
    values[i].arena_offset.reset();
  }
  Plan p;
  p.name = std::move(name);
  p.target = std::move(target);
  p.logical_digest = std::move(logical_digest);
  p.devices = devices;
  std::optional<uint64_t> sum = 0;
  for (size_t i = 0; i < n; ++i) {
    Operation& op = operations[i];
    for (auto j : op.inputs) {
      if (j >= i) invalid("operation " + op.name + " reads a later operation");
      values[j].last = i;
    }
    const Choice c = choose(op.candidates);
    sum = add_cost(sum, op.candidates[c.index].cost.estimate_ns);
    Step s;
    s.id = i;
    s.selected = c.index;
    s.selection_reason = c.reason;
    s.data_dependencies = op.inputs;
    s.order_dependencies = previous_step(i);
    s.operation = std::move(op);
    p.schedule.steps.push_back(std::move(s));
  }
  for (auto o : outputs) values[o].last = n;
  p.schedule.known_host_payload_peak_bytes = host_peak(values, n);
  p.schedule.values = std::move(values);
  p.schedule.outputs = std::move(outputs);
  p.schedule.activation_policy = "activations stay on the device; no host fallback; no arena reuse and no complete device budget is claimed here";
  p.schedule.cost_complete = sum.has_value();
  p.schedule.estimated_serial_ns = sum;
  p.limitations = {"inspection plan: the executor runs the token program, not this plan",
                   "kernel internals are opaque: boundary notes are not separately executable launches",
                   "workspace, temporaries and persistent-state sizes are settled when the backend prepares the program",
                   "costs are models or samples as their evidence says; overlap between steps is not modelled"};
  verify(p);
  return p;
}

void verify(const Plan& p) {
  if (p.format != kFormat || p.executable || p.policy != kPolicy || p.devices.empty() || p.devices.size() > 256 || p.logical_digest.empty()) invalid("not a serial device-resident inspection plan");
  std::set<uint32_t> devs(p.devices.begin(), p.devices.end());
  if (devs.size() != p.devices.size()) invalid("two ranks share a device");
  const Schedule& s = p.schedule;
  const size_t n = s.steps.size();
  if (n == 0 || n > 10000 || s.values.size() != n || s.outputs.empty() || s.memory_complete) invalid("physical schedule out of bounds");
  for (auto o : s.outputs)
    if (o >= n) invalid("an output names no step");
  std::vector<size_t> ends(n);
  for (size_t i = 0; i < n; ++i) ends[i] = i;
  size_t sequence = 0;
  std::optional<uint64_t> sum = 0;
  std::set<size_t> origins;
  for (size_t i = 0; i < n; ++i) {
    const Step& st = s.steps[i];
    const Operation& op = st.operation;
    if (st.id != i || st.stream != 0 || st.data_dependencies != op.inputs || st.order_dependencies != previous_step(i) || !st.reuse_dependencies.empty()) invalid("step " + std::to_string(i) + ": dependencies are not those of a serial plan");
    if (op.logical_nodes.empty()) invalid("step " + std::to_string(i) + " has no logical origin");
    for (auto j : op.logical_nodes)
      if (!origins.insert(j).second) invalid("logical node " + std::to_string(j) + " is claimed by two steps");
    for (auto j : op.inputs) {
      if (j >= i) invalid("step " + std::to_string(i) + " reads a later step");
      ends[j] = i;
    }
    const Choice c = choose(op.candidates);
    if (c.index != st.selected || c.reason != st.selection_reason) invalid("step " + std::to_string(i) + ": the recorded selection is not what the candidates imply");
    sum = add_cost(sum, op.candidates[c.index].cost.estimate_ns);
    if (op.collective) {
      const Collective& k = *op.collective;
      if (k.group != "all_ranks" || k.sequence != sequence || k.operation.empty() || k.dtype.empty() || k.elements_per_rank == 0) invalid("step " + std::to_string(i) + ": collective order or signature");
      ++sequence;
    }
  }
  for (auto o : s.outputs) ends[o] = n;
  for (size_t i = 0; i < n; ++i) {
    const Value& v = s.values[i];
    const auto& origin = s.steps[i].operation.logical_nodes;
    if (v.location != Location::Device || v.first != i || v.last != ends[i] || v.arena_offset || std::find(origin.begin(), origin.end(), v.logical_node) == origin.end()) invalid("value " + std::to_string(i) + ": lifetime, placement or origin is not what the steps imply");
    if (v.alignment && (*v.alignment == 0 || (*v.alignment & (*v.alignment - 1)))) invalid("value " + std::to_string(i) + ": alignment is not a power of two");
    if (v.payload_bytes) {
      uint64_t size = unit_bytes(v.dtype);
      if (v.shape.empty() || v.shape.size() > 8) invalid("value " + std::to_string(i) + ": a sized value has 1..8 dimensions");
      for (auto d : v.shape) {
        if (d == 0 || size > UINT64_MAX / d) invalid("value " + std::to_string(i) + ": shape is empty or overflows");
        size *= d;
      }
      if (size != *v.payload_bytes) invalid("value " + std::to_string(i) + ": payload bytes do not match dtype and shape");
    }
  }
  if (s.known_host_payload_peak_bytes != host_peak(s.values, n) || s.estimated_serial_ns != sum || s.cost_complete != sum.has_value()) invalid("the schedule's summary does not match its steps");
}

Json Plan::to_json() const {
  Json j = Json::object();
  j.set("format", format);
  j.set("name", name);
  j.set("target", target);
  j.set("logical_digest", logical_digest);
  j.set("policy", policy);
  j.set("executable", executable);
  Json ranks = Json::array(), all = Json::array();
  for (size_t i = 0; i < devices.size(); ++i) {
    Json r = Json::object();
    r.set("rank", (int64_t)i);
    r.set("device", devices[i]);
    r.set("schedule", 0);
    ranks.push(r);
    all.push((int64_t)i);
  }
  j.set("ranks", ranks);
  Json g = Json::object();
  g.set("id", "all_ranks");
  g.set("ranks", all);
  Json groups = Json::array();
  groups.push(g);
  j.set("groups", groups);
  Json s = Json::object();
  s.set("id", 0);
  Json steps = Json::array();
  for (auto& st : schedule.steps) {
    Json o = Json::object(), op = Json::object();
    o.set("id", (int64_t)st.id);
    op.set("name", st.operation.name);
    op.set("logical_nodes", sizes_json(st.operation.logical_nodes));
    op.set("inputs", sizes_json(st.operation.inputs));
    Json cs = Json::array();
    for (auto& c : st.operation.candidates) {
      Json k = Json::object();
      k.set("id", c.id);
      k.set("contract_revision", c.contract_revision);
      k.set("numerical_contract", c.numerical_contract);
      k.set("location", name_of(c.location, LOC_NAMES));
      k.set("eligible", c.eligible);
      k.set("rejection", c.rejection.empty() ? Json() : Json(c.rejection));
      k.set("workspace_bound_bytes", opt_json(c.workspace_bound_bytes));
      k.set("capture_qualified", c.capture_qualified);
      Json bs = Json::array();
      for (auto& b : c.boundaries) {
        Json bo = Json::object();
        bo.set("kind", name_of(b.kind, BOUNDARY_NAMES));
        bo.set("detail", b.detail);
        bs.push(bo);
      }
      k.set("boundaries", bs);
      Json un = Json::array();
      for (auto& u : c.unresolved) un.push(u);
      k.set("unresolved", un);
      Json cost = Json::object();
      cost.set("source", name_of(c.cost.source, COST_NAMES));
      cost.set("estimate_ns", opt_json(c.cost.estimate_ns));
      cost.set("upper_ns", opt_json(c.cost.upper_ns));
      cost.set("evidence", c.cost.evidence.empty() ? Json() : Json(c.cost.evidence));
      k.set("cost", cost);
      cs.push(k);
    }
    op.set("candidates", cs);
    if (st.operation.collective) {
      const Collective& c = *st.operation.collective;
      Json k = Json::object();
      k.set("group", c.group);
      k.set("operation", c.operation);
      k.set("dtype", c.dtype);
      k.set("elements_per_rank", c.elements_per_rank);
      k.set("sequence", (int64_t)c.sequence);
      op.set("collective", k);
    } else {
      op.set("collective", Json());
    }
    o.set("operation", op);
    o.set("selected", (int64_t)st.selected);
    o.set("selection_reason", st.selection_reason);
    o.set("stream", (int64_t)st.stream);
    o.set("data_dependencies", sizes_json(st.data_dependencies));
    o.set("order_dependencies", sizes_json(st.order_dependencies));
    o.set("reuse_dependencies", sizes_json(st.reuse_dependencies));
    steps.push(o);
  }
  s.set("steps", steps);
  Json vals = Json::array();
  for (auto& v : schedule.values) {
    Json o = Json::object();
    o.set("logical_node", (int64_t)v.logical_node);
    o.set("dtype", v.dtype.empty() ? Json() : Json(v.dtype));
    Json sh = Json::array();
    for (auto d : v.shape) sh.push((int64_t)d);
    o.set("shape", sh);
    o.set("layout", v.layout);
    o.set("location", name_of(v.location, LOC_NAMES));
    o.set("payload_bytes", opt_json(v.payload_bytes));
    o.set("alignment", opt_json(v.alignment));
    o.set("arena_offset", opt_json(v.arena_offset));
    Json lt = Json::array();
    lt.push((int64_t)v.first);
    lt.push((int64_t)v.last);
    o.set("lifetime", lt);
    vals.push(o);
  }
  s.set("values", vals);
  s.set("outputs", sizes_json(schedule.outputs));
  s.set("known_host_payload_peak_bytes", schedule.known_host_payload_peak_bytes);
  s.set("memory_complete", schedule.memory_complete);
  s.set("activation_policy", schedule.activation_policy);
  s.set("cost_complete", schedule.cost_complete);
  s.set("estimated_serial_ns", opt_json(schedule.estimated_serial_ns));
  Json scheds = Json::array();
  scheds.push(s);
  j.set("schedules", scheds);
  Json lim = Json::array();
  for (auto& l : limitations) lim.push(l);
  j.set("limitations", lim);
  return j;
}

Plan Plan::from_json(const Json& j) {
  only_fields(j, {"format", "name", "target", "logical_digest", "policy", "executable", "ranks", "groups", "schedules", "limitations"}, "physical plan");
  Plan p;
  p.format = j.at("format").as_string();
  p.name = j.at("name").as_string();
  p.target = j.at("target").as_string();
  p.logical_digest = j.at("logical_digest").as_string();
  p.policy = j.at("policy").as_string();
  p.executable = j.at("executable").as_bool();
  const JsonArray& ranks = j.at("ranks").as_array();
  for (size_t i = 0; i < ranks.size(); ++i) {
    if ((size_t)ranks[i].at("rank").as_int() != i || ranks[i].at("schedule").as_int() != 0) invalid("rank bindings must be dense and share schedule 0");
    p.devices.push_back((uint32_t)ranks[i].at("device").as_int());
  }
  const JsonArray& groups = j.at("groups").as_array();
  if (groups.size() != 1 || groups[0].at("id").as_string() != "all_ranks" || sizes_of(groups[0].at("ranks")).size() != ranks.size()) invalid("the one collective group is all_ranks");
  const JsonArray& scheds = j.at("schedules").as_array();
  if (scheds.size() != 1 || scheds[0].at("id").as_int() != 0) invalid("a serial plan has exactly one schedule");
  const Json& s = scheds[0];
  for (auto& o : s.at("steps").as_array()) {
    Step st;
    st.id = (size_t)o.at("id").as_int();
    const Json& op = o.at("operation");
    st.operation.name = op.at("name").as_string();
    st.operation.logical_nodes = sizes_of(op.at("logical_nodes"));
    st.operation.inputs = sizes_of(op.at("inputs"));
    for (auto& k : op.at("candidates").as_array()) {
      only_fields(k, {"id", "contract_revision", "numerical_contract", "location", "eligible", "rejection", "workspace_bound_bytes", "capture_qualified", "boundaries", "unresolved", "cost"}, "candidate");
      Candidate c;
      c.id = k.at("id").as_string();
      c.contract_revision = k.at("contract_revision").as_string();
      c.numerical_contract = k.at("numerical_contract").as_string();
      c.location = parse_enum<Location>(k.at("location").as_string(), LOC_NAMES, "location");
      c.eligible = k.at("eligible").as_bool();
      if (auto r = k.find("rejection"); r && !r->is_null()) c.rejection = r->as_string();
      c.workspace_bound_bytes = opt_of(k.find("workspace_bound_bytes"));
      c.capture_qualified = k.at("capture_qualified").as_bool();
      for (auto& b : k.at("boundaries").as_array()) c.boundaries.push_back({parse_enum<BoundaryKind>(b.at("kind").as_string(), BOUNDARY_NAMES, "boundary kind"), b.at("detail").as_string()});
      for (auto& u : k.at("unresolved").as_array()) c.unresolved.push_back(u.as_string());
      const Json& cost = k.at("cost");
      c.cost.source = parse_enum<CostSource>(cost.at("source").as_string(), COST_NAMES, "cost source");
      c.cost.estimate_ns = opt_of(cost.find("estimate_ns"));
      c.cost.upper_ns = opt_of(cost.find("upper_ns"));
      if (auto e = cost.find("evidence"); e && !e->is_null()) c.cost.evidence = e->as_string();
      st.operation.candidates.push_back(std::move(c));
    }
    if (auto k = op.find("collective"); k && !k->is_null()) {
      Collective c;
      c.group = k->at("group").as_string();
      c.operation = k->at("operation").as_string();
      c.dtype = k->at("dtype").as_string();
      c.elements_per_rank = (uint64_t)k->at("elements_per_rank").as_int();
      c.sequence = (size_t)k->at("sequence").as_int();
      st.operation.collective = c;
    }
    st.selected = (size_t)o.at("selected").as_int();
    st.selection_reason = o.at("selection_reason").as_string();
    st.stream = (size_t)o.at("stream").as_int();
    st.data_dependencies = sizes_of(o.at("data_dependencies"));
    st.order_dependencies = sizes_of(o.at("order_dependencies"));
    st.reuse_dependencies = sizes_of(o.at("reuse_dependencies"));
    p.schedule.steps.push_back(std::move(st));
  }
  for (auto& o : s.at("values").as_array()) {
    Value v;
    v.logical_node = (size_t)o.at("logical_node").as_int();
    if (auto d = o.find("dtype"); d && !d->is_null()) v.dtype = d->as_string();
    for (auto& d : o.at("shape").as_array()) v.shape.push_back((uint64_t)d.as_int());
    v.layout = o.at("layout").as_string();
    v.location = parse_enum<Location>(o.at("location").as_string(), LOC_NAMES, "location");
    v.payload_bytes = opt_of(o.find("payload_bytes"));
    v.alignment = opt_of(o.find("alignment"));
    v.arena_offset = opt_of(o.find("arena_offset"));
    const std::vector<size_t> lt = sizes_of(o.at("lifetime"));
    if (lt.size() != 2) invalid("a lifetime is [first, last]");
    v.first = lt[0];
    v.last = lt[1];
    p.schedule.values.push_back(std::move(v));
  }
  p.schedule.outputs = sizes_of(s.at("outputs"));
  p.schedule.known_host_payload_peak_bytes = (uint64_t)s.at("known_host_payload_peak_bytes").as_int();
  p.schedule.memory_complete = s.at("memory_complete").as_bool();
  p.schedule.activation_policy = s.at("activation_policy").as_string();
  p.schedule.cost_complete = s.at("cost_complete").as_bool();
  p.schedule.estimated_serial_ns = opt_of(s.find("estimated_serial_ns"));
  for (auto& l : j.at("limitations").as_array()) p.limitations.push_back(l.as_string());
  return p;
}

}  // namespace ifab::physical
