#include "device_buffer.h"

#include <algorithm>
#include <map>
#include <set>

namespace ifab::device_buffer {

namespace {

bool power_of_two(uint64_t a) { return a != 0 && (a & (a - 1)) == 0; }

struct Range {
  uint64_t begin, end;
  bool overlaps(const Range& o) const { return begin < o.end && o.begin < end; }
};

Range range_in(uint64_t offset, uint64_t bytes, uint64_t capacity, const char* what) {
  if (bytes == 0 || offset > UINT64_MAX - bytes || offset + bytes > capacity) invalid(std::string(what) + " lies outside its allocation");
  return {offset, offset + bytes};
}

const char* class_name(MemoryClass c) {
  static const char* n[] = {"weight", "state", "activation", "workspace", "input", "output"};
  return n[(int)c];
}
MemoryClass class_of(const std::string& s) {
  static const char* n[] = {"weight", "state", "activation", "workspace", "input", "output"};
  for (int i = 0; i < 6; ++i)
    if (s == n[i]) return (MemoryClass)i;
  invalid("unknown memory class " + s);
}
const char* dtype_name(DType d) { return d == DType::I8 ? "i8" : d == DType::Bf16 ? "bf16" : "f32"; }
DType dtype_of(const std::string& s) {
  if (s == "i8") return DType::I8;
  if (s == "bf16") return DType::Bf16;
  if (s == "f32") return DType::F32;
  invalid("unknown dtype " + s);
}

Json u64s(const std::vector<uint64_t>& v) {
  Json a = Json::array();
  for (auto x : v) a.push((int64_t)x);
  return a;
}
std::vector<uint64_t> u64s_of(const Json& j) {
  std::vector<uint64_t> v;
  for (auto& x : j.as_array()) {
    if (!x.is_int() || x.as_int() < 0) invalid("expected a non-negative integer");
    v.push_back((uint64_t)x.as_int());
  }
  return v;
}
void only_fields(const Json& o, std::initializer_list<const char*> known, const char* what) {
  for (auto& kv : o.as_object())
    if (std::none_of(known.begin(), known.end(), [&](const char* k) { return kv.first == k; })) invalid(std::string(what) + ": unknown field " + kv.first);
}
Json view_json(const TensorView& v) {
  Json o = Json::object();
  o.set("allocation", v.allocation);
  o.set("offset", v.offset);
  o.set("dtype", dtype_name(v.dtype));
  o.set("shape", u64s(v.shape));
  o.set("strides", u64s(v.strides));
  o.set("alignment", v.alignment);
  o.set("access", v.access == Access::Read ? "read" : "write");
  return o;
}
TensorView view_of(const Json& o) {
  only_fields(o, {"allocation", "offset", "dtype", "shape", "strides", "alignment", "access"}, "tensor view");
  TensorView v;
  v.allocation = (uint32_t)o.at("allocation").as_int();
  v.offset = (uint64_t)o.at("offset").as_int();
  v.dtype = dtype_of(o.at("dtype").as_string());
  v.shape = u64s_of(o.at("shape"));
  v.strides = u64s_of(o.at("strides"));
  v.alignment = (uint64_t)o.at("alignment").as_int();
  const std::string& a = o.at("access").as_string();
  if (a != "read" && a != "write") invalid("access is read or write");
  v.access = a == "read" ? Access::Read : Access::Write;
  return v;
}

}  // namespace

uint64_t dtype_bytes(DType d) { return d == DType::I8 ? 1 : d == DType::Bf16 ? 2 : 4; }

uint64_t TensorView::byte_span() const {
  if (shape.empty() || shape.size() > 8 || strides.size() != shape.size()) invalid("a tensor view has 1..8 dimensions and one stride per dimension");
  uint64_t run = 1;
  for (size_t k = shape.size(); k-- > 0;) {
    if (shape[k] == 0 || shape[k] > (uint64_t)INT64_MAX || run > (uint64_t)INT64_MAX || strides[k] != run) invalid("the kernel ABI takes contiguous views with positive strides");
    if (run > UINT64_MAX / shape[k]) invalid("tensor shape overflows");
    run *= shape[k];
  }
  if (run > UINT64_MAX / dtype_bytes(dtype)) invalid("tensor size overflows");
  return run * dtype_bytes(dtype);
}

void Invocation::verify() const {
  const bool hex = binary_sha256.size() == 64 && std::all_of(binary_sha256.begin(), binary_sha256.end(), [](unsigned char c) { return isxdigit(c); });
  if (format != kFormat || implementation.empty() || numerical_contract.empty() || !hex) invalid("invocation: format, implementation, numerical contract and a 64-digit binary sha256 are required");
  if (allocations.empty() || allocations.size() > 4096 || inputs.empty() || outputs.empty() || inputs.size() > 64 || outputs.size() > 64) invalid("invocation: 1..4096 allocations and 1..64 inputs and outputs");
  std::map<uint32_t, const Allocation*> table;
  for (auto& a : allocations) {
    if (!table.emplace(a.id, &a).second) invalid("allocation id " + std::to_string(a.id) + " is listed twice");
    if (a.bytes == 0 || !power_of_two(a.alignment) || a.rank != rank || a.device != device) invalid("allocation " + std::to_string(a.id) + ": empty, misaligned or on another rank / device");
    if (a.cls == MemoryClass::Weight && !a.read_only) invalid("allocation " + std::to_string(a.id) + ": weights are read-only");
  }
  std::set<uint32_t> used;
  std::vector<std::pair<uint32_t, Range>> reads, writes;
  auto add_views = [&](const std::vector<TensorView>& views, Access access, std::vector<std::pair<uint32_t, Range>>& out) {
    for (auto& v : views) {
      auto it = table.find(v.allocation);
      if (it == table.end()) invalid("a tensor view names an allocation that is not listed");
      const Allocation& a = *it->second;
      if (v.access != access || (access == Access::Write && a.read_only)) invalid("a view's access does not fit its port or its allocation");
      if (!power_of_two(v.alignment) || v.alignment < dtype_bytes(v.dtype) || a.alignment < v.alignment || v.offset % v.alignment) invalid("a view is not aligned as it claims");
      out.emplace_back(v.allocation, range_in(v.offset, v.byte_span(), a.bytes, "a tensor view"));
      used.insert(v.allocation);
    }
  };
  add_views(inputs, Access::Read, reads);
  add_views(outputs, Access::Write, writes);
  for (size_t i = 0; i < writes.size(); ++i) {
    for (auto& r : reads)
      if (r.first == writes[i].first && r.second.overlaps(writes[i].second)) invalid("an output overlaps an input: the ABI forbids writable aliases");
    for (size_t k = 0; k < i; ++k)
      if (writes[k].first == writes[i].first && writes[k].second.overlaps(writes[i].second)) invalid("two outputs overlap");
  }
  if (workspace) {
    auto it = table.find(workspace->allocation);
    if (it == table.end()) invalid("the workspace names an allocation that is not listed");
    const Allocation& a = *it->second;
    if (a.read_only || !power_of_two(workspace->alignment) || workspace->alignment > 4096 || a.alignment < workspace->alignment || workspace->offset % workspace->alignment) invalid("workspace access or alignment");
    const Range w = range_in(workspace->offset, workspace->bytes, a.bytes, "the workspace");
    for (auto* set : {&reads, &writes})
      for (auto& r : *set)
        if (r.first == workspace->allocation && r.second.overlaps(w)) invalid("the workspace overlaps a tensor");
    used.insert(workspace->allocation);
  }
  if (used.size() != table.size()) invalid("an allocation is listed that no view uses");
}

void Invocation::verify_prepared(const std::string& sha, const std::string& contract, uint64_t ws_bytes, uint64_t ws_alignment) const {
  verify();
  if (sha != binary_sha256 || contract != numerical_contract || !power_of_two(ws_alignment) || ws_alignment > 4096) invalid("the prepared implementation is not the one the record froze (binary, numerical contract or workspace alignment)");
  if (workspace ? (ws_bytes > workspace->bytes || ws_alignment > workspace->alignment) : ws_bytes != 0) invalid("the prepared workspace exceeds the frozen one: plan again, explicitly");
}

Json Invocation::to_json() const {
  Json j = Json::object();
  j.set("format", format);
  j.set("implementation", implementation);
  j.set("binary_sha256", binary_sha256);
  j.set("numerical_contract", numerical_contract);
  j.set("rank", rank);
  j.set("device", device);
  j.set("stream", stream);
  Json as = Json::array();
  for (auto& a : allocations) {
    Json o = Json::object();
    o.set("id", a.id);
    o.set("rank", a.rank);
    o.set("device", a.device);
    o.set("bytes", a.bytes);
    o.set("alignment", a.alignment);
    o.set("class", class_name(a.cls));
    o.set("read_only", a.read_only);
    as.push(o);
  }
  j.set("allocations", as);
  Json in = Json::array(), out = Json::array();
  for (auto& v : inputs) in.push(view_json(v));
  for (auto& v : outputs) out.push(view_json(v));
  j.set("inputs", in);
  j.set("outputs", out);
  if (workspace) {
    Json w = Json::object();
    w.set("allocation", workspace->allocation);
    w.set("offset", workspace->offset);
    w.set("bytes", workspace->bytes);
    w.set("alignment", workspace->alignment);
    j.set("workspace", w);
  } else {
    j.set("workspace", Json());
  }
  return j;
}

Invocation Invocation::from_json(const Json& j) {
  only_fields(j, {"format", "implementation", "binary_sha256", "numerical_contract", "rank", "device", "stream", "allocations", "inputs", "outputs", "workspace"}, "invocation");
  Invocation c;
  c.format = j.at("format").as_string();
  c.implementation = j.at("implementation").as_string();
  c.binary_sha256 = j.at("binary_sha256").as_string();
  c.numerical_contract = j.at("numerical_contract").as_string();
  c.rank = (uint32_t)j.at("rank").as_int();
  c.device = (uint32_t)j.at("device").as_int();
  c.stream = (uint32_t)j.at("stream").as_int();
  for (auto& o : j.at("allocations").as_array()) {
    only_fields(o, {"id", "rank", "device", "bytes", "alignment", "class", "read_only"}, "allocation");
    Allocation a;
    a.id = (uint32_t)o.at("id").as_int();
    a.rank = (uint32_t)o.at("rank").as_int();
    a.device = (uint32_t)o.at("device").as_int();
    a.bytes = (uint64_t)o.at("bytes").as_int();
    a.alignment = (uint64_t)o.at("alignment").as_int();
    a.cls = class_of(o.at("class").as_string());
    a.read_only = o.at("read_only").as_bool();
    c.allocations.push_back(a);
  }
  for (auto& o : j.at("inputs").as_array()) c.inputs.push_back(view_of(o));
  for (auto& o : j.at("outputs").as_array()) c.outputs.push_back(view_of(o));
  if (auto w = j.find("workspace"); w && !w->is_null()) {
    only_fields(*w, {"allocation", "offset", "bytes", "alignment"}, "workspace");
    Workspace ws;
    ws.allocation = (uint32_t)w->at("allocation").as_int();
    ws.offset = (uint64_t)w->at("offset").as_int();
    ws.bytes = (uint64_t)w->at("bytes").as_int();
    ws.alignment = (uint64_t)w->at("alignment").as_int();
    c.workspace = ws;
  }
  return c;
}

Json support() {
  Json j = Json::object();
  j.set("format", kFormat);
  j.set("kernel_abi", "IFKernelTensorV1");
  Json d = Json::array();
  for (auto n : {"i8", "bf16", "f32"}) d.push(n);
  j.set("dtypes", d);
  j.set("layout", "contiguous, positive strides");
  j.set("alias_policy", "outputs and workspace overlap nothing; inputs may overlap inputs");
  j.set("max_tensor_rank", 8);
  Json checks = Json::array();
  for (auto n : {"allocation id", "rank and device", "capacity", "alignment", "byte ranges", "absolute address aliases", "binary identity", "prepared workspace bound"}) checks.push(n);
  j.set("binding_checks", checks);
  return j;
}

BoundInvocation bind(const Invocation& call, const std::vector<ResidentAllocation>& residents) {
  call.verify();
  if (residents.size() != call.allocations.size()) invalid("bind: one resident allocation per listed allocation");
  std::map<uint32_t, const ResidentAllocation*> table;
  for (auto& r : residents)
    if (!table.emplace(r.id, &r).second) invalid("bind: resident allocation " + std::to_string(r.id) + " is given twice");
  for (auto& a : call.allocations) {
    auto it = table.find(a.id);
    if (it == table.end()) invalid("bind: no resident allocation with id " + std::to_string(a.id));
    const ResidentAllocation& r = *it->second;
    const uint64_t addr = (uint64_t)(uintptr_t)r.base;
    if (r.base == nullptr || r.rank != a.rank || r.device != a.device || r.bytes < a.bytes || addr % a.alignment || addr > UINT64_MAX - r.bytes)
      invalid("bind: resident allocation " + std::to_string(a.id) + " is null, elsewhere, smaller than recorded or misaligned");
  }
  struct Abs {
    Range r;
    bool write;
  };
  std::vector<Abs> spans;
  BoundInvocation out;
  auto describe = [&](const TensorView& v) {
    const ResidentAllocation& r = *table[v.allocation];
    IFKernelTensorV1 t{};
    t.struct_bytes = sizeof(IFKernelTensorV1);
    t.dtype = (uint32_t)v.dtype;
    t.rank = (uint32_t)v.shape.size();
    t.access = (uint32_t)v.access;
    t.data = (char*)r.base + v.offset;
    t.allocation_bytes = r.bytes - v.offset;
    for (size_t k = 0; k < v.shape.size(); ++k) {
      t.shape[k] = (int64_t)v.shape[k];
      t.strides[k] = (int64_t)v.strides[k];
    }
    const uint64_t begin = (uint64_t)(uintptr_t)t.data;
    spans.push_back({{begin, begin + v.byte_span()}, v.access == Access::Write});
    return t;
  };
  for (auto& v : call.inputs) out.inputs.push_back(describe(v));
  for (auto& v : call.outputs) out.outputs.push_back(describe(v));
  if (call.workspace) {
    const ResidentAllocation& r = *table[call.workspace->allocation];
    out.workspace = (char*)r.base + call.workspace->offset;
    out.workspace_bytes = call.workspace->bytes;
    const uint64_t begin = (uint64_t)(uintptr_t)out.workspace;
    spans.push_back({{begin, begin + out.workspace_bytes}, true});
  }
  // two ids may name the same memory: whatever is written must be disjoint from everything else in absolute addresses too
  for (size_t i = 0; i < spans.size(); ++i)
    for (size_t k = i + 1; k < spans.size(); ++k)
      if ((spans[i].write || spans[k].write) && spans[i].r.overlaps(spans[k].r)) invalid("bind: a written range overlaps another range in device memory");
  return out;
}

}  // namespace ifab::device_buffer
