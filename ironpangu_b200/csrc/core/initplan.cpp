#include "initplan.h"

#include <algorithm>
#include <cstring>
#include <filesystem>
#include <fstream>

namespace ifab::init {

using program::Instruction;
using program::Program;

size_t dtype_bytes(DType d) {
  switch (d) {
    case DType::I8: return 1;
    case DType::F8E4M3: return 1;
    case DType::Bf16: return 2;
    case DType::F32: return 4;
  }
  return 0;
}
const char* dtype_name(DType d) {
  switch (d) {
    case DType::I8: return "int8";
    case DType::F8E4M3: return "fp8_e4m3";
    case DType::Bf16: return "bf16";
    case DType::F32: return "f32";
  }
  return "?";
}
uint64_t Parameter::bytes() const {
  uint64_t n = dtype_bytes(dtype);
  for (auto d : dims) n *= d;
  return n;
}
uint64_t Plan::device_bytes() const {
  uint64_t n = 0;
  for (auto& p : parameters) n += (p.bytes() + 255) / 256 * 256;
  return n;
}

// ---------------------------------------------------------------------------------------------
bool Plan::reference_form() const {
  if (loads.size() != parameters.size()) return false;
  for (size_t i = 0; i < loads.size(); ++i)
    if (loads[i].dest != i || (uint32_t)loads[i].src_dtype > 3 || (uint32_t)parameters[i].dtype > 3) return false;
  return true;
}

std::string Plan::encode() const {
  ByteWriter w;
  w.raw(reference_form() ? "IFINIT01" : "IFINIT02");
  w.u32(rank);
  w.u32(device);
  w.str(provenance);
  w.u32((uint32_t)parameters.size());
  for (auto& p : parameters) {
    w.u32(p.id);
    w.str(p.name);
    w.u32((uint32_t)p.dtype);
    w.u32((uint32_t)p.dims.size());
    for (auto d : p.dims) w.u64(d);
  }
  w.u32((uint32_t)loads.size());
  for (auto& l : loads) {
    w.u32(l.tag);
    w.u32(l.dest);
    w.str(l.shard);
    w.u64(l.offset);
    w.u64(l.bytes);
    w.u32((uint32_t)l.src_dtype);
    if (l.tag == 2) {
      w.u64(l.row_bytes);
      w.u64(l.stride_bytes);
    }
  }
  return w.take();
}

Plan Plan::decode(std::string_view bytes) {
  ByteReader r(bytes);
  const std::string magic(r.raw(8));
  if (magic != "IFINIT01" && magic != "IFINIT02") invalid("not an initialization plan (IFINIT01 / IFINIT02)");
  const bool extended = magic == "IFINIT02";
  Plan p;
  p.rank = r.u32();
  p.device = r.u32();
  p.provenance = r.str(128);
  uint32_t np = r.u32();
  if (np > 200000) fail(ErrorKind::Capacity, "too many parameters");
  for (uint32_t i = 0; i < np; ++i) {
    Parameter q;
    q.id = r.u32();
    if (q.id != i) invalid("parameter ids must be dense and ordered");
    q.name = r.str(4096);
    uint32_t dt = r.u32();
    if (dt < 1 || dt > (extended ? 4u : 3u)) invalid("unknown parameter dtype");
    q.dtype = (DType)dt;
    uint32_t rank = r.u32();
    if (rank == 0 || rank > 6) invalid("parameter rank out of range");
    for (uint32_t k = 0; k < rank; ++k) {
      uint64_t d = r.u64();
      if (d == 0 || d > ((uint64_t)1 << 40)) invalid("parameter dimension out of range");
      q.dims.push_back(d);
    }
    p.parameters.push_back(std::move(q));
  }
  uint32_t nl = r.u32();
  if (nl > 2000000) fail(ErrorKind::Capacity, "too many load instructions");
  for (uint32_t i = 0; i < nl; ++i) {
    LoadSlice l;
    l.tag = r.u32();
    if (l.tag != 1 && l.tag != 2) invalid("unknown load tag");
    l.dest = r.u32();
    if (l.dest >= np) invalid("load destination out of range");
    l.shard = r.str(4096);
    if (l.shard.empty() || l.shard.find('/') != std::string::npos || l.shard.find("..") != std::string::npos) invalid("load names a shard outside the checkpoint directory");
    l.offset = r.u64();
    l.bytes = r.u64();
    uint32_t dt = r.u32();
    if (dt < 1 || dt > (extended ? 4u : 3u)) invalid("unknown source dtype");
    l.src_dtype = (DType)dt;
    if (l.tag == 2) {
      l.row_bytes = r.u64();
      l.stride_bytes = r.u64();
      if (l.row_bytes == 0 || l.stride_bytes < l.row_bytes || l.bytes % l.row_bytes) invalid("malformed strided load");
    }
    p.loads.push_back(std::move(l));
  }
  if (!r.done()) invalid("trailing bytes after the plan");
  if (!extended && !p.reference_form()) invalid("an IFINIT01 plan carries exactly one load per parameter, in parameter order");
  return p;
}

Json Plan::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.initialization.v1");
  j.set("rank", rank);
  j.set("device", device);
  j.set("provenance", provenance);
  j.set("device_bytes", device_bytes());
  Json ps = Json::array();
  for (auto& p : parameters) {
    Json o = Json::object();
    o.set("id", p.id);
    o.set("name", p.name);
    o.set("dtype", dtype_name(p.dtype));
    Json d = Json::array();
    for (auto x : p.dims) d.push((int64_t)x);
    o.set("dims", d);
    ps.push(o);
  }
  j.set("parameters", ps);
  Json ls = Json::array();
  for (auto& l : loads) {
    Json o = Json::object();
    o.set("kind", l.tag == 1 ? "slice" : "strided_rows");
    o.set("dest", l.dest);
    o.set("shard", l.shard);
    o.set("offset", l.offset);
    if (!l.tensor.empty()) o.set("tensor", l.tensor);
    o.set("bytes", l.bytes);
    o.set("src_dtype", dtype_name(l.src_dtype));
    if (l.tag == 2) {
      o.set("row_bytes", l.row_bytes);
      o.set("stride_bytes", l.stride_bytes);
    }
    ls.push(o);
  }
  j.set("loads", ls);
  return j;
}

// ---------------------------------------------------------------------------------------------
// safetensors
// ---------------------------------------------------------------------------------------------
namespace {
DType parse_st_dtype(const std::string& s, const std::string& where) {
  if (s == "BF16") return DType::Bf16;
  if (s == "F32") return DType::F32;
  if (s == "I8") return DType::I8;
  if (s == "F8_E4M3") return DType::F8E4M3;
  invalid(where + ": unsupported safetensors dtype " + s);
}
const char* st_dtype(DType d) {
  switch (d) {
    case DType::Bf16: return "BF16";
    case DType::F32: return "F32";
    case DType::I8: return "I8";
    case DType::F8E4M3: return "F8_E4M3";
  }
  return "?";
}
}  // namespace

Checkpoint Checkpoint::inspect(const std::string& dir) {
  namespace fs = std::filesystem;
  Checkpoint c;
  c.dir = dir;
  std::error_code ec;
  if (!fs::is_directory(dir, ec)) fail(ErrorKind::Io, dir + " is not a directory");
  std::vector<std::string> files;
  for (auto& e : fs::directory_iterator(dir, ec))
    if (e.path().extension() == ".safetensors") files.push_back(e.path().filename().string());
  std::sort(files.begin(), files.end());
  if (files.empty()) fail(ErrorKind::Io, "no .safetensors files under " + dir);
  for (auto& f : files) {
    std::string path = dir + "/" + f;
    std::ifstream in(path, std::ios::binary);
    if (!in) fail(ErrorKind::Io, "cannot open " + path);
    uint8_t lenb[8];
    in.read((char*)lenb, 8);
    if (!in) invalid(path + ": truncated header length");
    uint64_t hlen = 0;
    for (int i = 0; i < 8; ++i) hlen |= (uint64_t)lenb[i] << (8 * i);
    uint64_t fsize = fs::file_size(path, ec);
    if (hlen < 2 || hlen > (100u << 20) || 8 + hlen > fsize) invalid(path + ": header length out of bounds");
    std::string hdr(hlen, '\0');
    in.read(hdr.data(), (std::streamsize)hlen);
    if (!in) invalid(path + ": truncated header");
    Json j = Json::parse(hdr, 100u << 20);
    const uint64_t data_bytes = fsize - 8 - hlen;
    std::vector<std::pair<uint64_t, uint64_t>> ranges;
    for (auto& kv : j.as_object()) {
      if (kv.first == "__metadata__") continue;
      TensorInfo t;
      t.name = kv.first;
      t.file = f;
      t.dtype = parse_st_dtype(kv.second.at("dtype").as_string(), path + ":" + t.name);
      uint64_t n = dtype_bytes(t.dtype);
      for (auto& d : kv.second.at("shape").as_array()) {
        int64_t x = d.as_int();
        if (x <= 0) invalid(path + ":" + t.name + ": non-positive dimension");
        t.shape.push_back((uint64_t)x);
        if (n > ((uint64_t)1 << 50) / (uint64_t)x) invalid(path + ":" + t.name + ": size overflow");
        n *= (uint64_t)x;
      }
      auto& off = kv.second.at("data_offsets").as_array();
      if (off.size() != 2) invalid(path + ":" + t.name + ": data_offsets must have two entries");
      t.begin = (uint64_t)off[0].as_int();
      t.end = (uint64_t)off[1].as_int();
      if (t.end < t.begin || t.end > data_bytes || t.end - t.begin != n) invalid(path + ":" + t.name + ": data range does not match shape");
      t.data_start = 8 + hlen;
      ranges.emplace_back(t.begin, t.end);
      if (!c.tensors.emplace(t.name, t).second) invalid("tensor " + t.name + " appears in more than one shard");
    }
    std::sort(ranges.begin(), ranges.end());
    for (size_t i = 1; i < ranges.size(); ++i)
      if (ranges[i].first < ranges[i - 1].second) invalid(path + ": overlapping tensor ranges");
  }
  Sha256 h;
  for (auto& kv : c.tensors) {
    std::string line = kv.first + ":" + dtype_name(kv.second.dtype);
    for (auto d : kv.second.shape) line += "," + std::to_string(d);
    line += "\n";
    h.update(line.data(), line.size());
  }
  c.fingerprint = h.hex();
  return c;
}

Checkpoint Checkpoint::synthetic(const std::map<std::string, std::pair<DType, std::vector<uint64_t>>>& shapes) {
  Checkpoint c;
  Sha256 h;
  uint64_t cursor = 0;
  for (auto& kv : shapes) {
    TensorInfo t;
    t.name = kv.first;
    t.dtype = kv.second.first;
    t.shape = kv.second.second;
    // a virtual single shard, tensors back to back in name order after an 8-byte-aligned header stand-in
    t.file = "model.safetensors";
    t.data_start = 0;
    t.begin = cursor;
    uint64_t n = dtype_bytes(t.dtype);
    for (auto d : t.shape) n *= d;
    t.end = t.begin + n;
    cursor = t.end;
    c.tensors[t.name] = t;
    std::string line = kv.first + ":" + dtype_name(t.dtype);
    for (auto d : t.shape) line += "," + std::to_string(d);
    line += "\n";
    h.update(line.data(), line.size());
  }
  c.fingerprint = h.hex();
  return c;
}

const TensorInfo& Checkpoint::need(const std::string& name) const {
  auto it = tensors.find(name);
  if (it == tensors.end()) invalid("checkpoint has no tensor " + name);
  return it->second;
}

void write_safetensors(const std::string& path, const std::vector<std::pair<TensorInfo, std::string>>& tensors) {
  Json hdr = Json::object();
  uint64_t cursor = 0;
  for (auto& t : tensors) {
    Json o = Json::object();
    o.set("dtype", st_dtype(t.first.dtype));
    Json shp = Json::array();
    for (auto d : t.first.shape) shp.push((int64_t)d);
    o.set("shape", shp);
    Json off = Json::array();
    off.push((int64_t)cursor);
    cursor += t.second.size();
    off.push((int64_t)cursor);
    o.set("data_offsets", off);
    hdr.set(t.first.name, o);
  }
  std::string h = hdr.dump();
  while ((h.size() + 8) % 8) h += ' ';
  std::string out;
  uint64_t n = h.size();
  for (int i = 0; i < 8; ++i) out.push_back((char)((n >> (8 * i)) & 0xff));
  out += h;
  for (auto& t : tensors) out += t.second;
  write_file(path, out);
}

// ---------------------------------------------------------------------------------------------
// planner
// ---------------------------------------------------------------------------------------------
namespace {

struct Need {                      // one checkpoint tensor an instruction wants
  std::string tensor;              // checkpoint name (".weight" appended)
  std::vector<uint64_t> full;      // unsharded shape
  enum Shard { Full, Rows, Cols, Heads } shard = Full;
  DType device_dtype = DType::Bf16;
};
struct ParamSpec {
  std::string name;                // device parameter name
  DType dtype = DType::Bf16;
  std::vector<Need> parts;         // appended in order (packing)
  bool expert_stack = false;       // parts hold "{expert}"; replicated over the rank's experts
  bool optional = false;
  uint64_t experts = 0;
};

std::string expand_expert(const std::string& s, uint64_t e) {
  std::string out = s;
  size_t p = out.find("{expert}");
  if (p != std::string::npos) out.replace(p, 8, std::to_string(e));
  return out;
}

uint64_t attr_u(const Instruction& i, const char* k) {
  auto a = i.attr(k);
  if (!a) invalid("instruction " + i.name + " lacks attribute " + k);
  return (uint64_t)strtoull(a->c_str(), nullptr, 10);
}

std::vector<ParamSpec> specs_of(const Program& p) {
  std::vector<ParamSpec> out;
  const uint64_t tp = p.parallel.tp;
  auto in_width = [&](const Instruction& i, size_t k = 0) { return (uint64_t)p.instructions[i.inputs.at(k)].width; };
  auto norm_spec = [&](const Instruction& i, uint64_t width) {
    if (auto nw = i.attr("norm_weight")) {
      ParamSpec s;
      s.name = *nw;
      s.optional = i.attr("norm_optional") != nullptr;
      s.parts.push_back({*nw + ".weight", {width}, Need::Full, DType::Bf16});
      out.push_back(s);
    }
  };
  for (auto& i : p.instructions) {
    const std::string& op = i.op;
    if (op == "embedding") {
      ParamSpec s;
      s.name = *i.attr("weight");
      s.parts.push_back({s.name + ".weight", {attr_u(i, "vocab"), attr_u(i, "width")}, Need::Full, DType::Bf16});
      out.push_back(s);
    } else if (op == "norm" || op == "optional_norm") {
      ParamSpec s;
      s.name = *i.attr("weight");
      s.optional = op == "optional_norm";
      s.parts.push_back({s.name + ".weight", {(uint64_t)i.width}, Need::Full, DType::Bf16});
      out.push_back(s);
    } else if (op == "linear" || op == "linear_allreduce" || op == "lm_head") {
      const uint64_t K = in_width(i);
      norm_spec(i, K);
      const std::string pl = *i.attr("placement");
      const uint64_t w = attr_u(i, "width");
      ParamSpec s;
      s.name = *i.attr("weight");
      auto part = [&](const std::string& nm, uint64_t width) {
        if (pl == "tp_rows") return Need{nm + ".weight", {width * tp, K}, Need::Rows, DType::Bf16};
        if (pl == "tp_columns") return Need{nm + ".weight", {width, K * tp}, Need::Cols, DType::Bf16};
        return Need{nm + ".weight", {width, K}, Need::Full, DType::Bf16};
      };
      s.parts.push_back(part(s.name, w));
      if (auto pw = i.attr("paired_weight")) {
        uint64_t pwid = i.attr("paired_width") ? attr_u(i, "paired_width") : w;
        s.parts.push_back(part(*pw, pwid));
        s.name += "|" + *pw;
      }
      out.push_back(s);
    } else if (op == "mla_kv_write") {
      ParamSpec s;
      s.name = *i.attr("weight");
      s.parts.push_back({s.name + ".weight", {in_width(i, 0)}, Need::Full, DType::Bf16});
      out.push_back(s);
    } else if (op == "mhc_post") {
      norm_spec(i, in_width(i, 1));          // the branch norm folded into the mixing kernel, when there is one
    } else if (op == "mhc_pre" || op == "mhc_merge") {
      // the mixing module of a hyper-connection: four f32 tensors under the module's scope (no ".weight" suffix)
      const uint64_t S = attr_u(i, "streams"), total = in_width(i), M = S * S + 2 * S;
      const std::string base = *i.attr("weight");
      const std::pair<const char*, std::vector<uint64_t>> parts[4] = {{".phi", {M, total}}, {".gamma", {total}}, {".alpha", {3}}, {".beta", {M}}};
      for (auto& kv : parts) {
        ParamSpec s;
        s.name = base + kv.first;
        s.dtype = DType::F32;
        s.parts.push_back({s.name, kv.second, Need::Full, DType::F32});
        out.push_back(s);
      }
    } else if (op == "mome") {
      // depthwise taps of every channel of the model (a rank convolving its own channel range indexes into them)
      const bool sharded = i.attr("placement") && *i.attr("placement") == "tp_channels";
      ParamSpec s;
      s.name = *i.attr("weight");
      s.dtype = DType::F32;
      s.parts.push_back({s.name + ".weight", {(uint64_t)i.width * (sharded ? tp : 1), 1, attr_u(i, "taps")}, Need::Full, DType::F32});
      out.push_back(s);
    } else if (op == "sink_normalize") {
      const uint64_t count = attr_u(i, "count"), latent = attr_u(i, "latent"), rope = attr_u(i, "rope");
      const std::string base = *i.attr("weight");
      ParamSpec kv, pe, nw;
      kv.name = base + ".param_sink_compressed_kv";
      kv.parts.push_back({kv.name, {count, latent}, Need::Full, DType::Bf16});
      pe.name = base + ".param_sink_k_pe";
      pe.parts.push_back({pe.name, {count, rope}, Need::Full, DType::Bf16});
      nw.name = *i.attr("norm");
      nw.parts.push_back({nw.name + ".weight", {latent}, Need::Full, DType::Bf16});
      out.push_back(kv);
      out.push_back(pe);
      out.push_back(nw);
    } else if (op == "mla_q_absorb" || op == "mla_attention") {
      ParamSpec s;
      s.name = *i.attr("weight");
      uint64_t heads = attr_u(i, "heads"), latent = attr_u(i, "latent");
      uint64_t rows;
      if (op == "mla_q_absorb") rows = attr_u(i, "nope") + (i.attr("value") ? attr_u(i, "value") : attr_u(i, "nope"));
      else rows = (i.attr("nope") ? attr_u(i, "nope") : attr_u(i, "value")) + attr_u(i, "value");
      s.parts.push_back({s.name + ".weight", {heads * rows, latent}, Need::Rows, DType::Bf16});
      out.push_back(s);
    } else if (op == "router_topk") {
      const uint64_t K = in_width(i);
      norm_spec(i, K);
      ParamSpec s;
      s.name = *i.attr("weight");
      s.dtype = DType::F32;
      s.parts.push_back({s.name + ".weight", {attr_u(i, "experts"), K}, Need::Full, DType::F32});
      out.push_back(s);
      if (*i.attr("scoring") == "sigmoid_bias_group_topk") {
        ParamSpec b;
        b.name = *i.attr("weight") + ".e_score_correction_bias";
        b.dtype = DType::F32;
        b.optional = true;
        b.parts.push_back({b.name, {attr_u(i, "experts")}, Need::Full, DType::F32});
        out.push_back(b);
      }
    } else if (op == "moe_gate_up") {
      const uint64_t K = in_width(i), F = attr_u(i, "width");
      norm_spec(i, K);
      const Instruction& routes = p.instructions[i.inputs.at(1)];
      ParamSpec s;
      s.name = *i.attr("weight") + "|" + *i.attr("paired_weight");
      s.expert_stack = true;
      s.experts = attr_u(routes, "experts");
      s.parts.push_back({*i.attr("weight") + ".weight", {F, K}, Need::Full, DType::Bf16});
      s.parts.push_back({*i.attr("paired_weight") + ".weight", {F, K}, Need::Full, DType::Bf16});
      out.push_back(s);
      if (auto sw = i.attr("shared_weight")) {
        uint64_t fs = attr_u(i, "shared_width");
        ParamSpec q;
        q.name = *sw + "|" + *i.attr("shared_paired_weight");
        q.parts.push_back({*sw + ".weight", {fs * tp, K}, Need::Rows, DType::Bf16});
        q.parts.push_back({*i.attr("shared_paired_weight") + ".weight", {fs * tp, K}, Need::Rows, DType::Bf16});
        out.push_back(q);
      }
    } else if (op == "moe_down_allreduce") {
      const Instruction& act = p.instructions[i.inputs.at(0)];
      const Instruction& routes = p.instructions[i.inputs.at(1)];
      const uint64_t F = act.width, D = attr_u(i, "width");
      ParamSpec s;
      s.name = *i.attr("weight");
      s.expert_stack = true;
      s.experts = attr_u(routes, "experts");
      s.parts.push_back({s.name + ".weight", {D, F}, Need::Full, DType::Bf16});
      out.push_back(s);
      if (auto sw = i.attr("shared_weight")) {
        const Instruction& gu = act;
        uint64_t fs = attr_u(gu, "shared_width");
        ParamSpec q;
        q.name = *sw;
        q.parts.push_back({*sw + ".weight", {D, fs * tp}, Need::Cols, DType::Bf16});
        out.push_back(q);
      }
    }
  }
  // a weight used by several instructions (e.g. kv_b by absorb and attention) becomes one parameter
  std::vector<ParamSpec> uniq;
  std::map<std::string, size_t> seen;
  for (auto& s : out) {
    auto it = seen.find(s.name);
    if (it == seen.end()) {
      seen[s.name] = uniq.size();
      uniq.push_back(s);
    } else if (uniq[it->second].parts.size() != s.parts.size() || uniq[it->second].parts[0].full != s.parts[0].full) {
      invalid("weight " + s.name + " is requested with two different shapes");
    }
  }
  return uniq;
}

}  // namespace

std::map<std::string, std::pair<DType, std::vector<uint64_t>>> required_tensors(const Program& p) {
  std::map<std::string, std::pair<DType, std::vector<uint64_t>>> out;
  for (auto& s : specs_of(p)) {
    if (s.optional) continue;
    for (auto& n : s.parts) {
      if (s.expert_stack) {
        for (uint64_t e = 0; e < s.experts; ++e) out[expand_expert(n.tensor, e)] = {DType::Bf16, n.full};
      } else {
        out[n.tensor] = {n.device_dtype == DType::F32 ? DType::F32 : DType::Bf16, n.full};
      }
    }
  }
  return out;
}

std::vector<Plan> plan_all(const Program& p, const Checkpoint& ckpt) {
  const uint64_t tp = p.parallel.tp;
  auto specs = specs_of(p);
  std::vector<Plan> plans;
  for (uint32_t rank = 0; rank < tp; ++rank) {
    Plan plan;
    plan.rank = rank;
    plan.device = p.parallel.devices.at(rank);
    plan.provenance = ckpt.fingerprint;
    for (auto& s : specs) {
      // resolve tensors first so that optional weights vanish cleanly
      bool missing = false;
      for (auto& n : s.parts)
        if (!ckpt.has(s.expert_stack ? expand_expert(n.tensor, 0) : n.tensor)) missing = true;
      if (missing) {
        if (s.optional) continue;
        for (auto& n : s.parts) (void)ckpt.need(s.expert_stack ? expand_expert(n.tensor, 0) : n.tensor);
      }
      Parameter prm;
      prm.id = (uint32_t)plan.parameters.size();
      prm.name = s.name;
      prm.dtype = s.dtype;
      const uint64_t e_local = s.expert_stack ? s.experts / tp : 1;
      uint64_t rows_total = 0, cols = 0;
      std::vector<LoadSlice> loads;
      for (uint64_t el = 0; el < e_local; ++el) {
        for (auto& n : s.parts) {
          const std::string tname = s.expert_stack ? expand_expert(n.tensor, rank * e_local + el) : n.tensor;
          const TensorInfo& t = ckpt.need(tname);
          if (t.shape != n.full) {
            std::string want, got;
            for (auto d : n.full) want += std::to_string(d) + " ";
            for (auto d : t.shape) got += std::to_string(d) + " ";
            invalid("tensor " + tname + " has shape [" + got + "], the program needs [" + want + "]");
          }
          if (t.dtype != DType::Bf16 && t.dtype != n.device_dtype) invalid("tensor " + tname + ": unsupported source dtype " + dtype_name(t.dtype));
          if (t.dtype == DType::Bf16 && n.device_dtype != DType::Bf16 && n.device_dtype != DType::F32) invalid("tensor " + tname + ": only bf16->f32 conversion exists");
          const uint64_t eb = dtype_bytes(t.dtype);
          LoadSlice l;
          l.dest = prm.id;
          l.tensor = tname;
          l.shard = t.file;
          l.src_dtype = t.dtype;
          // a tensor of rank three or more is rows x (everything else): [channels, 1, taps] loads as [channels, taps]
          uint64_t inner = 1;
          for (size_t d = 1; d < n.full.size(); ++d) inner *= n.full[d];
          const uint64_t R = n.full.size() == 1 ? 1 : n.full[0], C = n.full.size() == 1 ? n.full[0] : inner;
          uint64_t r_local = R, c_local = C;
          switch (n.shard) {
            case Need::Full:
              l.tag = 1;
              l.offset = t.file_offset();
              l.bytes = R * C * eb;
              break;
            case Need::Rows:
            case Need::Heads:
              if (R % tp) invalid("tensor " + tname + ": rows not divisible by tp");
              r_local = R / tp;
              l.tag = 1;
              l.offset = t.file_offset() + rank * r_local * C * eb;
              l.bytes = r_local * C * eb;
              break;
            case Need::Cols:
              if (C % tp) invalid("tensor " + tname + ": columns not divisible by tp");
              c_local = C / tp;
              l.tag = 2;
              l.offset = t.file_offset() + rank * c_local * eb;
              l.row_bytes = c_local * eb;
              l.stride_bytes = C * eb;
              l.bytes = R * c_local * eb;
              break;
          }
          if (cols == 0) cols = c_local;
          if (cols != c_local) invalid("packed weights of " + s.name + " disagree on the inner dimension");
          rows_total += r_local;
          loads.push_back(std::move(l));
        }
      }
      if (s.expert_stack) prm.dims = {e_local, rows_total / e_local, cols};
      else if (s.parts[0].full.size() == 1) prm.dims = {cols};
      else prm.dims = {rows_total, cols};
      plan.parameters.push_back(std::move(prm));
      for (auto& l : loads) plan.loads.push_back(std::move(l));
    }
    plans.push_back(std::move(plan));
  }
  return plans;
}

// ---------------------------------------------------------------------------------------------
// execution
// ---------------------------------------------------------------------------------------------
void HostMemory::write(uint32_t param, uint64_t offset, const void* data, uint64_t bytes) {
  auto it = store.find(param);
  if (it == store.end() || offset + bytes > it->second.size()) fail(ErrorKind::Capacity, "write outside parameter " + std::to_string(param));
  memcpy(it->second.data() + offset, data, bytes);
}
void HostMemory::read(uint32_t param, uint64_t offset, void* out, uint64_t bytes) {
  auto it = store.find(param);
  if (it == store.end() || offset + bytes > it->second.size()) fail(ErrorKind::Capacity, "read outside parameter " + std::to_string(param));
  memcpy(out, it->second.data() + offset, bytes);
}

uint64_t execute(const Plan& plan, const Checkpoint& ckpt, DeviceMemory& mem, const ExecuteOptions& opt) {
  if (!ckpt.fingerprint.empty() && !plan.provenance.empty() && ckpt.fingerprint != plan.provenance)
    fail(ErrorKind::Stale, "initialization plan was made for a different checkpoint (metadata hash differs)");
  if (opt.staging_bytes < 4096) invalid("staging buffer too small");
  for (auto& p : plan.parameters) mem.allocate(p);
  std::vector<uint64_t> cursor(plan.parameters.size(), 0);
  std::vector<char> stage(opt.staging_bytes), conv;
  std::map<std::string, std::unique_ptr<std::ifstream>> files;
  uint64_t written = 0;
  std::map<std::string, uint64_t> sizes;
  for (auto& l : plan.loads) {
    const Parameter& prm = plan.parameters.at(l.dest);
    const std::string what = l.tensor.empty() ? l.shard + "@" + std::to_string(l.offset) : l.tensor;
    auto& f = files[l.shard];
    if (!f) {
      const std::string path = ckpt.dir + "/" + l.shard;
      f = std::make_unique<std::ifstream>(path, std::ios::binary);
      if (!*f) fail(ErrorKind::Io, "cannot open " + path);
      f->seekg(0, std::ios::end);
      sizes[l.shard] = (uint64_t)f->tellg();
    }
    const uint64_t file_bytes = sizes[l.shard];
    const bool widen = l.src_dtype == DType::Bf16 && prm.dtype == DType::F32;
    if (!widen && l.src_dtype != prm.dtype) invalid("load of " + what + ": no conversion from " + dtype_name(l.src_dtype) + " to " + dtype_name(prm.dtype));
    auto push = [&](const char* data, uint64_t n) {
      if (widen) {
        conv.resize(n * 2);
        const uint16_t* s = (const uint16_t*)data;
        uint32_t* d = (uint32_t*)conv.data();
        for (uint64_t i = 0; i < n / 2; ++i) d[i] = (uint32_t)s[i] << 16;
        mem.write(l.dest, cursor[l.dest], conv.data(), n * 2);
        if (opt.verify_upload) {
          std::vector<char> back(n * 2);
          mem.read(l.dest, cursor[l.dest], back.data(), n * 2);
          if (memcmp(back.data(), conv.data(), n * 2) != 0) fail(ErrorKind::Backend, "upload verification failed for " + what);
        }
        cursor[l.dest] += n * 2;
        written += n * 2;
      } else {
        mem.write(l.dest, cursor[l.dest], data, n);
        if (opt.verify_upload) {
          std::vector<char> back(n);
          mem.read(l.dest, cursor[l.dest], back.data(), n);
          if (memcmp(back.data(), data, n) != 0) fail(ErrorKind::Backend, "upload verification failed for " + what);
        }
        cursor[l.dest] += n;
        written += n;
      }
    };
    if (l.tag == 1) {
      if (l.offset + l.bytes > file_bytes) invalid("load of " + what + " runs past the end of " + l.shard);
      uint64_t done = 0;
      while (done < l.bytes) {
        uint64_t n = std::min<uint64_t>(stage.size(), l.bytes - done);
        f->seekg((std::streamoff)(l.offset + done));
        f->read(stage.data(), (std::streamsize)n);
        if (!*f) fail(ErrorKind::Io, "short read of " + what);
        push(stage.data(), n);
        done += n;
      }
    } else {
      const uint64_t rows = l.bytes / l.row_bytes;
      if (l.offset + (rows - 1) * l.stride_bytes + l.row_bytes > file_bytes) invalid("strided load of " + what + " runs past the end of " + l.shard);
      // pack as many rows as fit the staging buffer, then write once
      const uint64_t per = std::max<uint64_t>(1, stage.size() / l.row_bytes);
      if (l.row_bytes > stage.size()) stage.resize(l.row_bytes);
      for (uint64_t r0 = 0; r0 < rows; r0 += per) {
        uint64_t n = std::min(per, rows - r0);
        for (uint64_t r = 0; r < n; ++r) {
          f->seekg((std::streamoff)(l.offset + (r0 + r) * l.stride_bytes));
          f->read(stage.data() + r * l.row_bytes, (std::streamsize)l.row_bytes);
          if (!*f) fail(ErrorKind::Io, "short read of " + what);
        }
        push(stage.data(), n * l.row_bytes);
      }
    }
  }
  for (auto& p : plan.parameters)
    if (cursor[p.id] != p.bytes()) invalid("parameter " + p.name + " was filled with " + std::to_string(cursor[p.id]) + " of " + std::to_string(p.bytes()) + " bytes");
  return written;
}

}  // namespace ifab::init
