#include "bundle.h"
#include "physical.h"

#include <algorithm>
#include <cstdio>
#include <filesystem>
#include <sstream>
#include <unistd.h>

namespace ifab::bundle {

using program::Instruction;
using program::Program;
namespace fs = std::filesystem;

static uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
static uint64_t dtype_size(const std::string& d) {
  if (d == "f32" || d == "i32") return 4;
  if (d == "int8" || d == "fp8") return 1;
  return 2;
}

uint64_t value_bytes(const Program& p, const Instruction& ins, uint32_t tokens) {
  using graph::Kind;
  if (ins.kind == program::kKindView || ins.kind == program::kKindNone) return 0;
  switch ((Kind)ins.kind) {
    case Kind::Cache:
    case Kind::IndexCache: return 0;  // sequence state, owned by the page pool
    case Kind::Routes: return (uint64_t)tokens * ins.width * 8 + (uint64_t)tokens * strtoull(ins.attr("experts") ? ins.attr("experts")->c_str() : "0", nullptr, 10) * 4;
    case Kind::Experts: {
      // one row per route (+ one for the shared expert)
      uint64_t topk = 8;
      for (uint32_t in : ins.inputs)
        if (p.instructions[in].kind == (uint32_t)Kind::Routes) topk = p.instructions[in].width;
      return (uint64_t)tokens * (topk + 1) * ins.width * dtype_size(ins.dtype);
    }
    case Kind::Indices: return (uint64_t)tokens * ins.width * 4;
    case Kind::Quantized: return (uint64_t)tokens * (ins.width + 4);
    case Kind::HyperConnection: return (uint64_t)tokens * (ins.width * 2 + 64 * 4);
    default: return (uint64_t)tokens * ins.width * dtype_size(ins.dtype);
  }
}

Arena plan_arena(const Program& p, uint32_t tokens, const std::set<uint32_t>& pass_through) {
  Arena a;
  a.tokens = tokens;
  const uint32_t n = (uint32_t)p.instructions.size();
  // a view - and an instruction that passes its input through - keeps its source alive
  std::vector<uint32_t> root(n);
  for (uint32_t i = 0; i < n; ++i)
    root[i] = (p.instructions[i].kind == program::kKindView || pass_through.count(i)) ? root[p.instructions[i].inputs[0]] : i;
  std::vector<uint32_t> last(n);
  for (uint32_t i = 0; i < n; ++i) last[i] = i;
  for (uint32_t i = 0; i < n; ++i)
    for (uint32_t in : p.instructions[i].inputs) last[root[in]] = std::max(last[root[in]], i);
  last[root[p.output]] = n;  // the output outlives the step
  struct Live { uint64_t off, bytes; uint32_t until; };
  std::vector<Live> live;
  for (uint32_t i = 0; i < n; ++i) {
    const uint64_t need = pass_through.count(i) ? 0 : align_up(value_bytes(p, p.instructions[i], tokens), 512);
    // an in-place residual update may reuse its residual's slot, but the packing stays conservative:
    live.erase(std::remove_if(live.begin(), live.end(), [&](const Live& l) { return l.until < i; }), live.end());
    if (need == 0) continue;
    std::sort(live.begin(), live.end(), [](const Live& x, const Live& y) { return x.off < y.off; });
    uint64_t off = 0;
    for (auto& l : live) {
      if (off + need <= l.off) break;
      off = std::max(off, l.off + l.bytes);
    }
    live.push_back({off, need, last[i]});
    a.slots.push_back({i, off, need, i, last[i]});
    a.bytes = std::max(a.bytes, off + need);
  }
  // shared workspace: closed-form maxima over the instructions
  uint64_t ws = 0;
  for (auto& ins : p.instructions) {
    if (ins.op == "mla_attention" || ins.op == "latent_attention") {
      uint64_t heads = 0, latent = 512;
      if (auto h = ins.attr("heads")) heads = strtoull(h->c_str(), nullptr, 10) / p.parallel.tp;
      if (auto l = ins.attr("latent")) latent = strtoull(l->c_str(), nullptr, 10);
      ws = std::max<uint64_t>(ws, (uint64_t)tokens * std::max<uint64_t>(heads, 1) * 64 * (latent + 2) * 4);
    } else if (ins.op == "paged_attention") {
      ws = std::max<uint64_t>(ws, (uint64_t)tokens * ins.width * 64 * 4 + (uint64_t)tokens * 64 * 8 * 64);
    } else if (ins.op == "lm_head") {
      ws = std::max<uint64_t>(ws, ((uint64_t)ins.width / p.parallel.tp / 8 + 1) * 8 * 8);
    }
  }
  a.workspace_bytes = align_up(ws, 512);
  a.verify();
  return a;
}

void Arena::verify() const {
  for (size_t i = 0; i < slots.size(); ++i) {
    const ArenaSlot& s = slots[i];
    if (s.offset % 512 || s.bytes % 512 || s.bytes == 0) invalid("arena: slot " + std::to_string(i) + " is not 512-byte aligned");
    if (s.offset + s.bytes > bytes) invalid("arena: slot exceeds the arena");
    for (size_t k = 0; k < i; ++k) {
      const ArenaSlot& o = slots[k];
      bool time = !(o.last < s.first || s.last < o.first);
      bool space = !(o.offset + o.bytes <= s.offset || s.offset + s.bytes <= o.offset);
      if (time && space) invalid("arena: slots " + std::to_string(k) + " and " + std::to_string(i) + " overlap while both are live");
    }
  }
}

std::string Arena::encode(uint64_t program_fnv, uint64_t backend_fnv) const {
  std::ostringstream o;
  o << "IFARENA2 " << hex64(program_fnv) << " " << hex64(backend_fnv) << " " << bytes << " " << slots.size() << "\n";
  for (auto& s : slots) o << s.offset << " " << s.bytes << "\n";
  o << "pool\n";
  for (auto& s : slots) o << s.instruction << " " << s.first << " " << s.last << "\n";
  o << "tokens " << tokens << "\n";
  return o.str();
}
std::string Arena::encode_workspace(uint64_t program_fnv, uint64_t backend_fnv) const {
  return "IFWORKSPACE1 " + hex64(program_fnv) + " " + hex64(backend_fnv) + " " + std::to_string(workspace_bytes) + "\n";
}
Arena Arena::decode(const std::string& text, uint64_t* program_fnv, uint64_t* backend_fnv) {
  std::istringstream in(text);
  std::string magic, pf, bf;
  uint64_t bytes = 0;
  size_t n = 0;
  in >> magic >> pf >> bf >> bytes >> n;
  if (!in || (magic != "IFARENA2" && magic != "IFARENA1")) invalid("not an IFARENA file");
  if (n > 100000) fail(ErrorKind::Capacity, "arena: too many slots");
  Arena a;
  a.bytes = bytes;
  if (program_fnv) *program_fnv = strtoull(pf.c_str(), nullptr, 16);
  if (backend_fnv) *backend_fnv = strtoull(bf.c_str(), nullptr, 16);
  uint64_t prev_end = 0;
  (void)prev_end;
  for (size_t i = 0; i < n; ++i) {
    ArenaSlot s;
    in >> s.offset >> s.bytes;
    if (!in) invalid("arena: truncated slot table");
    a.slots.push_back(s);
  }
  std::string section;
  in >> section;
  if (section == "pool" || section == "bindings") {
    for (size_t i = 0; i < n; ++i) {
      in >> a.slots[i].instruction >> a.slots[i].first >> a.slots[i].last;
      if (!in) invalid("arena: truncated " + section + " section");
    }
    std::string key;
    if (in >> key && key == "tokens") in >> a.tokens;
  } else {
    invalid("arena: missing pool/bindings section");
  }
  a.verify();
  return a;
}

// ---------------------------------------------------------------------------------------------
std::string backend_fingerprint(const std::string& dir) {
  if (dir.empty()) return "";
  std::error_code ec;
  std::vector<std::string> files;
  for (auto& e : fs::directory_iterator(dir, ec)) {
    auto ext = e.path().extension().string();
    if (ext == ".cu" || ext == ".cuh" || ext == ".h") files.push_back(e.path().string());
  }
  std::sort(files.begin(), files.end());
  Sha256 h;
  for (auto& f : files) {
    std::string name = fs::path(f).filename().string();
    h.update(name.data(), name.size());
    std::string body = read_file(f);
    h.update(body.data(), body.size());
  }
  return h.hex();
}

// The program as a physical inspection plan (physical.h): one operation per instruction, each with the kernel the lowering
// selected and, where the library has another implementation of the same contract, that one as a second candidate with
// the reason it is not eligible in a decode program. Costs are a stream model (bytes the kernel must read at the measured
// copy rate of a B200 plus a fixed cost per launch), marked analytical with the model's name as evidence. "Logical nodes"
// are instruction numbers of the physical program: fused kernels cover several graph nodes, instructions are unique.
physical::Plan physical_plan(const Program& p, const std::string& backend_fp) {
  using namespace physical;
  const uint64_t tp = p.parallel.tp;
  const std::string revision = "ifab_kernels@" + (backend_fp.empty() ? std::string("unfingerprinted") : backend_fp.substr(0, 16));
  auto stream_cost = [](uint64_t bytes) {
    Cost c;
    c.source = CostSource::Analytical;
    c.estimate_ns = 2000 + bytes / 6400;       // 6.4 TB/s = 6400 bytes per ns
    c.upper_ns = 6000 + bytes / 3200;          // half that rate, and a cold launch
    c.evidence = "stream-model-1: weight bytes at 6.4 TB/s + 2 us per dependent launch";
    return c;
  };
  std::vector<Operation> ops;
  std::vector<Value> values;
  size_t sequence = 0;
  for (uint32_t k = 0; k < p.instructions.size(); ++k) {
    const Instruction& i = p.instructions[k];
    Operation op;
    op.name = i.name.empty() ? i.op : i.name;
    op.logical_nodes = {k};
    for (auto in : i.inputs) op.inputs.push_back(in);
    const bool launches = i.kernel != "view" && i.kernel != "none";
    const uint64_t K = i.inputs.empty() ? 0 : p.instructions[i.inputs[0]].width;
    uint64_t wbytes = 0;
    if (i.op == "linear" || i.op == "linear_allreduce" || i.op == "lm_head") wbytes = K * i.width * 2 * (i.attr("activation") ? 2 : 1) / (i.op == "lm_head" ? tp : 1);
    if (i.op == "embedding") wbytes = (uint64_t)i.width * 2;
    // the kernel field names the decode kernel and, after '|', the kernel that takes the same instruction for bulk rows
    const size_t bar = i.kernel.find('|');
    const std::string decode_kernel = i.kernel.substr(0, bar), bulk_kernel = bar == std::string::npos ? "" : i.kernel.substr(bar + 1);
    Candidate c;
    c.id = launches ? decode_kernel : "view";
    c.contract_revision = revision;
    c.numerical_contract = launches ? (i.dtype.empty() ? "none" : i.dtype) + std::string(" storage, f32 accumulation, sums in rank order") : "alias of its input";
    c.capture_qualified = true;
    c.workspace_bound_bytes = 0;
    if (i.op == "mla_attention" || i.op == "paged_attention") {
      c.workspace_bound_bytes.reset();
      c.unresolved.push_back("split-KV partials: sized from max_context when the engine prepares the program");
    }
    if (i.op == "moe_gate_up" || i.op == "moe_down_allreduce") c.unresolved.push_back("expert bytes depend on the routes of the step: the cost counts the launch only");
    if (launches) {
      c.cost = stream_cost(wbytes);
    } else {
      c.cost.source = CostSource::Analytical;
      c.cost.estimate_ns = c.cost.upper_ns = 0;
      c.cost.evidence = "no launch";
    }
    if (i.op == "embedding") c.boundaries.push_back({BoundaryKind::ControlUpload, "token ids, positions, slots and the page table are written by the engine before the step"});
    if (i.op == "lm_head") c.boundaries.push_back({BoundaryKind::RequestOutput, "the sampled token id (4 bytes per row) is what the engine reads after the step"});
    if (i.op == "kv_cache_append" || i.op == "mla_attention" || i.op == "paged_attention" || i.op == "mome") c.boundaries.push_back({BoundaryKind::PersistentState, "reads or writes a resident sequence state"});
    op.candidates.push_back(std::move(c));
    if (!bulk_kernel.empty()) {
      Candidate g = op.candidates[0];
      g.id = bulk_kernel;
      g.eligible = false;
      g.rejection = "the bulk-row kernel of this instruction (tensor cores): takes 9 or more rows per step, a decode step has at most 8";
      g.boundaries.clear();
      op.candidates.push_back(std::move(g));
    }
    if (i.op == "linear_allreduce" || i.op == "moe_down_allreduce" || i.op == "allreduce") {
      op.collective = Collective{"all_ranks", i.attr("bulk") ? "all_reduce_sum (reduce-scatter + all-gather in the GEMM epilogue)" : "all_reduce_sum (one-shot push in the kernel epilogue)", "f32", i.width, sequence++};
    } else if (i.op == "lm_head") {
      op.collective = Collective{"all_ranks", "argmax_exchange", "f32+i32", 2, sequence++};
    } else if (i.op == "gather") {
      op.collective = Collective{"all_ranks", "all_gather", "bf16", std::max<uint64_t>(1, i.width / tp), sequence++};
    }
    ops.push_back(std::move(op));
    Value v;
    v.logical_node = k;
    const std::string dt = i.dtype == "int8" ? "i8" : i.dtype;
    if ((dt == "bf16" || dt == "f32" || dt == "i8" || dt == "i32") && i.width > 0 && i.kind <= 3) {
      v.dtype = dt;
      v.shape = {1, i.width};
      v.payload_bytes = (uint64_t)i.width * (dt == "bf16" ? 2 : dt == "i8" ? 1 : 4);
      v.alignment = 512;
    }
    values.push_back(std::move(v));
  }
  return serial_plan(p.name, p.parallel.target, Sha256::of(p.encode()), p.parallel.devices, std::move(ops), std::move(values), {p.output});
}

// ---------------------------------------------------------------------------------------------
Json BundleSummary::to_json() const {
  Json j = Json::object();
  j.set("dir", dir);
  j.set("program_sha256", program_sha256);
  j.set("logical_nodes", (int64_t)logical_nodes);
  j.set("instructions", (int64_t)instructions);
  j.set("launches_per_token", (int64_t)launches);
  j.set("collectives_per_token", (int64_t)collectives);
  j.set("arena_bytes", arena_bytes);
  j.set("weight_bytes_per_rank", weight_bytes_per_rank);
  return j;
}

std::string html_view(const graph::Graph& g, const Program& p, const Arena& arena) {
  std::string data = "{\"graph\":" + g.to_json().dump() + ",\"program\":" + p.to_json().dump() + ",\"arena\":{\"bytes\":" + std::to_string(arena.bytes) +
                     ",\"workspace\":" + std::to_string(arena.workspace_bytes) + ",\"slots\":[";
  for (size_t i = 0; i < arena.slots.size(); ++i) {
    auto& s = arena.slots[i];
    data += (i ? "," : "") + std::string("[") + std::to_string(s.instruction) + "," + std::to_string(s.offset) + "," + std::to_string(s.bytes) + "," + std::to_string(s.first) + "," + std::to_string(s.last) + "]";
  }
  data += "]}}";
  // "</" must not appear inside the inline script
  for (size_t pos = 0; (pos = data.find("</", pos)) != std::string::npos; pos += 3) data.replace(pos, 2, "<\\/");
  std::string h =
      "<!doctype html><html><head><meta charset=\"utf-8\"><title>" + json_escape(g.name) + " - token program</title><style>"
      "body{font:13px/1.4 monospace;margin:0;display:flex;height:100vh}#l{width:46%;overflow:auto;border-right:1px solid #999}"
      "#r{flex:1;overflow:auto;padding:8px}table{border-collapse:collapse;width:100%}td,th{border-bottom:1px solid #ddd;padding:2px 6px;text-align:left}"
      "tr:hover{background:#eef}tr.sel{background:#cdf}.c{background:#ffd9a8}input{width:95%;margin:4px}h3{margin:6px 0}"
      "</style></head><body><div id=\"l\"><input id=\"q\" placeholder=\"filter by op / name\"><table id=\"t\"></table></div>"
      "<div id=\"r\"><h3 id=\"h\"></h3><pre id=\"d\"></pre></div><script>const D=" + data + ";\n"
      "const P=D.program.instructions,G=D.graph.nodes,T=document.getElementById('t'),Q=document.getElementById('q');\n"
      "function coll(o){return ['linear_allreduce','moe_down_allreduce','allreduce','gather','lm_head'].includes(o)}\n"
      "function row(i,k){return '<tr data-k=\"'+k+'\" class=\"'+(coll(i.op)?'c':'')+'\"><td>'+k+'</td><td>'+i.op+'</td><td>'+i.name+'</td><td>'+i.dtype+'['+i.width+']</td><td>'+i.kernel+'</td></tr>'}\n"
      "function draw(){const f=Q.value.toLowerCase();T.innerHTML='<tr><th>#</th><th>op</th><th>name</th><th>type</th><th>kernel</th></tr>'+P.map((i,k)=>[i,k]).filter(([i])=>!f||i.op.includes(f)||i.name.toLowerCase().includes(f)).map(([i,k])=>row(i,k)).join('')}\n"
      "function show(k){const i=P[k],n=G[i.logical_node];document.getElementById('h').textContent='#'+k+' '+i.op+'  '+i.name;\n"
      "const s=D.arena.slots.find(s=>s[0]==k);document.getElementById('d').textContent=JSON.stringify({instruction:i,arena_slot:s?{offset:s[1],bytes:s[2],live:[s[3],s[4]]}:null,logical:n,inputs:i.inputs.map(x=>x+' '+P[x].op+' '+P[x].name)},null,1)}\n"
      "T.onclick=e=>{const r=e.target.closest('tr');if(!r||!r.dataset.k)return;document.querySelectorAll('tr.sel').forEach(x=>x.classList.remove('sel'));r.classList.add('sel');show(+r.dataset.k)};Q.oninput=draw;draw();\n"
      "document.getElementById('h').textContent=D.graph.name+': '+G.length+' logical nodes, '+P.length+' instructions, '+D.program.launches_per_token+' launches/token, arena '+D.arena.bytes+' B';\n"
      "</script></body></html>\n";
  return h;
}

BundleSummary write_bundle(const BundleInputs& in, const std::string& out_dir) {
  if (path_exists(out_dir)) fail(ErrorKind::Io, "bundle output " + out_dir + " already exists; refusing to overwrite");
  graph::Graph g = graph::compile_source(in.source_text);
  Program p = program::lower(g, in.options);
  const std::string exec = p.encode();
  const std::string sha = Sha256::of(exec);
  init::Checkpoint ckpt = in.checkpoint_dir.empty() ? init::Checkpoint::synthetic(init::required_tensors(p)) : init::Checkpoint::inspect(in.checkpoint_dir);
  std::vector<init::Plan> plans = init::plan_all(p, ckpt);
  serving::Manifest man = serving::lower(p, sha);
  const uint32_t arena_tokens = std::max<uint32_t>(std::max(in.options.prefill_tokens, in.options.resident_sequences), 1);
  // optional norms whose gain no rank loads pass their rows through: the arena lets their source live on instead of a copy
  std::set<uint32_t> pass_through;
  for (uint32_t i = 0; i < p.instructions.size(); ++i) {
    const auto& ins = p.instructions[i];
    if (ins.op != "optional_norm" || ins.inputs.size() != 1 || !ins.attr("weight")) continue;
    const auto& src = p.instructions[ins.inputs[0]];
    if (src.kind != ins.kind || src.width != ins.width || src.dtype != ins.dtype || src.kind == program::kKindView) continue;
    bool loaded = false;
    for (const auto& pl : plans)
      for (const auto& prm : pl.parameters) loaded = loaded || prm.name == *ins.attr("weight");
    if (!loaded) pass_through.insert(i);
  }
  Arena arena = plan_arena(p, arena_tokens, pass_through);
  const std::string bfp = backend_fingerprint(in.kernel_source_dir);
  const uint64_t pf = fnv1a64(exec.data(), exec.size()), bf = fnv1a64(bfp.data(), bfp.size());

  fs::path out(out_dir);
  fs::path parent = out.parent_path().empty() ? fs::path(".") : out.parent_path();
  make_dirs(parent.string());
  fs::path stage = parent / (out.filename().string() + ".staging." + std::to_string((long)getpid()));
  std::error_code ec;
  fs::remove_all(stage, ec);
  make_dirs(stage.string());
  auto put = [&](const std::string& name, const std::string& data) { write_file((stage / name).string(), data); };
  try {
    put("execution.bin", exec);
    put("logical.bin", g.encode());
    put("model.inferfabric", in.source_text);   // the checked source travels with the bundle: host executors recompile it
    put("execution.json", g.to_json().dump(1));
    put("execution.dot", g.dot());
    put("execution.html", html_view(g, p, arena));
    put("device-program.json", p.to_json().dump(1));
    put("physical.json", physical_plan(p, bfp).to_json().dump(1));
    put("serving.json", man.to_json().dump(1));
    for (auto& pl : plans) {
      put("rank-" + std::to_string(pl.rank) + ".bin", pl.encode());
      put("rank-" + std::to_string(pl.rank) + ".init.json", pl.to_json().dump(1));
      put("arena-rank-" + std::to_string(pl.rank) + ".txt", arena.encode(pf, bf));
      put("workspace-rank-" + std::to_string(pl.rank) + ".txt", arena.encode_workspace(pf, bf));
    }
    Json aj = Json::object();
    aj.set("format", "inferfabric.arena.v1");
    aj.set("bytes", arena.bytes);
    aj.set("workspace_bytes", arena.workspace_bytes);
    aj.set("tokens", arena.tokens);
    aj.set("slots", (int64_t)arena.slots.size());
    aj.set("program_fingerprint", hex64(pf));
    aj.set("backend_fingerprint", hex64(bf));
    put("arena.json", aj.dump(1));
    Json idx = Json::object();
    idx.set("format", "inferfabric.token-bundle.v1");
    idx.set("model", g.name);
    idx.set("source", in.source_path);
    idx.set("source_sha256", Sha256::of(in.source_text));
    idx.set("program_sha256", sha);
    idx.set("program_magic", p.magic());
    idx.set("checkpoint_fingerprint", ckpt.fingerprint);
    idx.set("checkpoint", in.checkpoint_dir);
    idx.set("ranks", p.parallel.tp);
    idx.set("logical_nodes", (int64_t)g.nodes.size());
    idx.set("instructions", (int64_t)p.instructions.size());
    idx.set("launches_per_token", (int64_t)p.launches_per_token());
    idx.set("collectives_per_token", (int64_t)p.collectives_per_token());
    Json files = Json::array();
    for (auto& e : fs::directory_iterator(stage)) files.push(e.path().filename().string());
    std::sort(files.as_array().begin(), files.as_array().end(), [](const Json& a, const Json& b) { return a.as_string() < b.as_string(); });
    idx.set("files", files);
    put("plan.json", idx.dump(1));
    if (path_exists(out_dir)) fail(ErrorKind::Io, "bundle output " + out_dir + " appeared while compiling; refusing to overwrite");
    fs::rename(stage, out, ec);
    if (ec) fail(ErrorKind::Io, "cannot publish bundle: " + ec.message());
  } catch (...) {
    fs::remove_all(stage, ec);
    throw;
  }
  BundleSummary s;
  s.dir = out_dir;
  s.program_sha256 = sha;
  s.logical_nodes = g.nodes.size();
  s.instructions = p.instructions.size();
  s.launches = p.launches_per_token();
  s.collectives = p.collectives_per_token();
  s.arena_bytes = arena.bytes;
  s.weight_bytes_per_rank = plans.empty() ? 0 : plans[0].device_bytes();
  return s;
}

}  // namespace ifab::bundle
