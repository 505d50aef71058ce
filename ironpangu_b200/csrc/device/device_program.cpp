#include "device_program.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <map>
#include <set>

#include "../core/contract.h"
#include "../core/initplan.h"
#include "../kernels/ifab_kernels.h"

namespace ifab::device {
namespace {

void cu(cudaError_t e, const char* what) {
  if (e != cudaSuccess) fail(ErrorKind::Backend, std::string("device program: ") + what + ": " + cudaGetErrorString(e));
}
void kernel(int rc, const std::string& what) {
  if (rc != 0) fail(ErrorKind::Backend, "device program: " + what + " failed: " + ifab_error_string(rc) + " (code " + std::to_string(rc) + ")");
}
// every device allocation of the executor goes through here, so "nothing is allocated after readiness" is a counted fact
uint64_t g_device_allocations = 0;
void dmalloc(void** out, uint64_t bytes, const char* what) {
  cu(cudaMalloc(out, std::max<uint64_t>(bytes, 16)), what);
  ++g_device_allocations;
}
uint64_t fnv1a64(std::string_view s) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (unsigned char c : s) h = (h ^ c) * 0x100000001b3ull;
  return h;
}
std::vector<std::string> words(const std::string& line) {
  std::vector<std::string> out;
  size_t b = 0;
  while (b < line.size()) {
    while (b < line.size() && (line[b] == ' ' || line[b] == '\r')) ++b;
    size_t e = b;
    while (e < line.size() && line[e] != ' ' && line[e] != '\r') ++e;
    if (e > b) out.push_back(line.substr(b, e - b));
    b = e;
  }
  return out;
}
std::vector<std::string> lines(const std::string& text) {
  std::vector<std::string> out;
  size_t b = 0;
  while (b <= text.size()) {
    size_t e = text.find('\n', b);
    if (e == std::string::npos) e = text.size();
    out.push_back(text.substr(b, e - b));
    b = e + 1;
  }
  return out;
}

// Parameters of one rank in device memory, filled by the init-plan executor through a bounded pinned staging buffer.
class CudaMemory : public init::DeviceMemory {
 public:
  explicit CudaMemory(size_t staging_bytes) : staging_bytes_(staging_bytes) { cu(cudaMallocHost(&stage_, staging_bytes_), "pinned staging buffer"); }
  ~CudaMemory() override {
    if (stage_) cudaFreeHost(stage_);
    for (auto& kv : ptr) cudaFree(kv.second);
  }
  void allocate(const init::Parameter& p) override {
    void* d = nullptr;
    dmalloc(&d, p.bytes(), "parameter allocation");
    ptr[p.id] = d;
    size[p.id] = p.bytes();
  }
  void write(uint32_t param, uint64_t offset, const void* data, uint64_t bytes) override {
    if (offset + bytes > size.at(param)) invalid("device program: a load runs past the end of its parameter");
    const char* src = static_cast<const char*>(data);
    for (uint64_t done = 0; done < bytes;) {
      const uint64_t n = std::min<uint64_t>(staging_bytes_, bytes - done);
      std::memcpy(stage_, src + done, n);
      cu(cudaMemcpy(static_cast<char*>(ptr.at(param)) + offset + done, stage_, n, cudaMemcpyHostToDevice), "parameter upload");
      done += n;
      uploaded += n;
    }
  }
  void read(uint32_t param, uint64_t offset, void* out, uint64_t bytes) override {
    cu(cudaMemcpy(out, static_cast<char*>(ptr.at(param)) + offset, bytes, cudaMemcpyDeviceToHost), "parameter read-back");
  }
  std::map<uint32_t, void*> ptr;
  std::map<uint32_t, uint64_t> size;
  uint64_t uploaded = 0;

 private:
  size_t staging_bytes_;
  void* stage_ = nullptr;
};

struct Ins {
  std::string op, name, dtype;
  uint32_t width = 0;
  std::vector<uint32_t> in;
  std::map<std::string, std::string> a;
  bool has(const char* k) const { return a.count(k) != 0; }
  const std::string& s(const char* k) const {
    auto it = a.find(k);
    if (it == a.end()) invalid("device program: instruction " + name + " lacks attribute " + k);
    return it->second;
  }
  int i(const char* k) const { return std::stoi(s(k)); }
  float f(const char* k, float fallback) const { return has(k) ? std::stof(a.at(k)) : fallback; }
};
// a value: a strided row view into the arena (or into a parameter-free state)
struct Val {
  char* ptr = nullptr;     // row 0
  long ld = 0;             // elements per row
  int esize = 2;
};
struct HeadGroup {
  uint32_t qb = 0, write = 0, absorb = 0, qkv = 0;
  bool ok = false;
};
// grouped-query attention: {q, k, v projections of one normalised input, rotary on q and k, page append} feeding one attention
struct GqaGroup {
  uint32_t lq = 0, rq = 0, lk = 0, rk = 0, lv = 0, cache = 0, x = 0;
  void* packed = nullptr;      // [q | k | v] rows of the three matrices, one operand
  int rows = 0, k = 0;
};

}  // namespace

struct DeviceProgram::Impl {
  Options opt;
  std::string name;
  std::vector<Ins> ins;
  uint32_t context = 0, vocab = 0, eos = 0, residents = 1, rows = 1;
  int page_tokens = 16, max_pages = 0, num_pages = 0;
  int kps = 64, max_splits = 1;
  std::unique_ptr<CudaMemory> params;
  std::map<std::string, uint32_t> param_id;
  std::map<std::string, std::vector<uint64_t>> param_dims;
  // one device block: [arena | workspace | control]
  char* block = nullptr;
  uint64_t arena_bytes = 0, workspace_bytes = 0, block_bytes = 0;
  std::map<uint32_t, std::pair<uint64_t, uint64_t>> slot_of;   // instruction -> (offset, size)
  std::vector<Val> val;
  std::map<uint32_t, void*> cache_of;                           // cache-write instruction -> pages
  std::map<uint32_t, uint64_t> cache_bytes;                     // ... and their size (reset)
  std::map<uint32_t, HeadGroup> heads;                          // attention instruction -> its group
  std::set<uint32_t> head_members;
  bool fused_head = false;
  std::map<uint32_t, GqaGroup> gqa;                             // paged-attention instruction -> its group
  std::set<uint32_t> gqa_members;
  char *gqa_qkv = nullptr, *kv_pack = nullptr;                  // [rows, q | k | v] of a step; [rows, k | v] for an append outside a group
  long gqa_ld = 0, kv_pack_ld = 0;
  std::vector<void*> owned;                                     // packed operands and pack buffers
  // hyper-connected programs: mixing weights of a hyper-connection live behind its mixed row in the instruction's slot; token
  // convolutions keep the previous taps-1 rows per resident; sink rows are computed once from the parameters
  struct HcAux { float* post; float* comb; int S; };
  std::map<uint32_t, HcAux> hc_of;
  std::map<uint32_t, std::pair<void*, uint64_t>> conv_state;    // instruction -> (state, bytes)
  std::map<uint32_t, std::pair<const void*, int>> sink_rows;    // sink_normalize instruction -> (rows, count)
  std::map<uint32_t, std::pair<const void*, int>> sinks_of;     // cache-write instruction -> the sink rows its readers also attend to
  std::set<uint32_t> aliased;                                   // instructions that hand a value on without a launch
  std::set<uint32_t> packed;                                    // cache-write instructions whose pages hold packed int8 rows (656 bytes)
  std::map<uint32_t, void*> index_scales;                       // int8 index caches: one half-precision scale per row
  float* index_scores = nullptr;                                // selector scratch [rows, context]
  // control block (device): tokens | positions | slots | next ids | next values, page table; pinned mirror on the host
  int32_t *d_tokens = nullptr, *d_positions = nullptr, *d_slots = nullptr, *d_next = nullptr, *d_page_table = nullptr;
  float* d_next_vals = nullptr;
  int32_t *h_ctl = nullptr, *h_out = nullptr;
  char* fabric_block = nullptr;
  IfabFabric fab{};
  uint32_t* ticket = nullptr;
  cudaStream_t stream = nullptr;
  std::map<int, cudaGraphExec_t> graphs;
  uint64_t launches = 0, steps = 0, h2d = 0, d2h = 0;
  uint64_t launches_per_step_last = 0;
  uint64_t allocations_at_ready = 0;
  bool ready = false;

  ~Impl() {
    for (auto& g : graphs) cudaGraphExecDestroy(g.second);
    for (auto& c : cache_of) cudaFree(c.second);
    for (void* o : owned) cudaFree(o);
    for (auto& c : conv_state) cudaFree(c.second.first);
    if (block) cudaFree(block);
    if (fabric_block) cudaFree(fabric_block);
    if (d_page_table) cudaFree(d_page_table);
    if (h_ctl) cudaFreeHost(h_ctl);
    if (h_out) cudaFreeHost(h_out);
    if (stream) cudaStreamDestroy(stream);
  }

  void* P(const std::string& pname) const {
    auto it = param_id.find(pname);
    if (it == param_id.end()) invalid("device program: the bundle has no parameter " + pname);
    return params->ptr.at(it->second);
  }
  void* P_optional(const std::string& pname) const {
    auto it = param_id.find(pname);
    return it == param_id.end() ? nullptr : params->ptr.at(it->second);
  }
  const std::vector<uint64_t>& dims(const std::string& pname) const { return param_dims.at(pname); }

  Val lease(uint32_t k, uint64_t bytes, long ld, int esize) {
    auto it = slot_of.find(k);
    if (it == slot_of.end()) fail(ErrorKind::Backend, "device program: the arena has no slot for instruction " + std::to_string(k));
    if (bytes > it->second.second)
      fail(ErrorKind::Backend, "device program: instruction " + std::to_string(k) + " needs " + std::to_string(bytes) + " bytes, its arena slot holds " +
                                   std::to_string(it->second.second));
    return Val{block + it->second.first, ld, esize};
  }
  char* workspace(uint64_t bytes) const {
    if (bytes > workspace_bytes) fail(ErrorKind::Backend, "device program: a kernel needs " + std::to_string(bytes) + " bytes of workspace, the plan froze " + std::to_string(workspace_bytes));
    return block + arena_bytes;
  }

  void load(const std::string& bundle, const std::string& checkpoint);
  void dispatch(int T);
  void step(const int32_t* tokens, const int32_t* positions, const int32_t* slots, int T, int32_t* out);
};

void DeviceProgram::Impl::load(const std::string& bundle, const std::string& checkpoint) {
  cu(cudaSetDevice(opt.device), "cudaSetDevice");
  contract::validate_bundle(bundle);                      // kernel and binding contracts of the serialized program, before any allocation
  const Json prog = Json::parse(read_file(bundle + "/device-program.json", 256 << 20));
  const Json man = Json::parse(read_file(bundle + "/serving.json", 16 << 20));
  if (prog.at("parallel").at("tp").as_int() != 1) fail(ErrorKind::NotImplemented, "device program: this executor runs bundles compiled for tp = 1");
  name = prog.at("name").as_string();
  context = (uint32_t)prog.at("max_context").as_int();
  if (opt.context && opt.context < context) context = opt.context;
  eos = (uint32_t)prog.at("eos").as_int();
  vocab = (uint32_t)man.at("vocab").as_int();
  residents = opt.residents ? opt.residents : std::max<uint32_t>(1, (uint32_t)man.at("resident_sequences").as_int());
  for (auto& j : prog.at("instructions").as_array()) {
    Ins x;
    x.op = j.at("op").as_string();
    x.name = j.at("name").as_string();
    x.dtype = j.at("dtype").as_string();
    x.width = (uint32_t)j.at("width").as_int();
    for (auto& i : j.at("inputs").as_array()) x.in.push_back((uint32_t)i.as_int());
    for (auto& kv : j.at("attrs").as_object()) x.a[kv.first] = kv.second.is_string() ? kv.second.as_string() : kv.second.dump();
    ins.push_back(std::move(x));
  }
  // ---- parameters: the rank's init plan, executed into device memory ----
  const init::Plan plan = init::Plan::decode(read_file(bundle + "/rank-0.bin", 64 << 20));
  const init::Checkpoint ck = init::Checkpoint::inspect(checkpoint);
  params = std::make_unique<CudaMemory>(opt.staging_bytes);
  init::ExecuteOptions eo;
  eo.staging_bytes = opt.staging_bytes;
  for (auto& p : plan.parameters) {
    param_id[p.name] = p.id;
    param_dims[p.name] = p.dims;
  }
  init::execute(plan, ck, *params, eo);
  // ---- arena + workspace: one block, the compiler's offsets ----
  const std::string exec_bin = read_file(bundle + "/execution.bin", 256 << 20);
  const uint64_t fingerprint = fnv1a64(exec_bin);
  const auto al = lines(read_file(bundle + "/arena-rank-0.txt", 64 << 20));
  const auto head = words(al.at(0));
  if (head.size() != 5 || head[0] != "IFARENA2") invalid("device program: arena file is not IFARENA2");
  if (std::stoull(head[1], nullptr, 16) != fingerprint) invalid("device program: the arena was planned for another program");
  arena_bytes = std::stoull(head[3]);
  const size_t n = std::stoull(head[4]);
  if (al.size() < 2 * n + 3 || words(al[1 + n]).at(0) != "pool") invalid("device program: arena file is truncated");
  for (size_t i = 0; i < n; ++i) {
    const auto sz = words(al[1 + i]), own = words(al[2 + n + i]);
    const uint64_t off = std::stoull(sz.at(0)), size = std::stoull(sz.at(1));
    if (off % 512 || size % 512 || off + size > arena_bytes) invalid("device program: an arena slot is misaligned or outside the arena");
    slot_of[(uint32_t)std::stoul(own.at(0))] = {off, size};
  }
  const auto tok = words(al[2 + 2 * n]);
  rows = tok.size() == 2 && tok[0] == "tokens" ? (uint32_t)std::stoul(tok[1]) : 1;
  rows = std::max<uint32_t>(1, std::min<uint32_t>(8, rows));
  const auto ws = words(read_file(bundle + "/workspace-rank-0.txt", 1 << 20));
  if (ws.size() != 4 || ws[0] != "IFWORKSPACE1" || std::stoull(ws[1], nullptr, 16) != fingerprint) invalid("device program: the workspace file does not belong to this program");
  workspace_bytes = std::stoull(ws[3]);
  const uint64_t ctl_bytes = 4096;
  block_bytes = arena_bytes + workspace_bytes + ctl_bytes;
  dmalloc((void**)&block, block_bytes, "arena block");
  cu(cudaMemset(block, 0, block_bytes), "arena clear");
  char* ctl = block + arena_bytes + workspace_bytes;
  d_tokens = (int32_t*)ctl;
  d_positions = d_tokens + 8;
  d_slots = d_positions + 8;
  d_next = d_slots + 8;
  d_next_vals = (float*)(d_next + 8);
  cu(cudaMallocHost((void**)&h_ctl, 3 * 8 * sizeof(int32_t)), "pinned control block");
  cu(cudaMallocHost((void**)&h_out, 8 * sizeof(int32_t)), "pinned output block");
  cu(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "stream");
  // ---- sequence state: latent KV pages per resident, identity page table ----
  max_pages = (int)((context + page_tokens - 1) / page_tokens);
  num_pages = max_pages * (int)residents;
  std::vector<int32_t> table((size_t)num_pages);
  for (int i = 0; i < num_pages; ++i) table[(size_t)i] = i;
  dmalloc((void**)&d_page_table, table.size() * 4, "page table");
  cu(cudaMemcpy(d_page_table, table.data(), table.size() * 4, cudaMemcpyHostToDevice), "page table upload");
  max_splits = std::max(1, std::min(64, ((int)context + kps - 1) / kps));
  while ((long)max_splits * kps < (long)context) kps *= 2;
  // ---- a one-rank fabric: staging halves, flags, control words (the fused all-reduce kernels take the descriptor at any width) ----
  {
    const uint64_t data_half = 4 << 20, flag_half_words = 8 * 296, ll_half = 2 << 20;
    const uint64_t flag_bytes = (2 * flag_half_words * 8 + 255) / 256 * 256;
    const uint64_t off_flags = 2 * data_half, off_ctl = off_flags + flag_bytes, off_ll = off_ctl + 256, total = off_ll + 2 * ll_half;
    dmalloc((void**)&fabric_block, total, "fabric block");
    cu(cudaMemset(fabric_block, 0, total), "fabric clear");
    fab.data[0] = fabric_block;
    fab.flags[0] = (uint64_t*)(fabric_block + off_flags);
    fab.seq = (uint64_t*)(fabric_block + off_ctl);
    fab.done = (uint32_t*)(fabric_block + off_ctl + 8);
    fab.status = (uint32_t*)(fabric_block + off_ctl + 16);
    ticket = (uint32_t*)(fabric_block + off_ctl + 32);
    fab.rank = 0;
    fab.world = 1;
    fab.spin_limit = 4000000;
    fab.data_half_bytes = (uint32_t)data_half;
    fab.flag_half_words = (uint32_t)flag_half_words;
    fab.ll_half_bytes = (uint32_t)ll_half;
    fab.ll_offset = off_ll;
    fab.mc = nullptr;
  }
  // ---- values: views into the arena ----
  val.assign(ins.size(), Val{});
  const int T = (int)rows;
  for (uint32_t k = 0; k < ins.size(); ++k) {
    const Ins& x = ins[k];
    if (x.op == "view") continue;
    if (x.op == "mla_kv_write") {
      void* pages = nullptr;
      if (x.dtype == "int8_ds_mla") {
        if (x.width != 576) fail(ErrorKind::NotImplemented, "device program: the packed int8 cache holds 512 latent + 64 rotary columns");
        packed.insert(k);
      } else if (x.dtype != "bf16") {
        fail(ErrorKind::NotImplemented, "device program: cache dtype " + x.dtype + " has no device layout");
      }
      const uint64_t bytes = (uint64_t)num_pages * page_tokens * (packed.count(k) ? 656 : x.width * 2);
      dmalloc(&pages, bytes, "KV pages");
      cu(cudaMemset(pages, 0, bytes), "KV clear");
      cache_of[k] = pages;
      cache_bytes[k] = bytes;
    } else if (x.op == "index_cache_append") {
      const bool q8 = x.has("cache_dtype") && x.s("cache_dtype") == "int8";
      if (x.has("cache_dtype") && !q8 && x.s("cache_dtype") != "bf16") fail(ErrorKind::NotImplemented, "device program: index cache dtype " + x.s("cache_dtype"));
      void* pages = nullptr;
      const uint64_t bytes = (uint64_t)num_pages * page_tokens * x.width * (q8 ? 1 : 2);
      dmalloc(&pages, bytes, "index key pages");
      cu(cudaMemset(pages, 0, bytes), "index keys clear");
      cache_of[k] = pages;
      cache_bytes[k] = bytes;
      if (q8) {
        void* sc = nullptr;
        dmalloc(&sc, (uint64_t)num_pages * page_tokens * 2, "index key scales");
        cu(cudaMemset(sc, 0, (uint64_t)num_pages * page_tokens * 2), "index scales clear");
        index_scales[k] = sc;
        owned.push_back(sc);
      }
    } else if (x.op == "sparse_index") {
      val[k] = lease(k, (uint64_t)T * x.width * 4, x.width, 4);
      if (!index_scores) {
        dmalloc((void**)&index_scores, (uint64_t)rows * context * 4, "selector scores");
        owned.push_back(index_scores);
      }
    } else if (x.op == "mhc_pre" || x.op == "mhc_merge") {
      const int S = x.i("streams");
      if (S + S * S > 64) fail(ErrorKind::NotImplemented, "device program: a hyper-connection slot holds at most 64 mixing weights per row");
      val[k] = lease(k, (uint64_t)T * x.width * 2 + (uint64_t)T * 64 * 4, x.width, 2);     // mixed rows | post weights | stream-to-stream weights
      float* post = (float*)(val[k].ptr + (uint64_t)T * x.width * 2);
      hc_of[k] = HcAux{post, post + (uint64_t)T * S, S};
    } else if (x.op == "mhc_input") {
      val[k] = val[x.in.at(0)];                            // the mixed row of its hyper-connection
      aliased.insert(k);
    } else if (x.op == "optional_norm" && !slot_of.count(k)) {
      // compiled against a checkpoint without this gain: the rows pass through, the arena kept the source's slot alive
      if (P_optional(x.s("weight"))) invalid("device program: the bundle was compiled without " + x.s("weight") + ", the checkpoint has it");
      val[k] = val[x.in.at(0)];
      aliased.insert(k);
    } else if (x.op == "mome") {
      const uint64_t bytes = (uint64_t)residents * (x.i("taps") - 1) * x.width * 2;
      void* st = nullptr;
      dmalloc(&st, bytes, "convolution history");
      cu(cudaMemset(st, 0, bytes), "convolution history clear");
      conv_state[k] = {st, bytes};
      val[k] = lease(k, (uint64_t)T * x.width * 2, x.width, 2);
    } else if (x.op == "sink_normalize") {
      const int count = x.i("count"), lat = x.i("latent"), rope = x.i("rope");
      void* rows_ptr = nullptr;
      dmalloc(&rows_ptr, (uint64_t)count * (lat + rope) * 2, "sink rows");
      owned.push_back(rows_ptr);
      kernel(ifab_rmsnorm_bf16(P(x.s("weight") + ".param_sink_compressed_kv"), lat, P(x.s("norm")), rows_ptr, lat + rope, count, lat, x.f("eps", 1e-5f), 0, stream),
             x.name);
      cu(cudaMemcpy2DAsync((char*)rows_ptr + (size_t)lat * 2, (size_t)(lat + rope) * 2, P(x.s("weight") + ".param_sink_k_pe"), (size_t)rope * 2, (size_t)rope * 2,
                           count, cudaMemcpyDeviceToDevice, stream),
         "sink rows");
      cu(cudaStreamSynchronize(stream), "sink rows");
      sink_rows[k] = {rows_ptr, count};
      val[k] = Val{(char*)rows_ptr, lat + rope, 2};
      aliased.insert(k);
    } else if (x.op == "kv_cache_append") {
      // key pages, then value pages: [pages, page_tokens, local kv heads, head_dim] each
      if (x.has("cache_dtype") && x.s("cache_dtype") != "bf16") fail(ErrorKind::NotImplemented, "device program: K / V pages are bf16");
      void* pages = nullptr;
      const uint64_t bytes = (uint64_t)num_pages * page_tokens * x.width * 2;
      dmalloc(&pages, bytes, "K/V pages");
      cu(cudaMemset(pages, 0, bytes), "K/V clear");
      cache_of[k] = pages;
      cache_bytes[k] = bytes;
      kv_pack_ld = std::max<long>(kv_pack_ld, x.width);
    } else if (x.op == "router_topk") {
      const int E = x.i("experts");
      val[k] = lease(k, (uint64_t)T * x.width * 8 + (uint64_t)T * E * 4, x.width, 4);
    } else if (x.op == "moe_gate_up") {
      const uint32_t topk = ins[x.in.at(1)].width;
      val[k] = lease(k, (uint64_t)T * (topk + 1) * x.width * 2, (long)(topk + 1) * x.width, 2);
    } else if (x.op == "mla_q_absorb") {
      const long w = (long)x.i("heads") * (x.i("latent") + x.i("rope"));
      val[k] = lease(k, (uint64_t)T * w * 2, w, 2);
    } else if (x.op == "lm_head") {
      val[k] = Val{(char*)d_next, 1, 4};
    } else {
      const int es = x.dtype == "f32" ? 4 : 2;
      val[k] = lease(k, (uint64_t)T * x.width * es, x.width, es);
    }
  }
  for (uint32_t k = 0; k < ins.size(); ++k) {          // views: a column range of their source (sources precede them)
    const Ins& x = ins[k];
    if (x.op != "view") continue;
    const Val& src = val[x.in.at(0)];
    val[k] = Val{src.ptr + (long)x.i("start") * src.esize, src.ld, src.esize};
  }
  // ---- dispatcher: the attention group as one launch ----
  std::map<uint32_t, std::vector<uint32_t>> users;
  for (uint32_t k = 0; k < ins.size(); ++k)
    for (uint32_t j : ins[k].in) users[j].push_back(k);
  auto only_user = [&](uint32_t v, uint32_t u) { return users[v].size() == 1 && users[v][0] == u; };
  bool all_ok = true, any = false;
  for (uint32_t k = 0; k < ins.size(); ++k) {
    const Ins& x = ins[k];
    if (x.op != "mla_attention") continue;
    HeadGroup g;
    g.absorb = x.in.at(0);
    g.write = x.in.at(1);
    if (ins[g.absorb].op != "mla_q_absorb" || ins[g.write].op != "mla_kv_write") continue;
    g.qb = ins[g.absorb].in.at(0);
    const Ins &qb = ins[g.qb], &ab = ins[g.absorb];
    if (qb.op != "linear" || !qb.has("norm_weight") || qb.has("paired_weight")) continue;
    const Ins &vq = ins[qb.in.at(0)], &vl = ins[ins[g.write].in.at(0)], &vr = ins[ins[g.write].in.at(1)];
    if (vq.op != "view" || vl.op != "view" || vr.op != "view" || vq.in[0] != vl.in[0] || vq.in[0] != vr.in[0]) continue;
    g.qkv = vq.in[0];
    const int q_lora = vq.i("width"), latent = ab.i("latent"), rope = ab.i("rope"), nope = ab.i("nope"), vdim = x.i("value");
    const bool layout = vq.i("start") == 0 && vl.i("start") == q_lora && vr.i("start") == q_lora + latent;
    const bool priv = only_user(g.qb, g.absorb) && only_user(g.absorb, k) && only_user(g.write, k);
    g.ok = ins[g.write].dtype == "bf16" && x.in.size() == 2 && layout && priv && latent == 512 && rope == 64 && nope % 32 == 0 && nope <= 128 && vdim <= 128 && q_lora % 8 == 0 && ab.s("weight") == x.s("weight");
    heads[k] = g;
    any = true;
    all_ok = all_ok && g.ok;
  }
  const bool can = any && all_ok;
  fused_head = opt.fused_head < 0 ? (can && context <= 2048) : (opt.fused_head != 0 && can);
  if (fused_head)
    for (auto& kv : heads) {
      head_members.insert(kv.second.qb);
      head_members.insert(kv.second.write);
      head_members.insert(kv.second.absorb);
    }
  // ---- dispatcher: the grouped-query attention group as packed projection + rotate-and-append + attention ----
  for (uint32_t k = 0; k < ins.size(); ++k) {
    const Ins& x = ins[k];
    if (x.op != "paged_attention") continue;
    if (x.has("window") && x.i("window") > 0 && (uint32_t)x.i("window") < context) fail(ErrorKind::NotImplemented, "device program: windowed grouped-query attention has no kernel");
    GqaGroup g;
    g.rq = x.in.at(0);
    g.cache = x.in.at(1);
    if (ins[g.cache].op != "kv_cache_append" || ins[g.rq].op != "rotary_prefix") continue;
    g.rk = ins[g.cache].in.at(0);
    g.lv = ins[g.cache].in.at(1);
    if (ins[g.rk].op != "rotary_prefix" || ins[g.lv].op != "linear") continue;
    g.lq = ins[g.rq].in.at(0);
    g.lk = ins[g.rk].in.at(0);
    const Ins *L[3] = {&ins[g.lq], &ins[g.lk], &ins[g.lv]};
    bool ok = true;
    for (const Ins* l : L) ok = ok && l->op == "linear" && !l->has("paired_weight") && !l->has("activation") && l->in.at(0) == L[0]->in.at(0);
    for (const char* f : {"norm_weight", "norm_eps", "norm_optional"})
      for (const Ins* l : L) ok = ok && l->has(f) == L[0]->has(f) && (!l->has(f) || l->s(f) == L[0]->s(f));
    const Ins &rq = ins[g.rq], &rk = ins[g.rk];
    for (const char* f : {"head_dim", "rotary_dim", "theta"}) ok = ok && rq.s(f) == rk.s(f);
    ok = ok && rq.s("head_dim") == x.s("head_dim") && only_user(g.lq, g.rq) && only_user(g.lk, g.rk) && only_user(g.lv, g.cache) && only_user(g.rq, k) &&
         only_user(g.rk, g.cache) && only_user(g.cache, k);
    if (!ok) continue;
    g.x = L[0]->in.at(0);
    g.k = (int)dims(L[0]->s("weight")).at(1);
    for (const Ins* l : L) g.rows += (int)dims(l->s("weight")).at(0);
    dmalloc(&g.packed, (uint64_t)g.rows * g.k * 2, "packed q|k|v operand");
    owned.push_back(g.packed);
    uint64_t at = 0;
    for (const Ins* l : L) {
      const uint64_t bytes = dims(l->s("weight"))[0] * (uint64_t)g.k * 2;
      cu(cudaMemcpy((char*)g.packed + at, P(l->s("weight")), bytes, cudaMemcpyDeviceToDevice), "packing q|k|v");
      at += bytes;
    }
    gqa_ld = std::max<long>(gqa_ld, g.rows);
    for (uint32_t m : {g.lq, g.rq, g.lk, g.rk, g.lv, g.cache}) gqa_members.insert(m);
    gqa[k] = g;
  }
  if (gqa_ld) {
    dmalloc((void**)&gqa_qkv, (uint64_t)rows * gqa_ld * 2, "q|k|v rows of a step");
    owned.push_back(gqa_qkv);
  }
  if (kv_pack_ld) {
    dmalloc((void**)&kv_pack, (uint64_t)rows * kv_pack_ld * 2, "k|v rows of a step");
    owned.push_back(kv_pack);
  }
  allocations_at_ready = g_device_allocations;
  ready = true;
}

// Enqueue the program for T rows on `stream` (eagerly or under capture).
void DeviceProgram::Impl::dispatch(int T) {
  void* st = stream;
  uint32_t* status = fab.status;
  const bool head = fused_head && T <= 2;
  uint64_t count = 0;
  auto V = [&](uint32_t k) -> const Val& { return val[k]; };
  for (uint32_t k = 0; k < ins.size(); ++k) {
    const Ins& x = ins[k];
    if (x.op == "view" || aliased.count(k)) continue;
    if (head && head_members.count(k)) continue;
    if (gqa_members.count(k)) continue;
    const void* norm_w = x.has("norm_weight") ? (x.has("norm_optional") ? P_optional(x.s("norm_weight")) : P(x.s("norm_weight"))) : nullptr;
    const float eps = x.f("norm_eps", 1e-5f);
    ++count;
    if (head && heads.count(k)) {
      const HeadGroup& g = heads[k];
      const Ins &qb = ins[g.qb], &ab = ins[g.absorb], &wr = ins[g.write];
      const Val& qkv = V(g.qkv);
      kernel(ifab_mla_head_decode(qkv.ptr, qkv.ld, P(qb.s("norm_weight")), P(wr.s("weight")), qb.f("norm_eps", 1e-5f), ab.f("theta", 10000.f),
                                  P(qb.s("weight")), P(x.s("weight")), cache_of.at(g.write), d_positions, d_slots, d_page_table, max_pages, page_tokens,
                                  num_pages, nullptr, 0, x.i("window"), 1.f / std::sqrt((float)x.i("scale_dim")), T, x.i("heads"), ins[qb.in[0]].i("width"),
                                  ab.i("nope"), x.i("value"), V(k).ptr, V(k).ld, status, st),
             x.name);
    } else if (gqa.count(k)) {
      const GqaGroup& g = gqa[k];
      const Ins& lq = ins[g.lq];
      const int hd = x.i("head_dim"), H = x.i("heads"), KVH = x.i("kv_heads");
      const Val& in = V(g.x);
      const void* nw = lq.has("norm_weight") ? (lq.has("norm_optional") ? P_optional(lq.s("norm_weight")) : P(lq.s("norm_weight"))) : nullptr;
      char* kv = (char*)cache_of.at(g.cache);
      char* vpages = kv + (uint64_t)num_pages * page_tokens * KVH * hd * 2;
      const uint64_t scratch = (uint64_t)T * H * max_splits * (hd + 2) * 4;
      count += 3;                                                      // projection, rotate-and-append, split, merge
      kernel(ifab_gemv_bf16(in.ptr, in.ld, g.packed, nw, lq.f("norm_eps", 1e-5f), 0, nullptr, 0, gqa_qkv, gqa_ld, 0, T, g.rows, g.k, 0, st), lq.name);
      kernel(ifab_gqa_rope_kv_write(gqa_qkv, gqa_ld, d_positions, d_slots, d_page_table, max_pages, page_tokens, kv, vpages, num_pages, T, H, KVH, hd,
                                    ins[g.rq].i("rotary_dim"), ins[g.rq].f("theta", 10000.f), status, st),
             ins[g.cache].name);
      kernel(ifab_gqa_decode_attention(gqa_qkv, gqa_ld, kv, vpages, d_positions, d_slots, d_page_table, max_pages, page_tokens, num_pages, x.f("scale", 1.f), T, H,
                                       KVH, hd, kps, max_splits, (float*)workspace(scratch), scratch, V(k).ptr, V(k).ld, status, st),
             x.name);
    } else if (x.op == "index_cache_append") {
      const Val& key = V(x.in.at(0));
      auto sc = index_scales.find(k);
      if (sc != index_scales.end())
        kernel(ifab_index_cache_append_q8(key.ptr, key.ld, d_positions, d_slots, d_page_table, max_pages, page_tokens, num_pages, cache_of.at(k), sc->second, T,
                                          (int)x.width, status, st),
               x.name);
      else
        kernel(ifab_index_cache_append(key.ptr, key.ld, d_positions, d_slots, d_page_table, max_pages, page_tokens, num_pages, cache_of.at(k), T, (int)x.width,
                                       status, st),
               x.name);
    } else if (x.op == "sparse_index") {
      const Val &q = V(x.in.at(0)), &g = V(x.in.at(1));
      const uint32_t keys = x.in.at(2);
      if (q.ld != (long)ins[x.in[0]].width) fail(ErrorKind::NotImplemented, "device program: the index query must be a whole instruction result");
      auto sc = index_scales.find(keys);
      ++count;                                                         // score + select
      kernel(ifab_sparse_index_general(q.ptr, g.ptr, g.ld, g.esize == 2 ? 1 : 0, cache_of.at(keys), sc == index_scales.end() ? nullptr : sc->second, d_positions,
                                       d_slots, d_page_table, max_pages, page_tokens, num_pages, index_scores, (int)context, T, x.i("heads"), x.i("head_dim"),
                                       x.i("topk"), (int32_t*)V(k).ptr, status, st),
             x.name);
    } else if (x.op == "repeat") {
      const Val& in = V(x.in.at(0));
      const int n = x.i("count"), w = (int)ins[x.in[0]].width;
      for (int c = 0; c < n; ++c)
        cu(cudaMemcpy2DAsync(V(k).ptr + (size_t)c * w * 2, (size_t)V(k).ld * 2, in.ptr, (size_t)in.ld * 2, (size_t)w * 2, T, cudaMemcpyDeviceToDevice,
                             (cudaStream_t)st),
           "repeat");
      count += n - 1;
    } else if (x.op == "optional_norm") {
      const Val& in = V(x.in.at(0));
      const void* g = P_optional(x.s("weight"));
      if (g) kernel(ifab_rmsnorm_bf16(in.ptr, in.ld, g, V(k).ptr, V(k).ld, T, (int)x.width, x.f("eps", 1e-5f), 0, st), x.name);
      else cu(cudaMemcpy2DAsync(V(k).ptr, (size_t)V(k).ld * 2, in.ptr, (size_t)in.ld * 2, (size_t)x.width * 2, T, cudaMemcpyDeviceToDevice, (cudaStream_t)st), "pass-through");
    } else if (x.op == "mhc_pre" || x.op == "mhc_merge") {
      const HcAux& h = hc_of.at(k);
      const Val& in = V(x.in.at(0));
      const std::string b = x.s("weight");
      if (in.ld != (long)ins[x.in[0]].width) fail(ErrorKind::NotImplemented, "device program: the streams of a hyper-connection must be whole rows");
      kernel(ifab_mhc_pre_ticketed(in.ptr, (const float*)P(b + ".phi"), (const float*)P(b + ".gamma"), (const float*)P(b + ".alpha"), (const float*)P(b + ".beta"),
                                   V(k).ptr, h.post, h.comb, T, h.S, (int)x.width, x.i("sinkhorn"), x.f("eps", 1e-6f), ticket + 8, st),
             x.name);
    } else if (x.op == "mhc_post") {
      const HcAux& h = hc_of.at(x.in.at(0));
      const Val &br = V(x.in.at(1)), &X = V(x.in.at(2));
      const int W = (int)x.width / h.S;
      if (norm_w)
        kernel(ifab_mhc_post_norm(X.ptr, br.ptr, br.ld, norm_w, eps, h.post, h.comb, V(k).ptr, T, h.S, W, st), x.name);
      else
        kernel(ifab_mhc_post(X.ptr, br.ptr, br.ld, h.post, h.comb, V(k).ptr, T, h.S, W, st), x.name);
    } else if (x.op == "mome") {
      const Val& in = V(x.in.at(0));
      kernel(ifab_mome(in.ptr, in.ld, (const float*)P(x.s("weight")), conv_state.at(k).first, d_positions, d_slots, V(k).ptr, V(k).ld, T, (int)x.width, x.i("taps"), 0,
                       st),
             x.name);
    } else if (x.op == "swiglu") {
      if (x.in.size() == 2) {
        const Val &g = V(x.in[0]), &u = V(x.in[1]);
        kernel(ifab_swiglu_pair(g.ptr, g.ld, u.ptr, u.ld, V(k).ptr, V(k).ld, T, (int)x.width, st), x.name);
      } else {
        const Val& gu = V(x.in.at(0));
        kernel(ifab_swiglu_pair(gu.ptr, gu.ld, gu.ptr + (size_t)x.width * 2, gu.ld, V(k).ptr, V(k).ld, T, (int)x.width, st), x.name);
      }
    } else if (x.op == "rotary_prefix") {
      const Val& in = V(x.in.at(0));
      kernel(ifab_rope_prefix(in.ptr, in.ld, d_positions, V(k).ptr, V(k).ld, T, x.i("heads"), x.i("head_dim"), x.i("rotary_dim"), x.f("theta", 10000.f), st), x.name);
    } else if (x.op == "add") {
      const Val &a = V(x.in.at(0)), &b = V(x.in.at(1));
      if (x.dtype != "bf16" || a.esize != 2 || b.esize != 2) fail(ErrorKind::NotImplemented, "device program: add over f32 rows has no kernel");
      kernel(ifab_add_rows(a.ptr, a.ld, b.ptr, b.ld, V(k).ptr, V(k).ld, T, (int)x.width, st), x.name);
    } else if (x.op == "kv_cache_append") {
      // outside a group: k and v rows side by side in the pack buffer, then the append kernel with no query heads and no rotation
      const Val &kr = V(x.in.at(0)), &vr = V(x.in.at(1));
      const int hd = x.i("head_dim"), kvl = (int)x.width / (2 * hd);
      const size_t half = (size_t)kvl * hd * 2;
      cu(cudaMemcpy2DAsync(kv_pack, kv_pack_ld * 2, kr.ptr, kr.ld * 2, half, T, cudaMemcpyDeviceToDevice, (cudaStream_t)st), "k rows into the pack buffer");
      cu(cudaMemcpy2DAsync(kv_pack + half, kv_pack_ld * 2, vr.ptr, vr.ld * 2, half, T, cudaMemcpyDeviceToDevice, (cudaStream_t)st), "v rows into the pack buffer");
      char* kv = (char*)cache_of.at(k);
      count += 2;
      kernel(ifab_gqa_rope_kv_write(kv_pack, kv_pack_ld, d_positions, d_slots, d_page_table, max_pages, page_tokens, kv,
                                    kv + (uint64_t)num_pages * page_tokens * kvl * hd * 2, num_pages, T, 0, kvl, hd, 0, 2.f, status, st),
             x.name);
    } else if (x.op == "paged_attention") {
      const int hd = x.i("head_dim"), H = x.i("heads"), KVH = x.i("kv_heads");
      char* kv = (char*)cache_of.at(x.in.at(1));
      const uint64_t scratch = (uint64_t)T * H * max_splits * (hd + 2) * 4;
      const Val& q = V(x.in.at(0));
      ++count;
      kernel(ifab_gqa_decode_attention(q.ptr, q.ld, kv, kv + (uint64_t)num_pages * page_tokens * KVH * hd * 2, d_positions, d_slots, d_page_table, max_pages,
                                       page_tokens, num_pages, x.f("scale", 1.f), T, H, KVH, hd, kps, max_splits, (float*)workspace(scratch), scratch, V(k).ptr,
                                       V(k).ld, status, st),
             x.name);
    } else if (x.op == "embedding") {
      kernel(ifab_embedding_bf16(d_tokens, P(x.s("weight")), V(k).ptr, T, (int)x.width, x.i("vocab"), status, st), x.name);
    } else if (x.op == "linear") {
      const std::string pname = x.s("weight") + (x.has("paired_weight") ? "|" + x.s("paired_weight") : "");
      const bool swiglu = x.has("activation") && x.s("activation") == "swiglu";
      const auto& d = dims(pname);
      const Val& in = V(x.in.at(0));
      kernel(ifab_gemv_bf16(in.ptr, in.ld, P(pname), norm_w, eps, 0, nullptr, 0, V(k).ptr, V(k).ld, 0, T, (int)(swiglu ? d[0] / 2 : d[0]), (int)d[1],
                            swiglu ? 1 : 0, st),
             x.name);
    } else if (x.op == "linear_allreduce") {
      const auto& d = dims(x.s("weight"));
      const Val& in = V(x.in.at(0));
      const Val* res = x.in.size() > 1 ? &V(x.in[1]) : nullptr;
      kernel(ifab_gemv_allreduce_bf16(in.ptr, in.ld, P(x.s("weight")), res ? res->ptr : nullptr, res ? res->ld : 0, V(k).ptr, V(k).ld, nullptr, T, (int)d[0],
                                      (int)d[1], &fab, st),
             x.name);
    } else if (x.op == "norm") {
      const Val& in = V(x.in.at(0));
      kernel(ifab_rmsnorm_bf16(in.ptr, in.ld, P(x.s("weight")), V(k).ptr, V(k).ld, T, (int)x.width, x.f("eps", 1e-5f), 0, st), x.name);
    } else if (x.op == "mla_kv_write") {
      const Val &lat = V(x.in.at(0)), &kr = V(x.in.at(1));
      const int latent = (int)ins[x.in[0]].width, rope = (int)ins[x.in[1]].width;
      if (x.in.size() > 2) sinks_of[k] = sink_rows.at(x.in[2]);
      if (packed.count(k)) {
        if (kr.ptr != lat.ptr + (long)latent * 2 || kr.ld != lat.ld)
          kernel(ifab_mla_kv_write_q8_split(lat.ptr, lat.ld, kr.ptr, kr.ld, P(x.s("weight")), x.f("eps", 1e-5f), x.f("theta", 10000.f), d_positions, d_slots,
                                            d_page_table, max_pages, page_tokens, cache_of.at(k), num_pages, T, status, st),
                 x.name);
        else
          kernel(ifab_mla_kv_write_q8(lat.ptr, lat.ld, P(x.s("weight")), x.f("eps", 1e-5f), x.f("theta", 10000.f), d_positions, d_slots, d_page_table,
                                      max_pages, page_tokens, cache_of.at(k), num_pages, T, status, st),
                 x.name);
      } else if (kr.ptr != lat.ptr + (long)latent * 2 || kr.ld != lat.ld)
        // e.g. a convolved latent and the raw rotary columns of the projection: the kernel reads them where they are
        kernel(ifab_mla_kv_write_split(lat.ptr, lat.ld, kr.ptr, kr.ld, P(x.s("weight")), x.f("eps", 1e-5f), x.f("theta", 10000.f), d_positions, d_slots,
                                       d_page_table, max_pages, page_tokens, cache_of.at(k), num_pages, T, latent, rope, status, st),
               x.name);
      else
        kernel(ifab_mla_kv_write(lat.ptr, lat.ld, P(x.s("weight")), x.f("eps", 1e-5f), x.f("theta", 10000.f), d_positions, d_slots, d_page_table, max_pages,
                                 page_tokens, cache_of.at(k), num_pages, T, latent, rope, status, st),
               x.name);
    } else if (x.op == "mla_q_absorb") {
      const Val& q = V(x.in.at(0));
      const int nope = x.i("nope"), vdim = x.has("value") ? x.i("value") : nope;
      kernel(ifab_mla_q_absorb(q.ptr, q.ld, P(x.s("weight")), x.f("theta", 10000.f), d_positions, V(k).ptr, T, x.i("heads"), nope, x.i("rope"), x.i("latent"),
                               vdim, st),
             x.name);
    } else if (x.op == "mla_attention") {
      const int H = x.i("heads"), latent = x.i("latent"), vdim = x.i("value"), nope = x.has("nope") ? x.i("nope") : vdim;
      const uint64_t scratch = (uint64_t)T * H * max_splits * (latent + 2) * 4;
      ++count;                                                         // split + merge
      auto sk = sinks_of.find(x.in.at(1));
      const int32_t* picked = x.in.size() > 2 ? (const int32_t*)V(x.in[2]).ptr : nullptr;
      kernel(ifab_mla_decode_attention_indexed(V(x.in.at(0)).ptr, cache_of.at(x.in.at(1)), d_positions, d_slots, d_page_table, max_pages, page_tokens, num_pages,
                                               sk == sinks_of.end() ? nullptr : sk->second.first, sk == sinks_of.end() ? 0 : sk->second.second, x.i("window"),
                                               1.f / std::sqrt((float)x.i("scale_dim")), T, H, latent, packed.count(x.in[1]) ? -64 : 64, kps, max_splits,
                                               (float*)workspace(scratch), scratch, P(x.s("weight")), nope, vdim, V(k).ptr, V(k).ld, status, picked,
                                               picked ? (int)ins[x.in[2]].width : 0, st),
             x.name);
    } else if (x.op == "router_topk") {
      const int E = x.i("experts"), topk = x.i("topk");
      char* raw = V(k).ptr;
      int32_t* ids = (int32_t*)raw;
      float* wts = (float*)(raw + (uint64_t)rows * topk * 4);
      float* logits = (float*)(raw + (uint64_t)rows * topk * 8);
      const Val& in = V(x.in.at(0));
      const int scoring = x.s("scoring") == "softmax" ? 0 : 1;
      const int renorm = !(x.has("renorm") && x.s("renorm") == "false");
      kernel(ifab_router_topk(in.ptr, in.ld, norm_w, eps, (const float*)P(x.s("weight")), (const float*)P_optional(x.s("weight") + ".e_score_correction_bias"),
                              logits, ids, wts, T, (int)ins[x.in[0]].width, E, topk, scoring, renorm, x.f("scale", 1.f), ticket, nullptr, 0, st),
             x.name);
    } else if (x.op == "moe_gate_up") {
      const Ins& r = ins[x.in.at(1)];
      const std::string pname = x.s("weight") + "|" + x.s("paired_weight");
      const auto& d = dims(pname);        // [experts, 2F, D]
      const void* shared = x.has("shared_weight") ? P(x.s("shared_weight") + "|" + x.s("shared_paired_weight")) : nullptr;
      const int Fs = x.has("shared_weight") ? (int)(dims(x.s("shared_weight") + "|" + x.s("shared_paired_weight"))[0] / 2) : 0;
      const Val& in = V(x.in.at(0));
      kernel(ifab_moe_gate_up_decode(in.ptr, in.ld, norm_w, eps, (const int32_t*)V(x.in[1]).ptr, T, (int)d[2], (int)(d[1] / 2), r.i("topk"), 0, (int)d[0], P(pname),
                                     shared, Fs, V(k).ptr, st),
             x.name);
    } else if (x.op == "moe_down_allreduce") {
      const Ins& r = ins[x.in.at(1)];
      const auto& d = dims(x.s("weight"));   // [experts, D, F]
      const int topk = r.i("topk");
      char* raw = V(x.in[1]).ptr;
      const void* shared = x.has("shared_weight") ? P(x.s("shared_weight")) : nullptr;
      const int Fs = x.has("shared_weight") ? (int)dims(x.s("shared_weight"))[1] : 0;
      const Val* res = x.in.size() > 2 ? &V(x.in[2]) : nullptr;
      kernel(ifab_moe_down_allreduce_decode(V(x.in[0]).ptr, (const int32_t*)raw, (const float*)(raw + (uint64_t)rows * topk * 4), T, (int)d[1], (int)d[2], topk, 0,
                                            (int)d[0], P(x.s("weight")), shared, Fs, res ? res->ptr : nullptr, res ? res->ld : 0, V(k).ptr, V(k).ld, &fab, st),
             x.name);
    } else if (x.op == "lm_head") {
      const auto& d = dims(x.s("weight"));
      const uint64_t partial = ((d[0] + 7) / 8) * 8 * 2 * 4;
      const Val& in = V(x.in.at(0));
      kernel(ifab_lm_head_argmax(in.ptr, in.ld, norm_w, eps, P(x.s("weight")), nullptr, T, (int)d[0], (int)d[1], 0, workspace(partial), partial, d_next, d_next_vals, &fab,
                                 st),
             x.name);
    } else {
      fail(ErrorKind::NotImplemented, "device program: no kernel bound for instruction '" + x.op + "' (" + x.name + ")");
    }
  }
  launches_per_step_last = count;
}

void DeviceProgram::Impl::step(const int32_t* tokens, const int32_t* positions, const int32_t* slots, int T, int32_t* out) {
  if (T < 1 || T > (int)rows) invalid("device program: a launch group holds 1.." + std::to_string(rows) + " rows");
  for (int i = 0; i < T; ++i) {
    if (tokens[i] < 0 || (uint32_t)tokens[i] >= vocab) invalid("device program: token id outside the vocabulary");
    if (positions[i] < 0 || (uint32_t)positions[i] >= context) fail(ErrorKind::Capacity, "device program: a row lies beyond the context");
    if (slots[i] < 0 || (uint32_t)slots[i] >= residents) invalid("device program: resident slot out of range");
    h_ctl[i] = tokens[i];
    h_ctl[8 + i] = positions[i];
    h_ctl[16 + i] = slots[i];
  }
  cu(cudaMemcpyAsync(d_tokens, h_ctl, 3 * 8 * sizeof(int32_t), cudaMemcpyHostToDevice, stream), "control upload");
  h2d += 3 * 8 * sizeof(int32_t);
  auto it = graphs.find(T);
  if (it != graphs.end()) {
    cu(cudaGraphLaunch(it->second, stream), "graph launch");
  } else {
    dispatch(T);                                                  // the real run of this step, and the warm-up of the capture
    if (opt.graphs) {
      cu(cudaStreamSynchronize(stream), "synchronise before capture");
      cudaGraph_t g = nullptr;
      cu(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "begin capture");
      try {
        dispatch(T);                                              // records only
      } catch (...) {
        cudaStreamEndCapture(stream, &g);
        if (g) cudaGraphDestroy(g);
        throw;
      }
      cu(cudaStreamEndCapture(stream, &g), "end capture");
      cudaGraphExec_t exec = nullptr;
      cu(cudaGraphInstantiate(&exec, g, 0), "graph instantiate");
      cudaGraphDestroy(g);
      graphs[T] = exec;
    }
  }
  launches += launches_per_step_last;
  cu(cudaMemcpyAsync(h_out, d_next, 8 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream), "token download");
  uint32_t status = 0;
  cu(cudaMemcpyAsync(&h_out[0] + 0, d_next, T * sizeof(int32_t), cudaMemcpyDeviceToHost, stream), "token download");
  cu(cudaStreamSynchronize(stream), "step synchronise");
  cu(cudaMemcpy(&status, fab.status, 4, cudaMemcpyDeviceToHost), "status read");
  d2h += T * sizeof(int32_t) + 4;
  if (status != 0) fail(ErrorKind::Backend, "device program: kernel status word = " + std::to_string(status));
  for (int i = 0; i < T; ++i) out[i] = h_out[i];
  ++steps;
}

DeviceProgram::DeviceProgram(const std::string& bundle_dir, const std::string& checkpoint_dir, const Options& opt) : p_(std::make_unique<Impl>()) {
  p_->opt = opt;
  p_->load(bundle_dir, checkpoint_dir);
}
DeviceProgram::~DeviceProgram() = default;
uint32_t DeviceProgram::context() const { return p_->context; }
uint32_t DeviceProgram::vocab() const { return p_->vocab; }
uint32_t DeviceProgram::eos() const { return p_->eos; }
uint32_t DeviceProgram::residents() const { return p_->residents; }
uint32_t DeviceProgram::max_rows() const { return p_->rows; }
const std::string& DeviceProgram::name() const { return p_->name; }
void DeviceProgram::run_rows(const int32_t* tokens, const int32_t* positions, const int32_t* slots, int rows, int32_t* next_tokens) {
  cu(cudaSetDevice(p_->opt.device), "cudaSetDevice");
  p_->step(tokens, positions, slots, rows, next_tokens);
}
void DeviceProgram::reset() {
  for (auto& c : p_->conv_state) cu(cudaMemset(c.second.first, 0, c.second.second), "convolution history clear");
  for (auto& c : p_->cache_of) cu(cudaMemset(c.second, 0, p_->cache_bytes.at(c.first)), "KV clear");
  for (auto& c : p_->index_scales) cu(cudaMemset(c.second, 0, (uint64_t)p_->num_pages * p_->page_tokens * 2), "index scales clear");
}
Json DeviceProgram::audit() const {
  Json j = Json::object();
  j.set("format", "ifab.device-program-audit.v1");
  j.set("program", p_->name);
  j.set("steps", p_->steps);
  j.set("launches", p_->launches);
  j.set("launches_per_step", p_->launches_per_step_last);
  j.set("fused_head", p_->fused_head);
  Json widths = Json::array();
  for (auto& g : p_->graphs) widths.push((int64_t)g.first);
  j.set("graph_widths", widths);
  Json arena = Json::object();
  arena.set("bytes", p_->arena_bytes);
  arena.set("workspace_bytes", p_->workspace_bytes);
  arena.set("slots", (int64_t)p_->slot_of.size());
  arena.set("planned_rows", p_->rows);
  j.set("arena", arena);
  j.set("parameter_bytes_uploaded", p_->params ? p_->params->uploaded : 0);
  j.set("h2d_bytes", p_->h2d);
  j.set("d2h_bytes", p_->d2h);
  j.set("device_allocations_after_ready", g_device_allocations - p_->allocations_at_ready);   // this executor's own cudaMalloc calls
  return j;
}

// ---- the executor as a server engine ----------------------------------------------------------------------------------------
namespace {
class DeviceResidentEngine : public serve::ResidentEngine {
 public:
  DeviceResidentEngine(const std::string& bundle, const std::string& checkpoint, const Options& opt) : p_(bundle, checkpoint, opt), next_(p_.residents(), 0) {}
  serve::EngineInfo info() const override {
    serve::EngineInfo e;
    e.model = p_.name().empty() ? "ifab-program" : p_.name();
    e.residents = p_.residents();
    e.token_budget = e.chunk = std::max<uint32_t>(8, p_.max_rows());
    e.context = p_.context();
    e.vocab = p_.vocab();
    e.eos = p_.eos();
    e.has_eos = false;
    e.greedy_only = true;
    return e;
  }
  void admit(uint32_t resident, const serve::SamplingParams& s, uint32_t reserve) override {
    if (!s.greedy()) invalid("the device program engine samples greedily only");
    if (reserve > p_.context()) fail(ErrorKind::Capacity, "request does not fit the sequence slot");
    next_.at(resident) = 0;
  }
  std::vector<uint32_t> step(const paging::SequenceBatch& batch) override {
    // rows in slice order, cut into launch groups of at most max_rows; the token of a slice is that of its last row
    struct Row { int32_t token, position, slot; int slice; };
    std::vector<Row> rows;
    size_t off = 0;
    for (size_t s = 0; s < batch.slices.size(); ++s) {
      const auto& sl = batch.slices[s];
      if (sl.position != next_.at(sl.resident)) invalid("device program engine: resident " + std::to_string(sl.resident) + " stands at position " + std::to_string(next_[sl.resident]));
      for (uint32_t i = 0; i < sl.token_count; ++i)
        rows.push_back({batch.tokens[off + i], (int32_t)(sl.position + i), (int32_t)sl.resident, i + 1 == sl.token_count ? (int)s : -1});
      off += sl.token_count;
      next_[sl.resident] = sl.position + sl.token_count;
    }
    std::vector<uint32_t> out(batch.slices.size(), 0);
    const int G = (int)p_.max_rows();
    int32_t t[8], p[8], sl[8], nx[8];
    for (size_t r0 = 0; r0 < rows.size(); r0 += (size_t)G) {
      const int n = (int)std::min<size_t>((size_t)G, rows.size() - r0);
      for (int i = 0; i < n; ++i) {
        t[i] = rows[r0 + i].token;
        p[i] = rows[r0 + i].position;
        sl[i] = rows[r0 + i].slot;
      }
      p_.run_rows(t, p, sl, n, nx);
      for (int i = 0; i < n; ++i)
        if (rows[r0 + i].slice >= 0) out[(size_t)rows[r0 + i].slice] = (uint32_t)nx[i];
    }
    return out;
  }
  void release(uint32_t resident) override { next_.at(resident) = 0; }
  Json audit() override { return p_.audit(); }

 private:
  DeviceProgram p_;
  std::vector<uint32_t> next_;
};
}  // namespace

std::shared_ptr<serve::ResidentEngine> make_device_program_engine(const std::string& bundle, const std::string& checkpoint, const Options& opt) {
  return std::make_shared<DeviceResidentEngine>(bundle, checkpoint, opt);
}

}  // namespace ifab::device

// ---- C ABI --------------------------------------------------------------------------------------------------------------------
namespace {
thread_local std::string g_device_error;
template <typename F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const ifab::Error& e) {
    g_device_error = e.what();
    return 1 + (int)e.kind();
  } catch (const std::exception& e) {
    g_device_error = e.what();
    return 100;
  }
}
ifab::device::DeviceProgram* D(void* e) {
  if (!e) ifab::invalid("device program: null handle");
  return static_cast<ifab::device::DeviceProgram*>(e);
}
}  // namespace

extern "C" {
const char* ifab_device_program_error(void) { return g_device_error.c_str(); }
int ifab_device_program_open(const char* bundle, const char* checkpoint, int device, uint32_t residents, void** out) {
  return guarded([&] {
    ifab::device::Options o;
    o.device = device;
    o.residents = residents;
    *out = new ifab::device::DeviceProgram(bundle, checkpoint, o);
  });
}
int ifab_device_program_info(void* e, uint32_t* context, uint32_t* vocabulary, uint32_t* eos, uint32_t* residents, uint32_t* max_rows) {
  return guarded([&] {
    auto* p = D(e);
    if (context) *context = p->context();
    if (vocabulary) *vocabulary = p->vocab();
    if (eos) *eos = p->eos();
    if (residents) *residents = p->residents();
    if (max_rows) *max_rows = p->max_rows();
  });
}
int ifab_device_program_rows(void* e, const int32_t* tokens, const int32_t* positions, const int32_t* slots, uint32_t rows, int32_t* next_tokens) {
  return guarded([&] { D(e)->run_rows(tokens, positions, slots, (int)rows, next_tokens); });
}
int ifab_device_program_reset(void* e) {
  return guarded([&] { D(e)->reset(); });
}
int ifab_device_program_audit(void* e, char* out_json, uint64_t capacity) {
  return guarded([&] {
    const std::string s = D(e)->audit().dump();
    if (s.size() + 1 > capacity) ifab::fail(ifab::ErrorKind::Capacity, "device program: audit buffer too small");
    std::memcpy(out_json, s.c_str(), s.size() + 1);
  });
}
int ifab_device_program_close(void* e) {
  return guarded([&] { delete D(e); });
}
// For the server, which loads this library on demand: the executor as a ResidentEngine (a C++ object of the host core's type;
// both sides are built from the same headers). Returns null and leaves the reason in ifab_device_program_error().
void* ifab_device_program_engine_new(const char* bundle, const char* checkpoint, int device, uint32_t residents, uint32_t context) {
  void* out = nullptr;
  guarded([&] {
    ifab::device::Options o;
    o.device = device;
    o.residents = residents;
    o.context = context;
    out = new std::shared_ptr<ifab::serve::ResidentEngine>(ifab::device::make_device_program_engine(bundle, checkpoint, o));
  });
  return out;
}
}
