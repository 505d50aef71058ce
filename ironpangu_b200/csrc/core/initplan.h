// Per-rank weight initialization plans and the safetensors checkpoint reader.
//
// The planner walks the physical program, asks for every weight by its scoped name and emits, for
// each rank, a list of device parameters plus LoadSlice instructions: row shards (tp_rows) are one
// contiguous byte range, K shards (tp_columns) are strided source rows, expert weights keep only the
// rank's experts, paired projections are packed into one parameter. Plans are metadata only; the
// executor streams bytes from the checkpoint through a bounded staging buffer into a DeviceMemory.
// Reference: crates/inferfabric-compiler/src/token.rs:87-335 (planner), initialization.rs:8-49
// (IFINIT01), native/src/initialization_plan.cpp:66-278 (reader + executor).
#pragma once
#include <functional>

#include "program.h"

namespace ifab::init {

enum class DType : uint32_t { I8 = 1, Bf16 = 2, F32 = 3, F8E4M3 = 4 };
size_t dtype_bytes(DType d);
const char* dtype_name(DType d);

struct Parameter {
  uint32_t id = 0;
  std::string name;          // device-side name (the instruction's weight attribute)
  DType dtype = DType::Bf16;
  std::vector<uint64_t> dims;
  uint64_t bytes() const;
};

// Append `bytes` (after conversion) to parameter `dest`. tag 1 = contiguous range, tag 2 = strided
// rows (`row_bytes` taken every `stride_bytes`, starting at `offset`, until `bytes` source bytes).
// `shard` is the checkpoint FILE the bytes come from and `offset` an absolute offset in that file (the
// safetensors header included), as in the reference's LoadSlice (crates/inferfabric-ir/src/initialization.rs:
// 52-66): a plan is executable with nothing but the shard files. `tensor` names the checkpoint tensor for
// diagnostics and the JSON view; it is not part of the binary form.
struct LoadSlice {
  uint32_t tag = 1;
  uint32_t dest = 0;
  std::string shard;         // file name inside the checkpoint directory
  uint64_t offset = 0;       // absolute byte offset inside that file
  uint64_t bytes = 0;        // source bytes to move
  DType src_dtype = DType::Bf16;
  uint64_t row_bytes = 0, stride_bytes = 0;
  std::string tensor;        // informational: the checkpoint tensor the range lies in
};

struct Plan {
  uint32_t rank = 0, device = 0;
  std::string provenance;    // sha256 of the checkpoint metadata the plan was made against
  std::vector<Parameter> parameters;
  std::vector<LoadSlice> loads;

  // IFINIT01 when the plan has the reference's form (exactly one load per parameter, in parameter order, dtypes 1-3):
  // byte-for-byte what the reference's encoder writes for the same plan. Otherwise IFINIT02: the same layout, but
  // several loads may append to one parameter (expert stacks, packed pairs) and dtype 4 (fp8 e4m3) may appear.
  std::string encode() const;
  bool reference_form() const;
  static Plan decode(std::string_view bytes);
  Json to_json() const;
  uint64_t device_bytes() const;
};

// ---- checkpoint metadata (safetensors) -------------------------------------------------------------
struct TensorInfo {
  std::string name, file;
  DType dtype = DType::Bf16;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;   // byte range inside the file's data section
  uint64_t data_start = 0;       // file offset of the data section
  uint64_t file_offset() const { return data_start + begin; }
};
struct Checkpoint {
  std::string dir;
  std::map<std::string, TensorInfo> tensors;
  std::string fingerprint;       // sha256 over the sorted metadata

  // Parse every *.safetensors header under `dir` (bounds, overlap and dtype checks; no tensor data read).
  static Checkpoint inspect(const std::string& dir);
  // Metadata-only checkpoint for planning without files (name -> shape, all bf16 unless noted).
  static Checkpoint synthetic(const std::map<std::string, std::pair<DType, std::vector<uint64_t>>>& shapes);
  const TensorInfo& need(const std::string& name) const;
  bool has(const std::string& name) const { return tensors.count(name) != 0; }
};
// Write one safetensors file (used by tests and the weight synthesizer).
void write_safetensors(const std::string& path, const std::vector<std::pair<TensorInfo, std::string>>& tensors);

// Shapes of every checkpoint tensor the program needs (unsharded), derived from the program alone.
std::map<std::string, std::pair<DType, std::vector<uint64_t>>> required_tensors(const program::Program& p);

// One plan per rank. `ckpt` supplies shapes/dtypes; missing or mis-shaped tensors are errors
// (except weights of `norm_optional` instructions, which are skipped when absent).
std::vector<Plan> plan_all(const program::Program& p, const Checkpoint& ckpt);

// ---- execution -----------------------------------------------------------------------------------
class DeviceMemory {
 public:
  virtual ~DeviceMemory() = default;
  virtual void allocate(const Parameter& p) = 0;
  virtual void write(uint32_t param, uint64_t offset, const void* data, uint64_t bytes) = 0;
  virtual void read(uint32_t param, uint64_t offset, void* out, uint64_t bytes) { (void)param; (void)offset; (void)out; (void)bytes; fail(ErrorKind::NotImplemented, "read-back not supported"); }
};
class HostMemory : public DeviceMemory {
 public:
  void allocate(const Parameter& p) override { store[p.id].assign(p.bytes(), '\0'); }
  void write(uint32_t param, uint64_t offset, const void* data, uint64_t bytes) override;
  void read(uint32_t param, uint64_t offset, void* out, uint64_t bytes) override;
  std::map<uint32_t, std::string> store;
};
struct ExecuteOptions {
  size_t staging_bytes = 4 << 20;
  bool verify_upload = false;
};
// Stream the plan's slices from `ckpt` into `mem`. Returns the number of bytes written.
uint64_t execute(const Plan& plan, const Checkpoint& ckpt, DeviceMemory& mem, const ExecuteOptions& opt = {});

}  // namespace ifab::init
