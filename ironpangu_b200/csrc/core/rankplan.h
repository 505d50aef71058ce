// Model/mesh vocabulary and the structural rank-plan compiler.
//
// A Spec names a hybrid decoder (full-attention and gated-delta layers) and two meshes (prefill,
// decode). `compile` emits, for every rank of every role, an ordered list of kernel, communication
// and fence instructions that makes the distribution strategy explicit:
//   TP  column-parallel in-projections, row-parallel out-projections + AllReduce
//   SP  AllGather(tokens) before attention / ReduceScatter(tokens) after the row-parallel projection
//   CP  causal ring traversal of KV shards: Send/Receive per step + online-softmax merge kernel;
//       gated-delta layers hand their recurrent state to the next context rank in order
//   PD  prefill ranks end with a page transfer to the decode ranks
// Plans are backend-neutral (a mock backend executes them in tests); the artifact is content
// addressed and cached on disk. Reference: crates/inferfabric-model/src/lib.rs:31-157,
// crates/inferfabric-ir/src/lib.rs:8-93, crates/inferfabric-compiler/src/lib.rs:36-317.
#pragma once
#include "base.h"

namespace ifab::rankplan {

enum class Layer { Full, Delta };
enum class Role { Prefill, Decode };
const char* role_name(Role r);

struct Mesh {
  uint32_t tp = 1, cp = 1;
  bool sp = false;
  uint32_t ranks() const { return tp * cp; }
};
struct Model {
  std::string name;
  uint32_t hidden = 0, intermediate = 0, vocab = 0, query_heads = 0, kv_heads = 0, head_dim = 0;
  uint32_t delta_heads = 0, delta_dim = 0, conv_width = 0;
  std::vector<Layer> layers;
};
struct Spec {
  Model model;
  Mesh prefill, decode;
  uint32_t page_tokens = 16, token_budget = 1024;
  std::vector<uint32_t> batch_buckets{1}, context_buckets{512};
  void validate() const;
  uint32_t max_context() const { return context_buckets.empty() ? 0 : context_buckets.back(); }
  static Spec from_json(const Json& j);
  Json to_json() const;
};

enum class StateKind { Kv, Recurrent, Conv };
enum class CommKind { AllReduce, AllGather, ReduceScatter, Send, Receive };
const char* comm_name(CommKind k);

struct Instruction {
  enum class Kind { Kernel, Communication, Fence } kind = Kind::Kernel;
  std::string name;            // kernel name / fence label
  uint32_t layer = 0;
  CommKind comm = CommKind::AllReduce;
  uint32_t peer = 0;           // Send / Receive
  std::string group;           // "tp" | "cp" | "pd"
  uint64_t elements = 0;       // payload per token (symbolic)
};
struct Bucket { uint32_t batch = 1, context = 512; };
struct RankPlan {
  Role role = Role::Decode;
  uint32_t rank = 0, tp_rank = 0, cp_rank = 0;
  std::vector<Instruction> instructions;
  std::vector<std::pair<StateKind, uint32_t>> states;   // (kind, layer)
};
struct Artifact {
  std::string key;             // content key of (spec, target)
  std::string target;
  Spec spec;
  std::vector<RankPlan> plans;
  std::vector<Bucket> buckets;
  Json to_json() const;
  static Artifact from_json(const Json& j);
};

std::string content_key(const Spec& spec, const std::string& target);
Artifact compile(const Spec& spec, const std::string& target = "mock");
std::string encode(const Artifact& a);          // "PANGU\0\0\x01" + sha256 + JSON
Artifact decode(std::string_view bytes);
// On-disk cache: <dir>/<key>.inferfabric-bin, written atomically, verified on load.
Artifact cached(const Spec& spec, const std::string& target, const std::string& cache_dir, bool* hit = nullptr);

}  // namespace ifab::rankplan
