// Checkpoint-bound compile path of the hybrid decoder family (gated-delta layers + full-attention layers, the
// `qwen35_text_v1` contract): checkpoint metadata inspection, the typed mathematical plan, and its lowering to per-layer
// weight bindings.
//
//   inspect   reads config.json, model.safetensors.index.json and the safetensors HEADERS of every shard (never tensor
//             data): file names must be plain names inside the directory, header sizes and tensor ranges are bounds- and
//             overlap-checked and must tile the data section exactly, index and headers must agree, every tensor the
//             model's shape calls for must be present with the right dtype and shape; vision / multi-token-prediction
//             tensors are counted and left out; anything else is an error
//   compile   Spec + Checkpoint -> Plan: a single-assignment graph of typed nodes over symbolic dimensions (tokens,
//             requests, pages) with explicit states (paged keys / values, delta key-value state, conv history) and the
//             numerics of every operator spelled out in its attributes; validated (use before definition, duplicate
//             outputs, shape / dtype rule of every operator, every checkpoint weight bound exactly once where the contract says)
//   lower     Plan -> Program: per-layer weight bindings with the transform each needs (zero-centred RMS gains are stored
//             as w and used as 1 + w in f32), for a declared context bucket and a batch of 1..64 lanes
// The reference pins this path to one model's constants (crates/inferfabric-compiler/src/checkpoint.rs:89-188,
// bound.rs:200-240); here the dimensions come from the document's Spec and the checkpoint's config must agree with them.
// Reference: checkpoint.rs:190-334, bound.rs:42-518 and 520-830, lower.rs:9-134.
#pragma once
#include "initplan.h"
#include "rankplan.h"

namespace ifab::hybrid {

constexpr const char* kPrefix = "model.language_model.";
constexpr uint32_t kMaxModelLen = 262144;

struct Weight {
  std::string shard;               // file name
  init::DType dtype = init::DType::Bf16;
  std::vector<uint64_t> shape;
  uint64_t offset = 0;             // absolute file offset (8-byte length + header included)
  uint64_t bytes = 0;
};
struct Shard {
  uint64_t bytes = 0;
  std::string header_sha256;
};
struct Checkpoint {
  std::string config_sha256, index_sha256;
  std::map<std::string, Shard> shards;
  std::map<std::string, Weight> weights;      // the text model's tensors only
  std::map<std::string, uint64_t> excluded;   // "vision" / "mtp" -> tensor count
  std::string metadata_sha256;                // over all of the above; payload bytes are not covered
  Json to_json() const;
};

using Schema = std::map<std::string, std::pair<init::DType, std::vector<uint64_t>>>;
Schema schema(const rankplan::Model& m);
void validate_config(const Json& config, const rankplan::Model& m);
Checkpoint inspect(const std::string& directory, const rankplan::Model& m);

// ---- typed plan ------------------------------------------------------------------------------------
struct Dim {
  enum class Kind { Tokens, Requests, RequestBoundaries, Pages, Fixed } kind = Kind::Fixed;
  uint64_t n = 0;
  bool operator==(const Dim& o) const { return kind == o.kind && (kind != Kind::Fixed || n == o.n); }
  static Dim fixed(uint64_t v) { return {Kind::Fixed, v}; }
};
enum class Scalar { Bf16, Fp32, I64 };
struct Tensor {
  std::string name;
  std::vector<Dim> shape;
  Scalar dtype = Scalar::Bf16;
};
enum class StateKind { PagedKeys, PagedValues, DeltaKeyValue, ConvPreviousInputs };
struct State {
  Tensor tensor;
  StateKind kind;
  bool initially_zero = false;
};
enum class Op {
  Embedding, Linear, ZeroCenteredRms, Reshape, Split, TextRope, PagedAttention, Sigmoid, Silu, Multiply, Add, CausalConvSilu,
  L2Norm, DeltaDecay, DeltaRecurrence, GatedRms, SelectFrontier
};
const char* op_name(Op op);
struct Node {
  Op op = Op::Add;
  std::vector<std::string> inputs;
  std::vector<Tensor> outputs;
  std::map<std::string, std::string> attrs;    // weights, state names and the numerics contract of the operator, as text
};
struct Plan {
  std::string format = "inferfabric.typed-plan.v1";
  bool executable = false;                      // a mathematical plan: kernels are chosen by the lowering, not here
  std::string contract = "qwen35_text_v1";
  std::string key;                              // sha256 of the plan's JSON without the key
  rankplan::Spec spec;
  Checkpoint checkpoint;
  std::vector<Tensor> inputs;
  std::vector<State> states;
  std::vector<Node> nodes;
  std::string output;
  uint64_t text_weight_bytes = 0, recurrent_and_conv_bytes_per_request = 0, kv_bytes_per_page = 0;
  Json to_json() const;
};
Plan compile(const rankplan::Spec& spec, const Checkpoint& checkpoint);
// A self-contained HTML page of a typed plan document (the JSON `Plan::to_json` writes): model facts, states, and the operators
// grouped by layer with their shapes, weights and numerics attributes. Refuses documents of another format.
// Reference: crates/inferfabric-compiler/src/model_inspect.rs behind `explain-model`.
std::string html_view(const Json& typed_plan);
void validate(const Plan& plan);

// ---- lowering ----------------------------------------------------------------------------------------
enum class Transform { Identity, OnePlusFp32 };
struct Binding {
  std::string name;
  Transform transform = Transform::Identity;
};
struct Block {
  uint32_t layer = 0;
  rankplan::Layer kind = rankplan::Layer::Full;
  std::vector<Binding> bindings;
};
struct Program {
  std::string key, source_key;
  std::vector<Block> blocks;
  std::string embedding;
  Binding final_norm;
  uint32_t batch = 1, context = 0, page_tokens = 0;
  Json to_json() const;
};
// Only the canonical plan of (spec, checkpoint) lowers: an edited node list is refused.
Program lower_batch(const Plan& plan, uint32_t context, uint32_t batch);
inline Program lower(const Plan& plan, uint32_t context) { return lower_batch(plan, context, 1); }
Plan specialize_context(const Plan& plan, uint32_t context);

}  // namespace ifab::hybrid
