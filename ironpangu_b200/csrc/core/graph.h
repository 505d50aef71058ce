// Logical token graph: typed primitive nodes produced by the DSL expander, with a dimension-generic
// checker. The reference pins its checker to one model's constants
// (crates/inferfabric-authoring/src/execution.rs:105-452); here every dimension is an attribute and
// the rules are consistency rules (widths must agree, heads must divide by tp, ...).
#pragma once
#include "base.h"
#include "lang.h"

namespace ifab::graph {

enum class Kind : uint32_t { Tensor = 0, HyperConnection = 1, Routes = 2, Experts = 3, Cache = 4, Quantized = 5, IndexCache = 6, Indices = 7 };
const char* kind_name(Kind k);

struct Type {
  Kind kind = Kind::Tensor;
  uint32_t width = 0;   // columns per token (Routes: top-k; Cache: row width)
  uint32_t aux = 0;     // HyperConnection: streams; Routes: experts; Cache: rope columns / kv heads
};

struct Node {
  std::string name, op;
  std::vector<uint32_t> inputs;
  std::vector<std::pair<std::string, std::string>> attrs;  // sorted by key
  Type type;
  size_t byte = 0;
  std::vector<lang::Frame> frames;

  const std::string* attr(std::string_view key) const;
  const std::string& need(std::string_view key) const;
  int64_t int_attr(std::string_view key) const;
  double num_attr(std::string_view key) const;
  bool has(std::string_view key) const { return attr(key) != nullptr; }
};

// Parallel layout of a token program (tp == ep in {1,2,4,8}; one device per rank).
struct Parallel {
  std::string target = "b200_token_v1";
  uint32_t tp = 1, ep = 1;
  std::vector<uint32_t> devices{0};
  uint32_t max_num_seqs = 1, max_num_batched_tokens = 1, max_model_len = 512;
  void validate() const;
  Json to_json() const;
};

struct Graph {
  std::string name;
  std::vector<Node> nodes;
  uint32_t output = 0;
  uint32_t max_context = 512;
  uint32_t eos = 0;
  Parallel parallel;

  void validate() const;            // graph-level rules (topology, liveness, route provenance, ...)
  std::string encode() const;       // IFTOKN01
  static Graph decode(std::string_view bytes);
  std::string dot() const;          // Graphviz
  Json to_json() const;
  static Graph from_json(const Json& j);   // types are inferred again and the graph is validated: nothing is trusted
  std::map<std::string, size_t> op_histogram() const;
};

// Expanded DSL -> typed, validated graph. Throws Error(Invalid) with the source byte of the bad node.
Graph elaborate(const lang::Expanded& ex);
// Convenience: source text -> graph.
Graph compile_source(std::string_view source);

// Infer the output type of `node` from its inputs' types (exact attribute sets are enforced).
Type infer(const Node& node, const std::vector<Type>& inputs, const Parallel& par);

}  // namespace ifab::graph
