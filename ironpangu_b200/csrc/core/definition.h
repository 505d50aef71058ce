// Model definitions: the one value every authoring path ends in, and its JSON artifact.
//
// A `.inferfabric` document becomes one of four definitions, chosen by the plan's target or the model's contract field:
//   Execution  plan target b200_token_v1 / ascend_token_v1: a checked token graph + its parallel layout
//   Graph      plan target cpu_f32_v1: a static f32 graph for the CPU planner
//   Qwen       model field `contract = qwen35_text_v1 | qwen_structure_v1`: a hybrid decoder Spec (layer kinds, meshes, buckets);
//              the first form is bound to a checkpoint, the second is structure only
//   OpenPangu  model field `contract = openpangu_v2_tp_ep_v1`: the parallel layout of the 92B-class family alone
// Contract documents hold `key = value;` fields only (no graph members, no modules). `definition()` also accepts the JSON
// artifact {"format": "inferfabric.model", "version": 1, "definition": {"kind": ...}} (at most 16 MiB) that `encode`
// writes, and validates it exactly like a document. Nothing in either input is executed.
// Reference: crates/inferfabric-dsl/src/lib.rs:94-268, crates/inferfabric-authoring/src/lib.rs:9-80.
#pragma once
#include "cpu_plan.h"
#include "graph.h"
#include "rankplan.h"

namespace ifab::definition {

enum class Kind { Qwen, OpenPangu, Graph, Execution };
const char* kind_name(Kind k);

struct ModelDefinition {
  Kind kind = Kind::Graph;
  bool checkpoint = false;        // Qwen: true for qwen35_text_v1 (weights come from a checkpoint)
  rankplan::Spec spec;            // Qwen
  graph::Parallel parallel;       // OpenPangu, Execution
  cpu::LogicalGraph logical;      // Graph
  graph::Graph execution;         // Execution

  void validate() const;          // the checks of the definition's kind (Spec / Parallel / token graph / CPU plan compile)
  Json to_json() const;           // {"kind": "qwen" | "open_pangu" | "graph" | "execution", ...}
  static ModelDefinition from_json(const Json& j);
};

constexpr size_t kMaxArtifactBytes = (size_t)16 << 20;

ModelDefinition elaborate(const lang::Document& doc);
// DSL text, or (first non-blank byte '{') the JSON artifact.
ModelDefinition definition(std::string_view source);
std::string encode(const ModelDefinition& d);          // pretty JSON artifact; validates first
ModelDefinition decode(std::string_view bytes);        // validates after parsing; rejects other formats / versions / fields

// Conveniences mirroring the reference's `parse` / `parse_checkpoint`.
rankplan::Spec parse_spec(std::string_view source);               // any Qwen definition
rankplan::Spec parse_checkpoint_spec(std::string_view source);    // only the checkpoint-bound contract

}  // namespace ifab::definition
