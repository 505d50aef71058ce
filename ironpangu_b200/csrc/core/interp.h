// CPU interpreter of the logical token graph: the numerical oracle of every device plan.
//
// It executes one sequence token by token, simulating all tensor-parallel ranks (rank-local values
// are kept per rank, K-sharded partial sums are reduced in rank order) in f32 arithmetic and rounds
// to bf16 exactly where the device program stores bf16 tensors. The reference ships a scalar CPU
// model for its dense family (crates/inferfabric-cli/src/npu_probe/cpu_model.rs:47-151) and a CPU
// executor for f32 graphs (crates/inferfabric-plan/src/execute.rs:40-227); this interpreter covers
// the whole token-graph vocabulary instead.
#pragma once
#include "graph.h"
#include "initplan.h"

namespace ifab::interp {

struct Tensor {
  std::vector<uint64_t> shape;
  std::vector<float> data;
};

class Weights {
 public:
  // Load every tensor of a safetensors checkpoint (bf16 / f32 -> f32).
  static Weights from_checkpoint(const init::Checkpoint& ckpt);
  // Deterministic N(0, std) values rounded to bf16 (norm gains are 1 + N(0, std)); seed 0 by default.
  static Weights random(const std::map<std::string, std::pair<init::DType, std::vector<uint64_t>>>& shapes, uint64_t seed = 0, float std = 0.02f);
  // Write the tensors as one safetensors file (bf16, f32 for router weights) so a device run can load the same values.
  void save(const std::string& dir, const std::string& file = "model.safetensors") const;
  const Tensor& need(const std::string& name) const;
  const Tensor* find(const std::string& name) const;
  std::map<std::string, Tensor> tensors;
  std::map<std::string, init::DType> dtypes;
};

float bf16_round(float v);

class Interpreter {
 public:
  Interpreter(const graph::Graph& g, const Weights& w);
  // Feed `token` at `position` (positions must be consecutive from 0); returns the greedy next token.
  // `logits` (optional) receives the full-vocabulary f32 logits.
  uint32_t step(uint32_t token, uint32_t position, std::vector<float>* logits = nullptr);
  void reset();
  uint32_t vocab() const { return vocab_; }
  // The value node `name` produced in the last step, as JSON: {"ranks": [[...]]} for tensors (one row when replicated),
  // {"ids": [...], "weights": [...]} for routes and index selections, {"cache_rows": n} for caches. A probe for tests and
  // for debugging a device kernel against the oracle (the reference's probes: crates/inferfabric-cli/src/npu_probe.rs).
  Json watch(const std::string& name) const;

 private:
  struct Value {
    bool replicated = true;
    bool f32 = false;                          // true: unrounded f32 (partials, logits); false: bf16-valued
    std::vector<std::vector<float>> r;         // 1 (replicated) or tp vectors
    // Routes
    std::vector<uint32_t> ids;
    std::vector<float> wts;
    // Experts: per route row (per rank: rows of non-local routes stay empty)
    std::vector<std::vector<std::vector<float>>> rows;
    // HyperConnection
    std::vector<float> hc_x, hc_post, hc_comb;
    int cache = -1;                            // Cache / IndexCache state index
  };
  struct CacheState {
    uint32_t width = 0;
    std::vector<std::vector<float>> rows;      // one row per position
    std::vector<std::vector<float>> sinks;
  };
  struct ConvState {
    std::vector<std::vector<float>> hist;      // [ranks][(taps-1) * channels]
    uint32_t count = 0;
  };
  const std::vector<float>& at(const Value& v, uint32_t rank) const { return v.replicated ? v.r[0] : v.r[rank]; }
  void run_node(uint32_t i, uint32_t token, uint32_t position);

  const graph::Graph& g_;
  const Weights& w_;
  uint32_t tp_ = 1, vocab_ = 0;
  std::vector<Value> vals_;
  std::vector<CacheState> caches_;
  std::map<uint32_t, int> cache_of_node_;
  std::map<uint32_t, ConvState> conv_;
  uint32_t expected_pos_ = 0;
  int64_t logits_linear_ = -1;
};

}  // namespace ifab::interp
