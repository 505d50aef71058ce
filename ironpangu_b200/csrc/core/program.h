// Physical token program: the logical graph lowered to the instructions the B200 executor runs.
//
// Lowering = dtype assignment with explicit casts (CSE'd), view elimination for slices, and fusion
// selection that maps groups of logical nodes onto one sm_100a kernel each:
//   norm -> following linear / router / expert prologue
//   linear(tp_columns) + allreduce (+ residual add)            -> linear_allreduce
//   linear(paired) + swiglu                                    -> linear[activation=swiglu]
//   latent_attention + mla_value                               -> mla_attention
//   expert_linear + expert_swiglu_down + expert_reduce (+ shared expert partial) + allreduce (+ add)
//                                                              -> moe_gate_up + moe_down_allreduce
//   final linear(tp_rows) + gather at the output               -> lm_head (sharded logits / argmax)
// The reference performs the analogous step for CANN (crates/inferfabric-compiler/src/
// token_program.rs:157-943); the instruction record and the IFTOKN02-09 container are kept.
#pragma once
#include "graph.h"

namespace ifab::program {

// result kinds: graph::Kind values 0..7, plus
constexpr uint32_t kKindView = 8;   // aliases its input (no kernel)
constexpr uint32_t kKindNone = 9;   // produces nothing a later instruction reads

struct Instruction {
  uint32_t kind = 0;
  uint32_t width = 0;
  std::string name, op;
  std::vector<uint32_t> inputs;
  std::vector<std::pair<std::string, std::string>> attrs;
  std::string dtype;     // bf16 | f32 | int8 | i32 | none
  std::string kernel;    // C entry point that executes it ("view" / "none" when no launch)
  uint32_t logical_node = 0;

  const std::string* attr(std::string_view key) const;
};

struct Options {
  uint32_t resident_sequences = 1;           // sequence slots kept on device
  uint32_t prefill_tokens = 1;               // captured prefill width (1 = token at a time)
  std::vector<uint32_t> prefill_variants;    // exact captured widths, ascending (e.g. 2,4,8,16,32)
  bool uncaptured_prefill = false;           // eager chunk envelope of `prefill_tokens` rows
  bool shared_pages = false;                 // one page pool shared by all residents
  bool output_rows = false;                  // run the lm_head suffix on sampled rows only
  bool bulk_collectives = false;             // two-shot collectives for prefill-sized payloads
};

struct Program {
  std::string name;
  std::vector<Instruction> instructions;
  uint32_t output = 0;
  uint32_t max_context = 0, eos = 0;
  graph::Parallel parallel;
  Options options;
  std::vector<uint32_t> output_suffix;       // instruction ids that may run on sampled rows only

  void validate() const;
  std::string magic() const;                 // IFTOKN02 .. IFTOKN09 by feature set
  std::string encode() const;
  static Program decode(std::string_view bytes);
  Json to_json() const;                      // device-program.json (instructions + kernel recipes)
  std::map<std::string, size_t> op_histogram() const;
  size_t launches_per_token() const;         // instructions that launch a kernel
  size_t collectives_per_token() const;      // instructions that contain a cross-rank exchange
};

Program lower(const graph::Graph& g, const Options& opt = {});

// op -> kernel entry point table (the recipe book); unknown ops map to "unsupported".
const std::map<std::string, std::string>& recipes();

}  // namespace ifab::program
