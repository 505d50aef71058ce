// Compiled bundle: the directory that couples the offline compiler to the runtime.
//
//   execution.bin         physical program (IFTOKN02-09)        logical.bin       logical graph (IFTOKN01)
//   execution.json/.dot   logical graph, JSON and Graphviz       execution.html    self-contained viewer
//   device-program.json   instructions + kernel recipes          physical.json     inspection plan (costs, collectives)
//   rank-N.bin/.init.json per-rank weight plans (IFINIT01/02)     serving.json      serving manifest
//   arena-rank-N.txt      frozen activation arena (IFARENA2)     workspace-rank-N.txt  kernel scratch (IFWORKSPACE1)
//   arena.json            arena summary                           plan.json         bundle index (token-bundle.v1)
//
// Everything is written into a staging sibling first and renamed into place; an existing output
// directory is never overwritten. Reference: crates/inferfabric-compiler/src/token.rs:338-458,
// native/include/frozen_arena.h:14-99, token_physical.rs:14-273.
#pragma once
#include <set>
#include "initplan.h"
#include "physical.h"
#include "serving.h"

namespace ifab::bundle {

// ---- activation arena ------------------------------------------------------------------------------
struct ArenaSlot {
  uint32_t instruction = 0;
  uint64_t offset = 0, bytes = 0;
  uint32_t first = 0, last = 0;     // live interval in instruction order
};
struct Arena {
  uint64_t bytes = 0;
  uint32_t tokens = 1;               // query rows the layout was planned for
  std::vector<ArenaSlot> slots;
  uint64_t workspace_bytes = 0;      // shared kernel scratch (attention splits, argmax partials, route lists)
  std::string encode(uint64_t program_fnv, uint64_t backend_fnv) const;                 // IFARENA2 text
  std::string encode_workspace(uint64_t program_fnv, uint64_t backend_fnv) const;       // IFWORKSPACE1 text
  static Arena decode(const std::string& text, uint64_t* program_fnv = nullptr, uint64_t* backend_fnv = nullptr);
  void verify() const;               // 512-byte alignment, ascending, no two live-overlapping slots share bytes
};
// Live-interval first-fit packing of every instruction result for `tokens` query rows.
// `pass_through`: instructions that hand their first input on unchanged (an optional norm whose gain the checkpoint lacks): they
// get no slot, and their source's slot lives on for as long as they are read.
Arena plan_arena(const program::Program& p, uint32_t tokens, const std::set<uint32_t>& pass_through = {});
uint64_t value_bytes(const program::Program& p, const program::Instruction& ins, uint32_t tokens);

// ---- inspection plan -------------------------------------------------------------------------------
physical::Plan physical_plan(const program::Program& p, const std::string& backend_fingerprint);
// SHA-256 over the kernel sources that execute the program (sorted by file name); "" if dir is empty.
std::string backend_fingerprint(const std::string& kernel_source_dir);

// ---- bundle ------------------------------------------------------------------------------------------
struct BundleInputs {
  std::string source_path, source_text;
  std::string checkpoint_dir;        // empty: plan against the shapes the program itself implies
  std::string kernel_source_dir;     // for the backend fingerprint
  program::Options options;
  bool allow_stale_index_size = false;
};
struct BundleSummary {
  std::string dir, program_sha256;
  size_t logical_nodes = 0, instructions = 0, launches = 0, collectives = 0;
  uint64_t arena_bytes = 0, weight_bytes_per_rank = 0;
  Json to_json() const;
};
BundleSummary write_bundle(const BundleInputs& in, const std::string& out_dir);

std::string html_view(const graph::Graph& g, const program::Program& p, const Arena& arena);

}  // namespace ifab::bundle
