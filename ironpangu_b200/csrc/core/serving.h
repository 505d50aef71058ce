// Serving manifest: what a runtime must know to host a compiled token program - execution variants
// (decode / prefill / extend with their accepted query-token counts), per-layer sequence states
// (paged KV, paged index keys, fixed-size slots) with retention policy, request batches, prefix
// identity and the arithmetic history that guards prefix reuse.
// Reference: crates/inferfabric-ir/src/serving.rs:7-312, arithmetic_history.rs:8-98,
// crates/inferfabric-compiler/src/token_serving.rs:6-165.
#pragma once
#include "program.h"

namespace ifab::serving {

enum class Phase { Decode, Prefill, Extend };
const char* phase_name(Phase p);

struct Variant {
  std::string name;
  Phase phase = Phase::Decode;
  std::vector<uint32_t> query_tokens;   // exact accepted counts; empty = any count up to max_query_tokens
  uint32_t max_query_tokens = 1;
  bool captured = true;                 // replayed as a CUDA graph
  std::string numerics;                 // numerical class: tokens produced by different classes are not mixed in a prefix
  bool accepts_query_tokens(uint32_t n) const;
};

struct Storage {
  enum class Kind { Pages, Slot } kind = Kind::Pages;
  uint32_t page_tokens = 0;   // Pages
  uint32_t row_bytes = 0;     // Pages: bytes per token row
  uint64_t slot_bytes = 0;    // Slot
};
struct Retention {
  enum class Kind { Full, SlidingWindow } kind = Kind::Full;
  uint32_t window = 0;
};
struct State {
  std::string name;           // logical node that owns the state
  uint32_t component = 0;     // dense index used by the state pool
  std::string dtype;
  Storage storage;
  Retention retention;
};

// Rows a sliding-window state must keep so that `query` new rows can be appended to a window of
// `window` rows in pages of `page` rows without overwriting a row that is still visible.
uint32_t sliding_capacity(uint32_t context, uint32_t window, uint32_t query, uint32_t page);

struct Identity {
  std::string model, program_sha256, target;
  uint32_t tp = 1;
};

struct RequestSpan {          // one sequence's share of a batch
  uint32_t resident = 0;      // sequence slot
  uint32_t position = 0;      // position of its first query token
  uint32_t token_count = 0;
  bool sample = false;        // emit a token for the last row
};
struct Batch {
  std::string variant;
  std::vector<RequestSpan> spans;
  uint32_t total_tokens() const;
};

struct Manifest {
  Identity identity;
  uint32_t max_context = 0, vocab = 0, eos = 0;
  uint32_t resident_sequences = 1, max_batched_tokens = 1;
  std::vector<Variant> variants;
  std::vector<State> states;
  std::vector<std::string> limitations;

  void validate() const;
  // Check a batch against the manifest (variant exists and accepts the token counts, residents in
  // range and distinct, positions + counts inside the context, token budget).
  void validate_batch(const Batch& b) const;
  const Variant* find_variant(std::string_view name) const;
  // Smallest variant that can run `tokens` query tokens of one sequence in `phase`.
  const Variant* choose_variant(Phase phase, uint32_t tokens) const;
  Json to_json() const;
  static Manifest from_json(const Json& j);
  uint64_t state_bytes_per_sequence() const;
};

Manifest lower(const program::Program& p, const std::string& program_sha256);

// Prefix identity: two cached prefixes are interchangeable only if all of this matches.
struct PrefixIdentity {
  std::string program_sha256, weights_sha256, ns, salt;
  uint32_t page_tokens = 0;
  bool compatible(const PrefixIdentity& o) const;
};

// Which numerical class produced each span of a sequence. A prefix may be reused by a continuation
// only if the continuation would have produced the same classes for the same spans.
class ArithmeticHistory {
 public:
  struct Span { uint32_t begin, end; std::string numerics; };
  void check_append(uint32_t begin, uint32_t count) const;            // must extend the history contiguously
  void append_completed(uint32_t begin, uint32_t count, const std::string& numerics);
  ArithmeticHistory prefix(uint32_t tokens) const;
  bool same_prefix(const ArithmeticHistory& o, uint32_t tokens) const;
  uint32_t length() const { return spans_.empty() ? 0 : spans_.back().end; }
  const std::vector<Span>& spans() const { return spans_; }

 private:
  std::vector<Span> spans_;
};

}  // namespace ifab::serving
