// Page arithmetic shared by the host runtime and the device executors: page spans of a token range,
// per-resident page bindings (possibly permuted / non-contiguous), batch page tables, state-copy
// plans for prefix snapshots, the packed sequence batch handed to the device, the sliding-window
// ring layout and bounded buffer leases.
// Reference: native/src/page_binding.h, native/include/{paged_state_contract,sequence_batch,
// sliding_window_layout,bounded_buffers}.h, native/src/continuation_copy.inc.
#pragma once
#include "base.h"

namespace ifab::paging {

struct PageSpan { uint32_t page = 0, first_row = 0, rows = 0; };   // logical page index + row range
// Logical pages touched by tokens [begin, begin + count) with `page_tokens` rows per page.
std::vector<PageSpan> page_spans(uint32_t begin, uint32_t count, uint32_t page_tokens);

struct PagedStateContract {
  uint32_t page_tokens = 16, row_bytes = 0, pool_pages = 0, max_pages_per_sequence = 0;
  void validate() const;
  uint64_t pool_bytes() const { return (uint64_t)pool_pages * page_tokens * row_bytes; }
};

// Physical pages bound to each resident sequence of one paged state.
class ResidentPages {
 public:
  ResidentPages(PagedStateContract c, uint32_t residents);
  void bind(uint32_t resident, const std::vector<uint32_t>& pages);   // replaces the binding; pages must be unique pool-wide
  void release(uint32_t resident);
  void append(uint32_t resident, uint32_t page);
  const std::vector<uint32_t>& table(uint32_t resident) const;
  // Row-major [residents x max_pages_per_sequence] table, -1 padded (what the kernels read).
  std::vector<int32_t> batch_table() const;
  uint64_t row_offset(uint32_t resident, uint32_t position) const;     // byte offset of a token row in the pool
  struct CopyRange { uint64_t src, dst, bytes; };
  // Byte ranges that copy the first `tokens` rows of `src` into `dst` (both must have enough pages).
  std::vector<CopyRange> copy_plan(uint32_t src, uint32_t dst, uint32_t tokens) const;
  const PagedStateContract& contract() const { return c_; }

 private:
  PagedStateContract c_;
  std::vector<std::vector<uint32_t>> tables_;
  std::vector<int32_t> owner_;   // page -> resident or -1
};

// One sequence's slice of a packed batch.
struct SequenceSlice { uint32_t resident = 0, position = 0, token_count = 0; bool sample = false; };
struct SequenceBatch {
  std::vector<int32_t> tokens, positions, slots;   // one entry per query row
  std::vector<int32_t> sample_rows;                // row index of each sequence's sampled row (or -1)
  std::vector<SequenceSlice> slices;
  // Pack slices in order; rejects duplicates, empty slices, overflow of `max_rows` and of `context`.
  static SequenceBatch make(const std::vector<SequenceSlice>& slices, const std::vector<int32_t>& tokens, uint32_t max_rows,
                            uint32_t residents, uint32_t context);
};

// Ring layout of a sliding-window state: position p lives in ring row p % capacity.
struct SlidingWindowLayout {
  uint32_t window = 0, capacity = 0, page_tokens = 16;
  static SlidingWindowLayout make(uint32_t context, uint32_t window, uint32_t max_query, uint32_t page_tokens);
  uint32_t ring_row(uint32_t position) const { return position % capacity; }
  // first visible position for a query at `position`
  uint32_t first_visible(uint32_t position) const { return position + 1 > window ? position + 1 - window : 0; }
  // true when appending `count` rows at `position` cannot overwrite a row still visible to any of them
  bool append_is_safe(uint32_t position, uint32_t count) const;
};

// Bounded leases of same-sized scratch buffers (exact-size LIFO): exhaustion fails closed.
class BoundedBuffers {
 public:
  BoundedBuffers(uint64_t bytes_each, uint32_t count) : bytes_(bytes_each) {
    for (uint32_t i = count; i-- > 0;) free_.push_back(i);
  }
  uint32_t acquire(uint64_t bytes);
  void release(uint32_t id);
  size_t available() const { return free_.size(); }

 private:
  uint64_t bytes_;
  std::vector<uint32_t> free_;
};

}  // namespace ifab::paging
