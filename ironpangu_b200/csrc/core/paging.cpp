#include "paging.h"

#include <algorithm>
#include <set>

#include "serving.h"

namespace ifab::paging {

std::vector<PageSpan> page_spans(uint32_t begin, uint32_t count, uint32_t page_tokens) {
  if (page_tokens == 0) invalid("page_spans: page size is zero");
  std::vector<PageSpan> out;
  uint64_t pos = begin, end = (uint64_t)begin + count;
  while (pos < end) {
    uint32_t page = (uint32_t)(pos / page_tokens), row = (uint32_t)(pos % page_tokens);
    uint32_t rows = (uint32_t)std::min<uint64_t>(page_tokens - row, end - pos);
    out.push_back({page, row, rows});
    pos += rows;
  }
  return out;
}

void PagedStateContract::validate() const {
  if (page_tokens == 0 || row_bytes == 0 || pool_pages == 0 || max_pages_per_sequence == 0) invalid("paged state: all dimensions must be positive");
  if (max_pages_per_sequence > pool_pages) invalid("paged state: a sequence cannot own more pages than the pool holds");
  if (row_bytes % 16) invalid("paged state: rows must be a multiple of 16 bytes");
}

ResidentPages::ResidentPages(PagedStateContract c, uint32_t residents) : c_(c), tables_(residents), owner_(c.pool_pages, -1) { c_.validate(); }

void ResidentPages::bind(uint32_t resident, const std::vector<uint32_t>& pages) {
  if (resident >= tables_.size()) invalid("page binding: resident out of range");
  if (pages.size() > c_.max_pages_per_sequence) fail(ErrorKind::Capacity, "page binding: too many pages for one sequence");
  std::set<uint32_t> uniq;
  for (uint32_t p : pages) {
    if (p >= c_.pool_pages) invalid("page binding: page " + std::to_string(p) + " outside the pool");
    if (!uniq.insert(p).second) invalid("page binding: page listed twice");
    if (owner_[p] >= 0 && owner_[p] != (int32_t)resident) invalid("page binding: page " + std::to_string(p) + " belongs to resident " + std::to_string(owner_[p]));
  }
  release(resident);
  for (uint32_t p : pages) owner_[p] = (int32_t)resident;
  tables_[resident] = pages;
}
void ResidentPages::release(uint32_t resident) {
  if (resident >= tables_.size()) invalid("page binding: resident out of range");
  for (uint32_t p : tables_[resident]) owner_[p] = -1;
  tables_[resident].clear();
}
void ResidentPages::append(uint32_t resident, uint32_t page) {
  if (resident >= tables_.size()) invalid("page binding: resident out of range");
  if (page >= c_.pool_pages) invalid("page binding: page outside the pool");
  if (owner_[page] >= 0) invalid("page binding: page already bound");
  if (tables_[resident].size() >= c_.max_pages_per_sequence) fail(ErrorKind::Capacity, "page binding: sequence is at its page limit");
  owner_[page] = (int32_t)resident;
  tables_[resident].push_back(page);
}
const std::vector<uint32_t>& ResidentPages::table(uint32_t resident) const {
  if (resident >= tables_.size()) invalid("page binding: resident out of range");
  return tables_[resident];
}
std::vector<int32_t> ResidentPages::batch_table() const {
  std::vector<int32_t> t((size_t)tables_.size() * c_.max_pages_per_sequence, -1);
  for (size_t r = 0; r < tables_.size(); ++r)
    for (size_t k = 0; k < tables_[r].size(); ++k) t[r * c_.max_pages_per_sequence + k] = (int32_t)tables_[r][k];
  return t;
}
uint64_t ResidentPages::row_offset(uint32_t resident, uint32_t position) const {
  const auto& t = table(resident);
  const uint32_t lp = position / c_.page_tokens;
  if (lp >= t.size()) fail(ErrorKind::Capacity, "page binding: position beyond the bound pages");
  return ((uint64_t)t[lp] * c_.page_tokens + position % c_.page_tokens) * c_.row_bytes;
}
std::vector<ResidentPages::CopyRange> ResidentPages::copy_plan(uint32_t src, uint32_t dst, uint32_t tokens) const {
  if (src == dst) invalid("state copy: source and destination are the same resident");
  std::vector<CopyRange> out;
  for (auto& s : page_spans(0, tokens, c_.page_tokens)) {
    const auto &ts = table(src), &td = table(dst);
    if (s.page >= ts.size() || s.page >= td.size()) fail(ErrorKind::Capacity, "state copy: not enough pages bound");
    CopyRange r;
    r.src = ((uint64_t)ts[s.page] * c_.page_tokens + s.first_row) * c_.row_bytes;
    r.dst = ((uint64_t)td[s.page] * c_.page_tokens + s.first_row) * c_.row_bytes;
    r.bytes = (uint64_t)s.rows * c_.row_bytes;
    if (!out.empty() && out.back().src + out.back().bytes == r.src && out.back().dst + out.back().bytes == r.dst) out.back().bytes += r.bytes;
    else out.push_back(r);
  }
  return out;
}

SequenceBatch SequenceBatch::make(const std::vector<SequenceSlice>& slices, const std::vector<int32_t>& tokens, uint32_t max_rows,
                                  uint32_t residents, uint32_t context) {
  if (slices.empty()) invalid("sequence batch: empty");
  SequenceBatch b;
  std::set<uint32_t> seen;
  size_t cursor = 0;
  for (auto& s : slices) {
    if (s.token_count == 0) invalid("sequence batch: empty slice");
    if (s.resident >= residents) invalid("sequence batch: resident out of range");
    if (!seen.insert(s.resident).second) invalid("sequence batch: resident appears twice");
    if ((uint64_t)s.position + s.token_count > context) fail(ErrorKind::Capacity, "sequence batch: slice exceeds the context");
    if (cursor + s.token_count > tokens.size()) invalid("sequence batch: fewer tokens than the slices describe");
    if (b.tokens.size() + s.token_count > max_rows) fail(ErrorKind::Capacity, "sequence batch: more rows than the variant accepts");
    for (uint32_t k = 0; k < s.token_count; ++k) {
      b.tokens.push_back(tokens[cursor + k]);
      b.positions.push_back((int32_t)(s.position + k));
      b.slots.push_back((int32_t)s.resident);
    }
    cursor += s.token_count;
    b.sample_rows.push_back(s.sample ? (int32_t)b.tokens.size() - 1 : -1);
    b.slices.push_back(s);
  }
  if (cursor != tokens.size()) invalid("sequence batch: more tokens than the slices describe");
  return b;
}

SlidingWindowLayout SlidingWindowLayout::make(uint32_t context, uint32_t window, uint32_t max_query, uint32_t page_tokens) {
  if (window == 0) invalid("sliding window: window must be positive");
  SlidingWindowLayout l;
  l.window = window;
  l.page_tokens = page_tokens;
  l.capacity = serving::sliding_capacity(context, window, max_query, page_tokens);
  return l;
}
bool SlidingWindowLayout::append_is_safe(uint32_t position, uint32_t count) const {
  if (count == 0) return true;
  // rows [position, position+count) are written; the earliest query of the append still sees
  // positions >= first_visible(position). A written row p overwrites position p - capacity.
  const uint64_t last_written = (uint64_t)position + count - 1;
  if (last_written < capacity) return true;
  const uint64_t overwritten_newest = last_written - capacity;
  return overwritten_newest < first_visible(position);
}

uint32_t BoundedBuffers::acquire(uint64_t bytes) {
  if (bytes > bytes_) fail(ErrorKind::Capacity, "bounded buffers: request of " + std::to_string(bytes) + " bytes exceeds the planned " + std::to_string(bytes_));
  if (free_.empty()) fail(ErrorKind::Capacity, "bounded buffers: pool exhausted");
  uint32_t id = free_.back();
  free_.pop_back();
  return id;
}
void BoundedBuffers::release(uint32_t id) {
  if (std::find(free_.begin(), free_.end(), id) != free_.end()) invalid("bounded buffers: double release");
  free_.push_back(id);
}

}  // namespace ifab::paging
