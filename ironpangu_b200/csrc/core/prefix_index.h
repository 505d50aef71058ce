// Prefix index (compressed radix tree over token ids) and the LRU prefix cache built on it.
//
// Checkpoints are sequence-state snapshots taken at aligned token boundaries. `insert` records that
// a checkpoint covers a token prefix; `lookup` returns the longest recorded prefix of a query that
// ends on an alignment boundary and leaves at least one token to compute. Entries live in a
// namespace and carry a PrefixIdentity, so prefixes made by another program, checkpoint, salt or
// page size never match. The cache adds capacity, LRU eviction and pin counts on top.
// Reference: crates/inferfabric-runtime/src/prefix_index.rs:12-222,
// crates/inferfabric-native/src/prefix_cache.rs:16-232.
#pragma once
#include <list>
#include <memory>

#include "serving.h"
#include "state_pool.h"

namespace ifab::runtime {

struct CheckpointId { uint64_t value = 0; bool operator==(const CheckpointId& o) const { return value == o.value; } };
struct Match { CheckpointId id; uint32_t tokens = 0; };

class PrefixIndex {
 public:
  PrefixIndex(serving::PrefixIdentity identity, uint32_t alignment);
  // Record `id` for exactly `tokens` (length must be a positive multiple of the alignment). Returns false if
  // the same prefix is already recorded (the existing checkpoint is kept).
  bool insert(const serving::PrefixIdentity& identity, const std::vector<uint32_t>& tokens, CheckpointId id);
  // Longest recorded prefix of `tokens` with length <= tokens.size() - 1.
  std::optional<Match> lookup(const serving::PrefixIdentity& identity, const std::vector<uint32_t>& tokens) const;
  bool remove(CheckpointId id);
  size_t size() const { return count_; }
  bool empty() const { return count_ == 0; }
  uint64_t token_units() const { return token_units_; }   // tokens stored in edges (memory proxy)
  uint32_t alignment() const { return alignment_; }

 private:
  struct Node {
    std::vector<uint32_t> edge;                       // tokens on the edge from the parent
    std::map<uint32_t, std::unique_ptr<Node>> next;   // by first token of the child edge
    std::optional<CheckpointId> checkpoint;
  };
  bool remove_in(Node& n, CheckpointId id);
  serving::PrefixIdentity identity_;
  uint32_t alignment_;
  Node root_;
  size_t count_ = 0;
  uint64_t token_units_ = 0;
};

// LRU cache of sealed sequence snapshots keyed by token prefix.
class PrefixCache {
 public:
  struct Entry {
    CheckpointId id;
    std::vector<uint32_t> tokens;
    SealedLease snapshot;
    serving::ArithmeticHistory history;
    uint32_t pins = 0;
  };
  PrefixCache(serving::PrefixIdentity identity, uint32_t alignment, size_t capacity);
  // Publish a snapshot for `tokens`; evicts least-recently-used unpinned entries to make room. Returns the
  // evicted snapshots (the caller retires them in the state pool). nullopt id = not stored (duplicate / no room).
  std::optional<CheckpointId> publish(const std::vector<uint32_t>& tokens, SealedLease snapshot, const serving::ArithmeticHistory& history,
                                      std::vector<SealedLease>* evicted);
  // Longest usable prefix whose history matches what `variant_of` would produce; pins the entry until unpin().
  const Entry* restore(const std::vector<uint32_t>& tokens, const serving::ArithmeticHistory* expect = nullptr);
  void unpin(CheckpointId id);
  std::vector<SealedLease> clear();          // drops every unpinned entry
  size_t size() const { return entries_.size(); }
  uint64_t hits() const { return hits_; }
  uint64_t misses() const { return misses_; }

 private:
  PrefixIndex index_;
  serving::PrefixIdentity identity_;
  size_t capacity_;
  std::list<Entry> entries_;                 // front = most recently used
  uint64_t next_id_ = 1, hits_ = 0, misses_ = 0;
};

}  // namespace ifab::runtime
