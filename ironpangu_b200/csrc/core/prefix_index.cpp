#include "prefix_index.h"

#include <algorithm>

namespace ifab::runtime {

PrefixIndex::PrefixIndex(serving::PrefixIdentity identity, uint32_t alignment) : identity_(std::move(identity)), alignment_(alignment) {
  if (alignment == 0) invalid("prefix index: alignment must be positive");
}

bool PrefixIndex::insert(const serving::PrefixIdentity& identity, const std::vector<uint32_t>& tokens, CheckpointId id) {
  if (!identity_.compatible(identity)) invalid("prefix index: identity mismatch");
  if (tokens.empty() || tokens.size() % alignment_) invalid("prefix index: prefix length must be a positive multiple of " + std::to_string(alignment_));
  Node* cur = &root_;
  size_t pos = 0;
  while (pos < tokens.size()) {
    auto it = cur->next.find(tokens[pos]);
    if (it == cur->next.end()) {
      auto n = std::make_unique<Node>();
      n->edge.assign(tokens.begin() + pos, tokens.end());
      token_units_ += n->edge.size();
      n->checkpoint = id;
      cur->next[tokens[pos]] = std::move(n);
      ++count_;
      return true;
    }
    Node* child = it->second.get();
    size_t common = 0;
    while (common < child->edge.size() && pos + common < tokens.size() && child->edge[common] == tokens[pos + common]) ++common;
    if (common < child->edge.size()) {
      // split the edge at `common`
      auto mid = std::make_unique<Node>();
      mid->edge.assign(child->edge.begin(), child->edge.begin() + common);
      std::unique_ptr<Node> old = std::move(it->second);
      old->edge.erase(old->edge.begin(), old->edge.begin() + common);
      const uint32_t key = old->edge[0];
      mid->next[key] = std::move(old);
      Node* midp = mid.get();
      it->second = std::move(mid);
      child = midp;
    }
    pos += common;
    cur = child;
  }
  if (cur->checkpoint) return false;
  cur->checkpoint = id;
  ++count_;
  return true;
}

std::optional<Match> PrefixIndex::lookup(const serving::PrefixIdentity& identity, const std::vector<uint32_t>& tokens) const {
  if (!identity_.compatible(identity) || tokens.size() < 2) return std::nullopt;
  const size_t limit = tokens.size() - 1;   // at least one token must remain to produce logits
  const Node* cur = &root_;
  size_t pos = 0;
  std::optional<Match> best;
  while (pos < limit) {
    auto it = cur->next.find(tokens[pos]);
    if (it == cur->next.end()) break;
    const Node* child = it->second.get();
    if (pos + child->edge.size() > limit) break;
    if (!std::equal(child->edge.begin(), child->edge.end(), tokens.begin() + pos)) break;
    pos += child->edge.size();
    cur = child;
    if (cur->checkpoint && pos % alignment_ == 0) best = Match{*cur->checkpoint, (uint32_t)pos};
  }
  return best;
}

bool PrefixIndex::remove_in(Node& n, CheckpointId id) {
  for (auto it = n.next.begin(); it != n.next.end(); ++it) {
    Node& c = *it->second;
    if (c.checkpoint && *c.checkpoint == id) {
      c.checkpoint.reset();
      --count_;
      if (c.next.empty()) {
        token_units_ -= c.edge.size();
        n.next.erase(it);
      } else if (c.next.size() == 1) {
        // merge the only child into this edge
        std::unique_ptr<Node> only = std::move(c.next.begin()->second);
        c.edge.insert(c.edge.end(), only->edge.begin(), only->edge.end());
        c.checkpoint = only->checkpoint;
        auto grand = std::move(only->next);
        c.next = std::move(grand);
      }
      return true;
    }
    if (remove_in(c, id)) {
      if (!c.checkpoint && c.next.empty()) {
        token_units_ -= c.edge.size();
        n.next.erase(it);
      }
      return true;
    }
  }
  return false;
}
bool PrefixIndex::remove(CheckpointId id) { return remove_in(root_, id); }

// ---------------------------------------------------------------------------------------------
PrefixCache::PrefixCache(serving::PrefixIdentity identity, uint32_t alignment, size_t capacity)
    : index_(identity, alignment), identity_(std::move(identity)), capacity_(capacity) {}

std::optional<CheckpointId> PrefixCache::publish(const std::vector<uint32_t>& tokens, SealedLease snapshot, const serving::ArithmeticHistory& history,
                                                 std::vector<SealedLease>* evicted) {
  if (capacity_ == 0) return std::nullopt;
  if (history.length() != tokens.size()) invalid("prefix cache: history does not cover the prefix");
  while (entries_.size() >= capacity_) {
    auto victim = entries_.end();
    for (auto it = entries_.end(); it != entries_.begin();) {
      --it;
      if (it->pins == 0) { victim = it; break; }
    }
    if (victim == entries_.end()) return std::nullopt;   // everything is pinned
    index_.remove(victim->id);
    if (evicted) evicted->push_back(victim->snapshot);
    entries_.erase(victim);
  }
  CheckpointId id{next_id_++};
  if (!index_.insert(identity_, tokens, id)) return std::nullopt;
  entries_.push_front(Entry{id, tokens, snapshot, history, 0});
  return id;
}

const PrefixCache::Entry* PrefixCache::restore(const std::vector<uint32_t>& tokens, const serving::ArithmeticHistory* expect) {
  auto m = index_.lookup(identity_, tokens);
  if (!m) { ++misses_; return nullptr; }
  for (auto it = entries_.begin(); it != entries_.end(); ++it) {
    if (!(it->id == m->id)) continue;
    if (expect && !it->history.same_prefix(*expect, m->tokens)) { ++misses_; return nullptr; }
    ++it->pins;
    entries_.splice(entries_.begin(), entries_, it);
    ++hits_;
    return &entries_.front();
  }
  ++misses_;
  return nullptr;
}

void PrefixCache::unpin(CheckpointId id) {
  for (auto& e : entries_)
    if (e.id == id) {
      if (e.pins == 0) invalid("prefix cache: entry is not pinned");
      --e.pins;
      return;
    }
  invalid("prefix cache: unknown checkpoint");
}

std::vector<SealedLease> PrefixCache::clear() {
  std::vector<SealedLease> out;
  for (auto it = entries_.begin(); it != entries_.end();) {
    if (it->pins == 0) {
      index_.remove(it->id);
      out.push_back(it->snapshot);
      it = entries_.erase(it);
    } else {
      ++it;
    }
  }
  return out;
}

}  // namespace ifab::runtime
