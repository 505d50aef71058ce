#include "state_pool.h"

#include <algorithm>

namespace ifab::runtime {

using serving::Retention;
using serving::Storage;

StatePool::StatePool(const serving::Manifest& m, uint64_t epoch, uint32_t ranks, const std::map<Key, uint32_t>& capacities)
    : epoch_(epoch), ranks_(ranks), max_context_(m.max_context) {
  if (ranks == 0 || ranks > 64) invalid("state pool: ranks out of range");
  for (auto& s : m.states) {
    Component c;
    c.state = s;
    c.unit_bytes = s.storage.kind == Storage::Kind::Pages ? (uint64_t)s.storage.page_tokens * s.storage.row_bytes : s.storage.slot_bytes;
    c.free_units.resize(ranks);
    c.capacity.resize(ranks);
    for (uint32_t r = 0; r < ranks; ++r) {
      auto it = capacities.find({s.name, r});
      if (it == capacities.end()) invalid("state pool: no capacity given for " + s.name + " on rank " + std::to_string(r));
      c.capacity[r] = it->second;
      for (uint32_t u = it->second; u-- > 0;) c.free_units[r].push_back(u);   // unit 0 is handed out first
    }
    components_.push_back(std::move(c));
  }
  for (auto& kv : capacities) {
    bool known = false;
    for (auto& c : components_) known |= c.state.name == kv.first.first && kv.first.second < ranks;
    if (!known) invalid("state pool: capacity for unknown component " + kv.first.first);
  }
}

void StatePool::guard(uint64_t epoch) const {
  if (poisoned_) fail(ErrorKind::Backend, "state pool is poisoned");
  if (epoch != epoch_) fail(ErrorKind::Stale, "state pool: handle from epoch " + std::to_string(epoch) + ", pool is at " + std::to_string(epoch_));
}
StatePool::Record& StatePool::record(Lease l) {
  auto it = leases_.find(l.id);
  if (it == leases_.end() || it->second.generation != l.generation) fail(ErrorKind::Stale, "state pool: unknown or recycled lease");
  return it->second;
}
const StatePool::Record& StatePool::record(Lease l) const {
  auto it = leases_.find(l.id);
  if (it == leases_.end() || it->second.generation != l.generation) fail(ErrorKind::Stale, "state pool: unknown or recycled lease");
  return it->second;
}

Lease StatePool::reserve(uint64_t epoch, uint64_t request, uint32_t tokens) {
  guard(epoch);
  return reserve_impl(request, tokens, -1);
}
Lease StatePool::reserve_at_slot(uint64_t epoch, uint64_t request, uint32_t tokens, uint32_t slot) {
  guard(epoch);
  return reserve_impl(request, tokens, slot);
}

Lease StatePool::reserve_impl(uint64_t request, uint32_t tokens, int64_t slot) {
  if (tokens == 0) invalid("state pool: empty reservation");
  if (tokens > max_context_) fail(ErrorKind::Capacity, "state pool: reservation exceeds the model context");
  // first pass: can every component on every rank satisfy the request? (all-or-nothing)
  std::vector<uint32_t> need(components_.size()), ring(components_.size(), 0);
  for (size_t ci = 0; ci < components_.size(); ++ci) {
    const Component& c = components_[ci];
    if (c.state.storage.kind == Storage::Kind::Slot) {
      need[ci] = 1;
    } else {
      const uint32_t page = c.state.storage.page_tokens;
      uint32_t rows = tokens;
      if (c.state.retention.kind == Retention::Kind::SlidingWindow) {
        const uint32_t cap = serving::sliding_capacity(max_context_, c.state.retention.window, /*query*/ page, page);
        if (tokens > cap) {
          rows = cap;
          ring[ci] = cap;
        }
      }
      need[ci] = (rows + page - 1) / page;
    }
    for (uint32_t r = 0; r < ranks_; ++r) {
      if (c.state.storage.kind == Storage::Kind::Slot && slot >= 0) {
        auto& f = c.free_units[r];
        if (std::find(f.begin(), f.end(), (uint32_t)slot) == f.end()) fail(ErrorKind::Capacity, "state pool: slot " + std::to_string(slot) + " of " + c.state.name + " is taken");
      } else if (c.free_units[r].size() < need[ci]) {
        fail(ErrorKind::Capacity, "state pool: " + c.state.name + " on rank " + std::to_string(r) + " has " + std::to_string(c.free_units[r].size()) +
                                      " free units, " + std::to_string(need[ci]) + " needed");
      }
    }
  }
  Record rec;
  rec.generation = next_generation_++;
  rec.request = request;
  rec.tokens = tokens;
  for (size_t ci = 0; ci < components_.size(); ++ci) {
    Component& c = components_[ci];
    for (uint32_t r = 0; r < ranks_; ++r) {
      Binding b;
      b.component = c.state.name;
      b.rank = r;
      b.ring_tokens = ring[ci];
      auto& f = c.free_units[r];
      if (c.state.storage.kind == Storage::Kind::Slot && slot >= 0) {
        f.erase(std::find(f.begin(), f.end(), (uint32_t)slot));
        b.units.push_back((uint32_t)slot);
      } else {
        for (uint32_t k = 0; k < need[ci]; ++k) {
          b.units.push_back(f.back());
          f.pop_back();
        }
      }
      rec.bindings.push_back(std::move(b));
    }
  }
  Lease l{next_lease_++, rec.generation};
  leases_[l.id] = std::move(rec);
  return l;
}

const std::vector<Binding>& StatePool::bindings(uint64_t epoch, Lease lease) const {
  guard(epoch);
  const Record& r = record(lease);
  if (r.retired) fail(ErrorKind::Stale, "state pool: lease was retired");
  return r.bindings;
}

PageAddress StatePool::page_address(uint64_t epoch, Lease lease, const std::string& component, uint32_t rank, uint32_t position) const {
  guard(epoch);
  const Record& rec = record(lease);
  if (rec.retired) fail(ErrorKind::Stale, "state pool: lease was retired");
  if (position >= rec.tokens) fail(ErrorKind::Capacity, "state pool: position beyond the reservation");
  for (size_t ci = 0; ci < components_.size(); ++ci) {
    const Component& c = components_[ci];
    if (c.state.name != component) continue;
    for (auto& b : rec.bindings) {
      if (b.component != component || b.rank != rank) continue;
      PageAddress a;
      if (c.state.storage.kind == Storage::Kind::Slot) {
        a.unit = b.units[0];
        a.byte_offset = (uint64_t)a.unit * c.unit_bytes;
        return a;
      }
      const uint32_t page = c.state.storage.page_tokens;
      const uint32_t p = b.ring_tokens ? position % b.ring_tokens : position;
      a.unit = b.units.at(p / page);
      a.row = p % page;
      a.byte_offset = (uint64_t)a.unit * c.unit_bytes + (uint64_t)a.row * c.state.storage.row_bytes;
      return a;
    }
  }
  invalid("state pool: no component " + component + " on rank " + std::to_string(rank));
}

Borrow StatePool::borrow(uint64_t epoch, Lease lease) {
  guard(epoch);
  Record& r = record(lease);
  if (r.retired) fail(ErrorKind::Stale, "state pool: lease was retired");
  Borrow b{next_borrow_++, lease.id, lease.generation};
  ++r.borrowers;
  borrows_[b.id] = b;
  return b;
}
Borrow StatePool::borrow_sealed(uint64_t epoch, SealedLease s) {
  guard(epoch);
  auto it = leases_.find(s.lease);
  if (it == leases_.end() || it->second.generation != s.generation || !it->second.sealed) fail(ErrorKind::Stale, "state pool: sealed lease no longer exists");
  Borrow b{next_borrow_++, s.lease, s.generation};
  ++it->second.borrowers;
  borrows_[b.id] = b;
  return b;
}
const std::vector<Binding>& StatePool::borrowed_bindings(uint64_t epoch, Borrow b) const {
  guard(epoch);
  auto it = borrows_.find(b.id);
  if (it == borrows_.end() || it->second.generation != b.generation) fail(ErrorKind::Stale, "state pool: unknown borrow");
  return leases_.at(b.lease).bindings;
}
void StatePool::release(uint64_t epoch, Borrow b) {
  guard(epoch);
  auto it = borrows_.find(b.id);
  if (it == borrows_.end() || it->second.generation != b.generation) fail(ErrorKind::Stale, "state pool: unknown borrow");
  borrows_.erase(it);
  Record& r = leases_.at(b.lease);
  --r.borrowers;
  maybe_reclaim(b.lease);
}
void StatePool::check_idle(uint64_t epoch, Lease lease) const {
  guard(epoch);
  if (record(lease).in_flight) fail(ErrorKind::Invalid, "state pool: lease has work in flight");
}
SealedLease StatePool::seal(uint64_t epoch, Lease lease) {
  guard(epoch);
  Record& r = record(lease);
  if (r.retired) fail(ErrorKind::Stale, "state pool: lease was retired");
  if (r.in_flight) invalid("state pool: cannot seal a lease with work in flight");
  r.sealed = true;
  return SealedLease{lease.id, lease.generation};
}

Ticket StatePool::submit(uint64_t epoch, const std::vector<Lease>& writes, const std::vector<Borrow>& reads) {
  guard(epoch);
  if (writes.empty() && reads.empty()) invalid("state pool: empty submission");
  std::set<uint64_t> seen;
  for (auto& l : writes) {
    Record& r = record(l);
    if (r.retired) fail(ErrorKind::Stale, "state pool: lease was retired");
    if (r.sealed) invalid("state pool: a sealed lease is read-only");
    if (!seen.insert(l.id).second) invalid("state pool: lease submitted twice");
  }
  for (auto& b : reads) {
    auto it = borrows_.find(b.id);
    if (it == borrows_.end() || it->second.generation != b.generation) fail(ErrorKind::Stale, "state pool: unknown borrow");
    if (seen.count(b.lease)) invalid("state pool: lease is both written and read by one submission");
  }
  Flight f;
  for (auto& l : writes) f.leases.push_back(l.id);
  for (auto& b : reads) f.leases.push_back(b.lease);
  for (uint32_t r = 0; r < ranks_; ++r) f.pending_ranks.insert(r);
  for (uint64_t id : f.leases) ++leases_.at(id).in_flight;
  Ticket t{next_ticket_++};
  flights_[t.id] = std::move(f);
  return t;
}

void StatePool::complete(uint64_t epoch, Ticket t, uint32_t rank) {
  guard(epoch);
  auto it = flights_.find(t.id);
  if (it == flights_.end()) fail(ErrorKind::Stale, "state pool: unknown ticket");
  if (!it->second.pending_ranks.erase(rank)) invalid("state pool: rank " + std::to_string(rank) + " already completed this ticket");
  if (!it->second.pending_ranks.empty()) return;
  std::vector<uint64_t> ids = it->second.leases;
  flights_.erase(it);
  for (uint64_t id : ids) {
    --leases_.at(id).in_flight;
    maybe_reclaim(id);
  }
}

void StatePool::retire(uint64_t epoch, Lease lease) {
  guard(epoch);
  Record& r = record(lease);
  if (r.retired) fail(ErrorKind::Stale, "state pool: lease was already retired");
  r.retired = true;
  maybe_reclaim(lease.id);
}

void StatePool::maybe_reclaim(uint64_t id) {
  auto it = leases_.find(id);
  if (it == leases_.end()) return;
  Record& r = it->second;
  if (!r.retired || r.in_flight || r.borrowers) return;
  for (auto& b : r.bindings)
    for (auto& c : components_)
      if (c.state.name == b.component)
        for (auto u = b.units.rbegin(); u != b.units.rend(); ++u) c.free_units[b.rank].push_back(*u);
  leases_.erase(it);
}

std::vector<Usage> StatePool::usage() const {
  std::vector<Usage> out;
  for (auto& c : components_)
    for (uint32_t r = 0; r < ranks_; ++r) {
      Usage u;
      u.component = c.state.name;
      u.rank = r;
      u.capacity_units = c.capacity[r];
      u.occupied_units = c.capacity[r] - c.free_units[r].size();
      u.occupied_bytes = u.occupied_units * c.unit_bytes;
      for (auto& kv : leases_)
        if (kv.second.sealed)
          for (auto& b : kv.second.bindings)
            if (b.component == c.state.name && b.rank == r) u.sealed_bytes += b.units.size() * c.unit_bytes;
      out.push_back(std::move(u));
    }
  return out;
}

}  // namespace ifab::runtime
