// Sequence-state allocator: pages and slots for every (state component, rank) of a serving manifest.
//
// A request reserves a Lease covering `tokens` tokens; each paged component receives the page units
// it needs (a sliding-window component only its ring), each slot component one slot. Work that
// touches a lease is bracketed by submit() -> Ticket and one complete() per rank; until every rank
// completed, the lease can be neither sealed nor reclaimed. seal() freezes a lease into a read-only
// SealedLease (prefix snapshots) that outlives the owner's retire(); readers pin leases with
// borrow()/release(). Units return to the free lists only when the owner retired, no ticket is in
// flight and no borrower remains (deferred reclaim). Every handle carries a generation, so a stale
// handle never aliases a recycled physical unit, and the pool epoch rejects handles of an earlier
// engine incarnation. poison() fails every later call (fail closed after a backend error).
// Reference: crates/inferfabric-runtime/src/state_pool.rs:13-479.
#pragma once
#include <set>

#include "serving.h"

namespace ifab::runtime {

struct Lease { uint64_t id = 0, generation = 0; };
struct Borrow { uint64_t id = 0, lease = 0, generation = 0; };
struct Ticket { uint64_t id = 0; };
struct SealedLease { uint64_t lease = 0, generation = 0; };

struct Binding {             // units of one component on one rank
  std::string component;
  uint32_t rank = 0;
  std::vector<uint32_t> units;   // page ids (Pages) or one slot id (Slot)
  uint32_t ring_tokens = 0;      // > 0: positions wrap modulo this many tokens
};
struct PageAddress {
  uint32_t unit = 0;             // physical page / slot
  uint32_t row = 0;              // row inside the page
  uint64_t byte_offset = 0;      // unit * unit_bytes + row * row_bytes
};
struct Usage {
  std::string component;
  uint32_t rank = 0;
  uint64_t capacity_units = 0, occupied_units = 0, occupied_bytes = 0, sealed_bytes = 0;
  bool operator==(const Usage& o) const {
    return component == o.component && rank == o.rank && capacity_units == o.capacity_units && occupied_units == o.occupied_units &&
           occupied_bytes == o.occupied_bytes && sealed_bytes == o.sealed_bytes;
  }
};

class StatePool {
 public:
  using Key = std::pair<std::string, uint32_t>;   // (state name, rank)
  // `capacities`: units available per (component, rank); `ranks` = tensor-parallel width.
  StatePool(const serving::Manifest& manifest, uint64_t epoch, uint32_t ranks, const std::map<Key, uint32_t>& capacities);

  Lease reserve(uint64_t epoch, uint64_t request, uint32_t tokens);
  Lease reserve_at_slot(uint64_t epoch, uint64_t request, uint32_t tokens, uint32_t slot);   // pin the slot index (resident id)
  const std::vector<Binding>& bindings(uint64_t epoch, Lease lease) const;
  PageAddress page_address(uint64_t epoch, Lease lease, const std::string& component, uint32_t rank, uint32_t position) const;

  Borrow borrow(uint64_t epoch, Lease lease);
  Borrow borrow_sealed(uint64_t epoch, SealedLease sealed);
  const std::vector<Binding>& borrowed_bindings(uint64_t epoch, Borrow b) const;
  void release(uint64_t epoch, Borrow b);
  void check_idle(uint64_t epoch, Lease lease) const;        // no ticket in flight
  SealedLease seal(uint64_t epoch, Lease lease);

  Ticket submit(uint64_t epoch, const std::vector<Lease>& writes, const std::vector<Borrow>& reads);
  void complete(uint64_t epoch, Ticket t, uint32_t rank);
  void retire(uint64_t epoch, Lease lease);
  void poison() { poisoned_ = true; }
  bool poisoned() const { return poisoned_; }
  std::vector<Usage> usage() const;
  uint64_t epoch() const { return epoch_; }

 private:
  struct Component {
    serving::State state;
    uint64_t unit_bytes = 0;
    std::vector<std::vector<uint32_t>> free_units;   // per rank, LIFO
    std::vector<uint32_t> capacity;                  // per rank
  };
  struct Record {
    uint64_t generation = 0, request = 0;
    uint32_t tokens = 0;
    std::vector<Binding> bindings;
    bool retired = false, sealed = false;
    uint32_t in_flight = 0, borrowers = 0;
  };
  struct Flight {
    std::vector<uint64_t> leases;        // writes and reads alike keep their leases alive
    std::set<uint32_t> pending_ranks;
  };
  void guard(uint64_t epoch) const;
  Record& record(Lease l);
  const Record& record(Lease l) const;
  void maybe_reclaim(uint64_t id);
  Lease reserve_impl(uint64_t request, uint32_t tokens, int64_t slot);

  uint64_t epoch_;
  uint32_t ranks_;
  uint32_t max_context_;
  std::vector<Component> components_;
  std::map<uint64_t, Record> leases_;
  std::map<uint64_t, Borrow> borrows_;
  std::map<uint64_t, Flight> flights_;
  uint64_t next_lease_ = 1, next_borrow_ = 1, next_ticket_ = 1, next_generation_ = 1;
  bool poisoned_ = false;
};

}  // namespace ifab::runtime
