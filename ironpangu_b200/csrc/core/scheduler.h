// Continuous-batching scheduler.
//
// LiveScheduler owns the request queue and the resident sequence slots of one engine. Every engine
// step is planned in two halves so that any executor (mock, CPU ranks, CUDA engine behind a C ABI or
// a Python binding) can run it:
//   plan()    admit queued requests into free residents, then walk the residents round-robin from a
//             cursor: a sequence contributes either its next prefill chunk (bounded by the chunk size
//             and the remaining token budget) or one decode token; cancelled or back-pressured
//             sequences are skipped; planning stops at the first sequence whose quantum no longer fits
//             (the cursor stays there, so it is served first next time)
//   commit()  consumes the sampled tokens: appends, checks stop tokens / length, emits events, frees
//             residents of finished sequences
// New requests join a running decode batch without any recapture (widths are bucketed by the engine).
// Reference: frontend/src/program_worker.rs:204-398, frontend/src/native_worker.rs:28-40,
// crates/inferfabric-scheduler/src/{lib.rs:72-390,live.rs:32-291}.
#pragma once
#include <deque>

#include "paging.h"
#include "runtime.h"

namespace ifab::sched {

enum class Finish { Stop, Length, Cancelled, Error };
const char* finish_name(Finish f);

struct Event {
  uint64_t request = 0;
  std::optional<uint32_t> token;
  std::optional<Finish> finish;
};

struct Request {
  uint64_t id = 0;
  std::vector<uint32_t> prompt;
  uint32_t max_new_tokens = 16;
  std::vector<uint32_t> stop_tokens;
  uint32_t prefix_hit = 0;           // tokens restored from the prefix cache (already in the sequence state)
};

struct Capacity {
  uint32_t residents = 1;            // sequence slots
  uint32_t token_budget = 1;         // query rows per engine step
  uint32_t chunk = 1;                // longest prefill chunk per sequence and step
  uint32_t context = 512;            // prompt + generated tokens must fit
  uint32_t queue = 256;              // admission queue bound
  uint32_t vocab = 0;                // 0 = do not validate token ids
  void validate() const;
};

// Fair selection under a budget: starting at `cursor`, take eligible[i] while its cost fits what remains.
// Returns the chosen indices in service order and advances `cursor` to the first index that did not fit.
std::vector<size_t> select_round(const std::vector<uint32_t>& costs, size_t* cursor, uint32_t budget);

class LiveScheduler {
 public:
  explicit LiveScheduler(Capacity c);
  // Throws Capacity when the queue is full ("overloaded") and Invalid for malformed requests.
  void submit(Request r);
  // Cancels a queued or running request; returns the terminal event if the request was known.
  std::optional<Event> cancel(uint64_t id);
  // Marks a request as unable to accept output right now (its client is slow); it is skipped until cleared.
  void set_backpressure(uint64_t id, bool on);

  struct Plan {
    paging::SequenceBatch batch;
    std::vector<uint64_t> requests;     // request of each slice
    std::vector<uint32_t> released;     // residents freed since the previous plan (their state may be dropped)
    std::vector<std::pair<uint32_t, uint64_t>> admitted;   // (resident, request) admitted by this plan
    bool empty() const { return batch.slices.empty(); }
  };
  Plan plan();
  // `sampled[i]` is the token sampled for slice i (ignored for slices with sample == false).
  std::vector<Event> commit(const Plan& plan, const std::vector<uint32_t>& sampled);
  // The executor failed: every running and queued request ends with Finish::Error.
  std::vector<Event> fail_all();

  bool idle() const { return queue_.empty() && running_ == 0; }
  size_t queued() const { return queue_.size(); }
  size_t running() const { return running_; }
  uint64_t steps() const { return steps_; }
  const Capacity& capacity() const { return cap_; }

 private:
  struct Seq {
    bool active = false, cancelled = false, backpressure = false;
    Request req;
    uint32_t fed = 0;                  // prompt tokens already in the sequence state
    std::vector<uint32_t> generated;
    bool in_flight = false;
  };
  Capacity cap_;
  std::deque<Request> queue_;
  std::vector<Seq> seqs_;
  std::vector<uint32_t> released_;
  size_t cursor_ = 0, running_ = 0;
  uint64_t steps_ = 0;
};

// ---- offline simulation over the mock runtime (prefill / decode disaggregation) ---------------------
struct SimRequest { uint64_t id = 0; uint32_t prompt_tokens = 8, output_tokens = 4, arrival_tick = 0; std::optional<uint32_t> cancel_tick; };
struct SimCapacity { uint32_t decode_slots = 4, pages = 64, page_tokens = 16; };
struct SimReport {
  uint64_t ticks = 0, prefill_steps = 0, decode_steps = 0, transfers = 0, cancelled = 0, completed = 0;
  std::map<uint64_t, std::vector<uint32_t>> outputs;
  size_t leaked_allocations = 0;
  Json to_json() const;
};
SimReport run_mock(const rankplan::Artifact& artifact, std::vector<SimRequest> requests, SimCapacity cap, std::shared_ptr<runtime::Trace> trace = nullptr);

}  // namespace ifab::sched
