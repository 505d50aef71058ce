// Backend-neutral runtime: staged start-up with fault injection, bucket-selecting step, thread-per-rank
// worker group, deterministic mock backend, health guard, and the prefill->decode transfer protocol.
//
// Start-up walks Validate -> Compile -> Prepare -> Warmup -> Capture -> ValidateReplay -> Reset -> Ready;
// a failure at any stage (real or injected through `fail_at`) leaves the runtime Failed, never Ready,
// and every later call is refused (fail closed; recovery is an external restart).
// Reference: crates/inferfabric-runtime/src/lib.rs:17-655, crates/inferfabric-transfer/src/lib.rs:24-287.
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

#include "rankplan.h"

namespace ifab::runtime {

enum class Stage { Validate, Compile, Prepare, Warmup, Capture, ValidateReplay, Reset, Ready, Failed, Closed };
const char* stage_name(Stage s);

// Shared, thread-safe event trace asserted by tests.
class Trace {
 public:
  void add(const std::string& e);
  std::vector<std::string> events() const;
  size_t count(const std::string& needle) const;

 private:
  mutable std::mutex mu_;
  std::vector<std::string> events_;
};

struct StepInput { uint64_t request = 0; std::vector<uint32_t> tokens; uint32_t position = 0; };
struct StepOutput { uint64_t request = 0; uint32_t token = 0; uint32_t consumed = 0; };

class Backend {
 public:
  virtual ~Backend() = default;
  virtual std::string kind() const = 0;
  virtual void compile_kernels(const rankplan::Artifact& a) = 0;
  virtual void prepare(const rankplan::RankPlan& plan) = 0;
  virtual void upload_weights(const std::string& source) = 0;
  virtual uint64_t allocate(uint64_t bytes) = 0;
  virtual void release(uint64_t buffer) = 0;
  virtual void warmup(const rankplan::Spec& spec) = 0;
  virtual uint64_t capture(rankplan::Bucket bucket) = 0;
  virtual void validate_graph(uint64_t graph, rankplan::Bucket bucket) = 0;
  virtual void reset_scratch() = 0;
  virtual std::vector<StepOutput> execute(const rankplan::RankPlan& plan, const rankplan::Spec& spec, const std::vector<StepInput>& inputs,
                                          std::optional<uint64_t> graph) = 0;
  virtual void communicate(const rankplan::Instruction& ins) = 0;
  virtual void synchronize() = 0;
  virtual void close() = 0;
};

// Deterministic stand-in: tokens are a hash of (request, position); every call is traced.
class MockBackend : public Backend {
 public:
  explicit MockBackend(std::shared_ptr<Trace> trace, uint32_t rank = 0) : trace_(std::move(trace)), rank_(rank) {}
  std::string kind() const override { return "mock"; }
  void compile_kernels(const rankplan::Artifact& a) override;
  void prepare(const rankplan::RankPlan& plan) override;
  void upload_weights(const std::string& source) override;
  uint64_t allocate(uint64_t bytes) override;
  void release(uint64_t buffer) override;
  void warmup(const rankplan::Spec& spec) override;
  uint64_t capture(rankplan::Bucket bucket) override;
  void validate_graph(uint64_t graph, rankplan::Bucket bucket) override;
  void reset_scratch() override;
  std::vector<StepOutput> execute(const rankplan::RankPlan& plan, const rankplan::Spec& spec, const std::vector<StepInput>& inputs,
                                  std::optional<uint64_t> graph) override;
  void communicate(const rankplan::Instruction& ins) override;
  void synchronize() override;
  void close() override;
  uint64_t live_bytes() const { return live_bytes_; }
  static uint32_t token_for(uint64_t request, uint32_t position, uint32_t vocab);

 private:
  void log(const std::string& e) { trace_->add("rank" + std::to_string(rank_) + ":" + e); }
  std::shared_ptr<Trace> trace_;
  uint32_t rank_;
  std::map<uint64_t, uint64_t> buffers_;
  std::map<uint64_t, rankplan::Bucket> graphs_;
  uint64_t next_ = 1, live_bytes_ = 0;
  bool compiled_ = false, prepared_ = false, closed_ = false;
};

// A backend that is not built in this configuration: every call reports NotImplemented.
class UnavailableBackend : public Backend {
 public:
  explicit UnavailableBackend(std::string what) : what_(std::move(what)) {}
  std::string kind() const override { return what_; }
  void compile_kernels(const rankplan::Artifact&) override { no(); }
  void prepare(const rankplan::RankPlan&) override { no(); }
  void upload_weights(const std::string&) override { no(); }
  uint64_t allocate(uint64_t) override { no(); }
  void release(uint64_t) override { no(); }
  void warmup(const rankplan::Spec&) override { no(); }
  uint64_t capture(rankplan::Bucket) override { no(); }
  void validate_graph(uint64_t, rankplan::Bucket) override { no(); }
  void reset_scratch() override { no(); }
  std::vector<StepOutput> execute(const rankplan::RankPlan&, const rankplan::Spec&, const std::vector<StepInput>&, std::optional<uint64_t>) override { no(); }
  void communicate(const rankplan::Instruction&) override { no(); }
  void synchronize() override { no(); }
  void close() override {}

 private:
  [[noreturn]] void no() const { fail(ErrorKind::NotImplemented, what_ + " backend is not available in this build"); }
  std::string what_;
};

class Runtime {
 public:
  Runtime(rankplan::Artifact artifact, rankplan::Role role, uint32_t rank, std::unique_ptr<Backend> backend);
  // Runs the start-up stages in order; `fail_at` injects a failure when that stage is reached.
  void start(const std::string& weights, std::optional<Stage> fail_at = std::nullopt);
  // Executes one step in the smallest captured bucket that fits (batch, context).
  std::vector<StepOutput> step(const std::vector<StepInput>& inputs);
  void close();
  Stage stage() const { return stage_; }
  bool ready() const { return stage_ == Stage::Ready; }
  const rankplan::RankPlan& plan() const { return plan_; }

 private:
  void enter(Stage s, std::optional<Stage> fail_at);
  rankplan::Artifact artifact_;
  rankplan::RankPlan plan_;
  std::unique_ptr<Backend> backend_;
  Stage stage_ = Stage::Validate;
  std::map<std::pair<uint32_t, uint32_t>, uint64_t> graphs_;   // (batch, context) -> graph
};

// One thread per rank; `step` fans a command out and waits for all ranks (generation counter + condvar).
// A rank that throws marks the group failed: the submitter is woken and every later call fails.
class WorkerGroup {
 public:
  using Work = std::function<void(uint32_t rank, uint64_t generation)>;
  WorkerGroup(uint32_t ranks, Work work);
  ~WorkerGroup();
  void step();                       // throws if any rank failed (now or earlier)
  bool healthy() const { return !failed_.load(); }
  std::string failure() const;
  uint64_t generation() const { return generation_; }

 private:
  void loop(uint32_t rank);
  Work work_;
  std::vector<std::thread> threads_;
  mutable std::mutex mu_;
  std::condition_variable cv_work_, cv_done_;
  uint64_t generation_ = 0;
  uint32_t pending_ = 0;
  bool stopping_ = false;
  std::atomic<bool> failed_{false};
  std::string failure_;
};

// Flips to unhealthy exactly once; admission paths consult it before queueing work.
class HealthGuard {
 public:
  bool healthy() const { return healthy_.load(); }
  void fail(const std::string& why);
  std::string reason() const;

 private:
  std::atomic<bool> healthy_{true};
  mutable std::mutex mu_;
  std::string reason_;
};

// ---- prefill -> decode transfer ----------------------------------------------------------------------
struct TransferLease { uint64_t request = 0, epoch = 0, generation = 0; std::vector<uint32_t> pages; uint32_t slot = 0; uint32_t tokens = 0; };

class ResourcePool {
 public:
  ResourcePool(uint32_t pages, uint32_t slots, uint32_t page_tokens);
  TransferLease reserve(uint64_t request, uint64_t epoch, uint32_t tokens);
  void check(const TransferLease& l) const;                 // stale epoch / recycled generation are rejected
  TransferLease ensure(const TransferLease& l, uint32_t tokens);   // grow to cover `tokens`
  void retire(const TransferLease& l);                      // pages return after the next completion fence
  void completion_fence();
  size_t allocations() const { return live_.size(); }
  size_t retired() const { return limbo_pages_.size(); }
  size_t free_pages() const { return free_pages_.size(); }

 private:
  uint32_t page_tokens_;
  std::vector<uint32_t> free_pages_, free_slots_, limbo_pages_, limbo_slots_;
  std::map<uint64_t, TransferLease> live_;
  uint64_t next_generation_ = 1;
};

struct TransferManifest {       // what the prefill side hands over
  uint64_t request = 0, epoch = 0;
  std::string artifact_key;
  uint32_t consumed = 0;        // tokens whose state is included (exact boundary)
  uint32_t next_token = 0;
  std::vector<uint64_t> region_hashes;   // one per layer region
  uint64_t sampler_seed = 0, sampler_counter = 0;
};

class InMemoryTransport {
 public:
  enum class State { Reserved, InFlight, Complete, Committed, Acknowledged };
  InMemoryTransport(std::string artifact_key, uint32_t pages, uint32_t slots, uint32_t page_tokens);
  TransferLease reserve(uint64_t request, uint64_t epoch, uint32_t tokens);
  void transfer(const TransferManifest& m);         // Reserved -> InFlight (idempotent for an identical manifest)
  void complete(const TransferLease& l);            // InFlight -> Complete
  TransferManifest commit(const TransferLease& l);  // Complete -> Committed (idempotent)
  void acknowledge(const TransferLease& l);         // Committed -> Acknowledged (idempotent)
  void finish(const TransferLease& l);              // releases the lease after acknowledgement
  void abort(const TransferLease& l);
  void completion_fence() { pool_.completion_fence(); }
  size_t pending() const { return entries_.size(); }
  std::optional<State> state(uint64_t request) const;
  ResourcePool& pool() { return pool_; }

 private:
  struct Entry { TransferLease lease; State state; std::optional<TransferManifest> manifest; };
  Entry& entry(const TransferLease& l);
  std::string key_;
  ResourcePool pool_;
  std::map<uint64_t, Entry> entries_;
};

// Registered-memory transport between engines (e.g. over NVLink peer copies or a NIC). Interface only.
class RegisteredTransport {
 public:
  virtual ~RegisteredTransport() = default;
  virtual uint64_t register_region(void* base, uint64_t bytes) = 0;
  virtual void unregister_region(uint64_t registration) = 0;
  virtual uint64_t post_write(uint64_t registration, uint64_t offset, uint64_t bytes, uint32_t peer) = 0;
  virtual bool poll(uint64_t handle) = 0;
};
class UnavailableTransport : public RegisteredTransport {
 public:
  uint64_t register_region(void*, uint64_t) override { fail(ErrorKind::NotImplemented, "registered transport"); }
  void unregister_region(uint64_t) override { fail(ErrorKind::NotImplemented, "registered transport"); }
  uint64_t post_write(uint64_t, uint64_t, uint64_t, uint32_t) override { fail(ErrorKind::NotImplemented, "registered transport"); }
  bool poll(uint64_t) override { fail(ErrorKind::NotImplemented, "registered transport"); }
};

}  // namespace ifab::runtime
