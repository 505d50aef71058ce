#include "runtime.h"

#include <algorithm>

namespace ifab::runtime {

const char* stage_name(Stage s) {
  switch (s) {
    case Stage::Validate: return "validate";
    case Stage::Compile: return "compile";
    case Stage::Prepare: return "prepare";
    case Stage::Warmup: return "warmup";
    case Stage::Capture: return "capture";
    case Stage::ValidateReplay: return "validate_replay";
    case Stage::Reset: return "reset";
    case Stage::Ready: return "ready";
    case Stage::Failed: return "failed";
    case Stage::Closed: return "closed";
  }
  return "?";
}

void Trace::add(const std::string& e) {
  std::lock_guard<std::mutex> g(mu_);
  events_.push_back(e);
}
std::vector<std::string> Trace::events() const {
  std::lock_guard<std::mutex> g(mu_);
  return events_;
}
size_t Trace::count(const std::string& needle) const {
  std::lock_guard<std::mutex> g(mu_);
  size_t n = 0;
  for (auto& e : events_) n += e.find(needle) != std::string::npos;
  return n;
}

// ---------------------------------------------------------------------------------------------
void MockBackend::compile_kernels(const rankplan::Artifact& a) {
  log("compile " + a.key);
  compiled_ = true;
}
void MockBackend::prepare(const rankplan::RankPlan& plan) {
  if (!compiled_) invalid("mock: prepare before compile");
  log("prepare " + std::string(rankplan::role_name(plan.role)) + " rank " + std::to_string(plan.rank));
  prepared_ = true;
}
void MockBackend::upload_weights(const std::string& source) { log("weights " + source); }
uint64_t MockBackend::allocate(uint64_t bytes) {
  if (bytes == 0) invalid("mock: zero-byte allocation");
  buffers_[next_] = bytes;
  live_bytes_ += bytes;
  log("allocate " + std::to_string(bytes));
  return next_++;
}
void MockBackend::release(uint64_t buffer) {
  auto it = buffers_.find(buffer);
  if (it == buffers_.end()) invalid("mock: unknown buffer");
  live_bytes_ -= it->second;
  buffers_.erase(it);
  log("release");
}
void MockBackend::warmup(const rankplan::Spec& spec) { log("warmup ctx " + std::to_string(spec.max_context())); }
uint64_t MockBackend::capture(rankplan::Bucket b) {
  if (!prepared_) invalid("mock: capture before prepare");
  graphs_[next_] = b;
  log("capture " + std::to_string(b.batch) + "x" + std::to_string(b.context));
  return next_++;
}
void MockBackend::validate_graph(uint64_t graph, rankplan::Bucket b) {
  auto it = graphs_.find(graph);
  if (it == graphs_.end() || it->second.batch != b.batch || it->second.context != b.context) invalid("mock: graph does not match its bucket");
  log("validate_graph");
}
void MockBackend::reset_scratch() { log("reset"); }
uint32_t MockBackend::token_for(uint64_t request, uint32_t position, uint32_t vocab) {
  uint64_t h = request * 0x9e3779b97f4a7c15ull + position * 0xbf58476d1ce4e5b9ull;
  h ^= h >> 31;
  h *= 0x94d049bb133111ebull;
  h ^= h >> 29;
  return (uint32_t)(h % vocab);
}
std::vector<StepOutput> MockBackend::execute(const rankplan::RankPlan& plan, const rankplan::Spec& spec, const std::vector<StepInput>& inputs,
                                             std::optional<uint64_t> graph) {
  if (closed_) invalid("mock: execute after close");
  if (graph && !graphs_.count(*graph)) invalid("mock: unknown graph");
  for (auto& ins : plan.instructions)
    if (ins.kind == rankplan::Instruction::Kind::Communication) communicate(ins);
  std::vector<StepOutput> out;
  for (auto& in : inputs) {
    if (in.tokens.empty()) invalid("mock: empty step input");
    out.push_back({in.request, token_for(in.request, in.position + (uint32_t)in.tokens.size(), spec.model.vocab), (uint32_t)in.tokens.size()});
  }
  log("execute " + std::to_string(inputs.size()) + (graph ? " graph" : " eager"));
  return out;
}
void MockBackend::communicate(const rankplan::Instruction& ins) { log("comm " + ins.name + " " + ins.group); }
void MockBackend::synchronize() { log("sync"); }
void MockBackend::close() {
  closed_ = true;
  log("close");
}

// ---------------------------------------------------------------------------------------------
Runtime::Runtime(rankplan::Artifact artifact, rankplan::Role role, uint32_t rank, std::unique_ptr<Backend> backend)
    : artifact_(std::move(artifact)), backend_(std::move(backend)) {
  bool found = false;
  for (auto& p : artifact_.plans)
    if (p.role == role && p.rank == rank) {
      plan_ = p;
      found = true;
    }
  if (!found) invalid("runtime: artifact has no plan for this role/rank");
}

void Runtime::enter(Stage s, std::optional<Stage> fail_at) {
  stage_ = s;
  if (fail_at && *fail_at == s) fail(ErrorKind::Backend, std::string("injected failure at stage ") + stage_name(s));
}

void Runtime::start(const std::string& weights, std::optional<Stage> fail_at) {
  if (stage_ != Stage::Validate) invalid("runtime: start() may run once");
  try {
    enter(Stage::Validate, fail_at);
    artifact_.spec.validate();
    if (artifact_.key != rankplan::content_key(artifact_.spec, artifact_.target)) fail(ErrorKind::Stale, "runtime: artifact key does not match its contents");
    enter(Stage::Compile, fail_at);
    backend_->compile_kernels(artifact_);
    enter(Stage::Prepare, fail_at);
    backend_->prepare(plan_);
    backend_->upload_weights(weights);
    enter(Stage::Warmup, fail_at);
    backend_->warmup(artifact_.spec);
    enter(Stage::Capture, fail_at);
    if (plan_.role == rankplan::Role::Decode)
      for (auto& b : artifact_.buckets) graphs_[{b.batch, b.context}] = backend_->capture(b);
    enter(Stage::ValidateReplay, fail_at);
    for (auto& kv : graphs_) backend_->validate_graph(kv.second, {kv.first.first, kv.first.second});
    enter(Stage::Reset, fail_at);
    backend_->reset_scratch();
    backend_->synchronize();
    enter(Stage::Ready, fail_at);
  } catch (...) {
    stage_ = Stage::Failed;
    try { backend_->close(); } catch (...) {}
    throw;
  }
}

std::vector<StepOutput> Runtime::step(const std::vector<StepInput>& inputs) {
  if (stage_ != Stage::Ready) fail(ErrorKind::Backend, std::string("runtime is ") + stage_name(stage_) + ", not ready");
  if (inputs.empty()) invalid("runtime: empty step");
  std::optional<uint64_t> graph;
  if (plan_.role == rankplan::Role::Decode) {
    uint32_t ctx = 0;
    for (auto& in : inputs) ctx = std::max<uint32_t>(ctx, in.position + (uint32_t)in.tokens.size());
    // smallest bucket that fits
    for (auto& kv : graphs_)
      if (kv.first.first >= inputs.size() && kv.first.second >= ctx) {
        graph = kv.second;
        break;
      }
    if (!graph) fail(ErrorKind::Capacity, "runtime: no captured bucket fits batch " + std::to_string(inputs.size()) + " context " + std::to_string(ctx));
  } else {
    uint32_t budget = 0;
    for (auto& in : inputs) budget += (uint32_t)in.tokens.size();
    if (budget > artifact_.spec.token_budget) fail(ErrorKind::Capacity, "runtime: prefill step exceeds the token budget");
  }
  try {
    return backend_->execute(plan_, artifact_.spec, inputs, graph);
  } catch (...) {
    stage_ = Stage::Failed;
    throw;
  }
}

void Runtime::close() {
  if (stage_ == Stage::Closed) return;
  if (stage_ != Stage::Failed) backend_->close();
  stage_ = Stage::Closed;
}

// ---------------------------------------------------------------------------------------------
WorkerGroup::WorkerGroup(uint32_t ranks, Work work) : work_(std::move(work)) {
  if (ranks == 0 || ranks > 64) invalid("worker group: ranks out of range");
  for (uint32_t r = 0; r < ranks; ++r) threads_.emplace_back([this, r] { loop(r); });
}
WorkerGroup::~WorkerGroup() {
  {
    std::lock_guard<std::mutex> g(mu_);
    stopping_ = true;
  }
  cv_work_.notify_all();
  for (auto& t : threads_) t.join();
}
void WorkerGroup::loop(uint32_t rank) {
  uint64_t seen = 0;
  for (;;) {
    uint64_t gen;
    {
      std::unique_lock<std::mutex> l(mu_);
      cv_work_.wait(l, [&] { return stopping_ || generation_ != seen; });
      if (stopping_) return;
      gen = seen = generation_;
    }
    bool ok = true;
    std::string why;
    if (!failed_.load()) {
      try {
        work_(rank, gen);
      } catch (const std::exception& e) {
        ok = false;
        why = e.what();
      } catch (...) {
        ok = false;
        why = "unknown failure";
      }
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      if (!ok && !failed_.exchange(true)) failure_ = "rank " + std::to_string(rank) + ": " + why;
      --pending_;
    }
    cv_done_.notify_all();
  }
}
void WorkerGroup::step() {
  std::unique_lock<std::mutex> l(mu_);
  if (failed_.load()) fail(ErrorKind::Backend, "worker group failed earlier: " + failure_);
  pending_ = (uint32_t)threads_.size();
  ++generation_;
  cv_work_.notify_all();
  cv_done_.wait(l, [&] { return pending_ == 0; });
  if (failed_.load()) fail(ErrorKind::Backend, "worker group failed: " + failure_);
}
std::string WorkerGroup::failure() const {
  std::lock_guard<std::mutex> g(mu_);
  return failure_;
}

void HealthGuard::fail(const std::string& why) {
  std::lock_guard<std::mutex> g(mu_);
  if (healthy_.exchange(false)) reason_ = why;
}
std::string HealthGuard::reason() const {
  std::lock_guard<std::mutex> g(mu_);
  return reason_;
}

// ---------------------------------------------------------------------------------------------
ResourcePool::ResourcePool(uint32_t pages, uint32_t slots, uint32_t page_tokens) : page_tokens_(page_tokens) {
  if (pages == 0 || slots == 0 || page_tokens == 0) invalid("resource pool: sizes must be positive");
  for (uint32_t p = pages; p-- > 0;) free_pages_.push_back(p);
  for (uint32_t s = slots; s-- > 0;) free_slots_.push_back(s);
}
TransferLease ResourcePool::reserve(uint64_t request, uint64_t epoch, uint32_t tokens) {
  if (tokens == 0) invalid("resource pool: empty reservation");
  if (live_.count(request)) invalid("resource pool: request already holds a lease");
  const uint32_t need = (tokens + page_tokens_ - 1) / page_tokens_;
  if (free_pages_.size() < need || free_slots_.empty()) fail(ErrorKind::Capacity, "resource pool: out of pages or slots");
  TransferLease l;
  l.request = request;
  l.epoch = epoch;
  l.generation = next_generation_++;
  l.tokens = tokens;
  for (uint32_t k = 0; k < need; ++k) {
    l.pages.push_back(free_pages_.back());
    free_pages_.pop_back();
  }
  l.slot = free_slots_.back();
  free_slots_.pop_back();
  live_[request] = l;
  return l;
}
void ResourcePool::check(const TransferLease& l) const {
  auto it = live_.find(l.request);
  if (it == live_.end()) fail(ErrorKind::Stale, "resource pool: lease is not live");
  if (it->second.epoch != l.epoch) fail(ErrorKind::Stale, "resource pool: stale epoch");
  if (it->second.generation != l.generation) fail(ErrorKind::Stale, "resource pool: stale generation");
}
TransferLease ResourcePool::ensure(const TransferLease& l, uint32_t tokens) {
  check(l);
  TransferLease& cur = live_[l.request];
  const uint32_t need = (tokens + page_tokens_ - 1) / page_tokens_;
  if (need > cur.pages.size()) {
    if (free_pages_.size() < need - cur.pages.size()) fail(ErrorKind::Capacity, "resource pool: out of pages");
    while (cur.pages.size() < need) {
      cur.pages.push_back(free_pages_.back());
      free_pages_.pop_back();
    }
  }
  cur.tokens = std::max(cur.tokens, tokens);
  return cur;
}
void ResourcePool::retire(const TransferLease& l) {
  check(l);
  TransferLease cur = live_[l.request];
  live_.erase(l.request);
  for (uint32_t p : cur.pages) limbo_pages_.push_back(p);
  limbo_slots_.push_back(cur.slot);
}
void ResourcePool::completion_fence() {
  for (uint32_t p : limbo_pages_) free_pages_.push_back(p);
  for (uint32_t s : limbo_slots_) free_slots_.push_back(s);
  limbo_pages_.clear();
  limbo_slots_.clear();
}

InMemoryTransport::InMemoryTransport(std::string artifact_key, uint32_t pages, uint32_t slots, uint32_t page_tokens)
    : key_(std::move(artifact_key)), pool_(pages, slots, page_tokens) {}
TransferLease InMemoryTransport::reserve(uint64_t request, uint64_t epoch, uint32_t tokens) {
  TransferLease l = pool_.reserve(request, epoch, tokens);
  entries_[request] = Entry{l, State::Reserved, std::nullopt};
  return l;
}
InMemoryTransport::Entry& InMemoryTransport::entry(const TransferLease& l) {
  pool_.check(l);
  auto it = entries_.find(l.request);
  if (it == entries_.end()) fail(ErrorKind::Stale, "transport: unknown transfer");
  return it->second;
}
void InMemoryTransport::transfer(const TransferManifest& m) {
  auto it = entries_.find(m.request);
  if (it == entries_.end()) fail(ErrorKind::Stale, "transport: no reservation for request " + std::to_string(m.request));
  Entry& e = it->second;
  if (m.epoch != e.lease.epoch) fail(ErrorKind::Stale, "transport: manifest from a stale epoch");
  if (m.artifact_key != key_) invalid("transport: manifest was produced by a different artifact");
  if (m.consumed == 0 || m.consumed > e.lease.tokens) invalid("transport: consumed length outside the reservation");
  if (e.state != State::Reserved) {
    // duplicates of the same manifest are harmless; anything else is a protocol error
    if (e.manifest && e.manifest->consumed == m.consumed && e.manifest->next_token == m.next_token && e.manifest->region_hashes == m.region_hashes) return;
    invalid("transport: conflicting manifest for a transfer already in flight");
  }
  e.manifest = m;
  e.state = State::InFlight;
}
void InMemoryTransport::complete(const TransferLease& l) {
  Entry& e = entry(l);
  if (e.state == State::Complete || e.state == State::Committed || e.state == State::Acknowledged) return;
  if (e.state != State::InFlight) invalid("transport: complete before transfer");
  e.state = State::Complete;
}
TransferManifest InMemoryTransport::commit(const TransferLease& l) {
  Entry& e = entry(l);
  if (e.state == State::Committed || e.state == State::Acknowledged) return *e.manifest;
  if (e.state != State::Complete) invalid("transport: commit before completion");
  e.state = State::Committed;
  return *e.manifest;
}
void InMemoryTransport::acknowledge(const TransferLease& l) {
  Entry& e = entry(l);
  if (e.state == State::Acknowledged) return;
  if (e.state != State::Committed) invalid("transport: acknowledge before commit");
  e.state = State::Acknowledged;
}
void InMemoryTransport::finish(const TransferLease& l) {
  Entry& e = entry(l);
  if (e.state != State::Acknowledged) invalid("transport: finish before acknowledgement");
  pool_.retire(l);
  entries_.erase(l.request);
}
void InMemoryTransport::abort(const TransferLease& l) {
  entry(l);
  pool_.retire(l);
  entries_.erase(l.request);
}
std::optional<InMemoryTransport::State> InMemoryTransport::state(uint64_t request) const {
  auto it = entries_.find(request);
  if (it == entries_.end()) return std::nullopt;
  return it->second.state;
}

}  // namespace ifab::runtime
