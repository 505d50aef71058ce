// Serving core: the engine contract, engines, and the service that owns one engine on a worker thread.
//
//   ResidentEngine   what a model executor offers to the server: a fixed number of resident sequence slots, one
//                    packed step (prefill chunks and decode rows of several sequences at once -> one sampled token
//                    per sampling slice), per-slot sampling parameters, slot release. Nothing else crosses it.
//   MockEngine       deterministic CPU engine (token = hash of the sequence so far) with injectable latency and
//                    failures: drives the server in tests and in `ifab-server --mock`
//   PipeEngine       the same contract over a Unix-domain socket with newline-delimited JSON: the GPU engine lives
//                    in worker processes (one per GPU, PyTorch + the sm_100a kernel library); rank 0 connects here
//   Service          admission (bounded queue -> Overloaded, unhealthy -> Unavailable), the continuous-batching loop
//                    (LiveScheduler plan -> engine step -> commit), bounded per-request output streams with
//                    back-pressure, cancellation, fail-closed health, drain on shutdown, counters for /metrics
// Reference: frontend/src/{native_backend.rs,program_worker.rs,backend.rs}, vendor/rust/src/llm/src/backend.rs:13-21.
#pragma once
#include <condition_variable>
#include <future>
#include <thread>
#include <unordered_map>

#include "scheduler.h"

namespace ifab::serve {

struct SamplingParams {
  double temperature = 0.0;          // 0 = greedy
  int32_t top_k = 0;                 // 0 = off
  double top_p = 1.0, min_p = 0.0;
  double presence_penalty = 0.0, frequency_penalty = 0.0, repetition_penalty = 1.0;
  std::optional<uint64_t> seed;
  uint32_t max_tokens = 16, min_tokens = 0;
  std::vector<uint32_t> stop_token_ids;
  bool ignore_eos = false;
  int32_t logprobs = -1;             // -1 = none
  std::string cache_salt;            // prefix-cache isolation: requests share cached prefixes only with requests of the same salt
  bool greedy() const { return temperature <= 0.0 || top_k == 1; }
  void validate() const;             // throws Invalid
  Json to_json() const;
  static SamplingParams from_json(const Json& j, const SamplingParams& defaults);
  // Defaults of a deployment: the model-card recommendation (temperature 1, top-k 20, presence penalty 2, the rest neutral),
  // then every sampling key of `generation_config.json` in `dir_or_file` that is present and not null, then validation.
  // Reference: frontend/src/native_sampling.rs:16-39.
  static SamplingParams model_card();
  static SamplingParams deployment_defaults(const std::string& dir_or_file);
  // Request fields this engine does not implement (logit_bias, allowed_token_ids, structured outputs, prompt_logprobs ...):
  // a request carrying one is refused instead of being served without it. Reference: native_sampling.rs:44-67.
  static void refuse_unsupported(const Json& request);
};

struct EngineInfo {
  std::string model = "ifab";
  uint32_t residents = 1, token_budget = 8, chunk = 8, context = 512, vocab = 0, eos = 0, world = 1;
  bool greedy_only = false, has_eos = false;
  Json to_json() const;
  static EngineInfo from_json(const Json& j);
};

class ResidentEngine {
 public:
  virtual ~ResidentEngine() = default;
  virtual EngineInfo info() const = 0;
  // a request was admitted into `resident`; may throw Capacity / Invalid (the request then fails, the slot is released)
  virtual void admit(uint32_t resident, const SamplingParams& params, uint32_t reserve_tokens) { (void)resident; (void)params; (void)reserve_tokens; }
  // one engine step; returns one token per slice (ignored where slice.sample is false). Throws Backend on failure.
  virtual std::vector<uint32_t> step(const paging::SequenceBatch& batch) = 0;
  virtual void release(uint32_t resident) { (void)resident; }
  // transfer / execution audit of the engine (bytes moved each way, launch groups, prefix-cache traffic ...); engine thread only
  virtual Json audit() { return Json::object(); }
  virtual void shutdown() {}
};

class MockEngine : public ResidentEngine {
 public:
  explicit MockEngine(EngineInfo info, uint32_t step_micros = 0) : info_(std::move(info)), step_micros_(step_micros), history_(info_.residents) {}
  EngineInfo info() const override { return info_; }
  void admit(uint32_t resident, const SamplingParams&, uint32_t) override { history_.at(resident).clear(); }
  std::vector<uint32_t> step(const paging::SequenceBatch& batch) override;
  void release(uint32_t resident) override { history_.at(resident).clear(); }
  Json audit() override;
  void fail_after(uint64_t steps) { fail_after_ = steps; }      // the step with this ordinal throws Backend
  uint64_t steps() const { return steps_; }
  // the token the mock produces after `sequence`
  static uint32_t next_token(const std::vector<uint32_t>& sequence, uint32_t vocab);

 private:
  EngineInfo info_;
  uint32_t step_micros_;
  std::vector<std::vector<uint32_t>> history_;
  uint64_t steps_ = 0, rows_ = 0;
  std::optional<uint64_t> fail_after_;
};

// Client side of the engine-worker protocol. One request line, one response line:
//   {"op":"info"}                                              -> {"ok":true,"info":{...}}
//   {"op":"admit","resident":r,"reserve":n,"sampling":{...}}   -> {"ok":true}
//   {"op":"step","slices":[[resident,position,count,sample]..],"tokens":[..]} -> {"ok":true,"tokens":[..]}
//   {"op":"release","resident":r} / {"op":"shutdown"}          -> {"ok":true}
// An {"ok":false,"kind":"capacity|invalid|backend","error":"..."} response becomes the matching Error.
class PipeEngine : public ResidentEngine {
 public:
  // listens on `socket_path` and waits up to `accept_seconds` for the worker to connect
  // `watch_pid`: a child process expected to connect; when it exits first the wait ends at once with a Backend error
  PipeEngine(const std::string& socket_path, double accept_seconds, double io_seconds = 120.0, long watch_pid = 0);
  ~PipeEngine() override;
  EngineInfo info() const override { return info_; }
  void admit(uint32_t resident, const SamplingParams& params, uint32_t reserve_tokens) override;
  std::vector<uint32_t> step(const paging::SequenceBatch& batch) override;
  void release(uint32_t resident) override;
  Json audit() override;
  void shutdown() override;

 private:
  Json call(const Json& request);
  int listen_fd_ = -1, fd_ = -1;
  std::string path_, inbuf_;
  double io_seconds_;
  EngineInfo info_;
};

// ---- output stream of one request -------------------------------------------------------------------------------
struct StreamItem {
  std::optional<uint32_t> token;
  std::optional<sched::Finish> finish;
  std::string error;
  ErrorKind error_kind = ErrorKind::Backend;   // of a terminal Finish::Error: Capacity when admission refused the request after all
};

class Stream {
 public:
  explicit Stream(size_t capacity) : cap_(capacity) {}
  bool push(StreamItem item);                                   // false when full (never blocks)
  void push_terminal(StreamItem item);                          // always accepted
  std::optional<StreamItem> pop(double timeout_seconds);        // nullopt on timeout
  size_t free_slots() const;
  void close_reader() { reader_gone_.store(true); }             // the client went away
  bool reader_gone() const { return reader_gone_.load(); }

 private:
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<StreamItem> q_;
  size_t cap_;
  std::atomic<bool> reader_gone_{false};
};

struct GenerateRequest {
  std::string request_id;
  std::vector<uint32_t> prompt;
  SamplingParams sampling;
};

struct ServiceOptions {
  uint32_t queue = 256;            // admission bound
  uint32_t stream_capacity = 64;   // tokens buffered per request before it is back-pressured
  uint32_t idle_micros = 2000;
};

// cumulative latency histogram (Prometheus style): count of observations <= each bound, sum and total count
struct Histogram {
  static constexpr int N = 14;
  static constexpr double kBounds[N] = {0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.2, 0.5, 1.0, 2.0, 5.0, 10.0, 30.0};
  uint64_t bucket[N] = {};
  uint64_t count = 0;
  double sum = 0.0;
  void observe(double seconds) {
    for (int i = 0; i < N; ++i)
      if (seconds <= kBounds[i]) ++bucket[i];
    ++count;
    sum += seconds;
  }
};

struct Counters {
  uint64_t requests_total = 0, requests_finished = 0, requests_failed = 0, requests_cancelled = 0, rejected_overloaded = 0,
           rejected_unavailable = 0, prompt_tokens = 0, generated_tokens = 0, engine_steps = 0, batched_rows = 0, backpressure_skips = 0;
  double step_seconds = 0.0;
  uint32_t running = 0, queued = 0;
  Histogram ttft, inter_token;   // seconds from submission to the first token / between consecutive tokens of a request
};

class Service {
 public:
  Service(std::shared_ptr<ResidentEngine> engine, ServiceOptions opt = {});
  ~Service();
  const EngineInfo& info() const { return info_; }
  // Validates and queues; throws Invalid, Capacity (overloaded) or Backend (unavailable).
  std::shared_ptr<Stream> generate(GenerateRequest req);
  void abort(const std::string& request_id);
  void shutdown();
  bool healthy() const { return health_.healthy(); }
  std::string unhealthy_reason() const { return health_.reason(); }
  Counters counters() const;
  std::string metrics_text() const;     // Prometheus exposition format
  // The engine's audit record, fetched by the engine thread between two steps (throws Backend when the engine is down or
  // does not answer within `timeout_seconds`).
  Json engine_audit(double timeout_seconds = 10.0);

 private:
  void run();
  struct Live {
    std::string name; std::shared_ptr<Stream> stream; SamplingParams sampling; uint32_t reserve = 0;
    double t_submit = 0.0, t_last = 0.0;   // for the latency histograms
  };
  std::shared_ptr<ResidentEngine> engine_;
  EngineInfo info_;
  ServiceOptions opt_;
  runtime::HealthGuard health_;
  mutable std::mutex mu_;
  std::deque<std::pair<sched::Request, Live>> inbox_;
  uint32_t handing_over_ = 0;   // requests taken out of the inbox that the scheduler has not counted yet (guarded by mu_)
  std::vector<uint64_t> aborts_;
  std::unordered_map<std::string, uint64_t> ids_;
  uint64_t next_id_ = 1;
  std::atomic<bool> stop_{false};
  std::vector<std::shared_ptr<std::promise<Json>>> audit_waiters_;
  Counters counters_;
  std::thread worker_;
};

}  // namespace ifab::serve
