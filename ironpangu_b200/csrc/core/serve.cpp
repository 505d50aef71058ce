#include "serve.h"

#include <sys/stat.h>

#include <poll.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>

namespace ifab::serve {

namespace {
double now_seconds() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
double num(const Json& j, const char* key, double dflt) {
  const Json* v = j.find(key);
  if (!v || v->is_null()) return dflt;
  if (!v->is_number()) invalid(std::string("sampling: '") + key + "' must be a number");
  return v->as_double();
}
}  // namespace

// ---- sampling parameters ----------------------------------------------------------------------------------------
void SamplingParams::validate() const {
  if (!(temperature >= 0.0) || temperature > 100.0) invalid("sampling: temperature must be in [0, 100]");
  if (top_k < 0) invalid("sampling: top_k must be >= 0 (0 disables it)");
  if (!(top_p > 0.0) || top_p > 1.0) invalid("sampling: top_p must be in (0, 1]");
  if (!(min_p >= 0.0) || min_p > 1.0) invalid("sampling: min_p must be in [0, 1]");
  if (presence_penalty < -2.0 || presence_penalty > 2.0) invalid("sampling: presence_penalty must be in [-2, 2]");
  if (frequency_penalty < -2.0 || frequency_penalty > 2.0) invalid("sampling: frequency_penalty must be in [-2, 2]");
  if (!(repetition_penalty > 0.0) || repetition_penalty > 2.0) invalid("sampling: repetition_penalty must be in (0, 2]");
  if (max_tokens == 0) invalid("sampling: max_tokens must be positive");
  if (min_tokens > max_tokens) invalid("sampling: min_tokens exceeds max_tokens");
  if (logprobs >= 0) invalid("sampling: logprobs are not supported by this server");
}

Json SamplingParams::to_json() const {
  Json j = Json::object();
  j.set("temperature", temperature);
  j.set("top_k", (int64_t)top_k);
  j.set("top_p", top_p);
  j.set("min_p", min_p);
  j.set("presence_penalty", presence_penalty);
  j.set("frequency_penalty", frequency_penalty);
  j.set("repetition_penalty", repetition_penalty);
  if (seed) j.set("seed", (int64_t)*seed);
  j.set("max_tokens", (int64_t)max_tokens);
  if (!cache_salt.empty()) j.set("cache_salt", cache_salt);
  return j;
}

SamplingParams SamplingParams::from_json(const Json& j, const SamplingParams& d) {
  SamplingParams s = d;
  if (!j.is_object()) invalid("sampling parameters must be a JSON object");
  s.temperature = num(j, "temperature", d.temperature);
  s.top_k = (int32_t)num(j, "top_k", d.top_k);
  if (s.top_k < 0) s.top_k = 0;   // -1 is the conventional "off"
  s.top_p = num(j, "top_p", d.top_p);
  s.min_p = num(j, "min_p", d.min_p);
  s.presence_penalty = num(j, "presence_penalty", d.presence_penalty);
  s.frequency_penalty = num(j, "frequency_penalty", d.frequency_penalty);
  s.repetition_penalty = num(j, "repetition_penalty", d.repetition_penalty);
  if (const Json* v = j.find("seed"); v && !v->is_null()) s.seed = (uint64_t)v->as_int();
  if (const Json* v = j.find("max_tokens"); v && !v->is_null()) {
    if (v->as_int() <= 0) invalid("sampling: max_tokens must be positive");
    s.max_tokens = (uint32_t)v->as_int();
  }
  if (const Json* v = j.find("max_completion_tokens"); v && !v->is_null()) s.max_tokens = (uint32_t)std::max<int64_t>(1, v->as_int());
  if (const Json* v = j.find("min_tokens"); v && !v->is_null()) s.min_tokens = (uint32_t)std::max<int64_t>(0, v->as_int());
  if (const Json* v = j.find("ignore_eos"); v && !v->is_null()) s.ignore_eos = v->as_bool();
  if (const Json* v = j.find("stop_token_ids"); v && !v->is_null())
    for (auto& t : v->as_array()) s.stop_token_ids.push_back((uint32_t)t.as_int());
  if (const Json* v = j.find("cache_salt"); v && !v->is_null()) {
    if (!v->is_string() || v->as_string().size() > 256) invalid("sampling: cache_salt must be a string of at most 256 bytes");
    s.cache_salt = v->as_string();
  }
  if (const Json* v = j.find("logprobs"); v && !v->is_null()) s.logprobs = v->is_bool() ? (v->as_bool() ? 1 : -1) : (int32_t)v->as_int();
  return s;
}

SamplingParams SamplingParams::model_card() {
  SamplingParams s;
  s.temperature = 1.0;
  s.top_k = 20;
  s.presence_penalty = 2.0;
  return s;
}

SamplingParams SamplingParams::deployment_defaults(const std::string& dir_or_file) {
  SamplingParams s = model_card();
  std::string path = dir_or_file;
  struct stat st {};
  if (!path.empty() && ::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode)) path += "/generation_config.json";
  if (!path.empty() && ::stat(path.c_str(), &st) == 0) {
    const Json cfg = Json::parse(read_file(path, 1 << 20));
    if (!cfg.is_object()) invalid("generation config: " + path + " is not a JSON object");
    Json only = Json::object();
    for (const char* key : {"temperature", "top_k", "top_p", "min_p", "presence_penalty", "frequency_penalty", "repetition_penalty"})
      if (const Json* v = cfg.find(key); v && !v->is_null()) only.set(key, *v);
    const uint32_t keep = s.max_tokens;
    s = from_json(only, s);
    s.max_tokens = keep;
  } else if (!dir_or_file.empty() && ::stat(dir_or_file.c_str(), &st) != 0) {
    invalid("generation config: " + dir_or_file + " does not exist");
  }
  s.validate();
  return s;
}

void SamplingParams::refuse_unsupported(const Json& request) {
  static const char* const kUnsupported[] = {"logit_bias", "allowed_token_ids", "bad_words", "bad_words_token_ids", "structured_outputs",
                                             "guided_json", "guided_regex", "guided_choice", "guided_grammar", "response_format",
                                             "prompt_logprobs", "logprob_token_ids", "repetition_detection", "thinking_token_budget",
                                             "lora_request", "mm_features", "data_parallel_rank", "best_of", "use_beam_search"};
  auto scan = [](const Json& o) {
    if (!o.is_object()) return;
    for (const char* key : kUnsupported)
      if (const Json* v = o.find(key); v && !v->is_null())
        fail(ErrorKind::NotImplemented, std::string("sampling: '") + key + "' is not supported by this engine (supported: temperature, top_k, "
             "top_p, min_p, seed, repetition / presence / frequency penalties, min_tokens, stop_token_ids)");
  };
  scan(request);
  if (const Json* sp = request.find("sampling_params")) scan(*sp);
  if (const Json* n = request.find("n"); n && !n->is_null() && n->as_int() != 1) fail(ErrorKind::NotImplemented, "sampling: n != 1 is not supported");
  if (const Json* p = request.find("priority"); p && !p->is_null() && p->as_int() != 0) fail(ErrorKind::NotImplemented, "sampling: priority is not supported");
}

Json EngineInfo::to_json() const {
  Json j = Json::object();
  j.set("model", model);
  j.set("residents", residents);
  j.set("token_budget", token_budget);
  j.set("chunk", chunk);
  j.set("context", context);
  j.set("vocab", vocab);
  j.set("eos", eos);
  j.set("has_eos", has_eos);
  j.set("world", world);
  j.set("greedy_only", greedy_only);
  return j;
}

EngineInfo EngineInfo::from_json(const Json& j) {
  EngineInfo e;
  auto u = [&](const char* k, uint32_t d) { const Json* v = j.find(k); return v && !v->is_null() ? (uint32_t)v->as_int() : d; };
  if (const Json* v = j.find("model")) e.model = v->as_string();
  e.residents = u("residents", 1);
  e.token_budget = u("token_budget", 8);
  e.chunk = u("chunk", e.token_budget);
  e.context = u("context", 512);
  e.vocab = u("vocab", 0);
  e.eos = u("eos", 0);
  e.world = u("world", 1);
  if (const Json* v = j.find("has_eos")) e.has_eos = v->as_bool();
  if (const Json* v = j.find("greedy_only")) e.greedy_only = v->as_bool();
  if (e.residents == 0 || e.token_budget == 0 || e.chunk == 0 || e.context < 2) fail(ErrorKind::Backend, "engine reported an unusable capacity");
  return e;
}

// ---- mock engine --------------------------------------------------------------------------------------------------
uint32_t MockEngine::next_token(const std::vector<uint32_t>& seq, uint32_t vocab) {
  const uint64_t h = fnv1a64(seq.data(), seq.size() * sizeof(uint32_t));
  if (vocab <= 3) return 0;
  return 3 + (uint32_t)(h % (vocab - 3));
}

Json MockEngine::audit() {
  Json j = Json::object();
  j.set("steps", steps_);
  j.set("rows", rows_);
  return j;
}

std::vector<uint32_t> MockEngine::step(const paging::SequenceBatch& batch) {
  if (fail_after_ && steps_ >= *fail_after_) fail(ErrorKind::Backend, "mock engine: injected step failure");
  ++steps_;
  rows_ += batch.tokens.size();
  if (step_micros_) std::this_thread::sleep_for(std::chrono::microseconds(step_micros_));
  std::vector<uint32_t> out;
  size_t row = 0;
  for (const auto& sl : batch.slices) {
    auto& hist = history_.at(sl.resident);
    if (hist.size() != sl.position) fail(ErrorKind::Backend, "mock engine: slice position does not continue the resident's sequence");
    for (uint32_t k = 0; k < sl.token_count; ++k) hist.push_back((uint32_t)batch.tokens.at(row++));
    out.push_back(sl.sample ? next_token(hist, info_.vocab ? info_.vocab : 1024) : 0);
  }
  return out;
}

// ---- pipe engine ----------------------------------------------------------------------------------------------------
PipeEngine::PipeEngine(const std::string& socket_path, double accept_seconds, double io_seconds, long watch_pid)
    : path_(socket_path), io_seconds_(io_seconds) {
  sockaddr_un addr{};
  if (socket_path.size() >= sizeof(addr.sun_path)) invalid("engine socket path is too long");
  listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
  if (listen_fd_ < 0) fail(ErrorKind::Io, "engine socket: cannot create");
  addr.sun_family = AF_UNIX;
  std::strncpy(addr.sun_path, socket_path.c_str(), sizeof(addr.sun_path) - 1);
  ::unlink(socket_path.c_str());
  if (::bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)) != 0 || ::listen(listen_fd_, 1) != 0) {
    ::close(listen_fd_);
    listen_fd_ = -1;
    fail(ErrorKind::Io, "engine socket: cannot bind " + socket_path);
  }
  const double deadline = now_seconds() + accept_seconds;
  for (;;) {
    pollfd p{listen_fd_, POLLIN, 0};
    const double left = deadline - now_seconds();
    if (left <= 0) fail(ErrorKind::Backend, "engine worker did not connect in time");
    if (::poll(&p, 1, (int)(std::min(left, 0.5) * 1000)) > 0) break;
    if (watch_pid > 0) {
      int status = 0;
      if (::waitpid((pid_t)watch_pid, &status, WNOHANG) == (pid_t)watch_pid)
        fail(ErrorKind::Backend, "engine worker exited before connecting (status " + std::to_string(status) + ")");
    }
  }
  fd_ = ::accept(listen_fd_, nullptr, nullptr);
  if (fd_ < 0) fail(ErrorKind::Backend, "engine socket: accept failed");
  Json req = Json::object();
  req.set("op", "info");
  info_ = EngineInfo::from_json(call(req).at("info"));
}

PipeEngine::~PipeEngine() {
  if (fd_ >= 0) ::close(fd_);
  if (listen_fd_ >= 0) ::close(listen_fd_);
  if (!path_.empty()) ::unlink(path_.c_str());
}

Json PipeEngine::call(const Json& request) {
  if (fd_ < 0) fail(ErrorKind::Backend, "engine connection is closed");
  std::string line = request.dump();
  line.push_back('\n');
  size_t off = 0;
  while (off < line.size()) {
    const ssize_t n = ::send(fd_, line.data() + off, line.size() - off, MSG_NOSIGNAL);
    if (n <= 0) {
      ::close(fd_);
      fd_ = -1;
      fail(ErrorKind::Backend, "engine worker went away (send failed)");
    }
    off += (size_t)n;
  }
  const double deadline = now_seconds() + io_seconds_;
  for (;;) {
    const size_t nl = inbuf_.find('\n');
    if (nl != std::string::npos) {
      const std::string text = inbuf_.substr(0, nl);
      inbuf_.erase(0, nl + 1);
      Json r = Json::parse(text);
      const Json* ok = r.find("ok");
      if (ok && ok->as_bool()) return r;
      const std::string kind = r.find("kind") ? r.at("kind").as_string() : "backend";
      const std::string msg = r.find("error") ? r.at("error").as_string() : "engine error";
      if (kind == "capacity") fail(ErrorKind::Capacity, msg);
      if (kind == "invalid") invalid(msg);
      fail(ErrorKind::Backend, msg);
    }
    const double left = deadline - now_seconds();
    pollfd p{fd_, POLLIN, 0};
    if (left <= 0 || ::poll(&p, 1, (int)(left * 1000)) <= 0) {
      ::close(fd_);
      fd_ = -1;
      fail(ErrorKind::Backend, "engine worker did not answer in time");
    }
    char buf[65536];
    const ssize_t n = ::recv(fd_, buf, sizeof(buf), 0);
    if (n <= 0) {
      ::close(fd_);
      fd_ = -1;
      fail(ErrorKind::Backend, "engine worker went away (connection closed)");
    }
    inbuf_.append(buf, (size_t)n);
  }
}

void PipeEngine::admit(uint32_t resident, const SamplingParams& params, uint32_t reserve_tokens) {
  Json r = Json::object();
  r.set("op", "admit");
  r.set("resident", resident);
  r.set("reserve", reserve_tokens);
  r.set("sampling", params.to_json());
  call(r);
}

std::vector<uint32_t> PipeEngine::step(const paging::SequenceBatch& batch) {
  Json r = Json::object();
  r.set("op", "step");
  Json sl = Json::array();
  for (const auto& s : batch.slices) {
    Json one = Json::array();
    one.push((int64_t)s.resident);
    one.push((int64_t)s.position);
    one.push((int64_t)s.token_count);
    one.push((int64_t)(s.sample ? 1 : 0));
    sl.push(std::move(one));
  }
  r.set("slices", std::move(sl));
  Json toks = Json::array();
  for (int32_t t : batch.tokens) toks.push((int64_t)t);
  r.set("tokens", std::move(toks));
  const Json resp = call(r);
  std::vector<uint32_t> out;
  for (const auto& t : resp.at("tokens").as_array()) out.push_back((uint32_t)t.as_int());
  if (out.size() != batch.slices.size()) fail(ErrorKind::Backend, "engine returned a wrong number of tokens");
  return out;
}

void PipeEngine::release(uint32_t resident) {
  Json r = Json::object();
  r.set("op", "release");
  r.set("resident", resident);
  call(r);
}

Json PipeEngine::audit() {
  Json r = Json::object();
  r.set("op", "audit");
  const Json resp = call(r);
  const Json* a = resp.find("audit");
  return a ? *a : Json::object();
}

void PipeEngine::shutdown() {
  if (fd_ < 0) return;
  try {
    Json r = Json::object();
    r.set("op", "shutdown");
    call(r);
  } catch (const Error&) {
  }
}

// ---- streams ----------------------------------------------------------------------------------------------------
bool Stream::push(StreamItem item) {
  std::lock_guard<std::mutex> lk(mu_);
  if (q_.size() >= cap_) return false;
  q_.push_back(std::move(item));
  cv_.notify_one();
  return true;
}
void Stream::push_terminal(StreamItem item) {
  std::lock_guard<std::mutex> lk(mu_);
  q_.push_back(std::move(item));
  cv_.notify_one();
}
std::optional<StreamItem> Stream::pop(double timeout_seconds) {
  std::unique_lock<std::mutex> lk(mu_);
  if (!cv_.wait_for(lk, std::chrono::duration<double>(timeout_seconds), [&] { return !q_.empty(); })) return std::nullopt;
  StreamItem it = std::move(q_.front());
  q_.pop_front();
  return it;
}
size_t Stream::free_slots() const {
  std::lock_guard<std::mutex> lk(mu_);
  return q_.size() >= cap_ ? 0 : cap_ - q_.size();
}

// ---- service ------------------------------------------------------------------------------------------------------
Service::Service(std::shared_ptr<ResidentEngine> engine, ServiceOptions opt) : engine_(std::move(engine)), info_(engine_->info()), opt_(opt) {
  worker_ = std::thread([this] { run(); });
}

Service::~Service() { shutdown(); }

void Service::shutdown() {
  if (stop_.exchange(true)) {
    if (worker_.joinable()) worker_.join();
    return;
  }
  if (worker_.joinable()) worker_.join();
}

std::shared_ptr<Stream> Service::generate(GenerateRequest req) {
  req.sampling.validate();
  if (info_.greedy_only && !req.sampling.greedy()) invalid("this engine accepts greedy sampling only (temperature 0 or top_k 1)");
  if (req.prompt.empty()) invalid("request: empty prompt");
  if ((uint64_t)req.prompt.size() + req.sampling.max_tokens > info_.context)
    invalid("request: prompt (" + std::to_string(req.prompt.size()) + " tokens) + max_tokens (" + std::to_string(req.sampling.max_tokens) +
            ") exceeds the context of " + std::to_string(info_.context));
  if (info_.vocab)
    for (uint32_t t : req.prompt)
      if (t >= info_.vocab) invalid("request: token id outside the vocabulary");
  std::lock_guard<std::mutex> lk(mu_);
  if (!health_.healthy() || stop_.load()) {
    ++counters_.rejected_unavailable;
    fail(ErrorKind::Backend, "unavailable: " + (stop_.load() ? std::string("server is shutting down") : health_.reason()));
  }
  if (req.request_id.empty()) req.request_id = "req-" + std::to_string(next_id_);
  if (ids_.count(req.request_id)) invalid("request: duplicate request id");
  if (inbox_.size() + handing_over_ + counters_.queued >= opt_.queue) {
    ++counters_.rejected_overloaded;
    fail(ErrorKind::Capacity, "overloaded: the admission queue is full");
  }
  sched::Request r;
  r.id = next_id_++;
  r.prompt = std::move(req.prompt);
  r.max_new_tokens = req.sampling.max_tokens;
  r.stop_tokens = req.sampling.stop_token_ids;
  if (info_.has_eos && !req.sampling.ignore_eos) r.stop_tokens.push_back(info_.eos);
  Live live;
  live.name = req.request_id;
  live.stream = std::make_shared<Stream>(opt_.stream_capacity);
  live.sampling = req.sampling;
  live.reserve = (uint32_t)r.prompt.size() + r.max_new_tokens;
  live.t_submit = now_seconds();
  ids_[live.name] = r.id;
  ++counters_.requests_total;
  counters_.prompt_tokens += r.prompt.size();
  auto stream = live.stream;
  inbox_.emplace_back(std::move(r), std::move(live));
  return stream;
}

void Service::abort(const std::string& request_id) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = ids_.find(request_id);
  if (it != ids_.end()) aborts_.push_back(it->second);
}

Counters Service::counters() const {
  std::lock_guard<std::mutex> lk(mu_);
  return counters_;
}

std::string Service::metrics_text() const {
  const Counters c = counters();
  std::string s;
  auto line = [&](const char* name, const char* help, const char* type, double v) {
    s += std::string("# HELP ") + name + " " + help + "\n# TYPE " + name + " " + type + "\n" + name + " " + format_double(v) + "\n";
  };
  line("ifab_requests_total", "Requests accepted.", "counter", (double)c.requests_total);
  line("ifab_requests_finished_total", "Requests that ended with stop or length.", "counter", (double)c.requests_finished);
  line("ifab_requests_failed_total", "Requests that ended with an error.", "counter", (double)c.requests_failed);
  line("ifab_requests_cancelled_total", "Requests cancelled by the client.", "counter", (double)c.requests_cancelled);
  line("ifab_rejected_overloaded_total", "Requests refused because the admission queue was full.", "counter", (double)c.rejected_overloaded);
  line("ifab_rejected_unavailable_total", "Requests refused because the engine was unhealthy.", "counter", (double)c.rejected_unavailable);
  line("ifab_prompt_tokens_total", "Prompt tokens accepted.", "counter", (double)c.prompt_tokens);
  line("ifab_generation_tokens_total", "Tokens generated.", "counter", (double)c.generated_tokens);
  line("ifab_engine_steps_total", "Engine steps executed.", "counter", (double)c.engine_steps);
  line("ifab_engine_rows_total", "Query rows executed (prefill + decode).", "counter", (double)c.batched_rows);
  line("ifab_engine_step_seconds_total", "Time spent inside engine steps.", "counter", c.step_seconds);
  line("ifab_backpressure_skips_total", "Sequence quanta skipped because the client was slow.", "counter", (double)c.backpressure_skips);
  line("ifab_requests_running", "Requests holding a resident slot.", "gauge", (double)c.running);
  line("ifab_requests_waiting", "Requests in the admission queue.", "gauge", (double)c.queued);
  line("ifab_healthy", "1 while the engine is healthy.", "gauge", healthy() ? 1.0 : 0.0);
  auto histogram = [&](const char* name, const char* help, const Histogram& h) {
    s += std::string("# HELP ") + name + " " + help + "\n# TYPE " + name + " histogram\n";
    for (int i = 0; i < Histogram::N; ++i)
      s += std::string(name) + "_bucket{le=\"" + format_double(Histogram::kBounds[i]) + "\"} " + std::to_string(h.bucket[i]) + "\n";
    s += std::string(name) + "_bucket{le=\"+Inf\"} " + std::to_string(h.count) + "\n";
    s += std::string(name) + "_sum " + format_double(h.sum) + "\n" + name + "_count " + std::to_string(h.count) + "\n";
  };
  histogram("ifab_time_to_first_token_seconds", "Time from submission to the first generated token.", c.ttft);
  histogram("ifab_inter_token_latency_seconds", "Time between consecutive tokens of a request.", c.inter_token);
  return s;
}

Json Service::engine_audit(double timeout_seconds) {
  if (stop_.load() || !health_.healthy()) fail(ErrorKind::Backend, "engine is not serving");
  auto p = std::make_shared<std::promise<Json>>();
  auto f = p->get_future();
  {
    std::lock_guard<std::mutex> lk(mu_);
    audit_waiters_.push_back(p);
  }
  if (f.wait_for(std::chrono::duration<double>(timeout_seconds)) != std::future_status::ready)
    fail(ErrorKind::Backend, "engine audit timed out");
  return f.get();
}

void Service::run() {
  sched::Capacity cap;
  cap.residents = info_.residents;
  cap.token_budget = info_.token_budget;
  cap.chunk = std::min(info_.chunk, info_.token_budget);
  cap.context = info_.context;
  cap.queue = opt_.queue;
  cap.vocab = info_.vocab;
  sched::LiveScheduler sch(cap);
  std::unordered_map<uint64_t, Live> live;

  auto finish = [&](uint64_t id, StreamItem item) {
    auto it = live.find(id);
    if (it == live.end()) return;
    {
      std::lock_guard<std::mutex> lk(mu_);
      ids_.erase(it->second.name);
      if (item.finish == sched::Finish::Error) ++counters_.requests_failed;
      else if (item.finish == sched::Finish::Cancelled) ++counters_.requests_cancelled;
      else ++counters_.requests_finished;
    }
    it->second.stream->push_terminal(std::move(item));
    live.erase(it);
  };
  auto fail_everything = [&](const std::string& why) {
    for (auto& ev : sch.fail_all()) finish(ev.request, StreamItem{std::nullopt, sched::Finish::Error, why});
  };

  for (;;) {
    std::deque<std::pair<sched::Request, Live>> fresh;
    std::vector<uint64_t> aborts;
    std::vector<std::shared_ptr<std::promise<Json>>> audits;
    {
      std::lock_guard<std::mutex> lk(mu_);
      fresh.swap(inbox_);
      handing_over_ = (uint32_t)fresh.size();       // still counted at the door until the scheduler's queue length includes them
      aborts.swap(aborts_);
      audits.swap(audit_waiters_);
      counters_.queued = (uint32_t)sch.queued();
      counters_.running = (uint32_t)sch.running();
    }
    for (auto& w : audits) {
      try {
        w->set_value(engine_->audit());
      } catch (...) {
        w->set_exception(std::current_exception());
      }
    }
    for (auto& [req, lv] : fresh) {
      const uint64_t id = req.id;
      live.emplace(id, std::move(lv));
      try {
        sch.submit(std::move(req));
      } catch (const Error& e) {
        // the door counts the inbox, the requests being handed over and the scheduler's queue, so this is not expected; a
        // request the scheduler's queue cannot take is still refused as overloaded (429), like one refused at the door
        if (e.kind() == ErrorKind::Capacity) {
          std::lock_guard<std::mutex> lk(mu_);
          ++counters_.rejected_overloaded;
        }
        finish(id, StreamItem{std::nullopt, sched::Finish::Error, e.what(), e.kind()});
      }
    }
    if (!fresh.empty()) {
      std::lock_guard<std::mutex> lk(mu_);
      counters_.queued = (uint32_t)sch.queued();
      handing_over_ = 0;
    }
    for (auto& [id, lv] : live)
      if (lv.stream->reader_gone()) aborts.push_back(id);
    for (uint64_t id : aborts)
      if (auto ev = sch.cancel(id)) finish(id, StreamItem{std::nullopt, sched::Finish::Cancelled, ""});
    if (stop_.load()) {
      fail_everything("server is shutting down");
      break;
    }
    if (!health_.healthy()) {
      fail_everything("engine failed: " + health_.reason());
      std::this_thread::sleep_for(std::chrono::microseconds(opt_.idle_micros));
      continue;
    }
    uint64_t skipped = 0;
    for (auto& [id, lv] : live) {
      const bool full = lv.stream->free_slots() == 0;
      sch.set_backpressure(id, full);
      skipped += full ? 1 : 0;
    }
    sched::LiveScheduler::Plan plan = sch.plan();
    try {
      for (uint32_t r : plan.released) engine_->release(r);
    } catch (const Error& e) {
      health_.fail(std::string("release failed: ") + e.what());
      continue;
    }
    for (auto& [resident, id] : plan.admitted) {
      auto it = live.find(id);
      if (it == live.end()) continue;
      try {
        engine_->admit(resident, it->second.sampling, it->second.reserve);
      } catch (const Error& e) {
        if (e.kind() == ErrorKind::Backend) {
          health_.fail(std::string("admit failed: ") + e.what());
        } else {
          sch.cancel(id);   // the running step still carries its slice; commit() releases the resident
          finish(id, StreamItem{std::nullopt, sched::Finish::Error, e.what()});
        }
      }
    }
    if (plan.empty() || !health_.healthy()) {
      if (!plan.empty()) fail_everything("engine failed: " + health_.reason());
      std::this_thread::sleep_for(std::chrono::microseconds(opt_.idle_micros));
      continue;
    }
    std::vector<uint32_t> sampled;
    const double t0 = now_seconds();
    try {
      sampled = engine_->step(plan.batch);
    } catch (const std::exception& e) {
      health_.fail(std::string("step failed: ") + e.what());
      fail_everything("engine failed: " + health_.reason());
      continue;
    }
    const double dt = now_seconds() - t0;
    std::vector<sched::Event> events;
    try {
      events = sch.commit(plan, sampled);
    } catch (const Error& e) {
      health_.fail(std::string("commit failed: ") + e.what());
      fail_everything("engine failed: " + health_.reason());
      continue;
    }
    uint64_t generated = 0;
    Histogram ttft_now, itl_now;
    const double t_emit = now_seconds();
    // the step's counters first, the tokens second: a reader that sees the last token of a request must also see it counted
    for (auto& ev : events) {
      auto it = live.find(ev.request);
      if (it == live.end() || !ev.token) continue;
      ++generated;
      if (it->second.t_last == 0.0) ttft_now.observe(t_emit - it->second.t_submit);
      else itl_now.observe(t_emit - it->second.t_last);
      it->second.t_last = t_emit;
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      ++counters_.engine_steps;
      counters_.batched_rows += plan.batch.tokens.size();
      counters_.step_seconds += dt;
      counters_.generated_tokens += generated;
      counters_.backpressure_skips += skipped;
      for (const auto* pair : {&ttft_now, &itl_now}) {
        Histogram& dst = pair == &ttft_now ? counters_.ttft : counters_.inter_token;
        for (int i = 0; i < Histogram::N; ++i) dst.bucket[i] += pair->bucket[i];
        dst.count += pair->count;
        dst.sum += pair->sum;
      }
    }
    for (auto& ev : events) {
      auto it = live.find(ev.request);
      if (it == live.end()) continue;
      if (ev.token) {
        if (ev.finish) finish(ev.request, StreamItem{ev.token, ev.finish, ""});
        else it->second.stream->push(StreamItem{ev.token, std::nullopt, ""});
      } else if (ev.finish) {
        finish(ev.request, StreamItem{std::nullopt, ev.finish, *ev.finish == sched::Finish::Error ? "engine produced an invalid token" : ""});
      }
    }
  }
  // drain: free every resident, stop the engine
  try {
    for (uint32_t r : sch.plan().released) engine_->release(r);
    engine_->shutdown();
  } catch (const std::exception&) {
  }
  std::lock_guard<std::mutex> lk(mu_);
  for (auto& [req, lv] : inbox_) lv.stream->push_terminal(StreamItem{std::nullopt, sched::Finish::Error, "server is shutting down"});
  inbox_.clear();
}

}  // namespace ifab::serve
