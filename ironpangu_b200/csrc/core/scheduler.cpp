#include "scheduler.h"

#include <algorithm>

namespace ifab::sched {

const char* finish_name(Finish f) {
  switch (f) {
    case Finish::Stop: return "stop";
    case Finish::Length: return "length";
    case Finish::Cancelled: return "cancelled";
    case Finish::Error: return "error";
  }
  return "?";
}

void Capacity::validate() const {
  if (residents == 0 || residents > 1024) invalid("scheduler: residents must be 1..1024");
  if (token_budget == 0 || chunk == 0 || context == 0 || queue == 0) invalid("scheduler: capacities must be positive");
}

std::vector<size_t> select_round(const std::vector<uint32_t>& costs, size_t* cursor, uint32_t budget) {
  std::vector<size_t> out;
  const size_t n = costs.size();
  if (n == 0) return out;
  size_t start = *cursor % n;
  for (size_t k = 0; k < n; ++k) {
    const size_t i = (start + k) % n;
    if (costs[i] == 0) continue;   // not eligible this round
    if (costs[i] > budget) {
      *cursor = i;                 // served first next time, with a full budget
      return out;
    }
    budget -= costs[i];
    out.push_back(i);
  }
  *cursor = (start + 1) % n;       // everyone was served: rotate the starting point
  return out;
}

LiveScheduler::LiveScheduler(Capacity c) : cap_(c), seqs_(c.residents) { cap_.validate(); }

void LiveScheduler::submit(Request r) {
  if (r.prompt.empty()) invalid("request: empty prompt");
  if (r.max_new_tokens == 0) invalid("request: max_new_tokens must be positive");
  if ((uint64_t)r.prompt.size() + r.max_new_tokens > cap_.context) fail(ErrorKind::Capacity, "request: prompt + max_new_tokens exceeds the context");
  if (cap_.vocab)
    for (uint32_t t : r.prompt)
      if (t >= cap_.vocab) invalid("request: token id outside the vocabulary");
  if (r.prefix_hit >= r.prompt.size()) invalid("request: a restored prefix must leave at least one prompt token");
  for (auto& q : queue_)
    if (q.id == r.id) invalid("request: duplicate id");
  for (auto& s : seqs_)
    if (s.active && s.req.id == r.id) invalid("request: duplicate id");
  if (queue_.size() >= cap_.queue) fail(ErrorKind::Capacity, "scheduler: admission queue is full (overloaded)");
  queue_.push_back(std::move(r));
}

std::optional<Event> LiveScheduler::cancel(uint64_t id) {
  for (auto it = queue_.begin(); it != queue_.end(); ++it)
    if (it->id == id) {
      queue_.erase(it);
      return Event{id, std::nullopt, Finish::Cancelled};
    }
  for (size_t i = 0; i < seqs_.size(); ++i) {
    Seq& s = seqs_[i];
    if (!s.active || s.req.id != id || s.cancelled) continue;
    s.cancelled = true;
    if (!s.in_flight) {
      s.active = false;
      --running_;
      released_.push_back((uint32_t)i);
    }
    return Event{id, std::nullopt, Finish::Cancelled};
  }
  return std::nullopt;
}

void LiveScheduler::set_backpressure(uint64_t id, bool on) {
  for (auto& s : seqs_)
    if (s.active && s.req.id == id) s.backpressure = on;
}

LiveScheduler::Plan LiveScheduler::plan() {
  Plan p;
  p.released.swap(released_);
  // admission
  for (size_t i = 0; i < seqs_.size() && !queue_.empty(); ++i) {
    if (seqs_[i].active) continue;
    Seq& s = seqs_[i];
    s = Seq{};
    s.active = true;
    s.req = std::move(queue_.front());
    queue_.pop_front();
    s.fed = s.req.prefix_hit;
    ++running_;
    p.admitted.push_back({(uint32_t)i, s.req.id});
  }
  // quanta
  std::vector<uint32_t> costs(seqs_.size(), 0);
  for (size_t i = 0; i < seqs_.size(); ++i) {
    const Seq& s = seqs_[i];
    if (!s.active || s.cancelled || s.backpressure) continue;
    const uint32_t left = (uint32_t)s.req.prompt.size() - s.fed;
    costs[i] = left > 0 ? std::min({left, cap_.chunk, cap_.token_budget}) : 1;
  }
  std::vector<size_t> chosen = select_round(costs, &cursor_, cap_.token_budget);
  std::vector<paging::SequenceSlice> slices;
  std::vector<int32_t> tokens;
  for (size_t i : chosen) {
    Seq& s = seqs_[i];
    paging::SequenceSlice sl;
    sl.resident = (uint32_t)i;
    const uint32_t left = (uint32_t)s.req.prompt.size() - s.fed;
    if (left > 0) {
      sl.position = s.fed;
      sl.token_count = costs[i];
      sl.sample = costs[i] == left;          // the chunk that ends the prompt produces the first token
      for (uint32_t k = 0; k < costs[i]; ++k) tokens.push_back((int32_t)s.req.prompt[s.fed + k]);
    } else {
      sl.position = (uint32_t)s.req.prompt.size() + (uint32_t)s.generated.size() - 1;
      sl.token_count = 1;
      sl.sample = true;
      tokens.push_back((int32_t)s.generated.back());
    }
    s.in_flight = true;
    slices.push_back(sl);
    p.requests.push_back(s.req.id);
  }
  if (!slices.empty()) p.batch = paging::SequenceBatch::make(slices, tokens, cap_.token_budget, cap_.residents, cap_.context);
  return p;
}

std::vector<Event> LiveScheduler::commit(const Plan& plan, const std::vector<uint32_t>& sampled) {
  if (sampled.size() != plan.batch.slices.size()) invalid("scheduler: one sampled token per slice is required");
  std::vector<Event> ev;
  ++steps_;
  for (size_t k = 0; k < plan.batch.slices.size(); ++k) {
    const auto& sl = plan.batch.slices[k];
    Seq& s = seqs_.at(sl.resident);
    if (!s.active || s.req.id != plan.requests[k] || !s.in_flight) invalid("scheduler: commit does not match the outstanding plan");
    s.in_flight = false;
    if (s.cancelled) {      // cancelled while the step was running: the terminal event was already delivered
      s.active = false;
      --running_;
      released_.push_back(sl.resident);
      continue;
    }
    if (s.fed < s.req.prompt.size()) s.fed += sl.token_count;
    if (!sl.sample) continue;
    const uint32_t tok = sampled[k];
    if (cap_.vocab && tok >= cap_.vocab) {
      ev.push_back({s.req.id, std::nullopt, Finish::Error});
      s.active = false;
      --running_;
      released_.push_back(sl.resident);
      continue;
    }
    s.generated.push_back(tok);
    const bool stop = std::find(s.req.stop_tokens.begin(), s.req.stop_tokens.end(), tok) != s.req.stop_tokens.end();
    const bool length = s.generated.size() >= s.req.max_new_tokens;
    Event e{s.req.id, tok, std::nullopt};
    if (stop) e.finish = Finish::Stop;
    else if (length) e.finish = Finish::Length;
    ev.push_back(e);
    if (e.finish) {
      s.active = false;
      --running_;
      released_.push_back(sl.resident);
    }
  }
  return ev;
}

std::vector<Event> LiveScheduler::fail_all() {
  std::vector<Event> ev;
  for (auto& q : queue_) ev.push_back({q.id, std::nullopt, Finish::Error});
  queue_.clear();
  for (size_t i = 0; i < seqs_.size(); ++i)
    if (seqs_[i].active) {
      if (!seqs_[i].cancelled) ev.push_back({seqs_[i].req.id, std::nullopt, Finish::Error});
      seqs_[i].active = false;
      released_.push_back((uint32_t)i);
    }
  running_ = 0;
  return ev;
}

// ---------------------------------------------------------------------------------------------
Json SimReport::to_json() const {
  Json j = Json::object();
  j.set("ticks", ticks);
  j.set("prefill_steps", prefill_steps);
  j.set("decode_steps", decode_steps);
  j.set("transfers", transfers);
  j.set("cancelled", cancelled);
  j.set("completed", completed);
  j.set("leaked_allocations", (int64_t)leaked_allocations);
  Json o = Json::object();
  for (auto& kv : outputs) {
    Json a = Json::array();
    for (auto t : kv.second) a.push((int64_t)t);
    o.set(std::to_string(kv.first), a);
  }
  j.set("outputs", o);
  return j;
}

SimReport run_mock(const rankplan::Artifact& artifact, std::vector<SimRequest> requests, SimCapacity cap, std::shared_ptr<runtime::Trace> trace) {
  using namespace runtime;
  if (!trace) trace = std::make_shared<Trace>();
  const rankplan::Spec& spec = artifact.spec;
  Runtime prefill(artifact, rankplan::Role::Prefill, 0, std::make_unique<MockBackend>(trace, 0));
  Runtime decode(artifact, rankplan::Role::Decode, 0, std::make_unique<MockBackend>(trace, 100));
  prefill.start("metadata-only");
  decode.start("metadata-only");
  InMemoryTransport transport(artifact.key, cap.pages, cap.decode_slots, cap.page_tokens);
  struct Live { SimRequest r; uint32_t prefilled = 0; std::optional<TransferLease> lease; bool decoding = false; uint32_t next = 0; std::vector<uint32_t> out; bool done = false; };
  std::vector<Live> live;
  for (auto& r : requests) {
    if (r.prompt_tokens == 0 || r.output_tokens == 0) invalid("simulation: empty request");
    if (r.prompt_tokens + r.output_tokens > spec.max_context()) fail(ErrorKind::Capacity, "simulation: request exceeds the largest context bucket");
    live.push_back({r});
  }
  SimReport rep;
  const uint64_t epoch = 1;
  size_t rr = 0;
  for (uint64_t tick = 0; tick < 100000; ++tick) {
    bool all_done = true;
    for (auto& l : live) all_done &= l.done;
    if (all_done) break;
    rep.ticks = tick + 1;
    // cancellations
    for (auto& l : live)
      if (!l.done && l.r.cancel_tick && *l.r.cancel_tick <= tick) {
        if (l.lease) transport.abort(*l.lease);
        l.done = true;
        ++rep.cancelled;
      }
    transport.completion_fence();
    // chunked prefill, round robin under the token budget
    uint32_t budget = spec.token_budget;
    std::vector<StepInput> pin;
    std::vector<size_t> who;
    for (size_t k = 0; k < live.size() && budget > 0; ++k) {
      Live& l = live[(rr + k) % live.size()];
      if (l.done || l.decoding || l.r.arrival_tick > tick || l.prefilled >= l.r.prompt_tokens) continue;
      if (!l.lease) {
        try {
          l.lease = transport.reserve(l.r.id, epoch, l.r.prompt_tokens + l.r.output_tokens);
        } catch (const Error& e) {
          if (e.kind() == ErrorKind::Capacity) continue;   // wait for decode slots / pages
          throw;
        }
      }
      uint32_t n = std::min(budget, l.r.prompt_tokens - l.prefilled);
      StepInput in;
      in.request = l.r.id;
      in.position = l.prefilled;
      in.tokens.assign(n, 1);
      pin.push_back(in);
      who.push_back((rr + k) % live.size());
      budget -= n;
    }
    if (!live.empty()) rr = (rr + 1) % live.size();
    if (!pin.empty()) {
      auto outs = prefill.step(pin);
      ++rep.prefill_steps;
      for (size_t k = 0; k < outs.size(); ++k) {
        Live& l = live[who[k]];
        l.prefilled += outs[k].consumed;
        if (l.prefilled == l.r.prompt_tokens) {
          TransferManifest m;
          m.request = l.r.id;
          m.epoch = epoch;
          m.artifact_key = artifact.key;
          m.consumed = l.prefilled;
          m.next_token = outs[k].token;
          for (uint32_t layer = 0; layer < spec.model.layers.size(); ++layer) m.region_hashes.push_back(l.r.id * 1000 + layer);
          transport.transfer(m);
          transport.transfer(m);               // a duplicate delivery must be harmless
          transport.complete(*l.lease);
          TransferManifest got = transport.commit(*l.lease);
          transport.acknowledge(*l.lease);
          l.next = got.next_token;
          l.out.push_back(got.next_token);
          l.decoding = true;
          ++rep.transfers;
        }
      }
    }
    // decode batch
    std::vector<StepInput> din;
    std::vector<size_t> dwho;
    for (size_t i = 0; i < live.size(); ++i) {
      Live& l = live[i];
      if (l.done || !l.decoding) continue;
      if (l.out.size() >= l.r.output_tokens) continue;
      if (din.size() >= spec.batch_buckets.back()) break;
      StepInput in;
      in.request = l.r.id;
      in.position = l.r.prompt_tokens + (uint32_t)l.out.size() - 1;
      in.tokens = {l.next};
      din.push_back(in);
      dwho.push_back(i);
    }
    if (!din.empty()) {
      auto outs = decode.step(din);
      ++rep.decode_steps;
      for (size_t k = 0; k < outs.size(); ++k) {
        Live& l = live[dwho[k]];
        l.next = outs[k].token;
        l.out.push_back(outs[k].token);
      }
    }
    for (auto& l : live)
      if (!l.done && l.decoding && l.out.size() >= l.r.output_tokens) {
        transport.finish(*l.lease);
        l.done = true;
        ++rep.completed;
        rep.outputs[l.r.id] = l.out;
      }
  }
  transport.completion_fence();
  rep.leaked_allocations = transport.pool().allocations() + transport.pending();
  prefill.close();
  decode.close();
  return rep;
}

}  // namespace ifab::sched
