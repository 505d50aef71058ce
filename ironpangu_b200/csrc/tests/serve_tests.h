// Tests of the serving core against the mock engine (included by core_tests.cpp, uses its CHECK macros).
// Model: the reference's 20 program-worker tests with a Fake engine (frontend/src/program_worker.rs:400-995):
// admission bounds, continuous batching, back-pressure, cancellation, engine failure, shutdown drain.
#pragma once
#include <chrono>
#include <thread>

#include "api.h"
#include "serve.h"

namespace serve_tests {

using namespace ifab;
using namespace ifab::serve;

inline EngineInfo small_engine(uint32_t residents = 2, uint32_t budget = 4) {
  EngineInfo e;
  e.model = "fake";
  e.residents = residents;
  e.token_budget = budget;
  e.chunk = budget;
  e.context = 64;
  e.vocab = 300;
  e.eos = 2;
  e.has_eos = false;
  return e;
}

inline std::vector<uint32_t> expected_tokens(std::vector<uint32_t> prompt, uint32_t n, uint32_t vocab) {
  std::vector<uint32_t> out;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t t = MockEngine::next_token(prompt, vocab);
    out.push_back(t);
    prompt.push_back(t);
  }
  return out;
}

// drains a stream to its terminal item; returns the tokens and the terminal through out parameters
inline bool collect(Stream& s, std::vector<uint32_t>* tokens, StreamItem* last, double timeout = 5.0) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    auto it = s.pop(0.05);
    if (it) {
      if (it->token) tokens->push_back(*it->token);
      if (it->finish) {
        *last = *it;
        return true;
      }
    }
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout) return false;
  }
}

inline GenerateRequest request(std::vector<uint32_t> prompt, uint32_t max_tokens, std::string id = "") {
  GenerateRequest g;
  g.request_id = std::move(id);
  g.prompt = std::move(prompt);
  g.sampling.max_tokens = max_tokens;
  return g;
}

}  // namespace serve_tests

static void test_serve_batching_matches_sequential() {
  using namespace serve_tests;
  auto engine = std::make_shared<MockEngine>(small_engine(2, 4));
  Service svc(engine);
  // five requests over two residents: prompts longer than a chunk, different lengths, all interleaved
  std::vector<std::vector<uint32_t>> prompts = {{5, 6, 7, 8, 9, 10, 11}, {20}, {30, 31, 32}, {40, 41, 42, 43, 44}, {50, 51}};
  std::vector<std::shared_ptr<Stream>> streams;
  for (auto& p : prompts) streams.push_back(svc.generate(request(p, 6)));
  for (size_t i = 0; i < prompts.size(); ++i) {
    std::vector<uint32_t> got;
    StreamItem last;
    CHECK(collect(*streams[i], &got, &last));
    CHECK(last.finish && *last.finish == sched::Finish::Length);
    CHECK(got == expected_tokens(prompts[i], 6, 300));
  }
  const Counters c = svc.counters();
  CHECK(c.requests_total == 5 && c.requests_finished == 5 && c.generated_tokens == 30);
  CHECK(c.batched_rows > c.engine_steps);   // steps carried more than one row: sequences really shared steps
  CHECK(svc.metrics_text().find("ifab_generation_tokens_total 30") != std::string::npos);
}

static void test_serve_validation_and_admission() {
  using namespace serve_tests;
  EngineInfo info = small_engine(1, 2);
  info.greedy_only = true;
  auto engine = std::make_shared<MockEngine>(info, 20000);   // 20 ms per step keeps the queue occupied
  ServiceOptions opt;
  opt.queue = 2;
  Service svc(engine, opt);
  CHECK_THROWS(Invalid, svc.generate(request({}, 4)));
  CHECK_THROWS(Invalid, svc.generate(request({1, 2, 3}, 64)));            // prompt + max_tokens > context
  CHECK_THROWS(Invalid, svc.generate(request({1, 999}, 4)));              // outside the vocabulary
  GenerateRequest hot = request({1, 2}, 4);
  hot.sampling.temperature = 0.8;
  CHECK_THROWS(Invalid, svc.generate(hot));                               // greedy-only engine
  GenerateRequest lp = request({1, 2}, 4);
  lp.sampling.logprobs = 5;
  CHECK_THROWS(Invalid, svc.generate(lp));
  std::vector<std::shared_ptr<Stream>> held;
  bool overloaded = false;
  for (int i = 0; i < 8 && !overloaded; ++i) {
    try {
      held.push_back(svc.generate(request({7, 8, 9}, 8, "r" + std::to_string(i))));
    } catch (const Error& e) {
      overloaded = e.kind() == ErrorKind::Capacity;
    }
  }
  CHECK(overloaded);
  CHECK(svc.counters().rejected_overloaded >= 1);
  CHECK_THROWS(Invalid, svc.generate(request({7}, 2, "r0")));             // duplicate id while r0 is alive
  for (auto& s : held) {
    std::vector<uint32_t> got;
    StreamItem last;
    CHECK(collect(*s, &got, &last, 20.0));
    CHECK(last.finish && *last.finish == sched::Finish::Length && got.size() == 8);
  }
}

static void test_serve_backpressure_cancel_and_eos() {
  using namespace serve_tests;
  EngineInfo info = small_engine(2, 4);
  auto engine = std::make_shared<MockEngine>(info, 200);
  ServiceOptions opt;
  opt.stream_capacity = 2;
  Service svc(engine, opt);
  // a reader that does not read: the sequence stalls after `stream_capacity` tokens instead of running to the end
  auto slow = svc.generate(request({3, 4, 5}, 20, "slow"));
  auto fast = svc.generate(request({9, 9}, 10, "fast"));
  std::vector<uint32_t> got;
  StreamItem last;
  CHECK(collect(*fast, &got, &last));
  CHECK(got == expected_tokens({9, 9}, 10, 300));
  std::this_thread::sleep_for(std::chrono::milliseconds(50));
  CHECK(slow->free_slots() == 0);
  CHECK(svc.counters().backpressure_skips > 0);
  CHECK(svc.counters().generated_tokens < 10 + 20);                        // the slow one did not run ahead
  got.clear();
  CHECK(collect(*slow, &got, &last));                                      // reading releases it
  CHECK(got == expected_tokens({3, 4, 5}, 20, 300));
  // cancellation: explicit abort and a reader that goes away
  auto a = svc.generate(request({11, 12}, 40, "to-abort"));
  auto b = svc.generate(request({13}, 40, "gone"));
  svc.abort("to-abort");
  b->close_reader();
  got.clear();
  CHECK(collect(*a, &got, &last) && *last.finish == sched::Finish::Cancelled);
  got.clear();
  CHECK(collect(*b, &got, &last) && *last.finish == sched::Finish::Cancelled);
  CHECK(svc.counters().requests_cancelled == 2);
  // stop tokens: the second generated token of this prompt is used as a stop token
  const auto two = expected_tokens({21, 22}, 2, 300);
  GenerateRequest st = request({21, 22}, 10);
  st.sampling.stop_token_ids = {two[1]};
  auto s = svc.generate(st);
  got.clear();
  CHECK(collect(*s, &got, &last) && *last.finish == sched::Finish::Stop && got == two);
}

static void test_serve_engine_failure_and_shutdown() {
  using namespace serve_tests;
  auto engine = std::make_shared<MockEngine>(small_engine(2, 4), 100);
  engine->fail_after(3);
  Service svc(engine);
  auto s1 = svc.generate(request({1, 2, 3}, 30));
  auto s2 = svc.generate(request({4}, 30));
  std::vector<uint32_t> got;
  StreamItem last;
  CHECK(collect(*s1, &got, &last) && *last.finish == sched::Finish::Error && last.error.find("engine failed") != std::string::npos);
  CHECK(collect(*s2, &got, &last) && *last.finish == sched::Finish::Error);
  CHECK(!svc.healthy());
  CHECK_THROWS(Backend, svc.generate(request({5}, 2)));                    // fail closed: unavailable from now on
  CHECK(svc.counters().rejected_unavailable == 1);
  // shutdown drains running and queued requests with an error and refuses new ones
  auto engine2 = std::make_shared<MockEngine>(small_engine(1, 2), 5000);
  Service svc2(engine2);
  auto r1 = svc2.generate(request({1, 2, 3, 4, 5}, 40));
  auto r2 = svc2.generate(request({6}, 40));
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  svc2.shutdown();
  got.clear();
  CHECK(collect(*r1, &got, &last) && *last.finish == sched::Finish::Error && last.error.find("shutting down") != std::string::npos);
  CHECK(collect(*r2, &got, &last) && *last.finish == sched::Finish::Error);
  CHECK_THROWS(Backend, svc2.generate(request({5}, 2)));
}

static void test_api_tokenizer_and_sampling_json() {
  using namespace ifab::api;
  ByteTokenizer tok;
  const std::string text = "h\xC3\xA9llo \xE2\x82\xAC";
  CHECK(tok.decode(tok.encode(text)) == text);
  CHECK(tok.decode({3 + 0xC3}) == "\xEF\xBF\xBD");                          // truncated sequence -> replacement character
  CHECK(tok.decode({3 + 'a', 700, 3 + 'b'}) == "a<|700|>b");
  TextStream ts;
  CHECK(ts.feed(3 + 0xE2).empty() && ts.feed(3 + 0x82).empty() && ts.feed(3 + 0xAC) == "\xE2\x82\xAC");
  serve::SamplingParams d;
  d.temperature = 1.0;
  d.top_k = 20;
  const auto s = serve::SamplingParams::from_json(Json::parse("{\"temperature\":0.5,\"max_tokens\":7,\"top_k\":-1,\"seed\":11,\"stop_token_ids\":[4,5]}"), d);
  CHECK(s.temperature == 0.5 && s.max_tokens == 7 && s.top_k == 0 && s.seed && *s.seed == 11 && s.stop_token_ids.size() == 2);
  CHECK_THROWS(Invalid, serve::SamplingParams::from_json(Json::parse("{\"top_p\":0}"), d).validate());
  CHECK_THROWS(Invalid, serve::SamplingParams::from_json(Json::parse("{\"max_tokens\":0}"), d));
  CHECK_THROWS(Invalid, serve::SamplingParams::from_json(Json::parse("{\"temperature\":\"hot\"}"), d));
  // deployment defaults: the model-card recommendation, then the checkpoint's generation_config.json (null keys keep the default)
  const auto card = serve::SamplingParams::model_card();
  CHECK(card.temperature == 1.0 && card.top_k == 20 && card.top_p == 1.0 && card.presence_penalty == 2.0 && card.repetition_penalty == 1.0);
  char tmpl[] = "/tmp/ifab-gencfg-XXXXXX";
  const std::string dir = ::mkdtemp(tmpl);
  CHECK(serve::SamplingParams::deployment_defaults(dir).top_k == 20);                       // no file in the directory: the card
  write_file(dir + "/generation_config.json", "{\"temperature\":0.7,\"top_k\":null,\"top_p\":0.8,\"presence_penalty\":0,\"eos_token_id\":7,\"max_tokens\":999}");
  const auto dep = serve::SamplingParams::deployment_defaults(dir);
  CHECK(dep.temperature == 0.7 && dep.top_k == 20 && dep.top_p == 0.8 && dep.presence_penalty == 0.0 && dep.max_tokens == card.max_tokens);
  write_file(dir + "/generation_config.json", "{\"top_p\":0}");
  CHECK_THROWS(Invalid, serve::SamplingParams::deployment_defaults(dir));                   // defaults are validated like requests
  CHECK_THROWS(Invalid, serve::SamplingParams::deployment_defaults(dir + "/nothing-here"));
  // fields the engine does not implement are refused, at the top level and inside sampling_params
  CHECK_THROWS(NotImplemented, serve::SamplingParams::refuse_unsupported(Json::parse("{\"prompt\":\"x\",\"logit_bias\":{\"5\":1}}")));
  CHECK_THROWS(NotImplemented, serve::SamplingParams::refuse_unsupported(Json::parse("{\"token_ids\":[1],\"sampling_params\":{\"allowed_token_ids\":[1]}}")));
  serve::SamplingParams::refuse_unsupported(Json::parse("{\"prompt\":\"x\",\"logit_bias\":null,\"temperature\":0.2}"));
}
