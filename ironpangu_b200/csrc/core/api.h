// OpenAI-compatible routes over a serve::Service:
//   GET  /health /metrics /version /load /v1/models
//   POST /v1/completions /v1/chat/completions /tokenize /detokenize /inference/v1/generate
// Text goes through a byte-level tokenizer (ids 0 pad, 1 bos, 2 eos, 3 + byte); clients with their own tokenizer
// send token ids (`prompt` as an integer array, or /inference/v1/generate). Streaming responses are server-sent
// events over chunked transfer; a client that disconnects cancels its request.
// Reference: vendor/rust/src/server/src/routes.rs:75-120 (route set), frontend/src/native_backend.rs:221-293
// (admission errors), frontend/src/native_sampling.rs (defaults and validation).
#pragma once
#include "http.h"
#include "serve.h"

namespace ifab::api {

class ByteTokenizer {
 public:
  static constexpr uint32_t kPad = 0, kBos = 1, kEos = 2, kFirstByte = 3, kVocab = 259;
  std::vector<uint32_t> encode(std::string_view text) const;
  // ids outside the byte range render as <|id|>; invalid UTF-8 becomes U+FFFD
  std::string decode(const std::vector<uint32_t>& ids) const;
};

// incremental detokeniser: emits only complete UTF-8 sequences
class TextStream {
 public:
  std::string feed(uint32_t id);
  std::string flush();

 private:
  std::string pending_;
};

class Api {
 public:
  Api(serve::Service& service, serve::SamplingParams defaults) : svc_(service), defaults_(std::move(defaults)) {}
  void handle(const http::Request& req, http::ResponseWriter& w);

 private:
  struct Parsed { serve::GenerateRequest gen; bool stream = false; std::string model; };
  void completions(const http::Request& req, http::ResponseWriter& w, bool chat);
  void generate_tokens(const http::Request& req, http::ResponseWriter& w);
  std::vector<uint32_t> prompt_of(const Json& body, bool chat) const;
  serve::Service& svc_;
  serve::SamplingParams defaults_;
  ByteTokenizer tok_;
  std::atomic<uint64_t> counter_{0};
};

}  // namespace ifab::api
