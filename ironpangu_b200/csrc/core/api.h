// OpenAI-compatible routes over a serve::Service:
//   GET  /health /metrics /version /load /v1/models
//   POST /v1/completions /v1/chat/completions /tokenize /detokenize /inference/v1/generate
// Text goes through the configured tokenizer (tokenizer.h: bytes by default, byte-level BPE from a tokenizer.json) and chat
// messages through its prompt renderer; clients with their own tokenizer send token ids (`prompt` as an integer array, or /inference/v1/generate). Streaming responses are server-sent
// events over chunked transfer; a client that disconnects cancels its request.
// Reference: vendor/rust/src/server/src/routes.rs:75-120 (route set), frontend/src/native_backend.rs:221-293
// (admission errors), frontend/src/native_sampling.rs (defaults and validation).
#pragma once
#include "http.h"
#include "serve.h"
#include "tokenizer.h"

namespace ifab::api {

// the byte-level tokenizer and the incremental detokeniser live in tokenizer.h; the old names stay for their users
using ByteTokenizer = tok::ByteTokenizer;
class TextStream {        // incremental detokeniser over the byte tokenizer: emits only complete UTF-8 sequences
 public:
  TextStream() : d_(std::make_shared<tok::ByteTokenizer>(), false) {}
  std::string feed(uint32_t id) { return d_.feed(id); }
  std::string flush() { return d_.flush(); }

 private:
  tok::Detokenizer d_;
};

class Api {
 public:
  // `tokenizer`: bytes by default; a byte-level BPE tokenizer (tokenizer.json) for real vocabularies. `chat_style`: auto | chatml | plain.
  Api(serve::Service& service, serve::SamplingParams defaults, std::shared_ptr<tok::Tokenizer> tokenizer = nullptr, std::string chat_style = "auto")
      : svc_(service), defaults_(std::move(defaults)), tok_(tokenizer ? std::move(tokenizer) : std::make_shared<tok::ByteTokenizer>()),
        chat_style_(std::move(chat_style)) {}
  void handle(const http::Request& req, http::ResponseWriter& w);

 private:
  struct Parsed { serve::GenerateRequest gen; bool stream = false; std::string model; };
  void completions(const http::Request& req, http::ResponseWriter& w, bool chat);
  void generate_tokens(const http::Request& req, http::ResponseWriter& w);
  std::vector<uint32_t> prompt_of(const Json& body, bool chat) const;
  serve::Service& svc_;
  serve::SamplingParams defaults_;
  std::shared_ptr<tok::Tokenizer> tok_;
  std::string chat_style_;
  std::atomic<uint64_t> counter_{0};
};

}  // namespace ifab::api
