#include "chat_parse.h"
#include "api.h"

#include <chrono>

namespace ifab::api {

namespace {

int64_t unix_seconds() { return (int64_t)std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count(); }

// length of the UTF-8 sequence that starts with byte b (0 = not a start byte)
int utf8_len(unsigned char b) {
  if (b < 0x80) return 1;
  if ((b & 0xE0) == 0xC0) return 2;
  if ((b & 0xF0) == 0xE0) return 3;
  if ((b & 0xF8) == 0xF0) return 4;
  return 0;
}

// moves every complete, valid sequence from `in` to the result; replaces invalid bytes; leaves an incomplete tail in `in`

Json error_body(const std::string& message, const char* type, int code) {
  Json e = Json::object();
  e.set("message", message);
  e.set("type", type);
  e.set("code", (int64_t)code);
  Json j = Json::object();
  j.set("error", e);
  return j;
}

void send_error(http::ResponseWriter& w, const Error& e) {
  switch (e.kind()) {
    case ErrorKind::Invalid: w.send(400, "application/json", error_body(e.what(), "invalid_request_error", 400).dump()); break;
    case ErrorKind::Capacity: w.send(429, "application/json", error_body(e.what(), "overloaded", 429).dump()); break;
    case ErrorKind::NotImplemented: w.send(501, "application/json", error_body(e.what(), "unsupported", 501).dump()); break;
    case ErrorKind::Backend: w.send(503, "application/json", error_body(e.what(), "unavailable", 503).dump()); break;
    default: w.send(500, "application/json", error_body(e.what(), "internal_error", 500).dump()); break;
  }
}

const char* finish_reason(sched::Finish f) {
  switch (f) {
    case sched::Finish::Stop: return "stop";
    case sched::Finish::Length: return "length";
    case sched::Finish::Cancelled: return "abort";
    default: return "error";
  }
}

}  // namespace

std::vector<uint32_t> Api::prompt_of(const Json& body, bool chat) const {
  if (chat) {
    const Json& msgs = body.at("messages");
    if (!msgs.is_array() || msgs.size() == 0) invalid("'messages' must be a non-empty array");
    std::vector<tok::ChatMessage> rendered;
    if (const Json* tools = body.find("tools"); tools && !tools->is_null() && tools->size() > 0)
      rendered.push_back({"system", chat::render_tools(*tools)});
    for (const auto& m : msgs.as_array()) {
      const Json& content = m.at("content");
      std::string c;
      if (content.is_string()) {
        c = content.as_string();
      } else if (content.is_array()) {
        for (const auto& part : content.as_array()) {
          if (part.find("type") && part.at("type").as_string() != "text") invalid("only text content parts are supported");
          c += part.at("text").as_string();
        }
      } else {
        invalid("message content must be a string or an array of text parts");
      }
      rendered.push_back({m.at("role").as_string(), std::move(c)});
    }
    const std::string text = tok::render_chat(rendered, *tok_, chat_style_);
    std::vector<uint32_t> ids;
    if (tok_->bos() >= 0) ids.push_back((uint32_t)tok_->bos());
    for (uint32_t t : tok_->encode(text)) ids.push_back(t);
    return ids;
  }
  const Json& p = body.at("prompt");
  if (p.is_string()) return tok_->encode(p.as_string());
  if (p.is_array() && p.size() > 0) {
    const Json& first = p.as_array()[0];
    if (first.is_int()) {
      std::vector<uint32_t> ids;
      for (const auto& t : p.as_array()) {
        if (!t.is_int() || t.as_int() < 0) invalid("'prompt' token ids must be non-negative integers");
        ids.push_back((uint32_t)t.as_int());
      }
      return ids;
    }
    if (p.size() != 1) invalid("batched prompts are not supported: send one request per prompt");
    Json one = Json::object();
    one.set("prompt", first);
    return prompt_of(one, false);
  }
  invalid("'prompt' must be a string or an array of token ids");
}

void Api::completions(const http::Request& req, http::ResponseWriter& w, bool chat) {
  Json body;
  serve::GenerateRequest gen;
  bool stream = false;
  std::string model = svc_.info().model;
  try {
    body = Json::parse(req.body);
    if (!body.is_object()) invalid("the request body must be a JSON object");
    if (const Json* n = body.find("n"); n && !n->is_null() && n->as_int() != 1) invalid("'n' other than 1 is not supported");
    if (const Json* e = body.find("echo"); e && !e->is_null() && e->as_bool()) invalid("'echo' is not supported");
    if (const Json* s = body.find("stop"); s && !s->is_null() && !(s->is_array() && s->size() == 0))
      invalid("'stop' strings are not supported: use 'stop_token_ids'");
    if (const Json* s = body.find("stream"); s && !s->is_null()) stream = s->as_bool();
    if (const Json* m = body.find("model"); m && m->is_string()) model = m->as_string();
    gen.prompt = prompt_of(body, chat);
    serve::SamplingParams::refuse_unsupported(body);
    gen.sampling = serve::SamplingParams::from_json(body, defaults_);
    if (const Json* r = body.find("request_id"); r && r->is_string()) gen.request_id = r->as_string();
  } catch (const Error& e) {
    // anything wrong with the request body is the client's error, except a well-formed field this engine does not implement
    return send_error(w, Error(e.kind() == ErrorKind::NotImplemented ? ErrorKind::NotImplemented : ErrorKind::Invalid, e.what()));
  }
  const size_t prompt_tokens = gen.prompt.size();
  const std::string id = std::string(chat ? "chatcmpl-" : "cmpl-") + std::to_string(++counter_);
  if (gen.request_id.empty()) gen.request_id = id;
  std::shared_ptr<serve::Stream> out;
  try {
    out = svc_.generate(std::move(gen));
  } catch (const Error& e) {
    return send_error(w, e);
  }
  const int64_t created = unix_seconds();
  const char* object = chat ? (stream ? "chat.completion.chunk" : "chat.completion") : "text_completion";
  auto choice = [&](const std::string& text, const Json& finish, bool first) {
    Json c = Json::object();
    c.set("index", 0);
    if (chat) {
      Json d = Json::object();
      if (first || !stream) d.set("role", "assistant");
      d.set("content", text);
      c.set(stream ? "delta" : "message", d);
    } else {
      c.set("text", text);
    }
    c.set("finish_reason", finish);
    return c;
  };
  auto envelope = [&](Json choice_json) {
    Json j = Json::object();
    j.set("id", id);
    j.set("object", object);
    j.set("created", created);
    j.set("model", model);
    Json arr = Json::array();
    arr.push(std::move(choice_json));
    j.set("choices", arr);
    return j;
  };
  tok::Detokenizer ts(tok_);
  size_t completion_tokens = 0;
  if (stream) {
    if (!w.begin_stream("text/event-stream")) {
      out->close_reader();
      return;
    }
    bool first = true;
    for (;;) {
      auto item = out->pop(0.25);
      if (!item) {
        if (w.client_gone()) {
          out->close_reader();
          return;
        }
        continue;
      }
      std::string text;
      if (item->token) {
        ++completion_tokens;
        text = ts.feed(*item->token);
      }
      if (item->finish) text += ts.flush();
      Json finish = item->finish ? Json(finish_reason(*item->finish)) : Json(nullptr);
      Json ev = envelope(choice(text, finish, first));
      if (item->finish && !item->error.empty()) ev.set("error", item->error);
      first = false;
      if (!w.write_chunk("data: " + ev.dump() + "\n\n")) {
        out->close_reader();
        return;
      }
      if (item->finish) break;
    }
    w.write_chunk("data: [DONE]\n\n");
    w.end_stream();
    return;
  }
  std::string text, error;
  ErrorKind error_kind = ErrorKind::Backend;
  sched::Finish fin = sched::Finish::Error;
  for (;;) {
    auto item = out->pop(0.25);
    if (!item) {
      if (w.client_gone()) {
        out->close_reader();
        return;
      }
      continue;
    }
    if (item->token) {
      ++completion_tokens;
      text += ts.feed(*item->token);
    }
    if (item->finish) {
      fin = *item->finish;
      error = item->error;
      error_kind = item->error_kind;
      break;
    }
  }
  text += ts.flush();
  if (fin == sched::Finish::Error) return send_error(w, Error(error_kind, error.empty() ? "generation failed" : error));
  Json one = choice(text, Json(finish_reason(fin)), true);
  if (chat) {
    // reasoning sections and tool calls leave the content; a request may switch either parser off
    bool want_reasoning = true, want_tools = body.find("tools") != nullptr;
    if (const Json* k = body.find("chat_template_kwargs"); k && k->is_object())
      if (const Json* t = k->find("parse_reasoning"); t && !t->is_null()) want_reasoning = t->as_bool();
    const chat::Parsed parsed = chat::parse_assistant(text, want_reasoning, want_tools);
    one.set("message", chat::message_json(parsed, id));
    if (!parsed.tool_calls.empty() && fin != sched::Finish::Length) one.set("finish_reason", "tool_calls");
  }
  Json j = envelope(std::move(one));
  Json usage = Json::object();
  usage.set("prompt_tokens", (int64_t)prompt_tokens);
  usage.set("completion_tokens", (int64_t)completion_tokens);
  usage.set("total_tokens", (int64_t)(prompt_tokens + completion_tokens));
  j.set("usage", usage);
  w.send(200, "application/json", j.dump());
}

void Api::generate_tokens(const http::Request& req, http::ResponseWriter& w) {
  serve::GenerateRequest gen;
  bool stream = false;
  try {
    Json body = Json::parse(req.body);
    for (const auto& t : body.at("token_ids").as_array()) {
      if (!t.is_int() || t.as_int() < 0) invalid("'token_ids' must be non-negative integers");
      gen.prompt.push_back((uint32_t)t.as_int());
    }
    const Json* sp = body.find("sampling_params");
    serve::SamplingParams::refuse_unsupported(body);
    gen.sampling = sp && !sp->is_null() ? serve::SamplingParams::from_json(*sp, defaults_) : defaults_;
    if (const Json* s = body.find("stream"); s && !s->is_null()) stream = s->as_bool();
    if (const Json* r = body.find("request_id"); r && r->is_string()) gen.request_id = r->as_string();
    if (const Json* c = body.find("cache_salt"); c && c->is_string() && gen.sampling.cache_salt.empty()) gen.sampling.cache_salt = c->as_string();
  } catch (const Error& e) {
    // anything wrong with the request body is the client's error, except a well-formed field this engine does not implement
    return send_error(w, Error(e.kind() == ErrorKind::NotImplemented ? ErrorKind::NotImplemented : ErrorKind::Invalid, e.what()));
  }
  if (gen.request_id.empty()) gen.request_id = "gen-" + std::to_string(++counter_);
  const std::string id = gen.request_id;
  std::shared_ptr<serve::Stream> out;
  try {
    out = svc_.generate(std::move(gen));
  } catch (const Error& e) {
    return send_error(w, e);
  }
  if (stream && !w.begin_stream("text/event-stream")) {
    out->close_reader();
    return;
  }
  Json all = Json::array();
  for (;;) {
    auto item = out->pop(0.25);
    if (!item) {
      if (w.client_gone()) {
        out->close_reader();
        return;
      }
      continue;
    }
    if (item->token) all.push((int64_t)*item->token);
    if (stream) {
      Json ev = Json::object();
      ev.set("request_id", id);
      Json t = Json::array();
      if (item->token) t.push((int64_t)*item->token);
      ev.set("token_ids", t);
      ev.set("finish_reason", item->finish ? Json(finish_reason(*item->finish)) : Json(nullptr));
      if (!item->error.empty()) ev.set("error", item->error);
      if (!w.write_chunk("data: " + ev.dump() + "\n\n")) {
        out->close_reader();
        return;
      }
    }
    if (item->finish) {
      if (stream) {
        w.write_chunk("data: [DONE]\n\n");
        w.end_stream();
      } else if (*item->finish == sched::Finish::Error) {
        send_error(w, Error(item->error_kind, item->error.empty() ? "generation failed" : item->error));
      } else {
        Json j = Json::object();
        j.set("request_id", id);
        j.set("token_ids", all);
        j.set("finish_reason", finish_reason(*item->finish));
        w.send(200, "application/json", j.dump());
      }
      return;
    }
  }
}

void Api::handle(const http::Request& req, http::ResponseWriter& w) {
  const auto& info = svc_.info();
  const bool get = req.method == "GET", post = req.method == "POST";
  if (req.path == "/health") {
    if (!get) return w.send(405, "text/plain", "GET only\n");
    return svc_.healthy() ? w.send(200, "text/plain", "") : w.send(503, "text/plain", svc_.unhealthy_reason() + "\n");
  }
  if (req.path == "/metrics" && get) return w.send(200, "text/plain; version=0.0.4", svc_.metrics_text());
  if (req.path == "/version" && get) {
    Json j = Json::object();
    j.set("version", "0.1.0");
    return w.send(200, "application/json", j.dump());
  }
  if (req.path == "/load" && get) {
    const auto c = svc_.counters();
    Json j = Json::object();
    j.set("running", c.running);
    j.set("waiting", c.queued);
    j.set("residents", info.residents);
    return w.send(200, "application/json", j.dump());
  }
  if (req.path == "/audit" && get) {
    // engine-side transfer / execution audit plus the service counters, one JSON document
    const auto c = svc_.counters();
    Json j = Json::object(), svc = Json::object();
    svc.set("requests_finished", c.requests_finished);
    svc.set("requests_failed", c.requests_failed);
    svc.set("requests_cancelled", c.requests_cancelled);
    svc.set("running", c.running);
    svc.set("waiting", c.queued);
    j.set("service", svc);
    j.set("engine", svc_.engine_audit());
    return w.send(200, "application/json", j.dump());
  }
  if (req.path == "/v1/models" && get) {
    Json m = Json::object();
    m.set("id", info.model);
    m.set("object", "model");
    m.set("owned_by", "ifab");
    m.set("max_model_len", info.context);
    Json data = Json::array();
    data.push(m);
    Json j = Json::object();
    j.set("object", "list");
    j.set("data", data);
    return w.send(200, "application/json", j.dump());
  }
  if (!post) {
    if (req.path == "/v1/completions" || req.path == "/v1/chat/completions" || req.path == "/tokenize" || req.path == "/detokenize" ||
        req.path == "/inference/v1/generate")
      return w.send(405, "text/plain", "POST only\n");
    return;   // 404
  }
  if (req.path == "/v1/completions") return completions(req, w, false);
  if (req.path == "/v1/chat/completions") return completions(req, w, true);
  if (req.path == "/inference/v1/generate") return generate_tokens(req, w);
  if (req.path == "/tokenize" || req.path == "/detokenize") {
    try {
      Json body = Json::parse(req.body);
      Json j = Json::object();
      if (req.path == "/tokenize") {
        const std::vector<uint32_t> ids = body.find("messages") ? prompt_of(body, true) : prompt_of(body, false);
        Json a = Json::array();
        for (uint32_t t : ids) a.push((int64_t)t);
        j.set("tokens", a);
        j.set("count", (int64_t)ids.size());
        j.set("max_model_len", info.context);
      } else {
        std::vector<uint32_t> ids;
        for (const auto& t : body.at("tokens").as_array()) ids.push_back((uint32_t)t.as_int());
        j.set("prompt", tok_->decode(ids));
      }
      return w.send(200, "application/json", j.dump());
    } catch (const Error& e) {
      return send_error(w, Error(ErrorKind::Invalid, e.what()));
    }
  }
}

}  // namespace ifab::api
