#include "chat_parse.h"

namespace ifab::chat {
namespace {

const std::string kThinkOpen = "<think>", kThinkClose = "</think>", kToolOpen = "<tool_call>", kToolClose = "</tool_call>";

std::string trim(const std::string& s) {
  size_t b = 0, e = s.size();
  while (b < e && (s[b] == ' ' || s[b] == '\n' || s[b] == '\r' || s[b] == '\t')) ++b;
  while (e > b && (s[e - 1] == ' ' || s[e - 1] == '\n' || s[e - 1] == '\r' || s[e - 1] == '\t')) --e;
  return s.substr(b, e - b);
}

// one tool-call body: a JSON object with a string "name" and an object (or JSON-string) "arguments" / "parameters"
bool parse_call(const std::string& body, ToolCall* out) {
  try {
    const Json j = Json::parse(trim(body), 1 << 20);
    if (!j.is_object()) return false;
    const Json* name = j.find("name");
    if (!name || !name->is_string() || name->as_string().empty()) return false;
    const Json* args = j.find("arguments");
    if (!args) args = j.find("parameters");
    out->name = name->as_string();
    if (!args || args->is_null()) {
      out->arguments = "{}";
    } else if (args->is_object()) {
      out->arguments = args->dump();
    } else if (args->is_string()) {
      const Json inner = Json::parse(args->as_string(), 1 << 20);   // must itself be JSON
      if (!inner.is_object()) return false;
      out->arguments = inner.dump();
    } else {
      return false;
    }
    return true;
  } catch (const Error&) {
    return false;
  }
}

}  // namespace

Parsed parse_assistant(const std::string& text, bool want_reasoning, bool want_tools) {
  Parsed p;
  std::string rest = text;
  if (want_reasoning) {
    const size_t close = rest.find(kThinkClose);
    if (close != std::string::npos) {
      const size_t open = rest.find(kThinkOpen);
      const bool opened = open != std::string::npos && open < close;
      // text in front of an opening tag is content; without an opening tag everything up to the end tag is reasoning
      const size_t begin = opened ? open + kThinkOpen.size() : 0;
      p.reasoning = trim(rest.substr(begin, close - begin));
      p.has_reasoning = true;
      rest = (opened ? rest.substr(0, open) : std::string()) + rest.substr(close + kThinkClose.size());
    }
  }
  if (want_tools) {
    std::string kept;
    size_t at = 0;
    for (;;) {
      const size_t open = rest.find(kToolOpen, at);
      if (open == std::string::npos) break;
      const size_t close = rest.find(kToolClose, open + kToolOpen.size());
      if (close == std::string::npos) break;           // unterminated: stays text
      ToolCall call;
      if (parse_call(rest.substr(open + kToolOpen.size(), close - open - kToolOpen.size()), &call)) {
        kept += rest.substr(at, open - at);
        p.tool_calls.push_back(std::move(call));
      } else {
        kept += rest.substr(at, close + kToolClose.size() - at);
      }
      at = close + kToolClose.size();
    }
    kept += rest.substr(at);
    rest = kept;
  }
  p.content = trim(rest);
  return p;
}

std::string render_tools(const Json& tools) {
  if (!tools.is_array()) invalid("'tools' must be an array");
  std::string out = "# Tools\n\nYou may call one or more functions. Function signatures, one JSON object per line:\n<tools>\n";
  for (const auto& t : tools.as_array()) {
    if (!t.is_object()) invalid("every entry of 'tools' must be an object");
    const Json* type = t.find("type");
    if (type && type->is_string() && type->as_string() != "function") invalid("only tools of type 'function' are supported");
    const Json* fn = t.find("function");
    if (!fn || !fn->is_object() || !fn->find("name") || !fn->at("name").is_string()) invalid("a tool needs function.name");
    out += fn->dump() + "\n";
  }
  out += "</tools>\n\nFor each call return a JSON object with the function name and its arguments inside <tool_call></tool_call> tags:\n"
         "<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>\n";
  return out;
}

Json message_json(const Parsed& p, const std::string& id_prefix) {
  Json m = Json::object();
  m.set("role", "assistant");
  if (p.content.empty() && !p.tool_calls.empty()) m.set("content", Json(nullptr));
  else m.set("content", p.content);
  if (p.has_reasoning) m.set("reasoning_content", p.reasoning);
  if (!p.tool_calls.empty()) {
    Json calls = Json::array();
    for (size_t i = 0; i < p.tool_calls.size(); ++i) {
      Json c = Json::object(), f = Json::object();
      c.set("id", id_prefix + "-call-" + std::to_string(i));
      c.set("type", "function");
      f.set("name", p.tool_calls[i].name);
      f.set("arguments", p.tool_calls[i].arguments);
      c.set("function", f);
      calls.push(std::move(c));
    }
    m.set("tool_calls", calls);
  }
  return m;
}

}  // namespace ifab::chat
