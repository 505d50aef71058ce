// Post-processing of assistant text for the chat route: reasoning sections and tool calls.
//
//   <think> ... </think>                    -> message.reasoning_content (a closing tag without an opening one counts too:
//                                              templates that open the section in the prompt leave only the end in the output)
//   <tool_call> {"name": ..., "arguments": {...}} </tool_call>   (any number)  -> message.tool_calls[]
//
// Whatever does not parse stays in the content verbatim: a malformed block is text, never an error. `render_tools` is the
// other direction - the `tools` array of a request as a system block of the prompt, in the same tag vocabulary.
// Reference: vendored front end, parser crate (tool-call and reasoning parsers) and chat crate (templates)
// (vendor/rust/src/parser, vendor/rust/src/chat).
#pragma once
#include <string>
#include <vector>

#include "base.h"

namespace ifab::chat {

struct ToolCall {
  std::string name;
  std::string arguments;   // JSON text of the arguments object
};

struct Parsed {
  std::string content;     // text outside the recognised sections, trimmed of the whitespace the sections leave behind
  std::string reasoning;
  bool has_reasoning = false;
  std::vector<ToolCall> tool_calls;
};

Parsed parse_assistant(const std::string& text, bool want_reasoning = true, bool want_tools = true);

// The `tools` array of a chat request (OpenAI function schema) as prompt text; throws Invalid on a malformed entry.
std::string render_tools(const Json& tools);

// message JSON of a chat completion: role, content, and reasoning_content / tool_calls when present
Json message_json(const Parsed& p, const std::string& id_prefix);

}  // namespace ifab::chat
