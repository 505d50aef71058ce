#include "tokenizer.h"

#include <algorithm>
#include <climits>

namespace ifab::tok {

// ---------------------------------------------------------------------------------------------
// UTF-8 helpers
// ---------------------------------------------------------------------------------------------
namespace {

void append_utf8(std::string& out, uint32_t cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
}

// one code point starting at text[i]; malformed bytes decode as themselves (length 1) so that nothing is ever dropped
uint32_t next_cp(std::string_view text, size_t i, size_t* len) {
  const unsigned char c = (unsigned char)text[i];
  int n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
  if (i + n > text.size()) n = 1;
  for (int k = 1; k < n; ++k)
    if (((unsigned char)text[i + k] & 0xC0) != 0x80) n = 1;
  *len = (size_t)n;
  if (n == 1) return c;
  uint32_t cp = c & (0xFF >> (n + 1));
  for (int k = 1; k < n; ++k) cp = (cp << 6) | ((unsigned char)text[i + k] & 0x3F);
  return cp;
}

// The 256 byte values as printable characters: printable Latin-1 bytes stand for themselves, the other 68 are moved to
// U+0100 onwards in byte order (the table of the GPT-2 byte-level scheme).
struct ByteMap {
  uint32_t to_cp[256];
  std::unordered_map<uint32_t, uint8_t> to_byte;
  ByteMap() {
    uint32_t next = 256;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= 0x21 && b <= 0x7E) || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
      to_cp[b] = keep ? (uint32_t)b : next++;
      to_byte[to_cp[b]] = (uint8_t)b;
    }
  }
};
const ByteMap& byte_map() {
  static const ByteMap m;
  return m;
}

bool is_space(uint32_t c) { return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000; }
bool is_newline(uint32_t c) { return c == '\n' || c == '\r'; }
bool is_digit(uint32_t c) { return (c >= '0' && c <= '9') || (c >= 0x660 && c <= 0x669) || (c >= 0x6F0 && c <= 0x6F9) || (c >= 0x966 && c <= 0x96F) || (c >= 0xFF10 && c <= 0xFF19); }
// Letters: ASCII letters, and beyond ASCII every code point outside the blocks that hold spaces, punctuation and symbols.
bool is_letter(uint32_t c) {
  if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
  if (is_space(c) || is_digit(c)) return false;
  if (c < 0xC0) return c == 0xAA || c == 0xB5 || c == 0xBA;      // Latin-1 symbols: only the three letter-like ones
  if (c == 0xD7 || c == 0xF7) return false;                      // multiplication and division signs
  if (c >= 0x2000 && c <= 0x2BFF) return false;                  // general punctuation, arrows, math, box drawing, dingbats ...
  if (c >= 0x3000 && c <= 0x303F) return false;                  // CJK symbols and punctuation
  if (c >= 0xFE30 && c <= 0xFE6F) return false;                  // CJK compatibility forms, small form variants
  if ((c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) || (c >= 0xFF5B && c <= 0xFF65)) return false;
  if (c >= 0x1F000 && c <= 0x1FAFF) return false;                // emoji and pictographs
  if (c >= 0xE000 && c <= 0xF8FF) return false;                  // private use
  return true;
}

}  // namespace

std::string drain_utf8(std::string& in, bool final) {
  std::string out;
  size_t i = 0;
  while (i < in.size()) {
    const unsigned char c = (unsigned char)in[i];
    const int n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
    if (n == 0) { out += "\xEF\xBF\xBD"; ++i; continue; }
    if (i + n > in.size()) {
      // incomplete tail: keep it unless one of its bytes already rules a valid sequence out, or this is the end
      bool hopeless = false;
      for (size_t k = i + 1; k < in.size(); ++k) hopeless |= ((unsigned char)in[k] & 0xC0) != 0x80;
      if (!final && !hopeless) break;
      out += "\xEF\xBF\xBD";
      ++i;
      continue;
    }
    bool ok = true;
    for (int k = 1; k < n; ++k) ok &= ((unsigned char)in[i + k] & 0xC0) == 0x80;
    if (ok) { out.append(in, i, n); i += n; }
    else { out += "\xEF\xBF\xBD"; ++i; }
  }
  in.erase(0, i);
  return out;
}

std::string Tokenizer::decode(const std::vector<uint32_t>& ids, bool skip_special) const {
  std::string bytes;
  for (uint32_t id : ids) bytes += piece(id, skip_special);
  return drain_utf8(bytes, true);
}

// ---------------------------------------------------------------------------------------------
std::vector<uint32_t> ByteTokenizer::encode(std::string_view text) const {
  std::vector<uint32_t> ids;
  ids.reserve(text.size());
  for (unsigned char c : text) ids.push_back(kFirstByte + c);
  return ids;
}
std::string ByteTokenizer::piece(uint32_t id, bool) const {
  if (id < kFirstByte) return "";
  if (id >= kVocab) return "<|" + std::to_string(id) + "|>";
  return std::string(1, (char)(id - kFirstByte));
}

// ---------------------------------------------------------------------------------------------
BpeTokenizer::BpeTokenizer(std::string_view json_text) {
  const Json j = Json::parse(json_text, (size_t)64 << 20);
  const Json& model = j.at("model");
  if (const Json* t = model.find("type"); t && t->is_string() && t->as_string() != "BPE") invalid("tokenizer.json: model type " + t->as_string() + " is not byte-level BPE");
  bool byte_level = false;
  auto mentions_byte_level = [&](const Json* node, auto&& self) -> bool {
    if (!node || node->is_null()) return false;
    if (node->is_object()) {
      if (const Json* t = node->find("type"); t && t->is_string() && t->as_string() == "ByteLevel") return true;
      for (auto& kv : node->as_object())
        if (self(&kv.second, self)) return true;
    } else if (node->is_array()) {
      for (auto& x : node->as_array())
        if (self(&x, self)) return true;
    }
    return false;
  };
  byte_level = mentions_byte_level(j.find("pre_tokenizer"), mentions_byte_level) || mentions_byte_level(j.find("decoder"), mentions_byte_level);
  if (!byte_level) invalid("tokenizer.json: only byte-level BPE (a ByteLevel pre-tokenizer or decoder) is supported");
  const ByteMap& bm = byte_map();
  auto raw_bytes = [&](const std::string& standin) {
    std::string out;
    for (size_t i = 0; i < standin.size();) {
      size_t n;
      const uint32_t cp = next_cp(standin, i, &n);
      auto it = bm.to_byte.find(cp);
      if (it == bm.to_byte.end()) invalid("tokenizer.json: vocabulary entry '" + standin + "' is not in the byte-level alphabet");
      out.push_back((char)it->second);
      i += n;
    }
    return out;
  };
  size_t max_id = 0;
  for (auto& kv : model.at("vocab").as_object()) max_id = std::max(max_id, (size_t)kv.second.as_int());
  if (const Json* added = j.find("added_tokens"))
    for (auto& a : added->as_array()) max_id = std::max(max_id, (size_t)a.at("id").as_int());
  if (max_id > 4000000) fail(ErrorKind::Capacity, "tokenizer.json: ids above 4,000,000");
  pieces_.assign(max_id + 1, std::string());
  special_.assign(max_id + 1, 0);
  std::vector<uint8_t> defined(max_id + 1, 0);
  for (auto& kv : model.at("vocab").as_object()) {
    const uint32_t id = (uint32_t)kv.second.as_int();
    vocab_[kv.first] = id;
    pieces_[id] = raw_bytes(kv.first);
    defined[id] = 1;
  }
  uint32_t rank = 0;
  for (auto& m : model.at("merges").as_array()) {
    std::string key;
    if (m.is_string()) key = m.as_string();
    else if (m.is_array() && m.size() == 2) key = m.as_array()[0].as_string() + " " + m.as_array()[1].as_string();
    else invalid("tokenizer.json: a merge is \"left right\" or [left, right]");
    if (key.find(' ') == std::string::npos) invalid("tokenizer.json: malformed merge '" + key + "'");
    ranks_.emplace(std::move(key), rank++);
  }
  if (const Json* added = j.find("added_tokens")) {
    for (auto& a : added->as_array()) {
      const uint32_t id = (uint32_t)a.at("id").as_int();
      const std::string& content = a.at("content").as_string();
      if (content.empty()) continue;
      pieces_[id] = content;              // added tokens are stored as plain text, not in the stand-in alphabet
      defined[id] = 1;
      const Json* sp = a.find("special");
      special_[id] = sp && sp->is_bool() && sp->as_bool();
      added_.emplace_back(content, id);
    }
    std::sort(added_.begin(), added_.end(), [](auto& x, auto& y) { return x.first.size() != y.first.size() ? x.first.size() > y.first.size() : x.first < y.first; });
  }
  for (size_t id = 0; id <= max_id; ++id)
    if (!defined[id]) pieces_[id] = "<|" + std::to_string(id) + "|>";
  for (const char* name : {"<|endoftext|>", "<|im_end|>", "</s>", "<|end_of_text|>", "<|eot_id|>"})
    if (eos_ < 0) eos_ = token_id(name);
  for (const char* name : {"<|begin_of_text|>", "<s>", "<|startoftext|>"})
    if (bos_ < 0) bos_ = token_id(name);
}

std::shared_ptr<BpeTokenizer> BpeTokenizer::from_file(const std::string& path) { return std::make_shared<BpeTokenizer>(read_file(path, (size_t)64 << 20)); }

int64_t BpeTokenizer::token_id(std::string_view text) const {
  for (auto& a : added_)
    if (a.first == text) return a.second;
  return -1;
}

std::string BpeTokenizer::piece(uint32_t id, bool skip_special) const {
  if (id >= pieces_.size()) return "<|" + std::to_string(id) + "|>";
  if (skip_special && special_[id]) return "";
  return pieces_[id];
}

// Words in the order of the text. Rules, first match wins at every position:
//   1. a contraction suffix: ' followed by s t m d (any case) or re ve ll
//   2. an optional single character that is neither letter, digit nor newline, then one or more letters
//   3. one digit
//   4. an optional blank, then one or more characters that are neither space, letter nor digit, then any newlines
//   5. whitespace up to and including its last newline
//   6. whitespace followed by more text: all of it but the last character (which joins the next word); at the end: all of it
std::vector<std::string_view> BpeTokenizer::split_words(std::string_view text) {
  std::vector<std::string_view> words;
  std::vector<uint32_t> cps;
  std::vector<size_t> offs;
  for (size_t i = 0; i < text.size();) {
    size_t n;
    cps.push_back(next_cp(text, i, &n));
    offs.push_back(i);
    i += n;
  }
  offs.push_back(text.size());
  const size_t N = cps.size();
  auto lower = [](uint32_t c) { return c >= 'A' && c <= 'Z' ? c + 32 : c; };
  size_t i = 0;
  while (i < N) {
    size_t end = 0;
    const uint32_t c = cps[i];
    if (c == '\'' && i + 1 < N) {
      const uint32_t a = lower(cps[i + 1]), b = i + 2 < N ? lower(cps[i + 2]) : 0;
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) end = i + 3;
      else if (a == 's' || a == 't' || a == 'm' || a == 'd') end = i + 2;
    }
    if (!end) {
      size_t k = i;
      if (!is_letter(c) && !is_digit(c) && !is_newline(c) && k + 1 < N && is_letter(cps[k + 1])) ++k;
      if (is_letter(cps[k])) {
        while (k < N && is_letter(cps[k])) ++k;
        end = k;
      }
    }
    if (!end && is_digit(c)) end = i + 1;
    if (!end) {
      size_t k = i;
      if (c == ' ' && k + 1 < N) ++k;
      auto other = [&](uint32_t x) { return !is_space(x) && !is_letter(x) && !is_digit(x); };
      if (k < N && other(cps[k])) {
        while (k < N && other(cps[k])) ++k;
        while (k < N && is_newline(cps[k])) ++k;
        end = k;
      }
    }
    if (!end) {
      // c is whitespace here
      size_t k = i, last_newline = 0;
      bool any_newline = false;
      while (k < N && is_space(cps[k])) {
        if (is_newline(cps[k])) { any_newline = true; last_newline = k; }
        ++k;
      }
      if (any_newline) end = last_newline + 1;
      else if (k < N && k - i > 1) end = k - 1;
      else end = k > i ? k : i + 1;
    }
    words.push_back(text.substr(offs[i], offs[end] - offs[i]));
    i = end;
  }
  return words;
}

void BpeTokenizer::encode_word(std::string_view word, std::vector<uint32_t>& out) const {
  auto hit = cache_.find(std::string(word));
  if (hit != cache_.end()) {
    out.insert(out.end(), hit->second.begin(), hit->second.end());
    return;
  }
  const ByteMap& bm = byte_map();
  std::vector<std::string> sym;
  for (unsigned char b : word) {
    std::string s;
    append_utf8(s, bm.to_cp[b]);
    sym.push_back(std::move(s));
  }
  while (sym.size() > 1) {
    uint32_t best = UINT32_MAX;
    size_t at = 0;
    for (size_t k = 0; k + 1 < sym.size(); ++k) {
      auto it = ranks_.find(sym[k] + " " + sym[k + 1]);
      if (it != ranks_.end() && it->second < best) { best = it->second; at = k; }
    }
    if (best == UINT32_MAX) break;
    sym[at] += sym[at + 1];
    sym.erase(sym.begin() + (long)at + 1);
  }
  std::vector<uint32_t> ids;
  for (auto& s : sym) {
    auto it = vocab_.find(s);
    if (it != vocab_.end()) { ids.push_back(it->second); continue; }
    // a symbol the vocabulary lacks (possible only with a truncated vocabulary): fall back to its single characters
    for (size_t i = 0; i < s.size();) {
      size_t n;
      next_cp(s, i, &n);
      auto one = vocab_.find(s.substr(i, n));
      if (one == vocab_.end()) invalid("tokenizer: the vocabulary has no entry for byte stand-in '" + s.substr(i, n) + "'");
      ids.push_back(one->second);
      i += n;
    }
  }
  if (cache_.size() < 200000) cache_[std::string(word)] = ids;
  out.insert(out.end(), ids.begin(), ids.end());
}

std::vector<uint32_t> BpeTokenizer::encode(std::string_view text) const {
  std::vector<uint32_t> out;
  size_t start = 0, i = 0;
  auto flush = [&](size_t upto) {
    if (upto > start)
      for (auto w : split_words(text.substr(start, upto - start))) encode_word(w, out);
  };
  while (i < text.size()) {
    const std::pair<std::string, uint32_t>* match = nullptr;
    if (!added_.empty())
      for (auto& a : added_)
        if (text.compare(i, a.first.size(), a.first) == 0) { match = &a; break; }    // longest first
    if (match) {
      flush(i);
      out.push_back(match->second);
      i += match->first.size();
      start = i;
    } else {
      ++i;
    }
  }
  flush(text.size());
  return out;
}

// ---------------------------------------------------------------------------------------------
std::string Detokenizer::feed(uint32_t id) {
  pending_ += tok_->piece(id, skip_special_);
  return drain_utf8(pending_, false);
}
std::string Detokenizer::flush() { return drain_utf8(pending_, true); }

std::string render_chat(const std::vector<ChatMessage>& messages, const Tokenizer& tok, const std::string& style) {
  bool chatml = style == "chatml";
  if (style == "auto") chatml = tok.token_id("<|im_start|>") >= 0 && tok.token_id("<|im_end|>") >= 0;
  else if (style != "chatml" && style != "plain") invalid("chat template style is auto, chatml or plain");
  std::string text;
  for (auto& m : messages) {
    if (m.role.empty() || m.role.find_first_of("<>|\n") != std::string::npos) invalid("a message role is a plain word");
    if (chatml) text += "<|im_start|>" + m.role + "\n" + m.content + "<|im_end|>\n";
    else text += "<|" + m.role + "|>\n" + m.content + "\n";
  }
  text += chatml ? "<|im_start|>assistant\n" : "<|assistant|>\n";
  return text;
}

std::shared_ptr<Tokenizer> load_tokenizer(const std::string& spec) {
  if (spec.empty() || spec == "bytes") return std::make_shared<ByteTokenizer>();
  return BpeTokenizer::from_file(spec);
}

}  // namespace ifab::tok
