#include "base.h"

#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <sstream>
#include <unistd.h>

namespace ifab {

const char* error_kind_name(ErrorKind k) {
  switch (k) {
    case ErrorKind::Invalid: return "invalid";
    case ErrorKind::Capacity: return "capacity";
    case ErrorKind::NotImplemented: return "not implemented";
    case ErrorKind::Backend: return "backend";
    case ErrorKind::Stale: return "stale";
    case ErrorKind::Io: return "io";
  }
  return "?";
}

// ---------------------------------------------------------------------------------------------
bool Json::as_bool() const {
  if (auto p = std::get_if<bool>(&v_)) return *p;
  invalid("json: expected bool");
}
int64_t Json::as_int() const {
  if (auto p = std::get_if<int64_t>(&v_)) return *p;
  if (auto d = std::get_if<double>(&v_)) {
    if (std::floor(*d) == *d && std::fabs(*d) < 9.0e15) return (int64_t)*d;
  }
  invalid("json: expected integer");
}
double Json::as_double() const {
  if (auto p = std::get_if<double>(&v_)) return *p;
  if (auto i = std::get_if<int64_t>(&v_)) return (double)*i;
  invalid("json: expected number");
}
const std::string& Json::as_string() const {
  if (auto p = std::get_if<std::string>(&v_)) return *p;
  invalid("json: expected string");
}
const JsonArray& Json::as_array() const {
  if (auto p = std::get_if<JsonArray>(&v_)) return *p;
  invalid("json: expected array");
}
JsonArray& Json::as_array() {
  if (auto p = std::get_if<JsonArray>(&v_)) return *p;
  invalid("json: expected array");
}
const JsonObject& Json::as_object() const {
  if (auto p = std::get_if<JsonObject>(&v_)) return *p;
  invalid("json: expected object");
}
JsonObject& Json::as_object() {
  if (auto p = std::get_if<JsonObject>(&v_)) return *p;
  invalid("json: expected object");
}
const Json* Json::find(std::string_view key) const {
  if (!is_object()) return nullptr;
  for (auto& kv : std::get<JsonObject>(v_))
    if (kv.first == key) return &kv.second;
  return nullptr;
}
const Json& Json::at(std::string_view key) const {
  if (auto p = find(key)) return *p;
  invalid("json: missing key '" + std::string(key) + "'");
}
Json& Json::set(const std::string& key, Json value) {
  auto& o = as_object();
  for (auto& kv : o)
    if (kv.first == key) {
      kv.second = std::move(value);
      return kv.second;
    }
  o.emplace_back(key, std::move(value));
  return o.back().second;
}
void Json::push(Json value) { as_array().push_back(std::move(value)); }
size_t Json::size() const {
  if (is_array()) return std::get<JsonArray>(v_).size();
  if (is_object()) return std::get<JsonObject>(v_).size();
  return 0;
}

std::string json_escape(std::string_view s) {
  std::string out;
  out.reserve(s.size() + 2);
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char b[8];
          snprintf(b, sizeof b, "\\u%04x", c);
          out += b;
        } else {
          out += (char)c;
        }
    }
  }
  return out;
}

std::string format_double(double v) {
  if (std::isfinite(v) && std::floor(v) == v && std::fabs(v) < 1e15) {
    char b[32];
    snprintf(b, sizeof b, "%.1f", v);
    return b;
  }
  char b[40];
  snprintf(b, sizeof b, "%.17g", v);
  double back = strtod(b, nullptr);
  for (int prec = 1; prec < 17; ++prec) {
    char c[40];
    snprintf(c, sizeof c, "%.*g", prec, v);
    if (strtod(c, nullptr) == back) return c;
  }
  return b;
}

void Json::dump_to(std::string& out, int indent, int depth) const {
  auto nl = [&](int d) {
    if (indent < 0) return;
    out += '\n';
    out.append((size_t)(indent * d), ' ');
  };
  switch (type()) {
    case Type::Null: out += "null"; break;
    case Type::Bool: out += std::get<bool>(v_) ? "true" : "false"; break;
    case Type::Int: out += std::to_string(std::get<int64_t>(v_)); break;
    case Type::Double: {
      double d = std::get<double>(v_);
      out += std::isfinite(d) ? format_double(d) : "null";
      break;
    }
    case Type::String:
      out += '"';
      out += json_escape(std::get<std::string>(v_));
      out += '"';
      break;
    case Type::Array: {
      auto& a = std::get<JsonArray>(v_);
      if (a.empty()) { out += "[]"; break; }
      out += '[';
      for (size_t i = 0; i < a.size(); ++i) {
        if (i) out += ',';
        nl(depth + 1);
        a[i].dump_to(out, indent, depth + 1);
      }
      nl(depth);
      out += ']';
      break;
    }
    case Type::Object: {
      auto& o = std::get<JsonObject>(v_);
      if (o.empty()) { out += "{}"; break; }
      out += '{';
      for (size_t i = 0; i < o.size(); ++i) {
        if (i) out += ',';
        nl(depth + 1);
        out += '"';
        out += json_escape(o[i].first);
        out += indent < 0 ? "\":" : "\": ";
        o[i].second.dump_to(out, indent, depth + 1);
      }
      nl(depth);
      out += '}';
      break;
    }
  }
}
std::string Json::dump(int indent) const {
  std::string out;
  dump_to(out, indent, 0);
  return out;
}

namespace {
struct JsonParser {
  std::string_view s;
  size_t i = 0;
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  [[noreturn]] void err(const std::string& m) { invalid("json: " + m + " at byte " + std::to_string(i)); }
  Json value(int depth) {
    if (depth > 64) err("nesting too deep");
    ws();
    if (i >= s.size()) err("unexpected end");
    char c = s[i];
    if (c == '{') {
      ++i;
      JsonObject o;
      ws();
      if (i < s.size() && s[i] == '}') { ++i; return Json(std::move(o)); }
      for (;;) {
        ws();
        if (i >= s.size() || s[i] != '"') err("expected key");
        std::string k = string();
        for (auto& kv : o)
          if (kv.first == k) err("duplicate key '" + k + "'");
        ws();
        if (i >= s.size() || s[i] != ':') err("expected ':'");
        ++i;
        o.emplace_back(std::move(k), value(depth + 1));
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; break; }
        err("expected ',' or '}'");
      }
      return Json(std::move(o));
    }
    if (c == '[') {
      ++i;
      JsonArray a;
      ws();
      if (i < s.size() && s[i] == ']') { ++i; return Json(std::move(a)); }
      for (;;) {
        a.push_back(value(depth + 1));
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; break; }
        err("expected ',' or ']'");
      }
      return Json(std::move(a));
    }
    if (c == '"') return Json(string());
    if (s.compare(i, 4, "true") == 0) { i += 4; return Json(true); }
    if (s.compare(i, 5, "false") == 0) { i += 5; return Json(false); }
    if (s.compare(i, 4, "null") == 0) { i += 4; return Json(nullptr); }
    return number();
  }
  std::string string() {
    ++i;
    std::string out;
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c == '\\') {
        if (i >= s.size()) err("bad escape");
        char e = s[i++];
        switch (e) {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            if (i + 4 > s.size()) err("bad \\u escape");
            unsigned cp = 0;
            for (int k = 0; k < 4; ++k) {
              char h = s[i++];
              cp <<= 4;
              if (h >= '0' && h <= '9') cp |= (unsigned)(h - '0');
              else if (h >= 'a' && h <= 'f') cp |= (unsigned)(h - 'a' + 10);
              else if (h >= 'A' && h <= 'F') cp |= (unsigned)(h - 'A' + 10);
              else err("bad hex digit");
            }
            if (cp >= 0xD800 && cp <= 0xDBFF && i + 6 <= s.size() && s[i] == '\\' && s[i + 1] == 'u') {
              // a surrogate pair: two \u escapes name one code point beyond U+FFFF
              unsigned lo = 0;
              bool hex = true;
              for (int k = 0; k < 4; ++k) {
                const char h = s[i + 2 + k];
                lo <<= 4;
                if (h >= '0' && h <= '9') lo |= (unsigned)(h - '0');
                else if (h >= 'a' && h <= 'f') lo |= (unsigned)(h - 'a' + 10);
                else if (h >= 'A' && h <= 'F') lo |= (unsigned)(h - 'A' + 10);
                else hex = false;
              }
              if (hex && lo >= 0xDC00 && lo <= 0xDFFF) {
                cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                i += 6;
              }
            }
            if (cp >= 0xD800 && cp <= 0xDFFF) cp = 0xFFFD;   // a lone surrogate is not a character
            if (cp < 0x80) out += (char)cp;
            else if (cp < 0x800) { out += (char)(0xc0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3f)); }
            else if (cp < 0x10000) { out += (char)(0xe0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3f)); out += (char)(0x80 | (cp & 0x3f)); }
            else { out += (char)(0xf0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3f)); out += (char)(0x80 | ((cp >> 6) & 0x3f)); out += (char)(0x80 | (cp & 0x3f)); }
            break;
          }
          default: err("bad escape");
        }
      } else {
        out += c;
      }
    }
    if (i >= s.size()) err("unterminated string");
    ++i;
    return out;
  }
  Json number() {
    size_t b = i;
    bool is_float = false;
    if (i < s.size() && (s[i] == '-' || s[i] == '+')) ++i;
    while (i < s.size() && (isdigit((unsigned char)s[i]) || s[i] == '.' || s[i] == 'e' || s[i] == 'E' || s[i] == '-' || s[i] == '+')) {
      if (s[i] == '.' || s[i] == 'e' || s[i] == 'E') is_float = true;
      ++i;
    }
    if (b == i) err("unexpected character");
    std::string t(s.substr(b, i - b));
    if (!is_float) {
      errno = 0;
      char* end = nullptr;
      long long v = strtoll(t.c_str(), &end, 10);
      if (errno == 0 && end && *end == 0) return Json((int64_t)v);
    }
    char* end = nullptr;
    double d = strtod(t.c_str(), &end);
    if (!end || *end != 0) err("bad number");
    return Json(d);
  }
};
}  // namespace

Json Json::parse(std::string_view text, size_t max_bytes) {
  if (text.size() > max_bytes) fail(ErrorKind::Capacity, "json: document larger than limit");
  JsonParser p{text};
  Json v = p.value(0);
  p.ws();
  if (p.i != text.size()) p.err("trailing data");
  return v;
}

// ---------------------------------------------------------------------------------------------
static const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
static inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

Sha256::Sha256() {
  static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  memcpy(h_, init, sizeof init);
}
void Sha256::block(const uint8_t* p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h_[0], b = h_[1], c = h_[2], d = h_[3], e = h_[4], f = h_[5], g = h_[6], h = h_[7];
  for (int i = 0; i < 64; ++i) {
    uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
    uint32_t t1 = h + S1 + ch + K256[i] + w[i];
    uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
    uint32_t t2 = S0 + mj;
    h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h_[0] += a; h_[1] += b; h_[2] += c; h_[3] += d; h_[4] += e; h_[5] += f; h_[6] += g; h_[7] += h;
}
void Sha256::update(const void* data, size_t len) {
  const uint8_t* p = (const uint8_t*)data;
  total_ += len;
  while (len) {
    size_t n = std::min(len, 64 - fill_);
    memcpy(buf_ + fill_, p, n);
    fill_ += n; p += n; len -= n;
    if (fill_ == 64) { block(buf_); fill_ = 0; }
  }
}
std::string Sha256::hex() {
  uint64_t bits = total_ * 8;
  uint8_t pad = 0x80;
  update(&pad, 1);
  uint8_t z = 0;
  while (fill_ != 56) update(&z, 1);
  uint8_t len[8];
  for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
  update(len, 8);
  char out[65];
  for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", h_[i]);
  return std::string(out, 64);
}
std::string Sha256::of(std::string_view data) {
  Sha256 s;
  s.update(data.data(), data.size());
  return s.hex();
}
uint64_t fnv1a64(const void* data, size_t len, uint64_t seed) {
  const uint8_t* p = (const uint8_t*)data;
  uint64_t h = seed;
  for (size_t i = 0; i < len; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
  return h;
}
std::string hex64(uint64_t v) {
  char b[17];
  snprintf(b, sizeof b, "%016llx", (unsigned long long)v);
  return b;
}

// ---------------------------------------------------------------------------------------------
void ByteReader::need(size_t n) const {
  if (b_.size() - pos_ < n) invalid("binary: truncated input at byte " + std::to_string(pos_));
}
uint8_t ByteReader::u8() { need(1); return (uint8_t)b_[pos_++]; }
uint32_t ByteReader::u32() {
  need(4);
  uint32_t v = 0;
  for (int i = 0; i < 4; ++i) v |= (uint32_t)(uint8_t)b_[pos_ + i] << (8 * i);
  pos_ += 4;
  return v;
}
uint64_t ByteReader::u64() {
  need(8);
  uint64_t v = 0;
  for (int i = 0; i < 8; ++i) v |= (uint64_t)(uint8_t)b_[pos_ + i] << (8 * i);
  pos_ += 8;
  return v;
}
std::string ByteReader::str(size_t max_len) {
  uint32_t n = u32();
  if (n > max_len) fail(ErrorKind::Capacity, "binary: string longer than limit");
  need(n);
  std::string s(b_.substr(pos_, n));
  pos_ += n;
  return s;
}
std::string_view ByteReader::raw(size_t n) {
  need(n);
  auto v = b_.substr(pos_, n);
  pos_ += n;
  return v;
}

// ---------------------------------------------------------------------------------------------
std::string read_file(const std::string& path, size_t max_bytes) {
  std::ifstream f(path, std::ios::binary);
  if (!f) fail(ErrorKind::Io, "cannot open " + path);
  f.seekg(0, std::ios::end);
  std::streamoff n = f.tellg();
  if (n < 0) fail(ErrorKind::Io, "cannot stat " + path);
  if ((size_t)n > max_bytes) fail(ErrorKind::Capacity, path + " is larger than the limit");
  f.seekg(0);
  std::string s((size_t)n, '\0');
  f.read(s.data(), n);
  if (!f) fail(ErrorKind::Io, "short read of " + path);
  return s;
}
void write_file(const std::string& path, std::string_view data) {
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) fail(ErrorKind::Io, "cannot create " + path);
  f.write(data.data(), (std::streamsize)data.size());
  f.flush();
  if (!f) fail(ErrorKind::Io, "short write of " + path);
}
void write_file_atomic(const std::string& path, std::string_view data) {
  std::string tmp = path + ".tmp." + std::to_string((long)getpid());
  write_file(tmp, data);
  std::error_code ec;
  std::filesystem::rename(tmp, path, ec);
  if (ec) {
    std::filesystem::remove(tmp);
    fail(ErrorKind::Io, "cannot rename into " + path + ": " + ec.message());
  }
}
bool path_exists(const std::string& path) {
  std::error_code ec;
  return std::filesystem::exists(path, ec);
}
void make_dirs(const std::string& path) {
  std::error_code ec;
  std::filesystem::create_directories(path, ec);
  if (ec) fail(ErrorKind::Io, "cannot create directory " + path + ": " + ec.message());
}

}  // namespace ifab
