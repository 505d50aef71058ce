// Foundation of the host-side core: error vocabulary, a small JSON value with a bounded,
// duplicate-key-rejecting parser, SHA-256, FNV-1a, little-endian byte writer/reader and file helpers.
//
// Error kinds mirror the reference's model vocabulary (crates/inferfabric-model/src/lib.rs:6-13):
// Invalid, Capacity, NotImplemented, Backend, Stale, Io.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <string_view>
#include <utility>
#include <variant>
#include <vector>

namespace ifab {

enum class ErrorKind { Invalid, Capacity, NotImplemented, Backend, Stale, Io };
const char* error_kind_name(ErrorKind k);

class Error : public std::runtime_error {
 public:
  Error(ErrorKind kind, const std::string& msg) : std::runtime_error(msg), kind_(kind) {}
  ErrorKind kind() const { return kind_; }
  std::string describe() const { return std::string(error_kind_name(kind_)) + ": " + what(); }

 private:
  ErrorKind kind_;
};
[[noreturn]] inline void fail(ErrorKind k, const std::string& m) { throw Error(k, m); }
[[noreturn]] inline void invalid(const std::string& m) { throw Error(ErrorKind::Invalid, m); }

// ---------------------------------------------------------------------------------------------
// JSON
// ---------------------------------------------------------------------------------------------
class Json;
using JsonArray = std::vector<Json>;
using JsonObject = std::vector<std::pair<std::string, Json>>;  // insertion ordered

class Json {
 public:
  enum class Type { Null, Bool, Int, Double, String, Array, Object };
  Json() : v_(nullptr) {}
  Json(std::nullptr_t) : v_(nullptr) {}
  Json(bool b) : v_(b) {}
  Json(int i) : v_((int64_t)i) {}
  Json(unsigned i) : v_((int64_t)i) {}
  Json(int64_t i) : v_(i) {}
  Json(uint64_t i) : v_((int64_t)i) {}
  Json(double d) : v_(d) {}
  Json(const char* s) : v_(std::string(s)) {}
  Json(std::string s) : v_(std::move(s)) {}
  Json(JsonArray a) : v_(std::move(a)) {}
  Json(JsonObject o) : v_(std::move(o)) {}
  static Json array() { return Json(JsonArray{}); }
  static Json object() { return Json(JsonObject{}); }

  Type type() const { return (Type)v_.index(); }
  bool is_null() const { return type() == Type::Null; }
  bool is_bool() const { return type() == Type::Bool; }
  bool is_int() const { return type() == Type::Int; }
  bool is_number() const { return type() == Type::Int || type() == Type::Double; }
  bool is_string() const { return type() == Type::String; }
  bool is_array() const { return type() == Type::Array; }
  bool is_object() const { return type() == Type::Object; }

  bool as_bool() const;
  int64_t as_int() const;
  double as_double() const;
  const std::string& as_string() const;
  const JsonArray& as_array() const;
  JsonArray& as_array();
  const JsonObject& as_object() const;
  JsonObject& as_object();

  // object helpers
  const Json* find(std::string_view key) const;
  const Json& at(std::string_view key) const;            // throws Invalid when missing
  Json& set(const std::string& key, Json value);         // insert or replace; returns the stored value
  void push(Json value);                                 // array append
  size_t size() const;

  std::string dump(int indent = -1) const;
  // Parse with limits: `max_bytes` input size, nesting <= 64, duplicate object keys rejected.
  static Json parse(std::string_view text, size_t max_bytes = (size_t)64 << 20);

 private:
  void dump_to(std::string& out, int indent, int depth) const;
  std::variant<std::nullptr_t, bool, int64_t, double, std::string, JsonArray, JsonObject> v_;
};

std::string json_escape(std::string_view s);

// ---------------------------------------------------------------------------------------------
// hashing
// ---------------------------------------------------------------------------------------------
class Sha256 {
 public:
  Sha256();
  void update(const void* data, size_t len);
  std::string hex();  // finalises
  static std::string of(std::string_view data);

 private:
  void block(const uint8_t* p);
  uint32_t h_[8];
  uint8_t buf_[64];
  uint64_t total_ = 0;
  size_t fill_ = 0;
};
uint64_t fnv1a64(const void* data, size_t len, uint64_t seed = 0xcbf29ce484222325ull);
std::string hex64(uint64_t v);

// ---------------------------------------------------------------------------------------------
// little-endian binary writer / bounded reader
// ---------------------------------------------------------------------------------------------
class ByteWriter {
 public:
  void u8(uint8_t v) { b_.push_back((char)v); }
  void u32(uint32_t v) { for (int i = 0; i < 4; ++i) b_.push_back((char)((v >> (8 * i)) & 0xff)); }
  void u64(uint64_t v) { for (int i = 0; i < 8; ++i) b_.push_back((char)((v >> (8 * i)) & 0xff)); }
  void str(std::string_view s) { u32((uint32_t)s.size()); b_.append(s); }
  void raw(std::string_view s) { b_.append(s); }
  const std::string& bytes() const { return b_; }
  std::string take() { return std::move(b_); }

 private:
  std::string b_;
};

class ByteReader {
 public:
  explicit ByteReader(std::string_view b) : b_(b) {}
  uint8_t u8();
  uint32_t u32();
  uint64_t u64();
  std::string str(size_t max_len = 1 << 20);
  std::string_view raw(size_t n);
  bool done() const { return pos_ == b_.size(); }
  size_t pos() const { return pos_; }
  size_t remaining() const { return b_.size() - pos_; }

 private:
  void need(size_t n) const;
  std::string_view b_;
  size_t pos_ = 0;
};

// ---------------------------------------------------------------------------------------------
// files
// ---------------------------------------------------------------------------------------------
std::string read_file(const std::string& path, size_t max_bytes = (size_t)1 << 32);
void write_file(const std::string& path, std::string_view data);
// write to a sibling temporary then rename (readers never see a partial file)
void write_file_atomic(const std::string& path, std::string_view data);
bool path_exists(const std::string& path);
void make_dirs(const std::string& path);

std::string format_double(double v);

}  // namespace ifab
