#include "lang.h"

#include <algorithm>
#include <cstdlib>
#include <functional>

namespace ifab::lang {

namespace {

constexpr size_t kMaxSource = 1 << 20;
constexpr size_t kMaxTokens = 100000;
constexpr size_t kMaxModules = 256;
constexpr size_t kMaxNesting = 64;
constexpr size_t kMaxFold = 4096;
constexpr size_t kMaxNodes = 10000;
constexpr size_t kMaxSteps = 100000;
constexpr size_t kMaxRecordFields = 64;

struct Token {
  enum class Kind { Ident, Number, String, Punct, End };
  Kind kind;
  std::string text;
  size_t start, end;
};

[[noreturn]] void err_at(size_t byte, const std::string& m) { invalid("byte " + std::to_string(byte) + ": " + m); }

std::vector<Token> lex(std::string_view s) {
  if (s.size() > kMaxSource) fail(ErrorKind::Capacity, "DSL source exceeds 1 MiB");
  std::vector<Token> out;
  size_t i = 0;
  auto ident_start = [](unsigned char c) { return isalpha(c) || c == '_'; };
  auto ident_body = [](unsigned char c) { return isalnum(c) || c == '_' || c == '.'; };
  while (i < s.size()) {
    unsigned char c = (unsigned char)s[i];
    if (isspace(c)) { ++i; continue; }
    if (c == '#' || (c == '/' && i + 1 < s.size() && s[i + 1] == '/')) {
      while (i < s.size() && s[i] != '\n') ++i;
      continue;
    }
    size_t b = i;
    Token t;
    if (c == '"') {
      ++i;
      std::string body;
      bool closed = false;
      while (i < s.size()) {
        if (s[i] == '\\' && i + 1 < s.size()) { body += s[i + 1]; i += 2; continue; }
        if (s[i] == '"') { ++i; closed = true; break; }
        body += s[i++];
      }
      if (!closed) err_at(b, "unterminated string");
      t = {Token::Kind::String, body, b, i};
    } else if (ident_start(c)) {
      while (i < s.size() && ident_body((unsigned char)s[i])) ++i;
      t = {Token::Kind::Ident, std::string(s.substr(b, i - b)), b, i};
    } else if (isdigit(c) || c == '-') {
      ++i;
      while (i < s.size() && (isdigit((unsigned char)s[i]) || s[i] == '.' || s[i] == 'e' || s[i] == 'E' || s[i] == '+' || s[i] == '-')) ++i;
      t = {Token::Kind::Number, std::string(s.substr(b, i - b)), b, i};
    } else if (std::string_view("{}[]()<>=,:;").find((char)c) != std::string_view::npos) {
      ++i;
      t = {Token::Kind::Punct, std::string(1, (char)c), b, i};
    } else {
      err_at(i, "unsupported character");
    }
    out.push_back(std::move(t));
    if (out.size() > kMaxTokens) fail(ErrorKind::Capacity, "DSL token limit (100000)");
  }
  out.push_back({Token::Kind::End, "", s.size(), s.size()});
  return out;
}

class Parser {
 public:
  explicit Parser(std::vector<Token> t) : t_(std::move(t)) {}

  Document document() {
    expect_ident("language");
    expect_ident("inferfabric");
    if (peek().kind != Token::Kind::Number || peek().text != "1") err("unsupported language version (expected `language inferfabric 1;`)");
    ++p_;
    expect(";");
    Document d;
    while (is_ident("module")) {
      if (d.modules.size() >= kMaxModules) fail(ErrorKind::Capacity, "more than 256 modules");
      d.modules.push_back(module());
    }
    expect_ident("model");
    d.model_name = ident();
    d.model = members(true, 0);
    expect_ident("plan");
    d.plan_name = ident();
    expect_ident("for");
    d.plan_model = ident();
    if (d.plan_model != d.model_name) err("plan targets unknown model " + d.plan_model);
    d.plan = members(false, 0);
    if (peek().kind != Token::Kind::End) err("unexpected text after the plan block");
    return d;
  }

 private:
  const Token& peek(size_t k = 0) const { return t_[std::min(p_ + k, t_.size() - 1)]; }
  [[noreturn]] void err(const std::string& m) const { err_at(peek().start, m); }
  bool is(const char* punct) const { return peek().kind == Token::Kind::Punct && peek().text == punct; }
  bool is_ident(const char* w) const { return peek().kind == Token::Kind::Ident && peek().text == w; }
  void expect(const char* punct) {
    if (!is(punct)) err(std::string("expected '") + punct + "'");
    ++p_;
  }
  void expect_ident(const char* w) {
    if (!is_ident(w)) err(std::string("expected '") + w + "'");
    ++p_;
  }
  std::string ident() {
    if (peek().kind != Token::Kind::Ident) err("expected identifier");
    return t_[p_++].text;
  }

  Module module() {
    Module m;
    m.pos = peek().start;
    expect_ident("module");
    m.name = ident();
    if (m.name.find('.') != std::string::npos) err("module name cannot contain '.'");
    expect("(");
    while (!is(")")) {
      std::string p = ident();
      if (p.find('.') != std::string::npos) err("parameter name cannot contain '.'");
      if (std::find(m.params.begin(), m.params.end(), p) != m.params.end()) err("duplicate parameter " + p);
      m.params.push_back(p);
      if (!is(",")) break;
      ++p_;
    }
    expect(")");
    m.body = members(true, 0);
    return m;
  }

  // A bracketed list of numeric literals, read straight from the tokens: `[` number (`,` number)* `]`. `what` names the
  // list in diagnostics ("shape", "initializer"); each literal goes through `take` with its position for the message.
  template <class F>
  size_t literal_list(const char* what, F&& take) {
    if (!is("[")) err(std::string(what) + ": expected '[' and a list of numbers");
    ++p_;
    size_t n = 0;
    while (!is("]")) {
      const Token& t = peek();
      if (t.kind != Token::Kind::Number) err(std::string(what) + ": entry " + std::to_string(n) + " is not a number literal");
      take(t.text, n);
      ++p_;
      ++n;
      if (!is(",")) break;
      ++p_;
    }
    expect("]");
    return n;
  }

  // what follows the keyword of a graph-body declaration
  struct DeclForm {
    const char* keyword;
    Member::Kind kind;
    bool named, typed, initialised, valued;   // NAME / ": tensor<f32>[dims]" / "= [floats]" / "= expr" (or bare expr when unnamed)
  };
  static const DeclForm* decl_form(const std::string& key) {
    static const DeclForm forms[] = {
        {"input", Member::Kind::Input, true, true, false, false},   {"const", Member::Kind::Constant, true, true, true, false},
        {"state", Member::Kind::State, true, true, true, false},    {"update", Member::Kind::Update, true, false, false, true},
        {"let", Member::Kind::Let, true, false, false, true},       {"yield", Member::Kind::Yield, false, false, false, true},
    };
    for (const auto& f : forms)
      if (key == f.keyword) return &f;
    return nullptr;
  }

  void tensor_type(Member& m) {
    expect(":");
    expect_ident("tensor");
    expect("<");
    expect_ident("f32");
    expect(">");
    literal_list("shape", [&](const std::string& text, size_t i) {
      size_t v = 0;
      for (char c : text) {
        if (c < '0' || c > '9') err("shape: dimension " + std::to_string(i) + " ('" + text + "') is not a positive integer");
        if (v > (SIZE_MAX - 9) / 10) err("shape: dimension " + std::to_string(i) + " overflows");
        v = v * 10 + (size_t)(c - '0');
      }
      if (v == 0) err("shape: dimension " + std::to_string(i) + " is zero");
      m.dims.push_back(v);
    });
  }

  void initialiser(Member& m) {
    size_t want = 1;
    for (size_t d : m.dims) want *= d;
    const size_t got = literal_list("initializer", [&](const std::string& text, size_t i) {
      char* end = nullptr;
      const float f = strtof(text.c_str(), &end);
      if (end == text.c_str() || *end) err("initializer: entry " + std::to_string(i) + " ('" + text + "') is not a float");
      m.values.push_back(f);
    });
    if (got != want)
      err("initializer of " + m.name + " has " + std::to_string(got) + " values, its shape holds " + std::to_string(want));
  }

  std::vector<Member> members(bool graph_allowed, size_t depth) {
    if (depth > kMaxNesting) fail(ErrorKind::Capacity, "declaration nesting limit (64)");
    expect("{");
    std::vector<Member> out;
    for (; !is("}"); expect(";"), out.back().end = t_[p_ - 1].end) {
      if (peek().kind == Token::Kind::End) err("unclosed declaration");
      Member& m = out.emplace_back();
      m.start = peek().start;
      const std::string key = ident();
      const DeclForm* form = graph_allowed ? decl_form(key) : nullptr;
      if (!form) {                       // `name = expr`: a field of a record / weights scope
        m.kind = Member::Kind::Field;
        m.name = key;
        expect("=");
        m.expr = expr(depth + 1);
        continue;
      }
      m.kind = form->kind;
      if (form->named) m.name = ident();
      if (form->kind == Member::Kind::Let && m.name.find('.') != std::string::npos) err("binding name cannot contain '.'");
      if (form->typed) tensor_type(m);
      if (form->initialised || (form->valued && form->named)) expect("=");
      if (form->initialised) initialiser(m);
      if (form->valued) m.expr = expr(depth + 1);
    }
    expect("}");
    return out;
  }

  ExprPtr expr(size_t depth) {
    if (depth > kMaxNesting) fail(ErrorKind::Capacity, "expression nesting limit (64)");
    auto e = std::make_shared<Expr>();
    e->pos = peek().start;
    const Token& t = peek();
    if (t.kind == Token::Kind::String) { e->kind = Expr::Kind::String; e->text = t.text; ++p_; return e; }
    if (t.kind == Token::Kind::Number) { e->kind = Expr::Kind::Number; e->text = t.text; ++p_; return e; }
    if (is("[")) {
      ++p_;
      e->kind = Expr::Kind::List;
      while (!is("]")) {
        e->args.emplace_back("", expr(depth + 1));
        if (!is(",")) break;
        ++p_;
      }
      expect("]");
      return e;
    }
    if (t.kind != Token::Kind::Ident) err("expected expression");
    if (t.text == "fold") {
      ++p_;
      e->kind = Expr::Kind::Fold;
      e->index = ident();
      expect_ident("in");
      expect_ident("range");
      expect("(");
      e->start = expr(depth + 1);
      expect(",");
      e->end = expr(depth + 1);
      expect(")");
      expect_ident("carry");
      expect("(");
      e->carry = ident();
      expect("=");
      e->initial = expr(depth + 1);
      expect(")");
      e->body = members(true, depth + 1);
      return e;
    }
    e->text = ident();
    if (is("(")) {
      ++p_;
      e->kind = Expr::Kind::Call;
      while (!is(")")) {
        std::string key;
        if (peek().kind == Token::Kind::Ident && peek(1).kind == Token::Kind::Punct && peek(1).text == "=") {
          key = ident();
          ++p_;
        }
        e->args.emplace_back(key, expr(depth + 1));
        if (!is(",")) break;
        ++p_;
      }
      expect(")");
      return e;
    }
    e->kind = Expr::Kind::Name;
    return e;
  }

  std::vector<Token> t_;
  size_t p_ = 0;
};

// ---------------------------------------------------------------------------------------------
// Expansion
// ---------------------------------------------------------------------------------------------
struct Value {
  enum class Kind { Tensor, Number, String, Bool, Scope, Record, List };
  Kind kind = Kind::Number;
  std::string text;                        // node name / literal / scope path
  std::map<std::string, Value> fields;     // Record
  std::vector<Value> items;                // List
};
using Env = std::map<std::string, Value>;

const std::set<std::string> kStatic = {"weights", "child", "choose", "div", "mod", "eq", "lt", "record"};

std::string render(const Value& v) {
  switch (v.kind) {
    case Value::Kind::List: {
      std::string s = "[";
      for (size_t i = 0; i < v.items.size(); ++i) s += (i ? "," : "") + render(v.items[i]);
      return s + "]";
    }
    default: return v.text;
  }
}

class Expander {
 public:
  explicit Expander(const Document& d) : doc_(d) {
    for (auto& m : d.modules) {
      if (primitives().count(m.name) || kStatic.count(m.name)) err_at(m.pos, "module name shadows a builtin: " + m.name);
      if (!modules_.emplace(m.name, &m).second) err_at(m.pos, "duplicate module " + m.name);
    }
  }

  Expanded run() {
    Expanded out;
    out.model_name = doc_.model_name;
    out.plan_name = doc_.plan_name;
    Env env;
    bool yielded = false;
    for (auto& m : doc_.model) {
      tick(m.start);
      switch (m.kind) {
        case Member::Kind::Field: out.fields[m.name] = render(literal(eval(*m.expr, env, "", m.name, m), m)); break;
        case Member::Kind::Let: bind(env, m.name, eval(*m.expr, env, "", m.name, m), m); break;
        case Member::Kind::Yield: {
          if (yielded) err_at(m.start, "model yields more than once");
          Value v = eval(*m.expr, env, "", "yield", m);
          if (v.kind != Value::Kind::Tensor) err_at(m.start, "model must yield a tensor");
          out.output = v.text;
          yielded = true;
          break;
        }
        case Member::Kind::Input:
        case Member::Kind::Constant:
        case Member::Kind::State: {
          FlatNode n;
          n.name = m.name;
          n.op = m.kind == Member::Kind::Input ? "input" : m.kind == Member::Kind::Constant ? "const" : "state";
          std::string dims = "[";
          for (size_t i = 0; i < m.dims.size(); ++i) dims += (i ? "," : "") + std::to_string(m.dims[i]);
          n.attrs.emplace_back("shape", dims + "]");
          if (m.kind != Member::Kind::Input) {
            std::string vals = "[";
            for (size_t i = 0; i < m.values.size(); ++i) vals += (i ? "," : "") + format_double(m.values[i]);
            n.attrs.emplace_back("data", vals + "]");
          }
          n.byte = m.start;
          emit(std::move(n), m);
          Value v;
          v.kind = Value::Kind::Tensor;
          v.text = m.name;
          bind(env, m.name, v, m);
          break;
        }
        case Member::Kind::Update: {
          Value v = eval(*m.expr, env, "", m.name, m);
          if (v.kind != Value::Kind::Tensor) err_at(m.start, "update needs a tensor value");
          if (!env.count(m.name)) err_at(m.start, "update of unknown state " + m.name);
          out.fields["update." + m.name] = v.text;
          break;
        }
      }
    }
    if (!yielded) invalid("model does not yield an output");
    for (auto& m : doc_.plan) {
      if (m.kind != Member::Kind::Field) err_at(m.start, "plan blocks hold `key = value;` fields only");
      if (out.plan.count(m.name)) err_at(m.start, "duplicate plan field " + m.name);
      out.plan[m.name] = render_expr(*m.expr);
    }
    out.nodes = std::move(nodes_);
    out.steps = steps_;
    return out;
  }

 private:
  void tick(size_t byte) {
    if (++steps_ > kMaxSteps) fail(ErrorKind::Capacity, "byte " + std::to_string(byte) + ": compile-time expansion work limit (100000 steps)");
  }
  static void bind(Env& env, const std::string& name, Value v, const Member& site) {
    if (env.count(name)) err_at(site.start, "duplicate binding " + name);
    env[name] = std::move(v);
  }
  static Value literal(Value v, const Member& site) {
    if (v.kind == Value::Kind::Tensor || v.kind == Value::Kind::Record) err_at(site.start, "tensor supplied where a compile-time attribute is required");
    return v;
  }
  static long long integer(const Value& v, const Member& site) {
    if (v.kind != Value::Kind::Number) err_at(site.start, "expected compile-time integer");
    char* end = nullptr;
    long long x = strtoll(v.text.c_str(), &end, 10);
    if (!end || *end || x < 0) err_at(site.start, "expected nonnegative compile-time integer");
    return x;
  }
  static Value number(long long x) {
    Value v;
    v.kind = Value::Kind::Number;
    v.text = std::to_string(x);
    return v;
  }
  static Value boolean(bool b) {
    Value v;
    v.kind = Value::Kind::Bool;
    v.text = b ? "true" : "false";
    return v;
  }
  static std::string scoped(const std::string& base, const std::string& comp, const Member& site) {
    if (comp.empty()) err_at(site.start, "invalid weight scope component");
    size_t b = 0;
    while (b <= comp.size()) {
      size_t e = comp.find('.', b);
      if (e == std::string::npos) e = comp.size();
      std::string part = comp.substr(b, e - b);
      bool ok = !part.empty() && (part == "{expert}" || std::all_of(part.begin(), part.end(), [](unsigned char c) { return isalnum(c) || c == '_'; }));
      if (!ok) err_at(site.start, "invalid weight scope component '" + comp + "'");
      b = e + 1;
    }
    std::string path = base.empty() ? comp : base + "." + comp;
    if (path.size() > 1024) fail(ErrorKind::Capacity, "weight path longer than 1024 bytes");
    return path;
  }
  static std::string render_expr(const Expr& e) {
    switch (e.kind) {
      case Expr::Kind::Name:
      case Expr::Kind::Number:
      case Expr::Kind::String: return e.text;
      case Expr::Kind::List: {
        std::string s = "[";
        for (size_t i = 0; i < e.args.size(); ++i) s += (i ? "," : "") + render_expr(*e.args[i].second);
        return s + "]";
      }
      case Expr::Kind::Call: {
        std::string s = e.text + "(";
        for (size_t i = 0; i < e.args.size(); ++i) s += (i ? "," : "") + (e.args[i].first.empty() ? "" : e.args[i].first + "=") + render_expr(*e.args[i].second);
        return s + ")";
      }
      case Expr::Kind::Fold: err_at(e.pos, "fold is not allowed here");
    }
    return "";
  }

  Value resolve(const std::string& name, const Env& env, const Member& site) {
    auto it = env.find(name);
    if (it != env.end()) return it->second;
    size_t dot = name.find('.');
    if (dot != std::string::npos) {
      auto root = env.find(name.substr(0, dot));
      if (root != env.end()) {
        std::string tail = name.substr(dot + 1);
        if (root->second.kind == Value::Kind::Scope) {
          Value v;
          v.kind = Value::Kind::Scope;
          v.text = scoped(root->second.text, tail, site);
          return v;
        }
        const Value* cur = &root->second;
        size_t b = 0;
        while (b <= tail.size()) {
          size_t e = tail.find('.', b);
          if (e == std::string::npos) e = tail.size();
          std::string field = tail.substr(b, e - b);
          if (cur->kind != Value::Kind::Record) err_at(site.start, "field access requires a record");
          auto f = cur->fields.find(field);
          if (f == cur->fields.end()) err_at(site.start, "unknown record field " + field);
          cur = &f->second;
          b = e + 1;
        }
        return *cur;
      }
    }
    if (name == "true" || name == "false") return boolean(name == "true");
    // bare identifiers in attribute position (e.g. target names, dtypes) are not allowed inside graphs:
    err_at(site.start, "unknown binding " + name);
  }

  std::string unique(const std::string& want) {
    std::string n = want;
    for (int k = 2; !names_.insert(n).second; ++k) n = want + "~" + std::to_string(k);
    return n;
  }
  void emit(FlatNode n, const Member& site) {
    if (nodes_.size() >= kMaxNodes) fail(ErrorKind::Capacity, "byte " + std::to_string(site.start) + ": expanded graph exceeds 10000 nodes");
    n.frames = frames_;
    names_.insert(n.name);
    nodes_.push_back(std::move(n));
  }

  // `prefix` is the instance path of the enclosing module/fold; `hint` names the value being bound.
  Value eval(const Expr& e, const Env& env, const std::string& prefix, const std::string& hint, const Member& site) {
    tick(e.pos);
    switch (e.kind) {
      case Expr::Kind::Number: { Value v; v.kind = Value::Kind::Number; v.text = e.text; return v; }
      case Expr::Kind::String: { Value v; v.kind = Value::Kind::String; v.text = e.text; return v; }
      case Expr::Kind::Name: return resolve(e.text, env, site);
      case Expr::Kind::List: {
        Value v;
        v.kind = Value::Kind::List;
        for (auto& a : e.args) v.items.push_back(literal(eval(*a.second, env, prefix, hint, site), site));
        return v;
      }
      case Expr::Kind::Fold: return fold(e, env, prefix, hint, site);
      case Expr::Kind::Call: break;
    }
    const std::string& f = e.text;
    if (kStatic.count(f)) return builtin(e, env, prefix, hint, site);
    auto mod = modules_.find(f);
    if (mod != modules_.end()) return call_module(*mod->second, e, env, prefix, hint, site);
    if (!primitives().count(f)) err_at(e.pos, "unknown function or module " + f);
    FlatNode n;
    n.op = f;
    n.byte = site.start;
    int anon = 0;
    for (auto& a : e.args) {
      if (a.first.empty()) {
        Value v = eval(*a.second, env, prefix, hint + "." + std::to_string(anon++), site);
        if (v.kind != Value::Kind::Tensor) err_at(a.second->pos, "expected tensor/graph handle as positional argument of " + f);
        n.inputs.push_back(v.text);
      } else {
        // an attribute value that is a bare word no binding claims (a dtype, a cache layout, a selection mode) is the
        // word itself; the checker decides whether the operator knows it
        const Expr& ae = *a.second;
        Value v;
        if (ae.kind == Expr::Kind::Name && !env.count(ae.text) && ae.text.find('.') == std::string::npos &&
            ae.text != "true" && ae.text != "false") {
          tick(ae.pos);
          v.kind = Value::Kind::String;
          v.text = ae.text;
        } else {
          v = literal(eval(ae, env, prefix, hint, site), site);
        }
        for (auto& kv : n.attrs)
          if (kv.first == a.first) err_at(a.second->pos, "duplicate attribute " + a.first);
        n.attrs.emplace_back(a.first, render(v));
      }
    }
    std::sort(n.attrs.begin(), n.attrs.end());
    n.name = unique(prefix.empty() ? hint : prefix + "/" + hint);
    Value out;
    out.kind = Value::Kind::Tensor;
    out.text = n.name;
    emit(std::move(n), site);
    return out;
  }

  Value builtin(const Expr& e, const Env& env, const std::string& prefix, const std::string& hint, const Member& site) {
    const std::string& f = e.text;
    auto positional = [&](size_t n) {
      if (e.args.size() != n) err_at(e.pos, f + " takes " + std::to_string(n) + " argument(s)");
      for (auto& a : e.args)
        if (!a.first.empty()) err_at(e.pos, f + " takes positional arguments");
    };
    if (f == "weights") {
      positional(1);
      Value v = eval(*e.args[0].second, env, prefix, hint, site);
      if (v.kind != Value::Kind::String) err_at(e.pos, "weights(\"root\") needs a string");
      Value s;
      s.kind = Value::Kind::Scope;
      s.text = scoped("", v.text, site);
      return s;
    }
    if (f == "child") {
      positional(2);
      Value base = eval(*e.args[0].second, env, prefix, hint, site);
      if (base.kind != Value::Kind::Scope) err_at(e.pos, "child() needs a weight scope");
      Value c = eval(*e.args[1].second, env, prefix, hint, site);
      if (c.kind != Value::Kind::Number && c.kind != Value::Kind::String) err_at(e.pos, "child() component must be an integer or a string");
      if (c.kind == Value::Kind::Number) (void)integer(c, site);
      Value s;
      s.kind = Value::Kind::Scope;
      s.text = scoped(base.text, c.text, site);
      return s;
    }
    if (f == "choose") {
      positional(3);
      Value c = eval(*e.args[0].second, env, prefix, hint, site);
      if (c.kind != Value::Kind::Bool) err_at(e.pos, "choose() condition must be a compile-time boolean");
      return eval(*e.args[c.text == "true" ? 1 : 2].second, env, prefix, hint, site);  // the other branch is never expanded
    }
    if (f == "div" || f == "mod" || f == "eq" || f == "lt") {
      positional(2);
      long long a = integer(eval(*e.args[0].second, env, prefix, hint, site), site);
      long long b = integer(eval(*e.args[1].second, env, prefix, hint, site), site);
      if ((f == "div" || f == "mod") && b == 0) err_at(e.pos, "division by zero");
      if (f == "div") return number(a / b);
      if (f == "mod") return number(a % b);
      if (f == "eq") return boolean(a == b);
      return boolean(a < b);
    }
    // record(name = value, ...)
    if (e.args.empty() || e.args.size() > kMaxRecordFields) err_at(e.pos, "record() takes 1..64 named fields");
    Value r;
    r.kind = Value::Kind::Record;
    for (auto& a : e.args) {
      if (a.first.empty()) err_at(e.pos, "record() fields must be named");
      Value v = eval(*a.second, env, prefix, hint + "." + a.first, site);
      if (v.kind != Value::Kind::Tensor && v.kind != Value::Kind::Record) err_at(a.second->pos, "record fields hold graph handles");
      if (!r.fields.emplace(a.first, std::move(v)).second) err_at(e.pos, "duplicate record field " + a.first);
    }
    return r;
  }

  Value run_body(const std::vector<Member>& body, Env env, const std::string& prefix, const Member& outer) {
    std::optional<Value> result;
    for (auto& m : body) {
      tick(m.start);
      switch (m.kind) {
        case Member::Kind::Let: bind(env, m.name, eval(*m.expr, env, prefix, m.name, m), m); break;
        case Member::Kind::Yield:
          if (result) err_at(m.start, "body yields more than once");
          result = eval(*m.expr, env, prefix, "yield", m);
          break;
        default: err_at(m.start, "only let/yield are allowed inside modules and folds");
      }
    }
    if (!result) err_at(outer.start, "body does not yield a value");
    return *result;
  }

  Value call_module(const Module& mod, const Expr& e, const Env& env, const std::string& prefix, const std::string& hint, const Member& site) {
    if (std::find(stack_.begin(), stack_.end(), mod.name) != stack_.end()) err_at(e.pos, "recursive module call: " + mod.name);
    if (stack_.size() >= kMaxNesting) fail(ErrorKind::Capacity, "module call depth limit (64)");
    Env inner;
    size_t next = 0;
    for (auto& a : e.args) {
      std::string target;
      if (a.first.empty()) {
        if (next >= mod.params.size()) err_at(e.pos, "too many arguments for module " + mod.name);
        target = mod.params[next++];
      } else {
        if (std::find(mod.params.begin(), mod.params.end(), a.first) == mod.params.end()) err_at(e.pos, "module " + mod.name + " has no parameter " + a.first);
        target = a.first;
      }
      if (inner.count(target)) err_at(e.pos, "parameter " + target + " bound twice");
      inner[target] = eval(*a.second, env, prefix, hint + "." + target, site);
    }
    for (auto& p : mod.params)
      if (!inner.count(p)) err_at(e.pos, "missing argument " + p + " for module " + mod.name);
    stack_.push_back(mod.name);
    frames_.push_back({"module " + mod.name, e.pos});
    Value v = run_body(mod.body, std::move(inner), prefix.empty() ? hint : prefix + "/" + hint, site);
    frames_.pop_back();
    stack_.pop_back();
    return v;
  }

  Value fold(const Expr& e, const Env& env, const std::string& prefix, const std::string& hint, const Member& site) {
    long long a = integer(eval(*e.start, env, prefix, hint, site), site);
    long long b = integer(eval(*e.end, env, prefix, hint, site), site);
    if (b < a) err_at(e.pos, "fold range end before start");
    if ((size_t)(b - a) > kMaxFold) fail(ErrorKind::Capacity, "fold longer than 4096 iterations");
    Value carry = eval(*e.initial, env, prefix, hint + ".init", site);
    if (carry.kind != Value::Kind::Tensor && carry.kind != Value::Kind::Record) err_at(e.pos, "fold carry must be a graph handle or a record of handles");
    const std::string shape0 = shape_of(carry);
    for (long long i = a; i < b; ++i) {
      Env inner = env;
      inner[e.index] = number(i);
      inner[e.carry] = carry;
      frames_.push_back({"fold " + e.index + "=" + std::to_string(i), e.pos});
      carry = run_body(e.body, std::move(inner), (prefix.empty() ? hint : prefix + "/" + hint) + "[" + std::to_string(i) + "]", site);
      frames_.pop_back();
      if (shape_of(carry) != shape0) err_at(e.pos, "fold body changes the structure of the carried value");
    }
    return carry;
  }
  static std::string shape_of(const Value& v) {
    if (v.kind == Value::Kind::Tensor) return "h";
    if (v.kind != Value::Kind::Record) return "?";
    std::string s = "{";
    for (auto& kv : v.fields) s += kv.first + ":" + shape_of(kv.second) + ";";
    return s + "}";
  }

  const Document& doc_;
  std::map<std::string, const Module*> modules_;
  std::vector<FlatNode> nodes_;
  std::set<std::string> names_;
  std::vector<std::string> stack_;
  std::vector<Frame> frames_;
  size_t steps_ = 0;
};

}  // namespace

const std::set<std::string>& primitives() {
  static const std::set<std::string> p = {
      // token-program primitives
      "embedding", "cast", "quantize", "repeat", "mhc_pre", "mhc_merge", "mhc_input", "mhc_post", "norm", "optional_norm",
      "linear", "gather", "allreduce", "mome", "slice", "rope", "rotary_prefix", "concat", "mla_query", "mla_value",
      "sink_normalize", "cache_append", "cache_norm_rope_append", "latent_attention", "index_cache_append", "sparse_index",
      "swiglu", "router", "expert_linear", "expert_swiglu_down", "expert_reduce", "add",
      // dense-attention family (GQA models)
      "kv_cache_append", "paged_attention",
      // cpu_f32_v1 graph ops
      "mul", "relu", "matmul"};
  return p;
}

Document parse(std::string_view source) { return Parser(lex(source)).document(); }
Expanded expand(const Document& doc) { return Expander(doc).run(); }

}  // namespace ifab::lang
