// The `.inferfabric` model language, version 1: lexer, parser and compile-time expander.
//
// Surface (same as the reference front end, crates/inferfabric-dsl/src/syntax.rs:332-390 and
// expand.rs:160-575):
//   language inferfabric 1;
//   module Name(p, q) { let a = op(p, attr = 1); yield a; }
//   model M { context = 512; eos = 7; let w = weights("model"); let h = fold i in range(0, 46)
//             carry(x = e) { let y = Block(x, child(w.layers, i), i); yield y; }; yield logits; }
//   plan P for M { target = b200_token_v1; tp = 8; ep = 8; devices = [0,1,2,3,4,5,6,7]; ... }
//
// Expansion evaluates folds, `choose`, `div/mod/eq/lt`, `record`, `weights`/`child` scopes and
// module calls at compile time and leaves a flat list of primitive nodes with hygienic instance
// paths and source origins. Limits: 1 MiB source, 100,000 tokens, 256 modules, nesting 64,
// 4,096 fold iterations, 10,000 nodes, 100,000 evaluation steps; recursion is rejected.
#pragma once
#include <map>
#include <memory>
#include <set>

#include "base.h"

namespace ifab::lang {

struct Member;
struct Expr {
  enum class Kind { Name, String, Number, List, Call, Fold };
  Kind kind = Kind::Name;
  std::string text;                                            // name / string body / number literal / callee
  std::vector<std::pair<std::string, std::shared_ptr<Expr>>> args;  // call arguments ("" = positional) / list items
  // fold
  std::string index, carry;
  std::shared_ptr<Expr> start, end, initial;
  std::vector<Member> body;
  size_t pos = 0;
};
using ExprPtr = std::shared_ptr<Expr>;

struct Member {
  enum class Kind { Field, Input, Constant, State, Let, Yield, Update };
  Kind kind = Kind::Field;
  std::string name;            // bound name (Field/Let/Input/Constant/State/Update target)
  ExprPtr expr;                // Field/Let/Yield/Update value
  std::vector<size_t> dims;    // Input/Constant/State
  std::vector<float> values;   // Constant/State
  size_t start = 0, end = 0;
};

struct Module {
  std::string name;
  std::vector<std::string> params;
  std::vector<Member> body;
  size_t pos = 0;
};

struct Document {
  std::vector<Module> modules;
  std::string model_name;
  std::vector<Member> model;
  std::string plan_name, plan_model;
  std::vector<Member> plan;
};

Document parse(std::string_view source);

// ---- expansion -------------------------------------------------------------------------------
struct Frame {            // one step of the expansion stack that produced a node
  std::string what;       // "module Name" / "fold i=3"
  size_t byte = 0;
};
struct FlatNode {
  std::string name;                                   // unique instance path
  std::string op;                                     // primitive
  std::vector<std::string> inputs;                    // names of earlier nodes
  std::vector<std::pair<std::string, std::string>> attrs;  // attribute literals (sorted by key)
  size_t byte = 0;                                    // source byte of the defining member
  std::vector<Frame> frames;
};
struct Expanded {
  std::vector<FlatNode> nodes;
  std::string output;                                 // node yielded by the model
  std::map<std::string, std::string> fields;          // model-level `key = literal;` fields
  std::map<std::string, std::string> plan;            // plan-level fields (lists rendered as "[a,b]")
  std::string model_name, plan_name;
  size_t steps = 0;
};

// Set of primitive op names the expander passes through as graph nodes.
const std::set<std::string>& primitives();
Expanded expand(const Document& doc);

}  // namespace ifab::lang
