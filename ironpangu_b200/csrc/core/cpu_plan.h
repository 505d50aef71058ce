// CPU physical planner, verifier and executor for static f32 graphs (target cpu_f32_v1).
//
// Pipeline: logical graph -> typed (topological order, shape inference) -> dead-code elimination ->
// constant folding (bounded work) -> value compaction -> lifetime intervals -> first-fit arena
// offsets (64-byte lines) -> reuse dependencies -> kernel selection with a recorded reason.
// The verifier re-derives aliasing / lifetime / bounds facts from the finished plan alone.
// Reference: crates/inferfabric-plan/src/{ir,planner,verify,execute,binary}.rs.
#pragma once
#include <functional>

#include "base.h"
#include "lang.h"

namespace ifab::cpu {

enum class Op { Add, Mul, Relu, Matmul };
const char* op_name(Op op);

struct TensorDecl { std::string name; std::vector<size_t> shape; };
struct ConstantDecl { std::string name; std::vector<size_t> shape; std::vector<float> data; };
struct LogicalNode { std::string name; Op op; std::vector<std::string> inputs; };

struct LogicalGraph {
  uint32_t version = 1;
  std::string name;
  std::vector<TensorDecl> inputs;
  std::vector<ConstantDecl> constants, states;
  std::vector<LogicalNode> nodes;
  std::vector<std::string> outputs;
  std::map<std::string, std::string> updates;   // state <- node, committed together after a run
  static LogicalGraph from_json(const Json& j);
  Json to_json() const;
};
// cpu_f32_v1 model written in the DSL (input / const / state / update members, ops add mul relu matmul).
LogicalGraph from_dsl(std::string_view source);
LogicalGraph from_expanded(const lang::Expanded& ex);

enum class Storage { Input, Constant, State, Temporary };
enum class Kernel { AddF32V1, MulF32V1, ReluF32V1, MatmulNaiveF32V1, MatmulBlockedF32V1 };
const char* kernel_name(Kernel k);
Op kernel_op(Kernel k);

struct Buffer {
  std::string name;
  std::vector<size_t> shape;
  Storage storage = Storage::Temporary;
  std::vector<float> initial;          // constants / states
  bool has_offset = false;
  size_t offset = 0;                   // byte offset in the arena (temporaries only)
  bool has_lifetime = false;
  size_t first = 0, last = 0;          // step interval
  size_t elements() const;
  size_t bytes() const { return elements() * 4; }
};
struct Step {
  std::string name;
  Kernel kernel;
  std::vector<size_t> inputs;
  size_t output = 0;
  size_t rank = 0, stream = 0;
  std::vector<size_t> dependencies;        // producers of the inputs
  std::vector<size_t> reuse_dependencies;  // last readers of the bytes this step overwrites
  std::string selection_reason;
};
struct PhysicalPlan {
  uint32_t version = 1;
  std::string name, target = "cpu_f32_v1", policy = "first_fit_64";
  std::vector<Buffer> buffers;
  std::vector<Step> steps;
  std::vector<size_t> outputs;
  std::map<size_t, size_t> updates;        // state buffer <- value buffer
  size_t arena_bytes = 0;
  size_t folded_constants = 0, eliminated_nodes = 0;
  Json to_json() const;
  static PhysicalPlan from_json(const Json& j);
};

struct Options {
  bool debug_names = false;                         // keep eliminated nodes' names in the report
  std::map<std::string, Kernel> override_kernels;   // node name -> forced kernel (must implement the node's op)
  size_t fold_work_limit = 4096;
};
// What the pipeline looked like between its passes, for `plan --dump-ir`: the typed graph (every value with its inferred
// shape) and the optimised graph (dead nodes gone, constants folded), each as JSON.
struct Stages {
  Json typed, optimized;
};
PhysicalPlan compile(const LogicalGraph& g, const Options& opt = {}, Stages* stages = nullptr);
// A plan with some steps' kernels replaced: `overrides` maps step names to kernel names; a kernel must implement the step's
// operation and exist; offsets, lifetimes and dependencies are kept and the result is verified. (Reference: override_kernels
// behind `tune-plan`, crates/inferfabric-cli/src/physical.rs:70-76.)
PhysicalPlan tune(const PhysicalPlan& plan, const std::map<std::string, std::string>& overrides);
// A self-contained HTML page of a plan: steps with kernels and reasons, buffers with arena offsets and lifetimes.
std::string html_view(const PhysicalPlan& plan);
void verify(const PhysicalPlan& p);   // throws Error(Invalid) naming the violated rule

std::string encode_plan(const PhysicalPlan& p);      // IFPLAN01: magic, u64 length, sha256, JSON
PhysicalPlan decode_plan(std::string_view bytes);
Json manifest(std::string_view bytes);               // header facts without decoding the body

struct RunReport {
  std::map<std::string, std::vector<float>> outputs;
  size_t steps = 0, arena_bytes = 0;
  std::vector<std::string> kernels;
  Json to_json() const;
};
using CompiledKernel = std::function<void(const std::vector<const float*>& inputs, const std::vector<std::vector<size_t>>& shapes, float* out)>;
class Executor {
 public:
  explicit Executor(PhysicalPlan plan);
  void bind(const std::string& step_name, CompiledKernel k);   // override one step with a bound kernel
  RunReport run(const std::map<std::string, std::vector<float>>& inputs);
  const std::vector<float>& state(const std::string& name) const;

 private:
  PhysicalPlan plan_;
  std::vector<float> arena_;                       // 64-byte lines, sized arena_bytes
  std::map<size_t, std::vector<float>> resident_;  // constants and states
  std::map<std::string, CompiledKernel> bound_;
};

}  // namespace ifab::cpu
