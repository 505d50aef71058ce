// `ifab` command line: offline compiler, inspectors and the CPU oracle.
//
//   ifab compile-token MODEL.inferfabric CHECKPOINT|- OUTPUT_DIR [--resident-sequences N]
//        [--prefill-tokens N | --prefill-variants 2,4,8] [--uncaptured-prefill] [--shared-pages]
//        [--output-rows] [--bulk-collectives] [--kernel-dir DIR]
//   ifab explain MODEL.inferfabric            graph / program summary as JSON
//   ifab model-source MODEL.inferfabric       expanded primitive list (one node per line)
//   ifab synth-checkpoint MODEL.inferfabric OUT_DIR [--seed N]   random N(0,0.02) safetensors for the model
//   ifab interpret MODEL.inferfabric CHECKPOINT_DIR NEW_TOKENS TOKEN_ID...   greedy decode on the CPU oracle
//   ifab inspect FILE                         decode execution.bin / logical.bin / rank-N.bin / arena-rank-N.txt
//   ifab plan|execute|explain-plan ...        CPU f32 graph planner (see cpu_plan.h)
//   ifab compile SPEC.json OUT.bin            structural rank plans for TP/SP/CP/PD meshes
//   ifab demo                                 compile + run the built-in two-layer slice
//
// Verbs follow the reference CLI (crates/inferfabric-cli/src/main.rs:17-293).
#include <cstdio>
#include <cstring>
#include <iostream>

#include <sys/stat.h>

#include "config_audit.h"
#include "contract.h"
#include "bundle.h"
#include "cpu_plan.h"
#include "definition.h"
#include "hybrid.h"
#include "interp.h"
#include "rankplan.h"
#include "tokenizer.h"

using namespace ifab;

namespace {

int usage() {
  std::fprintf(stderr,
               "usage: ifab <command> ...\n"
               "  compile-token MODEL CHECKPOINT|- OUTPUT_DIR [flags]\n  explain MODEL\n  model-source MODEL\n"
               "  synth-checkpoint MODEL OUT_DIR [--seed N]\n  interpret MODEL CHECKPOINT_DIR NEW_TOKENS TOKEN...\n"
               "  validate-bundle BUNDLE_DIR\n  inspect-config CONFIG.json [OUT.json]\n  inspect-checkpoint DIR [OUT.json]\n  bind-checkpoint MODEL DIR [OUT.json]\n  plan-placement MODEL [DIR|-] [OUT.json]\n"
               "  inspect FILE\n  plan|plan-debug GRAPH.json|MODEL.inferfabric [OUT.ifplan] [--dump-ir DIR]\n  tune-plan PLAN.ifplan OVERRIDES.json OUT.ifplan\n"
               "  explain-plan PLAN.ifplan|GRAPH [--html OUT.html]\n  explain-model TYPED-PLAN.json --html OUT.html\n  execute GRAPH.json|MODEL.inferfabric INPUTS.json\n"
               "  compile SPEC.json|MODEL.inferfabric OUT.bin\n  compile-model MODEL.inferfabric|MODEL.json [OUT.json]\n"
               "  tokenize TOKENIZER TEXT_FILE\n  detokenize TOKENIZER IDS.json\n  render-chat TOKENIZER MESSAGES.json [auto|chatml|plain]\n"
               "  inspect-hybrid-checkpoint MODEL DIR [OUT.json]\n  compile-checkpoint MODEL DIR [OUT.json]\n  lower-checkpoint MODEL DIR CONTEXT [BATCH] [OUT.json]\n  demo\n");
  return 2;
}

std::vector<uint32_t> parse_list(const std::string& s) {
  std::vector<uint32_t> v;
  size_t b = 0;
  while (b < s.size()) {
    size_t e = s.find(',', b);
    if (e == std::string::npos) e = s.size();
    v.push_back((uint32_t)std::stoul(s.substr(b, e - b)));
    b = e + 1;
  }
  return v;
}

int compile_token(int argc, char** argv) {
  if (argc < 5) return usage();
  bundle::BundleInputs in;
  in.source_path = argv[2];
  in.source_text = read_file(argv[2], 1 << 20);
  in.checkpoint_dir = std::string(argv[3]) == "-" ? "" : argv[3];
  std::string out = argv[4];
  bool tokens_set = false, variants_set = false;
  for (int i = 5; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> std::string {
      if (i + 1 >= argc) invalid("flag " + a + " needs a value");
      return argv[++i];
    };
    if (a == "--resident-sequences") in.options.resident_sequences = (uint32_t)std::stoul(next());
    else if (a == "--prefill-tokens") { in.options.prefill_tokens = (uint32_t)std::stoul(next()); tokens_set = true; }
    else if (a == "--prefill-variants") { in.options.prefill_variants = parse_list(next()); variants_set = true; }
    else if (a == "--uncaptured-prefill") in.options.uncaptured_prefill = true;
    else if (a == "--shared-pages") in.options.shared_pages = true;
    else if (a == "--output-rows") in.options.output_rows = true;
    else if (a == "--bulk-collectives") in.options.bulk_collectives = true;
    else if (a == "--allow-stale-index-size") in.allow_stale_index_size = true;
    else if (a == "--kernel-dir") in.kernel_source_dir = next();
    else invalid("unknown flag " + a);
  }
  if (tokens_set && variants_set) invalid("--prefill-tokens and --prefill-variants are exclusive");
  if (variants_set) in.options.prefill_tokens = in.options.prefill_variants.back();
  if (in.options.prefill_tokens >= 4096) in.options.uncaptured_prefill = true;  // the long-chunk envelope runs eagerly
  auto s = bundle::write_bundle(in, out);
  std::cout << s.to_json().dump(1) << "\n";
  return 0;
}

int explain(const char* path) {
  // a document or a model artifact of any kind: contracts and CPU graphs are summarised, token graphs also lowered
  definition::ModelDefinition def = definition::definition(read_file(path, definition::kMaxArtifactBytes));
  if (def.kind != definition::Kind::Execution) {
    Json j = Json::object();
    j.set("kind", definition::kind_name(def.kind));
    if (def.kind == definition::Kind::Qwen) {
      j.set("checkpoint", def.checkpoint);
      j.set("model", def.spec.model.name);
      size_t full = 0;
      for (auto l : def.spec.model.layers) full += l == rankplan::Layer::Full;
      j.set("layers", (int64_t)def.spec.model.layers.size());
      j.set("full_attention_layers", (int64_t)full);
      j.set("delta_layers", (int64_t)(def.spec.model.layers.size() - full));
      j.set("prefill_ranks", def.spec.prefill.ranks());
      j.set("decode_ranks", def.spec.decode.ranks());
      j.set("max_context", def.spec.max_context());
    } else if (def.kind == definition::Kind::OpenPangu) {
      j.set("parallel", def.parallel.to_json());
    } else {
      j.set("model", def.logical.name);
      j.set("nodes", (int64_t)def.logical.nodes.size());
      cpu::PhysicalPlan plan = cpu::compile(def.logical);
      j.set("steps", (int64_t)plan.steps.size());
      j.set("arena_bytes", (int64_t)plan.arena_bytes);
    }
    std::cout << j.dump(1) << "\n";
    return 0;
  }
  graph::Graph g = std::move(def.execution);
  program::Program p = program::lower(g);
  Json j = Json::object();
  j.set("model", g.name);
  j.set("logical_nodes", (int64_t)g.nodes.size());
  Json oh = Json::object();
  for (auto& kv : g.op_histogram()) oh.set(kv.first, (int64_t)kv.second);
  j.set("logical_ops", oh);
  j.set("instructions", (int64_t)p.instructions.size());
  Json ph = Json::object();
  for (auto& kv : p.op_histogram()) ph.set(kv.first, (int64_t)kv.second);
  j.set("physical_ops", ph);
  j.set("launches_per_token", (int64_t)p.launches_per_token());
  j.set("collectives_per_token", (int64_t)p.collectives_per_token());
  j.set("parallel", g.parallel.to_json());
  auto need = init::required_tensors(p);
  uint64_t bytes = 0;
  for (auto& kv : need) {
    uint64_t n = init::dtype_bytes(kv.second.first);
    for (auto d : kv.second.second) n *= d;
    bytes += n;
  }
  j.set("checkpoint_tensors", (int64_t)need.size());
  j.set("checkpoint_bytes", bytes);
  std::cout << j.dump(1) << "\n";
  return 0;
}

int interpret(int argc, char** argv) {
  if (argc < 6) return usage();
  graph::Graph g = graph::compile_source(read_file(argv[2], 1 << 20));
  interp::Weights w = interp::Weights::from_checkpoint(init::Checkpoint::inspect(argv[3]));
  interp::Interpreter it(g, w);
  uint32_t steps = (uint32_t)std::stoul(argv[4]);
  uint32_t next = 0, pos = 0;
  for (int i = 5; i < argc; ++i) next = it.step((uint32_t)std::stoul(argv[i]), pos++);
  Json gen = Json::array();
  for (uint32_t s = 0; s < steps; ++s) {
    gen.push((int64_t)next);
    if (next == g.eos) break;
    next = it.step(next, pos++);
  }
  Json j = Json::object();
  j.set("generated", gen);
  std::cout << j.dump() << "\n";
  return 0;
}

int inspect(const char* path) {
  std::string bytes = read_file(path);
  if (bytes.compare(0, 8, "IFTOKN01") == 0) std::cout << graph::Graph::decode(bytes).to_json().dump(1) << "\n";
  else if (bytes.compare(0, 7, "IFTOKN0") == 0) std::cout << program::Program::decode(bytes).to_json().dump(1) << "\n";
  else if (bytes.compare(0, 7, "IFINIT0") == 0) std::cout << init::Plan::decode(bytes).to_json().dump(1) << "\n";
  else if (bytes.compare(0, 7, "IFARENA") == 0) {
    uint64_t pf = 0, bf = 0;
    bundle::Arena a = bundle::Arena::decode(bytes, &pf, &bf);
    Json j = Json::object();
    j.set("bytes", a.bytes);
    j.set("slots", (int64_t)a.slots.size());
    j.set("tokens", a.tokens);
    j.set("program_fingerprint", hex64(pf));
    j.set("backend_fingerprint", hex64(bf));
    std::cout << j.dump(1) << "\n";
  } else if (bytes.compare(0, 8, "IFPLAN01") == 0) std::cout << cpu::decode_plan(bytes).to_json().dump(1) << "\n";
  else if (bytes.compare(0, 5, "PANGU") == 0) std::cout << rankplan::decode(bytes).to_json().dump(1) << "\n";
  else invalid("unrecognised file format");
  return 0;
}

// ---- checkpoint metadata verbs (no tensor data is read) ------------------------------------------------------------
uint64_t tensor_bytes(const init::TensorInfo& t) { return t.end - t.begin; }

void write_or_print(const Json& j, const char* out) {
  if (out) write_file_atomic(out, j.dump(1) + "\n");
  else std::cout << j.dump(1) << "\n";
}

// inspect-checkpoint DIR [OUT.json]: every tensor of every *.safetensors header, totals per dtype and per layer
int inspect_checkpoint(int argc, char** argv) {
  if (argc < 3) return usage();
  init::Checkpoint ck = init::Checkpoint::inspect(argv[2]);
  Json j = Json::object(), tensors = Json::array(), by_dtype = Json::object();
  std::map<std::string, uint64_t> dt_bytes, layer_bytes;
  uint64_t total = 0;
  for (auto& kv : ck.tensors) {
    const init::TensorInfo& t = kv.second;
    Json e = Json::object(), shape = Json::array();
    for (auto d : t.shape) shape.push((int64_t)d);
    e.set("name", t.name);
    e.set("dtype", init::dtype_name(t.dtype));
    e.set("shape", shape);
    e.set("bytes", tensor_bytes(t));
    e.set("file", t.file);
    tensors.push(e);
    dt_bytes[init::dtype_name(t.dtype)] += tensor_bytes(t);
    total += tensor_bytes(t);
    size_t at = t.name.find("layers.");
    if (at != std::string::npos) {
      size_t end = t.name.find('.', at + 7);
      layer_bytes[t.name.substr(at + 7, end == std::string::npos ? std::string::npos : end - at - 7)] += tensor_bytes(t);
    }
  }
  for (auto& kv : dt_bytes) by_dtype.set(kv.first, kv.second);
  j.set("directory", ck.dir);
  j.set("fingerprint", ck.fingerprint);
  j.set("tensors", (int64_t)ck.tensors.size());
  j.set("bytes", total);
  j.set("bytes_by_dtype", by_dtype);
  j.set("layers", (int64_t)layer_bytes.size());
  j.set("executable", false);
  j.set("tensor_list", tensors);
  // the directory's config.json, when it is of the audited family, is summarised beside the inventory
  {
    struct stat st {};
    const std::string cfg = std::string(argv[2]) + "/config.json";
    if (::stat(cfg.c_str(), &st) == 0) {
      try {
        j.set("config_audit", config_audit::audit(read_file(cfg, config_audit::kMaxConfigBytes)));
      } catch (const Error& e) {
        j.set("config_audit_error", std::string(e.what()));
      }
    }
  }
  write_or_print(j, argc > 3 ? argv[3] : nullptr);
  std::cerr << "checkpoint metadata audit: " << ck.tensors.size() << " tensors, " << layer_bytes.size() << " layers, " << total << " bytes\n";
  return 0;
}

// bind-checkpoint MODEL DIR [OUT.json]: which checkpoint tensor feeds which model parameter; shape / dtype agreement;
// tensors of the checkpoint the model does not use (multi-token-prediction heads and the like) are listed as excluded
int bind_checkpoint(int argc, char** argv) {
  if (argc < 4) return usage();
  graph::Graph g = graph::compile_source(read_file(argv[2], 1 << 20));
  program::Program p = program::lower(g);
  init::Checkpoint ck = init::Checkpoint::inspect(argv[3]);
  auto need = init::required_tensors(p);
  Json j = Json::object(), bound = Json::array(), missing = Json::array(), mismatched = Json::array(), excluded = Json::array();
  uint64_t bound_bytes = 0, excluded_bytes = 0;
  for (auto& kv : need) {
    if (!ck.has(kv.first)) { missing.push(kv.first); continue; }
    const init::TensorInfo& t = ck.need(kv.first);
    if (t.shape != kv.second.second) {
      Json e = Json::object(), want = Json::array(), got = Json::array();
      for (auto d : kv.second.second) want.push((int64_t)d);
      for (auto d : t.shape) got.push((int64_t)d);
      e.set("name", kv.first);
      e.set("model_shape", want);
      e.set("checkpoint_shape", got);
      mismatched.push(e);
      continue;
    }
    Json e = Json::object();
    e.set("name", kv.first);
    e.set("checkpoint_dtype", init::dtype_name(t.dtype));
    e.set("device_dtype", init::dtype_name(kv.second.first));
    e.set("bytes", tensor_bytes(t));
    e.set("file", t.file);
    bound.push(e);
    bound_bytes += tensor_bytes(t);
  }
  for (auto& kv : ck.tensors)
    if (!need.count(kv.first)) { excluded.push(kv.first); excluded_bytes += tensor_bytes(kv.second); }
  j.set("model", g.name);
  j.set("checkpoint_fingerprint", ck.fingerprint);
  j.set("bound", (int64_t)bound.size());
  j.set("bound_bytes", bound_bytes);
  j.set("excluded_bytes", excluded_bytes);
  j.set("complete", missing.size() == 0 && mismatched.size() == 0);
  j.set("bindings", bound);
  j.set("missing", missing);
  j.set("mismatched", mismatched);
  j.set("excluded", excluded);
  write_or_print(j, argc > 4 ? argv[4] : nullptr);
  std::cerr << "bound " << bound.size() << " tensors (" << bound_bytes << " bytes); missing " << missing.size() << ", mismatched "
            << mismatched.size() << ", excluded " << excluded_bytes << " bytes\n";
  return (missing.size() || mismatched.size()) ? 1 : 0;
}

// plan-placement MODEL [DIR] [OUT.json]: per-rank placement summary of the parallel plan (parameters, bytes, load slices);
// without a checkpoint directory the shapes come from the model alone
int plan_placement(int argc, char** argv) {
  if (argc < 3) return usage();
  graph::Graph g = graph::compile_source(read_file(argv[2], 1 << 20));
  program::Program p = program::lower(g);
  const bool have_dir = argc > 3 && std::string(argv[3]) != "-";
  init::Checkpoint ck = have_dir ? init::Checkpoint::inspect(argv[3]) : init::Checkpoint::synthetic(init::required_tensors(p));
  std::vector<init::Plan> plans = init::plan_all(p, ck);
  Json j = Json::object(), ranks = Json::array();
  for (auto& pl : plans) {
    Json r = Json::object();
    uint64_t strided = 0, src = 0;
    for (auto& l : pl.loads) { src += l.bytes; if (l.tag == 2) ++strided; }
    r.set("rank", (int64_t)pl.rank);
    r.set("parameters", (int64_t)pl.parameters.size());
    r.set("device_bytes", pl.device_bytes());
    r.set("load_slices", (int64_t)pl.loads.size());
    r.set("strided_slices", (int64_t)strided);
    r.set("source_bytes", src);
    ranks.push(r);
  }
  j.set("model", g.name);
  j.set("parallel", g.parallel.to_json());
  j.set("ranks", ranks);
  j.set("executable", have_dir);
  write_or_print(j, argc > 4 ? argv[4] : nullptr);
  return 0;
}

cpu::LogicalGraph load_cpu_graph(const std::string& path) {
  std::string text = read_file(path, 16 << 20);
  if (path.size() > 12 && path.compare(path.size() - 12, 12, ".inferfabric") == 0) return cpu::from_dsl(text);
  return cpu::LogicalGraph::from_json(Json::parse(text));
}

int demo() {
  const char* src = R"(language inferfabric 1;
model Residual { input x: tensor<f32>[2, 2]; const weight: tensor<f32>[2, 2] = [1, 0, 0, 1];
  let projected = matmul(x, weight); let summed = add(projected, x); let output = relu(summed); yield output; }
plan Cpu for Residual { target = cpu_f32_v1; })";
  cpu::LogicalGraph lg = cpu::from_dsl(src);
  cpu::PhysicalPlan plan = cpu::compile(lg);
  cpu::verify(plan);
  cpu::Executor ex(plan);
  auto rep = ex.run({{"x", {1, -2, 3, 4}}});
  std::cout << rep.to_json().dump(1) << "\n";
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return usage();
  std::string cmd = argv[1];
  try {
    if (cmd == "compile-token") return compile_token(argc, argv);
    if (cmd == "explain-model" && argc >= 5 && std::string(argv[3]) == "--html") {
      // explain-model TYPED-PLAN.json --html MODEL.html: the typed plan of the checkpoint-bound path as a page
      const Json doc = Json::parse(read_file(argv[2], 64 << 20));
      write_file_atomic(argv[4], hybrid::html_view(doc));
      std::cout << doc.at("spec").at("model").at("layers").size() << " layers, " << doc.at("nodes").size() << " operators, "
                << doc.at("checkpoint").at("weights").size() << " weights, " << doc.at("states").size() << " state tensors; " << argv[4] << "\n";
      return 0;
    }
    if (cmd == "explain" || cmd == "explain-model") return argc < 3 ? usage() : explain(argv[2]);
    if (cmd == "model-source") {
      if (argc < 3) return usage();
      auto ex = lang::expand(lang::parse(read_file(argv[2], 1 << 20)));
      for (auto& n : ex.nodes) {
        std::cout << n.name << " = " << n.op << "(";
        for (size_t i = 0; i < n.inputs.size(); ++i) std::cout << (i ? ", " : "") << n.inputs[i];
        for (auto& kv : n.attrs) std::cout << ", " << kv.first << "=" << kv.second;
        std::cout << ")\n";
      }
      return 0;
    }
    if (cmd == "synth-checkpoint") {
      if (argc < 4) return usage();
      uint64_t seed = 0;
      for (int i = 4; i + 1 < argc; ++i)
        if (std::string(argv[i]) == "--seed") seed = std::stoull(argv[i + 1]);
      graph::Graph g = graph::compile_source(read_file(argv[2], 1 << 20));
      program::Program p = program::lower(g);
      auto need = init::required_tensors(p);
      uint64_t bytes = 0;
      for (auto& kv : need) {
        uint64_t n = 2;
        for (auto d : kv.second.second) n *= d;
        bytes += n;
      }
      if (bytes > ((uint64_t)8 << 30)) fail(ErrorKind::Capacity, "refusing to synthesize more than 8 GiB of weights on the host");
      interp::Weights::random(need, seed).save(argv[3]);
      std::cout << "{\"tensors\": " << need.size() << ", \"bytes\": " << bytes << "}\n";
      return 0;
    }
    if (cmd == "interpret") return interpret(argc, argv);
    if (cmd == "inspect") return argc < 3 ? usage() : inspect(argv[2]);
    if (cmd == "validate-bundle") {
      if (argc < 3) return usage();
      std::cout << contract::validate_bundle(argv[2]).dump(1) << "\n";
      return 0;
    }
    if (cmd == "inspect-config") {
      // inspect-config CONFIG.json [OUT.json]: layer forms, features, required operations and kernels of an MLA + MoE config
      if (argc < 3) return usage();
      write_or_print(config_audit::audit(read_file(argv[2], config_audit::kMaxConfigBytes)), argc > 3 ? argv[3] : nullptr);
      return 0;
    }
    if (cmd == "inspect-checkpoint") return inspect_checkpoint(argc, argv);
    if (cmd == "bind-checkpoint") return bind_checkpoint(argc, argv);
    if (cmd == "plan-placement") return plan_placement(argc, argv);
    if (cmd == "plan" || cmd == "plan-debug") {
      // plan GRAPH.json|MODEL.inferfabric [OUT.ifplan] [--dump-ir DIR]: compile for the CPU f32 target; DIR receives the pipeline's stages
      if (argc < 3) return usage();
      cpu::Options o;
      o.debug_names = cmd == "plan-debug";
      std::string out_path, dump_dir;
      for (int i = 3; i < argc; ++i) {
        if (std::string(argv[i]) == "--dump-ir" && i + 1 < argc) dump_dir = argv[++i];
        else out_path = argv[i];
      }
      const cpu::LogicalGraph g = load_cpu_graph(argv[2]);
      cpu::Stages stages;
      cpu::PhysicalPlan plan = cpu::compile(g, o, &stages);
      cpu::verify(plan);
      const std::string binary = cpu::encode_plan(plan);
      if (!out_path.empty()) write_file_atomic(out_path, binary);
      if (!dump_dir.empty()) {
        ::mkdir(dump_dir.c_str(), 0755);
        write_file_atomic(dump_dir + "/00-logical.json", g.to_json().dump(1) + "\n");
        write_file_atomic(dump_dir + "/01-typed.json", stages.typed.dump(1) + "\n");
        write_file_atomic(dump_dir + "/02-optimized.json", stages.optimized.dump(1) + "\n");
        write_file_atomic(dump_dir + "/03-physical.json", plan.to_json().dump(1) + "\n");
        write_file_atomic(dump_dir + "/04-bundle-manifest.json", cpu::manifest(binary).dump(1) + "\n");
      }
      std::cout << plan.to_json().dump(1) << "\n";
      return 0;
    }
    if (cmd == "tune-plan") {
      // tune-plan PLAN.ifplan OVERRIDES.json OUT.ifplan: {"step name": "kernel name", ...}
      if (argc < 5) return usage();
      const cpu::PhysicalPlan plan = cpu::decode_plan(read_file(argv[2], 64 << 20));
      std::map<std::string, std::string> overrides;
      const Json wanted = Json::parse(read_file(argv[3], 1 << 20));
      for (auto& kv : wanted.as_object()) overrides[kv.first] = kv.second.as_string();
      const cpu::PhysicalPlan tuned = cpu::tune(plan, overrides);
      write_file_atomic(argv[4], cpu::encode_plan(tuned));
      std::cout << tuned.to_json().dump(1) << "\n";
      return 0;
    }
    if (cmd == "explain-plan") {
      // explain-plan PLAN.ifplan|GRAPH [--html OUT.html]
      if (argc < 3) return usage();
      const std::string bytes = read_file(argv[2], 64 << 20);
      cpu::PhysicalPlan plan = bytes.rfind("IFPLAN01", 0) == 0 ? cpu::decode_plan(bytes) : cpu::compile(load_cpu_graph(argv[2]));
      cpu::verify(plan);
      if (argc >= 5 && std::string(argv[3]) == "--html") write_file_atomic(argv[4], cpu::html_view(plan));
      std::cout << plan.to_json().dump(1) << "\n";
      return 0;
    }
    if (cmd == "execute") {
      if (argc < 4) return usage();
      cpu::PhysicalPlan plan = cpu::compile(load_cpu_graph(argv[2]));
      cpu::verify(plan);
      cpu::Executor ex(plan);
      Json inputs = Json::parse(read_file(argv[3], 16 << 20));
      Json reports = Json::array();
      auto run_one = [&](const Json& step) {
        std::map<std::string, std::vector<float>> in;
        for (auto& kv : step.as_object()) {
          std::vector<float> v;
          for (auto& x : kv.second.as_array()) v.push_back((float)x.as_double());
          in[kv.first] = std::move(v);
        }
        reports.push(ex.run(in).to_json());
      };
      if (inputs.is_array()) for (auto& s : inputs.as_array()) run_one(s);
      else run_one(inputs);
      std::cout << reports.dump(1) << "\n";
      return 0;
    }
    if (cmd == "inspect-hybrid-checkpoint" || cmd == "compile-checkpoint" || cmd == "lower-checkpoint") {
      // the checkpoint-bound path of the hybrid decoder family: MODEL must carry the qwen35_text_v1 contract
      if (argc < 4) return usage();
      const rankplan::Spec spec = definition::parse_checkpoint_spec(read_file(argv[2], definition::kMaxArtifactBytes));
      const hybrid::Checkpoint ck = hybrid::inspect(argv[3], spec.model);
      Json out;
      int next = 4;
      if (cmd == "inspect-hybrid-checkpoint") {
        out = ck.to_json();
      } else {
        const hybrid::Plan plan = hybrid::compile(spec, ck);
        if (cmd == "compile-checkpoint") {
          out = plan.to_json();
        } else {
          if (argc < 5) return usage();
          const uint32_t context = (uint32_t)std::stoul(argv[4]);
          uint32_t batch = 1;
          next = 5;
          if (argc > 5 && std::string(argv[5]).find_first_not_of("0123456789") == std::string::npos) { batch = (uint32_t)std::stoul(argv[5]); next = 6; }
          out = hybrid::lower_batch(plan, context, batch).to_json();
        }
      }
      if (argc > next) write_file_atomic(argv[next], out.dump(1));
      else std::cout << out.dump(1) << "\n";
      return 0;
    }
    if (cmd == "tokenize" || cmd == "detokenize" || cmd == "render-chat") {
      // TOKENIZER = "bytes" or a tokenizer.json; tokenize TEXT_FILE -> ids (+ the words they came from); detokenize IDS.json -> text;
      // render-chat MESSAGES.json [STYLE] -> the prompt text and its ids
      if (argc < 4) return usage();
      std::shared_ptr<tok::Tokenizer> t = tok::load_tokenizer(argv[2]);
      Json out = Json::object();
      out.set("tokenizer", t->name());
      out.set("vocab_size", t->vocab_size());
      if (cmd == "tokenize") {
        const std::string text = read_file(argv[3], 64 << 20);
        Json ids = Json::array(), words = Json::array();
        for (auto id : t->encode(text)) ids.push((int64_t)id);
        if (t->name() == "bpe")
          for (auto w : tok::BpeTokenizer::split_words(text)) words.push(std::string(w));
        out.set("ids", ids);
        out.set("words", words);
      } else if (cmd == "detokenize") {
        std::vector<uint32_t> ids;
        const Json list = Json::parse(read_file(argv[3], 64 << 20));
        for (auto& x : list.as_array()) ids.push_back((uint32_t)x.as_int());
        out.set("text", t->decode(ids));
        out.set("text_without_special", t->decode(ids, true));
        tok::Detokenizer stream(t, false);
        Json parts = Json::array();
        for (auto id : ids) parts.push(stream.feed(id));
        parts.push(stream.flush());
        out.set("stream", parts);
      } else {
        std::vector<tok::ChatMessage> msgs;
        const Json list = Json::parse(read_file(argv[3], 16 << 20));
        for (auto& m : list.as_array()) msgs.push_back({m.at("role").as_string(), m.at("content").as_string()});
        const std::string text = tok::render_chat(msgs, *t, argc > 4 ? argv[4] : "auto");
        out.set("text", text);
        Json ids = Json::array();
        for (auto id : t->encode(text)) ids.push((int64_t)id);
        out.set("ids", ids);
      }
      std::cout << out.dump() << "\n";
      return 0;
    }
    if (cmd == "compile-model") {
      // any document -> the versioned JSON artifact (inferfabric.model); an artifact is re-validated and re-written
      if (argc < 3) return usage();
      const std::string out = definition::encode(definition::definition(read_file(argv[2], definition::kMaxArtifactBytes)));
      if (argc >= 4) write_file_atomic(argv[3], out);
      else std::cout << out << "\n";
      return 0;
    }
    if (cmd == "compile") {
      if (argc < 4) return usage();
      const std::string text = read_file(argv[2], 16 << 20);
      const std::string path = argv[2];
      const bool dsl = path.size() > 12 && path.compare(path.size() - 12, 12, ".inferfabric") == 0;
      rankplan::Spec spec = dsl ? definition::parse_spec(text) : rankplan::Spec::from_json(Json::parse(text));
      rankplan::Artifact art = rankplan::compile(spec);
      write_file_atomic(argv[3], rankplan::encode(art));
      std::cout << art.to_json().dump(1) << "\n";
      return 0;
    }
    if (cmd == "demo") return demo();
    return usage();
  } catch (const Error& e) {
    std::fprintf(stderr, "ifab: %s\n", e.describe().c_str());
    return 1;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "ifab: %s\n", e.what());
    return 1;
  }
}
