// C ABI of the host core for ctypes bindings. Every call returns a malloc'd, NUL-terminated JSON
// document (free it with ifab_core_free): the result object on success, {"error": {"kind", "message"}}
// on failure. No exception crosses the boundary.
#include <cstdlib>
#include <cstring>

#include "contract.h"
#include "bundle.h"
#include "interp.h"
#include "kernel_plugin.h"

using namespace ifab;

namespace {
char* dup(const std::string& s) {
  char* p = (char*)malloc(s.size() + 1);
  if (p) memcpy(p, s.c_str(), s.size() + 1);
  return p;
}
template <typename F>
char* guarded(F&& f) {
  try {
    return dup(f().dump());
  } catch (const Error& e) {
    Json err = Json::object(), body = Json::object();
    body.set("kind", error_kind_name(e.kind()));
    body.set("message", e.what());
    err.set("error", body);
    return dup(err.dump());
  } catch (const std::exception& e) {
    Json err = Json::object(), body = Json::object();
    body.set("kind", "backend");
    body.set("message", e.what());
    err.set("error", body);
    return dup(err.dump());
  }
}
program::Options options_from(const Json& j) {
  program::Options o;
  if (auto v = j.find("resident_sequences")) o.resident_sequences = (uint32_t)v->as_int();
  if (auto v = j.find("prefill_tokens")) o.prefill_tokens = (uint32_t)v->as_int();
  if (auto v = j.find("prefill_variants"))
    for (auto& x : v->as_array()) o.prefill_variants.push_back((uint32_t)x.as_int());
  if (auto v = j.find("uncaptured_prefill")) o.uncaptured_prefill = v->as_bool();
  if (auto v = j.find("shared_pages")) o.shared_pages = v->as_bool();
  if (auto v = j.find("output_rows")) o.output_rows = v->as_bool();
  if (auto v = j.find("bulk_collectives")) o.bulk_collectives = v->as_bool();
  return o;
}
}  // namespace

extern "C" {

void ifab_core_free(char* p) { free(p); }

// Compile DSL text to the logical graph + physical program (both returned as JSON).
char* ifab_core_compile(const char* source, const char* options_json) {
  return guarded([&] {
    graph::Graph g = graph::compile_source(source);
    program::Program p = program::lower(g, options_from(Json::parse(options_json && *options_json ? options_json : "{}")));
    Json out = Json::object();
    out.set("graph", g.to_json());
    out.set("program", p.to_json());
    out.set("program_sha256", Sha256::of(p.encode()));
    Json need = Json::object();
    for (auto& kv : init::required_tensors(p)) {
      Json t = Json::object();
      t.set("dtype", init::dtype_name(kv.second.first));
      Json s = Json::array();
      for (auto d : kv.second.second) s.push((int64_t)d);
      t.set("shape", s);
      need.set(kv.first, t);
    }
    out.set("required_tensors", need);
    return out;
  });
}

// Compile and publish a bundle directory.
char* ifab_core_write_bundle(const char* source_path, const char* checkpoint_dir, const char* out_dir, const char* kernel_dir,
                             const char* options_json) {
  return guarded([&] {
    bundle::BundleInputs in;
    in.source_path = source_path;
    in.source_text = read_file(source_path, 1 << 20);
    in.checkpoint_dir = checkpoint_dir ? checkpoint_dir : "";
    in.kernel_source_dir = kernel_dir ? kernel_dir : "";
    in.options = options_from(Json::parse(options_json && *options_json ? options_json : "{}"));
    return bundle::write_bundle(in, out_dir).to_json();
  });
}

// Run the CPU interpreter on a compiled source with a safetensors checkpoint directory.
// request: {"tokens": [...], "steps": n}; returns {"generated": [...], "logits_last": [...] (optional)}
char* ifab_core_interpret(const char* source, const char* checkpoint_dir, const char* request_json) {
  return guarded([&] {
    graph::Graph g = graph::compile_source(source);
    Json req = Json::parse(request_json);
    interp::Weights w = interp::Weights::from_checkpoint(init::Checkpoint::inspect(checkpoint_dir));
    interp::Interpreter it(g, w);
    std::vector<uint32_t> toks;
    for (auto& t : req.at("tokens").as_array()) toks.push_back((uint32_t)t.as_int());
    uint32_t steps = req.find("steps") ? (uint32_t)req.at("steps").as_int() : 0;
    bool want_logits = req.find("logits") && req.at("logits").as_bool();
    Json out = Json::object();
    Json gen = Json::array(), pl = Json::array();
    std::vector<float> logits;
    uint32_t next = 0;
    const bool all_logits = req.find("all_logits") && req.at("all_logits").as_bool();
    Json every = Json::array();
    // "watch": node names whose values are reported after every fed token (`watched`: one object per token)
    std::vector<std::string> watch;
    if (const Json* wj = req.find("watch"))
      for (auto& nm : wj->as_array()) watch.push_back(nm.as_string());
    Json watched = Json::array();
    for (size_t i = 0; i < toks.size(); ++i) {
      next = it.step(toks[i], (uint32_t)i, &logits);
      pl.push((int64_t)next);
      if (!watch.empty()) {
        Json at = Json::object();
        for (auto& nm : watch) at.set(nm, it.watch(nm));
        watched.push(std::move(at));
      }
      if (all_logits) {
        Json l = Json::array();
        for (float v : logits) l.push((double)v);
        every.push(std::move(l));
      }
    }
    if (all_logits) out.set("prompt_logits", every);
    if (!watch.empty()) out.set("watched", watched);
    out.set("prompt_argmax", pl);
    uint32_t pos = (uint32_t)toks.size();
    for (uint32_t s = 0; s < steps; ++s) {
      gen.push((int64_t)next);
      next = it.step(next, pos++, &logits);
    }
    out.set("generated", gen);
    if (want_logits) {
      Json l = Json::array();
      for (float v : logits) l.push((double)v);
      out.set("logits_last", l);
    }
    return out;
  });
}

// Read back a bundle's IFINIT01 plan as JSON (for loaders written in other languages).
char* ifab_core_read_init_plan(const char* path) {
  return guarded([&] { return init::Plan::decode(read_file(path)).to_json(); });
}
// Engine-side contract check of a bundle (kernel contracts of execution.bin, binding contracts of every rank-N.bin).
char* ifab_core_validate_bundle(const char* dir) {
  return guarded([&] { return contract::validate_bundle(dir); });
}
char* ifab_core_read_program(const char* path) {
  return guarded([&] { return program::Program::decode(read_file(path)).to_json(); });
}

// Load a kernel plugin that implements "inferfabric.swiglu.bf16.v1" for `target` and run it once on x [T, 2F] -> y [T, F]
// (bf16, row strides in elements). The pointers are host memory for target "cpu" and device memory for the CUDA target;
// `stream` is handed to the plugin unchanged and synchronising it is the caller's job. The plugin's prepared state only
// holds launch arguments, so releasing it right after the enqueue is safe.
char* ifab_core_plugin_swiglu(const char* path, const char* target, void* x, void* y, long T, long F, long ldx, long ldy, void* stream) {
  return guarded([&] {
    plugin::PluginKernel k(path, "inferfabric.swiglu.bf16.v1", target);
    IFKernelTensorV1 in = plugin::make_tensor(x, 2, {T, 2 * F}, 1), out = plugin::make_tensor(y, 2, {T, F}, 2);
    in.strides[0] = ldx;
    out.strides[0] = ldy;
    in.allocation_bytes = plugin::tensor_span_bytes(in);
    out.allocation_bytes = plugin::tensor_span_bytes(out);
    k.prepare({in}, {out});
    k.enqueue(nullptr, 0, stream);
    Json j = Json::object();
    j.set("contract", k.contract());
    j.set("workspace_bytes", k.workspace_bytes());
    return j;
  });
}

}  // extern "C"
