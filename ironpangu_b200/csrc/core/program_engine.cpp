#include "contract.h"
#include "program_engine.h"

#include <map>
#include <set>

#include "interp.h"

namespace ifab {
namespace {

thread_local std::string g_error;

// One compiled bundle executed by the CPU interpreter; every resident sequence slot owns an interpreter state.
class CpuProgram {
 public:
  CpuProgram(const std::string& bundle, const std::string& checkpoint, uint32_t preparation, uint32_t residents_override = 0,
             uint32_t context_override = 0)
      : graph_(graph::compile_source(read_file(bundle + "/model.inferfabric", 1 << 20))),   // checked again on load
        weights_(interp::Weights::from_checkpoint(init::Checkpoint::inspect(checkpoint))),
        preparation_(preparation != 0) {
    const Json man = Json::parse(read_file(bundle + "/serving.json"));
    context_ = (uint32_t)man.at("max_context").as_int();
    vocab_ = (uint32_t)man.at("vocab").as_int();
    eos_ = (uint32_t)man.at("eos").as_int();
    uint32_t residents = (uint32_t)man.at("resident_sequences").as_int();
    chunk_ = (uint32_t)man.at("max_batched_tokens").as_int();
    if (residents_override) residents = residents_override;
    if (context_override && context_override < context_) context_ = context_override;
    if (residents == 0) residents = 1;
    if (chunk_ < 8) chunk_ = 8;   // the host executor takes any run length; the manifest value only bounds device variants
    for (uint32_t i = 0; i < residents; ++i) slots_.push_back(std::make_unique<interp::Interpreter>(graph_, weights_));
    next_.assign(residents, 0);
    if (vocab_ == 0) vocab_ = slots_[0]->vocab();
  }

  uint32_t context() const { return context_; }
  uint32_t vocab() const { return vocab_; }
  uint32_t eos() const { return eos_; }
  uint32_t residents() const { return (uint32_t)slots_.size(); }
  uint32_t chunk() const { return chunk_; }
  uint32_t selected = 0;

  void check_slot(uint32_t slot) const {
    if (slot >= slots_.size()) invalid("program engine: resident slot " + std::to_string(slot) + " does not exist");
  }
  void reset_slot(uint32_t slot) {
    check_slot(slot);
    slots_[slot]->reset();
    next_[slot] = 0;
  }
  void reset_all() {
    for (uint32_t i = 0; i < slots_.size(); ++i) reset_slot(i);
  }
  // feeds `count` tokens of one sequence; returns the greedy token after the last one
  uint32_t feed(uint32_t slot, const uint32_t* tokens, uint32_t count, uint32_t position) {
    check_slot(slot);
    if (preparation_) fail(ErrorKind::Backend, "program engine: opened in preparation mode, generation is disabled");
    if (count == 0) invalid("program engine: empty token run");
    if (position != next_[slot]) invalid("program engine: resident " + std::to_string(slot) + " stands at position " + std::to_string(next_[slot]) +
                                         ", got " + std::to_string(position));
    if ((uint64_t)position + count > context_) fail(ErrorKind::Capacity, "program engine: the run passes the end of the context");
    uint32_t out = 0;
    for (uint32_t i = 0; i < count; ++i) {
      if (tokens[i] >= vocab_) invalid("program engine: token id outside the vocabulary");
      out = slots_[slot]->step(tokens[i], position + i);
    }
    next_[slot] = position + count;
    return out;
  }
  void copy(uint32_t src, uint32_t dst, uint32_t boundary) {
    check_slot(src);
    check_slot(dst);
    if (src == dst) invalid("program engine: source and destination are the same resident");
    if (next_[src] != boundary) invalid("program engine: the source resident is not at the boundary");
    if (next_[dst] != 0) invalid("program engine: the destination resident must be reset first");
    slots_[dst] = std::make_unique<interp::Interpreter>(*slots_[src]);
    next_[dst] = boundary;
  }
  void bind(const std::string& key, const int32_t* pages, uint32_t count) {
    std::set<int32_t> seen;
    for (uint32_t i = 0; i < count; ++i) {
      if (pages[i] < 0) invalid("program engine: negative page id in a binding");
      if (!seen.insert(pages[i]).second) invalid("program engine: duplicate page id in a binding");
    }
    bindings_[key].assign(pages, pages + count);
  }

 private:
  graph::Graph graph_;
  interp::Weights weights_;
  bool preparation_;
  uint32_t context_ = 0, vocab_ = 0, eos_ = 0, chunk_ = 8;
  std::vector<std::unique_ptr<interp::Interpreter>> slots_;
  std::vector<uint32_t> next_;
  std::map<std::string, std::vector<int32_t>> bindings_;
};

template <typename F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const Error& e) {
    g_error = e.describe();
    return 1 + (int)e.kind();
  } catch (const std::exception& e) {
    g_error = e.what();
    return 100;
  }
}
CpuProgram* P(void* engine) {
  if (!engine) invalid("program engine: null handle");
  return static_cast<CpuProgram*>(engine);
}

class CpuResidentEngine : public serve::ResidentEngine {
 public:
  CpuResidentEngine(const std::string& bundle, const std::string& checkpoint, uint32_t residents, uint32_t context)
      : p_(bundle, checkpoint, 0, residents, context), name_(bundle.substr(bundle.find_last_of('/') + 1)) {}
  serve::EngineInfo info() const override {
    serve::EngineInfo e;
    e.model = name_.empty() ? "ifab-program" : name_;
    e.residents = p_.residents();
    e.token_budget = e.chunk = p_.chunk();
    e.context = p_.context();
    e.vocab = p_.vocab();
    e.eos = p_.eos();
    e.has_eos = false;
    e.greedy_only = true;
    return e;
  }
  void admit(uint32_t resident, const serve::SamplingParams& s, uint32_t) override {
    if (!s.greedy()) invalid("the program engine samples greedily only");
    p_.reset_slot(resident);
  }
  std::vector<uint32_t> step(const paging::SequenceBatch& batch) override {
    std::vector<uint32_t> out;
    size_t off = 0;
    std::vector<uint32_t> toks;
    for (const auto& sl : batch.slices) {
      toks.assign(batch.tokens.begin() + off, batch.tokens.begin() + off + sl.token_count);
      out.push_back(p_.feed(sl.resident, toks.data(), sl.token_count, sl.position));
      off += sl.token_count;
    }
    return out;
  }
  void release(uint32_t resident) override { p_.reset_slot(resident); }

 private:
  CpuProgram p_;
  std::string name_;
};

}  // namespace

namespace serve {
std::shared_ptr<ResidentEngine> make_cpu_program_engine(const std::string& bundle, const std::string& checkpoint, uint32_t residents,
                                                        uint32_t context) {
  contract::validate_bundle(bundle);
  return std::make_shared<CpuResidentEngine>(bundle, checkpoint, residents, context);
}
}  // namespace serve
}  // namespace ifab

using namespace ifab;

extern "C" {

uint32_t ifab_program_abi_version(void) { return 1; }
const char* ifab_program_error(void) { return g_error.c_str(); }

int ifab_program_open(const char* bundle, const char* checkpoint, uint32_t preparation, void** out) {
  return guard([&] {
    if (!bundle || !checkpoint || !out) invalid("program engine: null argument");
    *out = nullptr;
    contract::validate_bundle(bundle);   // kernel and binding contracts of the serialized program, before anything is loaded
    *out = new CpuProgram(bundle, checkpoint, preparation);
  });
}
int ifab_program_close(void* engine) {
  return guard([&] { delete P(engine); });
}
int ifab_program_info(void* engine, uint32_t* context, uint32_t* vocabulary, uint32_t* eos) {
  return guard([&] {
    CpuProgram* p = P(engine);
    if (context) *context = p->context();
    if (vocabulary) *vocabulary = p->vocab();
    if (eos) *eos = p->eos();
  });
}
int ifab_program_reset(void* engine) {
  return guard([&] { P(engine)->reset_all(); });
}
int ifab_program_resident_capacity(void* engine, uint32_t* count) {
  return guard([&] { *count = P(engine)->residents(); });
}
int ifab_program_select_resident(void* engine, uint32_t slot) {
  return guard([&] {
    P(engine)->check_slot(slot);
    P(engine)->selected = slot;
  });
}
int ifab_program_reset_resident(void* engine, uint32_t slot) {
  return guard([&] { P(engine)->reset_slot(slot); });
}
int ifab_program_copy_resident(void* engine, uint32_t source, uint32_t destination, uint32_t boundary) {
  return guard([&] { P(engine)->copy(source, destination, boundary); });
}
int ifab_program_bind_pages(void* engine, uint32_t rank, const char* component, const int32_t* pages, uint32_t count) {
  return guard([&] {
    if (!component || (!pages && count)) invalid("program engine: null argument");
    P(engine)->bind("pages/" + std::to_string(rank) + "/" + component, pages, count);
  });
}
int ifab_program_bind_state(void* engine, uint32_t rank, uint32_t logical_node, const int32_t* pages, uint32_t count) {
  return guard([&] {
    if (!pages && count) invalid("program engine: null argument");
    P(engine)->bind("state/" + std::to_string(rank) + "/" + std::to_string(logical_node), pages, count);
  });
}
int ifab_program_shared_pages(void* engine, uint32_t* enabled) {
  return guard([&] {
    P(engine);
    *enabled = 0;
  });
}
int ifab_program_token(void* engine, uint32_t token, uint32_t position, uint32_t sample, uint32_t* output) {
  return guard([&] {
    CpuProgram* p = P(engine);
    const uint32_t t = p->feed(p->selected, &token, 1, position);
    if (sample && output) *output = t;
  });
}
int ifab_program_prefill_capacity(void* engine, uint32_t* count) {
  return guard([&] { *count = P(engine)->chunk(); });
}
int ifab_program_prefill_mode(void* engine, uint32_t* mode) {
  return guard([&] {
    P(engine);
    *mode = 1;
  });
}
int ifab_program_prefill_variants(void* engine, uint32_t* mask) {
  return guard([&] {
    const uint32_t c = P(engine)->chunk();
    uint32_t m = 0;
    for (uint32_t n = 1; n <= c && n < 32; ++n) m |= 1u << n;
    *mask = m;
  });
}
int ifab_program_prefill_sizes(void* engine, uint32_t* sizes, uint32_t capacity, uint32_t* count) {
  return guard([&] {
    const uint32_t c = P(engine)->chunk();
    uint32_t n = 0;
    for (uint32_t s = 1; s <= c; s *= 2)
      if (n < capacity) sizes[n++] = s;
    *count = n;
  });
}
int ifab_program_prefill(void* engine, const uint32_t* tokens, uint32_t count, uint32_t position, uint32_t sample, uint32_t* output) {
  return guard([&] {
    CpuProgram* p = P(engine);
    if (!tokens) invalid("program engine: null token array");
    if (count > p->chunk()) fail(ErrorKind::Capacity, "program engine: prefill run exceeds the prefill capacity");
    const uint32_t t = p->feed(p->selected, tokens, count, position);
    if (sample && output) *output = t;
  });
}
int ifab_program_batch(void* engine, const IfabProgramSequenceV1* sequences, uint32_t sequence_count, const uint32_t* tokens,
                       uint32_t token_count, uint32_t* outputs, uint32_t output_capacity, uint32_t* output_count) {
  return guard([&] {
    CpuProgram* p = P(engine);
    if (!sequences || !tokens || !output_count) invalid("program engine: null argument");
    uint64_t total = 0, samples = 0;
    std::set<uint32_t> seen;
    for (uint32_t i = 0; i < sequence_count; ++i) {
      p->check_slot(sequences[i].resident);
      if (!seen.insert(sequences[i].resident).second) invalid("program engine: a resident appears twice in one batch");
      total += sequences[i].token_count;
      samples += sequences[i].sample ? 1 : 0;
    }
    if (total != token_count) invalid("program engine: token_count does not match the sequences");
    if (samples > output_capacity) fail(ErrorKind::Capacity, "program engine: output array is too small");
    uint32_t off = 0, n = 0;
    for (uint32_t i = 0; i < sequence_count; ++i) {
      const uint32_t t = p->feed(sequences[i].resident, tokens + off, sequences[i].token_count, sequences[i].position);
      off += sequences[i].token_count;
      if (sequences[i].sample) outputs[n++] = t;
    }
    *output_count = n;
  });
}
int ifab_program_batch_capacity(void* engine, uint32_t* capacity) {
  return guard([&] { *capacity = P(engine)->residents(); });
}

}  // extern "C"
