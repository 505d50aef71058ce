#include "serving.h"

#include <algorithm>
#include <set>

namespace ifab::serving {

const char* phase_name(Phase p) {
  switch (p) {
    case Phase::Decode: return "decode";
    case Phase::Prefill: return "prefill";
    case Phase::Extend: return "extend";
  }
  return "?";
}
static Phase parse_phase(const std::string& s) {
  if (s == "decode") return Phase::Decode;
  if (s == "prefill") return Phase::Prefill;
  if (s == "extend") return Phase::Extend;
  invalid("unknown phase " + s);
}

bool Variant::accepts_query_tokens(uint32_t n) const {
  if (n == 0) return false;
  if (query_tokens.empty()) return n <= max_query_tokens;
  return std::find(query_tokens.begin(), query_tokens.end(), n) != query_tokens.end();
}

uint32_t sliding_capacity(uint32_t context, uint32_t window, uint32_t query, uint32_t page) {
  if (page == 0) invalid("page size is zero");
  if (window == 0 || window >= context) return (context + page - 1) / page * page;
  // the window, the rows being appended, and one page of slack so that a partially overwritten
  // page never holds visible rows
  uint64_t rows = (uint64_t)window + query + page - 1;
  rows = (rows + page - 1) / page * page;
  uint64_t full = ((uint64_t)context + page - 1) / page * page;
  return (uint32_t)std::min(rows, full);
}

uint32_t Batch::total_tokens() const {
  uint32_t n = 0;
  for (auto& s : spans) n += s.token_count;
  return n;
}

const Variant* Manifest::find_variant(std::string_view name) const {
  for (auto& v : variants)
    if (v.name == name) return &v;
  return nullptr;
}
const Variant* Manifest::choose_variant(Phase phase, uint32_t tokens) const {
  const Variant* best = nullptr;
  for (auto& v : variants) {
    if (v.phase != phase || !v.accepts_query_tokens(tokens)) continue;
    if (!best || v.max_query_tokens < best->max_query_tokens) best = &v;
  }
  return best;
}

void Manifest::validate() const {
  if (identity.model.empty() || identity.program_sha256.size() != 64) invalid("manifest: identity is incomplete");
  if (max_context == 0 || vocab == 0) invalid("manifest: context and vocab must be positive");
  if (eos >= vocab) invalid("manifest: eos outside the vocabulary");
  if (resident_sequences == 0 || max_batched_tokens == 0) invalid("manifest: capacities must be positive");
  if (variants.empty()) invalid("manifest: no execution variants");
  std::set<std::string> names;
  bool has_decode = false;
  for (auto& v : variants) {
    if (!names.insert(v.name).second) invalid("manifest: duplicate variant " + v.name);
    if (v.max_query_tokens == 0 || v.max_query_tokens > max_context) invalid("manifest: variant " + v.name + " has a bad token capacity");
    for (size_t i = 0; i < v.query_tokens.size(); ++i) {
      if (v.query_tokens[i] == 0 || v.query_tokens[i] > v.max_query_tokens) invalid("manifest: variant " + v.name + " lists a token count above its capacity");
      if (i && v.query_tokens[i] <= v.query_tokens[i - 1]) invalid("manifest: variant " + v.name + " token counts must ascend");
    }
    if (v.phase == Phase::Decode) {
      has_decode = true;
      if (v.max_query_tokens != 1 && v.query_tokens.empty()) invalid("manifest: decode variants take exactly one token per sequence");
    }
    if (v.numerics.empty()) invalid("manifest: variant " + v.name + " has no numerics class");
  }
  if (!has_decode) invalid("manifest: no decode variant");
  std::set<std::string> snames;
  for (size_t i = 0; i < states.size(); ++i) {
    const State& s = states[i];
    if (!snames.insert(s.name).second) invalid("manifest: duplicate state " + s.name);
    if (s.component != i) invalid("manifest: state components must be dense and ordered");
    if (s.storage.kind == Storage::Kind::Pages) {
      if (s.storage.page_tokens == 0 || s.storage.row_bytes == 0) invalid("manifest: paged state " + s.name + " needs page_tokens and row_bytes");
    } else if (s.storage.slot_bytes == 0) {
      invalid("manifest: slot state " + s.name + " needs slot_bytes");
    }
    if (s.retention.kind == Retention::Kind::SlidingWindow) {
      if (s.storage.kind != Storage::Kind::Pages) invalid("manifest: only paged states slide");
      if (s.retention.window == 0 || s.retention.window > max_context) invalid("manifest: bad window for " + s.name);
    }
  }
}

void Manifest::validate_batch(const Batch& b) const {
  const Variant* v = find_variant(b.variant);
  if (!v) invalid("batch: unknown variant " + b.variant);
  if (b.spans.empty()) invalid("batch: empty");
  if (b.total_tokens() > max_batched_tokens) fail(ErrorKind::Capacity, "batch: token budget exceeded");
  std::set<uint32_t> seen;
  for (auto& s : b.spans) {
    if (s.resident >= resident_sequences) invalid("batch: resident out of range");
    if (!seen.insert(s.resident).second) invalid("batch: resident appears twice");
    if (s.token_count == 0) invalid("batch: empty span");
    if (v->phase == Phase::Decode && s.token_count != 1) invalid("batch: decode spans carry one token");
    if (v->phase != Phase::Decode && !v->accepts_query_tokens(s.token_count)) invalid("batch: variant " + v->name + " does not accept " + std::to_string(s.token_count) + " tokens");
    if ((uint64_t)s.position + s.token_count > max_context) fail(ErrorKind::Capacity, "batch: span exceeds the context");
    if (v->phase == Phase::Prefill && s.position != 0) invalid("batch: prefill starts at position 0 (use extend)");
  }
}

uint64_t Manifest::state_bytes_per_sequence() const {
  uint64_t n = 0;
  for (auto& s : states) {
    if (s.storage.kind == Storage::Kind::Slot) {
      n += s.storage.slot_bytes;
    } else {
      uint32_t rows = s.retention.kind == Retention::Kind::SlidingWindow
                          ? sliding_capacity(max_context, s.retention.window, max_batched_tokens, s.storage.page_tokens)
                          : (max_context + s.storage.page_tokens - 1) / s.storage.page_tokens * s.storage.page_tokens;
      n += (uint64_t)rows * s.storage.row_bytes;
    }
  }
  return n;
}

Json Manifest::to_json() const {
  Json j = Json::object();
  j.set("format", "inferfabric.serving.v1");
  Json id = Json::object();
  id.set("model", identity.model);
  id.set("program_sha256", identity.program_sha256);
  id.set("target", identity.target);
  id.set("tp", identity.tp);
  j.set("identity", id);
  j.set("max_context", max_context);
  j.set("vocab", vocab);
  j.set("eos", eos);
  j.set("resident_sequences", resident_sequences);
  j.set("max_batched_tokens", max_batched_tokens);
  Json vs = Json::array();
  for (auto& v : variants) {
    Json o = Json::object();
    o.set("name", v.name);
    o.set("phase", phase_name(v.phase));
    Json q = Json::array();
    for (auto t : v.query_tokens) q.push((int64_t)t);
    o.set("query_tokens", q);
    o.set("max_query_tokens", v.max_query_tokens);
    o.set("captured", v.captured);
    o.set("numerics", v.numerics);
    vs.push(o);
  }
  j.set("variants", vs);
  Json ss = Json::array();
  for (auto& s : states) {
    Json o = Json::object();
    o.set("name", s.name);
    o.set("component", s.component);
    o.set("dtype", s.dtype);
    Json st = Json::object();
    if (s.storage.kind == Storage::Kind::Pages) {
      st.set("kind", "pages");
      st.set("page_tokens", s.storage.page_tokens);
      st.set("row_bytes", s.storage.row_bytes);
    } else {
      st.set("kind", "slot");
      st.set("slot_bytes", s.storage.slot_bytes);
    }
    o.set("storage", st);
    Json rt = Json::object();
    rt.set("kind", s.retention.kind == Retention::Kind::Full ? "full" : "sliding_window");
    if (s.retention.kind == Retention::Kind::SlidingWindow) rt.set("window", s.retention.window);
    o.set("retention", rt);
    ss.push(o);
  }
  j.set("states", ss);
  Json lim = Json::array();
  for (auto& l : limitations) lim.push(l);
  j.set("limitations", lim);
  j.set("state_bytes_per_sequence", state_bytes_per_sequence());
  return j;
}

Manifest Manifest::from_json(const Json& j) {
  if (j.at("format").as_string() != "inferfabric.serving.v1") invalid("not a serving manifest");
  Manifest m;
  const Json& id = j.at("identity");
  m.identity.model = id.at("model").as_string();
  m.identity.program_sha256 = id.at("program_sha256").as_string();
  m.identity.target = id.at("target").as_string();
  m.identity.tp = (uint32_t)id.at("tp").as_int();
  m.max_context = (uint32_t)j.at("max_context").as_int();
  m.vocab = (uint32_t)j.at("vocab").as_int();
  m.eos = (uint32_t)j.at("eos").as_int();
  m.resident_sequences = (uint32_t)j.at("resident_sequences").as_int();
  m.max_batched_tokens = (uint32_t)j.at("max_batched_tokens").as_int();
  for (auto& v : j.at("variants").as_array()) {
    Variant x;
    x.name = v.at("name").as_string();
    x.phase = parse_phase(v.at("phase").as_string());
    for (auto& t : v.at("query_tokens").as_array()) x.query_tokens.push_back((uint32_t)t.as_int());
    x.max_query_tokens = (uint32_t)v.at("max_query_tokens").as_int();
    x.captured = v.at("captured").as_bool();
    x.numerics = v.at("numerics").as_string();
    m.variants.push_back(std::move(x));
  }
  for (auto& s : j.at("states").as_array()) {
    State x;
    x.name = s.at("name").as_string();
    x.component = (uint32_t)s.at("component").as_int();
    x.dtype = s.at("dtype").as_string();
    const Json& st = s.at("storage");
    if (st.at("kind").as_string() == "pages") {
      x.storage.kind = Storage::Kind::Pages;
      x.storage.page_tokens = (uint32_t)st.at("page_tokens").as_int();
      x.storage.row_bytes = (uint32_t)st.at("row_bytes").as_int();
    } else {
      x.storage.kind = Storage::Kind::Slot;
      x.storage.slot_bytes = (uint64_t)st.at("slot_bytes").as_int();
    }
    const Json& rt = s.at("retention");
    if (rt.at("kind").as_string() == "sliding_window") {
      x.retention.kind = Retention::Kind::SlidingWindow;
      x.retention.window = (uint32_t)rt.at("window").as_int();
    }
    m.states.push_back(std::move(x));
  }
  if (auto l = j.find("limitations"))
    for (auto& s : l->as_array()) m.limitations.push_back(s.as_string());
  m.validate();
  return m;
}

Manifest lower(const program::Program& p, const std::string& program_sha256) {
  Manifest m;
  m.identity = {p.name, program_sha256, p.parallel.target, p.parallel.tp};
  m.max_context = p.max_context;
  m.eos = p.eos;
  m.resident_sequences = p.options.resident_sequences;
  m.max_batched_tokens = std::max<uint32_t>(p.parallel.max_num_batched_tokens, std::max(p.options.prefill_tokens, p.options.resident_sequences));
  for (auto& i : p.instructions)
    if (i.op == "embedding") m.vocab = (uint32_t)strtoul(i.attr("vocab")->c_str(), nullptr, 10);
  if (m.vocab == 0) m.vocab = p.instructions[p.output].width;

  Variant dec;
  dec.name = "decode";
  dec.phase = Phase::Decode;
  dec.max_query_tokens = 1;
  dec.numerics = "gemv_f32acc";
  m.variants.push_back(dec);
  if (!p.options.prefill_variants.empty()) {
    for (uint32_t n : p.options.prefill_variants) {
      for (Phase ph : {Phase::Prefill, Phase::Extend}) {
        Variant v;
        v.name = std::string(phase_name(ph)) + "_" + std::to_string(n);
        v.phase = ph;
        v.query_tokens = {n};
        v.max_query_tokens = n;
        v.numerics = n <= 8 ? "gemv_f32acc" : "tcgen05_f32acc";
        m.variants.push_back(v);
      }
    }
  } else if (p.options.prefill_tokens > 1) {
    for (Phase ph : {Phase::Prefill, Phase::Extend}) {
      Variant v;
      v.name = std::string(phase_name(ph)) + (p.options.uncaptured_prefill ? "_chunk" : "_" + std::to_string(p.options.prefill_tokens));
      v.phase = ph;
      v.max_query_tokens = p.options.prefill_tokens;
      if (!p.options.uncaptured_prefill) v.query_tokens = {p.options.prefill_tokens};
      v.captured = !p.options.uncaptured_prefill;
      v.numerics = p.options.prefill_tokens <= 8 ? "gemv_f32acc" : "tcgen05_f32acc";
      m.variants.push_back(v);
    }
  }
  // states
  std::vector<std::vector<uint32_t>> users(p.instructions.size());
  for (uint32_t k = 0; k < p.instructions.size(); ++k)
    for (uint32_t in : p.instructions[k].inputs) users[in].push_back(k);
  for (uint32_t k = 0; k < p.instructions.size(); ++k) {
    const auto& i = p.instructions[k];
    State s;
    s.component = (uint32_t)m.states.size();
    s.name = i.name;
    if (i.kind == (uint32_t)graph::Kind::Cache) {
      s.dtype = i.dtype;
      s.storage.kind = Storage::Kind::Pages;
      if (i.dtype == "int8_ds_mla") {
        // packed row: int8 latent + bf16 rope + one f32 scale per 128 latent columns
        uint32_t rope = 64, latent = i.width - rope;
        s.storage.page_tokens = 32;
        s.storage.row_bytes = latent + rope * 2 + latent / 128 * 4;
      } else if (i.dtype == "int8") {
        s.storage.page_tokens = 16;
        s.storage.row_bytes = i.width + 4;
      } else if (i.dtype == "int4") {
        s.storage.page_tokens = 16;
        s.storage.row_bytes = i.width / 2 + 4;
      } else {
        s.storage.page_tokens = 16;
        s.storage.row_bytes = i.width * 2;
      }
      uint32_t window = 0;
      bool all_windowed = !users[k].empty();
      for (uint32_t u : users[k]) {
        auto w = p.instructions[u].attr("window");
        uint32_t wv = w ? (uint32_t)strtoul(w->c_str(), nullptr, 10) : 0;
        auto sel = p.instructions[u].attr("selection");
        if (wv == 0 || (sel && *sel == "learned_indices")) all_windowed = false;
        window = std::max(window, wv);
      }
      if (all_windowed && window < p.max_context) {
        s.retention.kind = Retention::Kind::SlidingWindow;
        s.retention.window = window;
      }
      m.states.push_back(s);
    } else if (i.kind == (uint32_t)graph::Kind::IndexCache) {
      s.dtype = i.dtype;
      s.storage.kind = Storage::Kind::Pages;
      s.storage.page_tokens = 64;
      s.storage.row_bytes = i.dtype == "int8" ? i.width + 2 : i.width * 2;
      m.states.push_back(s);
    } else if (i.op == "mome") {
      uint32_t taps = (uint32_t)strtoul(i.attr("taps")->c_str(), nullptr, 10);
      s.dtype = "bf16";
      s.storage.kind = Storage::Kind::Slot;
      s.storage.slot_bytes = (uint64_t)(taps - 1) * i.width * 2;
      m.states.push_back(s);
    }
  }
  if (p.parallel.tp > 1) m.limitations.push_back("single node: all ranks must share one NVSwitch domain");
  m.limitations.push_back("greedy sampling on the fused lm_head path; other samplers read gathered logits");
  m.validate();
  return m;
}

bool PrefixIdentity::compatible(const PrefixIdentity& o) const {
  return program_sha256 == o.program_sha256 && weights_sha256 == o.weights_sha256 && ns == o.ns && salt == o.salt && page_tokens == o.page_tokens;
}

void ArithmeticHistory::check_append(uint32_t begin, uint32_t count) const {
  if (count == 0) invalid("history: empty span");
  if (begin != length()) invalid("history: span does not continue the sequence (expected position " + std::to_string(length()) + ")");
}
void ArithmeticHistory::append_completed(uint32_t begin, uint32_t count, const std::string& numerics) {
  check_append(begin, count);
  if (!spans_.empty() && spans_.back().numerics == numerics) spans_.back().end += count;
  else spans_.push_back({begin, begin + count, numerics});
}
ArithmeticHistory ArithmeticHistory::prefix(uint32_t tokens) const {
  if (tokens > length()) invalid("history: prefix longer than the sequence");
  ArithmeticHistory h;
  for (auto& s : spans_) {
    if (s.begin >= tokens) break;
    h.spans_.push_back({s.begin, std::min(s.end, tokens), s.numerics});
  }
  return h;
}
bool ArithmeticHistory::same_prefix(const ArithmeticHistory& o, uint32_t tokens) const {
  if (tokens > length() || tokens > o.length()) return false;
  auto a = prefix(tokens), b = o.prefix(tokens);
  if (a.spans_.size() != b.spans_.size()) return false;
  for (size_t i = 0; i < a.spans_.size(); ++i)
    if (a.spans_[i].begin != b.spans_[i].begin || a.spans_[i].end != b.spans_[i].end || a.spans_[i].numerics != b.spans_[i].numerics) return false;
  return true;
}

}  // namespace ifab::serving
