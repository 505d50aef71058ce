#include "interp.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>

namespace ifab::interp {

using graph::Kind;
using graph::Node;

// x -> rint(x / s) * s with s = max|x| / 127 kept in half precision (one scale per row)
static void quantize_row_int8(float* x, size_t n) {
  float mx = 0.f;
  for (size_t i = 0; i < n; ++i) mx = std::max(mx, std::fabs(x[i]));
  if (mx == 0.f) return;
  float s = mx / 127.f;
  {  // round the scale to half precision, ties to even: 11 significant bits, or multiples of 2^-24 below 2^-14 (subnormals)
    if (s < std::ldexp(1.f, -14)) {
      s = std::ldexp(std::nearbyint(std::ldexp(s, 24)), -24);
    } else {
      int e;
      const float m = std::frexp(s, &e);
      s = std::ldexp(std::nearbyint(std::ldexp(m, 11)), e - 11);
    }
    if (s == 0.f) return;
  }
  for (size_t i = 0; i < n; ++i) x[i] = std::max(-127.f, std::min(127.f, std::nearbyint(x[i] / s))) * s;
}

float bf16_round(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;  // inf / nan
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  float r;
  memcpy(&r, &u, 4);
  return r;
}
static uint16_t to_bf16_bits(float v) {
  float r = bf16_round(v);
  uint32_t u;
  memcpy(&u, &r, 4);
  return (uint16_t)(u >> 16);
}

// ---------------------------------------------------------------------------------------------
Weights Weights::from_checkpoint(const init::Checkpoint& ckpt) {
  Weights w;
  std::map<std::string, std::string> files;
  for (auto& kv : ckpt.tensors) {
    const init::TensorInfo& t = kv.second;
    auto it = files.find(t.file);
    if (it == files.end()) it = files.emplace(t.file, read_file(ckpt.dir + "/" + t.file)).first;
    const char* p = it->second.data() + t.data_start + t.begin;
    Tensor x;
    x.shape = t.shape;
    size_t n = 1;
    for (auto d : t.shape) n *= d;
    x.data.resize(n);
    if (t.dtype == init::DType::Bf16) {
      const uint16_t* s = (const uint16_t*)p;
      for (size_t i = 0; i < n; ++i) {
        uint32_t u = (uint32_t)s[i] << 16;
        memcpy(&x.data[i], &u, 4);
      }
    } else if (t.dtype == init::DType::F32) {
      memcpy(x.data.data(), p, n * 4);
    } else {
      fail(ErrorKind::NotImplemented, "interpreter loads bf16 and f32 tensors only (" + t.name + ")");
    }
    w.dtypes[kv.first] = t.dtype;
    w.tensors[kv.first] = std::move(x);
  }
  return w;
}

Weights Weights::random(const std::map<std::string, std::pair<init::DType, std::vector<uint64_t>>>& shapes, uint64_t seed, float std) {
  Weights w;
  for (auto& kv : shapes) {
    // one generator per tensor, keyed by its name, so values do not depend on which tensors exist
    uint64_t s = fnv1a64(kv.first.data(), kv.first.size(), 0x9e3779b97f4a7c15ull ^ (seed * 0x100000001b3ull + 1));
    auto next = [&]() {
      s ^= s << 13;
      s ^= s >> 7;
      s ^= s << 17;
      return s;
    };
    Tensor t;
    t.shape = kv.second.second;
    size_t n = 1;
    for (auto d : t.shape) n *= d;
    t.data.resize(n);
    const bool gain = kv.first.find("norm") != std::string::npos;
    for (size_t i = 0; i < n; i += 2) {
      double u1 = ((next() >> 11) + 1.0) / 9007199254740993.0, u2 = (next() >> 11) / 9007199254740992.0;
      double rad = std::sqrt(-2.0 * std::log(u1)), ang = 6.283185307179586 * u2;
      float a = (float)(rad * std::cos(ang)) * std, b = (float)(rad * std::sin(ang)) * std;
      if (gain) { a += 1.f; b += 1.f; }
      t.data[i] = kv.second.first == init::DType::F32 ? a : bf16_round(a);
      if (i + 1 < n) t.data[i + 1] = kv.second.first == init::DType::F32 ? b : bf16_round(b);
    }
    w.dtypes[kv.first] = kv.second.first;
    w.tensors[kv.first] = std::move(t);
  }
  return w;
}

void Weights::save(const std::string& dir, const std::string& file) const {
  make_dirs(dir);
  std::vector<std::pair<init::TensorInfo, std::string>> out;
  for (auto& kv : tensors) {
    init::TensorInfo t;
    t.name = kv.first;
    t.shape = kv.second.shape;
    auto dt = dtypes.find(kv.first);
    t.dtype = dt == dtypes.end() ? init::DType::Bf16 : dt->second;
    std::string bytes;
    if (t.dtype == init::DType::F32) {
      bytes.assign((const char*)kv.second.data.data(), kv.second.data.size() * 4);
    } else {
      bytes.resize(kv.second.data.size() * 2);
      uint16_t* d = (uint16_t*)bytes.data();
      for (size_t i = 0; i < kv.second.data.size(); ++i) d[i] = to_bf16_bits(kv.second.data[i]);
      t.dtype = init::DType::Bf16;
    }
    out.emplace_back(std::move(t), std::move(bytes));
  }
  init::write_safetensors(dir + "/" + file, out);
}

const Tensor* Weights::find(const std::string& name) const {
  auto it = tensors.find(name);
  return it == tensors.end() ? nullptr : &it->second;
}
const Tensor& Weights::need(const std::string& name) const {
  if (auto t = find(name)) return *t;
  invalid("weights: missing tensor " + name);
}

// ---------------------------------------------------------------------------------------------
namespace {

float dotf(const float* a, const float* b, size_t n) {
  float s = 0.f;
  for (size_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}
std::vector<float> rmsnorm(const std::vector<float>& x, const Tensor& w, float eps, bool zero_centered) {
  if (w.data.size() != x.size()) invalid("norm weight size mismatch");
  double ss = 0;
  for (float v : x) ss += (double)v * v;
  float inv = 1.f / std::sqrt((float)(ss / x.size()) + eps);
  std::vector<float> y(x.size());
  for (size_t i = 0; i < x.size(); ++i) y[i] = bf16_round(x[i] * inv * (zero_centered ? 1.f + w.data[i] : w.data[i]));
  return y;
}
void rope_inplace(float* x, uint32_t d, uint32_t pos, float theta) {
  const uint32_t half = d / 2;
  for (uint32_t i = 0; i < half; ++i) {
    float inv_freq = std::exp2(-(2.f * (float)i / (float)d) * std::log2(theta));
    float ang = (float)pos * inv_freq;
    float c = bf16_round(std::cos(ang)), s = bf16_round(std::sin(ang));
    float a = x[i], b = x[i + half];
    x[i] = bf16_round(a * c - b * s);
    x[i + half] = bf16_round(b * c + a * s);
  }
}
float silu(float v) { return v / (1.f + std::exp(-v)); }
std::string expert_name(const std::string& s, uint32_t e) {
  std::string out = s;
  size_t p = out.find("{expert}");
  if (p != std::string::npos) out.replace(p, 8, std::to_string(e));
  return out;
}

}  // namespace

Interpreter::Interpreter(const graph::Graph& g, const Weights& w) : g_(g), w_(w) {
  tp_ = g.parallel.tp;
  vals_.resize(g.nodes.size());
  for (uint32_t i = 0; i < g.nodes.size(); ++i) {
    const Node& n = g.nodes[i];
    if (n.type.kind == Kind::Cache || n.type.kind == Kind::IndexCache) {
      cache_of_node_[i] = (int)caches_.size();
      CacheState c;
      c.width = n.type.width;
      caches_.push_back(std::move(c));
    }
    if (n.op == "embedding") vocab_ = (uint32_t)n.int_attr("vocab");
  }
  // the vocabulary projection keeps f32 logits (the device lm_head kernel never rounds them)
  const Node& out = g.nodes[g.output];
  if (out.op == "gather" && g.nodes[out.inputs[0]].op == "linear") logits_linear_ = (int64_t)out.inputs[0];
  else if (out.op == "linear") logits_linear_ = (int64_t)g.output;
}

Json Interpreter::watch(const std::string& name) const {
  for (size_t i = 0; i < g_.nodes.size(); ++i) {
    if (g_.nodes[i].name != name) continue;
    const Value& v = vals_[i];
    Json j = Json::object();
    if (v.cache >= 0) {
      j.set("cache_rows", (int64_t)caches_[v.cache].rows.size());
      if (!caches_[v.cache].rows.empty()) {
        Json last = Json::array();
        for (float x : caches_[v.cache].rows.back()) last.push((double)x);
        j.set("last_row", last);
      }
      return j;
    }
    if (!v.ids.empty() || !v.wts.empty()) {
      Json ids = Json::array(), wts = Json::array();
      for (uint32_t x : v.ids) ids.push((int64_t)x);
      for (float x : v.wts) wts.push((double)x);
      j.set("ids", ids);
      j.set("weights", wts);
      return j;
    }
    Json ranks = Json::array();
    for (const auto& r : v.r) {
      Json row = Json::array();
      for (float x : r) row.push((double)x);
      ranks.push(std::move(row));
    }
    j.set("ranks", ranks);
    return j;
  }
  invalid("watch: the graph has no node named " + name);
}

void Interpreter::reset() {
  for (auto& c : caches_) c.rows.clear();
  conv_.clear();
  expected_pos_ = 0;
}

uint32_t Interpreter::step(uint32_t token, uint32_t position, std::vector<float>* logits) {
  if (position != expected_pos_) invalid("interpreter: positions must be consecutive (expected " + std::to_string(expected_pos_) + ")");
  if (position >= g_.max_context) fail(ErrorKind::Capacity, "interpreter: position beyond the model context");
  if (token >= vocab_) invalid("interpreter: token id outside the vocabulary");
  for (uint32_t i = 0; i < g_.nodes.size(); ++i) run_node(i, token, position);
  ++expected_pos_;
  const Value& out = vals_[g_.output];
  const std::vector<float>& l = out.r[0];
  if (logits) *logits = l;
  uint32_t best = 0;
  for (uint32_t i = 1; i < l.size(); ++i)
    if (l[i] > l[best]) best = i;
  return best;
}

void Interpreter::run_node(uint32_t idx, uint32_t token, uint32_t position) {
  const Node& n = g_.nodes[idx];
  Value& out = vals_[idx];
  out = Value{};
  auto in = [&](size_t k) -> const Value& { return vals_[n.inputs.at(k)]; };
  const std::string& op = n.op;
  const uint32_t tp = tp_;
  auto W = [&](const std::string& attr) -> const Tensor& { return w_.need(n.need(attr) + ".weight"); };
  // bring a value to bf16-valued form (f32 partials are rounded once)
  auto as_bf16 = [&](const Value& v, uint32_t rank) {
    std::vector<float> x = at(v, rank);
    if (v.f32)
      for (auto& e : x) e = bf16_round(e);
    return x;
  };
  // per-rank elementwise helper
  auto per_rank = [&](bool replicated, auto&& fn) {
    out.replicated = replicated;
    out.r.resize(replicated ? 1 : tp);
    for (uint32_t r = 0; r < out.r.size(); ++r) out.r[r] = fn(r);
  };

  if (op == "embedding") {
    const Tensor& t = W("weight");
    const uint32_t width = n.type.width;
    if (t.shape.size() != 2 || t.shape[1] != width || t.shape[0] != vocab_) invalid(n.name + ": embedding table shape mismatch");
    out.r = {std::vector<float>(t.data.begin() + (size_t)token * width, t.data.begin() + (size_t)(token + 1) * width)};
  } else if (op == "norm" || op == "optional_norm") {
    const Tensor* t = w_.find(n.need("weight") + ".weight");
    const Value& x = in(0);
    if (!t) {
      if (op == "optional_norm") { out = x; return; }
      invalid(n.name + ": missing norm weight");
    }
    const float eps = (float)n.num_attr("eps");
    const bool zc = n.has("zero_centered") && *n.attr("zero_centered") == "true";
    per_rank(x.replicated, [&](uint32_t r) { return rmsnorm(as_bf16(x, r), *t, eps, zc); });
  } else if (op == "linear") {
    const Value& x = in(0);
    const std::string& pl = n.need("placement");
    const uint32_t width = (uint32_t)n.int_attr("width");
    const Tensor& w0 = W("weight");
    const Tensor* w1 = n.has("paired_weight") ? &W("paired_weight") : nullptr;
    const uint32_t pwidth = w1 ? (n.has("paired_width") ? (uint32_t)n.int_attr("paired_width") : width) : 0;
    const bool keep_f32 = (int64_t)idx == logits_linear_;
    auto rnd = [&](float v) { return keep_f32 ? v : bf16_round(v); };
    out.f32 = keep_f32;
    if (pl == "replicated") {
      if (!x.replicated) invalid(n.name + ": replicated linear over a rank-local input");
      std::vector<float> xv = as_bf16(x, 0);
      const size_t K = xv.size();
      if (w0.shape != std::vector<uint64_t>{width, K}) invalid(n.name + ": weight shape mismatch");
      std::vector<float> y(width + pwidth);
      for (uint32_t j = 0; j < width; ++j) y[j] = rnd(dotf(&w0.data[(size_t)j * K], xv.data(), K));
      for (uint32_t j = 0; j < pwidth; ++j) y[width + j] = rnd(dotf(&w1->data[(size_t)j * K], xv.data(), K));
      out.r = {std::move(y)};
    } else if (pl == "tp_rows") {
      per_rank(false, [&](uint32_t r) {
        std::vector<float> xv = as_bf16(x, r);
        const size_t K = xv.size();
        if (w0.shape != std::vector<uint64_t>{(uint64_t)width * tp, K}) invalid(n.name + ": weight shape mismatch");
        std::vector<float> y(width + pwidth);
        for (uint32_t j = 0; j < width; ++j) y[j] = rnd(dotf(&w0.data[((size_t)r * width + j) * K], xv.data(), K));
        for (uint32_t j = 0; j < pwidth; ++j) y[width + j] = rnd(dotf(&w1->data[((size_t)r * pwidth + j) * K], xv.data(), K));
        return y;
      });
      if (tp == 1) out.replicated = true;
    } else {  // tp_columns: f32 partial per rank
      out.f32 = true;
      per_rank(false, [&](uint32_t r) {
        std::vector<float> xv = as_bf16(x, r);
        const size_t Kl = xv.size(), K = Kl * tp;
        if (w0.shape != std::vector<uint64_t>{width, K}) invalid(n.name + ": weight shape mismatch");
        std::vector<float> y(width);
        for (uint32_t j = 0; j < width; ++j) y[j] = dotf(&w0.data[(size_t)j * K + (size_t)r * Kl], xv.data(), Kl);
        return y;
      });
    }
  } else if (op == "allreduce") {
    const Value& x = in(0);
    std::vector<float> s(at(x, 0).size(), 0.f);
    for (uint32_t r = 0; r < tp; ++r) {
      const auto& v = at(x, r);
      for (size_t i = 0; i < s.size(); ++i) s[i] += v[i];
      if (x.replicated && tp > 1) invalid(n.name + ": allreduce of a replicated value");
    }
    out.f32 = true;
    out.r = {std::move(s)};
  } else if (op == "gather") {
    const Value& x = in(0);
    std::vector<float> s;
    for (uint32_t r = 0; r < tp; ++r) {
      const auto& v = at(x, r);
      s.insert(s.end(), v.begin(), v.end());
    }
    out.f32 = true;  // gathered values keep their precision (logits)
    out.r = {std::move(s)};
  } else if (op == "add") {
    const Value &a = in(0), &b = in(1);
    if (a.f32 && b.f32 && !a.replicated && !b.replicated) {
      out.f32 = true;
      per_rank(false, [&](uint32_t r) {
        std::vector<float> y = at(a, r);
        const auto& z = at(b, r);
        for (size_t i = 0; i < y.size(); ++i) y[i] += z[i];
        return y;
      });
    } else {
      per_rank(a.replicated && b.replicated, [&](uint32_t r) {
        std::vector<float> y = as_bf16(a, r), z = as_bf16(b, r);
        for (size_t i = 0; i < y.size(); ++i) y[i] = bf16_round(y[i] + z[i]);
        return y;
      });
    }
  } else if (op == "slice") {
    const Value& x = in(0);
    const size_t s = (size_t)n.int_attr("start"), w = (size_t)n.int_attr("width");
    out.f32 = x.f32;
    per_rank(x.replicated, [&](uint32_t r) { return std::vector<float>(at(x, r).begin() + s, at(x, r).begin() + s + w); });
  } else if (op == "concat") {
    const Value &a = in(0), &b = in(1);
    per_rank(a.replicated && b.replicated, [&](uint32_t r) {
      std::vector<float> y = as_bf16(a, r), z = as_bf16(b, r);
      y.insert(y.end(), z.begin(), z.end());
      return y;
    });
  } else if (op == "repeat") {
    const Value& x = in(0);
    const int64_t c = n.int_attr("count");
    per_rank(x.replicated, [&](uint32_t r) {
      std::vector<float> y;
      for (int64_t k = 0; k < c; ++k) y.insert(y.end(), at(x, r).begin(), at(x, r).end());
      return y;
    });
  } else if (op == "cast") {
    const Value& x = in(0);
    out.f32 = n.need("dtype") == "f32";
    per_rank(x.replicated, [&](uint32_t r) { return out.f32 ? at(x, r) : as_bf16(x, r); });
  } else if (op == "swiglu") {
    if (n.inputs.size() == 1) {
      const Value& x = in(0);
      per_rank(x.replicated, [&](uint32_t r) {
        std::vector<float> v = as_bf16(x, r);
        const size_t h = v.size() / 2;
        std::vector<float> y(h);
        for (size_t i = 0; i < h; ++i) y[i] = bf16_round(silu(v[i]) * v[h + i]);
        return y;
      });
    } else {
      const Value &a = in(0), &b = in(1);
      per_rank(a.replicated && b.replicated, [&](uint32_t r) {
        std::vector<float> gt = as_bf16(a, r), up = as_bf16(b, r);
        for (size_t i = 0; i < gt.size(); ++i) gt[i] = bf16_round(silu(gt[i]) * up[i]);
        return gt;
      });
    }
  } else if (op == "rope") {
    const Value& x = in(0);
    const float theta = (float)n.num_attr("theta");
    per_rank(x.replicated, [&](uint32_t r) {
      std::vector<float> y = as_bf16(x, r);
      rope_inplace(y.data(), (uint32_t)y.size(), position, theta);
      return y;
    });
  } else if (op == "rotary_prefix") {
    const Value& x = in(0);
    const uint32_t hd = (uint32_t)n.int_attr("head_dim"), rd = (uint32_t)n.int_attr("rotary_dim");
    const float theta = (float)n.num_attr("theta");
    per_rank(x.replicated, [&](uint32_t r) {
      std::vector<float> y = as_bf16(x, r);
      for (size_t h = 0; h + hd <= y.size(); h += hd) rope_inplace(&y[h], rd, position, theta);
      return y;
    });
  } else if (op == "mome") {
    // causal depthwise conv over the token stream with residual: y = x + [count >= taps-1] * sum_k s_k w_k
    const Value& x = in(0);
    const uint32_t taps = (uint32_t)n.int_attr("taps");
    const Tensor& w = W("weight");  // [channels_total, 1, taps]
    ConvState& st = conv_[idx];
    const bool sharded = n.has("placement") && *n.attr("placement") == "tp_channels";
    const uint32_t ranks = x.replicated ? 1 : tp;
    if (st.hist.empty()) st.hist.assign(ranks, {});
    per_rank(x.replicated, [&](uint32_t r) {
      std::vector<float> xv = as_bf16(x, r);
      const size_t C = xv.size();
      auto& h = st.hist[r];
      if (h.empty()) h.assign((size_t)(taps - 1) * C, 0.f);
      const size_t cbase = sharded ? (size_t)r * C : 0;
      std::vector<float> y(C);
      for (size_t c = 0; c < C; ++c) {
        float conv = xv[c] * w.data[(cbase + c) * taps + taps - 1];
        for (uint32_t k = 0; k + 1 < taps; ++k) conv += h[k * C + c] * w.data[(cbase + c) * taps + k];
        y[c] = bf16_round(xv[c] + (st.count + 1 >= taps ? conv : 0.f));
      }
      for (uint32_t k = 0; k + 2 < taps; ++k) std::copy(h.begin() + (k + 1) * C, h.begin() + (k + 2) * C, h.begin() + k * C);
      std::copy(xv.begin(), xv.end(), h.begin() + (size_t)(taps - 2) * C);
      return y;
    });
    if (n.inputs.size()) {
      // the count advances once per token, after all ranks ran
      st.count++;
    }
  } else if (op == "mhc_pre" || op == "mhc_merge") {
    const Value& x = in(0);
    const uint32_t S = (uint32_t)n.int_attr("streams"), iters = (uint32_t)n.int_attr("sinkhorn");
    const float eps = (float)n.num_attr("eps");
    std::vector<float> X = as_bf16(x, 0);
    const size_t Wd = X.size() / S, total = X.size();
    const std::string base = n.need("weight");
    const Tensor& phi = w_.need(base + ".phi");      // [S*S + 2S, S*W]
    const Tensor& gamma = w_.need(base + ".gamma");  // [S*W]
    const Tensor& alpha = w_.need(base + ".alpha");  // [3]
    const Tensor& beta = w_.need(base + ".beta");    // [S*S + 2S]
    const size_t M = (size_t)S * S + 2 * S;
    double ss = 0;
    for (float v : X) ss += (double)v * v;
    const float inv = 1.f / std::sqrt((float)(ss / total) + eps);
    std::vector<float> m(M);
    for (size_t j = 0; j < M; ++j) {
      float s = 0.f;
      for (size_t c = 0; c < total; ++c) s += phi.data[j * total + c] * gamma.data[c] * X[c];
      m[j] = inv * s;
    }
    auto sig = [](float v) { return 1.f / (1.f + std::exp(-v)); };
    std::vector<float> pre(S), post(S), R((size_t)S * S);
    for (uint32_t j = 0; j < S; ++j) pre[j] = sig(m[j] * alpha.data[0] + beta.data[j]) + 1e-6f;
    for (uint32_t j = 0; j < S; ++j) post[j] = 2.f * sig(m[S + j] * alpha.data[1] + beta.data[S + j]);
    for (size_t j = 0; j < (size_t)S * S; ++j) R[j] = m[2 * S + j] * alpha.data[2] + beta.data[2 * S + j];
    // Sinkhorn: row softmax, then alternate column / row normalisation
    for (uint32_t a = 0; a < S; ++a) {
      float mx = -INFINITY, sum = 0.f;
      for (uint32_t b = 0; b < S; ++b) mx = std::max(mx, R[a * S + b]);
      for (uint32_t b = 0; b < S; ++b) sum += (R[a * S + b] = std::exp(R[a * S + b] - mx));
      for (uint32_t b = 0; b < S; ++b) R[a * S + b] = R[a * S + b] / sum + 1e-6f;
    }
    auto col_norm = [&] {
      for (uint32_t b = 0; b < S; ++b) {
        float sum = 0.f;
        for (uint32_t a = 0; a < S; ++a) sum += R[a * S + b];
        for (uint32_t a = 0; a < S; ++a) R[a * S + b] /= (sum + 1e-6f);
      }
    };
    auto row_norm = [&] {
      for (uint32_t a = 0; a < S; ++a) {
        float sum = 0.f;
        for (uint32_t b = 0; b < S; ++b) sum += R[a * S + b];
        for (uint32_t b = 0; b < S; ++b) R[a * S + b] /= (sum + 1e-6f);
      }
    };
    col_norm();
    for (uint32_t it = 1; it < iters; ++it) {
      row_norm();
      col_norm();
    }
    std::vector<float> y(Wd, 0.f);
    for (uint32_t s = 0; s < S; ++s)
      for (size_t c = 0; c < Wd; ++c) y[c] += pre[s] * X[s * Wd + c];
    for (auto& v : y) v = bf16_round(v);
    out.r = {std::move(y)};
    out.hc_x = std::move(X);
    out.hc_post = std::move(post);
    out.hc_comb = std::move(R);
  } else if (op == "mhc_input") {
    out.r = in(0).r;
  } else if (op == "mhc_post") {
    const Value& hc = in(0);
    std::vector<float> br = as_bf16(in(1), 0);
    const size_t Wd = br.size(), S = hc.hc_post.size();
    std::vector<float> y(S * Wd);
    for (size_t i = 0; i < S; ++i)
      for (size_t c = 0; c < Wd; ++c) {
        float v = hc.hc_post[i] * br[c];
        for (size_t k = 0; k < S; ++k) v += hc.hc_comb[k * S + i] * hc.hc_x[k * Wd + c];
        y[i * Wd + c] = bf16_round(v);
      }
    out.r = {std::move(y)};
  } else if (op == "cache_norm_rope_append" || op == "cache_append") {
    CacheState& c = caches_[cache_of_node_.at(idx)];
    std::vector<float> row;
    if (op == "cache_norm_rope_append") {
      std::vector<float> lat = rmsnorm(as_bf16(in(0), 0), W("weight"), (float)n.num_attr("eps"), false);
      std::vector<float> kr = as_bf16(in(1), 0);
      rope_inplace(kr.data(), (uint32_t)kr.size(), position, (float)n.num_attr("theta"));
      if (n.has("cache_dtype") && n.need("cache_dtype") == "int8_ds_mla") {
        // packed int8 latent: one f32 scale per tile of 128 columns (max|v| / 127, 1 for an all-zero tile), values rounded half
        // away from zero and clamped to +-127; the rotary columns stay bf16. The row holds what attention will read back.
        for (size_t t0 = 0; t0 < lat.size(); t0 += 128) {
          const size_t t1 = std::min(lat.size(), t0 + 128);
          float amax = 0.f;
          for (size_t i = t0; i < t1; ++i) amax = std::max(amax, std::fabs(lat[i]));
          const float scale = amax > 0.f ? amax / 127.f : 1.f;
          for (size_t i = t0; i < t1; ++i) {
            const float q = lat[i] / scale;
            const int r = (int)(q >= 0.f ? q + 0.5f : q - 0.5f);
            lat[i] = (float)std::max(-127, std::min(127, r)) * scale;
          }
        }
      }
      row = lat;
      row.insert(row.end(), kr.begin(), kr.end());
      if (n.inputs.size() == 3 && c.sinks.empty()) {
        const auto& s = at(in(2), 0);
        for (size_t o = 0; o + row.size() <= s.size(); o += row.size()) c.sinks.emplace_back(s.begin() + o, s.begin() + o + row.size());
      }
    } else {
      row = as_bf16(in(0), 0);
    }
    if (c.rows.size() != position) invalid(n.name + ": cache rows out of step with positions");
    c.rows.push_back(std::move(row));
    out.cache = cache_of_node_.at(idx);
  } else if (op == "index_cache_append") {
    // one index key per position; an int8 index cache keeps rint(x / s) * s with one scale per row (s = max|x| / 127, the
    // scale itself held in half precision), which is what the selector later scores against
    CacheState& c = caches_[cache_of_node_.at(idx)];
    std::vector<float> row = as_bf16(in(0), 0);
    if (n.has("cache_dtype") && n.need("cache_dtype") == "int8") quantize_row_int8(row.data(), row.size());
    if (c.rows.size() != position) invalid(n.name + ": index cache rows out of step with positions");
    c.rows.push_back(std::move(row));
    out.cache = cache_of_node_.at(idx);
  } else if (op == "sparse_index") {
    // score(p) = sum_h w_h * relu(q_h . key_p) over the causal positions; the `topk` best positions (ties to the earlier
    // one), reported in ascending order. With an int8 index cache the query heads are quantised row-wise like the keys.
    const uint32_t H = (uint32_t)n.int_attr("heads"), D = (uint32_t)n.int_attr("head_dim"), K = (uint32_t)n.int_attr("topk");
    std::vector<float> q = as_bf16(in(0), 0), w = as_bf16(in(1), 0);
    const CacheState& c = caches_[in(2).cache];
    const Node& cn = g_.nodes[n.inputs[2]];
    if (cn.has("cache_dtype") && cn.need("cache_dtype") == "int8")
      for (uint32_t h = 0; h < H; ++h) quantize_row_int8(&q[(size_t)h * D], D);
    if (c.rows.size() != position + 1) invalid(n.name + ": the index cache must hold the current position before it is searched");
    std::vector<std::pair<float, uint32_t>> scored(position + 1);
    for (uint32_t p = 0; p <= position; ++p) {
      float sc = 0.f;
      for (uint32_t h = 0; h < H; ++h) sc += w[h] * std::max(0.f, dotf(&q[(size_t)h * D], c.rows[p].data(), D));
      scored[p] = {sc, p};
    }
    const size_t keep = std::min<size_t>(K, scored.size());
    std::partial_sort(scored.begin(), scored.begin() + keep, scored.end(),
                      [](const auto& a, const auto& b) { return a.first != b.first ? a.first > b.first : a.second < b.second; });
    out.ids.clear();
    for (size_t i = 0; i < keep; ++i) out.ids.push_back(scored[i].second);
    std::sort(out.ids.begin(), out.ids.end());
  } else if (op == "sink_normalize") {
    const std::string base = n.need("weight");
    const Tensor& kv = w_.need(base + ".param_sink_compressed_kv");
    const Tensor& pe = w_.need(base + ".param_sink_k_pe");
    const Tensor& nw = w_.need(n.need("norm") + ".weight");
    const uint32_t count = (uint32_t)n.int_attr("count"), lat = (uint32_t)n.int_attr("latent"), rp = (uint32_t)n.int_attr("rope");
    std::vector<float> y;
    for (uint32_t s = 0; s < count; ++s) {
      std::vector<float> l(kv.data.begin() + (size_t)s * lat, kv.data.begin() + (size_t)(s + 1) * lat);
      auto ln = rmsnorm(l, nw, (float)n.num_attr("eps"), false);
      y.insert(y.end(), ln.begin(), ln.end());
      y.insert(y.end(), pe.data.begin() + (size_t)s * rp, pe.data.begin() + (size_t)(s + 1) * rp);
    }
    out.r = {std::move(y)};
  } else if (op == "mla_query") {
    const Value& q = in(0);
    const uint32_t H = (uint32_t)n.int_attr("heads"), np = (uint32_t)n.int_attr("nope"), rp = (uint32_t)n.int_attr("rope"), lat = (uint32_t)n.int_attr("latent");
    const uint32_t vd = n.has("value") ? (uint32_t)n.int_attr("value") : np;
    const uint32_t hl = H / tp;
    const Tensor& kvb = W("weight");  // [H*(np+vd), lat]
    if (kvb.shape != std::vector<uint64_t>{(uint64_t)H * (np + vd), lat}) invalid(n.name + ": kv_b shape mismatch");
    const float theta = (float)n.num_attr("theta");
    const bool local = n.has("input_layout") && *n.attr("input_layout") == "rank_local";
    per_rank(false, [&](uint32_t r) {
      std::vector<float> qv = as_bf16(q, r);
      std::vector<float> y((size_t)hl * (lat + rp));
      for (uint32_t j = 0; j < hl; ++j) {
        const uint32_t h = r * hl + j;
        const float* qh = &qv[(size_t)(local ? j : h) * (np + rp)];
        for (uint32_t c = 0; c < lat; ++c) {
          float s = 0.f;
          for (uint32_t d = 0; d < np; ++d) s += qh[d] * kvb.data[((size_t)h * (np + vd) + d) * lat + c];
          y[(size_t)j * (lat + rp) + c] = bf16_round(s);
        }
        float* ro = &y[(size_t)j * (lat + rp) + lat];
        std::copy(qh + np, qh + np + rp, ro);
        rope_inplace(ro, rp, position, theta);
      }
      return y;
    });
    if (tp == 1) out.replicated = true;
  } else if (op == "latent_attention") {
    const Value& q = in(0);
    const CacheState& c = caches_[in(1).cache];
    const uint32_t roww = c.width, rp = g_.nodes[n.inputs[1]].type.aux, lat = roww - rp;
    const float scale = 1.f / std::sqrt((float)n.int_attr("scale_dim"));
    const int64_t window = n.int_attr("window");
    const bool learned = n.need("selection") == "learned_indices";
    const size_t lo = window > 0 && (int64_t)position + 1 > window ? position + 1 - (size_t)window : 0;
    // learned selection: the positions the indexer chose (always causal), further limited by the window when there is one
    std::vector<uint32_t> chosen;
    if (learned)
      for (uint32_t p : in(2).ids)
        if (p >= lo && p <= position) chosen.push_back(p);
    per_rank(q.replicated, [&](uint32_t r) {
      std::vector<float> qv = as_bf16(q, r);
      const size_t hl = qv.size() / roww;
      std::vector<float> y(hl * lat);
      std::vector<const std::vector<float>*> keys;
      for (auto& s : c.sinks) keys.push_back(&s);
      if (learned)
        for (uint32_t p : chosen) keys.push_back(&c.rows[p]);
      else
        for (size_t p = lo; p <= position; ++p) keys.push_back(&c.rows[p]);
      std::vector<float> sc(keys.size());
      for (size_t h = 0; h < hl; ++h) {
        float mx = -INFINITY;
        for (size_t k = 0; k < keys.size(); ++k) mx = std::max(mx, sc[k] = dotf(&qv[h * roww], keys[k]->data(), roww) * scale);
        float sum = 0.f;
        for (auto& s : sc) sum += (s = std::exp(s - mx));
        for (uint32_t cidx = 0; cidx < lat; ++cidx) {
          float a = 0.f;
          for (size_t k = 0; k < keys.size(); ++k) a += sc[k] * (*keys[k])[cidx];
          y[h * lat + cidx] = keys.empty() ? 0.f : bf16_round(a / sum);     // a selection the window leaves empty attends to nothing
        }
      }
      return y;
    });
  } else if (op == "mla_value") {
    const Value& x = in(0);
    const uint32_t H = (uint32_t)n.int_attr("heads"), lat = (uint32_t)n.int_attr("latent"), vd = (uint32_t)n.int_attr("value");
    const uint32_t np = n.has("nope") ? (uint32_t)n.int_attr("nope") : vd;
    const uint32_t hl = H / tp;
    const Tensor& kvb = W("weight");
    per_rank(x.replicated && tp == 1, [&](uint32_t r) {
      std::vector<float> xv = as_bf16(x, r);
      std::vector<float> y((size_t)hl * vd);
      for (uint32_t j = 0; j < hl; ++j) {
        const uint32_t h = r * hl + j;
        for (uint32_t v = 0; v < vd; ++v) y[(size_t)j * vd + v] = bf16_round(dotf(&kvb.data[((size_t)h * (np + vd) + np + v) * lat], &xv[(size_t)j * lat], lat));
      }
      return y;
    });
  } else if (op == "router") {
    std::vector<float> x = as_bf16(in(0), 0);
    const Tensor& w = W("weight");
    const uint32_t E = (uint32_t)n.int_attr("experts"), K = (uint32_t)n.int_attr("topk");
    if (w.shape != std::vector<uint64_t>{E, x.size()}) invalid(n.name + ": router weight shape mismatch");
    std::vector<float> logit(E), raw(E), sel(E);
    for (uint32_t e = 0; e < E; ++e) logit[e] = dotf(&w.data[(size_t)e * x.size()], x.data(), x.size());
    const bool softmax = n.need("scoring") == "softmax";
    if (softmax) {
      float mx = *std::max_element(logit.begin(), logit.end()), sum = 0.f;
      for (uint32_t e = 0; e < E; ++e) sum += (raw[e] = std::exp(logit[e] - mx));
      for (uint32_t e = 0; e < E; ++e) sel[e] = raw[e] = raw[e] / sum;
    } else {
      const Tensor* bias = w_.find(n.need("weight") + ".e_score_correction_bias");
      for (uint32_t e = 0; e < E; ++e) {
        raw[e] = 1.f / (1.f + std::exp(-logit[e]));
        sel[e] = raw[e] + (bias ? bias->data[e] : 0.f);
      }
    }
    float wsum = 0.f;
    for (uint32_t k = 0; k < K; ++k) {
      uint32_t best = 0;
      for (uint32_t e = 1; e < E; ++e)
        if (sel[e] > sel[best]) best = e;
      out.ids.push_back(best);
      out.wts.push_back(raw[best]);
      wsum += raw[best];
      sel[best] = -INFINITY;
    }
    const float scale = (float)n.num_attr("scale");
    const bool renorm = !n.has("renorm") || *n.attr("renorm") != "false";
    for (auto& v : out.wts) v = (softmax ? (renorm ? v / wsum : v) : v / (wsum + 1e-20f)) * scale;
  } else if (op == "expert_linear") {
    std::vector<float> x = as_bf16(in(0), 0);
    const Value& routes = in(1);
    const uint32_t E = g_.nodes[n.inputs[1]].type.aux, el = E / tp, F = (uint32_t)n.int_attr("width");
    out.replicated = false;
    out.rows.assign(tp, std::vector<std::vector<float>>(routes.ids.size()));
    for (size_t k = 0; k < routes.ids.size(); ++k) {
      const uint32_t e = routes.ids[k], r = e / el;
      const Tensor& g0 = w_.need(expert_name(n.need("weight"), e) + ".weight");
      std::vector<float> y;
      for (uint32_t j = 0; j < F; ++j) y.push_back(bf16_round(dotf(&g0.data[(size_t)j * x.size()], x.data(), x.size())));
      if (n.has("paired_weight")) {
        const Tensor& u0 = w_.need(expert_name(n.need("paired_weight"), e) + ".weight");
        for (uint32_t j = 0; j < F; ++j) y.push_back(bf16_round(dotf(&u0.data[(size_t)j * x.size()], x.data(), x.size())));
      }
      out.rows[r][k] = std::move(y);
    }
  } else if (op == "expert_swiglu_down") {
    const Value& gu = in(0);
    const Value& routes = in(n.inputs.size() - 1);
    const uint32_t D = (uint32_t)n.int_attr("width");
    out.replicated = false;
    out.f32 = true;
    out.rows.assign(tp, std::vector<std::vector<float>>(routes.ids.size()));
    for (uint32_t r = 0; r < tp; ++r)
      for (size_t k = 0; k < routes.ids.size(); ++k) {
        const auto& row = gu.rows[r][k];
        if (row.empty()) continue;
        std::vector<float> act;
        if (n.inputs.size() == 3) {
          const auto& up = in(1).rows[r][k];
          for (size_t i = 0; i < row.size(); ++i) act.push_back(bf16_round(silu(row[i]) * up[i]));
        } else {
          const size_t F = row.size() / 2;
          for (size_t i = 0; i < F; ++i) act.push_back(bf16_round(silu(row[i]) * row[F + i]));
        }
        const Tensor& wd = w_.need(expert_name(n.need("weight"), routes.ids[k]) + ".weight");
        if (wd.shape != std::vector<uint64_t>{D, act.size()}) invalid(n.name + ": expert down weight shape mismatch");
        std::vector<float> y(D);
        for (uint32_t j = 0; j < D; ++j) y[j] = dotf(&wd.data[(size_t)j * act.size()], act.data(), act.size());
        out.rows[r][k] = std::move(y);
      }
  } else if (op == "expert_reduce") {
    const Value& ex = in(0);
    const Value& routes = in(1);
    out.f32 = true;
    per_rank(false, [&](uint32_t r) {
      std::vector<float> y(n.type.width, 0.f);
      for (size_t k = 0; k < routes.ids.size(); ++k) {
        const auto& row = ex.rows[r][k];
        if (row.empty()) continue;
        for (size_t i = 0; i < y.size(); ++i) y[i] += routes.wts[k] * row[i];
      }
      return y;
    });
  } else if (op == "kv_cache_append") {
    CacheState& c = caches_[cache_of_node_.at(idx)];
    // rows are kept per rank: [k | v] of the rank's kv heads
    const Value &k = in(0), &v = in(1);
    const uint32_t ranks = k.replicated ? 1 : tp;
    std::vector<float> row;
    for (uint32_t r = 0; r < ranks; ++r) {
      auto kk = as_bf16(k, r), vv = as_bf16(v, r);
      row.insert(row.end(), kk.begin(), kk.end());
      row.insert(row.end(), vv.begin(), vv.end());
    }
    if (c.rows.size() != position) invalid(n.name + ": cache rows out of step with positions");
    c.rows.push_back(std::move(row));
    out.cache = cache_of_node_.at(idx);
  } else if (op == "paged_attention") {
    const Value& q = in(0);
    const CacheState& c = caches_[in(1).cache];
    const uint32_t H = (uint32_t)n.int_attr("heads"), KVH = (uint32_t)n.int_attr("kv_heads"), hd = (uint32_t)n.int_attr("head_dim");
    const float scale = (float)n.num_attr("scale");
    const int64_t window = n.has("window") ? n.int_attr("window") : 0;
    const size_t lo = window > 0 && (int64_t)position + 1 > window ? position + 1 - (size_t)window : 0;
    const uint32_t hl = H / tp, kvl = std::max(1u, KVH / tp), per_rank_row = 2 * kvl * hd;
    const bool kv_per_rank = c.rows[0].size() == (size_t)per_rank_row * tp && tp > 1;
    per_rank(q.replicated && tp == 1, [&](uint32_t r) {
      std::vector<float> qv = as_bf16(q, r);
      std::vector<float> y((size_t)hl * hd);
      const size_t base = kv_per_rank ? (size_t)r * per_rank_row : 0;
      for (uint32_t j = 0; j < hl; ++j) {
        const uint32_t kvh = j / (hl / kvl);
        std::vector<float> sc;
        float mx = -INFINITY;
        for (size_t p = lo; p <= position; ++p) {
          float s = dotf(&qv[(size_t)j * hd], &c.rows[p][base + (size_t)kvh * hd], hd) * scale;
          sc.push_back(s);
          mx = std::max(mx, s);
        }
        float sum = 0.f;
        for (auto& s : sc) sum += (s = std::exp(s - mx));
        for (uint32_t d = 0; d < hd; ++d) {
          float a = 0.f;
          for (size_t p = lo; p <= position; ++p) a += sc[p - lo] * c.rows[p][base + (size_t)(kvl + kvh) * hd + d];
          y[(size_t)j * hd + d] = bf16_round(a / sum);
        }
      }
      return y;
    });
  } else if (op == "quantize") {
    // symmetric per-token int8 simulated in f32: q = rint(x / s) * s with s = max|x| / 127
    const Value& x = in(0);
    per_rank(x.replicated, [&](uint32_t r) {
      std::vector<float> v = as_bf16(x, r);
      float mx = 0.f;
      for (float e : v) mx = std::max(mx, std::fabs(e));
      const float s = mx > 0 ? mx / 127.f : 1.f;
      for (auto& e : v) e = std::nearbyint(e / s) * s;
      return v;
    });
    out.f32 = true;
  } else {
    fail(ErrorKind::NotImplemented, "interpreter: primitive " + op + " (node " + n.name + ")");
  }
}

}  // namespace ifab::interp
