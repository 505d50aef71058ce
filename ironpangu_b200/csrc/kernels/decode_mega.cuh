// One persistent kernel per decode step of the MLA + MoE decoder.
//
// A decode step of this model is ~460 small dependent operators. Launched one by one (even from a CUDA
// graph with programmatic dependent launch) every operator pays a launch gap, a drain and a cold ramp of
// its weight stream: about 5 us each, 2.3 ms per token, no matter how many GPUs share the weights. This
// kernel runs the whole step as ONE cooperative launch of 2 CTAs per SM: the operators become phases
// separated by a grid-wide barrier (an arrive counter in L2 polled by one thread per CTA), all weights
// are streamed with the same 16-loads-in-flight GEMV core, and both all-reduces of a layer run inside
// their producing phase with the tagged 8-byte-store protocol of oneshot_ar.cuh.
//
// Phases per layer (each ends with a grid barrier):
//   1 qkv_a      RMSNorm(x) @ W_qkv_a                         -> qkv            [T, q_lora + 576]
//   2 q_b        RMSNorm(q_a) @ W_q_b                         -> q              [T, hl * 192]
//     kv_write   RMSNorm(latent), RoPE(k_pe) -> paged cache    (CTAs 0..T-1, same phase)
//   3 absorb     q_nope @ W_uk, RoPE(q_pe)                    -> q_lat          [T, hl, 576]
//   4 split      split-KV attention over the latent cache     -> scratch        [T, hl, splits, 514]
//   5 merge/v_up LSE merge, o_lat @ W_uv                      -> attn           [T, hl * 128]
//   6 o_proj     attn @ W_o, all-reduce, + x                  -> x
//   7 router     RMSNorm(x) @ W_router (f32)                  -> logits         [T, E]
//   8 gate/up    top-k (every CTA), SwiGLU of the local routes and of the shared shard -> act
//   9 down       score-weighted down projections, all-reduce, + x -> x
// then the vocabulary-sharded head with the greedy (value, index) exchange, and optionally the feedback
// of the sampled token into the next step's inputs.
//
// Every wait is bounded: a barrier or peer wait that runs out sets a status bit and an abort word that
// every other wait polls, after which all CTAs leave the kernel; the barrier state repairs itself at the
// end of every launch (the last CTA to leave re-bases it), so the next launch starts clean.
// Reference: the captured decode graph of token::Decoder (native/src/token_executor.h:1323-1448) replays
// the same operator list as separate device launches.
#pragma once
#include "gemv.cuh"
#include "mla_common.cuh"
#include "ifab_kernels.h"

namespace ifab::mega {

using namespace ifab::mla;

constexpr int THREADS = 256, WARPS = 8;
constexpr int MD = 16;                     // 16-byte weight loads a lane keeps in flight per batch (see gemv.cuh)
constexpr int MAX_TOPK = 16;
constexpr int MAX_ROUTES = 8 * MAX_TOPK;   // T * topk
constexpr int AR_ROWS = 8;                 // output rows one warp may own in an all-reduce phase

struct Layer {   // same layout as IfabMlaMoeLayer
  const bf16 *attn_norm, *qkv_a, *kv_a_norm, *q_a_norm, *q_b, *kv_b, *o_proj, *ffn_norm;
  const float *router, *router_bias;
  const bf16 *gate_up, *down, *shared_gate_up, *shared_down;
  bf16* cache;
  const bf16* sinks;
};

struct Params {
  const Layer* layers;
  int n_layers, D, hl, q_lora, nope, rope, vdim, E, el, e0, topk, F, Fs, vl, vocab_offset, vocab;
  int scoring, renorm, window, n_sinks, page_tokens, max_pages, num_pages, kps, max_splits;
  float route_scale, eps, theta, attn_scale;
  const bf16 *embed, *final_norm, *lm_head;
  int32_t *tokens, *positions;
  const int32_t *slots, *page_table;
  bf16 *x, *qkv, *q, *q_lat, *attn, *act;
  float *scratch, *router_logits;
  int32_t* route_ids;
  float* route_w;
  float2* partial;
  int32_t* next_ids;
  float *next_vals, *logits;
  uint32_t* bar;        // [0] arrivals  [1] base of this launch  [2] exit tickets  [3] abort
  unsigned long long* trace;   // optional: CTA 0 stores the global timer (ns) at kernel entry and after every barrier
  int T_live, feedback;
  FabricView fv;
  uint64_t* seq;
  uint32_t spin_limit;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Grid-wide barrier state of one CTA. `count` advances identically in every thread of every CTA.
struct GridBar {
  unsigned long long* trace;
  uint32_t* bar;
  uint32_t base, count, nblocks, limit;
  uint32_t* status;
  int* s_ok;   // shared: 1 while the launch is healthy
};

// true when every CTA arrived; false when the launch was aborted (timeout here or elsewhere)
__device__ __forceinline__ bool grid_sync(GridBar& g) {
  g.count += 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    red_release_gpu_add(g.bar, 1u);
    const uint32_t target = g.base + g.count * g.nblocks;
    bool ok = false;
    for (uint32_t i = 0; i < g.limit; ++i) {
      if ((int32_t)(ld_acquire_gpu(g.bar) - target) >= 0) { ok = true; break; }
      if ((i & 63) == 63 && ld_volatile_u32(g.bar + 3) != 0) break;
    }
    if (!ok) {
      if (ld_volatile_u32(g.bar + 3) == 0) atomicOr(g.status, IFAB_STATUS_PEER_TIMEOUT);
      atomicExch(g.bar + 3, 1u);
      *g.s_ok = 0;
    }
  }
  __syncthreads();
  if (g.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) g.trace[g.count] = global_timer_ns();
  return *g.s_ok != 0;
}

// 16-byte load that always goes to L2: activations are written by other CTAs of this very kernel
__device__ __forceinline__ uint4 ld_act16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float ld_act_bf16(const bf16* p) {
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __uint_as_float((uint32_t)u << 16);
}

// Stage t_live rows (K columns, row stride ld) into shared memory as bf16, RMS-normalised when norm_w is given.
// Rows >= t_live are zero filled. All threads; ends with __syncthreads().
template <int T>
__device__ __forceinline__ void stage_act(bf16* xs, const bf16* x, long ld, int t_live, int K, const bf16* norm_w, float eps,
                                          float* red /* T*33 floats */) {
  const int tid = threadIdx.x;
  const int chunks = K >> 3;
  for (int t = 0; t < T; ++t) {
    const bool live = t < t_live;
    for (int c = tid; c < chunks; c += THREADS)
      *reinterpret_cast<uint4*>(xs + t * K + c * 8) = live ? ld_act16(x + (long)t * ld + c * 8) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  if (norm_w == nullptr) return;
  const int warp = tid >> 5, lane = tid & 31;
  for (int t = 0; t < T; ++t) {
    float ss = 0.f;
    for (int c = tid; c < chunks; c += THREADS) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(xs + t * K + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    if (lane == 0) red[t * 33 + warp] = ss;
  }
  __syncthreads();
  if (tid < T) {
    float s = 0.f;
    for (int w = 0; w < WARPS; ++w) s += red[tid * 33 + w];
    red[tid * 33 + 32] = rsqrtf(s / (float)K + eps);
  }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const float inv = red[t * 33 + 32];
    for (int c = tid; c < chunks; c += THREADS) {
      float f[8], g[8];
      unpack8(*reinterpret_cast<const uint4*>(xs + t * K + c * 8), f);
      unpack8(*reinterpret_cast<const uint4*>(norm_w + c * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i];
      *reinterpret_cast<uint4*>(xs + t * K + c * 8) = pack8(f);
    }
  }
  __syncthreads();
}

// y[t][r] = dot(W[r, :], xs[t, :]) for the rows this warp owns (units of R rows, interleaved over all warps of the
// grid so that neighbouring warps stream neighbouring rows). epi(first_row, acc) runs on every lane with full sums.
// `first` holds the first weight batch of this warp's first unit when the caller issued it ahead of time
// (prefetch_first, before the grid barrier that publishes the activations: weights never change, so their loads may
// overlap the barrier and the staging of the activations).
template <int T, int R, class Epi>
__device__ __forceinline__ void gemv_phase(const bf16* W, int rows, int K, const bf16* xs, int gw, int GW, RowBatch<R, MD>& first,
                                           bool have_first, Epi epi) {
  const int units = (rows + R - 1) / R;
  for (int u = gw; u < units; u += GW) {
    const bf16* wrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wrow[r] = (u * R + r < rows) ? W + (size_t)(u * R + r) * K : nullptr;
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    if (have_first && u == gw) warp_rows_dot<T, R, MD>(wrow, xs, K, acc, first);
    else warp_rows_dot<T, R, MD>(wrow, xs, K, acc);
    warp_reduce_acc<T, R>(acc);
    epi(u * R, acc);
  }
}

template <int T, int R, class Epi>
__device__ __forceinline__ void gemv_phase(const bf16* W, int rows, int K, const bf16* xs, int gw, int GW, Epi epi) {
  RowBatch<R, MD> none;
  gemv_phase<T, R>(W, rows, K, xs, gw, GW, none, false, epi);
}

// issue the first weight batch of unit `gw` (rows gw*R .. gw*R+R-1) of a GEMV phase
template <int R>
__device__ __forceinline__ void prefetch_first(const bf16* W, int rows, int K, int gw, RowBatch<R, MD>& pf) {
  const bf16* wrow[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wrow[r] = (gw * R + r < rows) ? W + (size_t)(gw * R + r) * K : nullptr;
  prefetch_rows<R, MD>(wrow, K, pf);
}

// ---- all-reduce of row partials (tagged 8-byte stores, see oneshot_ar.cuh) ------------------------------------
struct ArCtx {
  FabricView fv;
  uint64_t epoch;
  uint32_t* status;
  uint32_t* abort_word;
};

// push one partial value of (row t, column col) of an [t_live x N] result to every peer
__device__ __forceinline__ void ar_push(const ArCtx& a, int t, int t_live, int col, int N, float v) {
  const uint32_t par = (uint32_t)(a.epoch & 1), tag = (uint32_t)a.epoch;
  const uint64_t word = ((uint64_t)tag << 32) | (uint64_t)__float_as_uint(v);
  for (int q = 0; q < a.fv.world; ++q) {
    if (q == a.fv.rank) continue;
    uint64_t* dst = reinterpret_cast<uint64_t*>(a.fv.data[q] + a.fv.ll_offset + (size_t)par * a.fv.ll_half_bytes) +
                    ((size_t)a.fv.rank * t_live + t) * N + col;
    st_relaxed_sys(dst, word);
  }
}
// rank-ordered sum of own + peers' partials; *ok is cleared when a peer did not deliver in time
__device__ __forceinline__ float ar_collect(const ArCtx& a, int t, int t_live, int col, int N, float own, bool* ok) {
  const uint32_t par = (uint32_t)(a.epoch & 1), tag = (uint32_t)a.epoch;
  const uint64_t* src = reinterpret_cast<const uint64_t*>(a.fv.data[a.fv.rank] + a.fv.ll_offset + (size_t)par * a.fv.ll_half_bytes);
  float v = 0.f;
  for (int q = 0; q < a.fv.world; ++q) {
    if (q == a.fv.rank) { v += own; continue; }
    const uint64_t* slot = src + ((size_t)q * t_live + t) * N + col;
    uint64_t got = 0;
    bool hit = false;
    for (uint32_t spin = 0; spin < a.fv.spin_limit; ++spin) {
      got = ld_relaxed_sys(slot);
      if ((uint32_t)(got >> 32) == tag) { hit = true; break; }
      if ((spin & 255) == 255 && ld_volatile_u32(a.abort_word) != 0) break;
    }
    if (!hit) {
      if (ld_volatile_u32(a.abort_word) == 0) atomicOr(a.status, IFAB_STATUS_PEER_TIMEOUT);
      atomicExch(a.abort_word, 1u);
      *ok = false;
      return v;
    }
    v += __uint_as_float((uint32_t)got);
  }
  return v;
}

}  // namespace ifab::mega
