// The whole MoE half of a decode layer as ONE launch (one or two token rows):
//
//   router projection + top-k  ||  shared-expert gate/up      (independent of each other)
//   routed gate/up of the local experts                        (needs the routes)
//   down projections, score-weighted sum, one-shot all-reduce  (needs every activation)
//
// A decode step at 8 GPUs is bound by the fixed cost of every dependent kernel (launch, drain, staging of the
// row, first-load latency: about 5 us each on a B200), not by bytes: a rank streams ~40 MB per layer. The
// separate router, gate/up and down kernels pay that cost three times and the router's 16 KB per expert cannot
// hide anything. Here the grid is sized to be co-resident (at most two CTAs per SM) and the three steps are
// separated by two in-grid signals instead of kernel boundaries:
//   * routes: each router CTA stores its logit and the launch number as ONE 8-byte word; every CTA works on the shared
//     expert meanwhile, then collects the E words (bounded polling, all requested at once) and selects the top-k itself -
//     no ticket, no "last CTA", no second signal, so the routes cost one trip to L2 after the slowest router CTA;
//   * activations: an arrive counter (release add, nothing returned) that the down CTAs poll; the first
//     down-projection weights of a CTA are already in registers when it waits.
// Rounding points and summation order are those of router_topk_kernel / moe_gate_up_kernel /
// moe_down_allreduce_kernel (decode_moe.cu), so the result is bit-identical to the three-kernel chain.
//
// Reference counterparts: router_projection/router_select, expert_gmm, expert_reduce and allreduce as separate
// instructions (native/src/token_executor.h:957-1205).
#include "gemv.cuh"
#include "moe_select.cuh"
#include "oneshot_ar.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

struct BlockParams {
  const bf16* x; long ldx;                 // residual stream rows [T, D]
  const bf16* norm_w; float eps;
  const float* w_router; const float* bias;
  int E, topk, scoring, renorm; float route_scale;
  const bf16* w_gu; const bf16* w_sgu;     // [e_local, 2F, D], [2Fs, D]
  const bf16* w_down; const bf16* w_sdown; // [e_local, D, F], [D, Fs]
  int T, D, F, Fs, e0, e_local;
  float* logits; int32_t* ids; float* wts; // router outputs [T, E], [T, topk], [T, topk]
  bf16* act;                               // [T, topk + 1, F] activations between gate/up and down
  bf16* y; long ldy;                       // x + all-reduced expert output (may alias x)
  uint32_t* sync;                          // [2]: arrive counter of the gate/up -> down barrier (zero between launches)
  uint64_t* tagged;                        // [T, E] router logits as (launch number << 32 | f32 bits)
  FabricView fv; uint64_t* seq; uint32_t* done;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_gpu(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_gpu(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// one thread waits for `*p == want`; false when the polls ran out
__device__ __forceinline__ bool wait_word(const uint32_t* p, uint32_t want, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ld_acquire_gpu(p) == want) return true;
    if (i > 128) __nanosleep(20);
  }
  return false;
}

constexpr int MAXS = MAX_TOPK + 1;
constexpr int MAXC = 6;   // 16-byte chunks per lane of one down-projection row (F <= 1536)

template <int T, int R>
__global__ void __launch_bounds__(256, 2) moe_block_kernel(BlockParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                 // [T][D] normalised rows
  bf16* as = xs + (size_t)T * p.D;                              // [topk + 1][F] activation rows of the current token
  constexpr int RPC = 8 * R;
  __shared__ float red[T * 33];
  __shared__ float part[8][T];
  __shared__ float slab[T * RPC];
  __shared__ int timed_out, wait_failed;
  __shared__ int32_t s_ids[T][MAX_TOPK];
  __shared__ float s_wts[T][MAX_TOPK];
  __shared__ const bf16* s_wd[T][MAXS];   // down weights of local route i of token t
  __shared__ int s_e[T][MAXS];            // local expert index of that route (-1: the shared expert)
  __shared__ float s_g[T][MAXS];
  __shared__ int s_k[T][MAXS];
  __shared__ int s_slot[T][MAXS];
  __shared__ int s_n[T];
  grid_dep_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const bool router_cta = (int)blockIdx.x < p.E;

  // item q of the gate/up work (shared pairs first, then the routed ones) belongs to warp (q / G) % 8 of CTA G - 1 - q % G:
  // consecutive items land on different CTAs, and the router CTAs (the first E) are reached last
  const int n_warps = G * 8;
  const int gw_rev = warp * G + (G - 1 - (int)blockIdx.x);
  const int shared_pairs = p.w_sgu ? (p.Fs + 1) / 2 : 0;
  const int quads = p.D >> 2;
  uint32_t epoch;

  auto shared_rows = [&](int item, const bf16* (&rows)[4]) {
    const int j0 = item * 2;
    rows[0] = p.w_sgu + (size_t)j0 * p.D;
    rows[1] = (j0 + 1 < p.Fs) ? p.w_sgu + (size_t)(j0 + 1) * p.D : nullptr;
    rows[2] = p.w_sgu + (size_t)(p.Fs + j0) * p.D;
    rows[3] = (j0 + 1 < p.Fs) ? p.w_sgu + (size_t)(p.Fs + j0 + 1) * p.D : nullptr;
  };
  auto shared_store = [&](int item, const float (&acc)[4][T]) {
    if (lane != 0) return;
    const int j0 = item * 2;
#pragma unroll
    for (int t = 0; t < T; ++t) {
      if (t >= p.T) continue;
      bf16* out = p.act + ((size_t)t * (p.topk + 1) + p.topk) * p.F;
      out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0][t])) * bf16_round(acc[2][t]));
      if (j0 + 1 < p.Fs) out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1][t])) * bf16_round(acc[3][t]));
    }
  };
  // shared-expert feature pairs of this warp from `first` on (no loads requested ahead)
  auto shared_items = [&](int first) {
    for (int item = first; item < shared_pairs; item += n_warps) {
      const bf16* rows[4];
      shared_rows(item, rows);
      float acc[4][T];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
      warp_rows_dot<T, 4>(rows, xs, p.D, acc);
      warp_reduce_acc<T, 4>(acc);
      shared_store(item, acc);
    }
  };

  // The two kinds of CTA take separate paths from here to the route wait, so that neither carries the other's
  // requested-ahead weights in registers. Both request weights (which depend on no kernel) before waiting for x.
  if (router_cta) {
    // ---- router: CTA e owns expert e; the last one to finish selects ---------------------------------------------------
    constexpr int PFQ = 4;
    float4 rpf[PFQ];
    const float4* wr = reinterpret_cast<const float4*>(p.w_router + (size_t)blockIdx.x * p.D);
#pragma unroll
    for (int j = 0; j < PFQ; ++j) {
      const int c = threadIdx.x + j * 256;
      rpf[j] = c < quads ? __ldg(wr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    grid_dep_wait();
    epoch = (uint32_t)(*reinterpret_cast<volatile uint64_t*>(p.seq) + 1);
    if (threadIdx.x == 0) { timed_out = 0; wait_failed = 0; }
    stage_x<T>(xs, p.x, p.ldx, 0, p.T, p.D, p.norm_w, p.eps, false, red);
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = 0.f;
    auto fma_quad = [&](const float4& wv, int c) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(xs + t * p.D + c * 4);
        const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
        acc[t] += wv.x * a.x + wv.y * a.y + wv.z * b.x + wv.w * b.y;
      }
    };
#pragma unroll
    for (int j = 0; j < PFQ; ++j) {
      const int c = threadIdx.x + j * 256;
      if (c < quads) fma_quad(rpf[j], c);
    }
    for (int c = threadIdx.x + PFQ * 256; c < quads; c += 256) fma_quad(__ldg(wr + c), c);
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) part[warp][t] = v;
    }
    __syncthreads();
    if (threadIdx.x < T && (int)threadIdx.x < p.T) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += part[w][threadIdx.x];
      p.logits[(long)threadIdx.x * p.E + blockIdx.x] = v;
      // the logit and the launch number as one 8-byte word: whoever reads the word with this launch's number has the logit
      st_relaxed_gpu(p.tagged + (size_t)threadIdx.x * p.E + blockIdx.x, ((uint64_t)epoch << 32) | (uint64_t)__float_as_uint(v));
    }
    shared_items(gw_rev);
  } else {
    // ---- shared expert gate/up (does not need the routes); the first feature pair is requested before the wait ----------
    const bf16* srows[4] = {nullptr, nullptr, nullptr, nullptr};
    RowBatch<4> spf;
    if (gw_rev < shared_pairs) shared_rows(gw_rev, srows);
    prefetch_rows<4>(srows, p.D, spf);
    grid_dep_wait();
    epoch = (uint32_t)(*reinterpret_cast<volatile uint64_t*>(p.seq) + 1);
    if (threadIdx.x == 0) { timed_out = 0; wait_failed = 0; }
    stage_x<T>(xs, p.x, p.ldx, 0, p.T, p.D, p.norm_w, p.eps, false, red);
    if (gw_rev < shared_pairs) {
      float acc[4][T];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
      warp_rows_dot<T, 4>(srows, xs, p.D, acc, spf);
      warp_reduce_acc<T, 4>(acc);
      shared_store(gw_rev, acc);
      shared_items(gw_rev + n_warps);
    }
  }

  // ---- routes: every CTA collects the E tagged logits and selects the top-k itself (no ticket, no second signal) -------
  if (warp < T && warp < p.T) {
    const int t = warp;
    float score[SELECT_PER_LANE];
    unsigned pend = 0;
#pragma unroll
    for (int i = 0; i < SELECT_PER_LANE; ++i) {
      score[i] = -INFINITY;
      if (lane + 32 * i < p.E) pend |= 1u << i;
    }
    bool all_in = false;
    for (uint32_t spin = 0; spin < p.fv.spin_limit; ++spin) {
      uint64_t got[SELECT_PER_LANE];
#pragma unroll
      for (int i = 0; i < SELECT_PER_LANE; ++i)
        if ((pend >> i) & 1u) got[i] = ld_relaxed_gpu(p.tagged + (size_t)t * p.E + lane + 32 * i);
#pragma unroll
      for (int i = 0; i < SELECT_PER_LANE; ++i)
        if (((pend >> i) & 1u) && (uint32_t)(got[i] >> 32) == epoch) {
          score[i] = __uint_as_float((uint32_t)got[i]);
          pend &= ~(1u << i);
        }
      if (__all_sync(0xffffffffu, pend == 0)) { all_in = true; break; }
      if (spin > 64) __nanosleep(20);
    }
    if (!all_in && lane == 0) {
      wait_failed = 1;
      atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
    select_topk_scores(score, p.bias, p.E, p.topk, p.scoring, p.renorm, p.route_scale, s_ids[t], s_wts[t]);
    __syncwarp();
    if (blockIdx.x == 0 && lane < p.topk) {
      p.ids[t * p.topk + lane] = s_ids[t][lane];
      p.wts[t * p.topk + lane] = s_wts[t][lane];
    }
    // route table of token `warp`, one slot per lane, compacted to the local routes with a ballot
    const int slot = lane;
    bool local = false;
    const bf16* w = nullptr;
    float g = 0.f;
    int k = 0, el = -1;
    if (slot < p.topk && all_in) {
      const int e = s_ids[t][slot];
      local = e >= p.e0 && e < p.e0 + p.e_local;
      if (e < 0 || e >= p.E) atomicOr(p.fv.status, IFAB_STATUS_BAD_INDEX);
      el = local ? e - p.e0 : 0;
      w = p.w_down + (size_t)el * p.D * p.F;
      g = s_wts[t][slot];
      k = p.F;
    } else if (slot == p.topk && p.w_sdown != nullptr) {
      local = true;
      w = p.w_sdown;
      g = 1.f;
      k = p.Fs;
      el = -1;
    }
    const unsigned m = __ballot_sync(0xffffffffu, local);
    const int n = __popc(m & ((1u << lane) - 1u));
    if (local) {
      s_wd[t][n] = w;
      s_e[t][n] = el;
      s_g[t][n] = g;
      s_k[t][n] = k;
      s_slot[t][n] = slot;
    }
    if (lane == 0) s_n[t] = __popc(m);
  }
  __syncthreads();

  // ---- routed gate/up: items (token, local route, feature pair) dealt to all warps of the grid --------------------------
  {
    const int pairs = (p.F + 1) / 2;
    int base = shared_pairs;   // item index of the first feature pair of the current (token, route)
    for (int t = 0; t < T; ++t) {
      if (t >= p.T) break;
      for (int i = 0; i < s_n[t]; ++i) {
        if (s_e[t][i] < 0) continue;   // the shared expert was done above
        const bf16* W = p.w_gu + (size_t)s_e[t][i] * 2 * p.F * p.D;
        // first item of this route that belongs to this warp
        int first = gw_rev - (base % n_warps);
        if (first < 0) first += n_warps;
        for (int pj = first; pj < pairs; pj += n_warps) {
          const int j0 = pj * 2;
          const bf16* rows[4];
          rows[0] = W + (size_t)j0 * p.D;
          rows[1] = (j0 + 1 < p.F) ? W + (size_t)(j0 + 1) * p.D : nullptr;
          rows[2] = W + (size_t)(p.F + j0) * p.D;
          rows[3] = (j0 + 1 < p.F) ? W + (size_t)(p.F + j0 + 1) * p.D : nullptr;
          float acc[4][1] = {{0.f}, {0.f}, {0.f}, {0.f}};
          warp_rows_dot<1, 4>(rows, xs + (size_t)t * p.D, p.D, acc);
          warp_reduce_acc<1, 4>(acc);
          if (lane == 0) {
            bf16* out = p.act + ((size_t)t * (p.topk + 1) + s_slot[t][i]) * p.F;
            out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0][0])) * bf16_round(acc[2][0]));
            if (j0 + 1 < p.F) out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1][0])) * bf16_round(acc[3][0]));
          }
        }
        base += pairs;
      }
    }
  }

  // ---- down projection: this CTA's RPC output columns; the first route's weights are requested before the wait ---------
  const int nbase = blockIdx.x * RPC, n0 = nbase + warp * R;
  const bool down_cta = nbase < p.D;
  uint4 wv[MAXC][R];
  auto request_route = [&](int t, int i) {
    const int k = s_k[t][i], kch = k >> 3;
    const bf16* wb = s_wd[t][i] + (size_t)n0 * k;
#pragma unroll
    for (int u = 0; u < MAXC; ++u) {
      const int c = lane + 32 * u;
#pragma unroll
      for (int r = 0; r < R; ++r)
        wv[u][r] = (c < kch && n0 + r < p.D) ? ld_stream16(wb + (size_t)r * k + c * 8) : make_uint4(0, 0, 0, 0);
    }
  };
  const bool requested = down_cta && s_n[0] > 0;
  if (requested) request_route(0, 0);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    // arrive with a release add that returns nothing; the down CTAs then poll the count itself: one trip to L2 each way
    // (the last CTA of the launch, inside the all-reduce epilogue, puts the counter back to zero)
    red_release_gpu_add(p.sync + 2, 1u);
    if (down_cta && !wait_word(p.sync + 2, (uint32_t)G, p.fv.spin_limit)) {
      wait_failed = 1;
      atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  if (down_cta) {
    for (int t = 0; t < T; ++t) {
      if (t >= p.T) {
        if (lane == 0)
#pragma unroll
          for (int r = 0; r < R; ++r) slab[t * RPC + warp * R + r] = 0.f;
        continue;
      }
      const int n_routes = s_n[t];
      __syncthreads();
      // activation rows of the local routes -> shared memory (L2 reads: they were written by other SMs)
      for (int i = 0; i < n_routes; ++i) {
        const int kch = s_k[t][i] >> 3;
        const bf16* src = p.act + ((size_t)t * (p.topk + 1) + s_slot[t][i]) * p.F;
        for (int c = threadIdx.x; c < kch; c += blockDim.x)
          *reinterpret_cast<uint4*>(as + (size_t)i * p.F + c * 8) = __ldcg(reinterpret_cast<const uint4*>(src + c * 8));
      }
      __syncthreads();
      float total[R];
#pragma unroll
      for (int r = 0; r < R; ++r) total[r] = 0.f;
      for (int i = 0; i < n_routes; ++i) {
        const int k = s_k[t][i], kch = k >> 3;
        if (!(requested && t == 0 && i == 0)) request_route(t, i);
        const float g = s_g[t][i];
        const bf16* arow = as + (size_t)i * p.F;
        float d[R];
#pragma unroll
        for (int r = 0; r < R; ++r) d[r] = 0.f;
#pragma unroll
        for (int u = 0; u < MAXC; ++u) {
          const int c = lane + 32 * u;
          if (c < kch) {
            float xf[8];
            unpack8(*reinterpret_cast<const uint4*>(arow + c * 8), xf);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              float wf[8];
              unpack8(wv[u][r], wf);
#pragma unroll
              for (int q = 0; q < 8; ++q) d[r] = fmaf(wf[q], xf[q], d[r]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) total[r] = fmaf(g, d[r], total[r]);
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = warp_sum(total[r]);
        if (lane == 0) slab[t * RPC + warp * R + r] = v;
      }
    }
  }
  __syncthreads();
  oneshot_allreduce_slab<T, RPC>(slab, p.fv, p.seq, p.done, nbase, p.T, p.D, p.x, p.ldx, p.y, p.ldy, nullptr, &timed_out, p.sync + 2);
}

template <int T, int R>
int launch_block(const BlockParams& p, int sms, cudaStream_t s) {
  auto k = moe_block_kernel<T, R>;
  const size_t smem = ((size_t)T * p.D + (size_t)(p.topk + 1) * p.F) * sizeof(bf16);
  if (int rc = opt_in_smem(k, smem)) return rc;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, 256, smem) != cudaSuccess || per_sm < 1) return -6;
  // every CTA must be resident at once (they wait on one another): never more than the device holds
  int grid = sms * (per_sm < 2 ? per_sm : 2);
  const int need = (p.D + 8 * R - 1) / (8 * R);
  if (grid < need || grid < p.E) return -7;
  return launch_chain(k, dim3(grid), dim3(256), smem, s, p);
}

}  // namespace

extern "C" int ifab_moe_block_decode(const void* x, long ldx, const void* norm_w, float eps, const float* w_router,
                                     const float* bias, int E, int topk, int scoring, int renorm, float route_scale,
                                     const void* w_gu, const void* w_shared_gu, const void* w_down,
                                     const void* w_shared_down, int T, int D, int F, int Fs, int e0, int e_local,
                                     float* logits, int32_t* ids, float* wts, void* act, void* y, long ldy,
                                     uint32_t* sync_words, const IfabFabric* fab, void* stream) {
  if (T < 1 || T > 2 || E > 256 || topk > MAX_TOPK || topk > E || D % 8 != 0 || F % 8 != 0 || Fs % 8 != 0 || Fs > F ||
      (F >> 3) > 32 * MAXC || ldx % 8 != 0)
    return -1;
  BlockParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.norm_w = (const bf16*)norm_w; p.eps = eps;
  p.w_router = w_router; p.bias = bias; p.E = E; p.topk = topk; p.scoring = scoring; p.renorm = renorm;
  p.route_scale = route_scale;
  p.w_gu = (const bf16*)w_gu; p.w_sgu = (const bf16*)w_shared_gu;
  p.w_down = (const bf16*)w_down; p.w_sdown = (const bf16*)w_shared_down;
  p.T = T; p.D = D; p.F = F; p.Fs = Fs; p.e0 = e0; p.e_local = e_local;
  p.logits = logits; p.ids = ids; p.wts = wts; p.act = (bf16*)act; p.y = (bf16*)y; p.ldy = ldy;
  p.sync = sync_words;
  p.tagged = reinterpret_cast<uint64_t*>(sync_words + 4);
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.seq = fab->seq; p.done = fab->done;
  if ((size_t)fab->world * T * D * sizeof(uint64_t) > fab->ll_half_bytes) return -3;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return -6;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // two CTAs per SM: 16 output columns per CTA cover D = 4096 with 256 CTAs; narrower models use 8 per CTA
  const int ctas = sms * 2;
  if (T <= 1) {
    if ((D + 7) / 8 <= ctas) return launch_block<1, 1>(p, sms, s);
    if ((D + 15) / 16 <= ctas) return launch_block<1, 2>(p, sms, s);
    return launch_block<1, 4>(p, sms, s);
  }
  if ((D + 7) / 8 <= ctas) return launch_block<2, 1>(p, sms, s);
  if ((D + 15) / 16 <= ctas) return launch_block<2, 2>(p, sms, s);
  return launch_block<2, 4>(p, sms, s);
}
