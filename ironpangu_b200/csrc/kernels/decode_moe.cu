// MoE decode path for sm_100a with owner-local expert parallelism (tokens and routes replicated on
// every rank, each rank evaluates the routes that land on its experts, partial outputs are summed
// by the fused all-reduce of the down projection).
//
//   router_topk_kernel        f32 router projection, one CTA per expert (+RMSNorm prologue); the
//                             last CTA to finish turns the logits into top-k ids and weights
//                             (softmax top-k or sigmoid+bias)
//   moe_gate_up_kernel        one CTA column per route: gate/up rows of the routed expert, SwiGLU
//   moe_down_allreduce_kernel score-weighted sum of the local experts' down projections (+ the
//                             tensor-parallel shard of the shared expert) + one-shot all-reduce
//   lm_head_argmax_kernel     vocabulary-sharded logits + greedy selection; the last CTA exchanges
//                             (value, index) pairs with the peers so every rank ends with the token
//
// Reference counterparts: router_projection/router_select, route_quantize, expert_gmm,
// expert_reduce and allreduce (native/src/token_executor.h:957-1205) and emit (:1206-1274).
#include "gemv.cuh"
#include "oneshot_ar.cuh"
#include "moe_select.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {


// ------------------------------------------------------------------------------------------------
struct RouterParams {
  const bf16* x; long ldx; const bf16* norm_w; float eps;
  const float* w; const float* bias;
  float* logits; int32_t* ids; float* wts;
  int T, D, E, topk, scoring, renorm; float scale;
  uint32_t* ticket;
  bf16* xn; long ldxn;     // optional: the normalised rows, for the expert kernels that follow (CTA 0 writes them)
};

// grid = E CTAs of 256 threads; thread i owns float4 columns i, i+256, ... of its expert's row
template <int T>
__global__ void __launch_bounds__(256) router_topk_kernel(RouterParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[T * 33];
  __shared__ float part[8][T];
  __shared__ int is_last;
  grid_dep_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x;
  const float4* wr = reinterpret_cast<const float4*>(p.w + (long)e * p.D);
  const int quads = p.D >> 2;
  constexpr int PFQ = 4;
  float4 pf[PFQ];
#pragma unroll
  for (int j = 0; j < PFQ; ++j) {
    const int c = threadIdx.x + j * 256;
    pf[j] = c < quads ? __ldg(wr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  grid_dep_wait();
  stage_x<T>(xs, p.x, p.ldx, 0, p.T, p.D, p.norm_w, p.eps, false, red);
  if (p.xn && blockIdx.x == 0) {
    for (int i = threadIdx.x; i < p.T * (p.D >> 3); i += blockDim.x) {
      const int t = i / (p.D >> 3), c = i % (p.D >> 3);
      *reinterpret_cast<uint4*>(p.xn + (long)t * p.ldxn + c * 8) = *reinterpret_cast<const uint4*>(xs + (size_t)t * p.D + c * 8);
    }
  }
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
    if (c < quads) fma_quad(pf[j], c);
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
    p.logits[(long)threadIdx.x * p.E + e] = v;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t tk = atomicAdd(p.ticket, 1u);
    is_last = (tk == gridDim.x - 1);
    if (is_last) *p.ticket = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // selection: warp t handles token t
  if (warp >= p.T) return;
  select_topk_row(p.logits + (long)warp * p.E, p.bias, p.E, p.topk, p.scoring, p.renorm, p.scale, p.ids + warp * p.topk,
                  p.wts + warp * p.topk);
}

// ------------------------------------------------------------------------------------------------
struct GateUpParams {
  const bf16* x; long ldx; const bf16* norm_w; float eps;
  const int32_t* ids; int T, D, F, topk, e0, e_local;
  const bf16* w_gu; const bf16* w_sgu; int Fs;
  bf16* act;
};

// grid: (ceil(F/16), T*topk + T). Column y < T*topk is route (t, k); columns after that are the shared
// expert of token t. Routes that belong to other ranks exit at once (after the dependency wait).
__global__ void __launch_bounds__(256) moe_gate_up_kernel(GateUpParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[33];
  grid_dep_launch();
  const int routes = p.T * p.topk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j0 = (blockIdx.x * 8 + warp) * 2;
  const bool shared_col = (int)blockIdx.y >= routes;
  const bf16* rows[4] = {nullptr, nullptr, nullptr, nullptr};
  RowBatch<4> pf;
  int t, slot, Fcur;
  const bf16* W;
  if (shared_col) {
    // the shared expert does not depend on the routes: its weight rows are prefetched before the wait
    t = blockIdx.y - routes;
    slot = p.topk;
    W = p.w_sgu;
    Fcur = W ? p.Fs : 0;
    if (j0 < Fcur) {
      rows[0] = W + (size_t)j0 * p.D;
      rows[1] = (j0 + 1 < Fcur) ? W + (size_t)(j0 + 1) * p.D : nullptr;
      rows[2] = W + (size_t)(Fcur + j0) * p.D;
      rows[3] = (j0 + 1 < Fcur) ? W + (size_t)(Fcur + j0 + 1) * p.D : nullptr;
    }
    prefetch_rows<4>(rows, p.D, pf);
    grid_dep_wait();
  } else {
    grid_dep_wait();
    t = blockIdx.y / p.topk;
    slot = blockIdx.y % p.topk;
    const int e = p.ids[blockIdx.y];
    if (e < p.e0 || e >= p.e0 + p.e_local) return;
    W = p.w_gu + (size_t)(e - p.e0) * 2 * p.F * p.D;
    Fcur = p.F;
    if (j0 < Fcur) {
      rows[0] = W + (size_t)j0 * p.D;
      rows[1] = (j0 + 1 < Fcur) ? W + (size_t)(j0 + 1) * p.D : nullptr;
      rows[2] = W + (size_t)(Fcur + j0) * p.D;
      rows[3] = (j0 + 1 < Fcur) ? W + (size_t)(Fcur + j0 + 1) * p.D : nullptr;
    }
    prefetch_rows<4>(rows, p.D, pf);
  }
  if ((int)blockIdx.x * 16 >= Fcur) return;
  stage_x<1>(xs, p.x, p.ldx, t, p.T, p.D, p.norm_w, p.eps, false, red);
  if (j0 >= Fcur) return;
  float acc[4][1] = {{0.f}, {0.f}, {0.f}, {0.f}};
  warp_rows_dot<1, 4>(rows, xs, p.D, acc, pf);
  warp_reduce_acc<1, 4>(acc);
  if (lane == 0) {
    bf16* out = p.act + ((size_t)t * (p.topk + 1) + slot) * p.F;
    out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0][0])) * bf16_round(acc[2][0]));
    if (j0 + 1 < Fcur) out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1][0])) * bf16_round(acc[3][0]));
  }
}

// ------------------------------------------------------------------------------------------------
struct DownParams {
  const bf16* act; const int32_t* ids; const float* wts;
  int T, D, F, topk, e0, e_local;
  const bf16* w_down; const bf16* w_sdown; int Fs;
  const bf16* residual; long ldr; bf16* y; long ldy;
  FabricView fv; uint64_t* seq; uint32_t* done;
};

// Every warp owns R output columns. The K dimension of all local routes of a token is flattened into
// one chunk space (route s contributes F/8 chunks, the shared shard Fs/8), so a lane keeps 16 loads
// in flight across route boundaries instead of draining per expert:
//   y[t][n] = sum_s wgt_s * dot(W_s[n, :], act[t][s][:])
template <int T, int R>
__global__ void __launch_bounds__(256) moe_down_allreduce_kernel(DownParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* as = reinterpret_cast<bf16*>(smem_raw);   // [(topk+1)][F] activation rows of the current token
  constexpr int RPC = 8 * R;
  constexpr int MAXS = MAX_TOPK + 1;
  __shared__ float slab[T * RPC];
  __shared__ int timed_out;
  __shared__ const bf16* s_w[MAXS];   // weight base of local route i
  __shared__ float s_g[MAXS];         // its score
  __shared__ int s_k[MAXS];           // its K extent
  __shared__ int s_cbeg[MAXS + 1];    // first flattened chunk of route i
  __shared__ int s_slot[MAXS];
  __shared__ int s_n;
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nbase = blockIdx.x * RPC, n0 = nbase + warp * R;
  if (threadIdx.x == 0) timed_out = 0;
  for (int t = 0; t < T; ++t) {
    if (t < p.T) {
      __syncthreads();
      if (warp == 0) {
        // route table, one slot per lane (expert id and score of all slots are requested at once, not one dependent global
        // load after the other), compacted to the local routes with a ballot
        const int slot = lane;
        bool local = false;
        const bf16* w = nullptr;
        float g = 0.f;
        int k = 0;
        if (slot < p.topk) {
          const int e = p.ids[t * p.topk + slot];
          local = e >= p.e0 && e < p.e0 + p.e_local;
          w = p.w_down + (size_t)(local ? e - p.e0 : 0) * p.D * p.F;
          g = p.wts[t * p.topk + slot];
          k = p.F;
        } else if (slot == p.topk && p.w_sdown != nullptr) {
          local = true;
          w = p.w_sdown;
          g = 1.f;
          k = p.Fs;
        }
        const unsigned m = __ballot_sync(0xffffffffu, local);
        const int n = __popc(m & ((1u << lane) - 1u));
        if (local) {
          s_w[n] = w;
          s_g[n] = g;
          s_k[n] = k;
          s_slot[n] = slot;
          s_cbeg[n] = n * (p.F >> 3);              // every route before the shared expert spans F
        }
        if (lane == 0) {
          const int total_n = __popc(m), shared = (int)((m >> p.topk) & 1u);
          s_cbeg[total_n] = (total_n - shared) * (p.F >> 3) + shared * (p.Fs >> 3);
          s_n = total_n;
        }
      }
      __syncthreads();
      const int n_routes = s_n;
      {
        // activation rows of the local routes -> shared memory: the chunks of all routes as one index space, eight loads in
        // flight per thread before the first store
        const int total_c = s_cbeg[n_routes], kch0 = max(1, p.F >> 3);
        constexpr int SB = 8;
        for (int q0 = threadIdx.x; q0 < total_c; q0 += (int)blockDim.x * SB) {
          uint4 v[SB];
          int dst[SB];
#pragma unroll
          for (int j = 0; j < SB; ++j) {
            const int q = q0 + (int)blockDim.x * j;
            dst[j] = -1;
            if (q < total_c) {
              const int i = min(q / kch0, n_routes - 1), c = q - s_cbeg[i];
              v[j] = *reinterpret_cast<const uint4*>(p.act + ((size_t)t * (p.topk + 1) + s_slot[i]) * p.F + c * 8);
              dst[j] = i * p.F + c * 8;
            }
          }
#pragma unroll
          for (int j = 0; j < SB; ++j)
            if (dst[j] >= 0) *reinterpret_cast<uint4*>(as + dst[j]) = v[j];
        }
      }
      __syncthreads();
      float total[R];
#pragma unroll
      for (int r = 0; r < R; ++r) total[r] = 0.f;
      constexpr int MAXC = 6;   // 16-byte chunks per lane and route the per-route form holds in registers (K <= 1536)
      if ((p.F >> 3) <= 32 * MAXC) {
        // One route at a time: weight base, score and activation row are loop invariants, a lane requests its (at most
        // MAXC) chunks of all R rows at once and the chunk loop is straight-line code. The flattened form below spends
        // three times the instructions per chunk on finding out which route a chunk belongs to.
        for (int i = 0; i < n_routes; ++i) {
          const int k = s_k[i], kch = k >> 3;
          const bf16* wb = s_w[i] + (size_t)n0 * k;
          uint4 wv[MAXC][R];
#pragma unroll
          for (int u = 0; u < MAXC; ++u) {
            const int c = lane + 32 * u;
#pragma unroll
            for (int r = 0; r < R; ++r)
              wv[u][r] = (c < kch && n0 + r < p.D) ? ld_stream16(wb + (size_t)r * k + c * 8) : make_uint4(0, 0, 0, 0);
          }
          const float g = s_g[i];
          const bf16* arow_s = as + (size_t)i * p.F;
          float d[R];
#pragma unroll
          for (int r = 0; r < R; ++r) d[r] = 0.f;
#pragma unroll
          for (int u = 0; u < MAXC; ++u) {
            const int c = lane + 32 * u;
            if (c < kch) {
              float xf[8];
              unpack8(*reinterpret_cast<const uint4*>(arow_s + c * 8), xf);
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
      } else {
      const int chunks = s_cbeg[n_routes];
        // all routed experts span cpr chunks; only a trailing shared-expert shard may differ
        const int cpr = p.F >> 3;
        const int n_exp_chunks = (n_routes > 0 && s_slot[n_routes - 1] == p.topk) ? s_cbeg[n_routes - 1] : chunks;
        constexpr int U = 16 / R;
        for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
          uint4 wv[U][R];
          int route[U], cc[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int c = c0 + u * 32;
            const int i = c < n_exp_chunks ? c / cpr : n_routes - 1;
            route[u] = i;
            cc[u] = c < n_exp_chunks ? c - i * cpr : c - n_exp_chunks;
            if (c < chunks) {
              const bf16* wb = s_w[i] + (size_t)n0 * s_k[i] + cc[u] * 8;
#pragma unroll
              for (int r = 0; r < R; ++r)
                wv[u][r] = (n0 + r < p.D) ? ld_stream16(wb + (size_t)r * s_k[i]) : make_uint4(0, 0, 0, 0);
            } else {
#pragma unroll
              for (int r = 0; r < R; ++r) wv[u][r] = make_uint4(0, 0, 0, 0);
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (c0 + u * 32 < chunks) {
              float xf[8];
              unpack8(*reinterpret_cast<const uint4*>(as + (size_t)route[u] * p.F + cc[u] * 8), xf);
              const float g = s_g[route[u]];
#pragma unroll
              for (int r = 0; r < R; ++r) {
                float wf[8], d = 0.f;
                unpack8(wv[u][r], wf);
#pragma unroll
                for (int k = 0; k < 8; ++k) d = fmaf(wf[k], xf[k], d);
                total[r] = fmaf(g, d, total[r]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = warp_sum(total[r]);
        if (lane == 0) slab[t * RPC + warp * R + r] = v;
      }
    }
  }
  __syncthreads();
  oneshot_allreduce_slab<T, RPC>(slab, p.fv, p.seq, p.done, nbase, p.T, p.D, p.residual, p.ldr, p.y, p.ldy, nullptr,
                                 &timed_out);
}

template <int T, int R>
int launch_down(const DownParams& p, cudaStream_t s) {
  const size_t smem = (size_t)(p.topk + 1) * p.F * sizeof(bf16);
  auto k = moe_down_allreduce_kernel<T, R>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid((p.D + 8 * R - 1) / (8 * R));
  return launch_chain(k, grid, dim3(256), smem, s, p);
}
template <int T>
int dispatch_down(const DownParams& p, cudaStream_t s) {
  if ((p.D + 7) / 8 <= 296) return launch_down<T, 1>(p, s);
  if ((p.D + 15) / 16 <= 296) return launch_down<T, 2>(p, s);
  if ((p.D + 31) / 32 <= 296) return launch_down<T, 4>(p, s);
  return -2;
}

// ------------------------------------------------------------------------------------------------
struct HeadParams {
  const bf16* x; long ldx; const bf16* norm_w; float eps;
  const bf16* w; float* logits;
  int T, V, K, vocab_offset;
  float2* partial;     // [grid][T] (value, index-as-int-bits)
  int32_t* out_ids; float* out_vals;
  FabricView fv; uint64_t* seq; uint32_t* done;
};

template <int T, int R>
__global__ void __launch_bounds__(256) lm_head_argmax_kernel(HeadParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[T * 33];
  __shared__ float bestv[8][T];
  __shared__ int besti[8][T];
  __shared__ int is_last;
  grid_dep_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * 8 + warp) * R;
  const bf16* rows[R];
#pragma unroll
  for (int r = 0; r < R; ++r) rows[r] = (n0 + r < p.V) ? p.w + (size_t)(n0 + r) * p.K : nullptr;
  RowBatch<R> pf;
  prefetch_rows<R>(rows, p.K, pf);
  grid_dep_wait();
  stage_x<T>(xs, p.x, p.ldx, 0, p.T, p.K, p.norm_w, p.eps, false, red);
  {
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    warp_rows_dot<T, R>(rows, xs, p.K, acc, pf);
    warp_reduce_acc<T, R>(acc);
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < T; ++t) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (n0 + r >= p.V) continue;
          if (p.logits && t < p.T) p.logits[(size_t)t * p.V + n0 + r] = acc[r][t];
          if (acc[r][t] > bv) { bv = acc[r][t]; bi = p.vocab_offset + n0 + r; }
        }
        bestv[warp][t] = bv;
        besti[warp][t] = bi;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < T) {
    const int t = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int w = 0; w < 8; ++w)
      if (bestv[w][t] > bv || (bestv[w][t] == bv && besti[w][t] < bi)) { bv = bestv[w][t]; bi = besti[w][t]; }
    p.partial[(size_t)blockIdx.x * T + t] = make_float2(bv, __int_as_float(bi));
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t tk = atomicAdd(p.done, 1u);
    is_last = (tk == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // final reduction over CTAs: warp t handles token t
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(p.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  const int world = p.fv.world, rank = p.fv.rank;
  if (warp < p.T) {
    const int t = warp;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < (int)gridDim.x; c += 32) {
      const float2 v = __ldcg(p.partial + (size_t)c * T + t);
      const int vi = __float_as_int(v.y);
      if (v.x > bv || (v.x == bv && vi < bi)) { bv = v.x; bi = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (world > 1) {
      // exchange: slot [parity][src rank][t] in every peer's staging area
      if (lane < world) {
        float2* dst = reinterpret_cast<float2*>(p.fv.data[lane] + (size_t)par * p.fv.data_half_bytes) + rank * T + t;
        *dst = make_float2(bv, __int_as_float(bi));
      }
    } else if (lane == 0) {
      p.out_ids[t] = bi;
      if (p.out_vals) p.out_vals[t] = bv;
    }
  }
  if (world > 1) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
      const int q = threadIdx.x;
      st_release_sys(p.fv.flags[q] + (size_t)par * p.fv.flag_half_words + rank, epoch);
      if (!wait_flag_bounded(p.fv.flags[rank] + (size_t)par * p.fv.flag_half_words + q, epoch, p.fv.spin_limit))
        atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
    __syncthreads();
    if (threadIdx.x < p.T) {
      const int t = threadIdx.x;
      const float2* src = reinterpret_cast<const float2*>(p.fv.data[rank] + (size_t)par * p.fv.data_half_bytes);
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int q = 0; q < world; ++q) {
        const float2 v = __ldcg(src + q * T + t);
        const int vi = __float_as_int(v.y);
        if (v.x > bv || (v.x == bv && vi < bi)) { bv = v.x; bi = vi; }
      }
      p.out_ids[t] = bi;
      if (p.out_vals) p.out_vals[t] = bv;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *p.done = 0;
    *p.seq = epoch;
    __threadfence();
  }
}

template <int T, int R>
int launch_head(const HeadParams& p, uint64_t partial_bytes, cudaStream_t s) {
  const size_t smem = (size_t)T * p.K * sizeof(bf16);
  auto k = lm_head_argmax_kernel<T, R>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid((p.V + 8 * R - 1) / (8 * R));
  if ((uint64_t)grid.x * T * sizeof(float2) > partial_bytes) return -5;
  return launch_chain(k, grid, dim3(256), smem, s, p);
}

}  // namespace

extern "C" int ifab_router_topk(const void* x, long ldx, const void* norm_w, float eps, const float* w_router,
                                const float* bias, float* logits, int32_t* ids, float* wts, int T, int D, int E,
                                int topk, int scoring, int renorm, float scale, uint32_t* ticket, void* xn, long ldxn, void* stream) {
  if (T < 1 || T > 8 || E > 256 || topk > MAX_TOPK || topk > E || D % 8 != 0 || (xn && ldxn % 8 != 0)) return -1;
  RouterParams p{(const bf16*)x, ldx, (const bf16*)norm_w, eps, w_router, bias, logits, ids, wts,
                 T, D, E, topk, scoring, renorm, scale, ticket, (bf16*)xn, ldxn};
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(E);
#define IFAB_ROUTER(TT)                                                      \
  {                                                                          \
    const size_t smem = (size_t)TT * D * sizeof(bf16);                       \
    if (int rc = opt_in_smem(router_topk_kernel<TT>, smem)) return rc;       \
    return launch_chain(router_topk_kernel<TT>, grid, dim3(256), smem, s, p); \
  }
  if (T <= 1) IFAB_ROUTER(1) else if (T <= 2) IFAB_ROUTER(2) else if (T <= 4) IFAB_ROUTER(4) else IFAB_ROUTER(8)
#undef IFAB_ROUTER
}

extern "C" int ifab_moe_gate_up_decode(const void* x, long ldx, const void* norm_w, float eps, const int32_t* ids, int T,
                                       int D, int F, int topk, int e0, int e_local, const void* w_gu,
                                       const void* w_shared_gu, int Fs, void* act, void* stream) {
  if (D % 8 != 0 || F % 8 != 0 || Fs % 8 != 0 || Fs > F) return -1;
  GateUpParams p{(const bf16*)x, ldx, (const bf16*)norm_w, eps, ids, T, D, F, topk, e0, e_local,
                 (const bf16*)w_gu, (const bf16*)w_shared_gu, Fs, (bf16*)act};
  dim3 grid((F + 15) / 16, T * topk + T);
  const size_t smem = (size_t)D * sizeof(bf16);
  if (int rc = opt_in_smem(moe_gate_up_kernel, smem)) return rc;
  return launch_chain(moe_gate_up_kernel, grid, dim3(256), smem, (cudaStream_t)stream, p);
}

extern "C" int ifab_moe_down_allreduce_decode(const void* act, const int32_t* ids, const float* wts, int T, int D, int F,
                                              int topk, int e0, int e_local, const void* w_down,
                                              const void* w_shared_down, int Fs, const void* residual, long ldr,
                                              void* y, long ldy, const IfabFabric* fab, void* stream) {
  if (T < 1 || T > 8 || F % 8 != 0 || Fs % 8 != 0 || topk > MAX_TOPK || Fs > F) return -1;
  DownParams p;
  p.act = (const bf16*)act; p.ids = ids; p.wts = wts;
  p.T = T; p.D = D; p.F = F; p.topk = topk; p.e0 = e0; p.e_local = e_local;
  p.w_down = (const bf16*)w_down; p.w_sdown = (const bf16*)w_shared_down; p.Fs = Fs;
  p.residual = (const bf16*)residual; p.ldr = ldr; p.y = (bf16*)y; p.ldy = ldy;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.seq = fab->seq; p.done = fab->done;
  if ((size_t)fab->world * T * D * sizeof(uint64_t) > fab->ll_half_bytes) return -3;
  if ((size_t)fab->world * 296 > fab->flag_half_words) return -4;
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return dispatch_down<1>(p, s);
  if (T <= 2) return dispatch_down<2>(p, s);
  if (T <= 4) return dispatch_down<4>(p, s);
  return dispatch_down<8>(p, s);
}

extern "C" int ifab_lm_head_argmax(const void* x, long ldx, const void* norm_w, float eps, const void* w, float* logits,
                                   int T, int V_local, int K, int vocab_offset, void* partial, uint64_t partial_bytes,
                                   int32_t* out_ids, float* out_vals, const IfabFabric* fab, void* stream) {
  if (T < 1 || T > 8 || K % 8 != 0) return -1;
  HeadParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.norm_w = (const bf16*)norm_w; p.eps = eps;
  p.w = (const bf16*)w; p.logits = logits; p.T = T; p.V = V_local; p.K = K; p.vocab_offset = vocab_offset;
  p.partial = (float2*)partial; p.out_ids = out_ids; p.out_vals = out_vals;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.seq = fab->seq; p.done = fab->done;
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return launch_head<1, 4>(p, partial_bytes, s);
  if (T <= 2) return launch_head<2, 4>(p, partial_bytes, s);
  if (T <= 4) return launch_head<4, 4>(p, partial_bytes, s);
  return launch_head<8, 2>(p, partial_bytes, s);
}
