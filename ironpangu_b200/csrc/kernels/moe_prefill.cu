// Prefill-side MoE plumbing around the grouped tcgen05 GEMM (tc_grouped.cu), for chunks of hundreds of tokens:
//
//   router_block_kernel   f32 router projection + top-k for blocks of 8 tokens (the decode router handles <= 8 rows
//                         per launch; a prefill chunk would need 64 launches)
//   moe_dispatch_kernel   routes of this rank's experts -> rows sorted by expert (stable: token-major inside an
//                         expert), per-expert counts, the 128-row tile table of the grouped GEMM and, for every
//                         (token, slot), the row that will hold its expert output (-1 = not on this rank)
//   moe_gather_kernel     permuted activation matrix: row r = normalised hidden state of the token of route r
//   moe_combine_kernel    out[token] = sum_slots score * expert_out[row(token, slot)] (+ shared expert) (+ residual)
//
// Everything is sized by device-side counts; the host never learns how many tokens an expert received.
// Reference counterparts: route_quantize (aclnnMoeInitRoutingV3) and expert_reduce (aclnnMoeFinalizeRoutingV2),
// native/src/token_executor.h:1054-1205.
#include <algorithm>

#include "gemv.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

constexpr int MAX_TOPK = 16;
constexpr int MAX_LOCAL = 256;

// ---- router for token blocks -----------------------------------------------------------------------------------
struct RouterBlockParams {
  const bf16* x; long ldx; const bf16* norm_w; float eps;
  const float* w; const float* bias;
  float* logits; int32_t* ids; float* wts; bf16* xn; long ldxn;
  int M, D, E, topk, scoring, renorm; float scale;
};

// one CTA per 8 tokens; warps stride over the experts, then warp t selects for token t
__global__ void __launch_bounds__(256) router_block_kernel(RouterBlockParams p) {
  constexpr int T = 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);               // [8][D] normalised
  float* lg = reinterpret_cast<float*>(xs + (size_t)T * p.D); // [8][E]
  __shared__ float red[T * 33];
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * T;
  stage_x<T>(xs, p.x, p.ldx, t0, p.M, p.D, p.norm_w, p.eps, false, red);
  if (p.xn) {   // the normalised rows are reused by the expert GEMMs
    for (int i = threadIdx.x; i < T * (p.D >> 3); i += blockDim.x) {
      const int t = i / (p.D >> 3), c = i % (p.D >> 3);
      if (t0 + t < p.M) *reinterpret_cast<uint4*>(p.xn + (long)(t0 + t) * p.ldxn + c * 8) = *reinterpret_cast<const uint4*>(xs + (size_t)t * p.D + c * 8);
    }
  }
  const int quads = p.D >> 2;
  for (int e = warp; e < p.E; e += 8) {
    const float4* wr = reinterpret_cast<const float4*>(p.w + (long)e * p.D);
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = 0.f;
    // eight 16-byte weight loads in flight per lane: issued one at a time the loop waits for L2 on every iteration
    constexpr int G = 8;
    for (int c0 = lane; c0 < quads; c0 += 32 * G) {
      float4 wv[G];
#pragma unroll
      for (int g = 0; g < G; ++g) wv[g] = (c0 + 32 * g < quads) ? __ldg(wr + c0 + 32 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int c = c0 + 32 * g;
        if (c < quads) {
#pragma unroll
          for (int t = 0; t < T; ++t) {
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(xs + (size_t)t * p.D + c * 4);
            const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
            acc[t] += wv[g].x * a.x + wv[g].y * a.y + wv[g].z * b.x + wv[g].w * b.y;
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(acc[t]);
      if (lane == 0) {
        lg[t * p.E + e] = v;
        if (p.logits && t0 + t < p.M) p.logits[(long)(t0 + t) * p.E + e] = v;
      }
    }
  }
  __syncthreads();
  const int t = warp;
  if (t0 + t >= p.M) return;
  constexpr int PER = 8;
  float score[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ei = lane + 32 * i;
    score[i] = (ei < p.E) ? lg[t * p.E + ei] : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  mx = warp_max(mx);
  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ei = lane + 32 * i;
    if (ei < p.E) {
      if (p.scoring == 0) {
        score[i] = __expf(score[i] - mx);
        denom += score[i];
        sel[i] = score[i];
      } else {
        score[i] = 1.f / (1.f + __expf(-score[i]));
        sel[i] = score[i] + (p.bias ? p.bias[ei] : 0.f);
      }
    } else {
      score[i] = 0.f;
      sel[i] = -INFINITY;
    }
  }
  denom = warp_sum(denom);
  float picked_w[MAX_TOPK];
  int picked_e[MAX_TOPK];
  float wsum = 0.f;
  for (int k = 0; k < p.topk; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int ei = lane + 32 * i;
      if (sel[i] > bv || (sel[i] == bv && ei < bi)) { bv = sel[i]; bi = ei; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    float raw = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (lane + 32 * i == bi) { raw = score[i]; sel[i] = -INFINITY; }
    }
    raw = warp_sum(raw);
    picked_e[k] = bi;
    picked_w[k] = (p.scoring == 0) ? raw / denom : raw;
    wsum += picked_w[k];
  }
  if (lane == 0) {
    for (int k = 0; k < p.topk; ++k) {
      float w = picked_w[k];
      if (p.scoring == 0) { if (p.renorm) w = w / wsum; }
      else w = w / (wsum + 1e-20f);
      p.ids[(long)(t0 + t) * p.topk + k] = picked_e[k];
      p.wts[(long)(t0 + t) * p.topk + k] = w * p.scale;
    }
  }
}

// ---- dispatch ---------------------------------------------------------------------------------------------------
struct DispatchParams {
  const int32_t* ids; int M, topk, e0, el;
  int32_t* counts;      // [el]
  int32_t* route_row;   // [M * topk]: row in the permuted matrix, -1 when the expert lives on another rank
  int32_t* perm_token;  // [M * topk]: token of permuted row r
  int4* tiles; int32_t* num_tiles; int32_t* total_rows; int max_tiles;
  int smem_routes;      // routes whose local expert ids fit the dynamic shared memory of the launch
};

// single CTA of 1024 threads: warp w ranks the routes of experts w, w + 32, ... with ballot prefix sums, so the order
// inside an expert is the route order (token-major) and the result does not depend on thread timing
__global__ void __launch_bounds__(1024) moe_dispatch_kernel(DispatchParams p) {
  __shared__ int s_count[MAX_LOCAL];
  __shared__ int s_off[MAX_LOCAL + 1];
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = p.M * p.topk;
  // the local expert of every route (or -1), staged once: the ballot scans below would otherwise wait on a global load each
  extern __shared__ short s_loc[];
  const bool staged = R <= p.smem_routes;
  if (staged) {
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
      const int e = p.ids[i] - p.e0;
      s_loc[i] = (short)((e >= 0 && e < p.el) ? e : -1);
    }
    __syncthreads();
  }
  auto local_of = [&](int i) -> int { return staged ? (int)s_loc[i] : p.ids[i] - p.e0; };
  // pass 1: counts
  for (int e = warp; e < p.el; e += 32) {
    int n = 0;
    for (int i0 = 0; i0 < R; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < R && local_of(i) == e;
      n += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) s_count[e] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < p.el; ++e) {
      s_off[e] = off;
      p.counts[e] = s_count[e];
      for (int r0 = 0; r0 < s_count[e]; r0 += 128) {
        if (nt < p.max_tiles) p.tiles[nt] = make_int4(e, off + r0, min(128, s_count[e] - r0), 0);
        ++nt;
      }
      off += s_count[e];
    }
    s_off[p.el] = off;
    *p.num_tiles = min(nt, p.max_tiles);
    *p.total_rows = off;
  }
  // routes of other ranks
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int e = p.ids[i] - p.e0;
    if (e < 0 || e >= p.el) p.route_row[i] = -1;
  }
  __syncthreads();
  // pass 2: placement
  for (int e = warp; e < p.el; e += 32) {
    int base = s_off[e];
    for (int i0 = 0; i0 < R; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < R && local_of(i) == e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = base + __popc(m & ((1u << lane) - 1));
        p.route_row[i] = r;
        p.perm_token[r] = i / p.topk;
      }
      base += __popc(m);
    }
  }
}

// xp[r, :] = xn[perm_token[r], :] for r < *total_rows (16-byte chunks, one warp per row)
__global__ void __launch_bounds__(256) moe_gather_kernel(const bf16* xn, long ldxn, const int32_t* perm_token, const int32_t* total_rows,
                                                         bf16* xp, long ldxp, int D, int rows_max) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = min(*total_rows, rows_max);
  for (int r = blockIdx.x * 8 + warp; r < total; r += gridDim.x * 8) {
    const bf16* src = xn + (long)perm_token[r] * ldxn;
    bf16* dst = xp + (long)r * ldxp;
    for (int c = lane; c < (D >> 3); c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
  }
}

struct CombineParams {
  const bf16* y; long ldy;             // expert outputs by permuted row
  const int32_t* route_row; const float* wts; int M, topk, D;
  const bf16* shared; long lds;        // optional shared-expert output [M, D]
  const bf16* residual; long ldr;      // optional
  float* out_f32; bf16* out; long ldo;
};

// one warp per token row; f32 accumulation in slot order (deterministic)
__global__ void __launch_bounds__(256) moe_combine_kernel(CombineParams p) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 8 + warp;
  if (m >= p.M) return;
  int rows[MAX_TOPK];
  float w[MAX_TOPK];
  for (int k = 0; k < p.topk; ++k) {
    rows[k] = p.route_row[(long)m * p.topk + k];
    w[k] = p.wts[(long)m * p.topk + k];
  }
  for (int c = lane; c < (p.D >> 3); c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < p.topk; ++k) {
      if (rows[k] < 0) continue;
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.y + (long)rows[k] * p.ldy + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[k], f[i], acc[i]);
    }
    if (p.shared) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.shared + (long)m * p.lds + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    if (p.out_f32) {
      float* o = p.out_f32 + (long)m * p.D + c * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = acc[i];
    }
    if (p.out) {
      if (p.residual) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(p.residual + (long)m * p.ldr + c * 8), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = bf16_round(acc[i]) + f[i];
      }
      *reinterpret_cast<uint4*>(p.out + (long)m * p.ldo + c * 8) = pack8(acc);
    }
  }
}

}  // namespace

extern "C" int ifab_router_block(const void* x, long ldx, const void* norm_w, float eps, const float* w_router, const float* bias,
                                 float* logits, int32_t* ids, float* wts, void* xn, long ldxn, int M, int D, int E, int topk,
                                 int scoring, int renorm, float scale, void* stream) {
  if (M < 1 || E > 256 || topk > MAX_TOPK || topk > E || D % 8) return -1;
  RouterBlockParams p{(const bf16*)x, ldx, (const bf16*)norm_w, eps, w_router, bias, logits, ids, wts, (bf16*)xn, ldxn,
                      M, D, E, topk, scoring, renorm, scale};
  const size_t smem = (size_t)8 * D * sizeof(bf16) + (size_t)8 * E * sizeof(float);
  if (int rc = opt_in_smem(router_block_kernel, smem)) return rc;
  return launch_chain(router_block_kernel, dim3((M + 7) / 8), dim3(256), smem, (cudaStream_t)stream, p);
}

extern "C" int ifab_moe_dispatch(const int32_t* ids, int M, int topk, int e0, int e_local, int32_t* counts, int32_t* route_row,
                                 int32_t* perm_token, int32_t* tiles, int32_t* num_tiles, int32_t* total_rows, int max_tiles,
                                 void* stream) {
  if (M < 1 || topk < 1 || topk > MAX_TOPK || e_local < 1 || e_local > MAX_LOCAL || max_tiles < 1) return -1;
  DispatchParams p{ids, M, topk, e0, e_local, counts, route_row, perm_token, reinterpret_cast<int4*>(tiles), num_tiles, total_rows,
                   max_tiles, 0};
  const size_t want = (size_t)M * topk * sizeof(short);
  const size_t smem = want <= 160 * 1024 ? want : 0;
  p.smem_routes = (int)(smem / sizeof(short));
  if (int rc = opt_in_smem(moe_dispatch_kernel, smem)) return rc;
  return launch_chain(moe_dispatch_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, p);
}

extern "C" int ifab_moe_gather(const void* xn, long ldxn, const int32_t* perm_token, const int32_t* total_rows, void* xp, long ldxp,
                               int D, int rows_max, void* stream) {
  if (D % 8 || ldxn % 8 || ldxp % 8 || rows_max < 1) return -1;
  const int grid = std::min(4 * 148, (rows_max + 7) / 8);
  return launch_chain(moe_gather_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const bf16*)xn, ldxn, perm_token, total_rows,
                      (bf16*)xp, ldxp, D, rows_max);
}

extern "C" int ifab_moe_combine(const void* y, long ldy, const int32_t* route_row, const float* wts, int M, int topk, int D,
                                const void* shared, long lds, const void* residual, long ldr, float* out_f32, void* out, long ldo,
                                void* stream) {
  if (D % 8 || ldy % 8 || topk > MAX_TOPK || (shared && lds % 8) || (residual && ldr % 8) || (out && ldo % 8)) return -1;
  CombineParams p{(const bf16*)y, ldy, route_row, wts, M, topk, D, (const bf16*)shared, lds, (const bf16*)residual, ldr, out_f32,
                  (bf16*)out, ldo};
  return launch_chain(moe_combine_kernel, dim3((M + 7) / 8), dim3(256), 0, (cudaStream_t)stream, p);
}
