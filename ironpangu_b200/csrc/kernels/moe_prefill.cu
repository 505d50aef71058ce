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

// one CTA per T tokens (8, or 4 when that is what fills the SMs); warps stride over the experts, then warp t selects for token t
template <int T>
__global__ void __launch_bounds__(256) router_block_kernel(RouterBlockParams p) {
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
  if (t >= T || t0 + t >= p.M) return;
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
};

// Single CTA of 1024 threads. Every warp owns a contiguous segment of the routes (route order = token-major), so the order inside
// an expert is the route order and the result does not depend on thread timing:
//   1  per warp and expert: how many routes of the segment go to the expert (lanes with the same expert find one another with
//      match.any; the lowest lane of a group adds the group's size to the warp's histogram in shared memory)
//   2  per expert: exclusive scan of the warps' counts (one thread per expert), then expert offsets, counts and the tile table
//   3  per warp: walk the segment again; a route's row = expert offset + routes of earlier warps + routes seen so far in this warp
//      + its rank inside the 32-route group
// Work per warp is its segment twice, instead of every route once per expert.
__global__ void __launch_bounds__(1024) moe_dispatch_kernel(DispatchParams p) {
  __shared__ int s_off[MAX_LOCAL + 1];
  extern __shared__ int s_hist[];          // [32 warps][el]: counts, then running row offsets
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = p.M * p.topk, el = p.el;
  const int per_warp = ((R + 31) / 32 + 31) / 32 * 32;       // segment length, a multiple of 32
  const int seg0 = warp * per_warp, seg1 = min(R, seg0 + per_warp);
  for (int i = threadIdx.x; i < 32 * el; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  int* hist = s_hist + warp * el;
  for (int i0 = seg0; i0 < seg1; i0 += 32) {
    const int i = i0 + lane;
    int e = -1;
    if (i < seg1) {
      e = p.ids[i] - p.e0;
      if (e < 0 || e >= el) {
        e = -1;
        p.route_row[i] = -1;                 // the expert lives on another rank
      }
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (same & ((1u << lane) - 1)) == 0) hist[e] += __popc(same);     // one lane per expert per group: no two lanes touch a word
    __syncwarp();
  }
  __syncthreads();
  // exclusive scan over the warps, per expert; the total lands in s_off (as a count for now)
  for (int e = threadIdx.x; e < el; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = s_hist[w * el + e];
      s_hist[w * el + e] = run;
      run += c;
    }
    s_off[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < el; ++e) {
      const int c = s_off[e];
      s_off[e] = off;
      p.counts[e] = c;
      for (int r0 = 0; r0 < c; r0 += 128) {
        if (nt < p.max_tiles) p.tiles[nt] = make_int4(e, off + r0, min(128, c - r0), 0);
        ++nt;
      }
      off += c;
    }
    s_off[el] = off;
    *p.num_tiles = min(nt, p.max_tiles);
    *p.total_rows = off;
  }
  __syncthreads();
  for (int i0 = seg0; i0 < seg1; i0 += 32) {
    const int i = i0 + lane;
    int e = -1;
    if (i < seg1) {
      e = p.ids[i] - p.e0;
      if (e < 0 || e >= el) e = -1;
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    if (e >= 0) {
      const int r = s_off[e] + hist[e] + __popc(same & ((1u << lane) - 1));
      p.route_row[i] = r;
      p.perm_token[r] = i / p.topk;
    }
    __syncwarp();
    if (e >= 0 && (same & ((1u << lane) - 1)) == 0) hist[e] += __popc(same);
    __syncwarp();
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

// One warp per (token row, column quarter); f32 accumulation in slot order (deterministic). The loads of all routes of a chunk are
// issued before the first is used: rows of different experts are unrelated addresses, one at a time they cost a memory latency each.
__global__ void __launch_bounds__(256) moe_combine_kernel(CombineParams p, int quarters) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * 8 + warp;
  const int m = item / quarters, q = item % quarters;
  if (m >= p.M) return;
  int rows[MAX_TOPK];
  float w[MAX_TOPK];
#pragma unroll
  for (int k = 0; k < MAX_TOPK; ++k) {
    rows[k] = k < p.topk ? p.route_row[(long)m * p.topk + k] : -1;
    w[k] = k < p.topk ? p.wts[(long)m * p.topk + k] : 0.f;
  }
  const int per = (p.D >> 3) / quarters;
  for (int cc = lane; cc < per; cc += 32) {
    const int c = q * per + cc;
    uint4 v[MAX_TOPK];
#pragma unroll
    for (int k = 0; k < MAX_TOPK; ++k)
      v[k] = rows[k] >= 0 ? *reinterpret_cast<const uint4*>(p.y + (long)rows[k] * p.ldy + c * 8) : make_uint4(0, 0, 0, 0);
    uint4 sh = make_uint4(0, 0, 0, 0), rs = make_uint4(0, 0, 0, 0);
    if (p.shared) sh = *reinterpret_cast<const uint4*>(p.shared + (long)m * p.lds + c * 8);
    if (p.out && p.residual) rs = *reinterpret_cast<const uint4*>(p.residual + (long)m * p.ldr + c * 8);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MAX_TOPK; ++k) {
      if (rows[k] < 0) continue;
      float f[8];
      unpack8(v[k], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[k], f[i], acc[i]);
    }
    if (p.shared) {
      float f[8];
      unpack8(sh, f);
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
        unpack8(rs, f);
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
  // eight tokens per CTA re-read the router matrix least often; with fewer than ~150 such CTAs half the SMs idle, so chunks of
  // up to ~1200 tokens run four tokens per CTA
  if ((M + 7) / 8 >= 148) {
    const size_t smem = (size_t)8 * D * sizeof(bf16) + (size_t)8 * E * sizeof(float);
    if (int rc = opt_in_smem(router_block_kernel<8>, smem)) return rc;
    return launch_chain(router_block_kernel<8>, dim3((M + 7) / 8), dim3(256), smem, (cudaStream_t)stream, p);
  }
  const size_t smem = (size_t)4 * D * sizeof(bf16) + (size_t)4 * E * sizeof(float);
  if (int rc = opt_in_smem(router_block_kernel<4>, smem)) return rc;
  return launch_chain(router_block_kernel<4>, dim3((M + 3) / 4), dim3(256), smem, (cudaStream_t)stream, p);
}

extern "C" int ifab_moe_dispatch(const int32_t* ids, int M, int topk, int e0, int e_local, int32_t* counts, int32_t* route_row,
                                 int32_t* perm_token, int32_t* tiles, int32_t* num_tiles, int32_t* total_rows, int max_tiles,
                                 void* stream) {
  if (M < 1 || topk < 1 || topk > MAX_TOPK || e_local < 1 || e_local > MAX_LOCAL || max_tiles < 1) return -1;
  DispatchParams p{ids, M, topk, e0, e_local, counts, route_row, perm_token, reinterpret_cast<int4*>(tiles), num_tiles, total_rows,
                   max_tiles};
  const size_t smem = (size_t)32 * e_local * sizeof(int);
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
  const int quarters = (D % 32 == 0 && D >= 1024) ? 4 : 1;      // four warps share a wide row
  return launch_chain(moe_combine_kernel, dim3((M * quarters + 7) / 8), dim3(256), 0, (cudaStream_t)stream, p, quarters);
}
