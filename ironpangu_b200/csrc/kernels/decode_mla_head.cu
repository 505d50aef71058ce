// The attention half of an MLA decode layer as ONE launch: one thread-block cluster of 8 CTAs per head.
//
//   input   qkv_a[t] = [ q_latent (q_lora) | kv latent (512) | k_pe (64) ]       (output of the qkv_a GEMV)
//   output  attn[t][h * vdim ...]                                                   (input of the o_proj GEMV)
//
// Between those two GEMVs the operator-per-launch path runs five small kernels (cache write, q_b GEMV, absorb, split
// attention, merge + value up-projection), each a few microseconds of launch and drain latency around very little work.
// Every one of those steps is local to a head except the cache row of the new token, so a cluster per head can run the
// whole chain with cluster barriers (distributed shared memory) where the chain needed kernel boundaries:
//
//   0  all CTAs: RMSNorm(q latent) into shared memory; the new cache row of every token (RMSNorm(latent) | RoPE(k_pe)) into
//      shared memory - every cluster computes it for itself, the first CTA of head 0 also writes it to the paged cache
//   1  q_b: the 192 rows of the head are split over the 64 warps of the cluster, results broadcast to all 8 CTAs
//   2  absorb: CTA c produces latent columns [64c, 64c+64) of q_nope W_UK, broadcast; every CTA rotates q_pe itself
//   3  attention: the visible keys are split over the 64 warps (online softmax per warp, fixed-order merge per CTA);
//      keys written in this step are read from shared memory, older ones from the paged cache
//   4  CTA c merges columns [64c, 64c+64) of the 8 CTA partials (log-sum-exp, fixed order) and multiplies them with its
//      K-slice of W_UV; the 8 partial [T, vdim] results are summed in CTA order by CTA 0 and stored
//
// Weights of steps 1, 2 and 4 do not depend on activations and are requested before the producer kernel has finished
// (programmatic dependent launch). The rounding points are those of the separate kernels (q, q_lat, cache rows and the
// merged latent output are rounded to bf16), so both paths agree to f32 summation order.
// Reference: mla_query + cache_norm_rope_append + latent_attention + mla_value (native/src/token_executor.h:613-909).
#include <cooperative_groups.h>

#include "gemv.cuh"
#include "mla_common.cuh"
#include "ifab_kernels.h"

namespace cg = cooperative_groups;
using namespace ifab;
using namespace ifab::mla;

namespace {

constexpr int C = 8;            // CTAs per cluster
constexpr int NW = C * 8;       // warps per cluster
constexpr int MAXQ = 192;       // nope + rope per head
constexpr int SLICE = LATENT / C;

struct HeadParams {
  const bf16* qkv; long ldqkv;
  const bf16* q_norm; const bf16* kv_norm; float eps, theta;
  const bf16* w_qb; const bf16* w_kvb;
  bf16* cache; const int32_t* positions; const int32_t* slots; const int32_t* page_table;
  int max_pages, page_tokens, num_pages;
  const bf16* sinks; int n_sinks, window; float scale;
  int T, H, q_lora, nope, vdim;
  bf16* out; long ldo;
  uint32_t* status;
  // weight ranges of LATER kernels of the layer, requested into L2 while this kernel (a latency-bound chain that leaves HBM idle) runs
  const char* pf[3]; unsigned long long pf_bytes[3];
};

// shared-memory carve-up (bytes), identical in every CTA of the cluster
struct Layout {
  size_t xs, red, qf, qlat, newrow, wacc, wml, part, os, outbuf, total;
};
__host__ __device__ inline Layout layout_for(int T, int q_lora) {
  Layout L;
  size_t o = 0;
  auto take = [&](size_t bytes) { const size_t at = o; o += (bytes + 15) & ~(size_t)15; return at; };
  // xs (steps 0-1) and outbuf (step 4) never live at the same time
  const size_t xs_bytes = (size_t)T * q_lora * 2, ob_bytes = (size_t)C * T * 128 * 4;
  L.xs = L.outbuf = take(xs_bytes > ob_bytes ? xs_bytes : ob_bytes);
  L.red = take((size_t)T * 33 * 4);
  L.qf = take((size_t)T * MAXQ * 4);
  L.qlat = take((size_t)T * ROW * 2);
  L.newrow = take((size_t)T * ROW * 2);
  L.wacc = take((size_t)8 * LATENT * 4);
  L.wml = take(16 * 4);
  L.part = take((size_t)T * (LATENT + 2) * 4);
  L.os = take((size_t)T * SLICE * 2);
  L.total = o;
  return L;
}

// Sum NV values per lane across the warp; afterwards lane l holds the total of value (l * NV) / 32 (+ k, k < NV / 32) in v[k].
template <int NV>
__device__ __forceinline__ void warp_reduce_scatter(float (&v)[NV], int lane) {
  int n = NV;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    if (n >= 2) {
      const bool upper = (lane & off) != 0;
      const int h = n / 2;
#pragma unroll
      for (int k = 0; k < NV / 2; ++k) {
        if (k < h) {
          const float send = upper ? v[k] : v[k + h];
          const float keep = upper ? v[k + h] : v[k];
          v[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
      }
      n = h;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
}

// RMS-normalised rows of x into shared memory in ONE pass when a row fits one 16-byte chunk per thread (K <= 8 * blockDim):
// every thread keeps its chunk of every row in registers between the sum of squares and the scaling, so the rows are read
// once and two block barriers suffice. Same arithmetic and rounding as stage_x.
template <int T>
__device__ __forceinline__ void stage_q(bf16* xs, const bf16* __restrict__ x, long ldx, int t_total, int K, const bf16* __restrict__ norm_w,
                                        float eps, float* red) {
  const int chunks = K >> 3, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
  if (chunks > (int)blockDim.x) {
    stage_x<T>(xs, x, ldx, 0, t_total, K, norm_w, eps, false, red);
    return;
  }
  float f[T][8], g[8];
  const bool has = tid < chunks;
  if (has) unpack8(*reinterpret_cast<const uint4*>(norm_w + tid * 8), g);
#pragma unroll
  for (int t = 0; t < T; ++t) {
    const uint4 v = (has && t < t_total) ? *reinterpret_cast<const uint4*>(x + (long)t * ldx + tid * 8) : make_uint4(0, 0, 0, 0);
    unpack8(v, f[t]);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[t][i] * f[t][i];
    ss = warp_sum(ss);
    if (lane == 0) red[t * 33 + warp] = ss;
  }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < T; ++t) {
    float s = 0.f;
    for (int w = 0; w < nwarp; ++w) s += red[t * 33 + w];
    const float inv = rsqrtf(s / (float)K + eps);
    if (has) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[t][i] = f[t][i] * inv * g[i];
      *reinterpret_cast<uint4*>(xs + t * K + tid * 8) = pack8(f[t]);
    }
  }
  __syncthreads();
}

template <int T>
__global__ void __launch_bounds__(256, (T <= 2 ? 2 : 1)) mla_head_decode_kernel(HeadParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const Layout L = layout_for(T, p.q_lora);
  bf16* xs = reinterpret_cast<bf16*>(smem + L.xs);
  float* red = reinterpret_cast<float*>(smem + L.red);
  float* qf = reinterpret_cast<float*>(smem + L.qf);          // [T][MAXQ] q of this head (bf16 values)
  bf16* qlat = reinterpret_cast<bf16*>(smem + L.qlat);        // [T][ROW] absorbed query
  bf16* newrow = reinterpret_cast<bf16*>(smem + L.newrow);    // [T][ROW] cache rows produced by this step
  float* wacc = reinterpret_cast<float*>(smem + L.wacc);      // [8 warps][LATENT]
  float* wml = reinterpret_cast<float*>(smem + L.wml);        // [8] m, [8] l
  float* part = reinterpret_cast<float*>(smem + L.part);      // [T][LATENT + 2] partial of this CTA
  bf16* os = reinterpret_cast<bf16*>(smem + L.os);            // [T][SLICE] merged output, this CTA's columns
  float* outbuf = reinterpret_cast<float*>(smem + L.outbuf);  // [C][T][128] (read on CTA 0 only)
  __shared__ int s_pos[8], s_slot[8];

  grid_dep_launch();
  {
    const long first = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 128, stride = (long)gridDim.x * blockDim.x * 128;
#pragma unroll
    for (int i = 0; i < 3; ++i)
      for (long off = first; off < (long)p.pf_bytes[i]; off += stride) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.pf[i] + off));
  }
  const int cr = (int)cluster.block_rank(), h = blockIdx.x / C;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gw = cr * 8 + warp;
  const int nq = p.nope + ROPE;
  // ---- weights that do not depend on activations: first q_b batch, absorb slice ----
  const int rpw = (nq + NW - 1) / NW;   // q rows per warp, <= 3
  const bf16* qrows[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int r = gw * rpw + i;
    qrows[i] = (i < rpw && r < nq) ? p.w_qb + ((long)h * nq + r) * p.q_lora : nullptr;
  }
  RowBatch<3, 12> pf;
  prefetch_rows<3, 12>(qrows, p.q_lora, pf);
  const int dpl = p.nope >> 5;          // q_nope elements per lane in the absorb step, <= 4
  const bf16* Wuk = p.w_kvb + (long)h * (p.nope + p.vdim) * LATENT + cr * SLICE + warp * 8;
  uint4 wv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) wv[j] = j < dpl ? ld_stream16(Wuk + (long)(lane * dpl + j) * LATENT) : make_uint4(0, 0, 0, 0);
  cluster.sync();                       // every CTA of the cluster runs: its shared memory may be written from here on
  grid_dep_wait();

  // ---- step 0: normalised q latent, new cache rows ----
  if (threadIdx.x < 8) {
    const bool live = (int)threadIdx.x < p.T;
    s_pos[threadIdx.x] = live ? p.positions[threadIdx.x] : -1;
    s_slot[threadIdx.x] = live ? p.slots[threadIdx.x] : -1;
  }
  stage_q<T>(xs, p.qkv, p.ldqkv, p.T, p.q_lora, p.q_norm, p.eps, red);
  // Ask for the cache rows this warp will score in step 3 now (L2 prefetch, nine 128-byte lines per row), so that their
  // HBM latency passes under steps 1 and 2. Lane j looks up the j-th key of the warp, so the page-table loads of a warp
  // are in flight together (one latency, not one per key); they also warm L1 for the lookups of step 3.
  for (int t = 0; t < T; ++t) {
    const int pos = s_pos[t];
    if (pos < 0) continue;
    int first, nctx;
    visible_range(pos, p.window, &first, &nctx);
    for (int k = gw + NW * lane; k < nctx; k += NW * 32) {
      const long r = cache_row_of(first + k, s_slot[t], p.page_table, p.max_pages, p.page_tokens, p.num_pages);
      if (r >= 0) {
        const char* row = reinterpret_cast<const char*>(p.cache + r * ROW);
#pragma unroll
        for (int i = 0; i < (ROW * 2 + 127) / 128; ++i) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + i * 128));
      }
    }
  }
  if (warp < T && warp < p.T && s_pos[warp] >= 0) {
    const int t = warp, pos = s_pos[t];
    const bf16* src = p.qkv + (long)t * p.ldqkv + p.q_lora;
    float f[16], g[16];
    unpack8(*reinterpret_cast<const uint4*>(src + lane * 8), f);
    unpack8(*reinterpret_cast<const uint4*>(src + 256 + lane * 8), f + 8);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss += f[i] * f[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)LATENT + p.eps);
    unpack8(*reinterpret_cast<const uint4*>(p.kv_norm + lane * 8), g);
    unpack8(*reinterpret_cast<const uint4*>(p.kv_norm + 256 + lane * 8), g + 8);
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = f[i] * inv * g[i];
    bf16* dst = newrow + t * ROW;
    *reinterpret_cast<uint4*>(dst + lane * 8) = pack8(f);
    *reinterpret_cast<uint4*>(dst + 256 + lane * 8) = pack8(f + 8);
    float c, s;
    rope_cos_sin(pos, lane, ROPE, p.theta, &c, &s);
    const float a = __bfloat162float(src[LATENT + lane]), b = __bfloat162float(src[LATENT + lane + ROPE / 2]);
    dst[LATENT + lane] = __float2bfloat16_rn(a * c - b * s);
    dst[LATENT + lane + ROPE / 2] = __float2bfloat16_rn(b * c + a * s);
    if (h == 0 && cr == 0) {
      __syncwarp();
      const long row = cache_row_of(pos, s_slot[t], p.page_table, p.max_pages, p.page_tokens, p.num_pages);
      if (row < 0) {
        if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_BAD_INDEX);
      } else {
        uint4* g4 = reinterpret_cast<uint4*>(p.cache + row * ROW);
        const uint4* s4 = reinterpret_cast<const uint4*>(dst);
        for (int i = lane; i < ROW / 8; i += 32) g4[i] = s4[i];
      }
    }
  }

  // ---- step 1: q_b rows of this head, broadcast to the cluster ----
  {
    float acc[3][T];
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[i][t] = 0.f;
    warp_rows_dot<T, 3, 12>(qrows, xs, p.q_lora, acc, pf);
    warp_reduce_acc<T, 3>(acc);
    if (lane < C) {
      float* dst = cluster.map_shared_rank(qf, lane);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int r = gw * rpw + i;
        if (i < rpw && r < nq) {
#pragma unroll
          for (int t = 0; t < T; ++t) dst[t * MAXQ + r] = bf16_round(acc[i][t]);
        }
      }
    }
  }
  cluster.sync();

  // ---- step 2: absorb (columns [64 cr + 8 warp, +8)), rotate q_pe ----
  {
    float v[T * 8];
#pragma unroll
    for (int i = 0; i < T * 8; ++i) v[i] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j < dpl) {
        float wf[8];
        unpack8(wv[j], wf);
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const float qd = qf[t * MAXQ + lane * dpl + j];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[t * 8 + i] = fmaf(qd, wf[i], v[t * 8 + i]);
        }
      }
    }
    warp_reduce_scatter<T * 8>(v, lane);
    constexpr int PER = (T * 8 + 31) / 32;          // values a lane owns after the scatter
    constexpr int DUP = 32 / (T * 8) > 0 ? 32 / (T * 8) : 1;   // lanes holding the same value
    if (lane % DUP == 0) {
#pragma unroll
      for (int k = 0; k < PER; ++k) {
        const int idx = (lane * T * 8) / 32 + k, t = idx >> 3, i = idx & 7;
        const bf16 val = __float2bfloat16_rn(v[k]);
        for (int d = 0; d < C; ++d) cluster.map_shared_rank(qlat, d)[t * ROW + cr * SLICE + warp * 8 + i] = val;
      }
    }
    for (int i = threadIdx.x; i < T * (ROPE / 2); i += blockDim.x) {
      const int t = i / (ROPE / 2), k = i % (ROPE / 2);
      float c, s;
      rope_cos_sin(s_pos[t] < 0 ? 0 : s_pos[t], k, ROPE, p.theta, &c, &s);
      const float a = qf[t * MAXQ + p.nope + k], b = qf[t * MAXQ + p.nope + k + ROPE / 2];
      qlat[t * ROW + LATENT + k] = __float2bfloat16_rn(a * c - b * s);
      qlat[t * ROW + LATENT + k + ROPE / 2] = __float2bfloat16_rn(b * c + a * s);
    }
  }
  // value up-projection slice of this thread: row j = tid / 2, columns 64 cr + 32 (tid % 2) + [0, 32)
  const int vj = threadIdx.x >> 1, vhalf = threadIdx.x & 1;
  uint4 wu[4];
  {
    const bf16* Wuv = p.w_kvb + ((long)h * (p.nope + p.vdim) + p.nope + vj) * LATENT + cr * SLICE + vhalf * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) wu[j] = vj < p.vdim ? ld_stream16(Wuv + j * 8) : make_uint4(0, 0, 0, 0);
  }
  cluster.sync();

  // ---- step 3: attention over the keys of every token, split over the 64 warps of the cluster ----
  for (int t = 0; t < T; ++t) {
    const int pos = s_pos[t];
    float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    if (pos >= 0) {
      int first, nctx;
      visible_range(pos, p.window, &first, &nctx);
      const int total = p.n_sinks + nctx, slot = s_slot[t];
      RowFrag q;
      load_row(qlat + t * ROW, lane, &q);
      constexpr int KB = 4;
      for (int kb = gw; kb < total; kb += NW * KB) {
        uint4 ra[KB], rb[KB];
        __nv_bfloat162 rr[KB];
        bool ok[KB];
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          const int k = kb + NW * j;
          ok[j] = k < total;
          if (!ok[j]) continue;
          const bf16* row;
          if (k < p.n_sinks) {
            row = p.sinks + (long)k * ROW;
          } else {
            const int kp = first + (k - p.n_sinks);
            row = nullptr;
#pragma unroll
            for (int t2 = 0; t2 < T; ++t2)
              if (s_pos[t2] == kp && s_slot[t2] == slot) row = newrow + t2 * ROW;
            if (row == nullptr) {
              const long r = cache_row_of(kp, slot, p.page_table, p.max_pages, p.page_tokens, p.num_pages);
              if (r < 0) {
                if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_BAD_INDEX);
                ok[j] = false;
                continue;
              }
              row = p.cache + r * ROW;
            }
          }
          ra[j] = *reinterpret_cast<const uint4*>(row + lane * 8);
          rb[j] = *reinterpret_cast<const uint4*>(row + 256 + lane * 8);
          rr[j] = *reinterpret_cast<const __nv_bfloat162*>(row + LATENT + lane * 2);
        }
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          if (!ok[j]) continue;
          RowFrag kf;
          unpack8(ra[j], kf.lat);
          unpack8(rb[j], kf.lat + 8);
          const float2 r2 = __bfloat1622float2(rr[j]);
          float s = q.rp[0] * r2.x + q.rp[1] * r2.y;
#pragma unroll
          for (int i = 0; i < 16; ++i) s = fmaf(q.lat[i], kf.lat[i], s);
          s = warp_sum(s) * p.scale;
          const float mn = fmaxf(m, s);
          const float corr = __expf(m - mn), pe = __expf(s - mn);
          l = l * corr + pe;
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = acc[i] * corr + pe * kf.lat[i];
          m = mn;
        }
      }
    }
    __syncthreads();   // wacc / wml of the previous token have been consumed
    if (lane == 0) {
      wml[warp] = m;
      wml[8 + warp] = l;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      wacc[warp * LATENT + lane * 8 + i] = acc[i];
      wacc[warp * LATENT + 256 + lane * 8 + i] = acc[8 + i];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) M = fmaxf(M, wml[w]);
    float wg[8], Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      wg[w] = (wml[w] == -INFINITY) ? 0.f : __expf(wml[w] - M);
      Lsum += wg[w] * wml[8 + w];
    }
    float* dst = part + t * (LATENT + 2);
    for (int c = threadIdx.x; c < LATENT; c += blockDim.x) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) v += wg[w] * wacc[w * LATENT + c];
      dst[c] = v;
    }
    if (threadIdx.x == 0) {
      dst[LATENT] = M;
      dst[LATENT + 1] = Lsum;
    }
  }
  cluster.sync();

  // ---- step 4: merge the 8 CTA partials on this CTA's 64 columns, multiply with the K-slice of W_UV ----
  for (int i = threadIdx.x; i < T * SLICE; i += blockDim.x) {
    const int t = i / SLICE, c = i % SLICE;
    float ms[C], M = -INFINITY;
#pragma unroll
    for (int r = 0; r < C; ++r) {
      ms[r] = cluster.map_shared_rank(part, r)[t * (LATENT + 2) + LATENT];
      M = fmaxf(M, ms[r]);
    }
    float Lsum = 0.f, v = 0.f;
#pragma unroll
    for (int r = 0; r < C; ++r) {
      const float* rp = cluster.map_shared_rank(part, r) + t * (LATENT + 2);
      const float w = (ms[r] == -INFINITY) ? 0.f : __expf(ms[r] - M);
      Lsum += w * rp[LATENT + 1];
      v += w * rp[cr * SLICE + c];
    }
    os[t * SLICE + c] = __float2bfloat16_rn(Lsum > 0.f ? v / Lsum : 0.f);
  }
  __syncthreads();
  {
    float wf[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) unpack8(wu[j], wf + 8 * j);
    float* ob = cluster.map_shared_rank(outbuf, 0) + (long)cr * T * 128;
#pragma unroll
    for (int t = 0; t < T; ++t) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float of[8];
        unpack8(*reinterpret_cast<const uint4*>(os + t * SLICE + vhalf * 32 + j * 8), of);
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(of[i], wf[j * 8 + i], d);
      }
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      if (vhalf == 0) ob[t * 128 + vj] = d;
    }
  }
  cluster.sync();
  if (cr == 0) {
    for (int i = threadIdx.x; i < T * 128; i += blockDim.x) {
      const int t = i >> 7, j = i & 127;
      if (t >= p.T || j >= p.vdim || s_pos[t] < 0) continue;
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < C; ++r) s += outbuf[((long)r * T + t) * 128 + j];
      p.out[(long)t * p.ldo + (long)h * p.vdim + j] = __float2bfloat16_rn(s);
    }
  }
}

template <int T>
int launch_head(const HeadParams& p, cudaStream_t s) {
  const Layout L = layout_for(T, p.q_lora);
  auto k = mla_head_decode_kernel<T>;
  if (int rc = opt_in_smem(k, L.total)) return rc;
  return launch_chain_cluster(k, dim3(C * p.H), dim3(256), C, L.total, s, p);
}

}  // namespace

// qkv: [T, q_lora + 576] (q latent | kv latent | k_pe), w_qb: [H * (nope + 64), q_lora], w_kvb: [H, nope + vdim, 512],
// cache: bf16 paged latent cache; out: [T, H * vdim]. T <= 8.
extern "C" int ifab_mla_head_decode_pf(const void* qkv, long ldqkv, const void* q_norm, const void* kv_norm, float eps, float theta,
                                       const void* w_qb, const void* w_kvb, void* cache, const int32_t* positions, const int32_t* slots,
                                       const int32_t* page_table, int max_pages, int page_tokens, int num_pages, const void* sinks,
                                       int n_sinks, int window, float scale, int T, int H, int q_lora, int nope, int vdim, void* out,
                                       long ldo, uint32_t* status, const void* pf0, uint64_t pf0_bytes, const void* pf1, uint64_t pf1_bytes,
                                       const void* pf2, uint64_t pf2_bytes, void* stream) {
  if (T < 1 || T > 8 || H < 1 || q_lora % 8 != 0 || ldqkv % 8 != 0 || nope % 32 != 0 || nope > 128 || vdim > 128 || vdim < 1) return -1;
  HeadParams p{(const bf16*)qkv, ldqkv, (const bf16*)q_norm, (const bf16*)kv_norm, eps, theta, (const bf16*)w_qb, (const bf16*)w_kvb,
               (bf16*)cache, positions, slots, page_table, max_pages, page_tokens, num_pages, (const bf16*)sinks, sinks ? n_sinks : 0,
               window, scale, T, H, q_lora, nope, vdim, (bf16*)out, ldo, status,
               {(const char*)pf0, (const char*)pf1, (const char*)pf2},
               {pf0 ? pf0_bytes : 0, pf1 ? pf1_bytes : 0, pf2 ? pf2_bytes : 0}};
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return launch_head<1>(p, s);
  if (T <= 2) return launch_head<2>(p, s);
  if (T <= 4) return launch_head<4>(p, s);
  return launch_head<8>(p, s);
}

extern "C" int ifab_mla_head_decode(const void* qkv, long ldqkv, const void* q_norm, const void* kv_norm, float eps, float theta,
                                    const void* w_qb, const void* w_kvb, void* cache, const int32_t* positions, const int32_t* slots,
                                    const int32_t* page_table, int max_pages, int page_tokens, int num_pages, const void* sinks,
                                    int n_sinks, int window, float scale, int T, int H, int q_lora, int nope, int vdim, void* out,
                                    long ldo, uint32_t* status, void* stream) {
  return ifab_mla_head_decode_pf(qkv, ldqkv, q_norm, kv_norm, eps, theta, w_qb, w_kvb, cache, positions, slots, page_table, max_pages, page_tokens,
                                 num_pages, sinks, n_sinks, window, scale, T, H, q_lora, nope, vdim, out, ldo, status, nullptr, 0, nullptr, 0, nullptr, 0,
                                 stream);
}
