// Multi-head latent attention, decode / short-chunk path, for sm_100a.
//
// The KV cache keeps ONE row per token shared by all heads: [latent(512) bf16 | rope(64) bf16], in
// pages of `page_tokens` rows addressed through a per-sequence page table. Queries are "absorbed":
// q_nope is multiplied by W_UK so scores are taken directly against the latent rows, and the
// value up-projection W_UV is applied once to the attention output.
//
//   mla_kv_write_kernel     RMSNorm(latent) + RoPE(k_pe) + paged scatter (one CTA per token)
//   mla_q_absorb_kernel     q_lat[h] = [ q_nope[h] W_UK[h] | RoPE(q_rope[h]) ]
//   mla_split_kernel        split-KV online-softmax attention over the paged cache (+ learned sink
//                           rows, sliding window); partial (m, l, acc) per split go to scratch
//   mla_merge_vup_kernel    log-sum-exp merge of the splits + W_UV up-projection -> [T, H*vdim]
//
// Every query row carries its own position and sequence slot, so the same kernels serve
// single-sequence decode, batched decode and short causal prefill chunks (rows of one chunk are
// written to the cache first; row i then sees keys <= position i).
//
// Reference counterparts: cache_norm_rope_append (KvRmsNormRopeCache), mla_query (BatchMatMul +
// rotary + concat), latent_attention (FusedInferAttentionSink) and mla_value
// (native/src/token_executor.h:613-909).
#include "gemv.cuh"
#include "mla_common.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::mla;

namespace {

// ------------------------------------------------------------------------------------------------
// `kr` (optional): the rotary columns when they do not follow the latent columns in `kv` (e.g. a convolved latent)
__global__ void __launch_bounds__(128) mla_kv_write_kernel(const bf16* kv, long ldkv, const bf16* kr, long ldkr, const bf16* norm_w, float eps,
                                                           float theta, const int32_t* positions, const int32_t* slots,
                                                           const int32_t* page_table, int max_pages, int page_tokens,
                                                           bf16* cache, int num_pages, int latent, int rope,
                                                           uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  const long row = cache_row_of(pos, slots[t], page_table, max_pages, page_tokens, num_pages);
  if (row < 0) {
    if (threadIdx.x == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    return;
  }
  __shared__ float red[4];
  const bf16* src = kv + (long)t * ldkv;
  bf16* dst = cache + row * (latent + rope);
  const int tid = threadIdx.x;
  float f[8];
  float ss = 0.f;
  const bool has = tid < latent / 8;
  if (has) {
    unpack8(*reinterpret_cast<const uint4*>(src + tid * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)latent + eps);
  if (has) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(norm_w + tid * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i];
    *reinterpret_cast<uint4*>(dst + tid * 8) = pack8(f);
  }
  const int half = rope / 2;
  if (tid < half) {
    float c, s;
    rope_cos_sin(pos, tid, rope, theta, &c, &s);
    const bf16* rs = kr ? kr + (long)t * ldkr : src + latent;
    const float a = __bfloat162float(rs[tid]), b = __bfloat162float(rs[tid + half]);
    dst[latent + tid] = __float2bfloat16_rn(a * c - b * s);
    dst[latent + tid + half] = __float2bfloat16_rn(b * c + a * s);
  }
}

// ------------------------------------------------------------------------------------------------
// grid (H, T, latent/128), 256 threads. A CTA produces 128 latent columns of one head: thread
// (ds, cg) = (tid / 16, tid % 16) owns 8 columns [cg*8, cg*8+8) and the 8 q_nope elements
// [ds*8, ds*8+8); its 8 weight loads (16 bytes each) are issued before the dependency wait, the 16
// d-slices are then summed through shared memory. CTA z == 0 also rotates the rope part.
__global__ void __launch_bounds__(256) mla_q_absorb_kernel(const bf16* q, long ldq, const bf16* w_kvb, float theta,
                                                           const int32_t* positions, bf16* q_lat, int H, int nope,
                                                           int rope, int latent, int vdim) {
  __shared__ float qs[256];
  __shared__ float part[16][129];
  grid_dep_launch();
  const int h = blockIdx.x, t = blockIdx.y, cbase = blockIdx.z * 128;
  const int cg = threadIdx.x & 15, ds = threadIdx.x >> 4;
  const bf16* W = w_kvb + (long)h * (nope + vdim) * latent + cbase + cg * 8;
  uint4 wv[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = ds * 8 + j;
    wv[j] = d < nope ? ld_stream16(W + (long)d * latent) : make_uint4(0, 0, 0, 0);
  }
  grid_dep_wait();
  const int pos = positions[t];
  const bf16* qrow = q + (long)t * ldq + (long)h * (nope + rope);
  for (int i = threadIdx.x; i < nope; i += blockDim.x) qs[i] = __bfloat162float(qrow[i]);
  __syncthreads();
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int d0 = ds * 8; d0 < nope; d0 += 128) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = d0 + j;
      if (d >= nope) break;
      float wf[8];
      unpack8(d0 == ds * 8 ? wv[j] : ld_stream16(W + (long)d * latent), wf);
      const float qd = qs[d];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(qd, wf[i], acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[ds][cg * 8 + i] = acc[i];
  __syncthreads();
  bf16* out = q_lat + ((long)t * H + h) * (latent + rope);
  if (threadIdx.x < 128) {
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) v += part[k][threadIdx.x];
    out[cbase + threadIdx.x] = __float2bfloat16_rn(v);
  }
  const int half = rope / 2;
  if (blockIdx.z == 0 && (int)threadIdx.x >= 128 && (int)threadIdx.x - 128 < half) {
    const int i = threadIdx.x - 128;
    float c, sn;
    rope_cos_sin(pos < 0 ? 0 : pos, i, rope, theta, &c, &sn);
    const float a = __bfloat162float(qrow[nope + i]), b2 = __bfloat162float(qrow[nope + i + half]);
    out[latent + i] = __float2bfloat16_rn(a * c - b2 * sn);
    out[latent + i + half] = __float2bfloat16_rn(b2 * c + a * sn);
  }
}

// ------------------------------------------------------------------------------------------------
struct AttnParams {
  const bf16* q_lat; const bf16* cache; const int32_t* positions; const int32_t* slots; const int32_t* page_table;
  int max_pages, page_tokens, num_pages;
  const bf16* sinks; int n_sinks, window; float scale;
  int T, H, kps, max_splits;
  float* scratch;   // [T][H][max_splits][LATENT + 2]
  uint32_t* status;
  int q8;           // cache rows are packed: 512 int8 | 64 bf16 rope | 4 f32 scales (one per 128 latent columns) = 656 bytes
  const int32_t* indices;   // optional learned selection [T][n_index]: the key positions a row attends to, ascending, -1 padded
  int n_index;
};

// keys of a query row: sink rows first, then either the window's positions or the selected ones
__device__ __forceinline__ void key_space(const AttnParams& p, int pos, int* first, int* nctx) {
  visible_range(pos, p.window, first, nctx);
  if (p.indices) *nctx = min(p.n_index, pos + 1);       // the selector emits min(topk, pos + 1) positions
}

constexpr int ROW_Q8 = LATENT + ROPE * 2 + 16;

template <int HG>
__global__ void __launch_bounds__(256) mla_split_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sm_acc = reinterpret_cast<float*>(smem_raw);            // [8][HG][LATENT]
  float* sm_m = sm_acc + 8 * HG * LATENT;                        // [8][HG]
  float* sm_l = sm_m + 8 * HG;                                   // [8][HG]
  grid_dep_launch();
  grid_dep_wait();
  const int split = blockIdx.x, hg = blockIdx.y, t = blockIdx.z;
  const int pos = p.positions[t];
  if (pos < 0) return;
  int first, nctx;
  key_space(p, pos, &first, &nctx);
  const int total = p.n_sinks + nctx;
  const int k_begin = split * p.kps;
  if (k_begin >= total) return;
  // the last split also takes every key beyond max_splits * keys_per_split, so a long context is slower, never clipped
  const int k_end = (split == p.max_splits - 1) ? total : min(total, k_begin + p.kps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = p.slots[t];

  RowFrag qf[HG];
#pragma unroll
  for (int g = 0; g < HG; ++g) load_row(p.q_lat + ((long)t * p.H + hg * HG + g) * ROW, lane, &qf[g]);
  float m[HG], l[HG], acc[HG][16];
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[g][i] = 0.f;
  }
  // Each warp owns keys k_begin + warp, +8, ...; the rows of a batch of KB keys are all requested
  // before the first score is computed, so their latencies overlap.
  constexpr int KB = 4;
  for (int kb = k_begin + warp; kb < k_end; kb += 8 * KB) {
    uint4 ra[KB], rb[KB];
    __nv_bfloat162 rr[KB];
    bool ok[KB], packed[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const int k = kb + 8 * j;
      ok[j] = k < k_end;
      const bf16* row = nullptr;
      packed[j] = false;
      if (ok[j]) {
        if (k < p.n_sinks) {
          row = p.sinks + (long)k * ROW;
        } else {
          int kp = first + (k - p.n_sinks);
          bool skip = false;
          if (p.indices) {
            kp = p.indices[(long)t * p.n_index + (k - p.n_sinks)];
            skip = kp < first || kp > pos;                 // padding, or a selected position the window no longer shows
          }
          const long r = skip ? 0 : cache_row_of(kp, slot, p.page_table, p.max_pages, p.page_tokens, p.num_pages);
          if (skip) {
            ok[j] = false;
          } else if (r < 0) {
            if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_BAD_INDEX);
            ok[j] = false;
          } else if (p.q8) {
            // packed row: this lane's 8 + 8 int8 latents travel in ra, the two tile scales in rb
            const unsigned char* r8 = reinterpret_cast<const unsigned char*>(p.cache) + r * ROW_Q8;
            const uint2 a8 = *reinterpret_cast<const uint2*>(r8 + lane * 8);
            const uint2 b8 = *reinterpret_cast<const uint2*>(r8 + 256 + lane * 8);
            ra[j] = make_uint4(a8.x, a8.y, b8.x, b8.y);
            rb[j].x = *reinterpret_cast<const uint32_t*>(r8 + LATENT + ROPE * 2 + 4 * (lane >> 4));
            rb[j].y = *reinterpret_cast<const uint32_t*>(r8 + LATENT + ROPE * 2 + 4 * (2 + (lane >> 4)));
            rr[j] = *reinterpret_cast<const __nv_bfloat162*>(r8 + LATENT + lane * 4);
            packed[j] = true;
          } else {
            row = p.cache + r * ROW;
          }
        }
      }
      if (ok[j] && !packed[j]) {
        ra[j] = *reinterpret_cast<const uint4*>(row + lane * 8);
        rb[j] = *reinterpret_cast<const uint4*>(row + 256 + lane * 8);
        rr[j] = *reinterpret_cast<const __nv_bfloat162*>(row + LATENT + lane * 2);
      }
    }
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      if (!ok[j]) continue;
      RowFrag kf;
      if (packed[j]) {
        const float sa = __uint_as_float(rb[j].x), sb = __uint_as_float(rb[j].y);
        const uint32_t w[4] = {ra[j].x, ra[j].y, ra[j].z, ra[j].w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int q = (int)(signed char)((w[i >> 2] >> (8 * (i & 3))) & 0xff);
          kf.lat[i] = (float)q * (i < 8 ? sa : sb);
        }
      } else {
        unpack8(ra[j], kf.lat);
        unpack8(rb[j], kf.lat + 8);
      }
      const float2 r2 = __bfloat1622float2(rr[j]);
      kf.rp[0] = r2.x;
      kf.rp[1] = r2.y;
#pragma unroll
      for (int g = 0; g < HG; ++g) {
        float s = qf[g].rp[0] * kf.rp[0] + qf[g].rp[1] * kf.rp[1];
#pragma unroll
        for (int i = 0; i < 16; ++i) s = fmaf(qf[g].lat[i], kf.lat[i], s);
        s = warp_sum(s) * p.scale;
        const float mn = fmaxf(m[g], s);
        const float corr = __expf(m[g] - mn), pe = __expf(s - mn);
        l[g] = l[g] * corr + pe;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[g][i] = acc[g][i] * corr + pe * kf.lat[i];
        m[g] = mn;
      }
    }
  }
#pragma unroll
  for (int g = 0; g < HG; ++g) {
    if (lane == 0) {
      sm_m[warp * HG + g] = m[g];
      sm_l[warp * HG + g] = l[g];
    }
    float* dst = sm_acc + ((long)warp * HG + g) * LATENT;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dst[lane * 8 + i] = acc[g][i];
      dst[256 + lane * 8 + i] = acc[g][8 + i];
    }
  }
  __syncthreads();
  // fixed-order merge of the 8 warps
  for (int g = 0; g < HG; ++g) {
    float M = -INFINITY;
    for (int w = 0; w < 8; ++w) M = fmaxf(M, sm_m[w * HG + g]);
    float wgt[8], L = 0.f;
    for (int w = 0; w < 8; ++w) {
      wgt[w] = (sm_m[w * HG + g] == -INFINITY) ? 0.f : __expf(sm_m[w * HG + g] - M);
      L += wgt[w] * sm_l[w * HG + g];
    }
    float* out = p.scratch + (((long)t * p.H + hg * HG + g) * p.max_splits + split) * (LATENT + 2);
    for (int c = threadIdx.x; c < LATENT; c += blockDim.x) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += wgt[w] * sm_acc[((long)w * HG + g) * LATENT + c];
      out[c] = v;
    }
    if (threadIdx.x == 0) {
      out[LATENT] = M;
      out[LATENT + 1] = L;
    }
  }
}

// grid (H, T): merge splits, then out[t][h*vdim + j] = sum_c o[c] * W_UV[h][j][c]
__global__ void __launch_bounds__(256) mla_merge_vup_kernel(AttnParams p, const bf16* w_kvb, int nope, int vdim,
                                                            bf16* out, long ldo) {
  __shared__ __align__(16) bf16 os[LATENT];
  __shared__ float wgt[64];
  __shared__ float Ls;
  grid_dep_launch();
  const int h = blockIdx.x, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int RV = 8;
  const bf16* W = w_kvb + ((long)h * (nope + vdim) + nope) * LATENT;
  const bf16* rows[RV];
#pragma unroll
  for (int r = 0; r < RV; ++r) rows[r] = (warp * RV + r < vdim) ? W + (long)(warp * RV + r) * LATENT : nullptr;
  RowBatch<RV> pf;
  prefetch_rows<RV>(rows, LATENT, pf);
  grid_dep_wait();
  const int pos = p.positions[t];
  if (pos < 0) return;
  int first, nctx;
  key_space(p, pos, &first, &nctx);
  const int total = p.n_sinks + nctx;
  int ns = (total + p.kps - 1) / p.kps;
  if (ns > p.max_splits) ns = p.max_splits;
  const float* base = p.scratch + ((long)t * p.H + h) * p.max_splits * (LATENT + 2);
  if (threadIdx.x == 0) {
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, base[(long)s * (LATENT + 2) + LATENT]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float ms = base[(long)s * (LATENT + 2) + LATENT];
      const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
      wgt[s] = w;
      L += w * base[(long)s * (LATENT + 2) + LATENT + 1];
    }
    Ls = L;
  }
  __syncthreads();
  const float invL = Ls > 0.f ? 1.f / Ls : 0.f;
  for (int c = threadIdx.x; c < LATENT; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < ns; ++s) v += wgt[s] * base[(long)s * (LATENT + 2) + c];
    os[c] = __float2bfloat16_rn(v * invL);
  }
  __syncthreads();
  for (int j0 = warp * RV, it = 0; j0 < vdim; j0 += 8 * RV, ++it) {
    if (it > 0) {
#pragma unroll
      for (int r = 0; r < RV; ++r) rows[r] = (j0 + r < vdim) ? W + (long)(j0 + r) * LATENT : nullptr;
      prefetch_rows<RV>(rows, LATENT, pf);
    }
    float acc[RV][1];
#pragma unroll
    for (int r = 0; r < RV; ++r) acc[r][0] = 0.f;
    warp_rows_dot<1, RV>(rows, os, LATENT, acc, pf);
    warp_reduce_acc<1, RV>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RV; ++r)
        if (j0 + r < vdim) out[(long)t * ldo + (long)h * vdim + j0 + r] = __float2bfloat16_rn(acc[r][0]);
    }
  }
}

template <int HG>
int launch_split(const AttnParams& p, cudaStream_t s) {
  const size_t smem = (size_t)(8 * HG * LATENT + 16 * HG) * sizeof(float);
  auto k = mla_split_kernel<HG>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid(p.max_splits, p.H / HG, p.T);
  return launch_chain(k, grid, dim3(256), smem, s, p);
}

}  // namespace

extern "C" int ifab_mla_kv_write(const void* kv, long ldkv, const void* norm_w, float eps, float theta,
                                 const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                 int max_pages, int page_tokens, void* cache, int num_pages, int T, int latent, int rope,
                                 uint32_t* status, void* stream) {
  if (latent % 8 != 0 || latent > 1024 || rope % 2 != 0 || rope > 256 || ldkv % 8 != 0) return -1;
  return launch_chain(mla_kv_write_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, (const bf16*)kv, ldkv, (const bf16*)nullptr, 0L,
                      (const bf16*)norm_w, eps, theta, positions, slots, page_table, max_pages, page_tokens,
                      (bf16*)cache, num_pages, latent, rope, status);
}

extern "C" int ifab_mla_kv_write_split(const void* latent_rows, long ldl, const void* rope_rows, long ldr, const void* norm_w, float eps, float theta,
                                       const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens,
                                       void* cache, int num_pages, int T, int latent, int rope, uint32_t* status, void* stream) {
  if (latent % 8 != 0 || latent > 1024 || rope % 2 != 0 || rope > 256 || ldl % 8 != 0 || !rope_rows) return -1;
  return launch_chain(mla_kv_write_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, (const bf16*)latent_rows, ldl, (const bf16*)rope_rows, ldr,
                      (const bf16*)norm_w, eps, theta, positions, slots, page_table, max_pages, page_tokens,
                      (bf16*)cache, num_pages, latent, rope, status);
}

extern "C" int ifab_mla_q_absorb(const void* q, long ldq, const void* w_kvb, float theta, const int32_t* positions,
                                 void* q_lat, int T, int H, int nope, int rope, int latent, int vdim, void* stream) {
  if (nope > 256 || nope % 8 != 0 || latent % 128 != 0 || rope % 2 != 0 || rope > 256) return -1;
  dim3 grid(H, T, latent / 128);
  return launch_chain(mla_q_absorb_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)q, ldq,
                      (const bf16*)w_kvb, theta, positions, (bf16*)q_lat, H, nope, rope, latent, vdim);
}

extern "C" int ifab_mla_decode_attention_indexed(const void* q_lat, const void* cache, const int32_t* positions,
                                         const int32_t* slots, const int32_t* page_table, int max_pages,
                                         int page_tokens, int num_pages, const void* sinks, int n_sinks, int window,
                                         float scale, int T, int H, int latent, int rope, int keys_per_split,
                                         int max_splits, float* scratch, uint64_t scratch_bytes, const void* w_kvb,
                                         int nope, int vdim, void* out, long ldo, uint32_t* status, const int32_t* indices, int n_index,
                                         void* stream) {
  if (indices && n_index < 1) return -1;
  if (latent != LATENT || (rope != ROPE && rope != -ROPE)) return -1;
  if (max_splits < 1 || max_splits > 64 || keys_per_split < 8) return -1;
  if ((uint64_t)T * H * max_splits * (LATENT + 2) * sizeof(float) > scratch_bytes) return -5;
  // a negative `rope` selects the packed int8 cache layout (656-byte rows written by ifab_mla_kv_write_q8)
  const int q8 = rope < 0 ? 1 : 0;
  if (q8) rope = -rope;
  AttnParams p{(const bf16*)q_lat, (const bf16*)cache, positions, slots, page_table, max_pages, page_tokens, num_pages,
               (const bf16*)sinks, sinks ? n_sinks : 0, window, scale, T, H, keys_per_split, max_splits, scratch, status, q8, indices, indices ? n_index : 0};
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (H % 4 == 0) rc = launch_split<4>(p, s);
  else if (H % 2 == 0) rc = launch_split<2>(p, s);
  else rc = launch_split<1>(p, s);
  if (rc) return rc;
  if (w_kvb == nullptr) return 0;   // split partials only: the caller merges (ifab_mla_merge) and up-projects with a GEMM
  dim3 grid(H, T);
  return launch_chain(mla_merge_vup_kernel, grid, dim3(256), 0, s, p, (const bf16*)w_kvb, nope, vdim, (bf16*)out, ldo);
}

extern "C" int ifab_mla_decode_attention(const void* q_lat, const void* cache, const int32_t* positions,
                                         const int32_t* slots, const int32_t* page_table, int max_pages,
                                         int page_tokens, int num_pages, const void* sinks, int n_sinks, int window,
                                         float scale, int T, int H, int latent, int rope, int keys_per_split,
                                         int max_splits, float* scratch, uint64_t scratch_bytes, const void* w_kvb,
                                         int nope, int vdim, void* out, long ldo, uint32_t* status, void* stream) {
  return ifab_mla_decode_attention_indexed(q_lat, cache, positions, slots, page_table, max_pages, page_tokens, num_pages, sinks, n_sinks, window, scale, T, H,
                                           latent, rope, keys_per_split, max_splits, scratch, scratch_bytes, w_kvb, nope, vdim, out, ldo, status, nullptr, 0,
                                           stream);
}
