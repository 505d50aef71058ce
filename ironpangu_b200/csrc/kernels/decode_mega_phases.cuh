// Phase bodies of the persistent decode-step kernel (see decode_mega.cuh for the overall design).
// Every function is called by all threads of a CTA; control flow that reaches a __syncthreads() is uniform per CTA.
#pragma once
#include "decode_mega.cuh"

namespace ifab::mega {

// x[t] = embed[tokens[t]]
__device__ __forceinline__ void phase_embedding(const Params& p) {
  for (int t = blockIdx.x; t < p.T_live; t += gridDim.x) {
    int id = p.tokens[t];
    if (id < 0 || id >= p.vocab) {
      if (threadIdx.x == 0) atomicOr(p.fv.status, IFAB_STATUS_BAD_INDEX);
      id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.embed + (long)id * p.D);
    uint4* dst = reinterpret_cast<uint4*>(p.x + (long)t * p.D);
    for (int c = threadIdx.x; c < p.D / 8; c += THREADS) dst[c] = src[c];
  }
}

// latent row of token t: RMSNorm(latent) | RoPE(k_pe) -> its page of the cache (whole CTA, threads < 128 carry data)
__device__ __forceinline__ void kv_write_cta(const Params& p, const Layer& L, int t, float* red /* >= 8 floats */) {
  const int pos = p.positions[t];
  if (pos < 0) return;
  const long row = cache_row_of(pos, p.slots[t], p.page_table, p.max_pages, p.page_tokens, p.num_pages);
  if (row < 0) {
    if (threadIdx.x == 0) atomicOr(p.fv.status, IFAB_STATUS_BAD_INDEX);
    return;
  }
  const int NQ = p.q_lora + ROW;
  const bf16* src = p.qkv + (long)t * NQ + p.q_lora;
  bf16* dst = L.cache + row * ROW;
  const int tid = threadIdx.x;
  float f[8];
  float ss = 0.f;
  const bool has = tid < LATENT / 8;
  if (has) {
    unpack8(ld_act16(src + tid * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)LATENT + p.eps);
  if (has) {
    float g[8];
    unpack8(*reinterpret_cast<const uint4*>(L.kv_a_norm + tid * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i];
    *reinterpret_cast<uint4*>(dst + tid * 8) = pack8(f);
  }
  const int half = ROPE / 2;
  if (tid < half) {
    float c, s;
    rope_cos_sin(pos, tid, ROPE, p.theta, &c, &s);
    const float a = ld_act_bf16(src + LATENT + tid), b = ld_act_bf16(src + LATENT + tid + half);
    dst[LATENT + tid] = __float2bfloat16_rn(a * c - b * s);
    dst[LATENT + tid + half] = __float2bfloat16_rn(b * c + a * s);
  }
  __syncthreads();
}

// q_lat[t][h] = q_nope @ W_uk[h] (512 columns in 4 units of 128) | RoPE(q_pe). smem: 256 + 16*129 floats.
__device__ __forceinline__ void phase_absorb(const Params& p, const Layer& L, float* smem) {
  float* qs = smem;
  float* part = smem + 256;   // [16][129]
  const int cz_n = LATENT / 128;
  const int units = p.hl * p.T_live * cz_n;
  const int qk = p.nope + p.rope;
  const int cg = threadIdx.x & 15, ds = threadIdx.x >> 4;
  for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
    const int cz = vb % cz_n, h = (vb / cz_n) % p.hl, t = vb / (cz_n * p.hl);
    const int cbase = cz * 128;
    const bf16* W = L.kv_b + (long)h * (p.nope + p.vdim) * LATENT + cbase + cg * 8;
    uint4 wv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = ds * 8 + j;
      wv[j] = d < p.nope ? ld_stream16(W + (long)d * LATENT) : make_uint4(0, 0, 0, 0);
    }
    const int pos = p.positions[t];
    const bf16* qrow = p.q + (long)t * p.hl * qk + (long)h * qk;
    for (int i = threadIdx.x; i < p.nope; i += THREADS) qs[i] = ld_act_bf16(qrow + i);
    __syncthreads();
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int d0 = ds * 8; d0 < p.nope; d0 += 128) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = d0 + j;
        if (d >= p.nope) break;
        float wf[8];
        unpack8(d0 == ds * 8 ? wv[j] : ld_stream16(W + (long)d * LATENT), wf);
        const float qd = qs[d];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(qd, wf[i], acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) part[ds * 129 + cg * 8 + i] = acc[i];
    __syncthreads();
    bf16* out = p.q_lat + ((long)t * p.hl + h) * ROW;
    if (threadIdx.x < 128) {
      float v = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) v += part[k * 129 + threadIdx.x];
      out[cbase + threadIdx.x] = __float2bfloat16_rn(v);
    }
    const int half = p.rope / 2;
    if (cz == 0 && (int)threadIdx.x >= 128 && (int)threadIdx.x - 128 < half) {
      const int i = threadIdx.x - 128;
      float c, sn;
      rope_cos_sin(pos < 0 ? 0 : pos, i, p.rope, p.theta, &c, &sn);
      const float a = ld_act_bf16(qrow + p.nope + i), b2 = ld_act_bf16(qrow + p.nope + i + half);
      out[LATENT + i] = __float2bfloat16_rn(a * c - b2 * sn);
      out[LATENT + i + half] = __float2bfloat16_rn(b2 * c + a * sn);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void load_row_cg(const bf16* row, int lane, RowFrag* f) {
  const uint4 a = ld_act16(row + lane * 8);
  const uint4 b = ld_act16(row + 256 + lane * 8);
  const uint32_t r = __ldcg(reinterpret_cast<const uint32_t*>(row + LATENT + lane * 2));
  unpack8(a, f->lat);
  unpack8(b, f->lat + 8);
  f->rp[0] = __uint_as_float(r << 16);
  f->rp[1] = __uint_as_float(r & 0xffff0000u);
}

// split-KV attention of HG heads over one key range; smem: (8*HG*512 + 16*HG) floats
template <int HG>
__device__ __forceinline__ void phase_split(const Params& p, const Layer& L, float* smem) {
  float* sm_acc = smem;                    // [8][HG][LATENT]
  float* sm_m = sm_acc + 8 * HG * LATENT;  // [8][HG]
  float* sm_l = sm_m + 8 * HG;             // [8][HG]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hgs = p.hl / HG;
  const int units = p.max_splits * hgs * p.T_live;
  for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
    const int split = vb % p.max_splits, hg = (vb / p.max_splits) % hgs, t = vb / (p.max_splits * hgs);
    const int pos = p.positions[t];
    if (pos < 0) continue;
    int first, nctx;
    visible_range(pos, p.window, &first, &nctx);
    const int total = p.n_sinks + nctx;
    const int k_begin = split * p.kps;
    if (k_begin >= total) continue;
    const int k_end = (split == p.max_splits - 1) ? total : min(total, k_begin + p.kps);   // the last split takes the tail
    const int slot = p.slots[t];
    RowFrag qf[HG];
#pragma unroll
    for (int g = 0; g < HG; ++g) load_row_cg(p.q_lat + ((long)t * p.hl + hg * HG + g) * ROW, lane, &qf[g]);
    float m[HG], l[HG], acc[HG][16];
#pragma unroll
    for (int g = 0; g < HG; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[g][i] = 0.f;
    }
    constexpr int KB = 4;
    for (int kb = k_begin + warp; kb < k_end; kb += 8 * KB) {
      uint4 ra[KB], rb[KB];
      uint32_t rr[KB];
      bool ok[KB];
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        const int k = kb + 8 * j;
        ok[j] = k < k_end;
        const bf16* row = nullptr;
        if (ok[j]) {
          if (k < p.n_sinks) {
            row = L.sinks + (long)k * ROW;
          } else {
            const long r = cache_row_of(first + (k - p.n_sinks), slot, p.page_table, p.max_pages, p.page_tokens, p.num_pages);
            if (r < 0) {
              if (lane == 0) atomicOr(p.fv.status, IFAB_STATUS_BAD_INDEX);
              ok[j] = false;
            } else {
              row = L.cache + r * ROW;
            }
          }
        }
        if (ok[j]) {
          ra[j] = ld_act16(row + lane * 8);
          rb[j] = ld_act16(row + 256 + lane * 8);
          rr[j] = __ldcg(reinterpret_cast<const uint32_t*>(row + LATENT + lane * 2));
        }
      }
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        if (!ok[j]) continue;
        RowFrag kf;
        unpack8(ra[j], kf.lat);
        unpack8(rb[j], kf.lat + 8);
        kf.rp[0] = __uint_as_float(rr[j] << 16);
        kf.rp[1] = __uint_as_float(rr[j] & 0xffff0000u);
#pragma unroll
        for (int g = 0; g < HG; ++g) {
          float s = qf[g].rp[0] * kf.rp[0] + qf[g].rp[1] * kf.rp[1];
#pragma unroll
          for (int i = 0; i < 16; ++i) s = fmaf(qf[g].lat[i], kf.lat[i], s);
          s = warp_sum(s) * p.attn_scale;
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
    for (int g = 0; g < HG; ++g) {
      float M = -INFINITY;
      for (int w = 0; w < 8; ++w) M = fmaxf(M, sm_m[w * HG + g]);
      float wgt[8], Lsum = 0.f;
      for (int w = 0; w < 8; ++w) {
        wgt[w] = (sm_m[w * HG + g] == -INFINITY) ? 0.f : __expf(sm_m[w * HG + g] - M);
        Lsum += wgt[w] * sm_l[w * HG + g];
      }
      float* out = p.scratch + (((long)t * p.hl + hg * HG + g) * p.max_splits + split) * (LATENT + 2);
      for (int c = threadIdx.x; c < LATENT; c += THREADS) {
        float v = 0.f;
        for (int w = 0; w < 8; ++w) v += wgt[w] * sm_acc[((long)w * HG + g) * LATENT + c];
        out[c] = v;
      }
      if (threadIdx.x == 0) {
        out[LATENT] = M;
        out[LATENT + 1] = Lsum;
      }
    }
    __syncthreads();
  }
}

// LSE merge of the splits of (t, h) and 32 rows of the value up-projection per unit; smem: bf16[512] + 65 floats
__device__ __forceinline__ void phase_merge_vup(const Params& p, const Layer& L, unsigned char* smem) {
  bf16* os = reinterpret_cast<bf16*>(smem);
  float* wgt = reinterpret_cast<float*>(smem + LATENT * sizeof(bf16));   // [64] + Ls
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvs = (p.vdim + 31) / 32;
  const int units = p.hl * p.T_live * nvs;
  for (int vb = blockIdx.x; vb < units; vb += gridDim.x) {
    const int vs = vb % nvs, h = (vb / nvs) % p.hl, t = vb / (nvs * p.hl);
    const int pos = p.positions[t];
    if (pos < 0) continue;
    constexpr int RV = 4;
    const bf16* W = L.kv_b + ((long)h * (p.nope + p.vdim) + p.nope) * LATENT;
    const int j0 = vs * 32 + warp * RV;
    const bf16* rows[RV];
#pragma unroll
    for (int r = 0; r < RV; ++r) rows[r] = (j0 + r < p.vdim) ? W + (long)(j0 + r) * LATENT : nullptr;
    RowBatch<RV, MD> pf;
    prefetch_rows<RV, MD>(rows, LATENT, pf);
    int first, nctx;
    visible_range(pos, p.window, &first, &nctx);
    const int total = p.n_sinks + nctx;
    int ns = (total + p.kps - 1) / p.kps;
    if (ns > p.max_splits) ns = p.max_splits;
    const float* base = p.scratch + ((long)t * p.hl + h) * p.max_splits * (LATENT + 2);
    if (threadIdx.x == 0) {
      float M = -INFINITY;
      for (int s = 0; s < ns; ++s) M = fmaxf(M, __ldcg(base + (long)s * (LATENT + 2) + LATENT));
      float Lsum = 0.f;
      for (int s = 0; s < ns; ++s) {
        const float ms = __ldcg(base + (long)s * (LATENT + 2) + LATENT);
        const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
        wgt[s] = w;
        Lsum += w * __ldcg(base + (long)s * (LATENT + 2) + LATENT + 1);
      }
      wgt[64] = Lsum;
    }
    __syncthreads();
    const float Ls = wgt[64];
    const float invL = Ls > 0.f ? 1.f / Ls : 0.f;
    for (int c = threadIdx.x; c < LATENT; c += THREADS) {
      float v = 0.f;
      for (int s = 0; s < ns; ++s) v += wgt[s] * __ldcg(base + (long)s * (LATENT + 2) + c);
      os[c] = __float2bfloat16_rn(v * invL);
    }
    __syncthreads();
    float acc[RV][1];
#pragma unroll
    for (int r = 0; r < RV; ++r) acc[r][0] = 0.f;
    warp_rows_dot<1, RV, MD>(rows, os, LATENT, acc, pf);
    warp_reduce_acc<1, RV>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RV; ++r)
        if (j0 + r < p.vdim) p.attn[(long)t * p.hl * p.vdim + (long)h * p.vdim + j0 + r] = __float2bfloat16_rn(acc[r][0]);
    }
    __syncthreads();
  }
}

}  // namespace ifab::mega
