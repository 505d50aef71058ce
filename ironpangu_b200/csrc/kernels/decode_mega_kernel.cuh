// The persistent decode-step kernel and its launcher (design: decode_mega.cuh; attention phases: decode_mega_phases.cuh).
#pragma once
#include "decode_mega_phases.cuh"

namespace ifab::mega {

// Shared-memory state of one CTA that is not phase-local.
template <int T>
struct CtaState {
  float red[T * 33];
  float own[WARPS][AR_ROWS][T];        // this rank's partial sums of the rows a warp owns in an all-reduce phase
  int rids[T][MAX_TOPK];               // routes of every token (all experts, global ids)
  float rw[T][MAX_TOPK];
  int route_t[MAX_ROUTES], route_slot[MAX_ROUTES], route_e[MAX_ROUTES];   // local routes, token-major
  int n_routes;
  const bf16* dw[MAX_TOPK + 1];        // down phase, current token: weight base, score, K extent, first chunk, slot
  float dg[MAX_TOPK + 1];
  int dk[MAX_TOPK + 1], dcbeg[MAX_TOPK + 2], dslot[MAX_TOPK + 1];
  int dn;
  float bestv[WARPS][T];
  int besti[WARPS][T];
  int ok;
};

// Row-parallel GEMV (rows of W over this rank's K shard) + all-reduce + residual add into x.
template <int T, int R>
__device__ __forceinline__ void ar_gemv_phase(const Params& p, const ArCtx& ar, const bf16* W, int K, const bf16* xs,
                                              CtaState<T>& st, int gw, int GW) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TL = p.T_live, D = p.D;
  const int units = (D + R - 1) / R;
  int nown = 0;
  for (int u = gw; u < units && (nown + 1) * R <= AR_ROWS; u += GW, ++nown) {
    const bf16* wrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wrow[r] = (u * R + r < D) ? W + (size_t)(u * R + r) * K : nullptr;
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    warp_rows_dot<T, R>(wrow, xs, K, acc);
    warp_reduce_acc<T, R>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) st.own[warp][nown * R + r][t] = acc[r][t];
    }
    __syncwarp();
    if (ar.fv.world > 1) {
      for (int i = lane; i < R * T; i += 32) {
        const int r = i / T, t = i % T, col = u * R + r;
        if (col < D && t < TL) ar_push(ar, t, TL, col, D, st.own[warp][nown * R + r][t]);
      }
    }
  }
  bool ok = true;
  for (int k = 0, u = gw; k < nown; ++k, u += GW) {
    for (int i = lane; i < R * T; i += 32) {
      const int r = i / T, t = i % T, col = u * R + r;
      if (col >= D || t >= TL) continue;
      float v = st.own[warp][k * R + r][t];
      if (ar.fv.world > 1) v = ar_collect(ar, t, TL, col, D, v, &ok);
      v = bf16_round(v) + ld_act_bf16(p.x + (long)t * D + col);
      p.x[(long)t * D + col] = __float2bfloat16_rn(v);
    }
  }
}

// f32 router projection: one warp per expert row
template <int T>
__device__ __forceinline__ void phase_router(const Params& p, const Layer& L, const bf16* xs, int gw, int GW) {
  const int lane = threadIdx.x & 31;
  const int quads = p.D >> 2;
  for (int e = gw; e < p.E; e += GW) {
    const float4* wr = reinterpret_cast<const float4*>(L.router + (long)e * p.D);
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = 0.f;
    for (int c0 = lane; c0 < quads; c0 += 32 * 8) {
      float4 wv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j * 32;
        wv[j] = c < quads ? __ldg(wr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = c0 + j * 32;
        if (c >= quads) continue;
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(xs + t * p.D + c * 4);
          const float2 a = __bfloat1622float2(xp[0]), b = __bfloat1622float2(xp[1]);
          acc[t] += wv[j].x * a.x + wv[j].y * a.y + wv[j].z * b.x + wv[j].w * b.y;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
      const float v = warp_sum(acc[t]);
      if (lane == 0 && t < p.T_live) p.router_logits[(long)t * p.E + e] = v;
    }
  }
}

// top-k of token `t` by one warp (softmax top-k or sigmoid + bias); highest score first, ties to the lowest expert
template <int T>
__device__ __forceinline__ void route_select(const Params& p, const Layer& L, CtaState<T>& st, int t) {
  const int lane = threadIdx.x & 31;
  constexpr int PER = 8;   // E <= 256
  float score[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ei = lane + 32 * i;
    score[i] = (ei < p.E) ? __ldcg(p.router_logits + (long)t * p.E + ei) : -INFINITY;
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
        sel[i] = score[i] + (L.router_bias ? L.router_bias[ei] : 0.f);
      }
    } else {
      score[i] = 0.f;
      sel[i] = -INFINITY;
    }
  }
  denom = warp_sum(denom);
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
    const float w = (p.scoring == 0) ? raw / denom : raw;
    wsum += w;
    if (lane == 0) {
      st.rids[t][k] = bi;
      st.rw[t][k] = w;
    }
  }
  __syncwarp();
  if (lane < p.topk) {
    float w = st.rw[t][lane];
    if (p.scoring == 0) { if (p.renorm) w = w / wsum; }
    else w = w / (wsum + 1e-20f);
    st.rw[t][lane] = w * p.route_scale;
  }
}

// routes of every token (every CTA computes them), then SwiGLU(gate, up) of the local routes and of the shared shard
template <int T>
__device__ __forceinline__ void phase_gate_up(const Params& p, const Layer& L, const bf16* xs, CtaState<T>& st, int gw, int GW) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TL = p.T_live, D = p.D, F = p.F;
  if (warp < TL) route_select<T>(p, L, st, warp);
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int t = 0; t < TL; ++t)
      for (int k = 0; k < p.topk; ++k) {
        const int e = st.rids[t][k];
        if (e < p.e0 || e >= p.e0 + p.el) continue;
        st.route_t[n] = t;
        st.route_slot[n] = k;
        st.route_e[n] = e - p.e0;
        ++n;
      }
    st.n_routes = n;
  }
  if (blockIdx.x == 0 && (int)threadIdx.x < TL * p.topk) {
    const int t = threadIdx.x / p.topk, k = threadIdx.x % p.topk;
    p.route_ids[t * p.topk + k] = st.rids[t][k];
    p.route_w[t * p.topk + k] = st.rw[t][k];
  }
  __syncthreads();
  const int per_route = F / 2;
  const int UR = st.n_routes * per_route;
  const int Fs = L.shared_gate_up ? p.Fs : 0;
  const int US = Fs / 2;
  for (int u = gw; u < UR + US; u += GW) {
    const bf16* rows[4];
    if (u < UR) {
      const int i = u / per_route, j0 = (u % per_route) * 2;
      const int t = st.route_t[i];
      const bf16* W = L.gate_up + (size_t)st.route_e[i] * 2 * F * D;
      rows[0] = W + (size_t)j0 * D;
      rows[1] = W + (size_t)(j0 + 1) * D;
      rows[2] = W + (size_t)(F + j0) * D;
      rows[3] = W + (size_t)(F + j0 + 1) * D;
      float acc[4][1] = {{0.f}, {0.f}, {0.f}, {0.f}};
      warp_rows_dot<1, 4>(rows, xs + t * D, D, acc);
      warp_reduce_acc<1, 4>(acc);
      if (lane == 0) {
        bf16* out = p.act + ((size_t)t * (p.topk + 1) + st.route_slot[i]) * F;
        out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0][0])) * bf16_round(acc[2][0]));
        out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1][0])) * bf16_round(acc[3][0]));
      }
    } else {
      const int j0 = (u - UR) * 2;
      const bf16* W = L.shared_gate_up;
      rows[0] = W + (size_t)j0 * D;
      rows[1] = W + (size_t)(j0 + 1) * D;
      rows[2] = W + (size_t)(Fs + j0) * D;
      rows[3] = W + (size_t)(Fs + j0 + 1) * D;
      float acc[4][T];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
      warp_rows_dot<T, 4>(rows, xs, D, acc);
      warp_reduce_acc<T, 4>(acc);
      if (lane == 0) {
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (t >= TL) continue;
          bf16* out = p.act + ((size_t)t * (p.topk + 1) + p.topk) * F;
          out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0][t])) * bf16_round(acc[2][t]));
          out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1][t])) * bf16_round(acc[3][t]));
        }
      }
    }
  }
}

// y[t][n] = sum over the local routes s of token t of score_s * dot(W_s[n, :], act[t][s][:]) (+ shared shard),
// all-reduce, + x. `as` = shared staging of one token's activation rows, (topk+1) * F bf16.
template <int T>
__device__ __forceinline__ void phase_down(const Params& p, const Layer& L, const ArCtx& ar, bf16* as, CtaState<T>& st, int gw, int GW) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int TL = p.T_live, D = p.D, F = p.F;
  for (int t = 0; t < TL; ++t) {
    __syncthreads();
    if (threadIdx.x == 0) {
      int n = 0, c = 0;
      for (int slot = 0; slot <= p.topk; ++slot) {
        if (slot < p.topk) {
          const int e = st.rids[t][slot];
          if (e < p.e0 || e >= p.e0 + p.el) continue;
          st.dw[n] = L.down + (size_t)(e - p.e0) * D * F;
          st.dg[n] = st.rw[t][slot];
          st.dk[n] = F;
        } else {
          if (L.shared_down == nullptr) continue;
          st.dw[n] = L.shared_down;
          st.dg[n] = 1.f;
          st.dk[n] = p.Fs;
        }
        st.dslot[n] = slot;
        st.dcbeg[n] = c;
        c += st.dk[n] >> 3;
        ++n;
      }
      st.dcbeg[n] = c;
      st.dn = n;
    }
    __syncthreads();
    const int n_routes = st.dn;
    for (int i = 0; i < n_routes; ++i) {
      const bf16* arow = p.act + ((size_t)t * (p.topk + 1) + st.dslot[i]) * F;
      for (int c = threadIdx.x; c < (st.dk[i] >> 3); c += THREADS)
        *reinterpret_cast<uint4*>(as + (size_t)i * F + c * 8) = ld_act16(arow + c * 8);
    }
    __syncthreads();
    // The K ranges of all local routes form one flattened chunk space (16-byte chunks; routed experts own F/8 of
    // them each, a trailing shared-expert shard Fs/8), so a lane keeps U loads in flight across route boundaries.
    // The (route, chunk) pair of a load advances incrementally in registers - no division - and is remembered as
    // one packed word: route << 20 | chunk index in `as`.
    const int chunks = st.dcbeg[n_routes];
    const int as_cpr = F >> 3;
    const int last = n_routes - 1;
    const int last_cpr = n_routes > 0 ? (st.dk[last] >> 3) : 0;
    constexpr int U = 8;
    int k = 0;
    for (int n0 = gw; n0 < D && k < AR_ROWS; n0 += GW, ++k) {
      float total = 0.f;
      int route = 0, cc = lane;
      int cur = (route == last) ? last_cpr : as_cpr;
      while (route < n_routes && cc >= cur) { cc -= cur; ++route; cur = (route == last) ? last_cpr : as_cpr; }
      for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
        uint4 wv[U];
        int where[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (route < n_routes) {
            where[u] = (route << 20) | (route * as_cpr + cc);
            wv[u] = ld_stream16(st.dw[route] + ((size_t)n0 * cur + cc) * 8);
            cc += 32;
            while (route < n_routes && cc >= cur) { cc -= cur; ++route; cur = (route == last) ? last_cpr : as_cpr; }
          } else {
            where[u] = -1;
            wv[u] = make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (where[u] >= 0) {
            float xf[8], wf[8], d = 0.f;
            unpack8(*reinterpret_cast<const uint4*>(as + (size_t)(where[u] & 0xfffff) * 8), xf);
            unpack8(wv[u], wf);
#pragma unroll
            for (int q = 0; q < 8; ++q) d = fmaf(wf[q], xf[q], d);
            total = fmaf(st.dg[where[u] >> 20], d, total);
          }
        }
      }
      total = warp_sum(total);
      if (lane == 0) st.own[warp][k][t] = total;
    }
  }
  __syncwarp();
  int nown = 0;
  for (int n0 = gw; n0 < D && nown < AR_ROWS; n0 += GW, ++nown) {
    if (ar.fv.world > 1 && lane < TL) ar_push(ar, lane, TL, n0, D, st.own[warp][nown][lane]);
  }
  bool ok = true;
  for (int k = 0, n0 = gw; k < nown; ++k, n0 += GW) {
    if (lane < TL) {
      const int t = lane;
      float v = st.own[warp][k][t];
      if (ar.fv.world > 1) v = ar_collect(ar, t, TL, n0, D, v, &ok);
      v = bf16_round(v) + ld_act_bf16(p.x + (long)t * D + n0);
      p.x[(long)t * D + n0] = __float2bfloat16_rn(v);
    }
  }
}

// vocabulary shard of the head: logits (optional) and the per-CTA best (value, index) of every token
template <int T>
__device__ __forceinline__ void phase_head(const Params& p, const bf16* xs, CtaState<T>& st, int gw, int GW) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float bv[T];
  int bi[T];
#pragma unroll
  for (int t = 0; t < T; ++t) {
    bv[t] = -INFINITY;
    bi[t] = 0x7fffffff;
  }
  gemv_phase<T, 2>(p.lm_head, p.vl, p.D, xs, gw, GW, [&](int r0, float (&acc)[2][T]) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r0 + r >= p.vl) continue;
#pragma unroll
      for (int t = 0; t < T; ++t) {
        if (p.logits && lane == 0 && t < p.T_live) p.logits[(size_t)t * p.vl + r0 + r] = acc[r][t];
        if (acc[r][t] > bv[t]) { bv[t] = acc[r][t]; bi[t] = p.vocab_offset + r0 + r; }
      }
    }
  });
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < T; ++t) {
      st.bestv[warp][t] = bv[t];
      st.besti[warp][t] = bi[t];
    }
  }
  __syncthreads();
  if (threadIdx.x < T) {
    const int t = threadIdx.x;
    float v = -INFINITY;
    int i = 0x7fffffff;
    for (int w = 0; w < WARPS; ++w)
      if (st.bestv[w][t] > v || (st.bestv[w][t] == v && st.besti[w][t] < i)) { v = st.bestv[w][t]; i = st.besti[w][t]; }
    p.partial[(size_t)blockIdx.x * T + t] = make_float2(v, __int_as_float(i));
  }
}

// CTA 0: reduce the per-CTA candidates, exchange (value, index) with the peers, publish the token (+ feedback)
template <int T>
__device__ __forceinline__ void phase_sample(const Params& p, uint64_t epoch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t par = (uint32_t)(epoch & 1);
  const int world = p.fv.world, rank = p.fv.rank, TL = p.T_live;
  __shared__ float s_v[T];
  __shared__ int s_i[T];
  if (warp < TL) {
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
      if (lane < world) {
        float2* dst = reinterpret_cast<float2*>(p.fv.data[lane] + (size_t)par * p.fv.data_half_bytes) + rank * T + t;
        *dst = make_float2(bv, __int_as_float(bi));
      }
    } else if (lane == 0) {
      s_v[t] = bv;
      s_i[t] = bi;
    }
  }
  if (world > 1) {
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < world) {
      const int q = threadIdx.x;
      st_release_sys(p.fv.flags[q] + (size_t)par * p.fv.flag_half_words + rank, epoch);
      if (!wait_flag_bounded(p.fv.flags[rank] + (size_t)par * p.fv.flag_half_words + q, epoch, p.fv.spin_limit))
        atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
    __syncthreads();
    if ((int)threadIdx.x < TL) {
      const int t = threadIdx.x;
      const float2* src = reinterpret_cast<const float2*>(p.fv.data[rank] + (size_t)par * p.fv.data_half_bytes);
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int q = 0; q < world; ++q) {
        const float2 v = __ldcg(src + q * T + t);
        const int vi = __float_as_int(v.y);
        if (v.x > bv || (v.x == bv && vi < bi)) { bv = v.x; bi = vi; }
      }
      s_v[t] = bv;
      s_i[t] = bi;
    }
  }
  __syncthreads();
  if ((int)threadIdx.x < TL) {
    const int t = threadIdx.x;
    p.next_ids[t] = s_i[t];
    if (p.next_vals) p.next_vals[t] = s_v[t];
    if (p.feedback) {
      p.tokens[t] = s_i[t];
      p.positions[t] = p.positions[t] + 1;
    }
  }
}

template <int T, int HG>
__device__ __forceinline__ void run_step(const Params& p, unsigned char* smem, CtaState<T>& st, GridBar& gb, uint64_t seq0) {
  const int warp = threadIdx.x >> 5;
  const int gw = blockIdx.x * WARPS + warp, GW = gridDim.x * WARPS;
  const int TL = p.T_live, D = p.D;
  bf16* xs = reinterpret_cast<bf16*>(smem);
  const int NQ = p.q_lora + ROW;
  const int qk = p.nope + p.rope;
  ArCtx ar{p.fv, 0, p.fv.status, p.bar + 3};

  phase_embedding(p);
  if (!grid_sync(gb)) return;
  for (int l = 0; l < p.n_layers; ++l) {
    const Layer L = p.layers[l];
    // 1: qkv_a
    stage_act<T>(xs, p.x, D, TL, D, L.attn_norm, p.eps, st.red);
    gemv_phase<T, 1>(L.qkv_a, NQ, D, xs, gw, GW, [&](int r0, float (&acc)[1][T]) {
      if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int t = 0; t < T; ++t)
          if (t < TL) p.qkv[(long)t * NQ + r0] = __float2bfloat16_rn(acc[0][t]);
      }
    });
    if (!grid_sync(gb)) return;
    // 2: kv_write (CTAs 0..T-1) and q_b
    if ((int)blockIdx.x < TL) kv_write_cta(p, L, blockIdx.x, st.red);
    stage_act<T>(xs, p.qkv, NQ, TL, p.q_lora, L.q_a_norm, p.eps, st.red);
    {
      const int rows = p.hl * qk;
      gemv_phase<T, 2>(L.q_b, rows, p.q_lora, xs, gw, GW, [&](int r0, float (&acc)[2][T]) {
        if ((threadIdx.x & 31) == 0) {
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t)
              if (t < TL && r0 + r < rows) p.q[(long)t * rows + r0 + r] = __float2bfloat16_rn(acc[r][t]);
        }
      });
    }
    if (!grid_sync(gb)) return;
    // 3: absorb
    phase_absorb(p, L, reinterpret_cast<float*>(smem));
    if (!grid_sync(gb)) return;
    // 4: split attention
    phase_split<HG>(p, L, reinterpret_cast<float*>(smem));
    if (!grid_sync(gb)) return;
    // 5: merge + value up-projection
    phase_merge_vup(p, L, smem);
    if (!grid_sync(gb)) return;
    // 6: o_proj + all-reduce + residual
    {
      const int Ko = p.hl * p.vdim;
      stage_act<T>(xs, p.attn, Ko, TL, Ko, nullptr, p.eps, st.red);
      ar.epoch = seq0 + 1 + 2 * (uint64_t)l;
      if (Ko > 2048) ar_gemv_phase<T, 1>(p, ar, L.o_proj, Ko, xs, st, gw, GW);
      else if (Ko > 1024) ar_gemv_phase<T, 2>(p, ar, L.o_proj, Ko, xs, st, gw, GW);
      else ar_gemv_phase<T, 4>(p, ar, L.o_proj, Ko, xs, st, gw, GW);
    }
    if (!grid_sync(gb)) return;
    // 7: router logits (the normalised x stays staged for phase 8)
    stage_act<T>(xs, p.x, D, TL, D, L.ffn_norm, p.eps, st.red);
    phase_router<T>(p, L, xs, gw, GW);
    if (!grid_sync(gb)) return;
    // 8: routes + gate/up
    phase_gate_up<T>(p, L, xs, st, gw, GW);
    if (!grid_sync(gb)) return;
    // 9: down + all-reduce + residual
    ar.epoch = seq0 + 2 + 2 * (uint64_t)l;
    phase_down<T>(p, L, ar, xs, st, gw, GW);
    if (!grid_sync(gb)) return;
  }
  stage_act<T>(xs, p.x, D, TL, D, p.final_norm, p.eps, st.red);
  phase_head<T>(p, xs, st, gw, GW);
  if (!grid_sync(gb)) return;
  if (blockIdx.x == 0) phase_sample<T>(p, seq0 + 2 * (uint64_t)p.n_layers + 1);
}

template <int T, int HG>
__global__ void __launch_bounds__(THREADS, 2) decode_step_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ CtaState<T> st;
  if (threadIdx.x == 0) st.ok = 1;
  GridBar gb{p.trace, p.bar, ld_volatile_u32(p.bar + 1), 0u, gridDim.x, p.spin_limit, p.fv.status, &st.ok};
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[0] = global_timer_ns();
  const uint64_t seq0 = *reinterpret_cast<volatile uint64_t*>(p.seq);
  __syncthreads();
  run_step<T, HG>(p, smem, st, gb, seq0);
  // leave: the last CTA to get here re-bases the barrier for the next launch and advances the call counter
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(p.bar + 2, 1u);
    if (ticket == gridDim.x - 1) {
      const bool healthy = ld_volatile_u32(p.bar + 3) == 0;
      p.bar[1] = ld_acquire_gpu(p.bar);
      p.bar[2] = 0;
      p.bar[3] = 0;
      if (healthy) *p.seq = seq0 + 2 * (uint64_t)p.n_layers + 1;
      __threadfence();
    }
  }
}

// dynamic shared memory one CTA needs
template <int T, int HG>
inline size_t step_smem(const Params& p) {
  size_t s = (size_t)T * p.D * sizeof(bf16);                                  // staged x
  s = std::max(s, (size_t)T * std::max(p.q_lora, p.hl * p.vdim) * sizeof(bf16));
  s = std::max(s, (size_t)(256 + 16 * 129) * sizeof(float));                  // absorb
  s = std::max(s, (size_t)(8 * HG * LATENT + 16 * HG) * sizeof(float));       // split attention
  s = std::max(s, (size_t)(p.topk + 1) * p.F * sizeof(bf16));                 // down: one token's activation rows
  return s;
}

// Returns 0, a negative IFAB error or a CUDA error. The grid is 2 CTAs per SM (or what fits), launched cooperatively.
template <int T, int HG>
int launch_step(Params& p, cudaStream_t stream) {
  auto k = decode_step_kernel<T, HG>;
  const size_t smem = step_smem<T, HG>(p);
  static int cached_dev = -1, cached_blocks = 0;
  static size_t cached_smem = 0;
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev)) return (int)e;
  if (dev != cached_dev || smem != cached_smem) {
    if (int rc = opt_in_smem(k, smem)) return rc;
    int per_sm = 0, sms = 0;
    if (cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, THREADS, smem)) return (int)e;
    if (cudaError_t e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) return (int)e;
    if (per_sm < 1) return -2;
    cached_blocks = sms * std::min(per_sm, 2);
    cached_dev = dev;
    cached_smem = smem;
  }
  const int grid = cached_blocks;
  const int GW = grid * WARPS;
  // every warp may own at most AR_ROWS output rows in an all-reduce phase
  const int Ko = p.hl * p.vdim, R = Ko > 2048 ? 1 : (Ko > 1024 ? 2 : 4);
  if ((((p.D + R - 1) / R + GW - 1) / GW) * R > AR_ROWS) return -2;
  if ((p.D + GW - 1) / GW > AR_ROWS) return -2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, k, p);
}

}  // namespace ifab::mega
