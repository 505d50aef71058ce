// Operators of the hyper-connection / hybrid model families that are not plain linears or attention:
//
//   mome_kernel          causal depthwise convolution over the token stream with residual (taps <= 4), state = the last
//                        taps-1 inputs of every sequence slot:  y = x + [pos + 1 >= taps] * sum_k w_k * x_{t-(taps-1)+k}
//   mhc_pre_kernel       manifold-constrained hyper-connection, pre step: RMS statistic of the S residual streams, the
//                        S*S + 2S mixing logits (phi . (gamma * X)), sigmoid gates, Sinkhorn-normalised S x S mixing
//                        matrix, and the branch input  y = sum_s pre_s * X_s
//   mhc_post_kernel      Y_i = post_i * branch + sum_k comb[k][i] * X_k
//   delta_rule_kernel    gated delta-rule recurrence of one decode token per (slot, head):
//                        S *= exp(g); r = v - k S; S += k^T (beta r); o = (q / sqrt(dk)) S      (state f32 [dk, dv])
//   index_score_kernel / index_select_kernel
//                        sparse-attention indexer: score(t, s) = sum_h w[t,h] * relu(q[t,h,:] . key[s,:]) over the paged
//                        index-key cache, then the top-k key positions of every query (exact threshold search)
// Numerics follow the CPU interpreter (csrc/core/interp.cpp) operation by operation; all mixing arithmetic is f32.
// Reference counterparts: aclnnAiInfraFusedCausalConv1d, ...ManifoldConstrainedHyperConnectionPre / SinkhornEnhance /
// HyperConnectionPost (native/src/token_executor.h:480-585), delta_prepare (native/src/inferfabric_acl.cpp:889-960),
// aclnnLightningIndexerEnhance (native/src/resident_index.h).
#include <algorithm>

#include <cuda_fp16.h>

#include "common.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

// ---- MoME ---------------------------------------------------------------------------------------------------------
// grid = ceil(C / 256); every thread owns one channel and walks the rows in order, so rows of one sequence inside a
// chunk see each other's inputs. state: bf16 [slots, taps-1, C], oldest first.
__global__ void __launch_bounds__(256) mome_kernel(const bf16* x, long ldx, const float* w /*[C, taps]*/, bf16* state, const int32_t* positions,
                                                   const int32_t* slots, bf16* y, long ldy, int T, int C, int taps, int c_offset) {
  grid_dep_launch();
  grid_dep_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float wk[4];
  for (int k = 0; k < taps; ++k) wk[k] = w[(long)(c_offset + c) * taps + k];
  for (int t = 0; t < T; ++t) {
    const int pos = positions[t];
    if (pos < 0) continue;
    bf16* h = state + (long)slots[t] * (taps - 1) * C + c;
    const float xv = __bfloat162float(x[(long)t * ldx + c]);
    float conv = xv * wk[taps - 1];
    for (int k = 0; k + 1 < taps; ++k) conv += __bfloat162float(h[(long)k * C]) * wk[k];
    y[(long)t * ldy + c] = __float2bfloat16_rn(xv + (pos + 1 >= taps ? conv : 0.f));
    for (int k = 0; k + 2 < taps; ++k) h[(long)k * C] = h[(long)(k + 1) * C];
    h[(long)(taps - 2) * C] = __float2bfloat16_rn(xv);
  }
}

// ---- mHC ----------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
  return s;
}

// The pre step runs as two launches. The mixing logits are S*S + 2S dot products over all S*W elements of the token's streams
// (1 MB of phi per token at S = 4, W = 2560): one CTA per (logit, token) streams its row of phi, so the read is spread over
// S*S + 2S + 1 SMs instead of one. The tail - gates, Sinkhorn, branch input - is one CTA per token.
//
// mhc_logits_kernel: grid (M + 1, T), M = S*S + 2S. CTA j < M: raw[t][j] = sum_c phi[j][c] * gamma[c] * X[t][c]; CTA M: the sum of
// squares. The M + 1 floats land in the first bytes of the token's row of y (the tail kernel reads them before it writes y).
__device__ __forceinline__ void mhc_mix_token(const bf16* X, const float* raw, long raw_stride, const float* alpha, const float* beta, bf16* y, float* post,
                                              float* comb, int S, int W, int iters, float eps, int t);
// With `tickets` (one zeroed word per token, left zero again): the CTA that finishes a token's sums last also runs the token's
// tail (mhc_mix_token) - the whole pre step in one launch.
template <bool FUSED>
__global__ void __launch_bounds__(256) mhc_logits_kernel(const bf16* X, const float* phi, const float* gamma, float* raw, long raw_stride, int S, int W,
                                                         uint32_t* tickets, const float* alpha, const float* beta, float* post, float* comb, int iters,
                                                         float eps) {
  __shared__ float red[8];
  __shared__ bool is_last;
  grid_dep_launch();
  grid_dep_wait();
  const int j = blockIdx.x, t = blockIdx.y, M = S * S + 2 * S;
  const long total = (long)S * W;
  const bf16* Xt = X + (long)t * total;
  float s = 0.f;
  if (j == M) {
    for (long c = threadIdx.x; c < total; c += blockDim.x) {
      const float v = __bfloat162float(Xt[c]);
      s += v * v;
    }
  } else {
    const float* pj = phi + (long)j * total;
    if ((total & 3) == 0) {
      const float4* p4 = reinterpret_cast<const float4*>(pj);
      const float4* g4 = reinterpret_cast<const float4*>(gamma);
      const uint2* x4 = reinterpret_cast<const uint2*>(Xt);
      auto dot4 = [](const float4& a, const float4& g, const uint2& xr) {
        const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.x));
        const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.y));
        return a.x * g.x * x01.x + a.y * g.y * x01.y + a.z * g.z * x23.x + a.w * g.w * x23.y;
      };
      // four independent chunks per trip: twelve 8 / 16-byte loads in flight per thread
      const long n4 = total / 4, step = blockDim.x;
      long c = threadIdx.x;
      for (; c + 3 * step < n4; c += 4 * step) {
        const float4 a0 = p4[c], a1 = p4[c + step], a2 = p4[c + 2 * step], a3 = p4[c + 3 * step];
        const float4 g0 = g4[c], g1 = g4[c + step], g2 = g4[c + 2 * step], g3 = g4[c + 3 * step];
        const uint2 x0 = x4[c], x1 = x4[c + step], x2 = x4[c + 2 * step], x3 = x4[c + 3 * step];
        s += dot4(a0, g0, x0) + dot4(a1, g1, x1) + dot4(a2, g2, x2) + dot4(a3, g3, x3);
      }
      for (; c < n4; c += step) s += dot4(p4[c], g4[c], x4[c]);
    } else {
      for (long c = threadIdx.x; c < total; c += blockDim.x) s += pj[c] * gamma[c] * __bfloat162float(Xt[c]);
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) raw[(long)t * raw_stride + j] = s;
  if (!FUSED) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t tk = atomicAdd(tickets + t, 1u);
    is_last = (tk == gridDim.x - 1);
    if (is_last) tickets[t] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  mhc_mix_token(X, raw, raw_stride, alpha, beta, reinterpret_cast<bf16*>(raw), post, comb, S, W, iters, eps, t);
}

// mhc_mix_kernel: one CTA per token. Reads the M + 1 raw sums, then: sigmoid gates (pre, post), the S x S logits through a row
// softmax and `iters` rounds of Sinkhorn normalisation (one thread per matrix entry, two buffers, one barrier per pass), and the
// branch input y = sum_s pre_s * X_s. S <= 8.
__device__ __forceinline__ void mhc_mix_token(const bf16* X, const float* raw, long raw_stride, const float* alpha, const float* beta, bf16* y, float* post,
                                              float* comb, int S, int W, int iters, float eps, int t) {
  __shared__ float m[8 * 8 + 16 + 1];
  __shared__ float R[2][64];
  __shared__ float pre_s[8];
  const int M = S * S + 2 * S, n = S * S, tid = threadIdx.x;
  const long total = (long)S * W;
  const bf16* Xt = X + (long)t * total;
  if (tid <= M) m[tid] = raw[(long)t * raw_stride + tid];
  __syncthreads();                                   // every raw sum is in shared memory before y (which held them) is written
  const float inv = 1.f / sqrtf(m[M] / (float)total + eps);
  if (tid < S) pre_s[tid] = 1.f / (1.f + expf(-(inv * m[tid] * alpha[0] + beta[tid]))) + 1e-6f;
  else if (tid < 2 * S) post[(long)t * S + (tid - S)] = 2.f / (1.f + expf(-(inv * m[tid] * alpha[1] + beta[tid])));
  const int a = tid / S, b = tid % S;
  if (tid < n) R[0][tid] = inv * m[2 * S + tid] * alpha[2] + beta[2 * S + tid];
  __syncthreads();
  int cur = 0;
  if (tid < n) {                                     // row softmax
    float mx = -INFINITY, sum = 0.f;
    for (int k = 0; k < S; ++k) mx = fmaxf(mx, R[0][a * S + k]);
    for (int k = 0; k < S; ++k) sum += expf(R[0][a * S + k] - mx);
    R[1][tid] = expf(R[0][tid] - mx) / sum + 1e-6f;
  }
  cur = 1;
  __syncthreads();
  // column pass, then (iters - 1) x (row pass, column pass)
  for (int pass = 0; pass < 2 * iters - 1; ++pass) {
    const bool column = (pass & 1) == 0;
    if (tid < n) {
      float sum = 0.f;
      for (int k = 0; k < S; ++k) sum += column ? R[cur][k * S + b] : R[cur][a * S + k];
      R[cur ^ 1][tid] = R[cur][tid] / (sum + 1e-6f);
    }
    cur ^= 1;
    __syncthreads();
  }
  if (tid < n) comb[(long)t * n + tid] = R[cur][tid];
  for (int c = tid; c < W; c += blockDim.x) {
    float v = 0.f;
    for (int k = 0; k < S; ++k) v += pre_s[k] * __bfloat162float(Xt[(long)k * W + c]);
    y[(long)t * W + c] = __float2bfloat16_rn(v);
  }
}

__global__ void __launch_bounds__(256) mhc_mix_kernel(const bf16* X, const float* raw, long raw_stride, const float* alpha, const float* beta, bf16* y,
                                                      float* post, float* comb, int S, int W, int iters, float eps) {
  grid_dep_launch();
  grid_dep_wait();
  mhc_mix_token(X, raw, raw_stride, alpha, beta, y, post, comb, S, W, iters, eps, blockIdx.x);
}

// grid (ceil(W/256), T): Y[t, i, c] = post[t, i] * branch[t, c] + sum_k comb[t, k, i] * X[t, k, c]
__global__ void __launch_bounds__(256) mhc_post_kernel(const bf16* X, const bf16* branch, long ldb, const float* post, const float* comb, bf16* Y,
                                                       int S, int W) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const bf16* Xt = X + (long)t * S * W;
  const float br = __bfloat162float(branch[(long)t * ldb + c]);
  float xv[8];
  for (int k = 0; k < S; ++k) xv[k] = __bfloat162float(Xt[(long)k * W + c]);
  for (int i = 0; i < S; ++i) {
    float v = post[(long)t * S + i] * br;
    for (int k = 0; k < S; ++k) v += comb[(long)t * S * S + k * S + i] * xv[k];
    Y[((long)t * S + i) * W + c] = __float2bfloat16_rn(v);
  }
}

// The same with RMSNorm(branch) * gain folded in: every CTA first reduces the whole branch row (W values, a few KB) to its
// statistic, then mixes its 256 columns. The normalised value is rounded to bf16 as the stand-alone norm would store it.
__global__ void __launch_bounds__(256) mhc_post_norm_kernel(const bf16* X, const bf16* branch, long ldb, const bf16* gain, float eps, const float* post,
                                                            const float* comb, bf16* Y, int S, int W) {
  __shared__ float red[8];
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const bf16* br_row = branch + (long)t * ldb;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = __bfloat162float(br_row[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  if (c >= W) return;
  const float inv = rsqrtf(ss / (float)W + eps);
  const float br = __bfloat162float(__float2bfloat16_rn(__bfloat162float(br_row[c]) * inv * __bfloat162float(gain[c])));
  const bf16* Xt = X + (long)t * S * W;
  float xv[8];
  for (int k = 0; k < S; ++k) xv[k] = __bfloat162float(Xt[(long)k * W + c]);
  for (int i = 0; i < S; ++i) {
    float v = post[(long)t * S + i] * br;
    for (int k = 0; k < S; ++k) v += comb[(long)t * S * S + k * S + i] * xv[k];
    Y[((long)t * S + i) * W + c] = __float2bfloat16_rn(v);
  }
}

// ---- gated delta rule, one token ------------------------------------------------------------------------------------
// grid (H, rows); blockDim = dv (<= 256); thread j owns column j of the state of (slot, head).
// q, k [rows, H, dk] bf16; v [rows, H, dv] bf16; g, beta [rows, H] f32; state f32 [slots, H, dk, dv]; out [rows, H, dv] bf16.
__global__ void __launch_bounds__(256) delta_rule_kernel(const bf16* q, const bf16* k, const bf16* v, const float* g, const float* beta,
                                                         float* state, const int32_t* slots, bf16* out, int H, int dk, int dv) {
  extern __shared__ float sm[];   // q [dk], k [dk]
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, r = blockIdx.y, j = threadIdx.x;
  const long qk = ((long)r * H + h) * dk;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    sm[i] = __bfloat162float(q[qk + i]) * rsqrtf((float)dk);
    sm[dk + i] = __bfloat162float(k[qk + i]);
  }
  __syncthreads();
  if (j >= dv) return;
  float* S = state + (((long)slots[r] * H + h) * dk) * dv + j;
  const float decay = expf(g[(long)r * H + h]);
  float ks = 0.f;
  for (int i = 0; i < dk; ++i) {
    const float s = S[(long)i * dv] * decay;
    S[(long)i * dv] = s;
    ks = fmaf(sm[dk + i], s, ks);
  }
  const float rj = (__bfloat162float(v[((long)r * H + h) * dv + j]) - ks) * beta[(long)r * H + h];
  float o = 0.f;
  for (int i = 0; i < dk; ++i) {
    const float s = fmaf(sm[dk + i], rj, S[(long)i * dv]);
    S[(long)i * dv] = s;
    o = fmaf(sm[i], s, o);
  }
  out[((long)r * H + h) * dv + j] = __float2bfloat16_rn(o);
}

// ---- sparse-attention indexer -----------------------------------------------------------------------------------------
// grid (ceil(ctx/8), T): one warp per key position; keys: paged bf16 [pages, page_tokens, dim]; scores f32 [T, ctx]
// Q8: the keys are int8 rows with one half-precision scale per row (index_cache_append_q8_kernel), and every query head is
// quantised the same way before scoring - the arithmetic of the CPU oracle for an int8 index cache.
template <bool Q8>
__global__ void __launch_bounds__(256) index_score_kernel(const bf16* q /*[T, Hi, dim]*/, const void* w_raw /*[T, Hi] f32, or bf16 rows of stride ldw*/,
                                                          long ldw, int w_bf16, const void* keys_raw,
                                                          const __half* key_scales, const int32_t* positions, const int32_t* slots,
                                                          const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores,
                                                          int ctx, int Hi, int dim, uint32_t* status) {
  extern __shared__ float qs[];   // [Hi][dim] then w [Hi]
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < Hi * dim; i += blockDim.x) qs[i] = __bfloat162float(q[(long)t * Hi * dim + i]);
  for (int i = threadIdx.x; i < Hi; i += blockDim.x)
    qs[Hi * dim + i] = w_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(w_raw)[(long)t * ldw + i]) : reinterpret_cast<const float*>(w_raw)[(long)t * ldw + i];
  __syncthreads();
  if (Q8) {
    for (int h = warp; h < Hi; h += (int)(blockDim.x >> 5)) {          // one warp per head row
      float amax = 0.f;
      for (int i = lane; i < dim; i += 32) amax = fmaxf(amax, fabsf(qs[h * dim + i]));
      amax = warp_max(amax);
      const float sc = __half2float(__float2half_rn(amax / 127.f));
      if (sc > 0.f)
        for (int i = lane; i < dim; i += 32) qs[h * dim + i] = fmaxf(-127.f, fminf(127.f, rintf(qs[h * dim + i] / sc))) * sc;
    }
    __syncthreads();
  }
  const int s = blockIdx.x * 8 + warp;
  if (s >= ctx) return;
  const int pos = positions[t];
  float sc = -INFINITY;
  if (pos >= 0 && s <= pos) {
    const int lp = s / page_tokens;
    const int page = lp < max_pages ? page_table[(long)slots[t] * max_pages + lp] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    } else {
      const long krow = (long)page * page_tokens + s % page_tokens;
      float kf[8];
      const int per = dim / 32;   // dim = 128 -> 4 elements per lane
      if (Q8) {
        const signed char* kr = reinterpret_cast<const signed char*>(keys_raw) + krow * dim;
        const float ks = __half2float(key_scales[krow]);
        for (int i = 0; i < per; ++i) kf[i] = (float)kr[lane * per + i] * ks;
      } else {
        const bf16* kr = reinterpret_cast<const bf16*>(keys_raw) + krow * dim;
        for (int i = 0; i < per; ++i) kf[i] = __bfloat162float(kr[lane * per + i]);
      }
      sc = 0.f;
      for (int h = 0; h < Hi; ++h) {
        float d = 0.f;
        for (int i = 0; i < per; ++i) d = fmaf(qs[h * dim + lane * per + i], kf[i], d);
        d = warp_sum(d);
        sc += qs[Hi * dim + h] * fmaxf(d, 0.f);
      }
    }
  }
  if (lane == 0) scores[(long)t * ctx + s] = sc;
}

// order-preserving map of f32 to u32
__device__ __forceinline__ uint32_t f2key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// one CTA per query: the k-th largest score is found by a bitwise search on the ordered key (32 counting passes), then
// positions with a larger score are emitted in ascending order, ties at the threshold filling what is left (lowest first)
__global__ void __launch_bounds__(256) index_select_kernel(const float* scores, const int32_t* positions, int ctx, int topk, int32_t* out) {
  __shared__ int red[8];
  __shared__ int s_count;
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const float* sc = scores + (long)t * ctx;
  const int n = min(ctx, positions[t] + 1);
  int32_t* o = out + (long)t * topk;
  if (n <= topk) {
    for (int i = threadIdx.x; i < topk; i += blockDim.x) o[i] = i < n ? i : -1;
    return;
  }
  auto count_ge = [&](uint32_t thr) {
    int c = 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) c += f2key(sc[i]) >= thr ? 1 : 0;
    c = (int)warp_sum((float)c);   // counts stay far below 2^24
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    int tot = 0;
    for (int w = 0; w < 8; ++w) tot += red[w];
    return tot;
  };
  uint32_t thr = 0;   // largest key value with count(key >= thr) >= topk
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t cand = thr | (1u << bit);
    if (count_ge(cand) >= topk) thr = cand;
  }
  const int above = thr == 0xffffffffu ? 0 : count_ge(thr + 1);
  // ordered emission by one warp (n is at most a few 10^4)
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int emitted = 0, ties_left = topk - above;
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      const uint32_t key = i < n ? f2key(sc[i]) : 0u;
      const bool gt = i < n && key > thr, eq = i < n && key == thr;
      const unsigned meq = __ballot_sync(0xffffffffu, eq);
      const int eq_rank = __popc(meq & ((1u << lane) - 1));
      const bool take = gt || (eq && eq_rank < ties_left);
      const unsigned mt = __ballot_sync(0xffffffffu, take);
      if (take) o[emitted + __popc(mt & ((1u << lane) - 1))] = i;
      emitted += __popc(mt);
      ties_left -= min(ties_left, __popc(meq));
    }
    for (int i = emitted + lane; i < topk; i += 32) o[i] = -1;
  }
}

}  // namespace

extern "C" int ifab_mome(const void* x, long ldx, const float* w, void* state, const int32_t* positions, const int32_t* slots, void* y,
                         long ldy, int T, int C, int taps, int c_offset, void* stream) {
  if (T < 1 || C < 1 || taps < 2 || taps > 4) return -1;
  return launch_chain(mome_kernel, dim3((C + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx, w, (bf16*)state, positions,
                      slots, (bf16*)y, ldy, T, C, taps, c_offset);
}

static int mhc_pre_launch(const void* X, const float* phi, const float* gamma, const float* alpha, const float* beta, void* y, float* post, float* comb,
                          int T, int S, int W, int sinkhorn_iters, float eps, uint32_t* tickets, void* stream) {
  const int M = S * S + 2 * S;
  // the raw sums of a token travel in the first (M + 1) floats of its row of y
  if (T < 1 || S < 1 || S > 8 || W < 1 || sinkhorn_iters < 1 || (W & 1) || (long)W * 2 < (long)(M + 1) * 4) return -1;
  if (tickets)
    return launch_chain(mhc_logits_kernel<true>, dim3(M + 1, T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)X, phi, gamma, (float*)y, (long)(W / 2), S,
                        W, tickets, alpha, beta, post, comb, sinkhorn_iters, eps);
  if (int rc = launch_chain(mhc_logits_kernel<false>, dim3(M + 1, T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)X, phi, gamma, (float*)y,
                            (long)(W / 2), S, W, (uint32_t*)nullptr, alpha, beta, post, comb, sinkhorn_iters, eps))
    return rc;
  return launch_chain(mhc_mix_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)X, (const float*)y, (long)(W / 2), alpha, beta, (bf16*)y,
                      post, comb, S, W, sinkhorn_iters, eps);
}

extern "C" int ifab_mhc_pre(const void* X, const float* phi, const float* gamma, const float* alpha, const float* beta, void* y, float* post,
                            float* comb, int T, int S, int W, int sinkhorn_iters, float eps, void* stream) {
  return mhc_pre_launch(X, phi, gamma, alpha, beta, y, post, comb, T, S, W, sinkhorn_iters, eps, nullptr, stream);
}

extern "C" int ifab_mhc_pre_ticketed(const void* X, const float* phi, const float* gamma, const float* alpha, const float* beta, void* y, float* post,
                                     float* comb, int T, int S, int W, int sinkhorn_iters, float eps, uint32_t* tickets, void* stream) {
  if (!tickets) return -1;
  return mhc_pre_launch(X, phi, gamma, alpha, beta, y, post, comb, T, S, W, sinkhorn_iters, eps, tickets, stream);
}

extern "C" int ifab_mhc_post(const void* X, const void* branch, long ldb, const float* post, const float* comb, void* Y, int T, int S, int W,
                             void* stream) {
  if (T < 1 || S < 1 || S > 8 || W < 1) return -1;
  return launch_chain(mhc_post_kernel, dim3((W + 255) / 256, T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)X, (const bf16*)branch, ldb,
                      post, comb, (bf16*)Y, S, W);
}

extern "C" int ifab_mhc_post_norm(const void* X, const void* branch, long ldb, const void* norm_w, float eps, const float* post, const float* comb, void* Y,
                                  int T, int S, int W, void* stream) {
  if (T < 1 || S < 1 || S > 8 || W < 1) return -1;
  return launch_chain(mhc_post_norm_kernel, dim3((W + 255) / 256, T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)X, (const bf16*)branch, ldb,
                      (const bf16*)norm_w, eps, post, comb, (bf16*)Y, S, W);
}

extern "C" int ifab_delta_rule_decode(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                                      const int32_t* slots, void* out, int rows, int H, int dk, int dv, void* stream) {
  if (rows < 1 || H < 1 || dk < 1 || dk > 512 || dv < 1 || dv > 256) return -1;
  const int threads = (std::max(dv, 32) + 31) / 32 * 32;
  return launch_chain(delta_rule_kernel, dim3(H, rows), dim3(threads), (size_t)2 * dk * sizeof(float), (cudaStream_t)stream, (const bf16*)q,
                      (const bf16*)k, (const bf16*)v, g, beta, state, slots, (bf16*)out, H, dk, dv);
}

// scores: scratch f32 [T, ctx]; out: int32 [T, topk], ascending key positions, -1 padded
// Gains `w` are f32 [T, heads] (w_bf16 = 0) or bf16 rows of stride ldw (w_bf16 = 1, e.g. a projection's result where it lies);
// key_scales = null: bf16 keys; else int8 keys with one half-precision scale per row.
extern "C" int ifab_sparse_index_general(const void* q, const void* w, long ldw, int w_bf16, const void* keys, const void* key_scales,
                                         const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens,
                                         int num_pages, float* scores, int ctx, int T, int heads, int dim, int topk, int32_t* out, uint32_t* status,
                                         void* stream) {
  if (T < 1 || ctx < 1 || heads < 1 || dim % 32 || dim > 256 || topk < 1 || ldw < heads) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)(heads * dim + heads) * sizeof(float);
  int rc;
  if (key_scales) {
    if ((rc = opt_in_smem(index_score_kernel<true>, smem))) return rc;
    rc = launch_chain(index_score_kernel<true>, dim3((ctx + 7) / 8, T), dim3(256), smem, s, (const bf16*)q, w, ldw, w_bf16, keys, (const __half*)key_scales,
                      positions, slots, page_table, max_pages, page_tokens, num_pages, scores, ctx, heads, dim, status);
  } else {
    if ((rc = opt_in_smem(index_score_kernel<false>, smem))) return rc;
    rc = launch_chain(index_score_kernel<false>, dim3((ctx + 7) / 8, T), dim3(256), smem, s, (const bf16*)q, w, ldw, w_bf16, keys, (const __half*)nullptr,
                      positions, slots, page_table, max_pages, page_tokens, num_pages, scores, ctx, heads, dim, status);
  }
  if (rc) return rc;
  return launch_chain(index_select_kernel, dim3(T), dim3(256), 0, s, (const float*)scores, positions, ctx, topk, out);
}

extern "C" int ifab_sparse_index(const void* q, const float* w, const void* keys, const int32_t* positions, const int32_t* slots,
                                 const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores, int ctx, int T,
                                 int heads, int dim, int topk, int32_t* out, uint32_t* status, void* stream) {
  return ifab_sparse_index_general(q, w, heads, 0, keys, nullptr, positions, slots, page_table, max_pages, page_tokens, num_pages, scores, ctx, T, heads, dim,
                                   topk, out, status, stream);
}

// The same over an int8 index cache: keys int8 [pages, page_tokens, dim], key_scales half [pages, page_tokens].
extern "C" int ifab_sparse_index_q8(const void* q, const float* w, const void* keys, const void* key_scales, const int32_t* positions,
                                    const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens, int num_pages, float* scores,
                                    int ctx, int T, int heads, int dim, int topk, int32_t* out, uint32_t* status, void* stream) {
  if (!key_scales) return -1;
  return ifab_sparse_index_general(q, w, heads, 0, keys, key_scales, positions, slots, page_table, max_pages, page_tokens, num_pages, scores, ctx, T, heads,
                                   dim, topk, out, status, stream);
}
