// Row operators of the hybrid decoder family (gated-delta layers + gated full-attention layers) that sit between its linears:
//
//   zc_rms_kernel          zero-centred RMSNorm over groups of `d` columns: y = x * rsqrt(mean(x^2) + eps) * (1 + w), f32 arithmetic,
//                          one warp per (row, group) - the hidden-wide norms (one group) and the per-head q / k norms
//   qk_prepare_kernel      full-attention layer: from q_proj's [heads, 2 * hd] rows (query half | gate half) and the k | v rows
//                          it writes the fused [q | k | v] row the rotary / cache-write kernel reads (q and k zero-centred
//                          RMS-normalised per head) and the gate half as its own row
//   sigmoid_mul_kernel     y = a * sigmoid(b), bf16 rounding of the sigmoid first (the gate is a bf16 tensor of the plan)
//   conv_silu_kernel       causal depthwise convolution (width <= 4) + SiLU over the token stream of every sequence slot;
//                          state = the previous width - 1 inputs per slot and channel, oldest first; a thread owns a channel
//                          and walks the rows in order, so rows of one sequence inside a chunk see one another
//   delta_prepare_kernel   per (row, head): q, k L2-normalised (sum of squares rounded to bf16 before eps is added),
//                          g = -exp(A_log) * softplus(a + dt_bias) in f32, beta = sigmoid(b) rounded to bf16; a row at
//                          position 0 clears the recurrent state of its sequence slot
//   gated_rms_kernel       y = (x * rsqrt(mean(x^2) + eps) * w) * silu(z) per head, f32 gain w (not 1 + w)
//
// All of them are launched with programmatic dependent launch like the rest of the decode chain. The recurrence itself is
// delta_rule_kernel (hc_ops.cu), attention is the GQA pair of decode_gqa.cu (partial rotary, head_dim 64 / 128 / 256).
// Reference: the typed plan of the checkpoint-bound compile path (crates/inferfabric-compiler/src/bound.rs:520-830) and the
// device operators behind it (native/src/inferfabric_acl.cpp:889-960 delta_prepare, native/src/qwen_model.cpp).
#include <cuda_fp16.h>

#include "common.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

__device__ __forceinline__ float siluf(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// grid = ceil(rows * groups / 8), 256 threads: one warp per (row, group)
__global__ void __launch_bounds__(256) zc_rms_kernel(const bf16* x, long ldx, const bf16* w, float eps, bf16* y, long ldy, int rows, int groups,
                                                    int d) {
  grid_dep_launch();
  grid_dep_wait();
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= rows * groups) return;
  const int r = item / groups, g = item % groups;
  const bf16* xr = x + (long)r * ldx + (long)g * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = __bfloat162float(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)d + eps);
  bf16* yr = y + (long)r * ldy + (long)g * d;
  for (int i = lane; i < d; i += 32) yr[i] = __float2bfloat16_rn(__bfloat162float(xr[i]) * inv * (1.f + __bfloat162float(w[i])));
}

// grid = ceil(T * (Hq + 2 * Hkv) / 8): one warp per (row, head of the fused output)
__global__ void __launch_bounds__(256) qk_prepare_kernel(const bf16* qg, long ldqg, const bf16* kv, long ldkv, const bf16* q_norm, const bf16* k_norm,
                                                        float eps, bf16* qkv, long ldqkv, bf16* gate, long ldg, int T, int Hq, int Hkv, int hd) {
  grid_dep_launch();
  grid_dep_wait();
  const int heads = Hq + 2 * Hkv;
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= T * heads) return;
  const int t = item / heads, h = item % heads;
  bf16* dst = qkv + (long)t * ldqkv + (long)h * hd;
  if (h >= Hq + Hkv) {     // value head: a copy
    const bf16* src = kv + (long)t * ldkv + (long)(h - Hq) * hd;
    for (int i = lane; i < hd; i += 32) dst[i] = src[i];
    return;
  }
  const bool is_q = h < Hq;
  const bf16* src = is_q ? qg + (long)t * ldqg + (long)h * 2 * hd : kv + (long)t * ldkv + (long)(h - Hq) * hd;
  const bf16* w = is_q ? q_norm : k_norm;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    const float v = __bfloat162float(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)hd + eps);
  for (int i = lane; i < hd; i += 32) dst[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * inv * (1.f + __bfloat162float(w[i])));
  if (is_q) {
    bf16* gd = gate + (long)t * ldg + (long)h * hd;
    for (int i = lane; i < hd; i += 32) gd[i] = src[hd + i];
  }
}

__global__ void __launch_bounds__(256) sigmoid_mul_kernel(const bf16* a, long lda, const bf16* b, long ldb, bf16* y, long ldy, int rows, int n) {
  grid_dep_launch();
  grid_dep_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * n) return;
  const int r = (int)(i / n), c = (int)(i % n);
  const float s = bf16_round(sigmoidf_(__bfloat162float(b[(long)r * ldb + c])));
  y[(long)r * ldy + c] = __float2bfloat16_rn(__bfloat162float(a[(long)r * lda + c]) * s);
}

// grid = ceil(C / 256); state bf16 [slots, C, width - 1], oldest first; w bf16 [C, width]
__global__ void __launch_bounds__(256) conv_silu_kernel(const bf16* x, long ldx, const bf16* w, bf16* state, const int32_t* positions,
                                                       const int32_t* slots, bf16* y, long ldy, int T, int C, int width) {
  grid_dep_launch();
  grid_dep_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float wk[4];
  for (int k = 0; k < width; ++k) wk[k] = __bfloat162float(w[(long)c * width + k]);
  for (int t = 0; t < T; ++t) {
    if (positions[t] < 0) continue;
    bf16* h = state + ((long)slots[t] * C + c) * (width - 1);
    if (positions[t] == 0)
      for (int k = 0; k + 1 < width; ++k) h[k] = __float2bfloat16_rn(0.f);      // a new sequence starts from an empty history
    const float xv = __bfloat162float(x[(long)t * ldx + c]);
    float acc = xv * wk[width - 1];
    for (int k = 0; k + 1 < width; ++k) acc = fmaf(__bfloat162float(h[k]), wk[k], acc);
    y[(long)t * ldy + c] = __float2bfloat16_rn(siluf(acc));
    for (int k = 0; k + 2 < width; ++k) h[k] = h[k + 1];
    h[width - 2] = __float2bfloat16_rn(xv);
  }
}

// grid = ceil(T * H / 8): one warp per (row, head). conv [T, 3 * H * d] (q | k | v), ab [T, 2 * H] (a | b) bf16.
__global__ void __launch_bounds__(256) delta_prepare_kernel(const bf16* conv, long ldc, const bf16* ab, long ldab, const float* a_log,
                                                           const float* dt_bias, float eps, bf16* q, bf16* k, float* g, float* beta,
                                                           const int32_t* positions, const int32_t* slots, float* state, int T, int H, int d) {
  grid_dep_launch();
  grid_dep_wait();
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= T * H) return;
  const int t = item / H, h = item % H;
  if (state != nullptr && positions[t] == 0) {      // a new sequence starts from an empty state
    float* S = state + ((long)slots[t] * H + h) * d * d;
    for (int i = lane; i < d * d; i += 32) S[i] = 0.f;
  }
  for (int which = 0; which < 2; ++which) {
    const bf16* src = conv + (long)t * ldc + ((long)which * H + h) * d;
    bf16* dst = (which == 0 ? q : k) + ((long)t * H + h) * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float v = __bfloat162float(src[i]);
      ss += v * v;
    }
    ss = bf16_round(warp_sum(ss));
    const float inv = rsqrtf(ss + eps);
    for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(__bfloat162float(src[i]) * inv);
  }
  if (lane == 0) {
    const float a = __bfloat162float(ab[(long)t * ldab + h]) + dt_bias[h];
    const float sp = a > 20.f ? a : log1pf(__expf(a));
    g[(long)t * H + h] = -__expf(a_log[h]) * sp;
    beta[(long)t * H + h] = bf16_round(sigmoidf_(__bfloat162float(ab[(long)t * ldab + H + h])));
  }
}

// grid = ceil(T * H / 8): one warp per (row, head); x [T, H, d] bf16, z rows with leading dimension ldz, w f32 [d]
__global__ void __launch_bounds__(256) gated_rms_kernel(const bf16* x, const bf16* z, long ldz, const float* w, float eps, bf16* y, long ldy, int T,
                                                       int H, int d) {
  grid_dep_launch();
  grid_dep_wait();
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= T * H) return;
  const int t = item / H, h = item % H;
  const bf16* xr = x + ((long)t * H + h) * d;
  const bf16* zr = z + (long)t * ldz + (long)h * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = __bfloat162float(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)d + eps);
  bf16* yr = y + (long)t * ldy + (long)h * d;
  for (int i = lane; i < d; i += 32) {
    yr[i] = __float2bfloat16_rn(__bfloat162float(xr[i]) * inv * w[i] * siluf(__bfloat162float(zr[i])));
  }
}

// Half-rotation RoPE over the first `rot` columns of every head of a row (pairs (i, i + rot / 2)), bf16-rounded cos / sin like the
// cache-write kernels; the other columns are copied. grid T, 256 threads.
__global__ void __launch_bounds__(256) rope_prefix_kernel(const bf16* x, long ldx, const int32_t* positions, bf16* y, long ldy, int heads, int hd, int rot,
                                                         float theta) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x, pos = positions[t], half = rot / 2;
  const bf16* xr = x + (long)t * ldx;
  bf16* yr = y + (long)t * ldy;
  for (int i = threadIdx.x; i < heads * hd; i += blockDim.x) {
    const int h = i / hd, c = i % hd;
    float v = __bfloat162float(xr[i]);
    if (c < rot && pos >= 0) {
      const int j = c < half ? c : c - half;
      const float inv_freq = exp2f(-(2.f * (float)j / (float)rot) * log2f(theta));
      float sn, cs;
      sincosf((float)pos * inv_freq, &sn, &cs);
      cs = bf16_round(cs);
      sn = bf16_round(sn);
      const float a = __bfloat162float(xr[h * hd + j]), b = __bfloat162float(xr[h * hd + j + half]);
      v = c < half ? a * cs - b * sn : b * cs + a * sn;
    }
    yr[i] = __float2bfloat16_rn(v);
  }
}

// Index keys of the step's rows into their pages: cache bf16 [pages, page_tokens, dim]. One warp per row.
__global__ void __launch_bounds__(256) index_cache_append_kernel(const bf16* key, long ldk, const int32_t* positions, const int32_t* slots,
                                                                const int32_t* page_table, int max_pages, int page_tokens, int num_pages, bf16* cache,
                                                                int T, int dim, uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const int pos = positions[t];
  if (pos < 0) return;
  const int lp = pos / page_tokens;
  const int page = lp < max_pages ? page_table[(long)slots[t] * max_pages + lp] : -1;
  if (page < 0 || page >= num_pages) {
    if (lane == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    return;
  }
  bf16* dst = cache + ((long)page * page_tokens + pos % page_tokens) * dim;
  for (int i = lane; i < dim; i += 32) dst[i] = key[(long)t * ldk + i];
}

// The same into an int8 index cache: q = rint(x / s) clamped to +-127 with one scale per row, s = max|x| / 127 rounded to half
// precision (what the CPU oracle keeps: rint(x / s) * s). cache int8 [pages, page_tokens, dim], scales half [pages, page_tokens].
__global__ void __launch_bounds__(256) index_cache_append_q8_kernel(const bf16* key, long ldk, const int32_t* positions, const int32_t* slots,
                                                                   const int32_t* page_table, int max_pages, int page_tokens, int num_pages,
                                                                   signed char* cache, __half* scales, int T, int dim, uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const int pos = positions[t];
  if (pos < 0) return;
  const int lp = pos / page_tokens;
  const int page = lp < max_pages ? page_table[(long)slots[t] * max_pages + lp] : -1;
  if (page < 0 || page >= num_pages) {
    if (lane == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    return;
  }
  const long row = (long)page * page_tokens + pos % page_tokens;
  float amax = 0.f;
  for (int i = lane; i < dim; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(key[(long)t * ldk + i])));
  amax = warp_max(amax);
  const __half sh = __float2half_rn(amax / 127.f);
  const float sc = __half2float(sh);
  if (lane == 0) scales[row] = sh;
  signed char* dst = cache + row * dim;
  for (int i = lane; i < dim; i += 32) {
    const float v = __bfloat162float(key[(long)t * ldk + i]);
    dst[i] = sc > 0.f ? (signed char)fmaxf(-127.f, fminf(127.f, rintf(v / sc))) : (signed char)0;
  }
}

// y = a + b, bf16 rows
__global__ void __launch_bounds__(256) add_rows_kernel(const bf16* a, long lda, const bf16* b, long ldb, bf16* y, long ldy, int rows, int n) {
  grid_dep_launch();
  grid_dep_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * n) return;
  const int r = (int)(i / n), c = (int)(i % n);
  y[(long)r * ldy + c] = __float2bfloat16_rn(__bfloat162float(a[(long)r * lda + c]) + __bfloat162float(b[(long)r * ldb + c]));
}

// y = silu(gate) * up, bf16 rows (gate and up may be column ranges of one projection or two projections)
__global__ void __launch_bounds__(256) swiglu_pair_kernel(const bf16* g, long ldg, const bf16* u, long ldu, bf16* y, long ldy, int rows, int n) {
  grid_dep_launch();
  grid_dep_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * n) return;
  const int r = (int)(i / n), c = (int)(i % n);
  const float a = __bfloat162float(g[(long)r * ldg + c]);
  y[(long)r * ldy + c] = __float2bfloat16_rn(a / (1.f + __expf(-a)) * __bfloat162float(u[(long)r * ldu + c]));
}

}  // namespace

extern "C" int ifab_swiglu_pair(const void* gate, long ldg, const void* up, long ldu, void* y, long ldy, int rows, int n, void* stream) {
  if (rows < 1 || n < 1) return -1;
  return launch_chain(swiglu_pair_kernel, dim3((unsigned)(((long)rows * n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, (const bf16*)gate, ldg,
                      (const bf16*)up, ldu, (bf16*)y, ldy, rows, n);
}

extern "C" int ifab_rope_prefix(const void* x, long ldx, const int32_t* positions, void* y, long ldy, int T, int heads, int head_dim, int rotary_dim,
                                float theta, void* stream) {
  if (T < 1 || heads < 1 || head_dim < 1 || rotary_dim < 2 || rotary_dim % 2 || rotary_dim > head_dim) return -1;
  return launch_chain(rope_prefix_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx, positions, (bf16*)y, ldy, heads, head_dim,
                      rotary_dim, theta);
}

extern "C" int ifab_index_cache_append(const void* key, long ldk, const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                       int max_pages, int page_tokens, int num_pages, void* cache, int T, int dim, uint32_t* status, void* stream) {
  if (T < 1 || dim < 1) return -1;
  return launch_chain(index_cache_append_kernel, dim3((T + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)key, ldk, positions, slots, page_table,
                      max_pages, page_tokens, num_pages, (bf16*)cache, T, dim, status);
}

extern "C" int ifab_index_cache_append_q8(const void* key, long ldk, const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                          int max_pages, int page_tokens, int num_pages, void* cache, void* scales, int T, int dim, uint32_t* status,
                                          void* stream) {
  if (T < 1 || dim < 1) return -1;
  return launch_chain(index_cache_append_q8_kernel, dim3((T + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)key, ldk, positions, slots,
                      page_table, max_pages, page_tokens, num_pages, (signed char*)cache, (__half*)scales, T, dim, status);
}

extern "C" int ifab_add_rows(const void* a, long lda, const void* b, long ldb, void* y, long ldy, int rows, int n, void* stream) {
  if (rows < 1 || n < 1) return -1;
  return launch_chain(add_rows_kernel, dim3((unsigned)(((long)rows * n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, (const bf16*)a, lda,
                      (const bf16*)b, ldb, (bf16*)y, ldy, rows, n);
}

extern "C" int ifab_zc_rmsnorm(const void* x, long ldx, const void* w, float eps, void* y, long ldy, int rows, int groups, int d, void* stream) {
  if (rows < 1 || groups < 1 || d < 1) return -1;
  return launch_chain(zc_rms_kernel, dim3((rows * groups + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx, (const bf16*)w, eps,
                      (bf16*)y, ldy, rows, groups, d);
}

extern "C" int ifab_hybrid_qk_prepare(const void* qg, long ldqg, const void* kv, long ldkv, const void* q_norm, const void* k_norm, float eps,
                                      void* qkv, long ldqkv, void* gate, long ldg, int T, int Hq, int Hkv, int hd, void* stream) {
  if (T < 1 || Hq < 1 || Hkv < 1 || hd < 1) return -1;
  return launch_chain(qk_prepare_kernel, dim3((T * (Hq + 2 * Hkv) + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)qg, ldqg,
                      (const bf16*)kv, ldkv, (const bf16*)q_norm, (const bf16*)k_norm, eps, (bf16*)qkv, ldqkv, (bf16*)gate, ldg, T, Hq, Hkv, hd);
}

extern "C" int ifab_sigmoid_mul(const void* a, long lda, const void* b, long ldb, void* y, long ldy, int rows, int n, void* stream) {
  if (rows < 1 || n < 1) return -1;
  return launch_chain(sigmoid_mul_kernel, dim3((unsigned)(((long)rows * n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, (const bf16*)a, lda,
                      (const bf16*)b, ldb, (bf16*)y, ldy, rows, n);
}

extern "C" int ifab_conv_silu(const void* x, long ldx, const void* w, void* state, const int32_t* positions, const int32_t* slots, void* y,
                              long ldy, int T, int C, int width, void* stream) {
  if (T < 1 || C < 1 || width < 2 || width > 4) return -1;
  return launch_chain(conv_silu_kernel, dim3((C + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx, (const bf16*)w,
                      (bf16*)state, positions, slots, (bf16*)y, ldy, T, C, width);
}

extern "C" int ifab_delta_prepare(const void* conv, long ldc, const void* ab, long ldab, const float* a_log, const float* dt_bias, float eps,
                                  void* q, void* k, float* g, float* beta, const int32_t* positions, const int32_t* slots, float* state, int T,
                                  int H, int d, void* stream) {
  if (T < 1 || H < 1 || d < 1 || (state != nullptr && (positions == nullptr || slots == nullptr))) return -1;
  return launch_chain(delta_prepare_kernel, dim3((T * H + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)conv, ldc, (const bf16*)ab,
                      ldab, a_log, dt_bias, eps, (bf16*)q, (bf16*)k, g, beta, positions, slots, state, T, H, d);
}

extern "C" int ifab_gated_rmsnorm(const void* x, const void* z, long ldz, const float* w, float eps, void* y, long ldy, int T, int H, int d,
                                  void* stream) {
  if (T < 1 || H < 1 || d < 1) return -1;
  return launch_chain(gated_rms_kernel, dim3((T * H + 7) / 8), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, (const bf16*)z, ldz, w, eps,
                      (bf16*)y, ldy, T, H, d);
}
