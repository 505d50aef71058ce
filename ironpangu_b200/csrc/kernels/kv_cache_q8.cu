// Packed int8 latent KV cache and activation quantisation.
//
// Packed row (656 bytes per token, 1.76x smaller than the 1152-byte bf16 row):
//   [0, 512)    latent, int8, symmetric per 128-column tile
//   [512, 640)  rotary key part, 64 bf16 (kept in bf16: it is small and precision-critical)
//   [640, 656)  4 f32 scales, one per latent tile
// A tile's scale is max|v| / 127 (1 for an all-zero tile) and values round half away from zero, clamped to +-127.
// The split-KV attention kernel reads these rows directly (ifab_mla_decode_attention with rope = -64).
//
//   mla_kv_write_q8_kernel   RMSNorm(latent) + RoPE(k_pe) + per-tile quantisation + paged write, one CTA per token
//   kv_dequantize_q8_kernel  packed rows -> bf16 rows (test / debugging utility)
//   quantize_int8_kernel     per-token or per-128-column symmetric int8 quantisation of activations [T, K]
// Reference counterparts: cache_c8_norm_rope_append (native/src/token_executor.h:760-794), the AscC
// cache_quantize / cache_dequantize kernels (native/kernels/cache_quantization.cpp:12-57), quantize / index_quantize
// (aclnnDynamicQuant, token_executor.h:406-418).
#include "mla_common.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::mla;

namespace {

constexpr int ROW_Q8 = LATENT + ROPE * 2 + 16;

__device__ __forceinline__ int quant_round(float v, float scale) {
  const float q = v / scale;   // IEEE division: bit-identical to the f32 reference
  const int r = (int)(q >= 0.f ? q + 0.5f : q - 0.5f);   // ties away from zero
  return max(-127, min(127, r));
}

// 128 threads; thread i owns latent columns [4i, 4i+4); a 128-column tile is one warp
// `kr` (optional): the rotary columns when they do not follow the latent columns in `kv`
__global__ void __launch_bounds__(128) mla_kv_write_q8_kernel(const bf16* kv, long ldkv, const bf16* kr, long ldkr, const bf16* norm_w, float eps, float theta,
                                                              const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                                              int max_pages, int page_tokens, unsigned char* cache, int num_pages,
                                                              uint32_t* status) {
  __shared__ float red[4];
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
  const bf16* src = kv + (long)t * ldkv;
  unsigned char* dst = cache + row * ROW_Q8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float f[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i] = __bfloat162float(src[tid * 4 + i]);
    ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)LATENT + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i] = bf16_round(f[i] * inv * __bfloat162float(norm_w[tid * 4 + i]));   // the value a bf16 cache would hold
    amax = fmaxf(amax, fabsf(f[i]));
  }
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 127.f : 1.f;
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) packed |= ((uint32_t)(quant_round(f[i], scale) & 0xff)) << (8 * i);
  reinterpret_cast<uint32_t*>(dst)[tid] = packed;
  if (lane == 0) reinterpret_cast<float*>(dst + LATENT + ROPE * 2)[warp] = scale;
  const int half = ROPE / 2;
  if (tid < half) {
    float c, s;
    rope_cos_sin(pos, tid, ROPE, theta, &c, &s);
    const bf16* rs = kr ? kr + (long)t * ldkr : src + LATENT;
    const float a = __bfloat162float(rs[tid]), b = __bfloat162float(rs[tid + half]);
    bf16* rp = reinterpret_cast<bf16*>(dst + LATENT);
    rp[tid] = __float2bfloat16_rn(a * c - b * s);
    rp[tid + half] = __float2bfloat16_rn(b * c + a * s);
  }
}

__global__ void __launch_bounds__(128) kv_dequantize_q8_kernel(const unsigned char* cache, bf16* out, long rows) {
  const long r = blockIdx.x;
  if (r >= rows) return;
  const unsigned char* src = cache + r * ROW_Q8;
  bf16* dst = out + r * ROW;
  const int tid = threadIdx.x;
  const float scale = reinterpret_cast<const float*>(src + LATENT + ROPE * 2)[tid >> 5];
  const uint32_t w = reinterpret_cast<const uint32_t*>(src)[tid];
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[tid * 4 + i] = __float2bfloat16_rn((float)(signed char)((w >> (8 * i)) & 0xff) * scale);
  if (tid < ROPE) dst[LATENT + tid] = reinterpret_cast<const bf16*>(src + LATENT)[tid];
}

// one warp per (row, group); group = whole row (group_cols = K) or 128 columns
__global__ void __launch_bounds__(256) quantize_int8_kernel(const bf16* x, long ldx, signed char* q, long ldq, float* scales, long lds,
                                                            int T, int K, int group_cols) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (K + group_cols - 1) / group_cols;
  const long unit = (long)blockIdx.x * 8 + warp;
  if (unit >= (long)T * groups) return;
  const int t = (int)(unit / groups), g = (int)(unit % groups);
  const int c0 = g * group_cols, c1 = min(K, c0 + group_cols);
  const bf16* xr = x + (long)t * ldx;
  float amax = 0.f;
  for (int c = c0 + lane; c < c1; c += 32) amax = fmaxf(amax, fabsf(__bfloat162float(xr[c])));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 127.f : 1.f;
  for (int c = c0 + lane; c < c1; c += 32) q[(long)t * ldq + c] = (signed char)quant_round(__bfloat162float(xr[c]), scale);
  if (lane == 0) scales[(long)t * lds + g] = scale;
}

}  // namespace

extern "C" int ifab_mla_kv_write_q8(const void* kv, long ldkv, const void* norm_w, float eps, float theta, const int32_t* positions,
                                    const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens, void* cache,
                                    int num_pages, int T, uint32_t* status, void* stream) {
  if (T < 1 || ldkv % 2) return -1;
  return launch_chain(mla_kv_write_q8_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, (const bf16*)kv, ldkv, (const bf16*)nullptr, 0L,
                      (const bf16*)norm_w, eps, theta, positions, slots, page_table, max_pages, page_tokens, (unsigned char*)cache, num_pages, status);
}

// the same with the rotary columns in rows of their own (latent_rows [T, >= 512], rope_rows [T, >= 64])
extern "C" int ifab_mla_kv_write_q8_split(const void* latent_rows, long ldl, const void* rope_rows, long ldr, const void* norm_w, float eps, float theta,
                                          const int32_t* positions, const int32_t* slots, const int32_t* page_table, int max_pages, int page_tokens,
                                          void* cache, int num_pages, int T, uint32_t* status, void* stream) {
  if (T < 1 || ldl % 2 || !rope_rows) return -1;
  return launch_chain(mla_kv_write_q8_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, (const bf16*)latent_rows, ldl, (const bf16*)rope_rows, ldr,
                      (const bf16*)norm_w, eps, theta, positions, slots, page_table, max_pages, page_tokens, (unsigned char*)cache, num_pages, status);
}

extern "C" int ifab_kv_dequantize_q8(const void* cache, void* out, long rows, void* stream) {
  if (rows < 1) return -1;
  kv_dequantize_q8_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>((const unsigned char*)cache, (bf16*)out, rows);
  return (int)cudaGetLastError();
}

// group_cols = K: one scale per row (scales [T, 1]); group_cols = 128: one per 128 columns (scales [T, ceil(K/128)])
extern "C" int ifab_quantize_int8(const void* x, long ldx, void* q, long ldq, float* scales, long lds, int T, int K, int group_cols,
                                  void* stream) {
  if (T < 1 || K < 1 || group_cols < 1) return -1;
  const long units = (long)T * ((K + group_cols - 1) / group_cols);
  return launch_chain(quantize_int8_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx,
                      (signed char*)q, ldq, scales, lds, T, K, group_cols);
}
