// Helpers shared by the MLA decode and prompt kernels: row geometry of the latent
// cache (512 latent + 64 rope columns per token), RoPE angles, page-table lookup, visible key range.
#pragma once
#include "common.cuh"

namespace ifab::mla {

constexpr int LATENT = 512;
constexpr int ROPE = 64;
constexpr int ROW = LATENT + ROPE;

__device__ __forceinline__ void rope_cos_sin(int pos, int i, int rope_dim, float theta, float* c, float* s) {
  // angle_i = pos / theta^(2i/rope_dim); cos/sin are rounded to bf16 like the tables of the reference
  const float inv_freq = exp2f(-(2.f * (float)i / (float)rope_dim) * log2f(theta));
  float sn, cs;
  sincosf((float)pos * inv_freq, &sn, &cs);
  *c = bf16_round(cs);
  *s = bf16_round(sn);
}

__device__ __forceinline__ long cache_row_of(int pos, int slot, const int32_t* page_table, int max_pages,
                                             int page_tokens, int num_pages) {
  const int lp = pos / page_tokens;
  if (lp >= max_pages) return -1;
  const int page = page_table[(long)slot * max_pages + lp];
  if (page < 0 || page >= num_pages) return -1;
  return (long)page * page_tokens + (pos % page_tokens);
}

// key-space of one query: sink rows first, then the visible context rows
__device__ __forceinline__ void visible_range(int pos, int window, int* first, int* count) {
  int n = pos + 1;
  if (window > 0 && n > window) n = window;
  *count = n;
  *first = pos + 1 - n;
}

// lane layout of one 576-wide row: latent elements [8l, 8l+8) and [256+8l, 256+8l+8), rope elements 2l, 2l+1
struct RowFrag {
  float lat[16];
  float rp[2];
};
__device__ __forceinline__ void load_row(const bf16* row, int lane, RowFrag* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(row + lane * 8);
  const uint4 b = *reinterpret_cast<const uint4*>(row + 256 + lane * 8);
  const __nv_bfloat162 r = *reinterpret_cast<const __nv_bfloat162*>(row + LATENT + lane * 2);
  unpack8(a, f->lat);
  unpack8(b, f->lat + 8);
  const float2 rr = __bfloat1622float2(r);
  f->rp[0] = rr.x;
  f->rp[1] = rr.y;
}

}  // namespace ifab::mla
