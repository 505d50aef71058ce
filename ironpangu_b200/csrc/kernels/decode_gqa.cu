// Grouped-query attention, decode / short-chunk path (dense model family), for sm_100a.
//
//   gqa_rope_kv_write_kernel  rotates q and k in place (half-rotation RoPE on the first rotary_dim
//                             columns of every head, device-computed angles) and scatters k / v rows
//                             into the paged caches [pages, page_tokens, kv_heads, head_dim]
//   gqa_split_kernel          split-KV online-softmax attention: one CTA per (split, kv head, query
//                             row) serves the G = Hq/Hkv query heads that share the kv head
//   gqa_merge_kernel          log-sum-exp merge of the splits -> [T, Hq*head_dim] bf16
//
// Query rows carry their own position and sequence slot (continuous batching: rows of different
// sequences and prefill chunks share one launch). Reference counterparts: attention_qk_prepare /
// paged_attention_prepare composites (native/src/inferfabric_acl.cpp:1236-1433).
#include "gemv.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

__device__ __forceinline__ void rope_cs(int pos, int i, int rot, float theta, float* c, float* s) {
  const float inv_freq = exp2f(-(2.f * (float)i / (float)rot) * log2f(theta));
  float sn, cs;
  sincosf((float)pos * inv_freq, &sn, &cs);
  *c = bf16_round(cs);
  *s = bf16_round(sn);
}
__device__ __forceinline__ long row_of(int pos, int slot, const int32_t* page_table, int max_pages, int page_tokens, int num_pages) {
  const int lp = pos / page_tokens;
  if (lp >= max_pages) return -1;
  const int page = page_table[(long)slot * max_pages + lp];
  if (page < 0 || page >= num_pages) return -1;
  return (long)page * page_tokens + (pos % page_tokens);
}

// grid T, 256 threads
__global__ void __launch_bounds__(256) gqa_rope_kv_write_kernel(bf16* qkv, long ld, const int32_t* positions, const int32_t* slots,
                                                                const int32_t* page_table, int max_pages, int page_tokens,
                                                                bf16* k_cache, bf16* v_cache, int num_pages, int Hq, int Hkv, int hd,
                                                                int rot, float theta, uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  if (pos < 0) return;
  bf16* row = qkv + (long)t * ld;
  const int half = rot / 2;
  // rotate q heads and k heads: (Hq + Hkv) * half pairs
  for (int i = threadIdx.x; i < (Hq + Hkv) * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    bf16* p = row + (long)h * hd;
    float c, s;
    rope_cs(pos, j, rot, theta, &c, &s);
    const float a = __bfloat162float(p[j]), b = __bfloat162float(p[j + half]);
    p[j] = __float2bfloat16_rn(a * c - b * s);
    p[j + half] = __float2bfloat16_rn(b * c + a * s);
  }
  __syncthreads();
  const long r = row_of(pos, slots[t], page_table, max_pages, page_tokens, num_pages);
  if (r < 0) {
    if (threadIdx.x == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    return;
  }
  const int kv_elems = Hkv * hd;
  const uint4* ksrc = reinterpret_cast<const uint4*>(row + (long)Hq * hd);
  const uint4* vsrc = reinterpret_cast<const uint4*>(row + (long)(Hq + Hkv) * hd);
  uint4* kdst = reinterpret_cast<uint4*>(k_cache + r * kv_elems);
  uint4* vdst = reinterpret_cast<uint4*>(v_cache + r * kv_elems);
  for (int c = threadIdx.x; c < kv_elems / 8; c += blockDim.x) {
    kdst[c] = ksrc[c];
    vdst[c] = vsrc[c];
  }
}

struct GqaParams {
  const bf16* q; long ldq; const bf16* k_cache; const bf16* v_cache;
  const int32_t* positions; const int32_t* slots; const int32_t* page_table;
  int max_pages, page_tokens, num_pages;
  float scale; int window;
  int T, Hq, Hkv, kps, max_splits;
  float* scratch;   // [T][Hq][max_splits][HD + 2]
  uint32_t* status;
};

// HD = head_dim (EPL = HD/32 elements per lane), G = query heads per kv head
template <int HD, int G>
__global__ void __launch_bounds__(256) gqa_split_kernel(GqaParams p) {
  constexpr int EPL = HD / 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sm_acc = reinterpret_cast<float*>(smem_raw);   // [8][G][HD]
  float* sm_m = sm_acc + 8 * G * HD;
  float* sm_l = sm_m + 8 * G;
  grid_dep_launch();
  grid_dep_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int pos = p.positions[t];
  if (pos < 0) return;
  int n = pos + 1;
  if (p.window > 0 && n > p.window) n = p.window;
  const int first = pos + 1 - n;
  const int k_begin = split * p.kps;
  if (k_begin >= n) return;
  // the last split also takes every key beyond max_splits * keys_per_split, so a long context is slower, never clipped
  const int k_end = (split == p.max_splits - 1) ? n : min(n, k_begin + p.kps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = p.slots[t];
  float qf[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bf16* qh = p.q + (long)t * p.ldq + (long)(kvh * G + g) * HD + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) qf[g][i] = __bfloat162float(qh[i]);
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[g][i] = 0.f;
  }
  const int kv_elems = p.Hkv * HD;
  constexpr int KB = 4;
  for (int kb = k_begin + warp; kb < k_end; kb += 8 * KB) {
    float kf[KB][EPL], vf[KB][EPL];
    bool ok[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const int k = kb + 8 * j;
      ok[j] = k < k_end;
      if (ok[j]) {
        const long r = row_of(first + k, slot, p.page_table, p.max_pages, p.page_tokens, p.num_pages);
        if (r < 0) {
          if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_BAD_INDEX);
          ok[j] = false;
        } else {
          const bf16* kr = p.k_cache + r * kv_elems + (long)kvh * HD + lane * EPL;
          const bf16* vr = p.v_cache + r * kv_elems + (long)kvh * HD + lane * EPL;
#pragma unroll
          for (int i = 0; i < EPL; i += 2) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + i));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr + i));
            kf[j][i] = a.x; kf[j][i + 1] = a.y;
            vf[j][i] = b.x; vf[j][i + 1] = b.y;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      if (!ok[j]) continue;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s = fmaf(qf[g][i], kf[j][i], s);
        s = warp_sum(s) * p.scale;
        const float mn = fmaxf(m[g], s);
        const float corr = __expf(m[g] - mn), pe = __expf(s - mn);
        l[g] = l[g] * corr + pe;
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[g][i] = acc[g][i] * corr + pe * vf[j][i];
        m[g] = mn;
      }
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      sm_m[warp * G + g] = m[g];
      sm_l[warp * G + g] = l[g];
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) sm_acc[((long)warp * G + g) * HD + lane * EPL + i] = acc[g][i];
  }
  __syncthreads();
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
    for (int w = 0; w < 8; ++w) M = fmaxf(M, sm_m[w * G + g]);
    float wgt[8], L = 0.f;
    for (int w = 0; w < 8; ++w) {
      wgt[w] = (sm_m[w * G + g] == -INFINITY) ? 0.f : __expf(sm_m[w * G + g] - M);
      L += wgt[w] * sm_l[w * G + g];
    }
    float* out = p.scratch + (((long)t * p.Hq + kvh * G + g) * p.max_splits + split) * (HD + 2);
    for (int c = threadIdx.x; c < HD; c += blockDim.x) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += wgt[w] * sm_acc[((long)w * G + g) * HD + c];
      out[c] = v;
    }
    if (threadIdx.x == 0) {
      out[HD] = M;
      out[HD + 1] = L;
    }
  }
}

// grid (Hq, T), HD threads
template <int HD>
__global__ void gqa_merge_kernel(GqaParams p, bf16* out, long ldo) {
  __shared__ float wgt[64];
  __shared__ float Ls;
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, t = blockIdx.y;
  const int pos = p.positions[t];
  if (pos < 0) return;
  int n = pos + 1;
  if (p.window > 0 && n > p.window) n = p.window;
  int ns = (n + p.kps - 1) / p.kps;
  if (ns > p.max_splits) ns = p.max_splits;
  const float* base = p.scratch + ((long)t * p.Hq + h) * p.max_splits * (HD + 2);
  if (threadIdx.x == 0) {
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, base[(long)s * (HD + 2) + HD]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float ms = base[(long)s * (HD + 2) + HD];
      const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
      wgt[s] = w;
      L += w * base[(long)s * (HD + 2) + HD + 1];
    }
    Ls = L;
  }
  __syncthreads();
  const float invL = Ls > 0.f ? 1.f / Ls : 0.f;
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < ns; ++s) v += wgt[s] * base[(long)s * (HD + 2) + c];
    out[(long)t * ldo + (long)h * HD + c] = __float2bfloat16_rn(v * invL);
  }
}

template <int HD, int G>
int launch_gqa(const GqaParams& p, bf16* out, long ldo, cudaStream_t s) {
  const size_t smem = (size_t)(8 * G * HD + 16 * G) * sizeof(float);
  auto k = gqa_split_kernel<HD, G>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid(p.max_splits, p.Hkv, p.T);
  if (int rc = launch_chain(k, grid, dim3(256), smem, s, p)) return rc;
  return launch_chain(gqa_merge_kernel<HD>, dim3(p.Hq, p.T), dim3(HD < 128 ? 64 : 128), 0, s, p, out, ldo);
}

template <int HD>
int dispatch_g(const GqaParams& p, bf16* out, long ldo, cudaStream_t s) {
  switch (p.Hq / p.Hkv) {
    case 1: return launch_gqa<HD, 1>(p, out, ldo, s);
    case 2: return launch_gqa<HD, 2>(p, out, ldo, s);
    case 4: return launch_gqa<HD, 4>(p, out, ldo, s);
    case 8: return launch_gqa<HD, 8>(p, out, ldo, s);
    default: return -1;
  }
}

}  // namespace

extern "C" int ifab_gqa_rope_kv_write(void* qkv, long ld, const int32_t* positions, const int32_t* slots,
                                      const int32_t* page_table, int max_pages, int page_tokens, void* k_cache, void* v_cache,
                                      int num_pages, int T, int Hq, int Hkv, int head_dim, int rotary_dim, float theta,
                                      uint32_t* status, void* stream) {
  if (head_dim % 8 || rotary_dim % 2 || rotary_dim > head_dim || ld % 8) return -1;
  return launch_chain(gqa_rope_kv_write_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (bf16*)qkv, ld, positions, slots,
                      page_table, max_pages, page_tokens, (bf16*)k_cache, (bf16*)v_cache, num_pages, Hq, Hkv, head_dim, rotary_dim,
                      theta, status);
}

extern "C" int ifab_gqa_decode_attention(const void* q, long ldq, const void* k_cache, const void* v_cache,
                                         const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                         int max_pages, int page_tokens, int num_pages, float scale, int T, int Hq, int Hkv,
                                         int head_dim, int keys_per_split, int max_splits, float* scratch,
                                         uint64_t scratch_bytes, void* out, long ldo, uint32_t* status, void* stream) {
  if (Hkv < 1 || Hq % Hkv || max_splits < 1 || max_splits > 64 || keys_per_split < 8) return -1;
  if ((uint64_t)T * Hq * max_splits * (head_dim + 2) * sizeof(float) > scratch_bytes) return -5;
  GqaParams p{(const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, positions, slots, page_table,
              max_pages, page_tokens, num_pages, scale, 0, T, Hq, Hkv, keys_per_split, max_splits, scratch, status};
  cudaStream_t s = (cudaStream_t)stream;
  switch (head_dim) {
    case 64: return dispatch_g<64>(p, (bf16*)out, ldo, s);
    case 128: return dispatch_g<128>(p, (bf16*)out, ldo, s);
    case 256: return dispatch_g<256>(p, (bf16*)out, ldo, s);
    default: return -1;
  }
}
