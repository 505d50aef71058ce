// Small kernels of the prefill path that have no decode counterpart:
//
//   mla_q_rope_kernel     rotary part of the absorbed query: q[t, h, nope:] -> q_lat[t, h, 512:576]
//                         (the latent part comes from a per-head tensor-core GEMM with W_uk)
//   mla_merge_kernel      log-sum-exp merge of the split-KV partials -> o_lat [T, H, 512] bf16
//                         (the value up-projection is a per-head tensor-core GEMM with W_uv afterwards)
//   allreduce_rows_kernel one-shot pull all-reduce of an f32 [rows, D] partial held in symmetric memory by every
//                         rank: every rank reads all partials through its peer mappings (plain loads), sums them in
//                         rank order, adds the residual and stores bf16. Used after the MoE combine of a prefill chunk.
#include <algorithm>

#include "mla_common.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::mla;

namespace {

__global__ void __launch_bounds__(64) mla_q_rope_kernel(const bf16* q, long ldq, const int32_t* positions, bf16* q_lat, int H,
                                                        int nope, int rope, float theta) {
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, t = blockIdx.y;
  const int half = rope / 2;
  const int i = threadIdx.x;
  if (i >= half) return;
  const int pos = positions[t];
  const bf16* qr = q + (long)t * ldq + (long)h * (nope + rope) + nope;
  bf16* out = q_lat + ((long)t * H + h) * ROW + LATENT;
  float c, s;
  rope_cos_sin(pos < 0 ? 0 : pos, i, rope, theta, &c, &s);
  const float a = __bfloat162float(qr[i]), b = __bfloat162float(qr[i + half]);
  out[i] = __float2bfloat16_rn(a * c - b * s);
  out[i + half] = __float2bfloat16_rn(b * c + a * s);
}

// rotary columns of every head of a [T, H * (nope + rope)] query matrix, rotated in place (thread i owns the pair i, i + rope / 2)
__global__ void __launch_bounds__(64) mla_q_rope_inplace_kernel(bf16* q, long ldq, const int32_t* positions, int nope, int rope, float theta) {
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, t = blockIdx.y;
  const int half = rope / 2;
  const int i = threadIdx.x;
  if (i >= half) return;
  const int pos = positions[t];
  bf16* qr = q + (long)t * ldq + (long)h * (nope + rope) + nope;
  float c, s;
  rope_cos_sin(pos < 0 ? 0 : pos, i, rope, theta, &c, &s);
  const float a = __bfloat162float(qr[i]), b = __bfloat162float(qr[i + half]);
  qr[i] = __float2bfloat16_rn(a * c - b * s);
  qr[i + half] = __float2bfloat16_rn(b * c + a * s);
}

// The latent cache rows of keys 0 .. ctx - 1 of one sequence slot, copied out of their pages into two dense matrices: the
// latent part [rows, 512] and the rotary part [rows, 64]; rows from ctx up to `rows` are zero. One CTA per row, one
// 16-byte chunk per thread.
__global__ void __launch_bounds__(72) mla_ctx_gather_kernel(const bf16* cache, const int32_t* page_table, int slot, int max_pages, int page_tokens,
                                                            int num_pages, int ctx, bf16* lat, bf16* pe, uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x, c = threadIdx.x;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (r < ctx) {
    const long row = cache_row_of(r, slot, page_table, max_pages, page_tokens, num_pages);
    if (row < 0) {
      if (c == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    } else {
      v = *reinterpret_cast<const uint4*>(cache + row * ROW + c * 8);
    }
  }
  if (c < LATENT / 8) *reinterpret_cast<uint4*>(lat + (long)r * LATENT + c * 8) = v;
  else *reinterpret_cast<uint4*>(pe + (long)r * ROPE + (c - LATENT / 8) * 8) = v;
}

// Keys and values 0 .. ctx - 1 of one sequence slot out of the paged GQA caches [pages, page_tokens, kv_heads * hd]: the keys as
// dense rows k[rows, W] (W = kv_heads * hd), the values TRANSPOSED as vt[W, ld] with one column per key - the operand layouts of
// the tensor-core prompt attention. Rows / columns from ctx up to `rows` are zero. One CTA per 32 keys: the values go through a
// shared-memory tile so that both the reads (along a cache row) and the writes (32 consecutive keys of one column) coalesce.
__global__ void __launch_bounds__(256) gqa_ctx_gather_kernel(const bf16* k_cache, const bf16* v_cache, const int32_t* page_table, int slot,
                                                             int max_pages, int page_tokens, int num_pages, int ctx, int W, bf16* k, bf16* vt,
                                                             long ldvt, uint32_t* status) {
  __shared__ bf16 tile[32][256 + 2];
  __shared__ long src_row[32];
  grid_dep_launch();
  grid_dep_wait();
  const int j0 = blockIdx.x * 32, t = threadIdx.x;
  if (t < 32) {
    const int j = j0 + t;
    long row = -1;
    if (j < ctx) {
      row = cache_row_of(j, slot, page_table, max_pages, page_tokens, num_pages);
      if (row < 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    }
    src_row[t] = row;
  }
  __syncthreads();
  for (int c0 = 0; c0 < W; c0 += 256) {
    const int c = c0 + t;
    for (int kk = 0; kk < 32; ++kk) {
      const long row = src_row[kk];
      bf16 kv = __float2bfloat16_rn(0.f), vv = kv;
      if (row >= 0 && c < W) {
        kv = k_cache[row * W + c];
        vv = v_cache[row * W + c];
      }
      if (c < W) k[(long)(j0 + kk) * W + c] = kv;
      tile[kk][t] = vv;
    }
    __syncthreads();
    const int key = t & 31;
    for (int cc = t >> 5; cc < 256 && c0 + cc < W; cc += 8) vt[(long)(c0 + cc) * ldvt + j0 + key] = tile[key][cc];
    __syncthreads();
  }
}

struct MergeParams {
  const float* scratch;   // [T][H][max_splits][LATENT + 2]
  const int32_t* positions;
  int n_sinks, window, kps, max_splits, H;
  bf16* o_lat;            // [T][H][LATENT]
};

__global__ void __launch_bounds__(256) mla_merge_kernel(MergeParams p) {
  __shared__ float wgt[64];
  __shared__ float Ls;
  grid_dep_launch();
  grid_dep_wait();
  const int h = blockIdx.x, t = blockIdx.y;
  const int pos = p.positions[t];
  bf16* out = p.o_lat + ((long)t * p.H + h) * LATENT;
  if (pos < 0) {
    for (int c = threadIdx.x; c < LATENT; c += blockDim.x) out[c] = __float2bfloat16_rn(0.f);
    return;
  }
  int first, nctx;
  visible_range(pos, p.window, &first, &nctx);
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
    out[c] = __float2bfloat16_rn(v * invL);
  }
}

struct ArRowsParams {
  const float* parts[IFAB_MAX_RANKS];   // parts[r]: rank r's partial as mapped here (parts[rank] is local)
  const bf16* residual; long ldr;
  bf16* out; long ldo;
  long rows; int D;
  FabricView fv; uint64_t* seq; uint32_t* done;
};

__global__ void __launch_bounds__(256) allreduce_rows_kernel(ArRowsParams p) {
  __shared__ int s_ok, s_last;
  grid_dep_launch();
  grid_dep_wait();
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(p.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  const int world = p.fv.world, rank = p.fv.rank;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (world > 1) {
    // this rank's partial was written by the previous kernel of the stream: tell every peer, then wait for theirs
    if (blockIdx.x == 0 && (int)threadIdx.x < world && (int)threadIdx.x != rank) {
      __threadfence_system();
      st_release_sys(p.fv.flags[threadIdx.x] + (size_t)par * p.fv.flag_half_words + rank, epoch);
    }
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
      if (!wait_flag_bounded(p.fv.flags[rank] + (size_t)par * p.fv.flag_half_words + threadIdx.x, epoch, p.fv.spin_limit)) {
        s_ok = 0;
        atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
      }
    }
    __syncthreads();
  }
  if (s_ok) {
    const long chunks = p.rows * (p.D >> 2);   // float4 chunks
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (long)gridDim.x * blockDim.x) {
      const long row = i / (p.D >> 2);
      const int c = (int)(i % (p.D >> 2)) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(p.parts[r] + row * p.D + c);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float o[4] = {acc.x, acc.y, acc.z, acc.w};
      if (p.residual) {
        const bf16* rr = p.residual + row * p.ldr + c;
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = bf16_round(o[k]) + __bfloat162float(rr[k]);
      }
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(p.out + row * p.ldo + c);
      dst[0] = __floats2bfloat162_rn(o[0], o[1]);
      dst[1] = __floats2bfloat162_rn(o[2], o[3]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(p.done, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    *p.done = 0;
    *p.seq = epoch;
    __threadfence();
  }
}

// Two-shot all-reduce through the NVLink switch (NVLS). Rank r owns the float4 chunks i with i % world == r:
//   1. flag exchange: every rank's partial is in its own memory and visible;
//   2. the owner reads the sum of a chunk over all ranks with ONE multimem.ld_reduce (the switch adds the eight copies)
//      and writes it back to all eight copies with ONE multimem.st: a rank receives and sends 1/world of what the
//      pull form above moves;
//   3. second flag exchange: every rank's copy now holds the complete sums; each rank converts its own copy
//      (bf16, + residual) with local loads only.
// Every element is reduced by exactly one rank, so all ranks end with bit-identical rows.
struct ArNvlsParams {
  float* part_local;      // this rank's copy of the partial / result buffer [rows, D]
  float* part_mc;         // multicast address of the same buffer
  const bf16* residual; long ldr;
  bf16* out; long ldo;
  long rows; int D;
  FabricView fv; uint64_t* seq; uint32_t* done;
  uint32_t* arrive;       // local counter for the in-grid barrier between steps 2 and 3
};

// all CTAs of the grid are resident (grid <= 2 per SM); CTA 0 talks to the peers
__device__ __forceinline__ bool nvls_rank_barrier(const ArNvlsParams& p, uint64_t want, int slot_base, uint32_t par) {
  // called by threads < world of CTA 0
  const int q = threadIdx.x, rank = p.fv.rank;
  if (q == rank) return true;
  st_release_sys(p.fv.flags[q] + (size_t)par * p.fv.flag_half_words + slot_base + rank, want);
  return wait_flag_bounded(p.fv.flags[rank] + (size_t)par * p.fv.flag_half_words + slot_base + q, want, p.fv.spin_limit);
}

__global__ void __launch_bounds__(256) allreduce_rows_nvls_kernel(ArNvlsParams p) {
  __shared__ int s_ok, s_last;
  grid_dep_launch();
  grid_dep_wait();
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(p.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  const int world = p.fv.world, rank = p.fv.rank;
  const uint32_t G = gridDim.x;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // in-grid barrier: CTA 0 does the cross-rank part, publishes `phase` in arrive[1]; the others wait for it
  auto grid_phase = [&](uint32_t phase, int slot_base) {
    __syncthreads();
    if (blockIdx.x == 0) {
      // wait until every CTA of this rank has finished the step before (its stores fenced)
      if (threadIdx.x == 0) {
        __threadfence_system();
        bool ok = false;
        for (uint32_t i = 0; i < p.fv.spin_limit; ++i) {
          if (*reinterpret_cast<volatile uint32_t*>(p.arrive) == (G - 1) * phase) { ok = true; break; }
          if (i > 64) __nanosleep(40);
        }
        if (!ok) { s_ok = 0; atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT); }
        __threadfence_system();
      }
      __syncthreads();
      if ((int)threadIdx.x < world && !nvls_rank_barrier(p, epoch, slot_base, par)) {
        s_ok = 0;
        atomicOr(p.fv.status, IFAB_STATUS_PEER_TIMEOUT);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.arrive + 1) = s_ok ? (uint32_t)epoch * 4u + phase : 0xffffffffu;
      }
    } else {
      if (threadIdx.x == 0) {
        __threadfence_system();
        atomicAdd(p.arrive, 1u);
        bool ok = false;
        const uint32_t want = (uint32_t)epoch * 4u + phase;
        for (uint32_t i = 0; i < p.fv.spin_limit; ++i) {
          const uint32_t v = *reinterpret_cast<volatile uint32_t*>(p.arrive + 1);
          if (v == want) { ok = true; break; }
          if (v == 0xffffffffu) break;
          if (i > 64) __nanosleep(40);
        }
        if (!ok) s_ok = 0;
        __threadfence();
      }
    }
    __syncthreads();
  };
  const long chunks = p.rows * (p.D >> 2);   // float4 chunks
  grid_phase(1, 0);                          // every rank's partial is complete
  if (s_ok) {
    for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * world + rank; i < chunks; i += (long)G * blockDim.x * world) {
      const float4 v = multimem_ld_reduce_f32x4(p.part_mc + i * 4);
      multimem_st_f32x4(p.part_mc + i * 4, v);
    }
  }
  grid_phase(2, world);                      // every owner's sums have reached every copy
  if (s_ok) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (long)G * blockDim.x) {
      const long row = i / (p.D >> 2);
      const int c = (int)(i % (p.D >> 2)) * 4;
      const float4 acc = __ldcg(reinterpret_cast<const float4*>(p.part_local + row * p.D + c));
      float o[4] = {acc.x, acc.y, acc.z, acc.w};
      if (p.residual) {
        const bf16* rr = p.residual + row * p.ldr + c;
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = bf16_round(o[k]) + __bfloat162float(rr[k]);
      }
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(p.out + row * p.ldo + c);
      dst[0] = __floats2bfloat162_rn(o[0], o[1]);
      dst[1] = __floats2bfloat162_rn(o[2], o[3]);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(p.done, 1u) == G - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    *p.done = 0;
    p.arrive[0] = 0;
    *p.seq = epoch;
    __threadfence();
  }
}

}  // namespace

extern "C" int ifab_mla_q_rope(const void* q, long ldq, const int32_t* positions, void* q_lat, int T, int H, int nope, int rope,
                               float theta, void* stream) {
  if (rope != ROPE || T < 1 || H < 1) return -1;
  return launch_chain(mla_q_rope_kernel, dim3(H, T), dim3(64), 0, (cudaStream_t)stream, (const bf16*)q, ldq, positions, (bf16*)q_lat, H,
                      nope, rope, theta);
}

extern "C" int ifab_mla_merge(const float* scratch, const int32_t* positions, int n_sinks, int window, int keys_per_split,
                              int max_splits, int T, int H, void* o_lat, void* stream) {
  if (max_splits < 1 || max_splits > 64 || T < 1 || H < 1) return -1;
  MergeParams p{scratch, positions, n_sinks, window, keys_per_split, max_splits, H, (bf16*)o_lat};
  return launch_chain(mla_merge_kernel, dim3(H, T), dim3(256), 0, (cudaStream_t)stream, p);
}

// parts[r] (r < world): rank r's f32 [rows, D] partial in symmetric memory as mapped into this process. Partials must be
// double buffered by the caller (alternate two symmetric buffers between consecutive calls).
extern "C" int ifab_allreduce_rows(const void* const* parts, const void* residual, long ldr, void* out, long ldo, long rows, int D,
                                   const IfabFabric* fab, void* stream) {
  if (rows < 1 || D % 4 || (residual && ldr % 4) || ldo % 4) return -1;
  ArRowsParams p;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) p.parts[r] = r < fab->world ? (const float*)parts[r] : nullptr;
  p.residual = (const bf16*)residual; p.ldr = ldr; p.out = (bf16*)out; p.ldo = ldo; p.rows = rows; p.D = D;
  p.seq = fab->seq; p.done = fab->done;
  if ((size_t)fab->world > fab->flag_half_words) return -4;
  const long chunks = rows * (D >> 2);
  const int grid = (int)std::min<long>(2 * 148, (chunks + 255) / 256);
  return launch_chain(allreduce_rows_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p);
}

// NVLS form of ifab_allreduce_rows: part_local / part_mc are this rank's mapping and the multicast mapping of ONE f32
// [rows, D] buffer in symmetric memory that holds this rank's partial on entry and the complete sums on exit (alternate two
// buffers between consecutive calls). arrive: 2 zeroed uint32 words on this device, used only by this kernel.
extern "C" int ifab_allreduce_rows_nvls(void* part_local, void* part_mc, const void* residual, long ldr, void* out, long ldo, long rows,
                                        int D, uint32_t* arrive, const IfabFabric* fab, void* stream) {
  if (rows < 1 || D % 4 || (residual && ldr % 4) || ldo % 4 || part_mc == nullptr || arrive == nullptr) return -1;
  ArNvlsParams p;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.part_local = (float*)part_local; p.part_mc = (float*)part_mc;
  p.residual = (const bf16*)residual; p.ldr = ldr; p.out = (bf16*)out; p.ldo = ldo; p.rows = rows; p.D = D;
  p.seq = fab->seq; p.done = fab->done; p.arrive = arrive;
  if ((size_t)2 * fab->world > fab->flag_half_words) return -4;
  const long chunks = rows * (D >> 2);
  // the CTAs wait on one another: never more than are resident at once (one per SM is enough to saturate the links)
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -6;
  }
  const int grid = (int)std::min<long>(sms, (chunks + 255) / 256);
  return launch_chain(allreduce_rows_nvls_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p);
}

extern "C" int ifab_mla_q_rope_inplace(void* q, long ldq, const int32_t* positions, int T, int H, int nope, int rope, float theta, void* stream) {
  if (rope != ROPE || T < 1 || H < 1) return -1;
  return launch_chain(mla_q_rope_inplace_kernel, dim3(H, T), dim3(64), 0, (cudaStream_t)stream, (bf16*)q, ldq, positions, nope, rope, theta);
}

// lat: [rows, 512], pe: [rows, 64] (rows >= ctx; the tail is zeroed)
extern "C" int ifab_gqa_ctx_gather(const void* k_cache, const void* v_cache, const int32_t* page_table, int slot, int max_pages, int page_tokens,
                                   int num_pages, int ctx, int rows, int width, void* k, void* vt, long ldvt, uint32_t* status, void* stream) {
  if (ctx < 1 || rows < ctx || rows % 32 || slot < 0 || width < 1 || ldvt < rows) return -1;
  return launch_chain(gqa_ctx_gather_kernel, dim3(rows / 32), dim3(256), 0, (cudaStream_t)stream, (const bf16*)k_cache, (const bf16*)v_cache,
                      page_table, slot, max_pages, page_tokens, num_pages, ctx, width, (bf16*)k, (bf16*)vt, ldvt, status);
}

extern "C" int ifab_mla_ctx_gather(const void* cache, const int32_t* page_table, int slot, int max_pages, int page_tokens, int num_pages, int ctx,
                                   int rows, void* lat, void* pe, uint32_t* status, void* stream) {
  if (ctx < 1 || rows < ctx || slot < 0) return -1;
  return launch_chain(mla_ctx_gather_kernel, dim3(rows), dim3(72), 0, (cudaStream_t)stream, (const bf16*)cache, page_table, slot, max_pages,
                      page_tokens, num_pages, ctx, (bf16*)lat, (bf16*)pe, status);
}
