// Decode-time expert FFN over block-scaled fp8 (e4m3) expert weights.
//
// Storage: a weight matrix [rows, K] is kept as one byte per element plus one f32 scale per 1 x 128 block of a row
// (scales[row][ceil(K / 128)]); the represented value is fp8(w[row][k]) * scale[row][k / 128]. Decode linears are bound
// by the HBM stream of the weights, so halving the bytes of the expert matrices - 3/4 of the bytes a token touches in a
// mixture-of-experts layer - is what this buys; the arithmetic stays f32: every lane converts its 16-byte chunk (16
// weights) to f32, forms the chunk's dot product with the bf16 activations staged in shared memory, and scales it once.
// The kernels mirror the bf16 ones of decode_moe.cu (same grids, same routing inputs, same fused all-reduce), only the
// chunk geometry differs: 16 elements per 16-byte load instead of 8.
// Reference: W8A8 expert matrices of the 92B program (dequantising grouped matmul, native/src/token_executor.h:640-700).
#include <cuda_fp8.h>

#include <algorithm>

#include "gemv.cuh"
#include "ifab_kernels.h"
#include "oneshot_ar.cuh"

using namespace ifab;

namespace {

constexpr int QBLOCK = 128;
constexpr int MAX_TOPK8 = 16;

// Dot product of one 16-byte chunk (16 fp8 weights) with 16 activations held as f16: the weights convert pairwise to f16
// (one instruction per pair) and multiply-accumulate as half2, eight terms per half, before ONE conversion to f32 - three
// times fewer instructions than converting every weight to f32, which is what makes the halved bytes show up as time.
// The activations are staged scaled by kXScale so that eight products of a weight (|w| <= 448 after block scaling) and an
// activation stay far inside the f16 range; the caller multiplies the result by 1 / kXScale together with the block scale.
constexpr float kXScale = 1.f / 16.f;
__device__ __forceinline__ float dot16_e4m3_f16(const uint4& w, const __half2* xh) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  __half2 acc = __float2half2_rn(0.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((ww[i] >> (16 * h)) & 0xffffu), __NV_E4M3);
      acc = __hfma2(*reinterpret_cast<const __half2*>(&hr), xh[i * 2 + h], acc);
    }
  }
  const float2 f = __half22float2(acc);
  return f.x + f.y;
}
// 8 bf16 -> 8 f16 scaled by kXScale
__device__ __forceinline__ uint4 bf16x8_to_scaled_f16(const uint4& v) {
  float f[8];
  unpack8(v, f);
  uint4 o;
  __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i] * kXScale, f[2 * i + 1] * kXScale);
  return o;
}

// ---- quantiser: one warp per (row, block) ------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_fp8_block_kernel(const bf16* __restrict__ w, long ldw, long rows, int K, uint8_t* q,
                                                                 float* scales) {
  const int nb = (K + QBLOCK - 1) / QBLOCK;
  const long item = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= rows * nb) return;
  const long row = item / nb;
  const int b = (int)(item % nb), lane = threadIdx.x & 31;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = b * QBLOCK + lane * 4 + i;
    v[i] = k < K ? __bfloat162float(w[row * ldw + k]) : 0.f;
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  if (lane == 0) scales[row * nb + b] = scale;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int k = b * QBLOCK + lane * 4 + i;
    if (k < K) q[row * (long)K + k] = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(v[i], scale), __NV_SATFINITE, __NV_E4M3);
  }
}

// ---- dequantiser: 16 values per thread (one 16-byte load, two 16-byte stores); K % 16 == 0 ------------------------------------------
// out = bf16(fp8(q) * scale): the operand form of the tensor-core prompt path, which widens one layer's experts at a time
__global__ void __launch_bounds__(256) dequantize_fp8_block_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales, long rows, int K,
                                                                   bf16* __restrict__ out) {
  grid_dep_launch();
  grid_dep_wait();
  const int per_row = K / 16, nb = (K + QBLOCK - 1) / QBLOCK;
  const long total = rows * per_row;
  for (long item = (long)blockIdx.x * blockDim.x + threadIdx.x; item < total; item += (long)gridDim.x * blockDim.x) {
    const long row = item / per_row;
    const int c = (int)(item % per_row) * 16;
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(q + row * (long)K + c));
    const float sc = scales[row * nb + c / QBLOCK];
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    float f[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = __half2float(__half(__nv_cvt_fp8_to_halfraw(b[i], __NV_E4M3))) * sc;
    uint4* dst = reinterpret_cast<uint4*>(out + row * (long)K + c);
    dst[0] = pack8(f);
    dst[1] = pack8(f + 8);
  }
}

// ---- gate/up -------------------------------------------------------------------------------------------
struct GateUp8Params {
  const bf16* x; long ldx; const bf16* norm_w; float eps;
  const int32_t* ids; int T, D, F, topk, e0, e_local;
  const uint8_t* w_gu; const float* s_gu; const uint8_t* w_sgu; const float* s_sgu; int Fs;
  bf16* act;
};

// grid: (ceil(F/16), T*topk + T), the layout of the bf16 kernel: a warp owns gate rows j0, j0+1 and up rows j0, j0+1.
__global__ void __launch_bounds__(256) moe_gate_up_fp8_kernel(GateUp8Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[33];
  grid_dep_launch();
  const int routes = p.T * p.topk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j0 = (blockIdx.x * 8 + warp) * 2;
  const bool shared_col = (int)blockIdx.y >= routes;
  const int nb = (p.D + QBLOCK - 1) / QBLOCK, chunks = p.D >> 4;
  const uint8_t* rows[4] = {nullptr, nullptr, nullptr, nullptr};
  const float* srow[4] = {nullptr, nullptr, nullptr, nullptr};
  int t, slot, Fcur;
  const uint8_t* W;
  const float* S;
  if (shared_col) {
    t = blockIdx.y - routes;
    slot = p.topk;
    W = p.w_sgu;
    S = p.s_sgu;
    Fcur = W ? p.Fs : 0;
  } else {
    grid_dep_wait();
    t = blockIdx.y / p.topk;
    slot = blockIdx.y % p.topk;
    const int e = p.ids[blockIdx.y];
    if (e < p.e0 || e >= p.e0 + p.e_local) return;
    W = p.w_gu + (size_t)(e - p.e0) * 2 * p.F * p.D;
    S = p.s_gu + (size_t)(e - p.e0) * 2 * p.F * nb;
    Fcur = p.F;
  }
  if (j0 < Fcur) {
    const int r[4] = {j0, j0 + 1, Fcur + j0, Fcur + j0 + 1};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if ((i & 1) && j0 + 1 >= Fcur) continue;
      rows[i] = W + (size_t)r[i] * p.D;
      srow[i] = S + (size_t)r[i] * nb;
    }
  }
  constexpr int U = 4;   // 16 chunks of 16 bytes in flight per lane, over 4 rows
  uint4 pf[U][4];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int c = lane + u * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) pf[u][i] = (c < chunks && rows[i]) ? ld_stream16(rows[i] + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
  }
  if (shared_col) grid_dep_wait();
  if ((int)blockIdx.x * 16 >= Fcur) return;
  stage_x<1>(xs, p.x, p.ldx, t, p.T, p.D, p.norm_w, p.eps, false, red);
  // the normalised row, in place, as scaled f16 (same 2 bytes per element)
  for (int c = threadIdx.x; c < (p.D >> 3); c += blockDim.x) {
    uint4* q = reinterpret_cast<uint4*>(xs + c * 8);
    *q = bf16x8_to_scaled_f16(*q);
  }
  __syncthreads();
  const __half2* xh = reinterpret_cast<const __half2*>(xs);
  if (j0 >= Fcur) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
    if (c0 != lane) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) pf[u][i] = (c < chunks && rows[i]) ? ld_stream16(rows[i] + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * 32;
      if (c < chunks) {
        __half2 xv[8];
        *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(xh + c * 8);
        *reinterpret_cast<uint4*>(xv + 4) = *reinterpret_cast<const uint4*>(xh + c * 8 + 4);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (rows[i] == nullptr) continue;
          acc[i] = fmaf(__ldg(srow[i] + (c >> 3)), dot16_e4m3_f16(pf[u][i], xv), acc[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = warp_sum(acc[i]);
  if (lane == 0) {
    constexpr float un = 1.f / kXScale;
    bf16* out = p.act + ((size_t)t * (p.topk + 1) + slot) * p.F;
    out[j0] = __float2bfloat16_rn(silu(bf16_round(acc[0] * un)) * bf16_round(acc[2] * un));
    if (j0 + 1 < Fcur) out[j0 + 1] = __float2bfloat16_rn(silu(bf16_round(acc[1] * un)) * bf16_round(acc[3] * un));
  }
}

// ---- down + all-reduce ---------------------------------------------------------------------------------
struct Down8Params {
  const bf16* act; const int32_t* ids; const float* wts;
  int T, D, F, topk, e0, e_local;
  const uint8_t* w_down; const float* s_down; const uint8_t* w_sdown; const float* s_sdown; int Fs;
  const bf16* residual; long ldr; bf16* y; long ldy;
  FabricView fv; uint64_t* seq; uint32_t* done;
};

// The K dimension of all local routes of a token is flattened into one space of 16-element chunks, as in the bf16 kernel:
//   y[t][n] = sum_s wgt_s * sum_blocks scale_s[n][b] * dot(W8_s[n, block b], act[t][s][block b])
template <int T, int R>
__global__ void __launch_bounds__(256) moe_down_fp8_allreduce_kernel(Down8Params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* as = reinterpret_cast<bf16*>(smem_raw);   // [(topk+1)][F] activation rows of the current token, held as scaled f16 (2 bytes each)
  constexpr int RPC = 8 * R;
  constexpr int MAXS = MAX_TOPK8 + 1;
  __shared__ float slab[T * RPC];
  __shared__ int timed_out;
  __shared__ const uint8_t* s_w[MAXS];
  __shared__ const float* s_sc[MAXS];
  __shared__ float s_g[MAXS];
  __shared__ int s_k[MAXS];
  __shared__ int s_cbeg[MAXS + 1];
  __shared__ int s_slot[MAXS];
  __shared__ int s_n;
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nbase = blockIdx.x * RPC, n0 = nbase + warp * R;
  if (threadIdx.x == 0) timed_out = 0;
  for (int t = 0; t < T; ++t) {
    if (t < p.T) {
      __syncthreads();
      if (warp == 0) {
        // route table, one slot per lane (ids and scores of all slots requested at once), compacted with a ballot
        const int slot = lane;
        bool local = false;
        const uint8_t* w = nullptr;
        const float* sc = nullptr;
        float g = 0.f;
        int k = 0;
        if (slot < p.topk) {
          const int e = p.ids[t * p.topk + slot];
          local = e >= p.e0 && e < p.e0 + p.e_local;
          const size_t el = local ? (size_t)(e - p.e0) : 0;
          w = p.w_down + el * p.D * p.F;
          sc = p.s_down + el * p.D * ((p.F + QBLOCK - 1) / QBLOCK);
          g = p.wts[t * p.topk + slot];
          k = p.F;
        } else if (slot == p.topk && p.w_sdown != nullptr) {
          local = true;
          w = p.w_sdown;
          sc = p.s_sdown;
          g = 1.f;
          k = p.Fs;
        }
        const unsigned m = __ballot_sync(0xffffffffu, local);
        const int n = __popc(m & ((1u << lane) - 1u));
        if (local) {
          s_w[n] = w;
          s_sc[n] = sc;
          s_g[n] = g;
          s_k[n] = k;
          s_slot[n] = slot;
          s_cbeg[n] = n * (p.F >> 4);              // every route before the shared expert spans F
        }
        if (lane == 0) {
          const int total_n = __popc(m), shared = (int)((m >> p.topk) & 1u);
          s_cbeg[total_n] = (total_n - shared) * (p.F >> 4) + shared * (p.Fs >> 4);
          s_n = total_n;
        }
      }
      __syncthreads();
      const int n_routes = s_n;
      {
        // activation rows of the local routes -> scaled f16 in shared memory: eight loads in flight per thread
        const int kch0 = max(1, p.F >> 3);
        const int shared_last = (n_routes > 0 && s_slot[n_routes - 1] == p.topk) ? 1 : 0;
        const int total_c = (n_routes - shared_last) * kch0 + shared_last * (p.Fs >> 3);
        constexpr int SB = 8;
        for (int q0 = threadIdx.x; q0 < total_c; q0 += (int)blockDim.x * SB) {
          uint4 v[SB];
          int dst[SB];
#pragma unroll
          for (int j = 0; j < SB; ++j) {
            const int q = q0 + (int)blockDim.x * j;
            dst[j] = -1;
            if (q < total_c) {
              const int i = min(q / kch0, n_routes - 1), c = q - i * kch0;
              v[j] = *reinterpret_cast<const uint4*>(p.act + ((size_t)t * (p.topk + 1) + s_slot[i]) * p.F + c * 8);
              dst[j] = i * p.F + c * 8;
            }
          }
#pragma unroll
          for (int j = 0; j < SB; ++j)
            if (dst[j] >= 0) *reinterpret_cast<uint4*>(as + dst[j]) = bf16x8_to_scaled_f16(v[j]);
        }
      }
      __syncthreads();
      float total[R];
#pragma unroll
      for (int r = 0; r < R; ++r) total[r] = 0.f;
      constexpr int MAXC = 4;   // 16-byte chunks (16 weights) per lane and route held in registers (K <= 2048)
      if ((p.F >> 4) <= 32 * MAXC) {
        // one route at a time, as in the bf16 kernel: base pointers, score and activation row are loop invariants
        for (int i = 0; i < n_routes; ++i) {
          const int k = s_k[i], kch = k >> 4, nbk = (k + QBLOCK - 1) / QBLOCK;
          const uint8_t* wb = s_w[i] + (size_t)n0 * k;
          const float* sb = s_sc[i] + (size_t)n0 * nbk;
          uint4 wv[MAXC][R];
          float sv[MAXC][R];
#pragma unroll
          for (int u = 0; u < MAXC; ++u) {
            const int c = lane + 32 * u;
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const bool in = c < kch && n0 + r < p.D;
              wv[u][r] = in ? ld_stream16(wb + (size_t)r * k + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
              sv[u][r] = in ? __ldg(sb + (size_t)r * nbk + (c >> 3)) : 0.f;
            }
          }
          const float g = s_g[i];
          const bf16* arow_s = as + (size_t)i * p.F;
          float acc[R];
#pragma unroll
          for (int r = 0; r < R; ++r) acc[r] = 0.f;
#pragma unroll
          for (int u = 0; u < MAXC; ++u) {
            const int c = lane + 32 * u;
            if (c < kch) {
              __half2 xv[8];
              const __half2* xa = reinterpret_cast<const __half2*>(arow_s) + c * 8;
              *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(xa);
              *reinterpret_cast<uint4*>(xv + 4) = *reinterpret_cast<const uint4*>(xa + 4);
#pragma unroll
              for (int r = 0; r < R; ++r) acc[r] = fmaf(sv[u][r], dot16_e4m3_f16(wv[u][r], xv), acc[r]);
            }
          }
#pragma unroll
          for (int r = 0; r < R; ++r) total[r] = fmaf(g * (1.f / kXScale), acc[r], total[r]);
        }
      } else {
      const int chunks = s_cbeg[n_routes];
        const int cpr = p.F >> 4;
        const int n_exp_chunks = (n_routes > 0 && s_slot[n_routes - 1] == p.topk) ? s_cbeg[n_routes - 1] : chunks;
        constexpr int U = 16 / R;
        for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
          uint4 wv[U][R];
          float sv[U][R];
          int route[U], cc[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int c = c0 + u * 32;
            const int i = c < n_exp_chunks ? c / cpr : n_routes - 1;
            route[u] = i;
            cc[u] = c < n_exp_chunks ? c - i * cpr : c - n_exp_chunks;
            if (c < chunks) {
              const int k = s_k[i], nbk = (k + QBLOCK - 1) / QBLOCK;
              const uint8_t* wb = s_w[i] + (size_t)n0 * k + (size_t)cc[u] * 16;
              const float* sb = s_sc[i] + (size_t)n0 * nbk + (cc[u] >> 3);
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const bool in = n0 + r < p.D;
                wv[u][r] = in ? ld_stream16(wb + (size_t)r * k) : make_uint4(0, 0, 0, 0);
                sv[u][r] = in ? __ldg(sb + (size_t)r * nbk) : 0.f;
              }
            } else {
#pragma unroll
              for (int r = 0; r < R; ++r) { wv[u][r] = make_uint4(0, 0, 0, 0); sv[u][r] = 0.f; }
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (c0 + u * 32 < chunks) {
              __half2 xv[8];
              const __half2* xa = reinterpret_cast<const __half2*>(as + (size_t)route[u] * p.F) + cc[u] * 8;
              *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(xa);
              *reinterpret_cast<uint4*>(xv + 4) = *reinterpret_cast<const uint4*>(xa + 4);
              const float g = s_g[route[u]] * (1.f / kXScale);
#pragma unroll
              for (int r = 0; r < R; ++r) total[r] = fmaf(g * sv[u][r], dot16_e4m3_f16(wv[u][r], xv), total[r]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = warp_sum(total[r]);
        if (lane == 0) slab[t * RPC + warp * R + r] = v;
      }
    }
  }
  __syncthreads();
  oneshot_allreduce_slab<T, RPC>(slab, p.fv, p.seq, p.done, nbase, p.T, p.D, p.residual, p.ldr, p.y, p.ldy, nullptr, &timed_out);
}

template <int T, int R>
int launch_down8(const Down8Params& p, cudaStream_t s) {
  const size_t smem = (size_t)(p.topk + 1) * p.F * sizeof(bf16);
  auto k = moe_down_fp8_allreduce_kernel<T, R>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid((p.D + 8 * R - 1) / (8 * R));
  return launch_chain(k, grid, dim3(256), smem, s, p);
}
template <int T>
int dispatch_down8(const Down8Params& p, cudaStream_t s) {
  if ((p.D + 7) / 8 <= 296) return launch_down8<T, 1>(p, s);
  if ((p.D + 15) / 16 <= 296) return launch_down8<T, 2>(p, s);
  if ((p.D + 31) / 32 <= 296) return launch_down8<T, 4>(p, s);
  return -2;
}

}  // namespace

// w: bf16 [rows, K] (row stride ldw); q: u8 [rows, K]; scales: f32 [rows, ceil(K / 128)]
extern "C" int ifab_quantize_fp8_block(const void* w, long ldw, long rows, int K, void* q, float* scales, void* stream) {
  if (rows < 1 || K < 1) return -1;
  const long items = rows * ((K + QBLOCK - 1) / QBLOCK);
  quantize_fp8_block_kernel<<<(unsigned)((items + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)w, ldw, rows, K, (uint8_t*)q, scales);
  return (int)cudaGetLastError();
}

// q: u8 [rows, K], scales: f32 [rows, ceil(K / 128)] -> out: bf16 [rows, K] (contiguous); K % 16 == 0
extern "C" int ifab_dequantize_fp8_block(const void* q, const float* scales, long rows, int K, void* out, void* stream) {
  if (rows < 1 || K < 16 || K % 16) return -1;
  const long items = rows * (K / 16);
  const unsigned blocks = (unsigned)std::min<long>((items + 255) / 256, 148L * 16);
  return launch_chain(dequantize_fp8_block_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const uint8_t*)q, scales, rows, K, (bf16*)out);
}

extern "C" int ifab_moe_gate_up_decode_fp8(const void* x, long ldx, const void* norm_w, float eps, const int32_t* ids, int T, int D, int F,
                                           int topk, int e0, int e_local, const void* w_gu, const float* s_gu, const void* w_shared_gu,
                                           const float* s_shared_gu, int Fs, void* act, void* stream) {
  if (D % 16 != 0 || F % 16 != 0 || Fs % 16 != 0 || Fs > F) return -1;
  GateUp8Params p{(const bf16*)x, ldx, (const bf16*)norm_w, eps, ids, T, D, F, topk, e0, e_local,
                  (const uint8_t*)w_gu, s_gu, (const uint8_t*)w_shared_gu, s_shared_gu, Fs, (bf16*)act};
  dim3 grid((F + 15) / 16, T * topk + T);
  const size_t smem = (size_t)D * sizeof(bf16);
  if (int rc = opt_in_smem(moe_gate_up_fp8_kernel, smem)) return rc;
  return launch_chain(moe_gate_up_fp8_kernel, grid, dim3(256), smem, (cudaStream_t)stream, p);
}

extern "C" int ifab_moe_down_allreduce_decode_fp8(const void* act, const int32_t* ids, const float* wts, int T, int D, int F, int topk,
                                                  int e0, int e_local, const void* w_down, const float* s_down, const void* w_shared_down,
                                                  const float* s_shared_down, int Fs, const void* residual, long ldr, void* y, long ldy,
                                                  const IfabFabric* fab, void* stream) {
  if (T < 1 || T > 8 || F % 16 != 0 || Fs % 16 != 0 || topk > MAX_TOPK8 || Fs > F) return -1;
  Down8Params p;
  p.act = (const bf16*)act; p.ids = ids; p.wts = wts;
  p.T = T; p.D = D; p.F = F; p.topk = topk; p.e0 = e0; p.e_local = e_local;
  p.w_down = (const uint8_t*)w_down; p.s_down = s_down; p.w_sdown = (const uint8_t*)w_shared_down; p.s_sdown = s_shared_down; p.Fs = Fs;
  p.residual = (const bf16*)residual; p.ldr = ldr; p.y = (bf16*)y; p.ldy = ldy;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  p.seq = fab->seq; p.done = fab->done;
  if ((size_t)fab->world * T * D * sizeof(uint64_t) > fab->ll_half_bytes) return -3;
  if ((size_t)fab->world * 296 > fab->flag_half_words) return -4;
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return dispatch_down8<1>(p, s);
  if (T <= 2) return dispatch_down8<2>(p, s);
  if (T <= 4) return dispatch_down8<4>(p, s);
  return dispatch_down8<8>(p, s);
}
