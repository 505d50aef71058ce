// Skinny-M (decode) matrix-vector core shared by the decode kernels.
//
// Decode-time linears have M = 1..8 tokens and are bound by the HBM stream of the weight matrix,
// so the design goal is bytes in flight, not tensor-core issue: every warp owns R weight rows,
// every lane issues 16-byte streaming loads that bypass L1, and 16 loads are outstanding per lane
// before the first FMA. Activations sit in shared memory as bf16 (optionally RMS-normalised while
// they are staged) and are re-read conflict-free by consecutive lanes.
//
// Weights never depend on the previous kernel, activations do. Every kernel is launched with
// programmatic dependent launch: it first releases its own dependents, issues the first batch of
// weight loads into registers (`prefetch_rows`), and only then waits for the producer of its
// activations (`grid_dep_wait`). The weight stream of kernel n+1 therefore overlaps the tail,
// drain and launch latency of kernel n.
#pragma once
#include "common.cuh"

namespace ifab {

// number of 16-byte chunks a lane keeps in flight per batch (DEPTH), split over the R rows of its warp. The
// operator-per-launch kernels use 16; the persistent decode-step kernel, which lives on 128 registers per thread
// with 16 resident warps per SM, uses 8.
template <int R, int DEPTH = 16>
struct Pf {
  static constexpr int U = DEPTH / R;
};

template <int R, int DEPTH = 16>
struct RowBatch {
  uint4 v[Pf<R, DEPTH>::U][R];
};

// issue the loads of the first batch (chunks lane, lane+32, ...) of R rows; rows may be nullptr
template <int R, int DEPTH = 16>
__device__ __forceinline__ void prefetch_rows(const bf16* const (&wrow)[R], int K, RowBatch<R, DEPTH>& pf) {
  const int lane = threadIdx.x & 31;
  const int chunks = K >> 3;
#pragma unroll
  for (int u = 0; u < Pf<R, DEPTH>::U; ++u) {
    const int c = lane + u * 32;
#pragma unroll
    for (int r = 0; r < R; ++r)
      pf.v[u][r] = (c < chunks && wrow[r] != nullptr) ? ld_stream16(wrow[r] + c * 8) : make_uint4(0, 0, 0, 0);
  }
}

// Stage T rows of x (bf16, K columns, row stride ldx) into shared memory. When norm_w != nullptr the
// rows are RMS-normalised on the way: y = bf16(x * rsqrt(mean(x^2) + eps) * (w or 1+w)).
// All threads of the block participate; ends with __syncthreads().
template <int T>
__device__ __forceinline__ void stage_x(bf16* xs, const bf16* __restrict__ x, long ldx, int t0, int t_total,
                                        int K, const bf16* __restrict__ norm_w, float eps, bool zero_centered,
                                        float* red /* >= T*33 floats */) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int chunks = K >> 3;
  for (int t = 0; t < T; ++t) {
    const bool live = (t0 + t) < t_total;
    const bf16* xr = x + (long)(t0 + t) * ldx;
    for (int c = tid; c < chunks; c += nthr) {
      uint4 v = live ? *reinterpret_cast<const uint4*>(xr + c * 8) : make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(xs + t * K + c * 8) = v;
    }
  }
  __syncthreads();
  if (norm_w == nullptr) return;
  const int warp = tid >> 5, lane = tid & 31, nwarp = nthr >> 5;
  for (int t = 0; t < T; ++t) {
    float ss = 0.f;
    for (int c = tid; c < chunks; c += nthr) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(xs + t * K + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    if (lane == 0) red[t * 33 + warp] = ss;
  }
  __syncthreads();
  if (tid < T) {
    float s = 0.f;
    for (int w = 0; w < nwarp; ++w) s += red[tid * 33 + w];
    red[tid * 33 + 32] = rsqrtf(s / (float)K + eps);
  }
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const float inv = red[t * 33 + 32];
    for (int c = tid; c < chunks; c += nthr) {
      float f[8], g[8];
      unpack8(*reinterpret_cast<const uint4*>(xs + t * K + c * 8), f);
      unpack8(*reinterpret_cast<const uint4*>(norm_w + c * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * (zero_centered ? 1.f + g[i] : g[i]);
      *reinterpret_cast<uint4*>(xs + t * K + c * 8) = pack8(f);
    }
  }
  __syncthreads();
}

// acc[r][t] += dot(w_row[r][0..K), xs[t][0..K)) over this lane's share of K. `pf` holds the first
// batch (already loaded by prefetch_rows); later batches are loaded here. Rows whose pointer is
// nullptr are skipped. Caller reduces across the warp afterwards.
template <int T, int R, int DEPTH = 16>
__device__ __forceinline__ void warp_rows_dot(const bf16* const (&wrow)[R], const bf16* xs, int K, float (&acc)[R][T],
                                              RowBatch<R, DEPTH>& pf) {
  const int lane = threadIdx.x & 31;
  const int chunks = K >> 3;
  constexpr int U = Pf<R, DEPTH>::U;
  for (int c0 = lane; c0 < chunks; c0 += 32 * U) {
    if (c0 != lane) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u * 32;
#pragma unroll
        for (int r = 0; r < R; ++r)
          pf.v[u][r] = (c < chunks && wrow[r] != nullptr) ? ld_stream16(wrow[r] + c * 8) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * 32;
      if (c < chunks) {
        float xf[T][8];
#pragma unroll
        for (int t = 0; t < T; ++t) unpack8(*reinterpret_cast<const uint4*>(xs + t * K + c * 8), xf[t]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float wf[8];
          unpack8(pf.v[u][r], wf);
#pragma unroll
          for (int t = 0; t < T; ++t) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[r][t] = fmaf(wf[i], xf[t][i], acc[r][t]);
          }
        }
      }
    }
  }
}

// convenience: prefetch + dot in one go (no overlap with a prologue)
template <int T, int R, int DEPTH = 16>
__device__ __forceinline__ void warp_rows_dot(const bf16* const (&wrow)[R], const bf16* xs, int K, float (&acc)[R][T]) {
  RowBatch<R, DEPTH> pf;
  prefetch_rows<R, DEPTH>(wrow, K, pf);
  warp_rows_dot<T, R, DEPTH>(wrow, xs, K, acc, pf);
}

template <int T, int R>
__device__ __forceinline__ void warp_reduce_acc(float (&acc)[R][T]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < T; ++t) acc[r][t] = warp_sum(acc[r][t]);
}

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

}  // namespace ifab
