// Decode-time (M = 1..8 tokens per tile) linear layers for sm_100a.
//
//   gemv_kernel            y = act(norm(x) W^T) (+ residual)         column-parallel / replicated linears
//   gemv_allreduce_kernel  y = sum_ranks(x_r W_r^T) + residual       row-parallel linear fused with a
//                          one-shot all-reduce over NVLink peer memory (push partial tiles to every
//                          peer, bounded flag wait, rank-ordered f32 sum) - no separate collective launch
//
// Counterparts in the reference: `linear` + `allreduce` instructions executed by aclnnMatmul and
// HcclAllReduce (native/src/token_executor.h:374-404); here both are one kernel.
#include "gemv.cuh"
#include "oneshot_ar.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

struct GemvParams {
  const bf16* x; long ldx;
  const bf16* w;            // [rows, K], K contiguous; rows = N (plain) or 2N (swiglu: gate rows then up rows)
  const bf16* norm_w; float eps; int zero_centered;
  const bf16* residual; long ldr;
  void* y; long ldy; int out_f32;
  int T, N, K, mode;
};

template <int T, int R>
__global__ void __launch_bounds__(256) gemv_kernel(GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[T * 33];
  grid_dep_launch();
  const int t0 = blockIdx.y * T;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * 8 + warp) * R;
  if (p.mode == 0) {
    const bf16* rows[R];
#pragma unroll
    for (int r = 0; r < R; ++r) rows[r] = (n0 + r < p.N) ? p.w + (long)(n0 + r) * p.K : nullptr;
    RowBatch<R> pf;
    prefetch_rows<R>(rows, p.K, pf);
    grid_dep_wait();
    stage_x<T>(xs, p.x, p.ldx, t0, p.T, p.K, p.norm_w, p.eps, p.zero_centered != 0, red);
    if (n0 >= p.N) return;
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    warp_rows_dot<T, R>(rows, xs, p.K, acc, pf);
    warp_reduce_acc<T, R>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (n0 + r >= p.N) continue;
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (t0 + t >= p.T) continue;
          float v = acc[r][t];
          if (p.residual) v = bf16_round(v) + __bfloat162float(p.residual[(long)(t0 + t) * p.ldr + n0 + r]);
          if (p.out_f32) reinterpret_cast<float*>(p.y)[(long)(t0 + t) * p.ldy + n0 + r] = v;
          else reinterpret_cast<bf16*>(p.y)[(long)(t0 + t) * p.ldy + n0 + r] = __float2bfloat16_rn(v);
        }
      }
    }
  } else {
    // swiglu: output feature j uses gate row j and up row N + j
    const bf16* rows[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool ok = n0 + r < p.N;
      rows[r] = ok ? p.w + (long)(n0 + r) * p.K : nullptr;
      rows[R + r] = ok ? p.w + (long)(p.N + n0 + r) * p.K : nullptr;
    }
    RowBatch<2 * R> pf;
    prefetch_rows<2 * R>(rows, p.K, pf);
    grid_dep_wait();
    stage_x<T>(xs, p.x, p.ldx, t0, p.T, p.K, p.norm_w, p.eps, p.zero_centered != 0, red);
    if (n0 >= p.N) return;
    float acc[2 * R][T];
#pragma unroll
    for (int r = 0; r < 2 * R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    warp_rows_dot<T, 2 * R>(rows, xs, p.K, acc, pf);
    warp_reduce_acc<T, 2 * R>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (n0 + r >= p.N) continue;
#pragma unroll
        for (int t = 0; t < T; ++t) {
          if (t0 + t >= p.T) continue;
          const float g = bf16_round(acc[r][t]), u = bf16_round(acc[R + r][t]);
          reinterpret_cast<bf16*>(p.y)[(long)(t0 + t) * p.ldy + n0 + r] = __float2bfloat16_rn(silu(g) * u);
        }
      }
    }
  }
}

template <int T, int R>
int launch_gemv(const GemvParams& p, cudaStream_t s) {
  const size_t smem = (size_t)T * p.K * sizeof(bf16);
  auto k = gemv_kernel<T, R>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid((p.N + 8 * R - 1) / (8 * R), (p.T + T - 1) / T);
  return launch_chain(k, grid, dim3(256), smem, s, p);
}

template <int T>
int dispatch_rows(const GemvParams& p, cudaStream_t s) {
  // pick rows-per-warp so that small N still spreads over the 148 SMs
  const int n = p.N * (p.mode ? 2 : 1);
  if (p.mode) {
    if (n >= 148 * 8 * 4 * 2) return launch_gemv<T, 2>(p, s);
    return launch_gemv<T, 1>(p, s);
  }
  if (n >= 148 * 8 * 4 * 2) return launch_gemv<T, 4>(p, s);
  if (n >= 148 * 8 * 2 * 2) return launch_gemv<T, 2>(p, s);
  return launch_gemv<T, 1>(p, s);
}

// ----------------------------------------------------------------------------------------------
// Row-parallel linear + one-shot all-reduce (protocol in oneshot_ar.cuh).
// Every CTA owns a slab of 8*R output columns for all T tokens; only same-index CTAs of the ranks
// synchronise, so the transfer of early slabs overlaps the math of late ones.
// ----------------------------------------------------------------------------------------------
struct ArParams {
  GemvParams g;
  FabricView fv;
  uint64_t* seq;         // local call counter (read by all CTAs, advanced by the last one)
  uint32_t* done;        // local ticket counter
  float* y_f32;          // optional f32 copy of the reduced output [T, N]
};

template <int T, int R>
__global__ void __launch_bounds__(256) gemv_allreduce_kernel(ArParams a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const GemvParams& p = a.g;
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  __shared__ float red[T * 33];
  __shared__ float slab[T * 8 * R];
  __shared__ int timed_out;
  grid_dep_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int RPC = 8 * R;
  const int nbase = blockIdx.x * RPC;
  const int n0 = nbase + warp * R;
  const bf16* rows[R];
#pragma unroll
  for (int r = 0; r < R; ++r) rows[r] = (n0 + r < p.N) ? p.w + (long)(n0 + r) * p.K : nullptr;
  RowBatch<R> pf;
  prefetch_rows<R>(rows, p.K, pf);
  grid_dep_wait();
  if (threadIdx.x == 0) timed_out = 0;
  stage_x<T>(xs, p.x, p.ldx, 0, p.T, p.K, p.norm_w, p.eps, p.zero_centered != 0, red);
  {
    float acc[R][T];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    warp_rows_dot<T, R>(rows, xs, p.K, acc, pf);
    warp_reduce_acc<T, R>(acc);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int t = 0; t < T; ++t) slab[t * RPC + warp * R + r] = acc[r][t];
    }
  }
  __syncthreads();
  oneshot_allreduce_slab<T, RPC>(slab, a.fv, a.seq, a.done, nbase, p.T, p.N, p.residual, p.ldr,
                                 reinterpret_cast<bf16*>(p.y), p.ldy, a.y_f32, &timed_out);
}

template <int T, int R>
int launch_ar(const ArParams& a, cudaStream_t s) {
  const size_t smem = (size_t)T * a.g.K * sizeof(bf16);
  auto k = gemv_allreduce_kernel<T, R>;
  if (int rc = opt_in_smem(k, smem)) return rc;
  dim3 grid((a.g.N + 8 * R - 1) / (8 * R));
  return launch_chain(k, grid, dim3(256), smem, s, a);
}

template <int T>
int dispatch_ar(const ArParams& a, cudaStream_t s) {
  // keep the grid <= 296 CTAs (two per SM) so every CTA of every rank is co-resident: CTAs with the
  // same index wait on one another across GPUs.
  const int n = a.g.N;
  if ((n + 7) / 8 <= 296) return launch_ar<T, 1>(a, s);
  if ((n + 15) / 16 <= 296) return launch_ar<T, 2>(a, s);
  if ((n + 31) / 32 <= 296) return launch_ar<T, 4>(a, s);
  return -2;
}

}  // namespace

extern "C" int ifab_gemv_bf16(const void* x, long ldx, const void* w, const void* norm_w, float eps, int zero_centered,
                              const void* residual, long ldr, void* y, long ldy, int out_f32, int T, int N, int K,
                              int mode, void* stream) {
  if (K % 8 != 0 || ldx % 8 != 0) return -1;
  GemvParams p{(const bf16*)x, ldx, (const bf16*)w, (const bf16*)norm_w, eps, zero_centered,
               (const bf16*)residual, ldr, y, ldy, out_f32, T, N, K, mode};
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return dispatch_rows<1>(p, s);
  if (T <= 2) return dispatch_rows<2>(p, s);
  if (T <= 4) return dispatch_rows<4>(p, s);
  return dispatch_rows<8>(p, s);
}

extern "C" int ifab_gemv_allreduce_bf16(const void* x, long ldx, const void* w, const void* residual, long ldr,
                                        void* y, long ldy, void* y_f32, int T, int N, int K,
                                        const IfabFabric* fab, void* stream) {
  if (K % 8 != 0 || ldx % 8 != 0 || T > 8 || T < 1) return -1;
  ArParams a;
  a.g = GemvParams{(const bf16*)x, ldx, (const bf16*)w, nullptr, 0.f, 0, (const bf16*)residual, ldr, y, ldy, 0, T, N, K, 0};
  if (int rc = fabric_view(fab, &a.fv)) return rc;
  a.seq = fab->seq;
  a.done = fab->done;
  a.y_f32 = (float*)y_f32;
  if ((size_t)fab->world * T * N * sizeof(uint64_t) > fab->ll_half_bytes) return -3;
  if ((size_t)fab->world * 296 > fab->flag_half_words) return -4;
  cudaStream_t s = (cudaStream_t)stream;
  if (T <= 1) return dispatch_ar<1>(a, s);
  if (T <= 2) return dispatch_ar<2>(a, s);
  if (T <= 4) return dispatch_ar<4>(a, s);
  return dispatch_ar<8>(a, s);
}
