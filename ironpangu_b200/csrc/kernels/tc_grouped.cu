// Grouped expert GEMM on tcgen05 for MoE prefill: rows of a permuted activation matrix are grouped by expert and
// every 128-row tile multiplies with the weights of ITS expert.
//
//   A        [rows, K]      activations sorted by expert (moe_dispatch + moe_gather of moe_prefill.cu)
//   B        [E, N, K]      one [N, K] weight matrix per local expert (3-D tensor map, expert = batch coordinate)
//   tiles    device table   {expert, first row, valid rows, 0} per 128-row tile, written by the dispatch kernel;
//            num_tiles      device scalar. The host does not know how many tokens each expert received, so the grid
//                           covers the worst case and CTAs beyond num_tiles leave at once - no host round trip.
// Modes:
//   plain    C[row, n] = A[row, :] . B[e][n, :]                                    (down projection)
//   swiglu   B holds gate rows [0, F) and up rows [F, 2F); one accumulator of 256 columns receives 128 gate and the
//            128 matching up columns (two TMA boxes per stage), the epilogue stores silu(gate) * up -> C[row, F]
// Rows of a tile that belong to the next expert (the tile is only partly valid) are computed and thrown away.
// Reference counterparts: expert_gmm + expert_act_quantize (native/src/token_executor.h:1054-1167).
#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

struct GroupedParams {
  const int4* tiles;
  const int32_t* num_tiles;
  bf16* c; long ldc;
  int N, K, F;          // F: columns of the swiglu output (N = 2F); unused in plain mode
  uint32_t* status;
  uint32_t spin_limit;
};

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(192) tc_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                         const __grid_constant__ CUtensorMap tmap_b, GroupedParams p) {
  extern __shared__ unsigned char smem_raw[];
  grid_dep_launch();
  grid_dep_wait();
  if ((int)blockIdx.y >= *p.num_tiles) return;
  const int4 tile = p.tiles[blockIdx.y];          // x expert, y first row, z valid rows
  Pipe<BN> pipe;
  pipe.setup(smem_raw, &tmap_a, &tmap_b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int NOUT = SWIGLU ? BN / 2 : BN;      // output columns per CTA
  const int n0 = blockIdx.x * NOUT;
  if (warp == 0 && lane == 0) {
    if (SWIGLU) pipe.produce(&tmap_a, &tmap_b, num_kb, tile.y, n0, tile.x, p.spin_limit, p.status, p.F + n0);
    else pipe.produce(&tmap_a, &tmap_b, num_kb, tile.y, n0, tile.x, p.spin_limit, p.status);
  } else if (warp == 1 && lane == 0) {
    pipe.mma(num_kb, p.spin_limit, p.status);
  } else if (warp >= 2) {
    if (pipe.wait_accumulator(p.spin_limit, p.status)) {
      const int q = warp & 3;
      const int r = q * 32 + lane;
      const bool live = r < tile.z;
      bf16* out = p.c + (long)(tile.y + r) * p.ldc;
      const int ncols = SWIGLU ? p.F : p.N;
      const uint32_t tm = pipe.tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < NOUT; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tm + (uint32_t)c0, v);
        if (SWIGLU) {
          float u[32];
          tmem_ld_32x32(tm + (uint32_t)(NOUT + c0), u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = bf16_round(v[i]);
            v[i] = g / (1.f + __expf(-g)) * bf16_round(u[i]);
          }
        } else {
          tmem_ld_wait();
        }
        const int col = n0 + c0;
        if (live && col < ncols) {
          const int nvalid = min(32, ncols - col);
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(out + col) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(out + col)[i] = pack8(v + 8 * i);
          } else {
            for (int i = 0; i < nvalid; ++i) out[col + i] = __float2bfloat16_rn(v[i]);
          }
        }
      }
    }
  }
  pipe.teardown();
}

template <int BN, bool SWIGLU>
int launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, const GroupedParams& p, int max_tiles, cudaStream_t s) {
  auto k = tc_grouped_kernel<BN, SWIGLU>;
  if (int rc = opt_in_smem(k, Cfg<BN>::SMEM)) return rc;
  constexpr int NOUT = SWIGLU ? BN / 2 : BN;
  const int ncols = SWIGLU ? p.F : p.N;
  dim3 grid((ncols + NOUT - 1) / NOUT, max_tiles);
  return launch_chain(k, grid, dim3(192), (size_t)Cfg<BN>::SMEM, s, ta, tb, p);
}

}  // namespace

// mode 0: C[rows, N] = A . B[e]^T;  mode 1: N = 2F, C[rows, F] = silu(A . gate[e]^T) * (A . up[e]^T).
// `tiles` holds max_tiles int4 entries of which the first *num_tiles are valid (both in device memory).
extern "C" int ifab_grouped_gemm_bf16(const void* a, long lda, int rows_max, const void* b, int experts, int N, int K,
                                      const int32_t* tiles, const int32_t* num_tiles, int max_tiles, void* c, long ldc, int mode,
                                      uint32_t* status, void* stream) {
  if (rows_max < 1 || experts < 1 || N < 8 || K < 8 || K % 8 || lda % 8 || ldc % 8 || max_tiles < 1 || max_tiles > 65535) return -1;
  if (mode == 1 && (N % 16)) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)rows_max, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  GroupedParams p{reinterpret_cast<const int4*>(tiles), num_tiles, (bf16*)c, ldc, N, K, N / 2, status, 4000000u};
  cudaStream_t s = (cudaStream_t)stream;
  if (mode == 1) {
    if (int rc = make_tmap_bf16_3d(&tb, b, (uint64_t)experts, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint64_t)N * K, 128)) return rc;
    return launch_grouped<256, true>(ta, tb, p, max_tiles, s);
  }
  if (N > 128) {
    if (int rc = make_tmap_bf16_3d(&tb, b, (uint64_t)experts, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint64_t)N * K, 256)) return rc;
    return launch_grouped<256, false>(ta, tb, p, max_tiles, s);
  }
  if (int rc = make_tmap_bf16_3d(&tb, b, (uint64_t)experts, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint64_t)N * K, 128)) return rc;
  return launch_grouped<128, false>(ta, tb, p, max_tiles, s);
}
