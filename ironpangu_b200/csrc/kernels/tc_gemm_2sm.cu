// bf16 GEMM on the 5th-generation tensor cores, two-SM form:  C[M,N] = A[M,K] * B[N,K]^T (+ residual), f32 accumulate.
//
// A cluster of two CTAs (a pair of SMs) owns one 256 x 256 output tile. Each CTA streams ITS 128 rows of A and ITS 128 rows
// of B (half of the tile's N) into its own shared memory - 32 KB per 64-wide K block instead of the 48 KB a lone CTA needs for
// a 128 x 256 tile - and the leader CTA issues tcgen05.mma.cta_group::2 (256 x 256 x 16 per instruction), which reads A and B
// from both CTAs' shared memory and accumulates into both CTAs' tensor memory (each CTA keeps its 128 rows x 256 columns).
//
//   warp 0 (both CTAs)   TMA producer: cp.async.bulk.tensor...cta_group::2 into this CTA's stage ring; the bytes of both CTAs
//                        complete on the LEADER's full barrier (its shared::cluster address, by mapa)
//   warp 1 (both CTAs)   allocates tensor memory (cta_group::2, collectively); in the leader one elected lane issues the MMAs and
//                        releases a stage in BOTH CTAs with tcgen05.commit...multicast::cluster
//   warps 2-5 (both)     epilogue of this CTA's 128 rows: tcgen05.ld, convert, residual, store
// Six stages of 32 KB. No TMA load is multicast: every CTA fetches its own tiles. Every mbarrier wait is bounded; a wait that
// runs out raises the CTA's abort flag and a status bit, and both CTAs still meet at the closing cluster barrier.
// Shapes: N % 32 == 0 (rows are stored 32 columns at a time), K % 8 == 0; M, N and K tails by TMA zero fill and masked stores.
// `ifab_gemm_bf16` uses these kernels from 256 rows and 256 columns up; below that a pair's 256 x 256 tile is mostly padding.
#include <algorithm>

#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

constexpr int TN = 256;                         // tile N (both CTAs together), also the accumulator's TMEM columns
constexpr int HALF_N = TN / 2;                  // B rows a CTA supplies
constexpr int STAGES2 = 6;
constexpr int A2_BYTES = BM * BK * 2, B2_BYTES = HALF_N * BK * 2, STAGE2_BYTES = A2_BYTES + B2_BYTES;
constexpr int SMEM2 = STAGES2 * STAGE2_BYTES + 1024 + 256;

struct Gemm2Params {
  void* c; long ldc; int out_f32;
  const bf16* residual; long ldr;
  int M, N, K;
  uint32_t* status;
  uint32_t spin_limit;
  int swiglu_f;   // > 0 (persistent kernel only): B = [gate rows 0..F) | up rows F..2F), C[M, F] = silu(A gate^T) * (A up^T)
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// this CTA's tile -> this CTA's shared memory; completion bytes go to the barrier at `bar_cluster_addr` (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

__device__ __forceinline__ void store_row32_2(const Gemm2Params& p, int row, int col, float* v) {
  if (row >= p.M || col >= (p.swiglu_f > 0 ? p.swiglu_f : p.N)) return;
  if (p.residual) {
    const bf16* r = p.residual + (long)row * p.ldr + col;
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + __bfloat162float(r[i]);
  }
  if (p.out_f32) {
    float* out = reinterpret_cast<float*>(p.c) + (long)row * p.ldc + col;
    if ((reinterpret_cast<uintptr_t>(out) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(out)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      for (int i = 0; i < 32; ++i) out[i] = v[i];
    }
  } else {
    bf16* out = reinterpret_cast<bf16*>(p.c) + (long)row * p.ldc + col;
    if ((reinterpret_cast<uintptr_t>(out) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(out)[i] = pack8(v + 8 * i);
    } else {
      for (int i = 0; i < 32; ++i) out[i] = __float2bfloat16_rn(v[i]);
    }
  }
}

// grid (2 * M / 256, N / 256), clusters of 2 along x; 192 threads
__global__ void __launch_bounds__(192) tc_gemm_2sm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                          Gemm2Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE2_BYTES);
  uint64_t* empty = full + STAGES2;
  uint64_t* acc_full = empty + STAGES2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int m0 = (int)(blockIdx.x >> 1) * 2 * BM + (int)rank * BM;
  const int n0 = (int)blockIdx.y * TN;
  const int num_kb = (p.K + BK - 1) / BK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, TN);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                            // the peer's barriers and tensor memory exist before anything is signalled or issued
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_launch();
  grid_dep_wait();
  if (warp == 0 && lane == 0) {
    // ---- producer (both CTAs) ----
    int issued = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % STAGES2;
      const uint32_t round = kb / STAGES2;
      if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, p.spin_limit)) { *abort_flag = 1; break; }
      if (*abort_flag) break;
      unsigned char* a_dst = smem + s * STAGE2_BYTES;
      if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE2_BYTES);        // this CTA's tiles and the peer's
      const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
      tma_load_2d_pair(a_dst, &tmap_a, bar, kb * BK, m0);
      tma_load_2d_pair(a_dst + A2_BYTES, &tmap_b, bar, kb * BK, n0 + (int)rank * HALF_N);
      issued = kb + 1;
    }
    if (*abort_flag && p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    (void)issued;
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer (leader only) ----
    constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, TN);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % STAGES2;
      if (!mbar_wait(&full[s], (kb / STAGES2) & 1, p.spin_limit) || *abort_flag) { ok = false; break; }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(smem + s * STAGE2_BYTES);
      const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + A2_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, kb > 0 || k > 0);
      umma_commit_pair(&empty[s]);               // frees the stage in both CTAs
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    umma_commit_pair(acc_full);                  // both CTAs' accumulators are complete (or abandoned)
  } else if (warp >= 2) {
    // ---- epilogue (both CTAs): this CTA's 128 rows ----
    const bool ready = mbar_wait(acc_full, 0, p.spin_limit);
    tc_fence_after();
    if (!ready) {
      *abort_flag = 1;
      if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    if (ready && !*abort_flag) {
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        store_row32_2(p, row, n0 + c0, v);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                            // nobody reads the peer's shared or tensor memory any more
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TN);
  }
}

// ---- persistent form -------------------------------------------------------------------------------------------------------
// One CTA pair per SM pair (at most 74 pairs) walks the 256 x 256 tiles round-robin. Tensor memory holds TWO accumulators
// (2 x 256 columns = all 512): while the epilogue warps of both CTAs drain tile j, the leader already issues the MMAs of tile
// j + 1 into the other half, and the producers keep the stage ring full across tile boundaries. An accumulator half goes back
// to the issuer when the eight epilogue warps of the pair (four per CTA) have arrived on the leader's acc_empty barrier.
// Tile order of the persistent walk: groups of RASTER_M tile rows, inside a group the row index runs fastest. The 74 pairs
// that work at the same time then share a few B tiles (each read by up to RASTER_M pairs back to back) and keep RASTER_M
// tile rows of A in L2, instead of sweeping all of B for every tile row (at 8192^3 B alone is 128 MB - more than L2).
constexpr int RASTER_M = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int* tm, int* tn) {
  const int per_group = RASTER_M * tiles_n;
  const int g = t / per_group, within = t - g * per_group;
  const int first = g * RASTER_M, rows = min(RASTER_M, tiles_m - first);
  *tm = first + within % rows;
  *tn = within / rows;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// grid (2 * pairs), clusters of 2; 192 threads
__global__ void __launch_bounds__(192) tc_gemm_2sm_persistent_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                                     Gemm2Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE2_BYTES);
  uint64_t* empty = full + STAGES2;
  uint64_t* acc_full = empty + STAGES2;          // [2], one arrival each (the leader's commit, multicast to both CTAs)
  uint64_t* acc_empty = acc_full + 2;            // [2], used in the leader only: eight arrivals each (epilogue warps of both CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = (int)(blockIdx.x >> 1), pairs = (int)(gridDim.x >> 1);
  // SwiGLU mode: a tile is 256 rows x 128 output columns; the leader CTA streams the 128 gate rows of B, its peer the 128
  // matching up rows, so the accumulator holds gate in columns 0..127 and up in 128..255
  const int F = p.swiglu_f;
  const int tiles_n = F > 0 ? (F + HALF_N - 1) / HALF_N : (p.N + TN - 1) / TN, tiles_m = (p.M + 2 * BM - 1) / (2 * BM), tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 2 * TN);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_launch();
  grid_dep_wait();
  if (warp == 0 && lane == 0) {
    // ---- producer (both CTAs): one ring across all tiles ----
    uint32_t it = 0;
    for (int t = pair; t < tiles && !*abort_flag; t += pairs) {
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, &tm, &tn);
      const int m0 = tm * 2 * BM + (int)rank * BM, n0 = F > 0 ? tn * HALF_N + (int)rank * F : tn * TN + (int)rank * HALF_N;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = (int)(it % STAGES2);
        const uint32_t round = it / STAGES2;
        if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, p.spin_limit)) { *abort_flag = 1; break; }
        if (*abort_flag) break;
        unsigned char* a_dst = smem + s * STAGE2_BYTES;
        if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE2_BYTES);
        const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
        tma_load_2d_pair(a_dst, &tmap_a, bar, kb * BK, m0);
        tma_load_2d_pair(a_dst + A2_BYTES, &tmap_b, bar, kb * BK, n0);
      }
    }
    if (*abort_flag && p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer (leader only) ----
    constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, TN);
    uint32_t it = 0;
    bool ok = true;
    int j = 0;
    for (int t = pair; t < tiles && ok; t += pairs, ++j) {
      const int b = j & 1;
      // the accumulator half must have been drained by the epilogue of tile j - 2
      if (j >= 2 && !mbar_wait(&acc_empty[b], ((j >> 1) - 1) & 1, p.spin_limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d = tmem_base + (uint32_t)(b * TN);
      for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
        const int s = (int)(it % STAGES2);
        if (!mbar_wait(&full[s], (it / STAGES2) & 1, p.spin_limit) || *abort_flag) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * STAGE2_BYTES);
        const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + A2_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, kb > 0 || k > 0);
        umma_commit_pair(&empty[s]);
      }
      umma_commit_pair(&acc_full[b]);
    }
    if (!ok) {
      *abort_flag = 1;
      if (p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
      // wake the epilogues of both CTAs for every tile they still expect, so that they run into their own bounded waits only once
      for (int b = 0; b < 2; ++b) umma_commit_pair(&acc_full[b]);
    }
  } else if (warp >= 2) {
    // ---- epilogue (both CTAs) ----
    const int q = warp & 3;
    int j = 0;
    for (int t = pair; t < tiles; t += pairs, ++j) {
      const int b = j & 1;
      const bool ready = mbar_wait(&acc_full[b], (j >> 1) & 1, p.spin_limit);
      tc_fence_after();
      if (!ready || *abort_flag) {
        *abort_flag = 1;
        if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
        break;
      }
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, &tm, &tn);
      const int m0 = tm * 2 * BM + (int)rank * BM, n0 = F > 0 ? tn * HALF_N : tn * TN;
      const int row = m0 + q * 32 + lane;
      const uint32_t tm_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * TN);
      if (F > 0) {
#pragma unroll 1
        for (int c0 = 0; c0 < HALF_N; c0 += 32) {
          float v[32], u[32];
          tmem_ld_32x32(tm_row + (uint32_t)c0, v);
          tmem_ld_32x32(tm_row + (uint32_t)(HALF_N + c0), u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = bf16_round(v[i]);
            v[i] = g / (1.f + __expf(-g)) * bf16_round(u[i]);
          }
          store_row32_2(p, row, n0 + c0, v);
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < TN; c0 += 32) {
          float v[32];
          tmem_ld_32x32(tm_row + (uint32_t)c0, v);
          tmem_ld_wait();
          store_row32_2(p, row, n0 + c0, v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[b]), 0));
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * TN);
  }
}

}  // namespace

// C[M,N] = A[M,K] * B[N,K]^T (+ residual) with CTA pairs on 256 x 256 tiles. N % 32 == 0, K % 8 == 0.
extern "C" int ifab_gemm_bf16_2sm(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32, const void* residual, long ldr,
                                  int M, int N, int K, uint32_t* status, void* stream) {
  if (M < 1 || N < 32 || N % 32 || K < 8 || K % 8 || lda % 8 || ldb % 8) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, HALF_N)) return rc;
  Gemm2Params p{c, ldc, out_f32, (const bf16*)residual, ldr, M, N, K, status, 4000000u, 0};
  if (int rc = opt_in_smem(tc_gemm_2sm_kernel, SMEM2)) return rc;
  dim3 grid(2 * ((M + 255) / 256), (N + 255) / 256);
  return launch_chain_cluster(tc_gemm_2sm_kernel, grid, dim3(192), 2, (size_t)SMEM2, (cudaStream_t)stream, ta, tb, p);
}

// The same with a persistent grid (one CTA pair per SM pair) and two accumulators in tensor memory.
extern "C" int ifab_gemm_bf16_2sm_persistent(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32, const void* residual,
                                             long ldr, int M, int N, int K, uint32_t* status, void* stream) {
  if (M < 1 || N < 32 || N % 32 || K < 8 || K % 8 || lda % 8 || ldb % 8) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, HALF_N)) return rc;
  Gemm2Params p{c, ldc, out_f32, (const bf16*)residual, ldr, M, N, K, status, 4000000u, 0};
  if (int rc = opt_in_smem(tc_gemm_2sm_persistent_kernel, SMEM2)) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = std::max(1, std::min(tiles, sms / 2));
  return launch_chain_cluster(tc_gemm_2sm_persistent_kernel, dim3(2 * pairs), dim3(192), 2, (size_t)SMEM2, (cudaStream_t)stream, ta, tb, p);
}

// C[M, F] = silu(A gate^T) * (A up^T) with B = [gate rows | up rows] ([2F, K]): the packed gate / up projection of a SwiGLU block in
// one persistent CTA-pair launch (gate and up of the same 128 output columns share an accumulator). F % 32 == 0, K % 8 == 0.
extern "C" int ifab_gemm_swiglu_bf16_2sm(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int M, int F, int K, uint32_t* status,
                                         void* stream) {
  if (M < 1 || F < 32 || F % 32 || K < 8 || K % 8 || lda % 8 || ldb % 8) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)2 * F, (uint64_t)K, (uint64_t)ldb, HALF_N)) return rc;
  Gemm2Params p{c, ldc, 0, nullptr, 0, M, 2 * F, K, status, 4000000u, F};
  if (int rc = opt_in_smem(tc_gemm_2sm_persistent_kernel, SMEM2)) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + 255) / 256) * ((F + HALF_N - 1) / HALF_N);
  const int pairs = std::max(1, std::min(tiles, sms / 2));
  return launch_chain_cluster(tc_gemm_2sm_persistent_kernel, dim3(2 * pairs), dim3(192), 2, (size_t)SMEM2, (cudaStream_t)stream, ta, tb, p);
}
