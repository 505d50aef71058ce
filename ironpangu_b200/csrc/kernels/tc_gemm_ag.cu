// Column-parallel bf16 GEMM fused with the all-gather of its activations:
//     C[M, N_local] = concat_ranks(A_r)[M, K] * B[N_local, K]^T,   A_r = rank r's [M / world, K] row shard
//
// The activations are sharded by rows (sequence parallel): rank r produced rows [r * Ml, (r + 1) * Ml) into a buffer in
// symmetric memory. There is no separate gather: the GEMM grid starts with the tiles of this rank's own shard (TMA from
// local memory). While the tensor cores work on a local tile, the four epilogue warps of that CTA - idle until the
// accumulator is complete - bring the same tile row of every remote shard over NVLink with plain peer loads (this CTA's
// slice of the K columns, exactly once per remote element) into a local staging matrix and count the tile row complete.
// The CTAs of the remote tiles, later in the grid, wait for that count and feed their main loop from the local copy with
// ordinary tiled TMA loads (no multicast, no TMA from peer memory). The transfer of the remote shards therefore hides
// under the tensor-core work on the local one.
//
// Forward progress: a remote-tile CTA spins (bounded) on a count that local-tile CTAs of the SAME grid bump. The local tiles
// have the lower block indices, and the hardware hands out CTAs of a grid in block-index order, so by the time a remote-tile
// CTA is resident every local-tile CTA is resident or done. CUDA does not document that order; if it ever changed, a grid
// larger than the device holds could fill the SMs with waiting CTAs - the waits would then run out, the status word would
// carry IFAB_STATUS_PEER_TIMEOUT and the output of those tiles would be missing, without a hang.
//
// Readiness: the shard of a rank is written by the kernel that precedes this one in that rank's stream. At kernel start
// CTA 0 publishes "my shard of call `epoch` is complete" to every peer (system fence + release store); a CTA whose rows
// live on rank s waits - bounded - for s's flag, then issues a cross-proxy fence before its first TMA load. The caller
// alternates two symmetric A buffers between consecutive calls (a rank reaches call n + 2 only after every peer entered
// call n + 1, i.e. finished reading call n).
// Reference: gather (HCCL AllGather) + linear(tp_columns) in the token program (native/src/token_executor.h:356-404).
#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

struct AgMaps {
  CUtensorMap a[IFAB_MAX_RANKS];
};

struct AgParams {
  const bf16* a_peer[IFAB_MAX_RANKS]; long lda;   // shards as mapped here
  bf16* staged; long lds;                          // local [M, K] staging matrix for remote tiles
  unsigned long long* tile_count;                  // local [M tiles]: grows by gridDim.x per call once a remote tile is complete
  bf16* c; long ldc;
  int M, N, K, rows_local, world, rank;
  uint64_t* flags[IFAB_MAX_RANKS];   // flags[r] = rank r's flag row (u64[8]); entry [s] = last call for which s's shard is complete
  uint64_t epoch;
  uint32_t* status;
  uint32_t spin_limit;
};

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// maps.a[r]: tensor map of rank r's shard (only [rank] is used for TMA); map_s: the staging matrix
template <int BN>
__global__ void __launch_bounds__(192) tc_gemm_ag_kernel(const __grid_constant__ AgMaps maps, const __grid_constant__ CUtensorMap map_s,
                                                         const __grid_constant__ CUtensorMap tmap_b, AgParams p) {
  extern __shared__ unsigned char smem_raw[];
  grid_dep_launch();
  grid_dep_wait();
  // this rank's shard is complete (previous kernel of the stream): tell everybody, once
  if (blockIdx.x == 0 && blockIdx.y == 0 && (int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
  }
  // own shard first: tile rows are rotated so that blockIdx.y = 0 is this rank's first tile
  const int tiles_m = gridDim.y;
  const int ty = (blockIdx.y + p.rank * (tiles_m / p.world)) % tiles_m;
  const int m0 = ty * BM, n0 = blockIdx.x * BN;
  const int src = min(m0 / p.rows_local, p.world - 1);
  const bool remote = src != p.rank;
  const CUtensorMap* ta = remote ? &map_s : &maps.a[p.rank];
  __shared__ int s_ready;
  Pipe<BN> pipe;
  pipe.setup(smem_raw, ta, &tmap_b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  if (warp == 0 && lane == 0) {
    bool ready = true;
    if (remote) {
      ready = false;
      const unsigned long long target = p.epoch * gridDim.x;
      for (uint32_t i = 0; i < p.spin_limit; ++i) {
        if (ld_acquire_gpu_u64(p.tile_count + ty) >= target) { ready = true; break; }
        if (i > 64) __nanosleep(40);
      }
      fence_proxy_async();   // the copied rows (generic-proxy stores of other CTAs) must be visible to the TMA engine
    }
    if (!ready) {
      if (p.status) atomicOr(p.status, IFAB_STATUS_PEER_TIMEOUT);
      *pipe.abort_flag = 1;
    }
    pipe.produce(ta, &tmap_b, ready ? num_kb : 0, remote ? m0 : m0 - src * p.rows_local, n0, -1, p.spin_limit, p.status);
  } else if (warp == 1 && lane == 0) {
    pipe.mma(num_kb, p.spin_limit, p.status);
  } else if (warp >= 2) {
    if (!remote && p.world > 1) {
      // While the tensor cores work on this local tile, the four epilogue warps bring the same tile row of every
      // remote shard over NVLink: this CTA's slice of the K columns, eight 16-byte loads in flight per thread.
      const int et = threadIdx.x - 64;
      const int chunks = p.K >> 3, per = (chunks + gridDim.x - 1) / gridDim.x;
      const int c_lo = blockIdx.x * per, width = max(0, min(chunks, c_lo + per) - c_lo);
      const int r0 = m0 - p.rank * p.rows_local;          // first row of the tile inside a shard
      const int rows = min(BM, p.rows_local - r0);
      const int total = rows * width;
      for (int j = 1; j < p.world; ++j) {
        const int s = (p.rank + j) % p.world;
        if (et == 0) {
          s_ready = wait_flag_bounded(p.flags[p.rank] + s, p.epoch, p.spin_limit) ? 1 : 0;
          if (!s_ready && p.status) atomicOr(p.status, IFAB_STATUS_PEER_TIMEOUT);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (s_ready) {
          const bf16* from = p.a_peer[s] + (long)r0 * p.lda;
          bf16* to = p.staged + (long)(s * p.rows_local + r0) * p.lds;
          constexpr int G = 8;
          for (int i0 = et; i0 < total; i0 += 128 * G) {
            uint4 buf[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int i = i0 + 128 * g;
              buf[g] = make_uint4(0u, 0u, 0u, 0u);
              if (i < total) buf[g] = __ldcg(reinterpret_cast<const uint4*>(from + (long)(i / width) * p.lda + (c_lo + i % width) * 8));
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int i = i0 + 128 * g;
              if (i < total) *reinterpret_cast<uint4*>(to + (long)(i / width) * p.lds + (c_lo + i % width) * 8) = buf[g];
            }
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) atomicAdd(p.tile_count + (s * (p.rows_local / BM) + r0 / BM), 1ull);
      }
    }
    if (pipe.wait_accumulator(p.spin_limit, p.status)) {
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
      const int rows_here = min(p.M, (src + 1) * p.rows_local);   // rows past the owner's shard are not part of the tile
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(pipe.tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        const int col = n0 + c0;
        if (row < rows_here && col < p.N) {
          bf16* out = p.c + (long)row * p.ldc + col;
          const int nvalid = min(32, p.N - col);
          if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(out)[i] = pack8(v + 8 * i);
          } else {
            for (int i = 0; i < nvalid; ++i) out[i] = __float2bfloat16_rn(v[i]);
          }
        }
      }
    }
  }
  pipe.teardown();
}

template <int BN>
int launch_ag(const AgMaps& maps, const CUtensorMap& ms, const CUtensorMap& tb, const AgParams& p, cudaStream_t s) {
  auto k = tc_gemm_ag_kernel<BN>;
  if (int rc = opt_in_smem(k, Cfg<BN>::SMEM)) return rc;
  // M tiles never straddle two owners: tiles are laid out per shard
  const int tiles_per_shard = (p.rows_local + BM - 1) / BM;
  dim3 grid((p.N + BN - 1) / BN, tiles_per_shard * p.world);
  return launch_chain(k, grid, dim3(192), (size_t)Cfg<BN>::SMEM, s, maps, ms, tb, p);
}

}  // namespace

// a_peers[r]: rank r's [rows_local, K] shard (row stride lda) in symmetric memory as mapped here; flag_peers[r]: rank r's u64[8]
// flag row. staged: local bf16 [world * rows_local, K] scratch (row stride lds); tile_count: local u64 [world * rows_local / 128],
// zeroed once, owned by this entry point. C is local [world * rows_local, N]. rows_local must be a multiple of 128 unless world == 1.
extern "C" int ifab_allgather_gemm_bf16(void* const* a_peers, long lda, const void* b, long ldb, void* c, long ldc, int rows_local, int N,
                                        int K, int world, int rank, void* const* flag_peers, void* staged, long lds, void* tile_count,
                                        uint64_t epoch, uint32_t* status, void* stream) {
  if (rows_local < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8 || world < 1 || world > IFAB_MAX_RANKS || rank < 0 || rank >= world) return -1;
  if (world > 1 && rows_local % BM) return -1;
  AgMaps maps;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) {
    const void* base = a_peers[r < world ? r : rank];
    if (int rc = make_tmap_bf16_2d(&maps.a[r], base, (uint64_t)rows_local, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  }
  CUtensorMap tb, ms;
  if (world > 1) {
    if (!staged || !tile_count || lds % 8) return -1;
    if (int rc = make_tmap_bf16_2d(&ms, staged, (uint64_t)rows_local * world, (uint64_t)K, (uint64_t)lds, BM)) return rc;
  } else {
    ms = maps.a[0];
  }
  const int BN = N > 128 ? 256 : 128;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN)) return rc;
  AgParams p;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) p.a_peer[r] = (const bf16*)a_peers[r < world ? r : rank];
  p.lda = lda; p.staged = (bf16*)staged; p.lds = lds; p.tile_count = (unsigned long long*)tile_count;
  p.c = (bf16*)c; p.ldc = ldc; p.M = rows_local * world; p.N = N; p.K = K; p.rows_local = rows_local; p.world = world; p.rank = rank;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) p.flags[r] = r < world ? (uint64_t*)flag_peers[r] : nullptr;
  p.epoch = epoch; p.status = status; p.spin_limit = 4000000u;
  cudaStream_t s = (cudaStream_t)stream;
  return BN == 256 ? launch_ag<256>(maps, ms, tb, p, s) : launch_ag<128>(maps, ms, tb, p, s);
}
