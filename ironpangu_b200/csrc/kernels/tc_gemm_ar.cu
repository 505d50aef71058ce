// Row-parallel bf16 GEMM fused with a two-shot all-reduce (reduce-scatter + all-gather) over NVLink peer
// memory:  Y = sum_ranks A_r[M,K_r] * B_r[N,K_r]^T (+ residual), every rank ends with the full result.
//
// Every rank runs the same grid of 128 x 128 tiles over its K shard (tcgen05 main loop of
// tc_gemm_core.cuh, 3-stage ring so that two CTAs share an SM and one tile's exchange overlaps another
// tile's main loop). Tile t is owned by rank t % world. A rank computes the tiles it does NOT own first (in
// index order) and its own tiles last, so by the time an owner reaches a tile the partials of the other ranks -
// pushed from the front of their grids - have normally arrived and the bounded wait falls through.
//   non-owner  accumulator -> bf16 tile in shared memory (the drained TMA ring) -> one bulk copy per row
//              (cp.async.bulk shared -> global) into slot (t, rank) of the OWNER's staging area -> one
//              system fence by one thread behind a CTA barrier -> flag; the CTA then exits, it never waits
//   owner      waits - bounded - for the other ranks' flags of its tile, sums the `world` partials in rank
//              order (its own partial rounded to bf16 like the others, so the result does not depend on
//              who owns a tile; eight 16-byte loads in flight per thread), adds the residual, rounds, and
//              stores the finished rows into the output buffer of EVERY rank (the output lives in symmetric
//              memory: out_peers[r] is rank r's buffer), then raises each peer's "final" flag of the tile
//   last CTA   (by ticket) waits for the final flags of the tiles this rank does not own, so when the
//              kernel completes on a rank its output is complete, then advances the call counter
// Bytes crossing NVLink per rank: 2 * (world-1)/world * M*N*2 - the minimum of a bf16 reduce-scatter +
// all-gather - and they move tile by tile underneath the main loops of later tiles. Owners wait only for
// non-owner CTAs, which never wait, so no cycle can form. No TMA multicast and no TMA load from peer memory is used: peers are written with
// non-tensor bulk stores from shared memory and staged partials are read back locally. Reference: linear(tp_columns) + allreduce on the bulk collective domain
// (native/src/token_executor.h:374-404, docs/validation/2026-10-18-bulk-domains).
#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

struct ArParams {
  bf16* out_peers[IFAB_MAX_RANKS];   // out_peers[rank] is the local output; same shape / ldc on every rank
  long ldc;
  const bf16* residual; long ldr;
  int M, N, K;
  FabricView fv;
  uint64_t* seq; uint32_t* done;
  int tiles_n, ntiles;
  uint32_t spin_limit;
};

template <int BN, int NSTAGES>
__global__ void __launch_bounds__(192) tc_gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                const __grid_constant__ CUtensorMap tmap_b, ArParams a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_flag_ok, s_last;
  Pipe<BN, NSTAGES> pipe;
  pipe.setup(smem_raw, &tmap_a, &tmap_b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int world = a.fv.world, rank = a.fv.rank;
  // block order: the tiles of the other owners in increasing index, then this rank's own tiles
  int tile = blockIdx.x;
  if (world > 1) {
    const int owned = (a.ntiles - rank + world - 1) / world, foreign = a.ntiles - owned;
    const int b = blockIdx.x;
    if (b < foreign) {
      const int g = b / (world - 1), i = b % (world - 1);
      tile = g * world + (i < rank ? i : i + 1);
    } else {
      tile = (b - foreign) * world + rank;
    }
  }
  const int m0 = (tile / a.tiles_n) * BM, n0 = (tile % a.tiles_n) * BN;
  const int num_kb = (a.K + BK - 1) / BK;
  const int owner = tile % world;
  grid_dep_launch();
  grid_dep_wait();
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(a.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  constexpr size_t TILE_BYTES = (size_t)BM * BN * 2;
  constexpr int ROW_PAD = BN + 8;                       // bf16 elements per padded shared-memory row
  auto half = [&](int r) { return a.fv.data[r] + (size_t)par * a.fv.data_half_bytes; };
  auto flags = [&](int r) { return a.fv.flags[r] + (size_t)par * a.fv.flag_half_words; };
  if (warp == 0 && lane == 0) {
    pipe.produce(&tmap_a, &tmap_b, num_kb, m0, n0, -1, a.spin_limit, a.fv.status);
  } else if (warp == 1 && lane == 0) {
    pipe.mma(num_kb, a.spin_limit, a.fv.status);
  } else if (warp >= 2) {
    const bool ok = pipe.wait_accumulator(a.spin_limit, a.fv.status);
    const int q = warp & 3, trow = q * 32 + lane, et = threadIdx.x - 64, ew = warp - 2;   // epilogue thread / warp ids
    const uint32_t tm = pipe.tmem_base + ((uint32_t)(q * 32) << 16);
    bf16* tile_s = reinterpret_cast<bf16*>(pipe.smem);   // the stage ring is drained once the accumulator is complete
    // accumulator -> bf16 rows in shared memory
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tm + (uint32_t)c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(tile_s + (size_t)trow * ROW_PAD + c0 + 8 * i) = pack8(v + 8 * i);
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    constexpr int CPR = BN / 8;                          // 16-byte chunks per row
    const int nvalid = min(BN, a.N - n0);                // valid columns of this tile (multiple of 8)
    if (world > 1 && rank != owner) {
      // ---- push the partial tile: one bulk copy per row (thread et owns row et) ----
      bf16* dst = reinterpret_cast<bf16*>(half(owner) + ((size_t)(tile / world) * world + rank) * TILE_BYTES);
      if (ok) bulk_store(dst + (size_t)et * BN, tile_s + (size_t)et * ROW_PAD, BN * 2);
      bulk_commit();
      bulk_wait_all();
      fence_proxy_async();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) {
        __threadfence_system();
        st_release_sys(flags(owner) + (size_t)tile * world + rank, epoch);
      }
    } else {
      // ---- owner (or single rank): reduce in rank order, add the residual, publish to every rank ----
      if (et == 0) s_flag_ok = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (world > 1 && et < world && et != rank) {
        if (!wait_flag_bounded(flags(rank) + (size_t)tile * world + et, epoch, a.fv.spin_limit)) {
          s_flag_ok = 0;
          atomicOr(a.fv.status, IFAB_STATUS_PEER_TIMEOUT);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool good = ok && s_flag_ok;
      if (good) {
        const bf16* stage = reinterpret_cast<const bf16*>(half(rank) + (size_t)(tile / world) * world * TILE_BYTES);
        // item i = 16-byte chunk (i % CPR) of row (i / CPR); a thread owns items et + 128 * k and keeps G of them in flight
        constexpr int G = 8, ITEMS = BM * CPR / 128;
        static_assert(ITEMS % G == 0, "items per thread must split into groups");
#pragma unroll 1
        for (int k0 = 0; k0 < ITEMS; k0 += G) {
          float v[G][8];
#pragma unroll
          for (int g = 0; g < G; ++g)
#pragma unroll
            for (int k = 0; k < 8; ++k) v[g][k] = 0.f;
#pragma unroll 1
          for (int src = 0; src < world; ++src) {
            uint4 raw[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int i = et + 128 * (k0 + g), r = i / CPR, c = i % CPR;
              raw[g] = src == rank ? *reinterpret_cast<const uint4*>(tile_s + (size_t)r * ROW_PAD + c * 8)
                                   : __ldcg(reinterpret_cast<const uint4*>(stage + (size_t)src * BM * BN + (size_t)r * BN + c * 8));
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
              float f[8];
              unpack8(raw[g], f);
#pragma unroll
              for (int k = 0; k < 8; ++k) v[g][k] += f[k];
            }
          }
          uint4 res[G];
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const int i = et + 128 * (k0 + g), r = i / CPR, c = i % CPR;
            const bool in = m0 + r < a.M && n0 + c * 8 < a.N;
            res[g] = (a.residual && in) ? *reinterpret_cast<const uint4*>(a.residual + (long)(m0 + r) * a.ldr + n0 + c * 8) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const int i = et + 128 * (k0 + g), r = i / CPR, c = i % CPR;
            if (a.residual) {
              float f[8];
              unpack8(res[g], f);
#pragma unroll
              for (int k = 0; k < 8; ++k) v[g][k] = bf16_round(v[g][k]) + f[k];
            }
            *reinterpret_cast<uint4*>(tile_s + (size_t)r * ROW_PAD + c * 8) = pack8(v[g]);
          }
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (good && m0 + et < a.M) {
        for (int dst = 0; dst < world; ++dst)
          bulk_store(a.out_peers[dst] + (long)(m0 + et) * a.ldc + n0, tile_s + (size_t)et * ROW_PAD, (uint32_t)nvalid * 2);
      }
      bulk_commit();
      bulk_wait_all();
      if (world > 1) {
        fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          __threadfence_system();
          for (int dst = 0; dst < world; ++dst)
            if (dst != rank) st_release_sys(flags(dst) + (size_t)a.ntiles * world + tile, epoch);
        }
      }
    }
  }
  pipe.teardown();
  // ---- the last CTA of this rank collects the final flags of the tiles owned by peers ----
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(a.done, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (world > 1) {
    for (int t = threadIdx.x; t < a.ntiles; t += blockDim.x) {
      if (t % world == rank) continue;
      if (!wait_flag_bounded(flags(rank) + (size_t)a.ntiles * world + t, epoch, a.fv.spin_limit)) atomicOr(a.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *a.done = 0;
    *a.seq = epoch;
    __threadfence();
  }
}

// 128 x 128 tiles with a 3-stage ring (97 KB of shared memory): two CTAs share an SM, so the exchange of one
// tile overlaps the tensor-core main loop of another.
constexpr int AR_BN = 128, AR_STAGES = 3;

int launch_ar(const CUtensorMap& ta, const CUtensorMap& tb, ArParams& a, cudaStream_t s) {
  using C = Cfg<AR_BN, AR_STAGES>;
  auto k = tc_gemm_allreduce_kernel<AR_BN, AR_STAGES>;
  if (int rc = opt_in_smem(k, C::SMEM)) return rc;
  static_assert((size_t)BM * (AR_BN + 8) * 2 <= (size_t)C::STAGES * C::STAGE_BYTES, "tile must fit the drained ring");
  a.tiles_n = (a.N + AR_BN - 1) / AR_BN;
  a.ntiles = a.tiles_n * ((a.M + BM - 1) / BM);
  if (a.fv.world > 1) {
    const size_t owned = (a.ntiles + a.fv.world - 1) / a.fv.world;
    if (owned * a.fv.world * (size_t)BM * AR_BN * 2 > a.fv.data_half_bytes) return -3;
    if ((size_t)a.ntiles * (a.fv.world + 1) > a.fv.flag_half_words) return -4;
  }
  return launch_chain(k, dim3(a.ntiles), dim3(192), (size_t)C::SMEM, s, ta, tb, a);
}

}  // namespace

// `out_peers`: world pointers to the output buffer of every rank as mapped into this process (entry `rank` is
// the local one). With world == 1 only entry 0 is used. N and ldc must be multiples of 8.
extern "C" int ifab_gemm_allreduce_bf16(const void* a, long lda, const void* b, long ldb, void* const* out_peers, long ldc,
                                        const void* residual, long ldr, int M, int N, int K, const IfabFabric* fab,
                                        void* stream) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8 || ldc % 8 || N % 8 || (residual && ldr % 8)) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)AR_BN)) return rc;
  ArParams p;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) p.out_peers[r] = r < fab->world ? (bf16*)out_peers[r] : nullptr;
  for (int r = 0; r < fab->world; ++r)
    if (p.out_peers[r] == nullptr || (reinterpret_cast<uintptr_t>(p.out_peers[r]) & 15)) return -1;
  p.ldc = ldc;
  p.residual = (const bf16*)residual;
  p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.seq = fab->seq;
  p.done = fab->done;
  p.spin_limit = 4000000u;
  cudaStream_t s = (cudaStream_t)stream;
  return launch_ar(ta, tb, p, s);
}
