// Row-parallel bf16 GEMM fused with a two-shot all-reduce (reduce-scatter + all-gather) over NVLink peer
// memory:  Y = sum_ranks A_r[M,K_r] * B_r[N,K_r]^T (+ residual), every rank ends with the full result.
//
// A persistent kernel, one CTA per SM, 128 x 256 tiles over this rank's K shard. Tensor memory holds TWO accumulators
// (2 x 256 columns): while the four epilogue warps exchange tile i with the other GPUs, the TMA producer and the MMA
// issuer are already running the main loop of tile i + 1 into the other accumulator, so the NVLink traffic of a tile
// moves underneath the tensor-core work of the next one. Tile t is owned by rank t % world; a rank works through the
// tiles it does NOT own first (in index order, strided over its CTAs) and its own tiles last, so by the time an owner
// reaches a tile the partials of the other ranks - pushed from the front of their schedules - have normally arrived.
// A tile is exchanged in four passes of 64 columns through one 18 KB shared-memory buffer, which leaves room for a
// 4-stage operand ring beside it:
//   non-owner  accumulator columns -> bf16 rows in shared memory -> one bulk copy per row (cp.async.bulk shared ->
//              global) into slot (t, rank) of the OWNER's staging area; after the last pass: completion of all copies
//              -> one system fence by one thread behind a barrier -> flag; the epilogue never waits for a peer
//   owner      bounded wait for the other ranks' flags of the tile, then per pass: accumulator columns -> bf16 -> sum of
//              the `world` partials in rank order (the own partial rounded to bf16 like the others, so the result does
//              not depend on who owns a tile; eight 16-byte loads in flight per thread) + residual -> rows stored into
//              the output buffer of EVERY rank (the output lives in symmetric memory: out_peers[r] is rank r's
//              buffer); after the last pass each peer's "final" flag of the tile
//   last CTA   (by ticket) waits for the final flags of the tiles this rank does not own, so when the
//              kernel completes on a rank its output is complete, then advances the call counter
// Bytes crossing NVLink per rank: 2 * (world-1)/world * M*N*2 - the minimum of a bf16 reduce-scatter +
// all-gather. Owners wait only for non-owner epilogues, which never wait, so no cycle can form; every wait (mbarrier
// or flag) is bounded and reports through the status word. No TMA multicast and no TMA load from peer memory is
// used: peers are written with non-tensor bulk stores from shared memory and staged partials are read back locally.
// Reference: linear(tp_columns) + allreduce on the bulk collective domain
// (native/src/token_executor.h:374-404, docs/validation/2026-10-18-bulk-domains).
#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

constexpr int AR_BN = 256, AR_STAGES = 4;
constexpr int AR_QN = 64;                                   // columns exchanged per epilogue pass (a quarter of the tile)
constexpr int AR_A_BYTES = BM * BK * 2, AR_B_BYTES = AR_BN * BK * 2, AR_STAGE_BYTES = AR_A_BYTES + AR_B_BYTES;
constexpr int AR_ROW_PAD = AR_QN + 8;                       // bf16 elements per padded row of the exchange buffer
constexpr int AR_TILE_SMEM = BM * AR_ROW_PAD * 2;
constexpr size_t AR_TILE_BYTES = (size_t)BM * AR_BN * 2;    // one staged partial tile in global memory
constexpr int AR_SMEM = AR_STAGES * AR_STAGE_BYTES + AR_TILE_SMEM + 1024 /*align*/ + 256 /*barriers*/;

struct ArParams {
  bf16* out_peers[IFAB_MAX_RANKS];   // out_peers[rank] is the local output; same shape / ldc on every rank
  long ldc;
  const bf16* residual; long ldr;
  int M, N, K;
  FabricView fv;
  uint64_t* seq; uint32_t* done;
  int tiles_n, ntiles;
  // reduce-scatter mode: rank r owns the row block [r * rows_per_rank, (r + 1) * rows_per_rank) and keeps the finished rows
  // in its own [rows_per_rank, N] shard (out_peers[rank], residual addressed shard-relative); nothing is gathered
  int scatter, rows_per_rank, tiles_per_rank;
  uint32_t spin_limit;
};

// owner of a tile and the index of the tile among its owner's tiles
__device__ __forceinline__ int owner_of(const ArParams& a, int tile, int* local) {
  if (!a.scatter) {
    *local = tile / a.fv.world;
    return tile % a.fv.world;
  }
  const int o = min(tile / a.tiles_per_rank, a.fv.world - 1);
  *local = tile - o * a.tiles_per_rank;
  return o;
}

// barrier 1 over the 128 epilogue threads that also ANDs a predicate, so that every warp takes the same branch
__device__ __forceinline__ bool epilogue_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)pred) : "memory");
  return r != 0;
}

// schedule position -> tile: the tiles of the other owners in increasing index, then this rank's own tiles
__device__ __forceinline__ int tile_at(const ArParams& a, int pos) {
  const int ntiles = a.ntiles, world = a.fv.world, rank = a.fv.rank;
  if (world == 1) return pos;
  if (a.scatter) {
    // row-block ownership: the other owners in ring order starting at rank + 1 (so that at any moment every GPU receives
    // from one sender), each owner's tiles in index order, then this rank's own block
    const int own = a.tiles_per_rank, foreign = ntiles - own;
    if (pos >= foreign) return rank * own + (pos - foreign);
    const int j = pos / own;
    return ((rank + 1 + j) % world) * own + pos % own;
  }
  const int owned = (ntiles - rank + world - 1) / world, foreign = ntiles - owned;
  if (pos < foreign) {
    const int g = pos / (world - 1), i = pos % (world - 1);
    return g * world + (i < rank ? i : i + 1);
  }
  return (pos - foreign) * world + rank;
}

__global__ void __launch_bounds__(192, 1) tc_gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                   const __grid_constant__ CUtensorMap tmap_b, ArParams a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_flag_ok, s_last;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  bf16* tile_s = reinterpret_cast<bf16*>(smem + AR_STAGES * AR_STAGE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + AR_STAGES * AR_STAGE_BYTES + AR_TILE_SMEM);
  uint64_t* empty = full + AR_STAGES;
  uint64_t* acc_full = empty + AR_STAGES;    // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AR_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * AR_BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int world = a.fv.world, rank = a.fv.rank;
  const int num_kb = (a.K + BK - 1) / BK;
  // this CTA's tiles: schedule positions blockIdx.x, + gridDim.x, ...
  const int my_tiles = (a.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  grid_dep_launch();
  grid_dep_wait();
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(a.seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  auto half = [&](int r) { return a.fv.data[r] + (size_t)par * a.fv.data_half_bytes; };
  auto flags = [&](int r) { return a.fv.flags[r] + (size_t)par * a.fv.flag_half_words; };

  if (warp == 0 && lane == 0) {
    // ---- TMA producer: one continuous ring of stages over all tiles of this CTA ----
    int it = 0, issued = 0;
    for (int i = 0; i < my_tiles && !*abort_flag; ++i) {
      const int tile = tile_at(a, blockIdx.x + i * gridDim.x);
      const int m0 = (tile / a.tiles_n) * BM, n0 = (tile % a.tiles_n) * AR_BN;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % AR_STAGES;
        const uint32_t round = it / AR_STAGES;
        if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, a.spin_limit)) { *abort_flag = 1; break; }
        if (*abort_flag) break;
        unsigned char* dst = smem + s * AR_STAGE_BYTES;
        mbar_expect_tx(&full[s], AR_STAGE_BYTES);
        tma_load_2d(dst, &tmap_a, &full[s], kb * BK, m0);
        tma_load_2d(dst + AR_A_BYTES, &tmap_b, &full[s], kb * BK, n0);
        issued = it + 1;
      }
    }
    if (*abort_flag) {
      // drain: every copy this thread issued must land before the CTA may exit
      for (int k = max(0, issued - AR_STAGES); k < issued; ++k) mbar_wait(&full[k % AR_STAGES], (k / AR_STAGES) & 1, a.spin_limit);
      atomicOr(a.fv.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: tile i accumulates into accumulator i & 1 ----
    constexpr uint32_t idesc = umma_idesc_bf16(BM, AR_BN);
    int it = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int acc = i & 1, use = i >> 1;
      if (use > 0 && !mbar_wait(&acc_empty[acc], (use - 1) & 1, a.spin_limit)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d = tmem_base + (uint32_t)(acc * AR_BN);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % AR_STAGES;
        if (!mbar_wait(&full[s], (it / AR_STAGES) & 1, a.spin_limit) || *abort_flag) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * AR_STAGE_BYTES);
        const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + AR_A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, kb > 0 || k > 0);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(&acc_full[acc]);
    }
    if (!ok) {
      *abort_flag = 1;
      atomicOr(a.fv.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
  } else if (warp >= 2) {
    // ---- epilogue warps: exchange tile i while the main loop of tile i + 1 runs ----
    const int q = warp & 3, trow = q * 32 + lane, et = threadIdx.x - 64;
    if (a.scatter) {
      // Reduce-scatter calls do not end with a gather; what keeps a fast rank from overwriting staging slots of this parity
      // half that a slow owner is still reducing is that finishing any call needs a push from every peer. This explicit check
      // states that condition instead of relying on it. Every rank leaves, per half, the epoch of the last call of this
      // kernel it finished there (its own copy in slot `rank`, one in every peer's slot table); all ranks make the same
      // calls, so the previous user of this half has the same epoch everywhere: wait until every peer has finished it.
      // (Other fused kernels advance the shared call counter too, so that call is not simply "two epochs ago".)
      const uint64_t* slots = flags(rank) + (size_t)a.fv.flag_half_words - world;
      const uint64_t prev = *reinterpret_cast<const volatile uint64_t*>(slots + rank);
      if (prev > 0 && et < world && et != rank && !wait_flag_bounded(slots + et, prev, a.fv.spin_limit))
        atomicOr(a.fv.status, IFAB_STATUS_PEER_TIMEOUT);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    for (int i = 0; i < my_tiles; ++i) {
      const int acc = i & 1, use = i >> 1;
      const int tile = tile_at(a, blockIdx.x + i * gridDim.x);
      const int m0 = (tile / a.tiles_n) * BM, n0 = (tile % a.tiles_n) * AR_BN;
      int local_idx;
      const int owner = owner_of(a, tile, &local_idx);
      const int out_row0 = a.scatter ? m0 - rank * a.rows_per_rank : m0;   // first row of the tile in the local output / residual
      const bool ok = epilogue_all(mbar_wait(&acc_full[acc], use & 1, a.spin_limit) && !*abort_flag);
      tc_fence_after();
      if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicOr(a.fv.status, IFAB_STATUS_MBAR_TIMEOUT);
        break;
      }
      // The tile is exchanged in four passes of 64 columns through one small shared-memory buffer (which leaves room
      // for a 4-stage operand ring); the accumulator goes back to the MMA issuer after the last pass has read it.
      const uint32_t tm = tmem_base + (uint32_t)(acc * AR_BN) + ((uint32_t)(q * 32) << 16);
      const bool pusher = world > 1 && rank != owner;
      bool good = true;
      if (!pusher) {
        if (et == 0) s_flag_ok = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (world > 1 && et < world && et != rank) {
          if (!wait_flag_bounded(flags(rank) + (size_t)tile * world + et, epoch, a.fv.spin_limit)) {
            s_flag_ok = 0;
            atomicOr(a.fv.status, IFAB_STATUS_PEER_TIMEOUT);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        good = s_flag_ok != 0;
      }
      bf16* push_dst = reinterpret_cast<bf16*>(half(owner) + ((size_t)local_idx * world + rank) * AR_TILE_BYTES);
      const bf16* stage = reinterpret_cast<const bf16*>(half(rank) + (size_t)local_idx * world * AR_TILE_BYTES);
#pragma unroll 1
      for (int qc = 0; qc < AR_BN; qc += AR_QN) {
        // the previous pass's bulk copies have finished READING the buffer
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < AR_QN; c0 += 32) {
          float v[32];
          tmem_ld_32x32(tm + (uint32_t)(qc + c0), v);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(tile_s + (size_t)trow * AR_ROW_PAD + c0 + 8 * k) = pack8(v + 8 * k);
        }
        if (qc + AR_QN == AR_BN) {
          tc_fence_before();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) mbar_arrive(&acc_empty[acc]);
        } else {
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const int ncols = min(AR_QN, a.N - (n0 + qc));     // valid columns of this pass (multiple of 8, may be <= 0)
        if (pusher) {
          // ---- push the partial rows: one bulk copy per row (thread et owns row et) ----
          fence_proxy_async_smem();   // thread et wrote row et itself
          bulk_store(push_dst + (size_t)et * AR_BN + qc, tile_s + (size_t)et * AR_ROW_PAD, AR_QN * 2);
          bulk_commit();
        } else {
          // ---- owner (or single rank): reduce in rank order, add the residual, publish to every rank ----
          if (good) {
            // item j = 16-byte chunk (j % CPQ) of row (j / CPQ); a thread owns items et + 128 * g, all G in flight at once
            constexpr int CPQ = AR_QN / 8, G = BM * CPQ / 128;
            uint4 res[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int j = et + 128 * g, r = j / CPQ, c = j % CPQ;
              const bool in = m0 + r < a.M && n0 + qc + c * 8 < a.N;
              res[g] = (a.residual && in) ? *reinterpret_cast<const uint4*>(a.residual + (long)(out_row0 + r) * a.ldr + n0 + qc + c * 8) : make_uint4(0, 0, 0, 0);
            }
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
                const int j = et + 128 * g, r = j / CPQ, c = j % CPQ;
                raw[g] = src == rank ? *reinterpret_cast<const uint4*>(tile_s + (size_t)r * AR_ROW_PAD + c * 8)
                                     : __ldcg(reinterpret_cast<const uint4*>(stage + (size_t)src * BM * AR_BN + (size_t)r * AR_BN + qc + c * 8));
              }
#pragma unroll
              for (int g = 0; g < G; ++g) {
                float f[8];
                unpack8(raw[g], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[g][k] += f[k];
              }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int j = et + 128 * g, r = j / CPQ, c = j % CPQ;
              if (a.residual) {
                float f[8];
                unpack8(res[g], f);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[g][k] = bf16_round(v[g][k]) + f[k];
              }
              *reinterpret_cast<uint4*>(tile_s + (size_t)r * AR_ROW_PAD + c * 8) = pack8(v[g]);
            }
          }
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (good && m0 + et < a.M && ncols > 0) {
            if (a.scatter) {
              bulk_store(a.out_peers[rank] + (long)(out_row0 + et) * a.ldc + n0 + qc, tile_s + (size_t)et * AR_ROW_PAD, (uint32_t)ncols * 2);
            } else {
              for (int dst = 0; dst < world; ++dst)
                bulk_store(a.out_peers[dst] + (long)(m0 + et) * a.ldc + n0 + qc, tile_s + (size_t)et * AR_ROW_PAD, (uint32_t)ncols * 2);
            }
          }
          bulk_commit();
        }
      }
      // every copy of the tile has landed: publish
      bulk_wait_all();
      if (world > 1) {
        fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          __threadfence_system();
          if (pusher) {
            st_release_sys(flags(owner) + (size_t)tile * world + rank, epoch);
          } else if (!a.scatter) {
            for (int dst = 0; dst < world; ++dst)
              if (dst != rank) st_release_sys(flags(dst) + (size_t)a.ntiles * world + tile, epoch);
          }
        }
      }
    }
  }
  // ---- teardown: free tensor memory, then the last CTA of this rank collects the final flags ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * AR_BN);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(a.done, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  if (world > 1 && !a.scatter) {
    for (int t = threadIdx.x; t < a.ntiles; t += blockDim.x) {
      if (t % world == rank) continue;
      if (!wait_flag_bounded(flags(rank) + (size_t)a.ntiles * world + t, epoch, a.fv.spin_limit)) atomicOr(a.fv.status, IFAB_STATUS_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  // "this rank has finished call `epoch`" (it no longer reads the staging slots of this parity half), for the guard above:
  // to every peer, and to the own slot table (the next call on this half reads which epoch to wait for)
  if (world > 1 && (int)threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flags(threadIdx.x) + (size_t)a.fv.flag_half_words - world + rank, epoch);
  }
  if (threadIdx.x == 0) {
    *a.done = 0;
    *a.seq = epoch;
    __threadfence();
  }
}

int launch_ar(const CUtensorMap& ta, const CUtensorMap& tb, ArParams& a, cudaStream_t s) {
  auto k = tc_gemm_allreduce_kernel;
  if (int rc = opt_in_smem(k, AR_SMEM)) return rc;
  a.tiles_n = (a.N + AR_BN - 1) / AR_BN;
  a.ntiles = a.tiles_n * ((a.M + BM - 1) / BM);
  if (a.fv.world > 1) {
    const size_t owned = a.scatter ? (size_t)a.tiles_per_rank : (size_t)(a.ntiles + a.fv.world - 1) / a.fv.world;
    if (owned * a.fv.world * AR_TILE_BYTES > a.fv.data_half_bytes) return -3;
    if ((size_t)a.ntiles * (a.fv.world + 1) + a.fv.world > a.fv.flag_half_words) return -4;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int grid = a.ntiles < sms ? a.ntiles : sms;
  return launch_chain(k, dim3(grid), dim3(192), (size_t)AR_SMEM, s, ta, tb, a);
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
  p.scatter = 0; p.rows_per_rank = 0; p.tiles_per_rank = 0;
  p.seq = fab->seq;
  p.done = fab->done;
  p.spin_limit = 4000000u;
  cudaStream_t s = (cudaStream_t)stream;
  return launch_ar(ta, tb, p, s);
}

// Reduce-scatter form: rank r ends with rows [r * M / world, (r + 1) * M / world) of sum_ranks A_r B_r^T (+ residual) in its
// own `out` shard [M / world, N] (row stride ldc); `residual` is the matching [M / world, N] shard. M / world must be a
// multiple of 128. Same staging / flag protocol as the all-reduce form; no gather, no final flags.
extern "C" int ifab_gemm_reduce_scatter_bf16(const void* a, long lda, const void* b, long ldb, void* out, long ldc, const void* residual,
                                             long ldr, int M, int N, int K, const IfabFabric* fab, void* stream) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8 || ldc % 8 || N % 8 || (residual && ldr % 8)) return -1;
  if (M % fab->world || (fab->world > 1 && (M / fab->world) % BM)) return -1;
  CUtensorMap ta, tb;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)AR_BN)) return rc;
  ArParams p;
  if (int rc = fabric_view(fab, &p.fv)) return rc;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) p.out_peers[r] = nullptr;
  if (out == nullptr || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  p.out_peers[fab->rank] = (bf16*)out;
  p.ldc = ldc;
  p.residual = (const bf16*)residual;
  p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.scatter = fab->world > 1 ? 1 : 0;
  p.rows_per_rank = M / fab->world;
  p.tiles_per_rank = ((M / fab->world + BM - 1) / BM) * ((N + AR_BN - 1) / AR_BN);
  p.seq = fab->seq;
  p.done = fab->done;
  p.spin_limit = 4000000u;
  return launch_ar(ta, tb, p, (cudaStream_t)stream);
}
