// Expert parallelism with sharded tokens: dispatch / combine all-to-all over NVLink peer memory.
//
// In this mode every rank holds its own tokens (a slice of a prefill chunk, or its share of a data-parallel decode
// batch) and the routed experts live on their owner ranks, so token rows travel to the experts and results travel
// back. Both directions are plain peer stores from inside the kernels that produce the data - there is no separate
// collective:
//
//   ep_dispatch_kernel  (sender)   consumes the router's top-k directly: ranks every local route inside its destination
//                                  (stable, route order), copies the normalised token row into slot (src, idx) of the
//                                  owner's receive buffer together with {local expert, idx}, then publishes the row count
//                                  of every destination with a release flag
//   ep_plan_kernel      (owner)    waits - bounded - for the counts of all sources, sorts the received rows by local expert
//                                  (stable) and emits the 128-row tile table of the grouped tcgen05 GEMM plus the gather list
//   ep_gather_kernel    (owner)    receive buffer -> expert-sorted activation matrix (feeds ifab_grouped_gemm_bf16)
//   ep_return_kernel    (owner)    expert outputs -> slot (owner, idx) of the SOURCE rank's return buffer, then a release flag
//   ep_combine_kernel   (sender)   waits for every owner's flag, out[t] = sum_k w[t,k] * ret[owner_k][idx_k] (+ shared) (+ residual)
//
// Buffers (symmetric, one per rank, peers mapped): recv [W * cap, D] bf16, recv_meta [W * cap] int2, ret [W * cap, D] bf16,
// ctl: counts [W] and two flag rows [W] (u64). cap = rows one source may send to one destination. A receive slot is only
// rewritten after its owner returned the previous results (the sender waits for all return flags before its next dispatch),
// and a return slot only after the sender consumed it, so no double buffering is needed. `epoch` grows by one per layer.
// Reference: the IR-level Send/Recv + expert_pack design of the rank-plan compiler (crates/inferfabric-ir/src/rank_plan.rs);
// the reference runtime itself only ships the replicated-token (owner-local) mode.
#include <algorithm>

#include "common.cuh"
#include "ifab_kernels.h"

using namespace ifab;

namespace {

constexpr int MAX_TOPK = 16;

struct EpCtl {              // layout of the control block of one rank
  uint64_t dispatch_flag[IFAB_MAX_RANKS];   // [src]: epoch once src's rows and count have landed
  uint64_t return_flag[IFAB_MAX_RANKS];     // [owner]: epoch once owner's results have landed
  int32_t count[IFAB_MAX_RANKS];            // [src]: rows src sent in this epoch
};

struct DispatchParams {
  const bf16* xn; long ldxn;                 // normalised local tokens [M, D]
  const int32_t* ids; int M, topk, D, el, world, rank, cap;
  int32_t* send_idx;                         // [M * topk]: row index inside (dst, this rank)'s segment
  bf16* recv[IFAB_MAX_RANKS]; int2* meta[IFAB_MAX_RANKS]; EpCtl* ctl[IFAB_MAX_RANKS];
  uint32_t* ticket; int32_t* dst_count;      // local scratch: [1], [W]
  uint64_t epoch; uint32_t* status;
  int smem_routes;                           // routes whose destinations fit the dynamic shared memory of the launch
};

// grid = any; CTA 0 ranks the routes first (other CTAs wait on a local flag), then all warps copy rows
__global__ void __launch_bounds__(256) ep_dispatch_kernel(DispatchParams p) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = p.M * p.topk;
  __shared__ int s_last;
  bool ranking_missing = false;
  if (blockIdx.x == 0) {
    // stable ranking of the routes inside every destination: warp w handles destinations w, w + 8, ...; the destination of
    // every route is staged in shared memory first (one coalesced pass), so the ballot scans do not wait on global loads
    extern __shared__ unsigned char s_dst[];
    const bool staged = R <= p.smem_routes;
    if (staged) {
      for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const int d = p.ids[i] / p.el;
        s_dst[i] = (unsigned char)((d >= 0 && d < p.world) ? d : 255);
      }
      __syncthreads();
    }
    for (int dst = warp; dst < p.world; dst += 8) {
      int base = 0;
      for (int i0 = 0; i0 < R; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < R && (staged ? (int)s_dst[i] == dst : p.ids[i] / p.el == dst);
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (hit) p.send_idx[i] = base + __popc(m & ((1u << lane) - 1));
        base += __popc(m);
      }
      if (lane == 0) {
        if (base > p.cap) {
          if (p.status) atomicOr(p.status, IFAB_STATUS_BAD_INDEX);
          base = p.cap;
        }
        p.dst_count[dst] = base;
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) atomicExch(p.ticket + 1, 1u);   // ranking done
  } else {
    if (threadIdx.x == 0) {
      s_last = 0;                                 // reused below; here: 1 = the ranking never arrived
      bool ranked = false;
      for (uint32_t spin = 0; spin < 4000000u; ++spin) {
        if (atomicAdd(p.ticket + 1, 0u) != 0) { ranked = true; break; }
        __nanosleep(64);
      }
      if (!ranked) {
        s_last = 1;
        if (p.status) atomicOr(p.status, IFAB_STATUS_PEER_TIMEOUT);
      }
    }
    __syncthreads();
    __threadfence();
    ranking_missing = s_last != 0;
    __syncthreads();
  }
  // copy rows: one warp per route
  // without the ranking the send indices are stale: copy nothing (the status word says why) and only take the ticket
  for (int i = blockIdx.x * 8 + warp; i < R && !ranking_missing; i += gridDim.x * 8) {
    const int e = p.ids[i], dst = e / p.el, idx = __ldcg(p.send_idx + i);
    if (dst < 0 || dst >= p.world || idx >= p.cap) continue;
    const bf16* src = p.xn + (long)(i / p.topk) * p.ldxn;
    bf16* out = p.recv[dst] + ((long)p.rank * p.cap + idx) * p.D;
#pragma unroll 4
    for (int c = lane; c < (p.D >> 3); c += 32) *reinterpret_cast<uint4*>(out + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
    if (lane == 0) p.meta[dst][(long)p.rank * p.cap + idx] = make_int2(e - dst * p.el, idx);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  // last CTA: every row of this rank has been stored; publish the counts
  if ((int)threadIdx.x < p.world) {
    const int dst = threadIdx.x;
    p.ctl[dst]->count[p.rank] = __ldcg(p.dst_count + dst);
    __threadfence_system();
    st_release_sys(&p.ctl[dst]->dispatch_flag[p.rank], p.epoch);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.ticket[0] = 0;
    p.ticket[1] = 0;
    __threadfence();
  }
}

struct PlanParams {
  const int2* meta; EpCtl* ctl; int world, cap, el, max_tiles;
  int32_t* perm;          // [W * cap]: receive-buffer row of sorted row r
  int4* tiles; int32_t* num_tiles; int32_t* total_rows;
  uint64_t epoch; uint32_t spin_limit; uint32_t* status;
  int smem_rows;          // received rows whose expert ids fit the dynamic shared memory of the launch
};

// single CTA of 1024 threads
__global__ void __launch_bounds__(1024) ep_plan_kernel(PlanParams p) {
  __shared__ int s_cnt[IFAB_MAX_RANKS];
  __shared__ int s_count[256], s_off[257];
  __shared__ int s_ok;
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    if (!wait_flag_bounded(&p.ctl->dispatch_flag[threadIdx.x], p.epoch, p.spin_limit)) {
      s_ok = 0;
      if (p.status) atomicOr(p.status, IFAB_STATUS_PEER_TIMEOUT);
    }
    s_cnt[threadIdx.x] = min(p.cap, *reinterpret_cast<volatile int32_t*>(&p.ctl->count[threadIdx.x]));
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) {
      *p.num_tiles = 0;
      *p.total_rows = 0;
    }
    return;
  }
  // the local expert of every received row, staged once in shared memory (source-major): the scans below read it twice per
  // expert and would otherwise wait on a global load per ballot
  extern __shared__ short s_exp[];
  const bool staged = p.world * p.cap <= p.smem_rows;
  if (staged) {
    for (int src = 0; src < p.world; ++src)
      for (int i = threadIdx.x; i < s_cnt[src]; i += blockDim.x) s_exp[src * p.cap + i] = (short)__ldcg(&p.meta[(long)src * p.cap + i]).x;
    __syncthreads();
  }
  auto expert_of = [&](int src, int i) -> int { return staged ? (int)s_exp[src * p.cap + i] : __ldcg(&p.meta[(long)src * p.cap + i]).x; };
  // counts per local expert, then stable placement (source-major, then arrival index)
  for (int e = warp; e < p.el; e += 32) {
    int n = 0;
    for (int src = 0; src < p.world; ++src)
      for (int i0 = 0; i0 < s_cnt[src]; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < s_cnt[src] && expert_of(src, i) == e;
        n += __popc(__ballot_sync(0xffffffffu, hit));
      }
    if (lane == 0) s_count[e] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < p.el; ++e) {
      s_off[e] = off;
      for (int r0 = 0; r0 < s_count[e]; r0 += 128) {
        if (nt < p.max_tiles) p.tiles[nt] = make_int4(e, off + r0, min(128, s_count[e] - r0), 0);
        ++nt;
      }
      off += s_count[e];
    }
    *p.num_tiles = min(nt, p.max_tiles);
    *p.total_rows = off;
  }
  __syncthreads();
  for (int e = warp; e < p.el; e += 32) {
    int base = s_off[e];
    for (int src = 0; src < p.world; ++src)
      for (int i0 = 0; i0 < s_cnt[src]; i0 += 32) {
        const int i = i0 + lane;
        const bool hit = i < s_cnt[src] && expert_of(src, i) == e;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (hit) p.perm[base + __popc(m & ((1u << lane) - 1))] = src * p.cap + i;
        base += __popc(m);
      }
  }
}

// xp[r] = recv[perm[r]] for r < *total_rows
__global__ void __launch_bounds__(256) ep_gather_kernel(const bf16* recv, const int32_t* perm, const int32_t* total_rows, bf16* xp, long ldxp, int D,
                                                        int rows_max) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = min(*total_rows, rows_max);
  for (int r = blockIdx.x * 8 + warp; r < total; r += gridDim.x * 8) {
    const bf16* src = recv + (long)perm[r] * D;
    bf16* dst = xp + (long)r * ldxp;
    for (int c = lane; c < (D >> 3); c += 32) *reinterpret_cast<uint4*>(dst + c * 8) = __ldcg(reinterpret_cast<const uint4*>(src + c * 8));
  }
}

struct ReturnParams {
  const bf16* y; long ldy; const int32_t* perm; const int32_t* total_rows; int D, cap, world, rank, rows_max;
  bf16* ret[IFAB_MAX_RANKS]; EpCtl* ctl[IFAB_MAX_RANKS];
  uint32_t* ticket; uint64_t epoch;
};

__global__ void __launch_bounds__(256) ep_return_kernel(ReturnParams p) {
  __shared__ int s_last;
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = min(*p.total_rows, p.rows_max);
  for (int r = blockIdx.x * 8 + warp; r < total; r += gridDim.x * 8) {
    const int row = p.perm[r], src = row / p.cap, idx = row % p.cap;
    bf16* out = p.ret[src] + ((long)p.rank * p.cap + idx) * p.D;
    const bf16* in = p.y + (long)r * p.ldy;
#pragma unroll 4
    for (int c = lane; c < (p.D >> 3); c += 32) *reinterpret_cast<uint4*>(out + c * 8) = *reinterpret_cast<const uint4*>(in + c * 8);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  if ((int)threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(&p.ctl[threadIdx.x]->return_flag[p.rank], p.epoch);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.ticket[0] = 0;
    __threadfence();
  }
}

struct CombineParams {
  const bf16* ret; EpCtl* ctl; const int32_t* ids; const int32_t* send_idx; const float* wts;
  int M, topk, D, el, world, cap;
  const bf16* shared; long lds; const bf16* residual; long ldr; bf16* out; long ldo;
  uint64_t epoch; uint32_t spin_limit; uint32_t* status;
  int col_splits;
};

// one warp per (token, column range)
__global__ void __launch_bounds__(256) ep_combine_kernel(CombineParams p) {
  __shared__ int s_ok;
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    if (!wait_flag_bounded(&p.ctl->return_flag[threadIdx.x], p.epoch, p.spin_limit)) {
      s_ok = 0;
      if (p.status) atomicOr(p.status, IFAB_STATUS_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  if (!s_ok) return;
  // a warp owns one token and one of `p.col_splits` column ranges, so that small batches still fill the GPU
  const int unit = blockIdx.x * 8 + warp, m = unit / p.col_splits, part = unit % p.col_splits;
  if (m >= p.M) return;
  const int chunks = p.D >> 3, per = (chunks + p.col_splits - 1) / p.col_splits;
  const int c_lo = part * per, c_hi = min(chunks, c_lo + per);
  long rows[MAX_TOPK];
  float w[MAX_TOPK];
#pragma unroll
  for (int k = 0; k < MAX_TOPK; ++k) {
    rows[k] = -1;
    w[k] = 0.f;
    if (k < p.topk) {
      const int i = m * p.topk + k, owner = p.ids[i] / p.el, idx = p.send_idx[i];
      rows[k] = (owner >= 0 && owner < p.world && idx < p.cap) ? (long)owner * p.cap + idx : -1;
      w[k] = p.wts[i];
    }
  }
  for (int c = c_lo + lane; c < c_hi; c += 32) {
    // all rows of the token are requested before the first one is used
    uint4 raw[MAX_TOPK];
#pragma unroll
    for (int k = 0; k < MAX_TOPK; ++k)
      raw[k] = (k < p.topk && rows[k] >= 0) ? __ldcg(reinterpret_cast<const uint4*>(p.ret + rows[k] * p.D + c * 8)) : make_uint4(0, 0, 0, 0);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MAX_TOPK; ++k) {
      if (k < p.topk) {
        float f[8];
        unpack8(raw[k], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[k], f[i], acc[i]);
      }
    }
    if (p.shared) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.shared + (long)m * p.lds + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    if (p.residual) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(p.residual + (long)m * p.ldr + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = bf16_round(acc[i]) + f[i];
    }
    *reinterpret_cast<uint4*>(p.out + (long)m * p.ldo + c * 8) = pack8(acc);
  }
}

}  // namespace

extern "C" {

// peers arrays hold `world` pointers (this rank's entry is the local buffer). scratch: uint32 [2] ticket + int32 [8] counts.
int ifab_ep_dispatch(const void* xn, long ldxn, const int32_t* ids, int M, int topk, int D, int e_local, int world, int rank, int cap,
                     int32_t* send_idx, void* const* recv_peers, void* const* meta_peers, void* const* ctl_peers, uint32_t* ticket,
                     int32_t* dst_count, uint64_t epoch, uint32_t* status, void* stream) {
  if (M < 1 || topk < 1 || topk > MAX_TOPK || D % 8 || ldxn % 8 || world < 1 || world > IFAB_MAX_RANKS || cap < 1) return -1;
  DispatchParams p;
  p.xn = (const bf16*)xn; p.ldxn = ldxn; p.ids = ids; p.M = M; p.topk = topk; p.D = D; p.el = e_local; p.world = world; p.rank = rank;
  p.cap = cap; p.send_idx = send_idx; p.ticket = ticket; p.dst_count = dst_count; p.epoch = epoch; p.status = status;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) {
    p.recv[r] = r < world ? (bf16*)recv_peers[r] : nullptr;
    p.meta[r] = r < world ? (int2*)meta_peers[r] : nullptr;
    p.ctl[r] = r < world ? (EpCtl*)ctl_peers[r] : nullptr;
  }
  const int grid = std::max(1, std::min(2 * 148, (M * topk + 7) / 8));
  const size_t smem = (size_t)std::min(M * topk, 40 * 1024);
  p.smem_routes = (int)smem;
  return launch_chain(ep_dispatch_kernel, dim3(grid), dim3(256), smem, (cudaStream_t)stream, p);
}

int ifab_ep_plan(const void* meta, void* ctl, int world, int cap, int e_local, int32_t* perm, int32_t* tiles, int32_t* num_tiles,
                 int32_t* total_rows, int max_tiles, uint64_t epoch, uint32_t spin_limit, uint32_t* status, void* stream) {
  if (world < 1 || world > IFAB_MAX_RANKS || e_local < 1 || e_local > 256 || max_tiles < 1) return -1;
  PlanParams p{(const int2*)meta, (EpCtl*)ctl, world, cap, e_local, max_tiles, perm, (int4*)tiles, num_tiles, total_rows, epoch, spin_limit, status, 0};
  const size_t want = (size_t)world * cap * sizeof(short);
  const size_t smem = want <= 160 * 1024 ? want : 0;
  p.smem_rows = (int)(smem / sizeof(short));
  if (int rc = opt_in_smem(ep_plan_kernel, smem)) return rc;
  return launch_chain(ep_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream, p);
}

int ifab_ep_gather(const void* recv, const int32_t* perm, const int32_t* total_rows, void* xp, long ldxp, int D, int rows_max, void* stream) {
  if (D % 8 || ldxp % 8 || rows_max < 1) return -1;
  const int grid = std::min(4 * 148, (rows_max + 7) / 8);
  return launch_chain(ep_gather_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const bf16*)recv, perm, total_rows, (bf16*)xp, ldxp, D,
                      rows_max);
}

int ifab_ep_return(const void* y, long ldy, const int32_t* perm, const int32_t* total_rows, int D, int cap, int world, int rank, int rows_max,
                   void* const* ret_peers, void* const* ctl_peers, uint32_t* ticket, uint64_t epoch, void* stream) {
  if (D % 8 || ldy % 8 || world < 1 || world > IFAB_MAX_RANKS) return -1;
  ReturnParams p;
  p.y = (const bf16*)y; p.ldy = ldy; p.perm = perm; p.total_rows = total_rows; p.D = D; p.cap = cap; p.world = world; p.rank = rank;
  p.rows_max = rows_max; p.ticket = ticket; p.epoch = epoch;
  for (int r = 0; r < IFAB_MAX_RANKS; ++r) {
    p.ret[r] = r < world ? (bf16*)ret_peers[r] : nullptr;
    p.ctl[r] = r < world ? (EpCtl*)ctl_peers[r] : nullptr;
  }
  const int grid = std::max(1, std::min(4 * 148, (rows_max + 7) / 8));
  return launch_chain(ep_return_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, p);
}

int ifab_ep_combine(const void* ret, void* ctl, const int32_t* ids, const int32_t* send_idx, const float* wts, int M, int topk, int D,
                    int e_local, int world, int cap, const void* shared, long lds, const void* residual, long ldr, void* out, long ldo,
                    uint64_t epoch, uint32_t spin_limit, uint32_t* status, void* stream) {
  if (D % 8 || topk > MAX_TOPK || ldo % 8 || world < 1 || world > IFAB_MAX_RANKS) return -1;
  CombineParams p{(const bf16*)ret, (EpCtl*)ctl, ids, send_idx, wts, M, topk, D, e_local, world, cap, (const bf16*)shared, lds,
                  (const bf16*)residual, ldr, (bf16*)out, ldo, epoch, spin_limit, status, 1};
  // column ranges per token so that at least ~2 CTAs per SM exist; a range keeps at least one 512-byte warp row
  int splits = 1;
  while (splits < 8 && (long)M * splits < 8L * 2 * 148 && (D >> 3) / (splits * 2) >= 32) splits *= 2;
  p.col_splits = splits;
  return launch_chain(ep_combine_kernel, dim3((M * splits + 7) / 8), dim3(256), 0, (cudaStream_t)stream, p);
}

}  // extern "C"
