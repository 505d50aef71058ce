// One-shot all-reduce epilogue used inside compute kernels (row-parallel linears, MoE combine).
//
// The calling CTA holds an f32 slab [T][RPC] of partial outputs for columns [nbase, nbase+RPC).
// Every value is pushed to every peer as ONE 8-byte store that carries the f32 payload in its low
// half and the low 32 bits of the call number in its high half. An aligned 8-byte store becomes
// visible as a unit, so the receiver needs neither a fence nor a separate flag: it polls the slot
// itself until the tag matches the call it is in (bounded), which makes the cost of the exchange one
// one-way NVLink store latency instead of two fenced round trips. The `world` partials are then summed
// in rank order (deterministic, independent of arrival order), the residual is added and bf16 stored.
// The only remote traffic is T*RPC*8 bytes per peer per CTA. Where the block has an NVLink multicast mapping (NVLS) the
// push is ONE multimem.st per value, which the switch replicates to every rank; the polling side is the same.
//
// Protocol state: `seq` numbers the fused-collective launches of this rank (all ranks run the same
// sequence); the last CTA of a launch advances it, so CUDA-graph replays get fresh tags. The tagged-store
// area (its own region of the symmetric block: no other protocol may write arbitrary bits there)
// is double buffered on the parity of the call number; a rank cannot be more than one call ahead
// of a peer because finishing call n needs that peer's push of call n, so a slot is never overwritten
// before its reader consumed it. A slot left over from an earlier call carries an older tag and is
// ignored (a false match would need exactly 2^32 calls between two uses of one slot).
#pragma once
#include "common.cuh"

namespace ifab {

template <int T, int RPC>
__device__ __forceinline__ void oneshot_allreduce_slab(const float* slab, const FabricView& fv, uint64_t* seq,
                                                       uint32_t* done, int nbase, int t_live, int N,
                                                       const bf16* __restrict__ residual, long ldr, bf16* y, long ldy,
                                                       float* y_f32, int* timed_out_smem, uint32_t* zero_on_last = nullptr) {
  const int world = fv.world, rank = fv.rank;
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  const uint32_t tag = (uint32_t)epoch;
  if (world > 1 && fv.mc != nullptr) {
    // NVLS: one multicast store per value; the switch writes it into slot [rank][t][col] of every rank (this one included)
    for (int i = threadIdx.x; i < T * RPC; i += blockDim.x) {
      const int t = i / RPC, c = i % RPC;
      if (t < t_live && nbase + c < N) {
        uint64_t* dst = reinterpret_cast<uint64_t*>(fv.mc + fv.ll_offset + (size_t)par * fv.ll_half_bytes) +
                        ((size_t)rank * t_live + t) * N + nbase + c;
        multimem_st_u64(dst, ((uint64_t)tag << 32) | (uint64_t)__float_as_uint(slab[t * RPC + c]));
      }
    }
  } else if (world > 1) {
    for (int i = threadIdx.x; i < world * T * RPC; i += blockDim.x) {
      const int q = i / (T * RPC), rem = i % (T * RPC), t = rem / RPC, c = rem % RPC;
      if (q != rank && t < t_live && nbase + c < N) {
        uint64_t* dst = reinterpret_cast<uint64_t*>(fv.data[q] + fv.ll_offset + (size_t)par * fv.ll_half_bytes) +
                        ((size_t)rank * t_live + t) * N + nbase + c;
        st_relaxed_sys(dst, ((uint64_t)tag << 32) | (uint64_t)__float_as_uint(slab[t * RPC + c]));
      }
    }
  }
  for (int i = threadIdx.x; i < T * RPC; i += blockDim.x) {
    const int t = i / RPC, c = i % RPC;
    if (t >= t_live || nbase + c >= N) continue;
    float v;
    if (world > 1) {
      // all peers' slots are requested at once and only the ones whose tag is still old are asked again: the wait is one
      // load latency after the slowest peer's store lands, not one per peer
      const uint64_t* src = reinterpret_cast<const uint64_t*>(fv.data[rank] + fv.ll_offset + (size_t)par * fv.ll_half_bytes);
      uint64_t got[IFAB_MAX_RANKS];
      unsigned pending = ((1u << world) - 1u) & ~(1u << rank);
      for (uint32_t spin = 0; spin < fv.spin_limit && pending; ++spin) {
#pragma unroll
        for (int q = 0; q < IFAB_MAX_RANKS; ++q)
          if ((pending >> q) & 1u) got[q] = ld_relaxed_sys(src + ((size_t)q * t_live + t) * N + nbase + c);
#pragma unroll
        for (int q = 0; q < IFAB_MAX_RANKS; ++q)
          if (((pending >> q) & 1u) && (uint32_t)(got[q] >> 32) == tag) pending &= ~(1u << q);
        if (pending && spin > 256) __nanosleep(32);
      }
      if (pending) {
        *timed_out_smem = 1;
        atomicOr(fv.status, IFAB_STATUS_PEER_TIMEOUT);
      }
      v = 0.f;
#pragma unroll
      for (int q = 0; q < IFAB_MAX_RANKS; ++q) {
        if (q >= world) break;
        v += (q == rank) ? slab[t * RPC + c] : (((pending >> q) & 1u) ? 0.f : __uint_as_float((uint32_t)got[q]));
      }
    } else {
      v = slab[t * RPC + c];
    }
    if (y_f32) y_f32[(long)t * N + nbase + c] = v;
    if (residual) v = bf16_round(v) + __bfloat162float(residual[(long)t * ldr + nbase + c]);
    y[(long)t * ldy + nbase + c] = __float2bfloat16_rn(v);
  }
  // advance the call counter once every CTA of this launch is done
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(done, 1u);
    if (ticket == gridDim.x - 1) {
      *done = 0;
      if (zero_on_last) *zero_on_last = 0;   // a counter of the calling kernel that every CTA has passed by now
      *seq = epoch;
      __threadfence();
    }
  }
}

}  // namespace ifab
