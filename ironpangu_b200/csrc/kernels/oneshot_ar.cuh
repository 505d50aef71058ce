// One-shot all-reduce epilogue used inside compute kernels (row-parallel linears, MoE combine).
//
// The calling CTA holds an f32 slab [T][RPC] of partial outputs for columns [nbase, nbase+RPC).
// It pushes the slab into slot `rank` of every peer's staging area, publishes one flag per
// (peer, cta), waits - bounded - for the same-index CTAs of the other ranks, sums the `world`
// partials in rank order (deterministic, independent of arrival order), adds the residual and
// stores bf16. Peer memory is written with plain stores and read back locally; the only remote
// traffic is T*RPC*4 bytes per peer per CTA.
//
// Protocol state: `seq` numbers the fused-collective launches of this rank (all ranks run the same
// sequence); the last CTA of a launch advances it, so CUDA-graph replays get fresh epochs. The
// staging area and the flags are double buffered on the parity of the call number; a rank cannot
// be more than one call ahead of a peer because finishing call n needs that peer's push of call n.
#pragma once
#include "common.cuh"

namespace ifab {

template <int T, int RPC>
__device__ __forceinline__ void oneshot_allreduce_slab(const float* slab, const FabricView& fv, uint64_t* seq,
                                                       uint32_t* done, int nbase, int t_live, int N,
                                                       const bf16* __restrict__ residual, long ldr, bf16* y, long ldy,
                                                       float* y_f32, int* timed_out_smem) {
  const int world = fv.world, rank = fv.rank;
  const uint64_t epoch = *reinterpret_cast<volatile uint64_t*>(seq) + 1;
  const uint32_t par = (uint32_t)(epoch & 1);
  if (world > 1) {
    for (int i = threadIdx.x; i < world * T * RPC; i += blockDim.x) {
      const int q = i / (T * RPC), rem = i % (T * RPC), t = rem / RPC, c = rem % RPC;
      if (t < t_live && nbase + c < N) {
        float* dst = reinterpret_cast<float*>(fv.data[q] + (size_t)par * fv.data_half_bytes) +
                     ((size_t)rank * t_live + t) * N + nbase + c;
        *dst = slab[t * RPC + c];
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
      const int q = threadIdx.x;
      st_release_sys(fv.flags[q] + (size_t)par * fv.flag_half_words + (size_t)rank * gridDim.x + blockIdx.x, epoch);
      const uint64_t* f = fv.flags[rank] + (size_t)par * fv.flag_half_words + (size_t)q * gridDim.x + blockIdx.x;
      if (!wait_flag_bounded(f, epoch, fv.spin_limit)) {
        *timed_out_smem = 1;
        atomicOr(fv.status, IFAB_STATUS_PEER_TIMEOUT);
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < T * RPC; i += blockDim.x) {
    const int t = i / RPC, c = i % RPC;
    if (t >= t_live || nbase + c >= N) continue;
    float v;
    if (world > 1) {
      v = 0.f;
      const float* src = reinterpret_cast<const float*>(fv.data[rank] + (size_t)par * fv.data_half_bytes);
      for (int q = 0; q < world; ++q) v += __ldcg(src + ((size_t)q * t_live + t) * N + nbase + c);
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
      *seq = epoch;
      __threadfence();
    }
  }
}

}  // namespace ifab
