// Shared main loop of the tcgen05 GEMM kernels: pipeline state in shared memory, the TMA producer
// role and the MMA issuer role. Kernels differ only in their epilogue (plain store, fused all-reduce,
// grouped / SwiGLU variants).
#pragma once
#include "tc_common.cuh"

namespace ifab::tc {

constexpr int BM = 128, BK = 64, UMMA_K = 16;

template <int BN, int NSTAGES = (BN == 256 ? 4 : 6)>
struct Cfg {
  static constexpr int STAGES = NSTAGES;
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, int NSTAGES = (BN == 256 ? 4 : 6)>
struct Pipe {
  unsigned char* smem;        // 1024-byte aligned stage ring
  uint64_t *full, *empty, *acc_full;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  uint32_t tmem_base;

  // all threads; allocates TMEM (warp 1), initialises barriers, ends with a CTA barrier
  __device__ __forceinline__ void setup(unsigned char* smem_raw, const CUtensorMap* ta, const CUtensorMap* tb) {
    using C = Cfg<BN, NSTAGES>;
    smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    empty = full + C::STAGES;
    acc_full = empty + C::STAGES;
    tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    if (threadIdx.x == 0) {
      for (int s = 0; s < C::STAGES; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      mbar_init(acc_full, 1);
      *abort_flag = 0;
      mbar_fence_init();
      tma_prefetch_desc(ta);
      tma_prefetch_desc(tb);
    }
    if ((threadIdx.x >> 5) == 1) tmem_alloc(tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = *tmem_slot;
  }

  // one thread. (ax, ay[, az]) / (bx, by[, bz]) = tile origins; k advances along x.
  // b_row_hi >= 0: the B tile is two boxes of BN/2 rows (tb's box is BN/2 rows): rows b_row.. fill the first half of
  // the stage's B area and rows b_row_hi.. the second half (paired gate / up projections under one accumulator).
  __device__ __forceinline__ void produce(const CUtensorMap* ta, const CUtensorMap* tb, int num_kb, int a_row, int b_row, int b_batch,
                                          uint32_t spin_limit, uint32_t* status, int b_row_hi = -1) {
    using C = Cfg<BN, NSTAGES>;
    int issued = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % C::STAGES;
      const uint32_t round = kb / C::STAGES;
      if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, spin_limit)) { *abort_flag = 1; break; }
      if (*abort_flag) break;
      unsigned char* a_dst = smem + s * C::STAGE_BYTES;
      mbar_expect_tx(&full[s], C::STAGE_BYTES);
      tma_load_2d(a_dst, ta, &full[s], kb * BK, a_row);
      if (b_batch >= 0) tma_load_3d(a_dst + C::A_BYTES, tb, &full[s], kb * BK, b_row, b_batch);
      else tma_load_2d(a_dst + C::A_BYTES, tb, &full[s], kb * BK, b_row);
      if (b_row_hi >= 0) {
        if (b_batch >= 0) tma_load_3d(a_dst + C::A_BYTES + C::B_BYTES / 2, tb, &full[s], kb * BK, b_row_hi, b_batch);
        else tma_load_2d(a_dst + C::A_BYTES + C::B_BYTES / 2, tb, &full[s], kb * BK, b_row_hi);
      }
      issued = kb + 1;
    }
    if (*abort_flag) {
      // drain: every copy this thread issued must land before the CTA may exit
      for (int kb = max(0, issued - C::STAGES); kb < issued; ++kb) mbar_wait(&full[kb % C::STAGES], (kb / C::STAGES) & 1, spin_limit);
      if (status) atomicOr(status, IFAB_STATUS_MBAR_TIMEOUT);
    }
  }

  // one thread
  __device__ __forceinline__ void mma(int num_kb, uint32_t spin_limit, uint32_t* status) {
    using C = Cfg<BN, NSTAGES>;
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % C::STAGES;
      if (!mbar_wait(&full[s], (kb / C::STAGES) & 1, spin_limit) || *abort_flag) { ok = false; break; }
      tc_fence_after();
      const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
      const uint64_t da = umma_desc_sw128(a_addr), db = umma_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        // advancing 16 bf16 = 32 bytes along K inside the swizzle atom = +2 in 16-byte units
        umma_bf16(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, kb > 0 || k > 0);
      }
      umma_commit(&empty[s]);   // frees the stage once these MMAs have read it
    }
    if (!ok) {
      *abort_flag = 1;
      if (status) atomicOr(status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    umma_commit(acc_full);      // accumulator complete (or abandoned: the epilogue checks the flag)
  }

  // epilogue warps: true when the accumulator is complete and usable
  __device__ __forceinline__ bool wait_accumulator(uint32_t spin_limit, uint32_t* status) {
    const bool ready = mbar_wait(acc_full, 0, spin_limit);
    tc_fence_after();
    if (!ready) {
      *abort_flag = 1;
      if ((threadIdx.x & 31) == 0 && status) atomicOr(status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    return ready && !*abort_flag;
  }

  // all threads
  __device__ __forceinline__ void teardown() {
    tc_fence_before();
    __syncthreads();
    if ((threadIdx.x >> 5) == 1) {
      tc_fence_after();
      tmem_dealloc(tmem_base, BN);
    }
  }
};

}  // namespace ifab::tc
