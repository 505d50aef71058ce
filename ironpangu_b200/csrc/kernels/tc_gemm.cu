// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] * B[N,K]^T (+ residual), f32 accumulate.
//
// One CTA per 128 x BN output tile, three roles:
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle) through a
//               ring of shared-memory stages, one mbarrier pair (full / empty) per stage
//   warp 1      allocates tensor memory, then one elected lane issues tcgen05.mma (128 x BN x 16 per
//               instruction, accumulator in TMEM) and releases stages with tcgen05.commit
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quarter), convert,
//               add the residual, store bf16 or f32
// A and B are both K-major ("NT"), which is how activations [tokens, K] and weights [out, K] are
// stored everywhere in this library, so no transposes are needed. M, N and K tails are handled by
// TMA zero fill plus masked stores. Used for prefill chunks and batched decode (M >= 16); the
// reference's counterpart is aclnnMatmul on [T<=4096, K] activations (token_executor.h:387-456).
#include "tc_common.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;

struct GemmParams {
  void* c; long ldc; int out_f32;
  const bf16* residual; long ldr;
  int M, N, K;
  uint32_t* status;
  uint32_t spin_limit;
};

template <int BN>
struct Cfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN>
__global__ void __launch_bounds__(192) tc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                      const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* empty = full + C::STAGES;
  uint64_t* acc_full = empty + C::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) tmem_alloc(tmem_slot, BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_launch();
  grid_dep_wait();

  if (warp == 0 && lane == 0) {
    // ---------------- producer ----------------
    int issued = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % C::STAGES;
      const uint32_t round = kb / C::STAGES;
      if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, p.spin_limit)) { *abort_flag = 1; break; }
      if (*abort_flag) break;
      unsigned char* a_dst = smem + s * C::STAGE_BYTES;
      mbar_expect_tx(&full[s], C::STAGE_BYTES);
      tma_load_2d(a_dst, &tmap_a, &full[s], kb * BK, m0);
      tma_load_2d(a_dst + C::A_BYTES, &tmap_b, &full[s], kb * BK, n0);
      issued = kb + 1;
    }
    if (*abort_flag) {
      // drain: every copy this thread issued must land before the CTA may exit
      for (int kb = max(0, issued - C::STAGES); kb < issued; ++kb) mbar_wait(&full[kb % C::STAGES], (kb / C::STAGES) & 1, p.spin_limit);
      if (p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % C::STAGES;
      if (!mbar_wait(&full[s], (kb / C::STAGES) & 1, p.spin_limit) || *abort_flag) { ok = false; break; }
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
      if (p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    umma_commit(acc_full);      // accumulator complete (or abandoned: the epilogue checks the flag)
  } else if (warp >= 2) {
    // ---------------- epilogue ----------------
    const bool ready = mbar_wait(acc_full, 0, p.spin_limit);
    tc_fence_after();
    if (!ready) {
      *abort_flag = 1;
      if (lane == 0 && p.status) atomicOr(p.status, IFAB_STATUS_MBAR_TIMEOUT);
    }
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int row = m0 + q * 32 + lane;
    if (ready && !*abort_flag) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        const int col = n0 + c0;
        if (row < p.M && col < p.N) {
          const int nvalid = min(32, p.N - col);
          if (p.residual) {
            const bf16* r = p.residual + (long)row * p.ldr + col;
            for (int i = 0; i < nvalid; ++i) v[i] = bf16_round(v[i]) + __bfloat162float(r[i]);
          }
          if (p.out_f32) {
            float* out = reinterpret_cast<float*>(p.c) + (long)row * p.ldc + col;
            if (nvalid == 32 && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(out)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
              for (int i = 0; i < nvalid; ++i) out[i] = v[i];
            }
          } else {
            bf16* out = reinterpret_cast<bf16*>(p.c) + (long)row * p.ldc + col;
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
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

template <int BN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t s) {
  auto k = tc_gemm_kernel<BN>;
  if (int rc = opt_in_smem(k, Cfg<BN>::SMEM)) return rc;
  dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM);
  return launch_chain(k, grid, dim3(192), (size_t)Cfg<BN>::SMEM, s, ta, tb, p);
}

}  // namespace

namespace ifab::tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -20;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16 || box_rows == 0 || box_rows > 256) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -21;
}

int make_tmap_bf16_3d(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint64_t bstride, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -20;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * 2) % 16 || (bstride * 2) % 16 || box_rows == 0 || box_rows > 256) return -1;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, bstride * 2};
  cuuint32_t box[3] = {64, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -21;
}

}  // namespace ifab::tc

// C[M,N] = A[M,K] * B[N,K]^T (+ residual). A: row stride lda, B: row stride ldb (elements), K % 8 == 0.
extern "C" int ifab_gemm_bf16(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32,
                              const void* residual, long ldr, int M, int N, int K, uint32_t* status, void* stream) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8) return -1;
  CUtensorMap ta, tb;
  const int BN = N > 128 ? 256 : 128;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN)) return rc;
  GemmParams p{c, ldc, out_f32, (const bf16*)residual, ldr, M, N, K, status, 4000000u};
  cudaStream_t s = (cudaStream_t)stream;
  return BN == 256 ? launch<256>(ta, tb, p, s) : launch<128>(ta, tb, p, s);
}
