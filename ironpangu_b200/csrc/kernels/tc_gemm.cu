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
#include <cstdlib>

#include "tc_gemm_core.cuh"
#include "ifab_kernels.h"

using namespace ifab;
using namespace ifab::tc;

namespace {

struct GemmParams {
  void* c; long ldc; int out_f32;
  const bf16* residual; long ldr;
  int M, N, K;
  uint32_t* status;
  uint32_t spin_limit;
};

// store 32 consecutive columns of one row (values already final)
__device__ __forceinline__ void store_row32(const GemmParams& p, int row, int col, float* v) {
  if (row >= p.M || col >= p.N) return;
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

template <int BN>
__global__ void __launch_bounds__(192) tc_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                      const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  Pipe<BN> pipe;
  pipe.setup(smem_raw, &tmap_a, &tmap_b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int num_kb = (p.K + BK - 1) / BK;
  grid_dep_launch();
  grid_dep_wait();
  if (warp == 0 && lane == 0) {
    pipe.produce(&tmap_a, &tmap_b, num_kb, m0, n0, -1, p.spin_limit, p.status);
  } else if (warp == 1 && lane == 0) {
    pipe.mma(num_kb, p.spin_limit, p.status);
  } else if (warp >= 2) {
    if (pipe.wait_accumulator(p.spin_limit, p.status)) {
      const int q = warp & 3;                       // TMEM lane quarter this warp may read
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        tmem_ld_32x32(pipe.tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        store_row32(p, row, n0 + c0, v);
      }
    }
  }
  pipe.teardown();
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

// IFAB_GEMM_2SM=0 keeps every shape on the one-CTA kernel (for A/B timing)
static bool two_sm_enabled() {
  static const bool on = [] {
    const char* v = getenv("IFAB_GEMM_2SM");
    return !(v && v[0] == '0');
  }();
  return on;
}

// C[M,N] = A[M,K] * B[N,K]^T (+ residual). A: row stride lda, B: row stride ldb (elements), K % 8 == 0.
extern "C" int ifab_gemm_bf16(const void* a, long lda, const void* b, long ldb, void* c, long ldc, int out_f32,
                              const void* residual, long ldr, int M, int N, int K, uint32_t* status, void* stream) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8) return -1;
  // from 256 x 256 up: CTA pairs (tcgen05.mma cta_group::2; same accumulation order, same bits) - persistent with two
  // accumulators when there is more than one tile per SM pair, one tile per pair otherwise
  if (M >= 256 && N >= 256 && N % 32 == 0 && two_sm_enabled()) {
    const long tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
    return tiles > 74 ? ifab_gemm_bf16_2sm_persistent(a, lda, b, ldb, c, ldc, out_f32, residual, ldr, M, N, K, status, stream)
                      : ifab_gemm_bf16_2sm(a, lda, b, ldb, c, ldc, out_f32, residual, ldr, M, N, K, status, stream);
  }
  CUtensorMap ta, tb;
  const int BN = N > 128 ? 256 : 128;
  if (int rc = make_tmap_bf16_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return rc;
  if (int rc = make_tmap_bf16_2d(&tb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN)) return rc;
  GemmParams p{c, ldc, out_f32, (const bf16*)residual, ldr, M, N, K, status, 4000000u};
  cudaStream_t s = (cudaStream_t)stream;
  return BN == 256 ? launch<256>(ta, tb, p, s) : launch<128>(ta, tb, p, s);
}

