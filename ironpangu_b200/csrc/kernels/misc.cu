// Symmetric-heap plumbing (CUDA IPC, one process per GPU) and small layout kernels.
#include "common.cuh"
#include "ifab_kernels.h"
#include <string.h>

using namespace ifab;

extern "C" int ifab_device_alloc(void** out, uint64_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return (int)e;
  }
  *out = p;
  return 0;
}
extern "C" int ifab_device_free(void* p) { return (int)cudaFree(p); }

extern "C" int ifab_ipc_export(void* p, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle, &h, 64);
  return 0;
}
extern "C" int ifab_ipc_import(const unsigned char handle[64], void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int ifab_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

extern "C" int ifab_set_pdl(int on) {
  pdl_enabled() = on ? 1 : 0;
  return 0;
}
extern "C" int ifab_set_device(int device) { return (int)cudaSetDevice(device); }
extern "C" int ifab_peek(void* dst_host, const void* src_device, uint64_t bytes) {
  return (int)cudaMemcpy(dst_host, src_device, bytes, cudaMemcpyDeviceToHost);
}
extern "C" int ifab_poke(void* dst_device, const void* src_host, uint64_t bytes) {
  return (int)cudaMemcpy(dst_device, src_host, bytes, cudaMemcpyHostToDevice);
}

extern "C" const char* ifab_error_string(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "invalid argument (shape / alignment outside the kernel's contract)";
    case -2: return "output width too large for a co-resident fused-collective grid";
    case -3: return "fabric staging area too small for this call";
    case -4: return "fabric flag area too small for this call";
    case -5: return "scratch buffer too small";
    case -6: return "the call needs more split workspace than the library's built-in array holds (ifab_gqa_decode_attention_static)";
    case -7: return "the kernel's co-resident grid does not fit this device";
    case -10: return "invalid fabric descriptor";
    default: break;
  }
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown error";
}

namespace {

__global__ void embedding_kernel(const int32_t* ids, const bf16* table, bf16* out, int D, int vocab, uint32_t* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && status) atomicOr(status, IFAB_STATUS_BAD_INDEX);
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (long)id * D);
  uint4* dst = reinterpret_cast<uint4*>(out + (long)t * D);
  for (int c = threadIdx.x; c < D / 8; c += blockDim.x) dst[c] = src[c];
}

__global__ void __launch_bounds__(256) rmsnorm_kernel(const bf16* x, long ldx, const bf16* w, bf16* y, long ldy, int D,
                                                      float eps, int zero_centered) {
  __shared__ float red[8];
  __shared__ float inv_s;
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const bf16* xr = x + (long)t * ldx;
  float ss = 0.f;
  for (int c = threadIdx.x; c < D / 8; c += blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
    inv_s = rsqrtf(s / (float)D + eps);
  }
  __syncthreads();
  const float inv = inv_s;
  for (int c = threadIdx.x; c < D / 8; c += blockDim.x) {
    float f[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), f);
    unpack8(*reinterpret_cast<const uint4*>(w + c * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * (zero_centered ? 1.f + g[i] : g[i]);
    *reinterpret_cast<uint4*>(y + (long)t * ldy + c * 8) = pack8(f);
  }
}

// act[t, c] = silu(gu[t, c]) * gu[t, F + c]: the activation of a gate/up projection whose GEMM has no SwiGLU epilogue
// (the all-gather GEMM of the sequence-parallel block)
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const bf16* gu, long ldg, bf16* act, long lda, int F) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const bf16* g = gu + (long)t * ldg;
  for (int c = threadIdx.x; c < F / 8; c += blockDim.x) {
    float a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(g + c * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(g + F + c * 8), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = a[i] / (1.f + __expf(-a[i])) * b[i];
    *reinterpret_cast<uint4*>(act + (long)t * lda + c * 8) = pack8(a);
  }
}

}  // namespace

extern "C" int ifab_swiglu_rows_bf16(const void* gu, long ldg, void* act, long lda, int T, int F, void* stream) {
  if (F % 8 != 0 || ldg % 8 != 0 || lda % 8 != 0) return -1;
  return launch_chain(swiglu_rows_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)gu, ldg, (bf16*)act, lda, F);
}

extern "C" int ifab_embedding_bf16(const int32_t* ids, const void* table, void* out, int T, int D, int vocab,
                                   uint32_t* status, void* stream) {
  if (D % 8 != 0) return -1;
  return launch_chain(embedding_kernel, dim3(T), dim3(128), 0, (cudaStream_t)stream, ids, (const bf16*)table, (bf16*)out,
                      D, vocab, status);
}

extern "C" int ifab_rmsnorm_bf16(const void* x, long ldx, const void* w, void* y, long ldy, int T, int D, float eps,
                                 int zero_centered, void* stream) {
  if (D % 8 != 0 || ldx % 8 != 0 || ldy % 8 != 0) return -1;
  return launch_chain(rmsnorm_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x, ldx, (const bf16*)w,
                      (bf16*)y, ldy, D, eps, zero_centered);
}
