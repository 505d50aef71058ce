// Shared device helpers for the sm_100a kernels: bf16 packing, warp/block reductions,
// status words and the bounded cross-GPU flag protocol used by the fused collectives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "ifab_kernels.h"


// Status word bits written by kernels instead of trapping. The host reads the word after a step.
#define IFAB_STATUS_OK 0u
#define IFAB_STATUS_PEER_TIMEOUT 1u   // a bounded wait on a peer flag ran out
#define IFAB_STATUS_MBAR_TIMEOUT 2u   // a bounded wait on an mbarrier ran out
#define IFAB_STATUS_BAD_INDEX 4u      // a page / expert / token index was out of range and skipped

typedef __nv_bfloat16 bf16;

namespace ifab {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 8 bf16 packed in a uint4 -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// streaming 16-byte load that does not pollute L1 (weights are read once per step)
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. Every kernel of the decode chain is launched with the
// programmatic-stream-serialization attribute: it may start while its predecessor is still
// running. `grid_dep_launch` lets the successor start; `grid_dep_wait` blocks until the predecessor
// grid has completed and its writes are visible. Before the wait a kernel may only read data that
// no kernel writes (weights) and must not write global memory; every kernel of the chain executes
// the wait, so completion order stays transitive.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline int& pdl_enabled() {
  static int on = 1;
  return on;
}

// Launch `kernel` on `s`, with programmatic dependent launch unless it was switched off.
template <typename... KArgs, typename... Args>
inline int launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with thread-block clusters of `cluster_x` CTAs along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline int launch_chain_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster_x, size_t smem, cudaStream_t s,
                                Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename KernelT>
inline int opt_in_smem(KernelT kernel, size_t smem) {
  // the 48 KB default covers static + dynamic shared memory together, so opt in well below it
  if (smem <= 32 * 1024) return 0;
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

// ---------------------------------------------------------------------------------------------
// Cross-GPU flag protocol. Flags are 64-bit epochs in memory that every rank maps. A writer
// publishes its data with plain stores, then one thread issues a system-scope release store of
// the epoch; a reader spins (bounded) with system-scope acquire loads. The spin never exceeds
// `limit` polls: when it runs out the caller records IFAB_STATUS_PEER_TIMEOUT and carries on so
// the kernel always terminates and the context stays usable.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// returns true when the flag reached `want` within `limit` polls
__device__ __forceinline__ bool wait_flag_bounded(const uint64_t* p, uint64_t want, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ld_acquire_sys(p) >= want) return true;
    if (i > 64) __nanosleep(40);
  }
  return false;
}

// View of the symmetric heap handed to every fused collective kernel (by value).
//   data[r]  : rank r's staging area as mapped into this process (data[rank] is local)
//   flags[r] : rank r's flag words
//   seq      : local device counter bumped once per forward pass (same value on all ranks)
//   status   : local status word
struct FabricView {
  char* data[IFAB_MAX_RANKS];
  uint64_t* flags[IFAB_MAX_RANKS];
  const uint64_t* seq;
  uint32_t* status;
  int rank;
  int world;
  uint32_t spin_limit;
  uint32_t data_half_bytes;   // bytes of one parity half of the staging area
  uint32_t flag_half_words;   // flag words of one parity half
  uint32_t ll_half_bytes;     // one parity half of the tagged-store area (used only by oneshot_ar.cuh)
  uint64_t ll_offset;         // its byte offset from data[r]
  char* mc;                   // multicast mapping of the block (NVLS), or nullptr
};

// NVLink multicast (NVLS): one store that the switch delivers to the same offset of every rank's block
__device__ __forceinline__ void multimem_st_u64(uint64_t* mc_addr, uint64_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_addr), "l"(v) : "memory");
}
// the sum over all ranks of the four floats at this offset, reduced inside the switch
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, const float4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// host: build the by-value device view from the C descriptor
inline int fabric_view(const IfabFabric* f, FabricView* v) {
  if (f == nullptr || f->world < 1 || f->world > IFAB_MAX_RANKS || f->rank < 0 || f->rank >= f->world) return -10;
  for (int i = 0; i < IFAB_MAX_RANKS; ++i) {
    v->data[i] = (char*)f->data[i];
    v->flags[i] = (uint64_t*)f->flags[i];
  }
  v->seq = f->seq;
  v->status = f->status;
  v->rank = f->rank;
  v->world = f->world;
  v->spin_limit = f->spin_limit;
  v->data_half_bytes = f->data_half_bytes;
  v->flag_half_words = f->flag_half_words;
  v->ll_half_bytes = f->ll_half_bytes;
  v->ll_offset = f->ll_offset;
  v->mc = (char*)f->mc;
  return 0;
}

}  // namespace ifab
