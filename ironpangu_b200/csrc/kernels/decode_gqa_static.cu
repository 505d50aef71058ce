// Split-KV paged GQA decode attention for callers that must not allocate.
//
// ifab_gqa_decode_attention() takes its split-partials workspace from the caller, which in practice
// means a cudaMalloc or a framework allocator call somewhere up the stack. Some callers cannot make
// one: a C or C++ serving loop that links this library without a tensor framework and has handed all
// of the device's free memory to its KV cache, a callback running under an allocator lock, or a
// latency-critical path where an allocation could synchronise the device. For them this file keeps
// the workspace inside the library image: a fixed array in device global memory that exists as soon
// as the module is loaded on a device.
//
// Consequences of that choice, all of which a caller has to know:
//   * the workspace has a fixed size (IFAB_GQA_STATIC_SCRATCH_BYTES); a call that needs more is
//     refused with IFAB_ERR_STATIC_SCRATCH and a message, nothing is launched
//   * the address of the array is looked up once per device, on the first call made while that
//     device is current. That first call should be made outside any stream capture; later calls only
//     launch kernels
//   * every call on a device uses the same array, so two calls that can overlap on the GPU (different
//     streams without an ordering between them) race on it. Issue calls on one stream, or order them
//   * the array keeps whatever the previous call left in it. Nothing here needs it zeroed: each call
//     writes every partial it later reads (the merge reads split s of a head only when that split
//     holds at least one key, and exactly those splits are written by the same call)
// The arithmetic is the one of ifab_gqa_decode_attention - this entry point forwards to it with the
// built-in workspace - so results are bit-identical to a call with a caller-provided buffer.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "ifab_kernels.h"

namespace {

constexpr int kMaxDevices = 64;

// the workspace: [T][Hq][max_splits][head_dim + 2] f32 partials (accumulator, running max, running sum)
static __device__ __align__(256) unsigned char g_gqa_static_scratch[IFAB_GQA_STATIC_SCRATCH_BYTES];

// device ordinal -> address of the array on that device (each device has its own copy of a __device__ variable)
std::atomic<float*> g_scratch_addr[kMaxDevices];

// formats into the caller's buffer (if any); snprintf does not allocate
void explain(char* err, uint64_t err_len, const char* fmt, ...) {
  if (!err || !err_len) return;
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(err, (size_t)err_len, fmt, ap);
  va_end(ap);
}

// Looks the address up on first use for the current device; no allocation, the array is part of the module.
int static_scratch(float** out, char* err, uint64_t err_len) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    explain(err, err_len, "cudaGetDevice failed (CUDA error %d)", (int)e);
    return (int)e;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    explain(err, err_len, "device ordinal %d is outside the %d supported", dev, kMaxDevices);
    return -1;
  }
  float* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    void* sym = nullptr;
    e = cudaGetSymbolAddress(&sym, g_gqa_static_scratch);
    if (e != cudaSuccess || !sym) {
      explain(err, err_len, "cudaGetSymbolAddress of the built-in workspace failed on device %d (CUDA error %d)", dev, (int)e);
      return e != cudaSuccess ? (int)e : -1;
    }
    p = static_cast<float*>(sym);
    g_scratch_addr[dev].store(p, std::memory_order_release);   // concurrent first calls store the same value
  }
  *out = p;
  return 0;
}

}  // namespace

extern "C" int ifab_gqa_decode_attention_static(const void* q, long ldq, const void* k_cache, const void* v_cache,
                                                const int32_t* positions, const int32_t* slots, const int32_t* page_table,
                                                int max_pages, int page_tokens, int num_pages, float scale, int T, int Hq,
                                                int Hkv, int head_dim, int keys_per_split, int max_splits, void* out, long ldo,
                                                uint32_t* status, void* stream, char* err, uint64_t err_len) {
  if (err && err_len) err[0] = '\0';
  if (T < 1 || Hq < 1 || head_dim < 1 || max_splits < 1) {
    explain(err, err_len, "T, Hq, head_dim and max_splits must be positive (T=%d, Hq=%d, head_dim=%d, max_splits=%d)", T, Hq, head_dim,
            max_splits);
    return -1;
  }
  const uint64_t need = (uint64_t)T * (uint64_t)Hq * (uint64_t)max_splits * (uint64_t)(head_dim + 2) * sizeof(float);
  if (need > (uint64_t)IFAB_GQA_STATIC_SCRATCH_BYTES) {
    explain(err, err_len,
            "this call needs %llu bytes of split workspace (T*Hq*max_splits*(head_dim+2)*4) but the built-in array holds %llu; "
            "lower max_splits or T, or use ifab_gqa_decode_attention with your own buffer",
            (unsigned long long)need, (unsigned long long)IFAB_GQA_STATIC_SCRATCH_BYTES);
    return IFAB_ERR_STATIC_SCRATCH;
  }
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch, err, err_len)) return rc;
  const int rc = ifab_gqa_decode_attention(q, ldq, k_cache, v_cache, positions, slots, page_table, max_pages, page_tokens, num_pages,
                                           scale, T, Hq, Hkv, head_dim, keys_per_split, max_splits, scratch,
                                           (uint64_t)IFAB_GQA_STATIC_SCRATCH_BYTES, out, ldo, status, stream);
  if (rc) explain(err, err_len, "ifab_gqa_decode_attention refused the call or a launch failed (code %d)", rc);
  return rc;
}
