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
//   * the address of the array on the current device is looked up on every call (cudaGetSymbolAddress, a
//     host-side query that allocates nothing), so it stays right across a device reset or a new context.
//     The first call on a device may load the module: make it outside any stream capture
//   * every call on a device uses the same array, so two calls that can overlap on the GPU (different
//     streams without an ordering between them) race on it. Issue calls on one stream, or order them
//   * the array keeps whatever the previous call left in it. Nothing here needs it zeroed: each call
//     writes every partial it later reads (the merge reads split s of a head only when that split
//     holds at least one key, and exactly those splits are written by the same call)
// The arithmetic is the one of ifab_gqa_decode_attention - this entry point forwards to it with the
// built-in workspace - so results are bit-identical to a call with a caller-provided buffer.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "ifab_kernels.h"

namespace {

// the workspace: [T][Hq][max_splits][head_dim + 2] f32 partials (accumulator, running max, running sum)
static __device__ __align__(256) unsigned char g_gqa_static_scratch[IFAB_GQA_STATIC_SCRATCH_BYTES];

// formats into the caller's buffer (if any); snprintf does not allocate
void explain(char* err, uint64_t err_len, const char* fmt, ...) {
  if (!err || !err_len) return;
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(err, (size_t)err_len, fmt, ap);
  va_end(ap);
}

// The array's address on the current device (each device has its own copy of a __device__ variable). In host code the
// array's name is only a handle for this query, never a device pointer. Nothing is cached: the query is cheap and a cached
// pointer would be stale after a device reset.
int static_scratch(float** out, char* err, uint64_t err_len) {
  void* sym = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&sym, g_gqa_static_scratch);
  if (e != cudaSuccess || !sym) {
    int dev = -1;
    (void)cudaGetDevice(&dev);
    explain(err, err_len, "cudaGetSymbolAddress of the built-in workspace failed on device %d (CUDA error %d)", dev, (int)e);
    return e != cudaSuccess ? (int)e : -1;
  }
  *out = static_cast<float*>(sym);
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
            "raise keys_per_split (the last split covers the tail of any context) together with a lower max_splits, or lower T, "
            "or use ifab_gqa_decode_attention with your own buffer",
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

extern "C" uint64_t ifab_gqa_static_scratch_bytes(void) { return (uint64_t)IFAB_GQA_STATIC_SCRATCH_BYTES; }
extern "C" int ifab_err_static_scratch(void) { return IFAB_ERR_STATIC_SCRATCH; }
