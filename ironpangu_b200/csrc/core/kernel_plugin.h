// Kernel plugin ABI (version 1) and its loader.
//
// A plugin is a shared object that exports `inferfabric_kernel_v1(requested_version)` and returns a table with a
// contract name (what it computes, e.g. "inferfabric.swiglu.bf16.v1"), a target (which device stack it was built for)
// and three entry points: prepare (host-only: validate tensors, allocate metadata, say how much workspace is needed),
// enqueue (launch on the given stream: no allocation, no synchronisation) and release. The structs are plain C data
// with explicit sizes so that plugins built against this header keep working when fields are appended.
// The ABI is the public one of the reference (native/include/inferfabric_kernel_v1.h), so existing plugin sources
// only need a new target; the loader mirrors compiled_kernel.cpp: dlopen, ABI / contract / target checks, tensor
// aliasing checks, a single-enqueue guard and fail-closed ownership of the prepared state.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
/* dtypes follow the initialization plan: I8 = 1, BF16 = 2, F32 = 3; access: read = 1, write = 2; strides in elements */
typedef struct {
  uint32_t struct_bytes, dtype, rank, access;
  void* data;
  uint64_t allocation_bytes;
  int64_t shape[8], strides[8];
} IFKernelTensorV1;
typedef struct {
  void* state;
  uint64_t workspace_bytes, workspace_alignment;
} IFKernelPreparedV1;
typedef struct {
  uint32_t struct_bytes, abi_version;
  const char* contract;
  const char* target;
  int32_t (*prepare)(const IFKernelTensorV1* inputs, uint32_t input_count, const IFKernelTensorV1* outputs, uint32_t output_count,
                     IFKernelPreparedV1* out);
  int32_t (*enqueue)(void* state, void* workspace, uint64_t bytes, void* stream);
  void (*release)(void* state);
} IFKernelV1;
typedef const IFKernelV1* (*IFKernelEntryV1)(uint32_t requested_version);
#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
#include <string>
#include <vector>

#include "base.h"

namespace ifab::plugin {

constexpr const char* kCudaTarget = "cuda-sm100a";

// One loaded plugin bound to one set of tensors. Not copyable; release() runs in the destructor.
class PluginKernel {
 public:
  // Throws Io (cannot load), Stale (ABI / contract / target mismatch), Invalid (tensor checks), Backend (prepare failed).
  PluginKernel(const std::string& path, const std::string& contract, const std::string& target);
  ~PluginKernel();
  PluginKernel(const PluginKernel&) = delete;
  PluginKernel& operator=(const PluginKernel&) = delete;

  const std::string& contract() const { return contract_; }
  // Validates the tensors (sizes, dtypes, writable outputs that alias nothing else) and calls the plugin's prepare.
  void prepare(const std::vector<IFKernelTensorV1>& inputs, const std::vector<IFKernelTensorV1>& outputs);
  uint64_t workspace_bytes() const { return prepared_.workspace_bytes; }
  uint64_t workspace_alignment() const { return prepared_.workspace_alignment; }
  // One enqueue may be in flight at a time: call completed() after the caller has fenced the stream.
  void enqueue(void* workspace, uint64_t workspace_bytes, void* stream);
  void completed() { in_flight_ = false; }

 private:
  void* handle_ = nullptr;
  const IFKernelV1* table_ = nullptr;
  std::string contract_;
  IFKernelPreparedV1 prepared_{};
  bool is_prepared_ = false, in_flight_ = false;
};

uint64_t dtype_bytes(uint32_t dtype);                                   // throws Invalid for unknown dtypes
uint64_t tensor_span_bytes(const IFKernelTensorV1& t);                   // bytes from data to one past the last element
IFKernelTensorV1 make_tensor(void* data, uint32_t dtype, const std::vector<int64_t>& shape, uint32_t access, uint64_t allocation_bytes = 0);

}  // namespace ifab::plugin
#endif
