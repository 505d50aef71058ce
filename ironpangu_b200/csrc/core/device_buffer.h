// Device-buffer contract of one kernel invocation, and its checked binding to the plugin ABI's tensor descriptors.
//
// An Invocation names the implementation (with the sha256 of its binary and its numerical contract), the rank / device /
// stream it runs on, the allocations it may touch and, as views into those allocations, its inputs, outputs and workspace.
// `verify` proves from the record alone: ids unique, everything on the invocation's rank and device, weights read-only,
// views contiguous with positive strides, aligned, inside their allocation, outputs overlapping nothing (read / read
// overlap is allowed), the workspace overlapping no tensor, and no allocation listed that nothing uses. `verify_prepared`
// compares what the backend's prepare step reported (binary identity, numerical contract, workspace size and alignment)
// with the frozen record: a larger workspace is an error, never a silent re-plan. `bind` resolves the views against
// resident allocations supplied by the caller (id, base address, capacity, rank, device) into IFKernelTensorV1
// descriptors, re-checking aliasing on ABSOLUTE addresses, since two ids may name overlapping memory.
// Nothing here allocates on a device, copies, launches, synchronises or dereferences a device address.
// Reference: crates/inferfabric-plan/src/device_buffer.rs:10-436.
#pragma once
#include <optional>

#include "base.h"
#include "kernel_plugin.h"

namespace ifab::device_buffer {

constexpr const char* kFormat = "inferfabric.device-buffer.v1";

enum class DType { I8 = 1, Bf16 = 2, F32 = 3 };       // the values are the ABI tags
uint64_t dtype_bytes(DType d);
enum class Access { Read = 1, Write = 2 };
enum class MemoryClass { Weight, State, Activation, Workspace, Input, Output };

struct Allocation {
  uint32_t id = 0, rank = 0, device = 0;
  uint64_t bytes = 0, alignment = 256;
  MemoryClass cls = MemoryClass::Activation;
  bool read_only = false;
};
struct TensorView {
  uint32_t allocation = 0;
  uint64_t offset = 0;
  DType dtype = DType::Bf16;
  std::vector<uint64_t> shape, strides;       // strides in elements; the ABI takes contiguous views only
  uint64_t alignment = 16;
  Access access = Access::Read;
  uint64_t byte_span() const;                 // throws Invalid unless 1..8 dims, all positive, contiguous
};
struct Workspace {
  uint32_t allocation = 0;
  uint64_t offset = 0, bytes = 0, alignment = 256;
};
struct Invocation {
  std::string format = kFormat, implementation, binary_sha256, numerical_contract;
  uint32_t rank = 0, device = 0, stream = 0;
  std::vector<Allocation> allocations;
  std::vector<TensorView> inputs, outputs;
  std::optional<Workspace> workspace;         // absent = the invocation is frozen at zero workspace

  void verify() const;
  void verify_prepared(const std::string& binary_sha256, const std::string& numerical_contract, uint64_t workspace_bytes,
                       uint64_t workspace_alignment) const;
  Json to_json() const;
  static Invocation from_json(const Json& j);
};

// What the contract supports, for tools that want to show it.
Json support();

// A device allocation owned by the caller for as long as anything bound to it may run. The address is taken on trust
// (nothing can prove that it belongs to the device) and is never dereferenced here.
struct ResidentAllocation {
  uint32_t id = 0;
  void* base = nullptr;
  uint64_t bytes = 0;
  uint32_t rank = 0, device = 0;
};
struct BoundInvocation {
  std::vector<IFKernelTensorV1> inputs, outputs;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
};
BoundInvocation bind(const Invocation& call, const std::vector<ResidentAllocation>& residents);

}  // namespace ifab::device_buffer
