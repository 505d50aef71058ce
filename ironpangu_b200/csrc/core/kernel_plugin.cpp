#include "kernel_plugin.h"

#include <dlfcn.h>

#include <cstring>

namespace ifab::plugin {

uint64_t dtype_bytes(uint32_t dtype) {
  switch (dtype) {
    case 1: return 1;
    case 2: return 2;
    case 3: return 4;
    default: invalid("plugin tensor: unknown dtype " + std::to_string(dtype));
  }
}

uint64_t tensor_span_bytes(const IFKernelTensorV1& t) {
  if (t.rank == 0 || t.rank > 8) invalid("plugin tensor: rank must be 1..8");
  int64_t last = 0;
  for (uint32_t i = 0; i < t.rank; ++i) {
    if (t.shape[i] <= 0 || t.strides[i] < 0) invalid("plugin tensor: shape must be positive and strides non-negative");
    last += (t.shape[i] - 1) * t.strides[i];
  }
  return (uint64_t)(last + 1) * dtype_bytes(t.dtype);
}

IFKernelTensorV1 make_tensor(void* data, uint32_t dtype, const std::vector<int64_t>& shape, uint32_t access, uint64_t allocation_bytes) {
  if (shape.empty() || shape.size() > 8) invalid("plugin tensor: rank must be 1..8");
  IFKernelTensorV1 t{};
  t.struct_bytes = sizeof(IFKernelTensorV1);
  t.dtype = dtype;
  t.rank = (uint32_t)shape.size();
  t.access = access;
  t.data = data;
  int64_t stride = 1;
  for (size_t i = shape.size(); i-- > 0;) {
    t.shape[i] = shape[i];
    t.strides[i] = stride;
    stride *= shape[i];
  }
  t.allocation_bytes = allocation_bytes ? allocation_bytes : tensor_span_bytes(t);
  return t;
}

PluginKernel::PluginKernel(const std::string& path, const std::string& contract, const std::string& target) : contract_(contract) {
  handle_ = ::dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!handle_) {
    const char* why = ::dlerror();   // a second call would return NULL: the message is consumed by the first
    fail(ErrorKind::Io, "kernel plugin: cannot load " + path + ": " + (why ? why : "unknown error"));
  }
  auto entry = reinterpret_cast<IFKernelEntryV1>(::dlsym(handle_, "inferfabric_kernel_v1"));
  auto refuse = [&](ErrorKind k, const std::string& why) {
    ::dlclose(handle_);
    handle_ = nullptr;
    fail(k, "kernel plugin " + path + ": " + why);
  };
  if (!entry) refuse(ErrorKind::Stale, "does not export inferfabric_kernel_v1");
  table_ = entry(1);
  if (!table_) refuse(ErrorKind::Stale, "does not offer ABI version 1");
  if (table_->struct_bytes < sizeof(IFKernelV1) || table_->abi_version != 1) refuse(ErrorKind::Stale, "ABI table has an unexpected size or version");
  if (!table_->contract || contract != table_->contract)
    refuse(ErrorKind::Stale, std::string("implements contract '") + (table_->contract ? table_->contract : "") + "', wanted '" + contract + "'");
  if (!table_->target || target != table_->target)
    refuse(ErrorKind::Stale, std::string("was built for target '") + (table_->target ? table_->target : "") + "', this runtime is '" + target + "'");
  if (!table_->prepare || !table_->enqueue || !table_->release) refuse(ErrorKind::Stale, "has a null entry point");
}

PluginKernel::~PluginKernel() {
  if (is_prepared_ && table_) table_->release(prepared_.state);   // the caller fenced completion (contract of the ABI)
  if (handle_) ::dlclose(handle_);
}

void PluginKernel::prepare(const std::vector<IFKernelTensorV1>& inputs, const std::vector<IFKernelTensorV1>& outputs) {
  if (is_prepared_) invalid("kernel plugin: prepare was already called");
  struct Range { const char* lo; const char* hi; bool write; };
  std::vector<Range> ranges;
  auto check = [&](const IFKernelTensorV1& t, bool output) {
    if (t.struct_bytes != sizeof(IFKernelTensorV1)) invalid("plugin tensor: struct_bytes does not match this ABI");
    if (!t.data) invalid("plugin tensor: null data pointer");
    const uint64_t span = tensor_span_bytes(t);
    if (span > t.allocation_bytes) invalid("plugin tensor: the view extends past its allocation");
    if (output && !(t.access & 2)) invalid("plugin tensor: an output must be writable");
    if (!output && (t.access & 2)) invalid("plugin tensor: an input must be read-only");
    ranges.push_back({(const char*)t.data, (const char*)t.data + span, output});
  };
  for (auto& t : inputs) check(t, false);
  for (auto& t : outputs) check(t, true);
  for (size_t i = 0; i < ranges.size(); ++i)
    for (size_t j = i + 1; j < ranges.size(); ++j)
      if ((ranges[i].write || ranges[j].write) && ranges[i].lo < ranges[j].hi && ranges[j].lo < ranges[i].hi)
        invalid("plugin tensors: an output overlaps another tensor");
  IFKernelPreparedV1 out{};
  const int32_t rc = table_->prepare(inputs.data(), (uint32_t)inputs.size(), outputs.data(), (uint32_t)outputs.size(), &out);
  if (rc != 0) {
    if (out.state) table_->release(out.state);
    fail(ErrorKind::Backend, "kernel plugin '" + contract_ + "': prepare failed with code " + std::to_string(rc));
  }
  if (out.workspace_alignment == 0) out.workspace_alignment = 1;
  if (out.workspace_alignment & (out.workspace_alignment - 1)) {
    if (out.state) table_->release(out.state);
    fail(ErrorKind::Backend, "kernel plugin '" + contract_ + "': workspace alignment is not a power of two");
  }
  prepared_ = out;
  is_prepared_ = true;
}

void PluginKernel::enqueue(void* workspace, uint64_t workspace_bytes, void* stream) {
  if (!is_prepared_) invalid("kernel plugin: enqueue before prepare");
  if (in_flight_) invalid("kernel plugin: the previous enqueue has not been reported complete");
  if (workspace_bytes < prepared_.workspace_bytes) fail(ErrorKind::Capacity, "kernel plugin: workspace is smaller than prepare() asked for");
  if (prepared_.workspace_bytes && ((uintptr_t)workspace & (prepared_.workspace_alignment - 1))) invalid("kernel plugin: workspace is misaligned");
  in_flight_ = true;   // stays set on failure too: the caller must fence before release
  const int32_t rc = table_->enqueue(prepared_.state, workspace, workspace_bytes, stream);
  if (rc != 0) fail(ErrorKind::Backend, "kernel plugin '" + contract_ + "': enqueue failed with code " + std::to_string(rc));
}

}  // namespace ifab::plugin
