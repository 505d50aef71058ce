// Example kernel plugin for the CUDA target ("cuda-sm100a"): contract "inferfabric.swiglu.bf16.v1".
// input x [T, 2F] bf16 (gate columns then up columns) -> y [T, F] bf16 = silu(gate) * up in f32. prepare() only checks
// shapes and records pointers; enqueue() launches one kernel on the caller's stream and allocates nothing.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <new>

#include "../core/kernel_plugin.h"

namespace {

struct State { const __nv_bfloat16* x; __nv_bfloat16* y; long T, F, ldx, ldy; };

__global__ void swiglu_kernel(State s) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= s.T * s.F) return;
  const long t = i / s.F, j = i % s.F;
  const float g = __bfloat162float(s.x[t * s.ldx + j]), u = __bfloat162float(s.x[t * s.ldx + s.F + j]);
  s.y[t * s.ldy + j] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
}

int32_t prepare(const IFKernelTensorV1* in, uint32_t n_in, const IFKernelTensorV1* out, uint32_t n_out, IFKernelPreparedV1* prepared) {
  prepared->state = nullptr;
  prepared->workspace_bytes = 0;
  prepared->workspace_alignment = 1;
  if (n_in != 1 || n_out != 1 || in[0].dtype != 2 || out[0].dtype != 2 || in[0].rank != 2 || out[0].rank != 2) return 1;
  if (in[0].shape[0] != out[0].shape[0] || in[0].shape[1] != 2 * out[0].shape[1] || in[0].strides[1] != 1 || out[0].strides[1] != 1) return 2;
  State* s = new (std::nothrow) State{(const __nv_bfloat16*)in[0].data, (__nv_bfloat16*)out[0].data, (long)out[0].shape[0],
                                      (long)out[0].shape[1], (long)in[0].strides[0], (long)out[0].strides[0]};
  if (!s) return 3;
  prepared->state = s;
  return 0;
}

int32_t enqueue(void* state, void*, uint64_t, void* stream) {
  const State* s = (const State*)state;
  const long n = s->T * s->F;
  swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*s);
  return (int32_t)cudaGetLastError();
}

void release(void* state) { delete (State*)state; }

const IFKernelV1 table = {sizeof(IFKernelV1), 1, "inferfabric.swiglu.bf16.v1", "cuda-sm100a", prepare, enqueue, release};

}  // namespace

extern "C" const IFKernelV1* inferfabric_kernel_v1(uint32_t requested_version) { return requested_version == 1 ? &table : nullptr; }
