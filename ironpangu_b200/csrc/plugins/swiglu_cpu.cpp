// Example kernel plugin for the host target: contract "inferfabric.swiglu.bf16.v1" on CPU memory.
// input  x [T, 2F] bf16 (gate columns then up columns), output y [T, F] bf16 = silu(gate) * up, computed in f32.
// It exists to exercise the plugin loader without a device; the CUDA build of the same contract is swiglu_cuda.cu.
#include <cmath>
#include <cstring>
#include <new>

#include "../core/kernel_plugin.h"

namespace {

struct State { const uint16_t* x; uint16_t* y; int64_t T, F, ldx, ldy; };

float from_bf16(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);   // round to nearest even
  return (uint16_t)(u >> 16);
}

int32_t prepare(const IFKernelTensorV1* in, uint32_t n_in, const IFKernelTensorV1* out, uint32_t n_out, IFKernelPreparedV1* prepared) {
  prepared->state = nullptr;
  prepared->workspace_bytes = 0;
  prepared->workspace_alignment = 1;
  if (n_in != 1 || n_out != 1 || in[0].dtype != 2 || out[0].dtype != 2 || in[0].rank != 2 || out[0].rank != 2) return 1;
  if (in[0].shape[0] != out[0].shape[0] || in[0].shape[1] != 2 * out[0].shape[1] || in[0].strides[1] != 1 || out[0].strides[1] != 1) return 2;
  State* s = new (std::nothrow) State{(const uint16_t*)in[0].data, (uint16_t*)out[0].data, out[0].shape[0], out[0].shape[1], in[0].strides[0],
                                      out[0].strides[0]};
  if (!s) return 3;
  prepared->state = s;
  return 0;
}

int32_t enqueue(void* state, void*, uint64_t, void*) {
  const State* s = (const State*)state;
  for (int64_t t = 0; t < s->T; ++t)
    for (int64_t j = 0; j < s->F; ++j) {
      const float g = from_bf16(s->x[t * s->ldx + j]), u = from_bf16(s->x[t * s->ldx + s->F + j]);
      s->y[t * s->ldy + j] = to_bf16(g / (1.f + std::exp(-g)) * u);
    }
  return 0;
}

void release(void* state) { delete (State*)state; }

const IFKernelV1 table = {sizeof(IFKernelV1), 1, "inferfabric.swiglu.bf16.v1", "cpu", prepare, enqueue, release};

}  // namespace

extern "C" const IFKernelV1* inferfabric_kernel_v1(uint32_t requested_version) { return requested_version == 1 ? &table : nullptr; }
