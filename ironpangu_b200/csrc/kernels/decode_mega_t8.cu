// Instantiations of the persistent decode-step kernel for up to 8 query rows per step (one file per width so
// that the widths compile in parallel).
#include <algorithm>

#include "decode_mega_kernel.cuh"

namespace ifab::mega {
template int launch_step<8, 1>(Params&, cudaStream_t);
}  // namespace ifab::mega
