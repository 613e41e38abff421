// Instantiations of the FFMA register-tiled kernel family for one element type.
#include "simt_kernel.cuh"

namespace ksmm {
int simt_launch_f16(const Problem& p, int config, cudaStream_t stream) {
  return simt_launch_typed<__half, __half>(p, config, stream);
}
}  // namespace ksmm
