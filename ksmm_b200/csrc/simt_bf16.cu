// Instantiations of the FFMA register-tiled kernel family for one element type.
#include "simt_kernel.cuh"

namespace ksmm {
int simt_launch_bf16(const Problem& p, int config, cudaStream_t stream) {
  return simt_launch_typed<__nv_bfloat16, __nv_bfloat16>(p, config, stream);
}
}  // namespace ksmm
