// Instantiations of the FFMA register-tiled kernel family for one element type.
#include "simt_kernel.cuh"

namespace ksmm {
int simt_launch_f32(const Problem& p, int config, cudaStream_t stream) {
  return simt_launch_typed<float, float>(p, config, stream);
}
}  // namespace ksmm

namespace ksmm {
int simt_default_config_for(const Problem& p) { return simt_default_config(p); }
int simt_num_configs() { return kNumSimtConfigs; }
}  // namespace ksmm
