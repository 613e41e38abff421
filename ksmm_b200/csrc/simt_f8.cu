// Instantiations of the FFMA register-tiled kernel family for fp8-e4m3 inputs
// (fp32 accumulation; bf16, fp16 or fp32 output).
#include "simt_kernel.cuh"

namespace ksmm {
int simt_launch_f8(const Problem& p, int config, cudaStream_t stream) {
  switch (p.out_dtype) {
    case KSMM_BF16: return simt_launch_typed<f8e4m3, __nv_bfloat16>(p, config, stream);
    case KSMM_F16: return simt_launch_typed<f8e4m3, __half>(p, config, stream);
    case KSMM_F32: return simt_launch_typed<f8e4m3, float>(p, config, stream);
    default: return set_error(KSMM_ERR_UNSUPPORTED, "fp8 input needs a bf16, fp16 or fp32 output");
  }
}
}  // namespace ksmm
