// Host-side helpers shared by the tensor-core kernel translation units.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ksmm {
namespace tc {

// Rank-`rank` tiled tensor map with 128-byte swizzle (or none); dims/strides
// innermost first, strides in elements (the stride of dim 0 is implicitly 1).
// atom32 selects the 128-byte swizzle that permutes 32-byte pieces by (row % 4), the
// layout of an MN-major tf32 UMMA operand.
int encode_map(CUtensorMap* tm, int dt, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_elems, const uint32_t* box, bool swizzle128 = true,
               bool atom32 = false);
// Device address of the per-device status word (0 = no device-side timeout).
int* status_word();
int num_sms();
// false when the environment variable KSMM_NO_PDL is set (read once): launches are then plain ones
bool pdl_enabled();

// Launch with the programmatic-stream-serialisation attribute (see grid_dep_wait in tc_ptx.cuh).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace tc
}  // namespace ksmm
