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

}  // namespace tc
}  // namespace ksmm
