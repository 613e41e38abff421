// Out-of-place 2-D transpose (1-, 2- and 4-byte elements) used by the
// layout-conversion path: a batch-first factor that no direct kernel covers is
// run as transpose -> batch-last kernel -> transpose.
//
// One CTA moves a 64 x 64 tile through shared memory: 16-byte global loads
// along the input rows, element-wise shared stores into a padded tile, strided
// shared reads along the tile columns, 16-byte global stores in which the lanes
// of a warp follow the output rows (whole 128-byte lines per warp).  Edges and
// unaligned shapes fall back to element accesses.
#include "common.cuh"

namespace ksmm {

template <typename T>
__global__ void __launch_bounds__(256)
    transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t rows, int64_t cols,
                     int vec_ok, unsigned tiles_x) {
  constexpr int TILE = 64;
  constexpr int V = 16 / sizeof(T);            // elements per 16-byte vector
  // one extra 4-byte word per tile row keeps the column reads of a warp on distinct banks
  constexpr int PITCH = TILE + 4 / static_cast<int>(sizeof(T));
  __shared__ T tile[TILE][PITCH];
  // tiles are numbered row-major in one grid dimension (either extent may exceed 65535 tiles)
  const int64_t r0 = static_cast<int64_t>(blockIdx.x / tiles_x) * TILE;
  const int64_t c0 = static_cast<int64_t>(blockIdx.x % tiles_x) * TILE;
  const int tid = threadIdx.x;

  // ---- load: rows r0.., columns c0.. --------------------------------------------
  const bool full = vec_ok && (r0 + TILE <= rows) && (c0 + TILE <= cols);
  if (full) {
    constexpr int VPR = TILE / V;  // vectors per tile row
    for (int v = tid; v < TILE * VPR; v += 256) {
      const int r = v / VPR, cv = v % VPR;
      const uint4 raw = *reinterpret_cast<const uint4*>(in + (r0 + r) * cols + c0 + cv * V);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int q = 0; q < V; ++q) tile[r][cv * V + q] = e[q];
    }
  } else {
    for (int v = tid; v < TILE * TILE; v += 256) {
      const int r = v / TILE, c = v % TILE;
      if (r0 + r < rows && c0 + c < cols) tile[r][c] = in[(r0 + r) * cols + c0 + c];
    }
  }
  __syncthreads();
  // ---- store: output rows c0.., output columns r0.. ----------------------------------
  if (full) {
    constexpr int VPR = TILE / V;
    for (int v = tid; v < TILE * VPR; v += 256) {
      // lanes walk along an output row, so that a warp writes whole 128-byte lines
      const int c = v / VPR, rv = v % VPR;
      uint4 raw;
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int q = 0; q < V; ++q) e[q] = tile[rv * V + q][c];
      *reinterpret_cast<uint4*>(out + (c0 + c) * rows + r0 + rv * V) = raw;
    }
  } else {
    for (int v = tid; v < TILE * TILE; v += 256) {
      const int c = v / TILE, r = v % TILE;
      if (r0 + r < rows && c0 + c < cols) out[(c0 + c) * rows + r0 + r] = tile[r][c];
    }
  }
}

// in: rows x cols row-major, out: cols x rows row-major; `es` = element size in bytes
int launch_transpose(const void* in, void* out, int64_t rows, int64_t cols, int es,
                     cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return KSMM_OK;
  const int64_t gx = (cols + 63) / 64, gy = (rows + 63) / 64;
  if (gx * gy > 0x7fffffffLL)
    return set_error(KSMM_ERR_UNSUPPORTED, "transpose of %lld x %lld exceeds the grid limits",
                     static_cast<long long>(rows), static_cast<long long>(cols));
  const int V = 16 / es;
  const int vec_ok = (rows % V == 0) && (cols % V == 0) &&
                     reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const unsigned grid = static_cast<unsigned>(gx * gy), tx = static_cast<unsigned>(gx);
  if (es == 4)
    transpose_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(in),
                                                         static_cast<uint32_t*>(out), rows, cols, vec_ok, tx);
  else if (es == 2)
    transpose_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(in),
                                                         static_cast<uint16_t*>(out), rows, cols, vec_ok, tx);
  else
    transpose_kernel<uint8_t><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(in),
                                                        static_cast<uint8_t*>(out), rows, cols, vec_ok, tx);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "transpose launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace ksmm
