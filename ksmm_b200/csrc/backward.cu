// Backward of one Kronecker-sparse factor.
//
//   forward    Y4[i,j,l,n] = sum_k W[i,j,k,l] X4[i,k,l,n]
//   dX         dX4[i,k,l,n] = sum_j W[i,j,k,l] dY4[i,j,l,n]: the same multiplication with pattern
//              (a,c,b,d) and every b x c block transposed, so it runs on the forward kernels once
//              the blocks have been transposed (transpose_blocks_kernel below);
//   dW         dW[i,j,k,l] = sum_n dY4[i,j,l,n] X4[i,k,l,n]: a*d independent (c x B) @ (B x b)
//              products whose contraction runs over the batch.  In kernel format the result of block
//              (i,l) is the row-major (c, b) matrix dWk[(i*d + l)*c + k, j].
//
// dW on the tensor cores (16-bit inputs, fp32 accumulation in TMEM): accumulator rows are k (128 per
// tile), columns are j (up to 256), the K dimension of the MMAs is the batch, 64 entries per stage.
// Batch-last rows of X and dY hold consecutive batch entries: both are K-major operands fetched by
// the 4-D maps over (batch, d, features, a) that the forward kernel uses for its input.  Batch-first
// (d = 1) rows hold consecutive features: both are MN-major operands.  Blocks have few tiles, so the
// batch is split over CTAs; every CTA writes an fp32 partial tile and a second kernel sums the
// partials in a fixed order (bitwise repeatable) and converts.  Other cases (fp32, batch-first with
// d > 1, unaligned shapes) take a plain FFMA kernel.
//
// Roles of the tensor kernel (192 threads): warp 0 TMA producer, warp 1 TMEM owner and MMA issuer,
// warps 2..5 epilogue.  Waits are bounded and report through the device status word.
//
// The reference has no backward: Kernel.backward is a stub
// (src/ksmm_py/layer/kronecker_sparse/kernel.py:323-329).
#include <cuda.h>

#include <algorithm>
#include <atomic>

#include "tc_host.h"
#include "tc_kernel.h"
#include "tc_ptx.cuh"

namespace ksmm {

// ---------------------------------------------------------------------------
// block transposes of kernel-format weights: (nblk, c, b) -> (nblk, b, c)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    transpose_blocks_kernel(const T* __restrict__ in, T* __restrict__ out, int c, int b) {
  __shared__ T tile[32][33];
  const int64_t base = static_cast<int64_t>(blockIdx.z) * c * b;
  const int k0 = blockIdx.y * 32, j0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8)
    if (k0 + r < c && j0 + tx < b) tile[r][tx] = in[base + static_cast<int64_t>(k0 + r) * b + j0 + tx];
  __syncthreads();
  for (int r = ty; r < 32; r += 8)
    if (j0 + r < b && k0 + tx < c) out[base + static_cast<int64_t>(j0 + r) * c + k0 + tx] = tile[tx][r];
}

int launch_transpose_blocks(const void* in, void* out, int64_t nblk, int c, int b, int es,
                            cudaStream_t stream) {
  if (nblk <= 0) return KSMM_OK;
  if (nblk > 65535)
    return set_error(KSMM_ERR_UNSUPPORTED, "weight transpose: %lld blocks exceed the grid limit",
                     static_cast<long long>(nblk));
  dim3 grid((b + 31) / 32, (c + 31) / 32, static_cast<unsigned>(nblk));
  if (grid.y > 65535) return set_error(KSMM_ERR_UNSUPPORTED, "weight transpose: c too large");
  if (es == 4)
    transpose_blocks_kernel<uint32_t><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(in),
                                                                static_cast<uint32_t*>(out), c, b);
  else if (es == 2)
    transpose_blocks_kernel<uint16_t><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(in),
                                                                static_cast<uint16_t*>(out), c, b);
  else
    transpose_blocks_kernel<uint8_t><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(in),
                                                               static_cast<uint8_t*>(out), c, b);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "weight transpose launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

// ---------------------------------------------------------------------------
// dW, FFMA fallback: one thread per (k, j) of a 16 x 16 tile, the batch in steps of 32 through
// shared memory; any type, layout and alignment
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
    wgrad_simt_kernel(const T* __restrict__ x, const T* __restrict__ g, T* __restrict__ dw, int64_t batch,
                      int a, int b, int c, int d, int bs_last) {
  __shared__ float xs[16][33], gs[16][33];
  const int blk = blockIdx.z, i = blk / d, l = blk % d;
  const int k0 = blockIdx.y * 16, j0 = blockIdx.x * 16;
  const int tk = threadIdx.x >> 4, tj = threadIdx.x & 15;
  const int64_t n_in = static_cast<int64_t>(a) * c * d, n_out = static_cast<int64_t>(a) * b * d;
  float acc = 0.f;
  for (int64_t n0 = 0; n0 < batch; n0 += 32) {
    for (int e = threadIdx.x; e < 16 * 32; e += 256) {
      // batch-last: lanes walk the batch; batch-first: lanes walk the features
      const int r = bs_last ? e >> 5 : e & 15, nn = bs_last ? e & 31 : e >> 4;
      const int64_t n = n0 + nn;
      float xv = 0.f, gv = 0.f;
      if (n < batch) {
        if (k0 + r < c) {
          const int64_t f = (static_cast<int64_t>(i) * c + k0 + r) * d + l;
          xv = ElemTraits<T>::to_float(x[bs_last ? f * batch + n : n * n_in + f]);
        }
        if (j0 + r < b) {
          const int64_t f = (static_cast<int64_t>(i) * b + j0 + r) * d + l;
          gv = ElemTraits<T>::to_float(g[bs_last ? f * batch + n : n * n_out + f]);
        }
      }
      xs[r][nn] = xv;
      gs[r][nn] = gv;
    }
    __syncthreads();
#pragma unroll
    for (int nn = 0; nn < 32; ++nn) acc = fmaf(xs[tk][nn], gs[tj][nn], acc);
    __syncthreads();
  }
  if (k0 + tk < c && j0 + tj < b)
    dw[(static_cast<int64_t>(blk) * c + k0 + tk) * b + j0 + tj] = ElemTraits<T>::from_float(acc);
}

namespace tc {

struct ParamsW {
  int a, b, c, d;
  int64_t batch;
  int tiles_k, tiles_j, splits;
  int nchunks;  // ceil(batch / 64)
  uint32_t idesc;
  float* part;  // (splits, a*d, c, b) fp32
  int* status;
};

constexpr int kThreadsW = 6 * 32;

template <bool BS_LAST, int NT, int SX>
struct CfgW {
  static constexpr int A_BYTES = 128 * 128;  // 128 k x 64 batch entries (either order)
  static constexpr int B_BYTES = NT * 128;   // NT j x 64 batch entries
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NBAR = 2 * SX + 1;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = SX * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = NT;
  static_assert(NT == 64 || NT == 128 || NT == 256, "j tile");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM, so that the TMEM allocation never waits");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
};

template <bool BS_LAST, int NT, int SX>
__global__ void __launch_bounds__(kThreadsW, 1)
    ksmm_tc_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG,
                         const ParamsW P) {
  using C = CfgW<BS_LAST, NT, SX>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t ring0 = sm0;
  const uint32_t bar0 = ring0 + SX * C::STAGE_BYTES;
  uint8_t* bar_gen = sm_gen + SX * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (SX + s); };
  const uint32_t tfull_bar = bar0 + 8u * (2 * SX);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < SX; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // CTA -> (split, block, k tile, j tile); the split owns a contiguous range of 64-entry chunks
  uint32_t t = blockIdx.x;
  const int tj = static_cast<int>(t % P.tiles_j); t /= P.tiles_j;
  const int tk = static_cast<int>(t % P.tiles_k); t /= P.tiles_k;
  const int sp = static_cast<int>(t % P.splits);
  const int blk = static_cast<int>(t / P.splits);
  const int i = blk / P.d, l = blk % P.d;
  const int k0 = tk * 128, j0 = tj * NT;
  const int ch_begin = static_cast<int>(static_cast<int64_t>(sp) * P.nchunks / P.splits);
  const int ch_end = static_cast<int>(static_cast<int64_t>(sp + 1) * P.nchunks / P.splits);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t si = 0, sph = 0;
      for (int ch = ch_begin; ch < ch_end; ++ch) {
        if (!mbar_wait<64>(empty_bar(si), sph ^ 1u, abort_flag, P.status, 51)) break;
        const uint32_t dst = ring0 + si * C::STAGE_BYTES;
        const uint32_t bar = full_bar(si);
        mbar_expect_tx(bar, C::STAGE_BYTES);
        const int n0 = ch * 64;
        if constexpr (BS_LAST) {
          tma_load_4d(dst, &tmX, bar, n0, l, k0, i);
          tma_load_4d(dst + C::A_BYTES, &tmG, bar, n0, l, j0, i);
        } else {
          // 64 batch rows x 64 features per box; M / N groups of 64 follow one another
          tma_load_3d(dst, &tmX, bar, k0, blk, n0);
          tma_load_3d(dst + 64 * 128, &tmX, bar, k0 + 64, blk, n0);
#pragma unroll
          for (int jb = 0; jb < NT / 64; ++jb)
            tma_load_3d(dst + C::A_BYTES + jb * 64 * 128, &tmG, bar, j0 + jb * 64, blk, n0);
        }
        if (++si == SX) { si = 0; sph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      // descriptor words that never change: SBO = 1024 bytes, version 1, 128-byte swizzle
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      // K-major (batch-last): 32 bytes per k step inside the swizzle row, LBO unused;
      // MN-major (batch-first): LBO = one 64-wide group (64 rows x 128 bytes), 16 rows per k step
      constexpr uint32_t kLbo = BS_LAST ? (1u << 16) : (static_cast<uint32_t>((64 * 128) >> 4) << 16);
      constexpr uint32_t kStep = BS_LAST ? (32u >> 4) : ((16u * 128u) >> 4);
      uint32_t si = 0, sph = 0;
      bool ok = true;
      for (int ch = ch_begin; ch < ch_end; ++ch) {
        if (!mbar_wait<0>(full_bar(si), sph, abort_flag, P.status, 52)) { ok = false; break; }
        tc_fence_after();
        const uint32_t asrc = ring0 + si * C::STAGE_BYTES, bsrc = asrc + C::A_BYTES;
        const uint32_t alo = (asrc >> 4) | kLbo, blo = (bsrc >> 4) | kLbo;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t adesc = (static_cast<uint64_t>(kDescHi) << 32) | (alo + k * kStep);
          const uint64_t bdesc = (static_cast<uint64_t>(kDescHi) << 32) | (blo + k * kStep);
          umma<2>(tmem_base, adesc, bdesc, P.idesc, (ch != ch_begin || k != 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(si));
        if (++si == SX) { si = 0; sph ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  } else {
    // epilogue: lane = accumulator row k; 32 columns (j) per TMEM load, stored as fp32 partials
    const int q = warp & 3;
    int got = 1;
    if (lane == 0) got = mbar_wait<128>(tfull_bar, 0u, abort_flag, P.status, 53) ? 1 : 0;
    got = __shfl_sync(0xffffffffu, got, 0);
    if (got && ch_end > ch_begin) {
      tc_fence_after();
      const int k = k0 + q * 32 + lane;
      float* row = P.part + ((static_cast<int64_t>(sp) * P.a * P.d + blk) * P.c + k) * P.b + j0;
      const bool vec = (P.b % 4 == 0);
#pragma unroll 1
      for (int cg = 0; cg < NT / 32; ++cg) {
        if (j0 + cg * 32 >= P.b) break;
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + cg * 32, r);
        tmem_ld_wait();
        if (k < P.c) {
          if (vec && j0 + cg * 32 + 32 <= P.b) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(row + cg * 32 + e) =
                  make_float4(__uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                              __uint_as_float(r[e + 3]));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (j0 + cg * 32 + e < P.b) row[cg * 32 + e] = __uint_as_float(r[e]);
          }
        }
      }
    } else if (got) {
      // a split without chunks (more splits than chunks): its partial tile is zero
      const int k = k0 + q * 32 + lane;
      if (k < P.c) {
        float* row = P.part + ((static_cast<int64_t>(sp) * P.a * P.d + blk) * P.c + k) * P.b + j0;
        for (int e = 0; e < NT && j0 + e < P.b; ++e) row[e] = 0.f;
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// sums the partial tiles of the splits in a fixed order and converts to the weights' type
template <typename T>
__global__ void __launch_bounds__(256)
    wgrad_reduce_kernel(const float* __restrict__ part, T* __restrict__ dw, int64_t elems, int splits) {
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; e < elems;
       e += static_cast<int64_t>(gridDim.x) * 256) {
    float s = 0.f;
    for (int q = 0; q < splits; ++q) s += part[q * elems + e];
    dw[e] = ElemTraits<T>::from_float(s);
  }
}

static int wgrad_splits(const Problem& p, int nt) {
  const int64_t tiles = static_cast<int64_t>(p.a) * p.d * ((p.c + 127) / 128) * ((p.b + nt - 1) / nt);
  const int64_t nchunks = (p.batch + 63) / 64;
  int sms = num_sms();
  if (sms <= 0) sms = 148;
  int64_t s = (2 * sms + tiles - 1) / tiles;   // about two CTAs' worth of work per SM
  if (s > nchunks / 8) s = nchunks / 8;        // at least eight chunks per split
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return static_cast<int>(s);
}

static int wgrad_nt(const Problem& p) { return p.b <= 64 ? 64 : (p.b <= 128 ? 128 : 256); }

template <bool BS_LAST, int NT, int SX>
static int launch_w(const Problem& p, const void* grad_out, float* part, int splits, cudaStream_t stream) {
  using C = CfgW<BS_LAST, NT, SX>;
  auto kern = ksmm_tc_wgrad_kernel<BS_LAST, NT, SX>;
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess)
      return set_error(KSMM_ERR_CUDA, "cannot reserve %d bytes of shared memory: %s", C::SMEM_BYTES,
                       cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const uint64_t a = p.a, b = p.b, c = p.c, d = p.d, B = p.batch;
  CUtensorMap tmX, tmG;
  int st;
  if (BS_LAST) {
    const uint64_t xd[4] = {B, d, c, a};
    const uint64_t xs[4] = {1, B, d * B, c * d * B};
    const uint32_t xb[4] = {64, 1, 128, 1};
    if ((st = encode_map(&tmX, p.in_dtype, 4, p.in, xd, xs, xb)) != KSMM_OK) return st;
    const uint64_t gd[4] = {B, d, b, a};
    const uint64_t gs[4] = {1, B, d * B, b * d * B};
    const uint32_t gb[4] = {64, 1, static_cast<uint32_t>(NT), 1};
    if ((st = encode_map(&tmG, p.in_dtype, 4, grad_out, gd, gs, gb)) != KSMM_OK) return st;
  } else {
    const uint64_t xd[3] = {c, a, B};
    const uint64_t xs[3] = {1, c, a * c};
    const uint32_t xb[3] = {64, 1, 64};
    if ((st = encode_map(&tmX, p.in_dtype, 3, p.in, xd, xs, xb)) != KSMM_OK) return st;
    const uint64_t gd[3] = {b, a, B};
    const uint64_t gs[3] = {1, b, a * b};
    const uint32_t gb[3] = {64, 1, 64};
    if ((st = encode_map(&tmG, p.in_dtype, 3, grad_out, gd, gs, gb)) != KSMM_OK) return st;
  }
  ParamsW P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_k = (p.c + 127) / 128;
  P.tiles_j = (p.b + NT - 1) / NT;
  P.splits = splits;
  P.nchunks = static_cast<int>((p.batch + 63) / 64);
  P.part = part;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;
  // fp32 accumulate, M = 128, N = NT; batch-last: both operands K-major; batch-first: both MN-major
  P.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (BS_LAST ? 0u : ((1u << 15) | (1u << 16))) |
            (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  const int64_t grid = static_cast<int64_t>(p.a) * p.d * splits * P.tiles_k * P.tiles_j;
  if (grid <= 0 || grid > 0x7fffffffLL)
    return set_error(KSMM_ERR_UNSUPPORTED, "weight gradient: %lld tiles exceed the grid limit",
                     static_cast<long long>(grid));
  kern<<<static_cast<unsigned>(grid), kThreadsW, C::SMEM_BYTES, stream>>>(tmX, tmG, P);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "weight-gradient kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace tc

// can the tensor-core dW kernel run this problem (p.in = X, p.out = dW; grad_out separately)?
bool wgrad_tc_supported(const Problem& p, const void* grad_out, bool check_pointers) {
  if (p.in_dtype != KSMM_F16 && p.in_dtype != KSMM_BF16) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  if (p.bs_last) {
    if ((p.batch * 2) % 16 != 0) return false;
  } else {
    if (p.d != 1 || (p.c * 2) % 16 != 0 || (p.b * 2) % 16 != 0) return false;
  }
  if (check_pointers &&
      (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(grad_out) % 16))
    return false;
  return true;
}

size_t wgrad_workspace_bytes(const Problem& p) {
  if (!wgrad_tc_supported(p, nullptr, false)) return 0;
  const size_t elems = static_cast<size_t>(p.a) * p.b * p.c * p.d;
  return static_cast<size_t>(tc::wgrad_splits(p, tc::wgrad_nt(p))) * elems * sizeof(float);
}

// p.in = X, p.out = dW (kernel format, input dtype); grad_out = dY
int wgrad_launch(const Problem& p, const void* grad_out, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream) {
  const int64_t elems = static_cast<int64_t>(p.a) * p.b * p.c * p.d;
  if (p.batch == 0) {
    cudaError_t e = cudaMemsetAsync(p.out, 0, elems * dtype_size(p.in_dtype), stream);
    return e == cudaSuccess ? KSMM_OK : set_error(KSMM_ERR_CUDA, "memset failed: %s", cudaGetErrorString(e));
  }
  if (wgrad_tc_supported(p, grad_out, true) && workspace &&
      reinterpret_cast<uintptr_t>(workspace) % 16 == 0 && workspace_bytes >= wgrad_workspace_bytes(p)) {
    const int nt = tc::wgrad_nt(p);
    const int splits = tc::wgrad_splits(p, nt);
    float* part = static_cast<float*>(workspace);
    int st;
    if (p.bs_last)
      st = nt == 64 ? tc::launch_w<true, 64, 8>(p, grad_out, part, splits, stream)
                    : (nt == 128 ? tc::launch_w<true, 128, 6>(p, grad_out, part, splits, stream)
                                 : tc::launch_w<true, 256, 4>(p, grad_out, part, splits, stream));
    else
      st = nt == 64 ? tc::launch_w<false, 64, 8>(p, grad_out, part, splits, stream)
                    : (nt == 128 ? tc::launch_w<false, 128, 6>(p, grad_out, part, splits, stream)
                                 : tc::launch_w<false, 256, 4>(p, grad_out, part, splits, stream));
    if (st != KSMM_OK) return st;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>((elems + 255) / 256, 148 * 8));
    if (p.in_dtype == KSMM_F16)
      tc::wgrad_reduce_kernel<__half><<<grid, 256, 0, stream>>>(part, static_cast<__half*>(p.out), elems, splits);
    else
      tc::wgrad_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(part, static_cast<__nv_bfloat16*>(p.out),
                                                                     elems, splits);
    count_launch();
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
      return set_error(KSMM_ERR_CUDA, "weight-gradient reduction launch failed: %s", cudaGetErrorString(err));
    return KSMM_OK;
  }
  const int64_t nblk = static_cast<int64_t>(p.a) * p.d;
  if (nblk > 65535 || (p.c + 15) / 16 > 65535)
    return set_error(KSMM_ERR_UNSUPPORTED, "weight gradient: too many blocks for the fallback kernel");
  dim3 grid((p.b + 15) / 16, (p.c + 15) / 16, static_cast<unsigned>(nblk));
  if (p.in_dtype == KSMM_F32)
    wgrad_simt_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(p.in),
                                                       static_cast<const float*>(grad_out),
                                                       static_cast<float*>(p.out), p.batch, p.a, p.b, p.c, p.d,
                                                       p.bs_last);
  else if (p.in_dtype == KSMM_F16)
    wgrad_simt_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(p.in),
                                                        static_cast<const __half*>(grad_out),
                                                        static_cast<__half*>(p.out), p.batch, p.a, p.b, p.c, p.d,
                                                        p.bs_last);
  else if (p.in_dtype == KSMM_BF16)
    wgrad_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p.in), static_cast<const __nv_bfloat16*>(grad_out),
        static_cast<__nv_bfloat16*>(p.out), p.batch, p.a, p.b, p.c, p.d, p.bs_last);
  else
    return set_error(KSMM_ERR_UNSUPPORTED, "weight gradients exist for fp32, fp16 and bf16");
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "weight-gradient kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace ksmm
