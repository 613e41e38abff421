// tcgen05 kernel for batch-first factors with d = 2 or 4 (16-bit) whose input has
// been regrouped by block: X'[n, (i, l, k)] instead of X[n, (i, k, l)].
//
// With the d blocks of a block row stored one after the other, the input tile
// of block (i, l) is a plain K-major TMA tile, so the transposer stage of
// tc_bsfirst_d.cu and two of its four hand-offs per chunk disappear, and a
// chunk carries eight MMAs instead of four.  The output is the natural
// batch-first layout: the d accumulators of a block row live side by side in
// TMEM and the epilogue interleaves them (l fastest) into contiguous row
// segments, exactly as in tc_bsfirst_d.cu.
//
// One stage holds the input tiles of two blocks l (2 x 128 rows x 64 k) and their
// weights (2 x 64 k x NJ); a row tile takes (d / 2) * ceil(c / 64) chunks.  Who
// regroups the input: the factor before it in a chain (the epilogue of the d = 1
// kernel can store in this order, which is how chains use this kernel) or the
// small regrouping kernel in this file (configuration 1 of a single factor; the
// extra pass costs more than the kernel saves, so it is not the default).
// Measured for (1,768,192,4) fp16 at 25088 rows inside a chain: 66 us against 85 us
// for tc_bsfirst_d.cu.  The input tile is re-read once per j tile and the weights
// once per row tile, both from L2 (about 460 MB in all): that traffic, not the
// hand-offs, is what bounds this kernel.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 TMEM owner and MMA
// issuer, warps 2..9 epilogue (TMEM lane quarter = warp index mod 4).  Bounded
// waits and status reporting are as in tc_kernel.cu.
//
// Reference counterpart: kernel_bs_first_half
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_half.cuh:107-620).
#include <cuda.h>

#include <atomic>

#include "tc_host.h"
#include "tc_kernel.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace tc {

struct ParamsP {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  uint32_t rows;        // a * tiles_n: (block row, batch tile) pairs
  uint32_t row_groups;  // CTAs per j tile
  int nkc;              // ceil(c / 64) k chunks per block
  uint32_t idesc;
  float alpha;
  const void* bias;
  int out_dtype;
  int act;  // ksmm_activation_t
  int* status;
};

constexpr int kThreadsP = (2 + kEpilogueWarps) * 32;

template <int D, int NJ_, int ST_, int STGN>
struct CfgP {
  static constexpr int NJ = NJ_;                    // j columns per accumulator (64 or 128)
  static constexpr int ST = ST_;
  static constexpr int AL_BYTES = 128 * 128;        // one block's input tile: 128 rows x 64 k
  static constexpr int A_BYTES = 2 * AL_BYTES;      // two blocks per stage
  static constexpr int WL_BYTES = 64 * 128;         // one block's 64 k rows x 64 j
  static constexpr int WJB_BYTES = 2 * WL_BYTES;    // one TMA box: two blocks
  static constexpr int W_BYTES = (NJ / 64) * WJB_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  static constexpr int STG_TILE_BYTES = 32 * 128;   // 32 rows x 64 output elements
  static constexpr int STG_WARP_BYTES = STGN * STG_TILE_BYTES;
  static constexpr int STG_BYTES = kEpilogueWarps * STG_WARP_BYTES;
  static constexpr int NBAR = 2 * ST + 4;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STG_BYTES + ST * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int BUF_COLS = D * NJ;           // d accumulators side by side
  static constexpr int NBUF = BUF_COLS <= 256 ? 2 : 1;
  static constexpr int TMEM_COLS = 512;
  static_assert(NJ == 64 || NJ == 128, "j tile");
  static_assert(D == 2 || D == 4, "d = 2 or 4");
  static_assert(BUF_COLS <= 512, "TMEM capacity");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM, so that the TMEM allocation never waits");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
};

template <int D, int NJ_, int ST_, int STGN>
__global__ void __launch_bounds__(kThreadsP, 1)
    ksmm_tc_bsfirst_dp_kernel(const __grid_constant__ CUtensorMap tmX,
                              const __grid_constant__ CUtensorMap tmW,
                              const __grid_constant__ CUtensorMap tmY, const ParamsP P) {
  using C = CfgP<D, NJ_, ST_, STGN>;
  constexpr int ST = C::ST;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t stg0 = sm0;                     // epilogue staging tiles
  const uint32_t stage0 = stg0 + C::STG_BYTES;   // [input tiles of two blocks | their weights]
  const uint32_t bar0 = stage0 + ST * C::STAGE_BYTES;
  uint8_t* bar_gen = sm_gen + (bar0 - sm0);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto free_bar = [&](int s) { return bar0 + 8u * (ST + s); };
  auto tfull_bar = [&](int q) { return bar0 + 8u * (2 * ST + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (2 * ST + 2 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(free_bar(s), 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(tfull_bar(q), 1);
      mbar_init(tempty_bar(q), kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmX);
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmY);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above overlaps the tail of the previous kernel in the stream; memory comes after this
  grid_dep_wait();
  grid_dep_launch();

  const int nkc = P.nkc;
  const int tj = static_cast<int>(blockIdx.x % P.tiles_j);
  const uint32_t rc = blockIdx.x / P.tiles_j;
  const uint32_t row_begin = static_cast<uint32_t>(static_cast<uint64_t>(rc) * P.rows / P.row_groups);
  const uint32_t row_end = static_cast<uint32_t>(static_cast<uint64_t>(rc + 1) * P.rows / P.row_groups);
  const int j0 = tj * C::NJ;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0;
      bool ok = true;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        const int i = static_cast<int>(row / P.tiles_n);
        const int n0 = static_cast<int>(row % P.tiles_n) * 128;
        for (int lp = 0; lp < D / 2 && ok; ++lp) {
          for (int kc = 0; kc < nkc; ++kc) {
            if (!mbar_wait<64>(free_bar(si), sph ^ 1u, abort_flag, P.status, 51)) { ok = false; break; }
            const uint32_t sb = stage0 + si * C::STAGE_BYTES;
            mbar_expect_tx(full_bar(si), C::STAGE_BYTES);
            // regrouped input seen as (k, n, l, i): two tiles of 128 rows x 64 k
            tma_load_4d(sb, &tmX, full_bar(si), kc * 64, n0, lp * 2, i);
            // weights (a*d*c, b) seen as (b, c, a*d): per 64 columns, two blocks of 64 k rows
#pragma unroll
            for (int jb = 0; jb < C::NJ / 64; ++jb)
              tma_load_3d(sb + C::A_BYTES + jb * C::WJB_BYTES, &tmW, full_bar(si), j0 + jb * 64, kc * 64,
                          i * D + lp * 2);
            if (++si == ST) { si = 0; sph ^= 1u; }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0, ut = 0;
      bool ok = true;
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
        if (!mbar_wait<0>(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 52)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dcol = tmem_base + buf * C::BUF_COLS;
        for (int lp = 0; lp < D / 2 && ok; ++lp) {
          for (int kc = 0; kc < nkc; ++kc) {
            if (!mbar_wait<0>(full_bar(si), sph, abort_flag, P.status, 53)) { ok = false; break; }
            tc_fence_after();
            const uint32_t ab = stage0 + si * C::STAGE_BYTES, wb = ab + C::A_BYTES;
#pragma unroll
            for (int l2 = 0; l2 < 2; ++l2) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                // input tile: K-major rows of 64 k, 128-byte swizzle; a k step is 32 bytes in the row
                const uint64_t adesc = make_desc(ab + l2 * C::AL_BYTES + ks * 32, 16, 1024, 2);
                // weights: MN-major, 128-byte swizzle; LBO = next 64-j box, SBO = next 8 k rows
                const uint64_t bdesc = make_desc(wb + l2 * C::WL_BYTES + ks * 2048, C::WJB_BYTES, 1024, 2);
                umma<2>(dcol + (lp * 2 + l2) * C::NJ, adesc, bdesc, P.idesc, (kc | ks) != 0 ? 1u : 0u);
              }
            }
            umma_commit(free_bar(si));
            if (++si == ST) { si = 0; sph ^= 1u; }
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    const int ew = warp - 2;
    const int q = warp & 3;
    const int grp = ew >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool plain = (P.alpha == 1.f) && (P.bias == nullptr) && (P.act == 0);
    const uint32_t stg = stg0 + ew * C::STG_WARP_BYTES;
    constexpr int JB = 64 / D;  // j values in one 64-element output box
    uint32_t ut = 0, sti = 0;
    KSMM_TRACE_DECL;
    const bool etron = ew == 0 && lane == 0;
    for (uint32_t row = row_begin; row < row_end; ++row, ++ut) {
      const int i = static_cast<int>(row / P.tiles_n);
      const int n0 = static_cast<int>(row % P.tiles_n) * 128;
      const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
      int got = 1;
      if (etron) KSMM_TRACE(3, 20);
      if (lane == 0) got = mbar_wait<128>(tfull_bar(buf), bph, abort_flag, P.status, 17) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      if (etron) KSMM_TRACE(3, 21);
      tc_fence_after();
      const bool warp_active = n0 + q * 32 < P.batch;
      int jlim = P.b - j0;  // j columns of this tile that exist
      if (jlim > C::NJ) jlim = C::NJ;
      // iterations of this warp: cb = grp, grp + 2, ... while cb * JB < jlim
      int n_it = warp_active ? ((jlim + JB - 1) / JB - grp + 1) / 2 : 0;
      bool released = false;
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int cb = grp + 2 * it;
        const int jj0 = cb * JB;
        uint32_t r[D][JB];
#pragma unroll
        for (int l = 0; l < D; ++l) {
          const uint32_t ta = tmem_base + lane_addr + buf * C::BUF_COLS + l * C::NJ + jj0;
          if constexpr (JB == 16) {
            tmem_ld16(ta, r[l]);
          } else {
            tmem_ld32(ta, r[l]);
          }
        }
        tmem_ld_wait();
        if (it == n_it - 1) {
          // the accumulators are in registers: the MMA warp may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(buf));
          released = true;
        }
        if (!plain) {
          // bias of the 64 output elements (jj, l) of this tile: one coalesced 4-byte load per lane
          // (elements 2 lane and 2 lane + 1), then broadcast by shuffle
          uint32_t bpair = 0;
          if (P.bias != nullptr) {
            const int64_t e0 = (static_cast<int64_t>(i) * P.b + j0 + jj0) * D + 2 * lane;
            if (j0 + jj0 + (2 * lane) / D < P.b) {
              const uint16_t* bp = static_cast<const uint16_t*>(P.bias) + e0;
              bpair = (reinterpret_cast<uintptr_t>(bp) & 3) == 0
                          ? *reinterpret_cast<const uint32_t*>(bp)
                          : (static_cast<uint32_t>(bp[0]) | (static_cast<uint32_t>(bp[1]) << 16));
            }
          }
#pragma unroll
          for (int jj = 0; jj < JB; ++jj)
#pragma unroll
            for (int l = 0; l < D; ++l) {
              const int e = jj * D + l;
              const uint32_t pr = __shfl_sync(0xffffffffu, bpair, e >> 1);
              const uint16_t hv = static_cast<uint16_t>((e & 1) ? (pr >> 16) : (pr & 0xffffu));
              const float bv = P.out_dtype == KSMM_BF16 ? __uint_as_float(static_cast<uint32_t>(hv) << 16)
                                                        : __half2float(__ushort_as_half(hv));
              r[l][jj] = __float_as_uint(fmaf(P.alpha, __uint_as_float(r[l][jj]), bv));
            }
          if (P.act == KSMM_ACT_GELU) {
#pragma unroll
            for (int l = 0; l < D; ++l)
#pragma unroll
              for (int jj = 0; jj < JB; ++jj) r[l][jj] = __float_as_uint(gelu_16bit(__uint_as_float(r[l][jj])));
          } else if (P.act == KSMM_ACT_RELU) {
#pragma unroll
            for (int l = 0; l < D; ++l)
#pragma unroll
              for (int jj = 0; jj < JB; ++jj) r[l][jj] = __float_as_uint(fmaxf(__uint_as_float(r[l][jj]), 0.f));
          }
        }
        // the staging tile about to be written must have been read by its last store
        if (lane == 0) bulk_wait_read<STGN - 1>();
        __syncwarp();
        // output element (jj, l) sits at jj * D + l: words pair (l, l + 1) of one jj
        const uint32_t tile = stg + (STGN > 1 ? (sti * C::STG_TILE_BYTES) : 0u);
        const uint32_t rowaddr = tile + lane * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int widx = ch * 4 + e;           // word index within the 128-byte row
            const int jj = widx / (D / 2);
            const int l = (widx % (D / 2)) * 2;
            w[e] = pack2(__uint_as_float(r[l][jj]), __uint_as_float(r[l + 1][jj]), P.out_dtype);
          }
          const uint32_t chunk = static_cast<uint32_t>(ch ^ (lane & 7));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + chunk * 16),
                       "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmY, tile, (j0 + jj0) * D, i, n0 + q * 32);
          bulk_commit();
        }
        if (STGN > 1) sti = (sti + 1 == STGN) ? 0u : sti + 1;
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
      }
      if (etron) KSMM_TRACE(3, 27);
    }
    if (lane == 0) bulk_wait<0>();
    __syncwarp();
  }

  // ===================== teardown =====================
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


template <int D, int NJ_, int ST_, int STGN>
static int launch_p(const Problem& p, const void* regrouped, cudaStream_t stream) {
  using C = CfgP<D, NJ_, ST_, STGN>;
  auto kern = ksmm_tc_bsfirst_dp_kernel<D, NJ_, ST_, STGN>;
  static std::atomic<bool> attr_set[64];  // zero-initialised; set once per device (a repeated set is harmless)
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess)
      return set_error(KSMM_ERR_CUDA, "cannot reserve %d bytes of shared memory: %s",
                       C::SMEM_BYTES, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const uint64_t a = p.a, b = p.b, c = p.c, d = p.d, B = p.batch;
  CUtensorMap tmX, tmW, tmY;
  int st;
  {
    // regrouped input [n][i][l][k] seen as (k, n, l, i): box = two tiles of 128 rows x 64 k
    const uint64_t dims[4] = {c, B, d, a};
    const uint64_t str[4] = {1, a * c * d, c, c * d};
    const uint32_t box[4] = {64, 128, 2, 1};
    if ((st = encode_map(&tmX, p.in_dtype, 4, regrouped, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // weights (a*d*c, b) row-major seen as (b, c, a*d); box = 64 j x 64 k rows x two blocks
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {64, 64, 2};
    if ((st = encode_map(&tmW, p.in_dtype, 3, p.w, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // output rows: (b*d, a, batch); one epilogue warp stores 64 elements x 32 rows
    const uint64_t dims[3] = {b * d, a, B};
    const uint64_t str[3] = {1, b * d, a * b * d};
    const uint32_t box[3] = {64, 1, 32};
    if ((st = encode_map(&tmY, p.out_dtype, 3, p.out, dims, str, box, true)) != KSMM_OK) return st;
  }
  ParamsP P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + 127) / 128);
  P.tiles_j = static_cast<int>((b + C::NJ - 1) / C::NJ);
  P.nkc = (p.c + 63) / 64;
  P.alpha = p.alpha;
  P.bias = p.bias;
  P.out_dtype = p.out_dtype;
  P.act = p.activation;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;
  // fp32 accumulate, A K-major, B MN-major, N = NJ, M = 128
  P.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) |
            (static_cast<uint32_t>(C::NJ >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  const int sms = num_sms();
  if (sms <= 0) return set_error(KSMM_ERR_NO_DEVICE, "no CUDA device");
  const int64_t rows = static_cast<int64_t>(P.tiles_n) * p.a;
  if (rows <= 0 || rows > 0x7fffffffLL || P.tiles_j > sms)
    return set_error(KSMM_ERR_UNSUPPORTED, "tensor-core family: work-split limits exceeded");
  P.rows = static_cast<uint32_t>(rows);
  int64_t groups = sms / P.tiles_j;
  if (groups > rows) groups = rows;
  P.row_groups = static_cast<uint32_t>(groups);
  const unsigned grid = static_cast<unsigned>(groups * P.tiles_j);
  cudaError_t err = launch_pdl(kern, grid, kThreadsP, C::SMEM_BYTES, stream, tmX, tmW, tmY, P);
  count_launch();
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

// out[n, (i*d + l)*c + k] = in[n, (i*c + k)*d + l] for 2-byte elements: one CTA moves the c*d
// elements of one block row of 8 batch entries through shared memory (16-byte global accesses).
template <int D>
__global__ void __launch_bounds__(256)
    regroup_by_block_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int64_t batch,
                            int a, int c) {
  extern __shared__ uint16_t seg[];  // [8 rows][c * D]
  const int cd = c * D;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 8;
  const int i = blockIdx.y;
  const int64_t row_elems = static_cast<int64_t>(a) * cd;
  const int vec_per_row = cd / 8;
  for (int v = threadIdx.x; v < 8 * vec_per_row; v += 256) {
    const int r = v / vec_per_row, q = v % vec_per_row;
    if (n0 + r < batch)
      *reinterpret_cast<uint4*>(seg + r * cd + q * 8) =
          *reinterpret_cast<const uint4*>(in + (n0 + r) * row_elems + static_cast<int64_t>(i) * cd + q * 8);
  }
  __syncthreads();
  for (int v = threadIdx.x; v < 8 * vec_per_row; v += 256) {
    const int r = v / vec_per_row, q = v % vec_per_row;  // output vector q: block l, k = k0 .. k0 + 7
    const int l = (q * 8) / c, k0 = (q * 8) % c;
    if (n0 + r < batch) {
      uint16_t e[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) e[t] = seg[r * cd + (k0 + t) * D + l];
      uint4 pk;
      pk.x = e[0] | (static_cast<uint32_t>(e[1]) << 16);
      pk.y = e[2] | (static_cast<uint32_t>(e[3]) << 16);
      pk.z = e[4] | (static_cast<uint32_t>(e[5]) << 16);
      pk.w = e[6] | (static_cast<uint32_t>(e[7]) << 16);
      *reinterpret_cast<uint4*>(out + (n0 + r) * row_elems + static_cast<int64_t>(i) * cd + q * 8) = pk;
    }
  }
}

}  // namespace tc

bool tc_bsfirst_dp_supported(const Problem& p, bool check_pointers) {
  if (!tc_bsfirst_d_supported(p, check_pointers)) return false;
  // 16-byte pieces of the regrouped rows must not straddle blocks; one block row fits in shared memory
  return p.c % 8 == 0 && static_cast<int64_t>(p.c) * p.d <= 3072 && p.batch <= 8LL * 0x7fffffff &&
         p.a <= 65535;
}

size_t tc_bsfirst_dp_scratch_bytes(const Problem& p) {
  if (p.in_regrouped) return 0;
  const size_t bytes = static_cast<size_t>(p.batch) * p.a * p.c * p.d * 2;
  return (bytes + 255) / 256 * 256;
}

int tc_bsfirst_dp_launch(const Problem& p, cudaStream_t stream) {
  if (p.in_regrouped) {
    // a chain's previous factor stored its output in this order already
    if (p.d == 4)
      return p.b > 64 ? tc::launch_p<4, 128, 3, 1>(p, p.in, stream) : tc::launch_p<4, 64, 4, 1>(p, p.in, stream);
    return p.b > 64 ? tc::launch_p<2, 128, 3, 1>(p, p.in, stream) : tc::launch_p<2, 64, 4, 1>(p, p.in, stream);
  }
  // 1. regroup the input by block into the scratch
  void* scratch = nullptr;
  int st = layout_scratch(p, tc_bsfirst_dp_scratch_bytes(p), stream, &scratch);
  if (st != KSMM_OK) return st;
  {
    const dim3 grid(static_cast<unsigned>((p.batch + 7) / 8), static_cast<unsigned>(p.a));
    const size_t smem = static_cast<size_t>(8) * p.c * p.d * 2;
    auto in = static_cast<const uint16_t*>(p.in);
    auto out = static_cast<uint16_t*>(scratch);
    if (p.d == 4)
      tc::regroup_by_block_kernel<4><<<grid, 256, smem, stream>>>(in, out, p.batch, p.a, p.c);
    else
      tc::regroup_by_block_kernel<2><<<grid, 256, smem, stream>>>(in, out, p.batch, p.a, p.c);
    count_launch();
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
      return set_error(KSMM_ERR_CUDA, "regrouping kernel launch failed: %s", cudaGetErrorString(err));
  }
  // 2. <d, j tile, stages, staging tiles per epilogue warp>
  if (p.d == 4)
    return p.b > 64 ? tc::launch_p<4, 128, 3, 1>(p, scratch, stream) : tc::launch_p<4, 64, 4, 1>(p, scratch, stream);
  return p.b > 64 ? tc::launch_p<2, 128, 3, 1>(p, scratch, stream) : tc::launch_p<2, 64, 4, 1>(p, scratch, stream);
}

}  // namespace ksmm
