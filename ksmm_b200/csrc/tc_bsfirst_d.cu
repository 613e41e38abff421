// tcgen05 kernel for batch-first factors with d > 1 (16-bit inputs, d = 2 or 4).
//
// In the batch-first layout a row of the input holds, for one block row i_a,
// the c*d values x[n, i_a, k, l] with l fastest.  Block (i_a, l) contracts over
// k at a stride of d elements, which neither TMA (16-byte granularity) nor a
// UMMA operand descriptor can express.  This kernel therefore
//   1. fetches the contiguous 128-byte pieces of 128 input rows with TMA
//      ("raw" chunk: 64 elements = 64/d values of k for each of the d blocks),
//   2. lets four "transposer" warps split the chunk by l into d K-major operand
//      tiles in shared memory (16-byte loads, byte permutes, 4/8-byte stores),
//   3. issues, per chunk, d MMAs of 128 (batch rows) x 64 (j) into d
//      accumulators that live side by side in TMEM, and
//   4. in the epilogue interleaves the d accumulators back (l fastest), so that
//      every output row segment is contiguous and leaves through TMA stores.
// All d blocks of a block row are therefore handled by one CTA, the input is
// read in full 128-byte lines and the output is written in full lines; the
// reference instead issues 2-byte accesses at stride d
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_half.cuh:402-413, 609-618).
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 TMEM owner and MMA
// issuer, warps 2..5 transposers, warps 6..13 epilogue (TMEM lane quarter =
// warp index mod 4).  Work split, weight-stationary / streaming flavours,
// bounded waits and status reporting are as in tc_kernel.cu.
#include <cuda.h>

#include "tc_host.h"
#include "tc_kernel.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace tc {

struct ParamsD {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  uint32_t rows;        // a * tiles_n: (block row, batch tile) pairs
  uint32_t row_groups;  // CTAs per j tile
  int nchunks;          // ceil(c * d / 64) raw chunks per row
  uint32_t idesc;
  float alpha;
  const void* bias;
  int out_dtype;
  int* status;
};

constexpr int kThreadsD = (2 + 4 + kEpilogueWarps) * 32;

template <int D, int NJ_, bool WRES, int NWC, int SX>
struct CfgD {
  static constexpr int NJ = NJ_;                    // j columns per accumulator (64 or 128)
  static constexpr int KCL = 64 / D;                // k values per block in one raw chunk
  static constexpr int RAW_BYTES = 128 * 128;       // 128 rows x 64 elements
  static constexpr int A_BYTES = 128 * 128;         // d tiles of 128 rows x KCL elements
  static constexpr int AL_BYTES = A_BYTES / D;      // one block's tile
  static constexpr int WBOX_BYTES = KCL * 128;      // one weight box: KCL rows x 64 j
  static constexpr int WL_BYTES = (NJ / 64) * WBOX_BYTES;  // one block's weights for one raw chunk
  static constexpr int WCH_BYTES = D * WL_BYTES;    // weights that go with one raw chunk
  static constexpr int STAGE_BYTES = RAW_BYTES + A_BYTES + (WRES ? 0 : WCH_BYTES);
  static constexpr int STG_WARP_BYTES = 32 * 128;
  static constexpr int STG_BYTES = kEpilogueWarps * STG_WARP_BYTES;
  static constexpr int NBAR = 3 * SX + 2 + 4;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = NWC * WCH_BYTES + SX * STAGE_BYTES + STG_BYTES + BAR_BYTES + 1024;
  static constexpr int BUF_COLS = D * NJ;           // d accumulators side by side
  static constexpr int NBUF = BUF_COLS <= 256 ? 2 : 1;  // double-buffered when TMEM has room
  static constexpr int TMEM_COLS = 512;
  static_assert(NJ == 64 || NJ == 128, "j tile");
  static_assert(BUF_COLS <= 512, "TMEM capacity");
  static_assert(D == 2 || D == 4, "d = 2 or 4");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM, so that the TMEM allocation never waits");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
};

template <int D, int NJ_, bool WRES, int NWC, int SX>
__global__ void __launch_bounds__(kThreadsD, 1)
    ksmm_tc_bsfirst_d_kernel(const __grid_constant__ CUtensorMap tmX,
                             const __grid_constant__ CUtensorMap tmW,
                             const __grid_constant__ CUtensorMap tmY, const ParamsD P) {
  using C = CfgD<D, NJ_, WRES, NWC, SX>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t wres0 = sm0;                          // resident weights (weight-stationary)
  const uint32_t ring0 = wres0 + NWC * C::WCH_BYTES;   // stages: raw chunk, operand tiles, (weights)
  const uint32_t stg0 = ring0 + SX * C::STAGE_BYTES;
  const uint32_t bar0 = stg0 + C::STG_BYTES;
  uint8_t* bar_gen = sm_gen + NWC * C::WCH_BYTES + SX * C::STAGE_BYTES + C::STG_BYTES;
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto a_full = [&](int s) { return bar0 + 8u * (SX + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (2 * SX + s); };
  const uint32_t wfull_bar = bar0 + 8u * (3 * SX);
  const uint32_t wempty_bar = bar0 + 8u * (3 * SX + 1);
  auto tfull_bar = [&](int q) { return bar0 + 8u * (3 * SX + 2 + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (3 * SX + 4 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SX; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(a_full(s), 4);  // one arrival per transposer warp
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(wfull_bar, 1);
    mbar_init(wempty_bar, 1);
    for (int q = 0; q < 2; ++q) {
      mbar_init(tfull_bar(q), 1);
      mbar_init(tempty_bar(q), kEpilogueWarps);
    }
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

  const int nchunks = P.nchunks;
  const int tj = static_cast<int>(blockIdx.x % P.tiles_j);
  const uint32_t rc = blockIdx.x / P.tiles_j;
  const uint32_t row_begin = static_cast<uint32_t>(static_cast<uint64_t>(rc) * P.rows / P.row_groups);
  const uint32_t row_end = static_cast<uint32_t>(static_cast<uint64_t>(rc + 1) * P.rows / P.row_groups);
  const int j0 = tj * C::NJ;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0, wph = 0;
      int cur_i = -1;
      bool ok = true;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        const int i = static_cast<int>(row / P.tiles_n);
        const int n0 = static_cast<int>(row % P.tiles_n) * 128;
        if (WRES && i != cur_i) {
          if (!mbar_wait<64>(wempty_bar, wph ^ 1u, abort_flag, P.status, 11)) { ok = false; break; }
          wph ^= 1u;
          mbar_expect_tx(wfull_bar, nchunks * C::WCH_BYTES);
          for (int qc = 0; qc < nchunks; ++qc)
#pragma unroll
            for (int l = 0; l < D; ++l)
#pragma unroll
              for (int jb = 0; jb < C::NJ / 64; ++jb)
                tma_load_3d(wres0 + qc * C::WCH_BYTES + l * C::WL_BYTES + jb * C::WBOX_BYTES, &tmW,
                            wfull_bar, j0 + jb * 64, qc * C::KCL, i * D + l);
          cur_i = i;
        }
        for (int qc = 0; qc < nchunks; ++qc) {
          if (!mbar_wait<64>(empty_bar(si), sph ^ 1u, abort_flag, P.status, 12)) { ok = false; break; }
          const uint32_t dst = ring0 + si * C::STAGE_BYTES;
          const uint32_t bar = raw_full(si);
          mbar_expect_tx(bar, C::RAW_BYTES + (WRES ? 0 : C::WCH_BYTES));
          tma_load_3d(dst, &tmX, bar, qc * 64, i, n0);
          if constexpr (!WRES) {
#pragma unroll
            for (int l = 0; l < D; ++l)
#pragma unroll
              for (int jb = 0; jb < C::NJ / 64; ++jb)
                tma_load_3d(dst + C::RAW_BYTES + C::A_BYTES + l * C::WL_BYTES + jb * C::WBOX_BYTES,
                            &tmW, bar, j0 + jb * 64, qc * C::KCL, i * D + l);
          }
          if (++si == SX) { si = 0; sph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0, wph = 0, ut = 0;
      int cur_i = -1;
      bool ok = true;
      // operand tiles written by the transposers: K-major, no swizzle, core matrices of
      // 8 rows x 16 bytes; LBO = 128 bytes between the core matrices of one MMA along k,
      // SBO = (KCL / 8) * 128 bytes between groups of 8 rows
      constexpr uint32_t kASbo = (C::KCL / 8) * 128;
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        const int i = static_cast<int>(row / P.tiles_n);
        if (WRES && i != cur_i) {
          if (!mbar_wait<0>(wfull_bar, wph, abort_flag, P.status, 13)) { ok = false; break; }
          wph ^= 1u;
          cur_i = i;
        }
        const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
        if (!mbar_wait<0>(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 14)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dcol = tmem_base + buf * C::BUF_COLS;
        for (int qc = 0; qc < nchunks; ++qc) {
          if (!mbar_wait<0>(a_full(si), sph, abort_flag, P.status, 15)) { ok = false; break; }
          tc_fence_after();
          const uint32_t abase = ring0 + si * C::STAGE_BYTES + C::RAW_BYTES;
          const uint32_t wbase = WRES ? wres0 + qc * C::WCH_BYTES : abase + C::A_BYTES;
#pragma unroll
          for (int ks = 0; ks < C::KCL / 16; ++ks) {
#pragma unroll
            for (int l = 0; l < D; ++l) {
              const uint64_t adesc = make_desc(abase + l * C::AL_BYTES + ks * 256, 128, kASbo, 0);
              // weights: MN-major, 128-byte swizzle; LBO = next 64-j box, SBO = next 8 k rows
              const uint64_t bdesc =
                  make_desc(wbase + l * C::WL_BYTES + ks * 2048, C::WBOX_BYTES, 1024, 2);
              umma<2>(dcol + l * C::NJ, adesc, bdesc, P.idesc, (qc | ks) != 0 ? 1u : 0u);
            }
          }
          umma_commit(empty_bar(si));
          if (++si == SX) { si = 0; sph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));
        if (WRES && (row + 1 == row_end || static_cast<int>((row + 1) / P.tiles_n) != i))
          umma_commit(wempty_bar);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ===================== transposers =====================
    // Thread t handles the 16-byte pieces t, t + 128, ... of the raw chunk
    // (piece = row m, position p within the row).  A piece holds 8/d values of
    // k for each of the d blocks, l fastest; they are regrouped by block and
    // stored into that block's K-major tile.
    const int tt = (warp - 2) * 32 + lane;
    uint32_t si = 0, sph = 0;
    bool ok = true;
    for (uint32_t row = row_begin; row < row_end && ok; ++row) {
      for (int qc = 0; qc < nchunks; ++qc) {
        int got = 1;
        if (lane == 0) got = mbar_wait<32>(raw_full(si), sph, abort_flag, P.status, 16) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        const uint32_t rbase = ring0 + si * C::STAGE_BYTES;
        const uint32_t abase = rbase + C::RAW_BYTES;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int pq = tt + it * 128;
          const int m = pq >> 3, p = pq & 7;
          uint32_t w0, w1, w2, w3;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                       : "r"(rbase + m * 128 + p * 16)
                       : "memory");
          if constexpr (D == 4) {
            // piece = (k0: l0 l1 | l2 l3), (k1: l0 l1 | l2 l3); k0 = 2p
            const uint32_t o0 = __byte_perm(w0, w2, 0x5410);  // l0: k0, k1
            const uint32_t o1 = __byte_perm(w0, w2, 0x7632);  // l1
            const uint32_t o2 = __byte_perm(w1, w3, 0x5410);  // l2
            const uint32_t o3 = __byte_perm(w1, w3, 0x7632);  // l3
            // k = 2p: core column (2p) / 8 = p / 4, byte offset ((2p) % 8) * 2 = (p % 4) * 4
            const uint32_t off = (m >> 3) * ((C::KCL / 8) * 128) + (p >> 2) * 128 + (m & 7) * 16 +
                                 (p & 3) * 4;
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(abase + 0 * C::AL_BYTES + off), "r"(o0) : "memory");
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(abase + 1 * C::AL_BYTES + off), "r"(o1) : "memory");
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(abase + 2 * C::AL_BYTES + off), "r"(o2) : "memory");
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(abase + 3 * C::AL_BYTES + off), "r"(o3) : "memory");
          } else {
            // piece = (k0: l0 l1), (k1: l0 l1), (k2: l0 l1), (k3: l0 l1); k0 = 4p
            const uint32_t a0 = __byte_perm(w0, w1, 0x5410), a1 = __byte_perm(w2, w3, 0x5410);  // l0
            const uint32_t b0 = __byte_perm(w0, w1, 0x7632), b1 = __byte_perm(w2, w3, 0x7632);  // l1
            // k = 4p: core column p / 2, byte offset ((4p) % 8) * 2 = (p % 2) * 8
            const uint32_t off = (m >> 3) * ((C::KCL / 8) * 128) + (p >> 1) * 128 + (m & 7) * 16 +
                                 (p & 1) * 8;
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(abase + 0 * C::AL_BYTES + off), "r"(a0), "r"(a1) : "memory");
            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(abase + 1 * C::AL_BYTES + off), "r"(b0), "r"(b1) : "memory");
          }
        }
        fence_proxy_async();  // the tiles are read by the tensor core through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(si));
        if (++si == SX) { si = 0; sph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    const int ew = warp - 6;
    const int q = warp & 3;
    const int grp = ew >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool plain = (P.alpha == 1.f) && (P.bias == nullptr);
    const uint32_t stg = stg0 + ew * C::STG_WARP_BYTES;
    constexpr int JB = 64 / D;  // j values in one 64-element output box
    uint32_t ut = 0;
    for (uint32_t row = row_begin; row < row_end; ++row, ++ut) {
      const int i = static_cast<int>(row / P.tiles_n);
      const int n0 = static_cast<int>(row % P.tiles_n) * 128;
      const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
      int got = 1;
      if (lane == 0) got = mbar_wait<128>(tfull_bar(buf), bph, abort_flag, P.status, 17) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      const bool warp_active = n0 + q * 32 < P.batch;
      if (warp_active) {
#pragma unroll 1
        for (int cb = grp; cb < C::BUF_COLS / 64; cb += kEpilogueWarps / 4) {
          const int jj0 = cb * JB;
          if (j0 + jj0 >= P.b) break;
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
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
          if (!plain) {
#pragma unroll
            for (int l = 0; l < D; ++l)
#pragma unroll
              for (int jj = 0; jj < JB; ++jj) {
                float bv = 0.f;
                if (P.bias != nullptr && j0 + jj0 + jj < P.b)
                  bv = bias_at(P.bias, (static_cast<int64_t>(i) * P.b + j0 + jj0 + jj) * D + l,
                               P.out_dtype);
                r[l][jj] = __float_as_uint(fmaf(P.alpha, __uint_as_float(r[l][jj]), bv));
              }
          }
          // output element (jj, l) sits at jj * D + l: words pair (l, l + 1) of one jj
          const uint32_t rowaddr = stg + lane * 128;
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
            tma_store_3d(&tmY, stg, (j0 + jj0) * D, i, n0 + q * 32);
            bulk_commit();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
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

template <int D, int NJ_, bool WRES, int NWC, int SX>
static int launch_d(const Problem& p, cudaStream_t stream) {
  using C = CfgD<D, NJ_, WRES, NWC, SX>;
  auto kern = ksmm_tc_bsfirst_d_kernel<D, NJ_, WRES, NWC, SX>;
  static bool attr_set[64] = {false};
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
    // input rows: (c*d, a, batch); raw chunk = 64 contiguous elements of 128 rows, no swizzle
    const uint64_t dims[3] = {c * d, a, B};
    const uint64_t str[3] = {1, c * d, a * c * d};
    const uint32_t box[3] = {64, 1, 128};
    if ((st = encode_map(&tmX, p.in_dtype, 3, p.in, dims, str, box, false)) != KSMM_OK) return st;
  }
  {
    // weights (a*d*c, b) row-major seen as (b, c, a*d); box = 64 j x KCL k rows of one block
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {64, static_cast<uint32_t>(C::KCL), 1};
    if ((st = encode_map(&tmW, p.in_dtype, 3, p.w, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // output rows: (b*d, a, batch); one epilogue warp stores 64 elements x 32 rows
    const uint64_t dims[3] = {b * d, a, B};
    const uint64_t str[3] = {1, b * d, a * b * d};
    const uint32_t box[3] = {64, 1, 32};
    if ((st = encode_map(&tmY, p.out_dtype, 3, p.out, dims, str, box, true)) != KSMM_OK) return st;
  }
  ParamsD P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + 127) / 128);
  P.tiles_j = static_cast<int>((b + C::NJ - 1) / C::NJ);
  P.nchunks = static_cast<int>((c * d + 63) / 64);
  P.alpha = p.alpha;
  P.bias = p.bias;
  P.out_dtype = p.out_dtype;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;
  // fp32 accumulate, A K-major, B MN-major, N = 64, M = 128
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
  kern<<<grid, kThreadsD, C::SMEM_BYTES, stream>>>(tmX, tmW, tmY, P);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace tc

bool tc_bsfirst_d_supported(const Problem& p, bool check_pointers) {
  if (p.bs_last || (p.d != 2 && p.d != 4)) return false;
  if (p.in_dtype != KSMM_F16 && p.in_dtype != KSMM_BF16) return false;
  if (p.out_dtype != p.in_dtype) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  // tensor-map strides are multiples of 16 bytes: input and output rows, weight rows
  if ((static_cast<int64_t>(p.c) * p.d) % 8 != 0 || (static_cast<int64_t>(p.b) * p.d) % 8 != 0 ||
      p.b % 8 != 0)
    return false;
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16)
      return false;
  }
  return true;
}

int tc_bsfirst_d_launch(const Problem& p, cudaStream_t stream) {
  // <d, j tile, weight-stationary, resident weight chunks, ring stages>
  const int nchunks = (p.c * p.d + 63) / 64;
  const bool wide_j = p.b > 64;  // 128-wide j tiles halve the re-reads of the input
  if (p.d == 4) {
    if (wide_j) return tc::launch_d<4, 128, false, 0, 4>(p, stream);
    if (nchunks <= 12) return tc::launch_d<4, 64, true, 12, 3>(p, stream);
    return tc::launch_d<4, 64, false, 0, 4>(p, stream);
  }
  if (wide_j) {
    if (nchunks <= 6) return tc::launch_d<2, 128, true, 6, 3>(p, stream);
    return tc::launch_d<2, 128, false, 0, 4>(p, stream);
  }
  if (nchunks <= 12) return tc::launch_d<2, 64, true, 12, 3>(p, stream);
  return tc::launch_d<2, 64, false, 0, 4>(p, stream);
}

}  // namespace ksmm
