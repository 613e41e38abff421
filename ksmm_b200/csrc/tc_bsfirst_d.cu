// tcgen05 kernel for batch-first factors with d > 1 (16-bit inputs, d = 2 or 4).
//
// In the batch-first layout a row of the input holds, for one block row i_a,
// the c*d values x[n, i_a, k, l] with l fastest.  Block (i_a, l) contracts over
// k at a stride of d elements, which neither TMA (16-byte granularity) nor a
// UMMA operand descriptor can express.  This kernel therefore
//   1. fetches the contiguous 128-byte pieces of 128 input rows with TMA
//      ("raw" chunk: 64 elements = 64/d values of k for each of the d blocks),
//   2. lets four "transposer" warps split the chunk by l into d K-major operand
//      tiles in shared memory (16-byte loads, byte permutes, 16-byte stores),
//   3. issues, per chunk, 4 MMAs of 128 (batch rows) x 64 or 128 (j) x 16 into d
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
// warp index mod 4).  A CTA keeps one j tile and walks a contiguous range of
// (block row, batch tile) pairs; the weights of a chunk are streamed beside the
// raw input (they stay in L2).  Bounded waits and status reporting are as in
// tc_kernel.cu.
//
// What limits this kernel is not memory but the hand-offs between the roles:
// with every load, store, permute and MMA removed, the barrier skeleton alone
// (producer -> transposers -> MMA thread -> epilogue) takes about half of the
// run time, around 700 SM cycles per 64-element chunk against 256 cycles of
// tensor-pipe work.
#include <cuda.h>

#include <atomic>

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
  int act;  // ksmm_activation_t
  int* status;
};

constexpr int kThreadsD = (2 + 4 + kEpilogueWarps) * 32;

// Rings: SR raw input chunks (TMA -> transposers), SA split-tile buffers
// (transposers -> MMA) and, in the streaming flavour, SW weight chunks (TMA ->
// MMA).  STGN is the number of staging tiles per epilogue warp.
template <int D, int NJ_, int SR, int SW, int SA_, int STGN>
struct CfgD {
  static constexpr int NJ = NJ_;                    // j columns per accumulator (64 or 128)
  static constexpr int KCL = 64 / D;                // k values per block in one raw chunk
  static constexpr int RAW_BYTES = 128 * 128;       // 128 rows x 64 elements
  // split operand tiles (K-major, no swizzle): [k / 8][m / 8][m % 8][16 bytes]
  static constexpr int A_SBO = 128;                 // bytes between groups of 8 rows
  static constexpr int A_LBO = 16 * 128;            // bytes between core columns along k
  static constexpr int AL_BYTES = (KCL / 8) * A_LBO;  // one block's tile
  static constexpr int A_BYTES = D * AL_BYTES;
  static constexpr int SA = SA_;                    // split-tile buffers
  // weights of one raw chunk: [64-j box][block l][KCL rows][64 j], one TMA box per 64 j
  static constexpr int WL_BYTES = KCL * 128;        // one block's KCL rows x 64 j
  static constexpr int WJB_BYTES = D * WL_BYTES;    // one box: all d blocks (8 KB)
  static constexpr int WCH_BYTES = (NJ / 64) * WJB_BYTES;
  static constexpr int STG_TILE_BYTES = 32 * 128;     // 32 rows x 64 output elements
  static constexpr int STG_WARP_BYTES = STGN * STG_TILE_BYTES;
  static constexpr int STG_BYTES = kEpilogueWarps * STG_WARP_BYTES;
  static constexpr int NBAR = 2 * SR + 2 * SA + 2 * SW + 4;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES =
      STG_BYTES + SW * WCH_BYTES + SR * RAW_BYTES + SA * A_BYTES + BAR_BYTES + 1024;
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

template <int D, int NJ_, int SR, int SW, int SA_, int STGN>
__global__ void __launch_bounds__(kThreadsD, 1)
    ksmm_tc_bsfirst_d_kernel(const __grid_constant__ CUtensorMap tmX,
                             const __grid_constant__ CUtensorMap tmW,
                             const __grid_constant__ CUtensorMap tmY, const ParamsD P) {
  using C = CfgD<D, NJ_, SR, SW, SA_, STGN>;
  constexpr int SA = C::SA;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  // 1024-byte aligned regions first (swizzled weights and epilogue tiles), then the rest
  const uint32_t stg0 = sm0;                            // epilogue staging tiles
  const uint32_t wring0 = stg0 + C::STG_BYTES;          // streamed weight chunks
  const uint32_t rring0 = wring0 + SW * C::WCH_BYTES;   // raw input chunks
  const uint32_t aring0 = rring0 + SR * C::RAW_BYTES;   // split operand tiles
  const uint32_t bar0 = aring0 + SA * C::A_BYTES;
  uint8_t* bar_gen = sm_gen + (bar0 - sm0);
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto raw_empty = [&](int s) { return bar0 + 8u * (SR + s); };
  auto a_full = [&](int s) { return bar0 + 8u * (2 * SR + s); };
  auto a_empty = [&](int s) { return bar0 + 8u * (2 * SR + SA + s); };
  auto w_full = [&](int s) { return bar0 + 8u * (2 * SR + 2 * SA + s); };
  auto w_empty = [&](int s) { return bar0 + 8u * (2 * SR + 2 * SA + SW + s); };
  auto tfull_bar = [&](int q) { return bar0 + 8u * (2 * SR + 2 * SA + 2 * SW + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (2 * SR + 2 * SA + 2 * SW + 2 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SR; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(raw_empty(s), 4);  // one arrival per transposer warp
    }
    for (int s = 0; s < SA; ++s) {
      mbar_init(a_full(s), 4);
      mbar_init(a_empty(s), 1);
    }
    for (int s = 0; s < SW; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
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

  const int nchunks = P.nchunks;
  const int tj = static_cast<int>(blockIdx.x % P.tiles_j);
  const uint32_t rc = blockIdx.x / P.tiles_j;
  const uint32_t row_begin = static_cast<uint32_t>(static_cast<uint64_t>(rc) * P.rows / P.row_groups);
  const uint32_t row_end = static_cast<uint32_t>(static_cast<uint64_t>(rc + 1) * P.rows / P.row_groups);
  const int j0 = tj * C::NJ;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t ri = 0, rph = 0, wi = 0, wph = 0;
      bool ok = true;
      KSMM_TRACE_DECL;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        const int i = static_cast<int>(row / P.tiles_n);
        const int n0 = static_cast<int>(row % P.tiles_n) * 128;
        for (int qc = 0; qc < nchunks; ++qc) {
          KSMM_TRACE(0, 1);
          if (!mbar_wait<64>(raw_empty(ri), rph ^ 1u, abort_flag, P.status, 12)) { ok = false; break; }
          KSMM_TRACE(0, 2);
          mbar_expect_tx(raw_full(ri), C::RAW_BYTES);
          tma_load_3d(rring0 + ri * C::RAW_BYTES, &tmX, raw_full(ri), qc * 64, i, n0);
          if (++ri == SR) { ri = 0; rph ^= 1u; }
          KSMM_TRACE(0, 3);
          if (!mbar_wait<64>(w_empty(wi), wph ^ 1u, abort_flag, P.status, 13)) { ok = false; break; }
          KSMM_TRACE(0, 4);
          mbar_expect_tx(w_full(wi), C::WCH_BYTES);
#pragma unroll
          for (int jb = 0; jb < C::NJ / 64; ++jb)
            tma_load_3d(wring0 + wi * C::WCH_BYTES + jb * C::WJB_BYTES, &tmW, w_full(wi),
                        j0 + jb * 64, qc * C::KCL, i * D);
          if (++wi == SW) { wi = 0; wph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t ai = 0, aph = 0, wi = 0, wph = 0, ut = 0;
      bool ok = true;
      KSMM_TRACE_DECL;
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
        KSMM_TRACE(1, 10);
        if (!mbar_wait<0>(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 15)) { ok = false; break; }
        KSMM_TRACE(1, 11);
        tc_fence_after();
        const uint32_t dcol = tmem_base + buf * C::BUF_COLS;
        for (int qc = 0; qc < nchunks; ++qc) {
          KSMM_TRACE(1, 14);
          if (!mbar_wait<0>(w_full(wi), wph, abort_flag, P.status, 16)) { ok = false; break; }
          const uint32_t wbase = wring0 + wi * C::WCH_BYTES;
          KSMM_TRACE(1, 12);
          if (!mbar_wait<0>(a_full(ai), aph, abort_flag, P.status, 17)) { ok = false; break; }
          KSMM_TRACE(1, 13);
          tc_fence_after();
          KSMM_TRACE(1, 18);
          const uint32_t abase = aring0 + ai * C::A_BYTES;
#pragma unroll
          for (int ks = 0; ks < C::KCL / 16; ++ks) {
#pragma unroll
            for (int l = 0; l < D; ++l) {
              // split tile: K-major, no swizzle (core matrices of 8 rows x 16 bytes)
              const uint64_t adesc =
                  make_desc(abase + l * C::AL_BYTES + ks * 2 * C::A_LBO, C::A_LBO, C::A_SBO, 0);
              // weights: MN-major, 128-byte swizzle; LBO = next 64-j box, SBO = next 8 k rows
              const uint64_t bdesc =
                  make_desc(wbase + l * C::WL_BYTES + ks * 2048, C::WJB_BYTES, 1024, 2);
              umma<2>(dcol + l * C::NJ, adesc, bdesc, P.idesc, (qc | ks) != 0 ? 1u : 0u);
            }
          }
          KSMM_TRACE(1, 19);
          umma_commit(a_empty(ai));  // the split tiles and the weight slot are free again
          umma_commit(w_empty(wi));
          KSMM_TRACE(1, 16);
          if (++ai == SA) { ai = 0; aph ^= 1u; }
          if (++wi == SW) { wi = 0; wph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));
        KSMM_TRACE(1, 17);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ===================== transposers =====================
    // A raw chunk holds, per row m, 128 bytes = eight 16-byte pieces, stored by
    // TMA with the 128-byte swizzle (piece p of row m sits at p ^ (m % 8)).  One
    // unit of work is half a row (4 pieces = 32 elements = 32/d values of k for
    // each of the d blocks, l fastest): its values are regrouped by block into
    // runs of 8 consecutive k, i.e. whole 16-byte rows of the K-major core
    // matrices.  Eight neighbouring lanes take eight consecutive rows of the
    // same half, which makes both the swizzled loads and the stores conflict-free.
    const int tt = (warp - 2) * 32 + lane;
    uint32_t ri = 0, rph = 0, ai = 0, aph = 0;
    bool ok = true;
    KSMM_TRACE_DECL;
    const bool tron = warp == 2 && lane == 0;
    for (uint32_t row = row_begin; row < row_end && ok; ++row) {
      for (int qc = 0; qc < nchunks; ++qc) {
        int got = 1;
        if (tron) KSMM_TRACE(2, 30);
        if (lane == 0) got = mbar_wait<32>(raw_full(ri), rph, abort_flag, P.status, 18) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        if (tron) KSMM_TRACE(2, 31);
        const uint32_t rbase = rring0 + ri * C::RAW_BYTES;
        const uint32_t abase = aring0 + ai * C::A_BYTES;
        uint32_t w[2][4][4];
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int u = tt + it * 128;
          const int m = ((u >> 4) << 3) | (u & 7), half = (u >> 3) & 1;
#pragma unroll
          for (int pj = 0; pj < 4; ++pj)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[it][pj][0]), "=r"(w[it][pj][1]), "=r"(w[it][pj][2]), "=r"(w[it][pj][3])
                         : "r"(rbase + m * 128 + (((half * 4 + pj) ^ (m & 7)) << 4))
                         : "memory");
        }
        // the raw chunk is in registers: hand its slot back to the producer at once
        __syncwarp();
        if (tron) KSMM_TRACE(2, 32);
        if (lane == 0) {
          mbar_arrive(raw_empty(ri));
          got = mbar_wait<32>(a_empty(ai), aph ^ 1u, abort_flag, P.status, 19) ? 1 : 0;
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        if (tron) KSMM_TRACE(2, 33);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int u = tt + it * 128;
          const int half = (u >> 3) & 1;
          const uint32_t dst = abase + (u >> 4) * C::A_SBO + (u & 7) * 16;
          if constexpr (D == 4) {
            // piece pj = (k = 2 pj: l0 l1 | l2 l3), (k = 2 pj + 1: l0 l1 | l2 l3)
#pragma unroll
            for (int l = 0; l < 4; ++l) {
              uint32_t o[4];
#pragma unroll
              for (int pj = 0; pj < 4; ++pj)
                o[pj] = __byte_perm(w[it][pj][l >> 1], w[it][pj][2 + (l >> 1)], (l & 1) ? 0x7632 : 0x5410);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + l * C::AL_BYTES + half * C::A_LBO),
                           "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                           : "memory");
            }
          } else {
            // piece pj = (k = 4 pj .. 4 pj + 3), each word (l0 l1); 16 values of k per block:
            // pieces 0, 1 fill core column 2 half, pieces 2, 3 core column 2 half + 1
#pragma unroll
            for (int l = 0; l < 2; ++l)
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {
                const uint32_t sel = l ? 0x7632 : 0x5410;
                const uint32_t o0 = __byte_perm(w[it][2 * cc][0], w[it][2 * cc][1], sel);
                const uint32_t o1 = __byte_perm(w[it][2 * cc][2], w[it][2 * cc][3], sel);
                const uint32_t o2 = __byte_perm(w[it][2 * cc + 1][0], w[it][2 * cc + 1][1], sel);
                const uint32_t o3 = __byte_perm(w[it][2 * cc + 1][2], w[it][2 * cc + 1][3], sel);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                                 dst + l * C::AL_BYTES + (2 * half + cc) * C::A_LBO),
                             "r"(o0), "r"(o1), "r"(o2), "r"(o3)
                             : "memory");
              }
          }
        }
        fence_proxy_async();  // the tiles are read by the tensor core through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(ai));
        if (tron) KSMM_TRACE(2, 34);
        if (++ri == SR) { ri = 0; rph ^= 1u; }
        if (++ai == SA) { ai = 0; aph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    const int ew = warp - 6;
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

template <int D, int NJ_, int SR, int SW, int SA_, int STGN>
static int launch_d(const Problem& p, cudaStream_t stream) {
  using C = CfgD<D, NJ_, SR, SW, SA_, STGN>;
  auto kern = ksmm_tc_bsfirst_d_kernel<D, NJ_, SR, SW, SA_, STGN>;
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
    // input rows: (c*d, a, batch); raw chunk = 64 contiguous elements of 128 rows, 128-byte swizzle
    const uint64_t dims[3] = {c * d, a, B};
    const uint64_t str[3] = {1, c * d, a * c * d};
    const uint32_t box[3] = {64, 1, 128};
    if ((st = encode_map(&tmX, p.in_dtype, 3, p.in, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // weights (a*d*c, b) row-major seen as (b, c, a*d); box = 64 j x KCL k rows x the d blocks of a row
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {64, static_cast<uint32_t>(C::KCL), static_cast<uint32_t>(D)};
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
  P.act = p.activation;
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
  cudaError_t err = launch_pdl(kern, grid, kThreadsD, C::SMEM_BYTES, stream, tmX, tmW, tmY, P);
  count_launch();
  if (err == cudaSuccess) err = cudaGetLastError();
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
  // <d, j tile, raw stages, weight stages, split-tile buffers, staging tiles per epilogue warp>;
  // 128-wide j tiles halve the re-reads of the input
  if (p.d == 4)
    return p.b > 64 ? tc::launch_d<4, 128, 5, 5, 2, 1>(p, stream) : tc::launch_d<4, 64, 6, 8, 2, 1>(p, stream);
  return p.b > 64 ? tc::launch_d<2, 128, 5, 5, 2, 1>(p, stream) : tc::launch_d<2, 64, 6, 8, 2, 1>(p, stream);
}

}  // namespace ksmm

#ifdef KSMM_TC_TRACE
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace_d(unsigned long long* host) {
  using namespace ksmm;
  return static_cast<int>(cudaMemcpyFromSymbol(host, tc::g_trace, sizeof(tc::g_trace)));
}
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace_d_clear() {
  using namespace ksmm;
  static unsigned long long zeros[4][8192];
  return static_cast<int>(cudaMemcpyToSymbol(tc::g_trace, zeros, sizeof(zeros)));
}
#endif
