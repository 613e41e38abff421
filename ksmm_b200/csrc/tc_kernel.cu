// tcgen05 / TMEM / TMA KSMM kernel family (KSMM_ALGO_TC) for fp16, bf16 and
// fp8-e4m3 inputs with fp32 accumulation.
//
// One factor with pattern (a,b,c,d) is a*d independent (b x c) blocks, each
// contracted with a (c x batch) slice of the input.  The output is cut into
// tiles of 128 accumulator rows x NT columns.  A persistent CTA (one per SM) keeps
// one j tile (CTA index modulo the number of j tiles) and walks a contiguous range
// of rows (row = block x batch tile); CTAs that differ only in the j tile walk the
// same rows at the same time and share the input tile in L2.  Two flavours per tile
// configuration: weight-stationary (all k chunks of the CTA's weight tile stay in
// shared memory, only the input streams through the ring) when the weight tile
// fits, else streaming (a ring stage holds one k chunk of both operands).
//
//   batch-last : D[j (128 rows), n (NT cols)] = W_blk[j,k] * X_blk[k,n]
//                A = weights tile, MN-major, straight from the reference's
//                (a*d*c, b) storage; B = input slice, MN-major, fetched by a
//                4-D tensor map over (batch, d, c, a) so that the stride-d rows
//                of the slice land densely in shared memory.
//   batch-first (d == 1):
//                D[n (128 rows), j (NT cols)] = X_blk[n,k] * W_blk[j,k]
//                A = input rows, K-major; B = weights tile, MN-major.
//
// In both layouts the contiguous dimension of the output is the TMEM column
// dimension, so each epilogue thread owns a run of consecutive output
// elements: it converts them, writes 16-byte chunks into a 128-byte-swizzled
// staging tile, and one thread issues a TMA store of the tile.  The epilogue
// applies alpha, the bias (one coalesced load per tile, broadcast by shuffles) and
// an optional activation; in a chain it can store a batch-first 16-bit output
// regrouped by the blocks of the next factor (see tc_bsfirst_dp.cu).
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM allocator and
// single-thread MMA issuer, warps 2..9 = epilogue (TMEM lane quarter = warp
// index mod 4; each warp converts and stores its own 32-row sub-tiles, so the
// epilogue has no block-level barrier).  Ring stages and the resident weight tile
// are guarded by full/empty mbarriers; the accumulator is double-buffered in
// TMEM (2 x NT columns) so the epilogue of one tile overlaps the MMAs of the next.
//
// Every mbarrier wait is bounded (about two seconds); on expiry the kernel
// records a code in a device status word, stops issuing work, releases TMEM
// and returns.  Rows/columns/k beyond the problem extents are zero-filled by
// TMA on load and clipped by TMA on store, so no shape needs to divide a tile.
//
// Reference counterpart: kernel_bs_{first,last}_half{2,4}
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_half.cuh:107-1092, CUDA-core
// fp16 math with fp16 accumulation) and kernel_bs_{first,last}_fp8
// (src/ksmm_cu/src/template_kernels_fp8.cuh:22-370).
#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include <mutex>

#include "tc_kernel.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace tc {

// one status word per device that loads the module; 0 = no device-side timeout
__device__ int g_tc_status_word = 0;

struct Params {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  uint32_t rows;        // tiles_n * a * d: (block, batch tile) pairs
  uint32_t row_groups;  // CTAs per j tile; each walks a contiguous range of rows
  int nk;
  uint32_t idesc;
  float alpha;
  const void* bias;
  int out_dtype;
  int* status;
  int act;         // ksmm_activation_t
  int rg_d, rg_c;  // batch-first, 16-bit: store regrouped for the next factor's (c, d); 0 = natural order
  // Grouped launch: `groups` problems of the same pattern in one grid (weights and outputs of the
  // groups are stacked; the input is shared, or stacked as well when gx = 1).  A CTA's j tile slot
  // encodes (group, j tile), so the groups of one input tile run at the same time and share it in L2.
  int groups, gx;
  int tiles_jg;    // tiles_j * groups
  const void* residual;  // added after the activation; output's layout and type; or nullptr
};

// WRES = true  ("weight-stationary"): the CTA's weight tile (all NWC k chunks of
//   it) stays in shared memory while the CTA walks its rows; only input chunks
//   stream through the ring (SX stages of one chunk each).
// WRES = false ("streaming"): a ring stage holds one k chunk of both operands
//   (NWC = 0); used when the weight tile is too large to keep.
// IN_LAST / OUT_LAST: layout of the input and of the output.  The accumulator's rows are output
// features when the output is batch-last (weights = M-side operand) and batch entries when it is
// batch-first (input = M-side operand); the input operand is MN-major when the input is batch-last
// (rows of the tile = k, consecutive batch entries) and K-major when it is batch-first (rows =
// batch entries, consecutive k).  The two mixed combinations (d = 1 only) let a chain change its
// layout inside a factor at no cost.
template <bool IN_LAST, bool OUT_LAST, int ES, int OS, int NT, int KC, bool WRES, int NWC, int SX, int STGN = 1>
struct Cfg {
  static constexpr int NBOX = 128 / ES;        // elements in one 128-byte box row
  static constexpr int UK = 32 / ES;           // k extent of one MMA
  static constexpr int M_BYTES = 128 * KC * ES;  // one k chunk of the M-side operand
  static constexpr int N_BYTES = NT * KC * ES;   // one k chunk of the N-side operand
  static constexpr int XB = OUT_LAST ? N_BYTES : M_BYTES;  // input chunk
  static constexpr int WB = OUT_LAST ? M_BYTES : N_BYTES;  // weight chunk
  static constexpr int XN = OUT_LAST ? NT : 128;           // batch entries per tile
  static constexpr int WJ = OUT_LAST ? 128 : NT;           // output features per tile
  static constexpr int STAGE_BYTES = XB + (WRES ? 0 : WB);
  static constexpr int CB = 128 / OS;          // output elements in one staging row
  static constexpr int STG_TILE_BYTES = 32 * 128;  // one warp's 32 rows x 128 bytes
  // STGN staging tiles per epilogue warp: with two, a warp fills one while the TMA store of the
  // other is still reading shared memory
  static constexpr int STG_WARP_BYTES = STGN * STG_TILE_BYTES;
  static constexpr int STG_BYTES = kEpilogueWarps * STG_WARP_BYTES;
  static constexpr int NBAR = 2 * SX + 2 + 4;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = NWC * WB + SX * STAGE_BYTES + STG_BYTES + BAR_BYTES + 1024;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static constexpr int TMEM_COLS = 2 * NT;
  // CTAs that fit one SM: their TMEM allocations must fit together, so that an allocation never waits
  static constexpr int CTAS = SMEM_BYTES <= 115712 ? 2 : 1;
  static_assert(CTAS * TMEM_COLS <= 512, "tensor memory of the CTAs resident on one SM");
  static_assert(NT == 64 || NT == 128 || NT == 256, "TMEM allocation must be a power of two");
  static_assert(KC % UK == 0 && KC % 8 == 0, "k chunk");
  static_assert(IN_LAST || KC == NBOX, "batch-first input chunks are one 128-byte k box");
  static_assert(IN_LAST || XN <= 256, "a batch-first input chunk is one TMA box of XN rows");
  static_assert(NT % NBOX == 0, "N tile must be whole 128-byte box rows");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
  static_assert(WRES ? NWC > 0 : NWC == 0, "resident weight chunks exist in weight-stationary mode only");
};

template <bool IN_LAST, bool OUT_LAST, int ES, int OS, int NT, int KC, bool WRES, int NWC, int SX, int STGN>
__global__ void __launch_bounds__(kThreads, Cfg<IN_LAST, OUT_LAST, ES, OS, NT, KC, WRES, NWC, SX, STGN>::CTAS)
    ksmm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmY, const Params P) {
  using C = Cfg<IN_LAST, OUT_LAST, ES, OS, NT, KC, WRES, NWC, SX, STGN>;
  constexpr bool BS_LAST = OUT_LAST;  // orientation of the accumulator and of the epilogue
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;  // 1024-byte alignment for the 128-byte swizzle
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t wres0 = sm0;                           // resident weight tile (weight-stationary)
  const uint32_t ring0 = wres0 + NWC * C::WB;           // stage ring
  const uint32_t stg0 = ring0 + SX * C::STAGE_BYTES;    // epilogue staging, one tile per warp
  const uint32_t bar0 = stg0 + C::STG_BYTES;
  uint8_t* bar_gen = sm_gen + NWC * C::WB + SX * C::STAGE_BYTES + C::STG_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (SX + s); };
  const uint32_t wfull_bar = bar0 + 8u * (2 * SX);
  const uint32_t wempty_bar = bar0 + 8u * (2 * SX + 1);
  auto tfull_bar = [&](int q) { return bar0 + 8u * (2 * SX + 2 + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (2 * SX + 4 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SX; ++s) {
      mbar_init(full_bar(s), 1);
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

  // Work split: CTA c keeps one j tile (tj = c mod tiles_j) and walks a
  // contiguous range of rows, a row being one (block, batch tile) pair.  CTAs
  // that differ only in tj walk the same rows at the same time and share the
  // input tile in L2; the weight tile changes only when the block changes.
  const uint32_t d = P.d;
  const int nk = P.nk;
  const int tjg = static_cast<int>(blockIdx.x % P.tiles_jg);
  const int grp_id = tjg / P.tiles_j;
  const int tj = tjg % P.tiles_j;
  const uint32_t rc = blockIdx.x / P.tiles_jg;
  const uint32_t row_begin = static_cast<uint32_t>(static_cast<uint64_t>(rc) * P.rows / P.row_groups);
  const uint32_t row_end = static_cast<uint32_t>(static_cast<uint64_t>(rc + 1) * P.rows / P.row_groups);
  const int j0 = tj * (BS_LAST ? 128 : NT);
  // offsets of this CTA's group in the stacked tensors: weight blocks, block rows of a batch-last
  // input / output, batch rows of a batch-first input / output, bias elements
  const int wblk0 = grp_id * P.a * P.d;
  const int xi0 = P.gx ? grp_id * P.a : 0, yi0 = grp_id * P.a;
  const int xn0 = P.gx ? grp_id * static_cast<int>(P.batch) : 0, yn0 = grp_id * static_cast<int>(P.batch);
  (void)xi0; (void)xn0; (void)yi0; (void)yn0;
  const int64_t bias0 = static_cast<int64_t>(grp_id) * P.a * P.b * P.d;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0, wph = 0;  // ring position / phase, weight-tile phase
      int cur_blk = -1;
      KSMM_TRACE_DECL;
      bool ok = true;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        const int blk = static_cast<int>(row / P.tiles_n);
        const int tn = static_cast<int>(row % P.tiles_n);
        const int i = blk / d, l = blk % d;
        const int n0 = tn * C::XN;
        if (WRES && blk != cur_blk) {
          // new block: fetch its weight tile once the MMAs on the old one are done
          if (!mbar_wait<64>(wempty_bar, wph ^ 1u, abort_flag, P.status, 1)) { ok = false; break; }
          wph ^= 1u;
          mbar_expect_tx(wfull_bar, nk * C::WB);
          for (int kc = 0; kc < nk; ++kc) {
#pragma unroll
            for (int wb = 0; wb < C::WJ / C::NBOX; ++wb)
              tma_load_3d(wres0 + kc * C::WB + wb * KC * 128, &tmW, wfull_bar, j0 + wb * C::NBOX,
                          kc * KC, blk + wblk0);
          }
          cur_blk = blk;
        }
        for (int kc = 0; kc < nk; ++kc) {
          KSMM_TRACE(0, 3);
          if (!mbar_wait<64>(empty_bar(si), sph ^ 1u, abort_flag, P.status, 2)) { ok = false; break; }
          KSMM_TRACE(0, 4);
          const uint32_t dst = ring0 + si * C::STAGE_BYTES;
          const uint32_t bar = full_bar(si);
          mbar_expect_tx(bar, C::STAGE_BYTES);
          if constexpr (IN_LAST) {
#pragma unroll
            for (int xb = 0; xb < C::XN / C::NBOX; ++xb)
              tma_load_4d(dst + xb * KC * 128, &tmX, bar, n0 + xb * C::NBOX, l, kc * KC, i + xi0);
          } else {
            tma_load_3d(dst, &tmX, bar, kc * KC, i, n0 + xn0);
          }
          if constexpr (!WRES) {
#pragma unroll
            for (int wb = 0; wb < C::WJ / C::NBOX; ++wb)
              tma_load_3d(dst + C::XB + wb * KC * 128, &tmW, bar, j0 + wb * C::NBOX, kc * KC, blk + wblk0);
          }
          KSMM_TRACE(0, 5);
          if (++si == SX) { si = 0; sph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      // descriptor words that never change: SBO = 1024 bytes, version 1, 128-byte swizzle
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLboMN = static_cast<uint32_t>((KC * 128) >> 4) << 16;  // MN-major operands
      constexpr uint32_t kLboK = 1u << 16;                                       // unused for K-major
      constexpr uint32_t kStepMN = (C::UK * 128) >> 4;  // descriptor address step per MMA, MN-major
      constexpr uint32_t kStepK = (C::UK * ES) >> 4;    // K-major: UK elements inside the swizzle row
      const uint32_t idesc = P.idesc;
      uint32_t si = 0, sph = 0, wph = 0, ut = 0;
      int cur_blk = -1;
      bool ok = true;
      KSMM_TRACE_DECL;
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        const int blk = static_cast<int>(row / P.tiles_n);
        if (WRES && blk != cur_blk) {
          if (!mbar_wait<0>(wfull_bar, wph, abort_flag, P.status, 3)) { ok = false; break; }
          wph ^= 1u;
          cur_blk = blk;
        }
        const uint32_t buf = ut & 1u, bph = (ut >> 1) & 1u;
        KSMM_TRACE(1, 10);
        if (!mbar_wait<0>(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 4)) { ok = false; break; }
        tc_fence_after();
        KSMM_TRACE(1, 11);
        const uint32_t dcol = tmem_base + buf * NT;
        for (int kc = 0; kc < nk; ++kc) {
          KSMM_TRACE(1, 14);
          if (!mbar_wait<0>(full_bar(si), sph, abort_flag, P.status, 5)) { ok = false; break; }
          KSMM_TRACE(1, 15);
          const uint32_t xsrc = ring0 + si * C::STAGE_BYTES;
          const uint32_t wsrc = WRES ? wres0 + kc * C::WB : xsrc + C::XB;
          const uint32_t xlo = (xsrc >> 4) | (IN_LAST ? kLboMN : kLboK);
          const uint32_t wlo = (wsrc >> 4) | kLboMN;
#pragma unroll
          for (int k = 0; k < KC / C::UK; ++k) {
            const uint32_t xl = xlo + k * (IN_LAST ? kStepMN : kStepK);
            const uint32_t wl = wlo + k * kStepMN;
            const uint64_t xdesc = (static_cast<uint64_t>(kDescHi) << 32) | xl;
            const uint64_t wdesc = (static_cast<uint64_t>(kDescHi) << 32) | wl;
            // batch-last: A = weights, B = input slice; batch-first: A = input rows, B = weights
            umma<ES>(dcol, BS_LAST ? wdesc : xdesc, BS_LAST ? xdesc : wdesc, idesc,
                     (kc | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(si));  // frees the stage once these MMAs have read it
          KSMM_TRACE(1, 16);
          if (++si == SX) { si = 0; sph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));  // accumulator complete
        KSMM_TRACE(1, 17);
        if (WRES && (row + 1 == row_end || static_cast<int>((row + 1) / P.tiles_n) != blk))
          umma_commit(wempty_bar);  // last use of this weight tile
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    // Warp w owns TMEM lane quarter w mod 4 (32 output rows) and the column boxes
    // (w - 2) / 4, (w - 2) / 4 + kEpilogueWarps / 4, ...  Each warp converts its
    // 32 x CB sub-tile into its own swizzled staging tile and issues its own TMA
    // store, so the epilogue needs no block-level barrier.
    const int ew = warp - 2;
    const int q = warp & 3;
    const int grp = ew >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool plain = (P.alpha == 1.f) && (P.bias == nullptr) && (P.act == 0);
    const uint32_t stg_base = stg0 + ew * C::STG_WARP_BYTES;
    uint32_t ut = 0, sti = 0;
    KSMM_TRACE_DECL;
    const int trole = (ew == 0) ? 2 : 3;
    const bool tron = (ew == 0 || ew == 5) && lane == 0;
    (void)trole; (void)tron;
    for (uint32_t row = row_begin; row < row_end; ++row, ++ut) {
      const int blk = static_cast<int>(row / P.tiles_n);
      const int tn = static_cast<int>(row % P.tiles_n);
      const int i = blk / d, l = blk % d;
      const int n0 = tn * C::XN;
      const uint32_t buf = ut & 1u, bph = (ut >> 1) & 1u;
      if (tron) KSMM_TRACE(trole, 20);
      int got = 1;
      if (lane == 0) got = mbar_wait<128>(tfull_bar(buf), bph, abort_flag, P.status, 6) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      if (tron) KSMM_TRACE(trole, 21);
      // rows of this warp that exist (warp-uniform): j rows (batch-last) or batch rows
      const int row_limit = BS_LAST ? P.b - j0 : static_cast<int>(min(P.batch - n0, static_cast<int64_t>(128)));
      const bool warp_active = (q * 32) < row_limit;
      const int col_limit = BS_LAST ? static_cast<int>(min(P.batch - n0, static_cast<int64_t>(NT))) : P.b - j0;
      float bias_row = 0.f;
      if (BS_LAST && P.bias != nullptr && q * 32 + lane < row_limit)
        bias_row = bias_at(P.bias, bias0 + (static_cast<int64_t>(i) * P.b + j0 + q * 32 + lane) * d + l,
                           P.out_dtype);
      if (warp_active) {
#pragma unroll 1
        for (int cbi = grp; cbi < NT / C::CB; cbi += kEpilogueWarps / 4) {
          if (cbi * C::CB >= col_limit) break;
          // the staging tile about to be written has been read by the store that used it last
          if (lane == 0) bulk_wait_read<STGN - 1>();
          __syncwarp();
          const uint32_t stg = stg_base + (STGN > 1 ? sti * C::STG_TILE_BYTES : 0u);
          if (STGN > 1) sti = (sti + 1 == STGN) ? 0u : sti + 1;
          uint32_t r[C::CB];
#pragma unroll
          for (int h = 0; h < C::CB / 32; ++h)
            tmem_ld32(tmem_base + lane_addr + buf * NT + cbi * C::CB + h * 32, r + h * 32);
          tmem_ld_wait();
          if (tron) KSMM_TRACE(trole, 23);
          if (!plain) {
            // batch-first: the bias of the tile's columns comes through one coalesced load per lane
            // and shuffles (16-bit: columns 2 lane, 2 lane + 1; fp32: column lane);
            // batch-last: one value per accumulator row
            uint32_t braw = 0;
            if (!BS_LAST && P.bias != nullptr) {
              const int col = cbi * C::CB + (OS == 2 ? 2 * lane : lane);
              if (col < col_limit) {
                const int64_t e0 = bias0 + static_cast<int64_t>(i) * P.b + j0 + col;
                if constexpr (OS == 2) {
                  // (col_limit is even for 16-bit outputs: b * 2 bytes is a multiple of 16)
                  const uint16_t* bp = static_cast<const uint16_t*>(P.bias) + e0;
                  braw = (reinterpret_cast<uintptr_t>(bp) & 3) == 0
                             ? *reinterpret_cast<const uint32_t*>(bp)
                             : (static_cast<uint32_t>(bp[0]) | (static_cast<uint32_t>(bp[1]) << 16));
                } else {
                  braw = static_cast<const uint32_t*>(P.bias)[e0];
                }
              }
            }
#pragma unroll
            for (int e = 0; e < C::CB; ++e) {
              float bv = bias_row;
              if (!BS_LAST) {
                if constexpr (OS == 2) {
                  const uint32_t pr = __shfl_sync(0xffffffffu, braw, e >> 1);
                  const uint16_t hv = static_cast<uint16_t>((e & 1) ? (pr >> 16) : (pr & 0xffffu));
                  bv = P.out_dtype == KSMM_BF16 ? __uint_as_float(static_cast<uint32_t>(hv) << 16)
                                                : __half2float(__ushort_as_half(hv));
                } else {
                  bv = __uint_as_float(__shfl_sync(0xffffffffu, braw, e));
                }
              }
              r[e] = __float_as_uint(fmaf(P.alpha, __uint_as_float(r[e]), bv));
            }
            if (P.act == KSMM_ACT_GELU) {
#pragma unroll
              for (int e = 0; e < C::CB; ++e) r[e] = __float_as_uint(OS == 2 ? gelu_16bit(__uint_as_float(r[e])) : apply_activation(__uint_as_float(r[e]), 1));
            } else if (P.act == KSMM_ACT_RELU) {
#pragma unroll
              for (int e = 0; e < C::CB; ++e) r[e] = __float_as_uint(fmaxf(__uint_as_float(r[e]), 0.f));
            }
          }
          if (P.residual != nullptr && q * 32 + lane < row_limit) {
            // this thread's CB outputs are consecutive in memory (128 bytes): eight 16-byte loads
            const int64_t base = BS_LAST
                ? ((static_cast<int64_t>(i) * P.b + j0 + q * 32 + lane) * d + l) * P.batch + n0 + cbi * C::CB
                : (static_cast<int64_t>(n0) + q * 32 + lane) * (static_cast<int64_t>(P.a) * P.b) +
                      static_cast<int64_t>(i) * P.b + j0 + cbi * C::CB;
            const uint4* rp = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(P.residual) + base * OS);
            constexpr int EPC = 16 / OS;  // elements per 16-byte piece
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              if (cbi * C::CB + ch * EPC < col_limit) {
                const uint4 v = __ldg(rp + ch);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < EPC; ++e) {
                  float rv;
                  if constexpr (OS == 4) {
                    rv = __uint_as_float(w4[e]);
                  } else {
                    const uint16_t hv = static_cast<uint16_t>((e & 1) ? (w4[e >> 1] >> 16) : (w4[e >> 1] & 0xffffu));
                    rv = P.out_dtype == KSMM_BF16 ? __uint_as_float(static_cast<uint32_t>(hv) << 16)
                                                  : __half2float(__ushort_as_half(hv));
                  }
                  r[ch * EPC + e] = __float_as_uint(__uint_as_float(r[ch * EPC + e]) + rv);
                }
              }
            }
          }
          const uint32_t rowaddr = stg + lane * 128;
          if (!BS_LAST && OS == 2 && P.rg_d != 0) {
            // regrouped store: element e of the 64 goes to (e % d2) * (64 / d2) + e / d2; the tile is
            // not swizzled (its TMA box rows are 64 / d2 elements wide)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (P.rg_d == 4) {
                  const int l2 = ch >> 1, t = (ch & 1) * 4 + e;
                  w[e] = pack2(__uint_as_float(r[(2 * t) * 4 + l2]), __uint_as_float(r[(2 * t + 1) * 4 + l2]),
                               P.out_dtype);
                } else {
                  const int l2 = ch >> 2, t = (ch & 3) * 4 + e;
                  w[e] = pack2(__uint_as_float(r[(2 * t) * 2 + l2]), __uint_as_float(r[(2 * t + 1) * 2 + l2]),
                               P.out_dtype);
                }
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ch * 16),
                           "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                           : "memory");
            }
          } else if constexpr (OS == 2) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack2(__uint_as_float(r[ch * 8 + 2 * e]),
                             __uint_as_float(r[ch * 8 + 2 * e + 1]), P.out_dtype);
              const uint32_t chunk = static_cast<uint32_t>(ch ^ (lane & 7));
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + chunk * 16),
                           "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                           : "memory");
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              const uint32_t chunk = static_cast<uint32_t>(ch ^ (lane & 7));
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + chunk * 16),
                           "r"(r[ch * 4 + 0]), "r"(r[ch * 4 + 1]), "r"(r[ch * 4 + 2]),
                           "r"(r[ch * 4 + 3])
                           : "memory");
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (tron) KSMM_TRACE(trole, 25);
          if (lane == 0) {
            if constexpr (BS_LAST) {
              tma_store_4d(&tmY, stg, n0 + cbi * C::CB, l, j0 + q * 32, i + yi0);
            } else if (P.rg_d != 0) {
              // output seen as (k2, l2, i2, n): the tile starts at feature m0 = i*b + j0 + 64*cbi
              const int m0 = i * P.b + j0 + cbi * C::CB, seg = P.rg_c * P.rg_d;
              tma_store_4d(&tmY, stg, (m0 % seg) / P.rg_d, 0, m0 / seg, n0 + q * 32);
            } else {
              tma_store_3d(&tmY, stg, j0 + cbi * C::CB, i, n0 + q * 32 + yn0);
            }
            bulk_commit();
          }
        }
      }
      // this warp's TMEM reads of the buffer are complete: hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
      if (tron) KSMM_TRACE(trole, 27);
    }
    if (lane == 0) bulk_wait<0>();  // all stores have left shared memory and are visible
    __syncwarp();
  }

  // ===================== teardown =====================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory is handed to another CTA
    __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static CUtensorMapDataType tm_dtype(int dt) {
  switch (dt) {
    case KSMM_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case KSMM_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case KSMM_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// rank-R tiled map with 128-byte swizzle (16-byte or, with atom32, 32-byte atoms) or none;
// dims/strides innermost first, strides in elements (stride of dim 0 is implicitly 1)
int encode_map(CUtensorMap* tm, int dt, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_elems, const uint32_t* box, bool swizzle128, bool atom32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_error(KSMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  const uint64_t esz = dtype_size(dt);
  for (int r = 0; r < rank; ++r) {
    gdim[r] = dims[r];
    bx[r] = box[r];
    es[r] = 1;
    if (r > 0) gstr[r - 1] = strides_elems[r] * esz;
  }
  CUresult res = fn(tm, tm_dtype(dt), rank, const_cast<void*>(base), gdim, gstr, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? (atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B)
                               : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return set_error(KSMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d)",
                     static_cast<int>(res), rank);
  return KSMM_OK;
}

// Tile configurations (N tile, k rows per stage for 16-bit inputs, stages); see
// launch_cfg.  8-bit inputs use twice the k rows; batch-first stages always
// hold one 128-byte k box.  Configuration 4 (N tile 64) is narrower than one
// 128-byte fp8 box row and exists for 16-bit inputs only.
static constexpr int kNumConfigs = 8;

int* status_word() {
  // one status word per device, owned by the module image
  static std::atomic<int*> ptrs[64];  // zero-initialised; every thread resolves the same address
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int* cached = ptrs[dev].load(std::memory_order_acquire);
  if (!cached) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status_word) != cudaSuccess) return nullptr;
    cached = static_cast<int*>(p);
    ptrs[dev].store(cached, std::memory_order_release);
  }
  return cached;
}

bool pdl_enabled() {
  static const bool on = std::getenv("KSMM_NO_PDL") == nullptr;
  return on;
}

int num_sms() {
  static std::atomic<int> sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int n = sms[dev].load(std::memory_order_relaxed);
  if (!n) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

template <bool IN_LAST, bool OUT_LAST, int ES, int OS, int NT, int KC, bool WRES, int NWC, int SX, int STGN = 1>
static int launch_one(const Problem& p, cudaStream_t stream) {
  using C = Cfg<IN_LAST, OUT_LAST, ES, OS, NT, KC, WRES, NWC, SX, STGN>;
  auto kern = ksmm_tc_kernel<IN_LAST, OUT_LAST, ES, OS, NT, KC, WRES, NWC, SX, STGN>;
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
  const uint64_t G = p.groups > 1 ? p.groups : 1, GX = (G > 1 && !p.group_shared_input) ? G : 1;
  CUtensorMap tmX, tmW, tmY;
  int st;
  {
    // weights (a*d*c, b) row-major seen as (b, c, a*d); the groups' weights follow one another
    const uint64_t dims[3] = {b, c, G * a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {static_cast<uint32_t>(C::NBOX), static_cast<uint32_t>(KC), 1};
    if ((st = encode_map(&tmW, p.in_dtype, 3, p.w, dims, str, box)) != KSMM_OK) return st;
  }
  Params P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.nk = (p.c + KC - 1) / KC;
  P.alpha = p.alpha;
  P.bias = p.bias;
  P.out_dtype = p.out_dtype;
  P.act = p.activation;
  P.rg_d = (!OUT_LAST && OS == 2) ? p.out_regroup_d : 0;
  P.rg_c = p.out_regroup_c;
  P.groups = static_cast<int>(G);
  P.gx = GX > 1 ? 1 : 0;
  P.residual = p.residual;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;  // f16 / e4m3 = 0, bf16 = 1
  // fp32 accumulate; bit 15 / 16: the A / B operand is MN-major.  Weights always are; the input
  // is when it is batch-last.  A = weights for a batch-last output, else the input.
  const uint32_t a_mn = (OUT_LAST || IN_LAST) ? 1u : 0u, b_mn = (!OUT_LAST || IN_LAST) ? 1u : 0u;
  uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn << 15) | (b_mn << 16) |
                   (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  if (IN_LAST) {
    const uint64_t xd[4] = {B, d, c, GX * a};
    const uint64_t xs[4] = {1, B, d * B, c * d * B};
    const uint32_t xb[4] = {static_cast<uint32_t>(C::NBOX), 1, static_cast<uint32_t>(KC), 1};
    if ((st = encode_map(&tmX, p.in_dtype, 4, p.in, xd, xs, xb)) != KSMM_OK) return st;
  } else {
    const uint64_t xd[3] = {c, a, GX * B};
    const uint64_t xs[3] = {1, c, a * c};
    const uint32_t xb[3] = {static_cast<uint32_t>(KC), 1, static_cast<uint32_t>(C::XN)};
    if ((st = encode_map(&tmX, p.in_dtype, 3, p.in, xd, xs, xb)) != KSMM_OK) return st;
  }
  if (OUT_LAST) {
    const uint64_t yd[4] = {B, d, b, G * a};
    const uint64_t ys[4] = {1, B, d * B, b * d * B};
    const uint32_t yb[4] = {static_cast<uint32_t>(C::CB), 1, 32, 1};  // one epilogue warp's rows
    if ((st = encode_map(&tmY, p.out_dtype, 4, p.out, yd, ys, yb)) != KSMM_OK) return st;
  } else if (p.out_regroup_d > 0 && OS == 2) {
    // regrouped output (k2, l2, i2, n): a staging tile of 64 features is d2 runs of 64 / d2
    const uint64_t c2 = p.out_regroup_c, d2 = p.out_regroup_d;
    const uint64_t yd[4] = {c2, d2, a * b / (c2 * d2), B};
    const uint64_t ys[4] = {1, c2, c2 * d2, a * b};
    const uint32_t yb[4] = {static_cast<uint32_t>(C::CB / d2), static_cast<uint32_t>(d2), 1, 32};
    if ((st = encode_map(&tmY, p.out_dtype, 4, p.out, yd, ys, yb, false)) != KSMM_OK) return st;
  } else {
    const uint64_t yd[3] = {b, a, G * B};
    const uint64_t ys[3] = {1, b, a * b};
    const uint32_t yb[3] = {static_cast<uint32_t>(C::CB), 1, 32};
    if ((st = encode_map(&tmY, p.out_dtype, 3, p.out, yd, ys, yb)) != KSMM_OK) return st;
  }
  P.tiles_n = static_cast<int>((B + C::XN - 1) / C::XN);
  P.tiles_j = static_cast<int>((b + C::WJ - 1) / C::WJ);
  P.idesc = idesc;
  const int sms = num_sms();
  if (sms <= 0) return set_error(KSMM_ERR_NO_DEVICE, "no CUDA device");
  P.tiles_jg = P.tiles_j * static_cast<int>(G);
  const int64_t rows = static_cast<int64_t>(P.tiles_n) * p.a * p.d;
  const int slots = sms * C::CTAS;  // CTAs resident at the same time
  if (rows <= 0 || rows > 0x7fffffffLL || P.tiles_jg > sms)
    return set_error(KSMM_ERR_UNSUPPORTED,
                     "tensor-core family: %lld rows x %d j tiles exceed the work-split limits",
                     static_cast<long long>(rows), P.tiles_jg);
  P.rows = static_cast<uint32_t>(rows);
  int64_t groups = slots / P.tiles_jg;
  if (groups > rows) groups = rows;
  P.row_groups = static_cast<uint32_t>(groups);
  const unsigned grid = static_cast<unsigned>(groups * P.tiles_jg);
  cudaError_t err = launch_pdl(kern, grid, kThreads, C::SMEM_BYTES, stream, tmX, tmW, tmY, P);
  count_launch();
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

// Tile configurations.  Each has a weight-stationary and a streaming flavour;
// the first is used when all k chunks of the weight tile fit in its NWC slots.
//   <layout, ES, OS, N tile, bytes of k per chunk row, resident weight chunks,
//    ring stages (weight-stationary), ring stages (streaming)>
template <bool IN_LAST, bool OUT_LAST, int ES, int OS, int NT, int KCB, int NWC, int SX_W, int SX_S, int STGN = 1>
static int launch_flavour(const Problem& p, cudaStream_t stream) {
  constexpr int KC = KCB / ES;
  const int nk = (p.c + KC - 1) / KC;
  if (nk <= NWC) return launch_one<IN_LAST, OUT_LAST, ES, OS, NT, KC, true, NWC, SX_W, STGN>(p, stream);
  return launch_one<IN_LAST, OUT_LAST, ES, OS, NT, KC, false, 0, SX_S, STGN>(p, stream);
}

template <bool BS_LAST, int ES, int OS>
static int launch_cfg(const Problem& p, int config, cudaStream_t stream) {
  // batch-last, 16-bit: input chunk = NT x 64 x 2 bytes, weight chunk = 16 KB
  // batch-first, 16-bit: input chunk = 16 KB, weight chunk = NT x 64 x 2 bytes
  if constexpr (BS_LAST) {
    switch (config) {
      case 0: return launch_flavour<true, true, ES, OS, 256, 128, 3, 4, 4>(p, stream);
      case 1: return launch_flavour<true, true, ES, OS, 128, 128, 6, 6, 6>(p, stream);
      case 2: return launch_flavour<true, true, ES, OS, 256, 128, 1, 5, 4>(p, stream);
      case 3: return launch_flavour<true, true, ES, OS, 128, 128, 3, 8, 6>(p, stream);
      case 4:
        if constexpr (ES == 2) return launch_flavour<true, true, ES, OS, 64, 128, 6, 8, 8>(p, stream);
        break;
      case 5:  // two CTAs per SM: short rings, more independent pipelines in flight
        return launch_flavour<true, true, ES, OS, 128, 128, 1, 3, 2>(p, stream);
      case 6:  // two staging tiles per epilogue warp, short blocks
        return launch_flavour<true, true, ES, OS, 256, 128, 1, 4, 3, 2>(p, stream);
      case 7:  // two staging tiles per epilogue warp
        return launch_flavour<true, true, ES, OS, 256, 128, 3, 3, 3, 2>(p, stream);
    }
  } else {
    switch (config) {
      case 0: return launch_flavour<false, false, ES, OS, 256, 128, 3, 6, 4>(p, stream);
      case 1: return launch_flavour<false, false, ES, OS, 128, 128, 6, 6, 6>(p, stream);
      case 2: return launch_flavour<false, false, ES, OS, 256, 128, 1, 10, 4>(p, stream);
      case 3: return launch_flavour<false, false, ES, OS, 128, 128, 3, 8, 6>(p, stream);
      case 4:
        if constexpr (ES == 2) return launch_flavour<false, false, ES, OS, 64, 128, 6, 8, 8>(p, stream);
        break;
      case 5:
        return launch_flavour<false, false, ES, OS, 128, 128, 1, 3, 2>(p, stream);
      case 6:
        return launch_flavour<false, false, ES, OS, 256, 128, 1, 8, 3, 2>(p, stream);
      case 7:
        return launch_flavour<false, false, ES, OS, 256, 128, 3, 4, 3, 2>(p, stream);
    }
  }
  return set_error(KSMM_ERR_BAD_ARGUMENT, "tensor-core family: no configuration %d", config);
}

// Layout-changing factors (d = 1, 16-bit): the tile shapes of the output's layout, configurations
// 0, 1 and 4 of it (the other two differ only in ring depth).
template <bool IN_LAST>
static int launch_mixed(const Problem& p, int config, cudaStream_t stream) {
  constexpr bool OUT_LAST = !IN_LAST;
  if (config == 2 || config == 6 || config == 7) config = 0;
  if (config == 3 || config == 5) config = 1;
  switch (config) {
    case 0: return launch_flavour<IN_LAST, OUT_LAST, 2, 2, 256, 128, 3, OUT_LAST ? 4 : 6, 4>(p, stream);
    case 1: return launch_flavour<IN_LAST, OUT_LAST, 2, 2, 128, 128, 6, 6, 6>(p, stream);
    case 4: return launch_flavour<IN_LAST, OUT_LAST, 2, 2, 64, 128, 6, 8, 8>(p, stream);
  }
  return set_error(KSMM_ERR_BAD_ARGUMENT, "tensor-core family: no configuration %d", config);
}

}  // namespace tc

int tc_num_configs() { return tc::kNumConfigs; }

bool tc_config_supported(const Problem& p, int config, bool check_pointers) {
  if (config < 0 || config >= tc::kNumConfigs) return false;
  if (p.groups > 1) {
    // grouped launches exist in the 16-bit / 8-bit kernel of this file only; batch-first outputs of
    // the groups follow one another row-wise, so a partly filled last store box would spill into
    // the next group: the batch has to be a whole number of 32-row boxes
    if (p.in_dtype == KSMM_F32 || (!p.bs_last && (p.d != 1 || p.batch % 32 != 0))) return false;
    if (p.out_regroup_d || p.in_regrouped) return false;
    if (static_cast<int64_t>(p.groups) * p.batch > 0x7fffffffLL ||
        static_cast<int64_t>(p.groups) * p.a * p.d > 0x7fffffffLL)
      return false;
  }
  const bool out_last = p.out_bs_last < 0 ? p.bs_last != 0 : p.out_bs_last != 0;
  if (out_last != (p.bs_last != 0)) {
    // a factor that changes the layout: 16-bit, d = 1, no groups, no regrouping
    if (p.d != 1 || p.groups > 1 || p.out_regroup_d || p.in_regrouped) return false;
    if (p.in_dtype == KSMM_F32) return config >= 0 && config <= 3 && tc_f32x3_supported(p, check_pointers);
    if ((p.in_dtype != KSMM_F16 && p.in_dtype != KSMM_BF16) || p.out_dtype != p.in_dtype) return false;
    if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
    if (p.b % 8 != 0 || p.c % 8 != 0 || p.batch % 8 != 0) return false;   // 16-byte strides on both sides
    if (check_pointers && (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
                           reinterpret_cast<uintptr_t>(p.out) % 16))
      return false;
    return true;
  }
  if (p.in_dtype == KSMM_F32) return config >= 0 && config <= 3 && tc_f32x3_supported(p, check_pointers);
  if (!p.bs_last && p.d != 1) {
    if (p.d % 8 == 0) return config == 0 && tc_bsfirst_g_supported(p, check_pointers);
    return config == 0 ? tc_bsfirst_d_supported(p, check_pointers)
                       : (config == 1 && tc_bsfirst_dp_supported(p, check_pointers));
  }
  if (config == 4 && p.in_dtype == KSMM_F8E4M3) return false;
  const int es = dtype_size(p.in_dtype), os = dtype_size(p.out_dtype);
  if (p.in_dtype == KSMM_F16 || p.in_dtype == KSMM_BF16) {
    if (p.out_dtype != p.in_dtype) return false;
  } else if (p.in_dtype != KSMM_F8E4M3) {
    return false;
  }
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  // tensor-map rules: every global stride is a multiple of 16 bytes
  if ((static_cast<int64_t>(p.b) * es) % 16 != 0) return false;
  if (p.bs_last) {
    if ((p.batch * es) % 16 != 0 || (p.batch * os) % 16 != 0) return false;
  } else {
    if (p.d != 1) return false;
    if ((static_cast<int64_t>(p.c) * es) % 16 != 0) return false;
    if ((static_cast<int64_t>(p.b) * os) % 16 != 0) return false;
  }
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16)
      return false;
  }
  return true;
}

bool tc_can_regroup_output(const Problem& p) {
  // the 16-bit batch-first d = 1 kernel, whole 64-feature staging tiles that stay inside one
  // block row of the next factor
  if (p.bs_last || p.d != 1 || (p.in_dtype != KSMM_F16 && p.in_dtype != KSMM_BF16)) return false;
  if (p.out_dtype != p.in_dtype || p.b % 64 != 0) return false;
  const int d2 = p.out_regroup_d, c2 = p.out_regroup_c;
  if ((d2 != 2 && d2 != 4) || c2 <= 0 || (c2 * d2) % 64 != 0 || c2 % 8 != 0) return false;
  return (static_cast<int64_t>(p.a) * p.b) % (static_cast<int64_t>(c2) * d2) == 0 && tc_default_config(p) >= 0;
}

// true if the kernel that tc_launch would run for `p` adds p.residual in its epilogue (the 16-bit /
// 8-bit kernel of this file; the other kernels of the family leave it to a pass after them)
bool tc_fuses_residual(const Problem& p) {
  if (p.in_dtype == KSMM_F32) return false;
  const bool out_last = p.out_bs_last < 0 ? p.bs_last != 0 : p.out_bs_last != 0;
  if (out_last == (p.bs_last != 0) && !p.bs_last && p.d != 1) return false;
  if (p.groups > 1 || p.out_regroup_d) return false;
  return reinterpret_cast<uintptr_t>(p.residual) % 16 == 0;
}

int tc_default_config(const Problem& p) {
  if (!tc_config_supported(p, 0, true)) return -1;
  // tiny blocks are bandwidth problems that the FFMA family tiles more tightly
  if (p.b < 32 || p.c < 16) return -1;
  // fp32 on the tensor cores: the accumulator truncates once per k step of 8, so the default
  // stops at c = 1024 (relative error about 2e-6 at c = 768); longer sums take the FFMA family
  if (p.in_dtype == KSMM_F32) return p.c <= 1024 ? 0 : -1;
  // batch-first, d = 2 or 4: the in-kernel split (configuration 0).  Configuration 1 (regrouping pass,
  // then the kernel without the transposer stage) measured slower for a single factor (94 us
  // against 85 us for (1,768,192,4) fp16); chains use its kernel when the previous factor can
  // store the intermediate regrouped for free.
  const bool out_last = p.out_bs_last < 0 ? p.bs_last != 0 : p.out_bs_last != 0;
  if (out_last == (p.bs_last != 0) && !p.bs_last && p.d != 1) {
    // The eight-block kernel moves 16-byte pieces that lie d elements apart: at d = 16 it beats the
    // layout conversion (39 against 61 us for (1,64,64,16) fp16 at 25088 rows), at d = 24 the two
    // are level, beyond that the conversion wins by far (299 against 734 us for (1,48,48,96)).
    // It stays available as configuration 0 of the family.
    if (p.d % 8 == 0 && p.d > 16) return -1;
    return 0;
  }
  // 64 x 64 blocks are copies with one MMA chunk per tile: two smaller CTAs per SM keep more loads
  // and stores in flight (configuration 5; tuned at batch 25088: 23.0 against 24.0 us batch-last,
  // 24.1 against 26.5 us batch-first for the 16-block patterns)
  const bool small16 = p.in_dtype != KSMM_F8E4M3 && p.b <= 64 && p.c <= 64 && p.batch >= 4096;
  if (out_last) return small16 ? 5 : (p.batch >= 256 * 148 / 2 || p.batch >= 4096 ? 0 : 1);
  return p.b > 128 ? 0 : (p.b > 64 ? 1 : (small16 ? 5 : 4));
}

int tc_launch(const Problem& p, int config, cudaStream_t stream) {
  if (config < 0) config = tc_default_config(p);
  if (config < 0 || !tc_config_supported(p, config, true))
    return set_error(KSMM_ERR_UNSUPPORTED,
                     "tensor-core family cannot run pattern (%d,%d,%d,%d) batch %lld dtype %d "
                     "bs_last %d (alignment or layout rule)",
                     p.a, p.b, p.c, p.d, static_cast<long long>(p.batch), p.in_dtype, p.bs_last);
  const bool last = p.bs_last != 0;
  const bool out_last = p.out_bs_last < 0 ? last : p.out_bs_last != 0;
  if (p.in_dtype == KSMM_F32) return tc_f32x3_launch(p, config, stream);
  if (out_last != last) return last ? tc::launch_mixed<true>(p, config, stream) : tc::launch_mixed<false>(p, config, stream);
  if (!last && p.d != 1) {
    if (p.d % 8 == 0) return tc_bsfirst_g_launch(p, stream);
    return config == 1 ? tc_bsfirst_dp_launch(p, stream) : tc_bsfirst_d_launch(p, stream);
  }
  if (p.out_regroup_d > 0 && !tc_can_regroup_output(p))
    return set_error(KSMM_ERR_UNSUPPORTED, "this factor cannot store a regrouped output");
  if (p.in_dtype == KSMM_F8E4M3) {
    if (p.out_dtype == KSMM_F32)
      return last ? tc::launch_cfg<true, 1, 4>(p, config, stream)
                  : tc::launch_cfg<false, 1, 4>(p, config, stream);
    return last ? tc::launch_cfg<true, 1, 2>(p, config, stream)
                : tc::launch_cfg<false, 1, 2>(p, config, stream);
  }
  return last ? tc::launch_cfg<true, 2, 2>(p, config, stream)
              : tc::launch_cfg<false, 2, 2>(p, config, stream);
}

#ifdef KSMM_TC_TRACE
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace(unsigned long long* host) {
  cudaDeviceSynchronize();
  return static_cast<int>(cudaMemcpyFromSymbol(host, tc::g_trace, sizeof(tc::g_trace)));
}
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace_clear() {
  static unsigned long long zeros[4][8192];
  return static_cast<int>(cudaMemcpyToSymbol(tc::g_trace, zeros, sizeof(zeros)));
}
#endif

// One warp waits on an mbarrier that nothing ever arrives on, through the same bounded wait as
// the kernels above but with a caller-chosen limit: the wait runs out, the status word takes
// `code`, the warp returns.  Lets a test see the whole timeout path (device flag ->
// tc_check_device -> KSMM_ERR_DEVICE_TIMEOUT) without a faulting or hanging kernel.
namespace tc {
__global__ void __launch_bounds__(32) wait_probe_kernel(long long limit_cycles, int code, int* status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_wait<64>(b, 0u, &abort_flag, status, code, limit_cycles);
  __syncwarp();
}
}  // namespace tc

int tc_wait_probe(long long limit_cycles, int code, cudaStream_t stream) {
  int* w = tc::status_word();
  if (!w) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  tc::wait_probe_kernel<<<1, 32, 0, stream>>>(limit_cycles, code, w);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "wait probe launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

int tc_check_device(cudaStream_t stream) {
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "stream synchronisation failed: %s", cudaGetErrorString(e));
  int* w = tc::status_word();
  if (!w) return KSMM_OK;
  int code = 0;
  e = cudaMemcpy(&code, w, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "cannot read the device status word: %s",
                     cudaGetErrorString(e));
  if (code != 0) {
    int zero = 0;
    cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return set_error(KSMM_ERR_DEVICE_TIMEOUT,
                     "a tensor-core kernel gave up waiting (code %d: 1 producer/input slot, "
                     "2 producer/weight stage, 3 mma/accumulator, 4 mma/input, 5 mma/weights, "
                     "6 epilogue/accumulator)",
                     code);
  }
  return KSMM_OK;
}

}  // namespace ksmm
