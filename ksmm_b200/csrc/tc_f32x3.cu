// fp32 factors on the tensor cores: tcgen05 kind::tf32 with a three-term split
// ("3xTF32"), fp32 accumulation in TMEM.  Kernel family KSMM_ALGO_TC for fp32
// inputs, batch-last (any d) and batch-first (d = 1).
//
// A tf32 operand keeps the upper 19 bits of an fp32 value; the tensor core
// ignores the other 13 mantissa bits (it truncates, it does not round).  Every
// fp32 operand v is therefore used twice: once as it is (the hardware sees
// hi = trunc(v)) and once as lo = v - trunc(v), which is exact in fp32.  The
// product x * w is accumulated as
//     hi(x) hi(w) + lo(x) hi(w) + hi(x) lo(w),
// two MMAs per k step (hi(x) against the stacked rows [hi(w) | lo(w)], N = 2 NJ,
// and lo(x) against hi(w), N = NJ); the dropped lo * lo term and the truncation of lo
// itself are of relative size 2^-22.  The tensor core also truncates when it
// adds into the fp32 accumulator, once per MMA, and that error grows with the
// number of accumulations: the two small terms therefore go to an accumulator
// of their own (their truncation is 2^-11 times smaller) and are added to the
// leading one in the epilogue, which leaves c / 8 truncating additions on the
// leading accumulator.  Relative Frobenius error against an fp64 oracle: about
// 5e-7 to 8e-7 for c <= 192 and 2e-6 for c = 768, inside the 1e-5 of the reference's own
// fp32 check (src/ksmm_cu/src/template_sparse_mm.cu:873-880); the default
// dispatch uses this kernel up to c = 1024.  The exact FFMA kernels stay
// available as KSMM_ALGO_SIMT.
//
// Operand tiles come from TMA in the layout the tensor core reads, so the raw
// tile is the hi operand as it stands.  The batch-last input X[(i, k, l), n] and
// the weights W[(i, l, k), j] have k as their row index: they are MN-major
// operands, which for 32-bit elements use the 128-byte swizzle with 32-byte
// atoms (tile of 32 x-values by 32 k rows of 128 bytes; the 32-byte piece p of row k
// sits at p ^ (k % 4); CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B on the TMA side,
// descriptor layout type 1 on the MMA side).  The batch-first input rows hold
// consecutive k: K-major, plain 128-byte swizzle.  Two groups of four
// "splitter" warps only add the lo tiles, element by element at the same
// offsets (16-byte loads and stores).  The lo weights follow the hi weights
// directly, so the two together are one operand of 2 NJ rows.
//
// Three forms, chosen by the launcher:
//  * j tile of 128 columns: both operands from shared memory, one stage holds
//    [X hi | X lo | W hi | W lo].  The accumulators (2 buffers x 2 x 128 columns)
//    fill the tensor memory.
//  * j tile of 96 or 64 columns (TS): the input operand is read from tensor
//    memory.  The input splitters read the raw tile (one accumulator row = one
//    thread, through the swizzle) and write hi and lo with tcgen05.st into one of
//    two operand buffers of 64 columns behind the accumulators; a stage is
//    [X raw | W hi | W lo].  This removes the lo tile of the input and the tensor
//    core's reads of the input operand from the shared-memory pipe, the unit
//    that bounds the first form.
//  * the same with resident weights (WR; batch-last, 96 columns, c <= 192): the
//    hi and lo weights of the CTA's j tile stay in shared memory for all batch
//    tiles of a block (loaded and split once per block, after the MMAs of the
//    previous block have completed), a stage is the raw input tile alone, and
//    the four weight warps join the epilogue as a third column group, so that
//    each of the twelve warps stores 32 of the 96 columns.  On short blocks the
//    epilogue's stores, not the main loop, set the time per tile.
//
// Warp roles (576 threads): warp 0 TMA producer, warp 1 TMEM owner and MMA
// issuer, warps 2..5 input splitters, warps 6..9 weight splitters, warps
// 10..17 epilogue (TMEM lane quarter = warp index mod 4, which also fixes the
// accumulator rows an input splitter can write).  Accumulator rows
// are batch entries, columns are j.  A CTA keeps one j tile and walks a
// contiguous range of (block, batch tile) pairs.  Per chunk of 32 k there are three
// hand-offs: TMA -> splitters (one barrier for both tiles), splitters -> MMA
// thread (one arrival per splitter warp), MMA commit -> producer; an operand
// buffer in tensor memory is free again when the commit of the chunk two
// iterations back has arrived.  Waits are bounded and
// report through the status word as in tc_kernel.cu.
//
// Shapes: b a multiple of 32 and, batch-last, a batch that is a multiple of 32 (the tiles are
// addressed in atoms of 32 columns); batch-first needs d = 1 and c a multiple of 4.
//
// Reference counterparts: kernel_bs_last_float / kernel_bs_first_float
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_float.cuh:301-491, 51-299).
#include <cuda.h>

#include <atomic>

#include "tc_host.h"
#include "tc_kernel.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace tc {

struct ParamsF {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  uint32_t rows;        // blocks * tiles_n: (block, batch tile) pairs
  uint32_t row_groups;  // CTAs per j tile
  int nchunks;          // ceil(c / 32)
  uint32_t idesc;   // N = NJ
  uint32_t idesc2;  // N = 2 NJ
  float alpha;
  const float* bias;
  float* out;  // batch-last: the epilogue stores straight from registers
  int act;     // ksmm_activation_t
  int* status;
};

constexpr int kThreadsF = (2 + 4 + 4 + kEpilogueWarps) * 32;
constexpr int kKC = 32;  // k values per chunk (128 bytes of fp32)

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// same MMA with the A operand (128 rows x 8 k, one 32-bit column per k) read from tensor memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ uint32_t lo_part(uint32_t v) {
  return __float_as_uint(__uint_as_float(v) - __uint_as_float(v & 0xFFFFE000u));
}

// ST stages of [X hi | X lo | W hi | W lo]; with TS the input operand lives in tensor memory and a
// stage is [X raw | W hi | W lo].
// With WR (needs TS and c <= 32 kMaxResident) the hi and lo weights of the CTA's j tile stay in shared
// memory for all batch tiles of a block, and a stage is the raw input tile alone.
constexpr int kMaxResident = 6;  // chunks of 32 k

// IN_LAST / BS_LAST: layout of the input / of the output.  The accumulator's rows are batch entries
// in every form, so the input side (tensor map, producer, splitter, operand descriptors) and the
// output side (epilogue, stores, bias index) combine freely; the two mixed forms need d = 1.
template <bool IN_LAST, bool BS_LAST, int NJ_, int ST_, bool TS_, bool DIRECT_, bool WR_>
struct CfgF {
  static constexpr int NJ = NJ_;                    // j columns per accumulator (64, 96 or 128)
  static constexpr int ST = ST_;
  static constexpr bool TS = TS_;
  static constexpr bool WR = WR_;
  static_assert(!WR || (TS && BS_LAST && IN_LAST && DIRECT_),
                "resident weights come with the tensor-memory input operand and direct stores");
  static constexpr int XT_BYTES = kKC * 128 * 4;    // 32 k x 128 batch entries (either order)
  static constexpr int WT_BYTES = kKC * NJ * 4;     // 32 k x NJ columns
  static constexpr int W_OFF = TS ? XT_BYTES : 2 * XT_BYTES;
  static constexpr int STAGE_BYTES = WR ? XT_BYTES : W_OFF + 2 * WT_BYTES;
  static constexpr int WRES_BYTES = WR ? kMaxResident * 2 * WT_BYTES : 0;
  static constexpr int STG_WARP_BYTES = 32 * 128;   // 32 rows of 32 fp32
  // batch-last can do without staging: a warp's 32 lanes hold 32 consecutive batch entries of
  // one output row, so a plain store already writes a whole 128-byte line
  static constexpr bool DIRECT = BS_LAST && DIRECT_;
  static constexpr int STG_BYTES = DIRECT ? 0 : kEpilogueWarps * STG_WARP_BYTES;
  // barriers per stage: tiles landed, lo tiles written, stage free; tmem full/empty
  // + weights landed, weights split (resident weights only)
  static constexpr int NBAR = 3 * ST + 6;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = STG_BYTES + WRES_BYTES + ST * STAGE_BYTES + BAR_BYTES + 1024;
  static constexpr int NBUF = 2;
  static constexpr int BUF_COLS = 2 * NJ;  // leading accumulator | small-terms accumulator
  // TS: two operand buffers of [hi: 32 k | lo: 32 k] columns behind the accumulators
  static constexpr int A_COL0 = NBUF * BUF_COLS;
  static constexpr int A_BUF_COLS = 2 * kKC;
  static constexpr int USED_COLS = A_COL0 + (TS ? 2 * A_BUF_COLS : 0);
  // allocations are powers of two
  static constexpr int TMEM_COLS = USED_COLS <= 128 ? 128 : (USED_COLS <= 256 ? 256 : 512);
  static_assert(USED_COLS <= 512, "tensor memory budget");
  static_assert(NJ == 64 || NJ == 96 || NJ == 128, "j tile");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM, so that the TMEM allocation never waits");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
};

template <bool IN_LAST, bool BS_LAST, int NJ_, int ST_, bool TS_, bool DIRECT_, bool WR_>
__global__ void __launch_bounds__(kThreadsF, 1)
    ksmm_tc_f32x3_kernel(const __grid_constant__ CUtensorMap tmX,
                         const __grid_constant__ CUtensorMap tmW,
                         const __grid_constant__ CUtensorMap tmY, const ParamsF P) {
  using C = CfgF<IN_LAST, BS_LAST, NJ_, ST_, TS_, DIRECT_, WR_>;
  constexpr int ST = C::ST;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t stg0 = sm0;                     // epilogue staging tiles
  const uint32_t wres0 = stg0 + C::STG_BYTES;    // resident weights: per chunk [hi | lo]
  const uint32_t stage0 = wres0 + C::WRES_BYTES;  // operand stages
  const uint32_t bar0 = stage0 + ST * C::STAGE_BYTES;
  uint8_t* bar_gen = sm_gen + (bar0 - sm0);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };             // TMA: X hi and W hi landed
  auto split_bar = [&](int s) { return bar0 + 8u * (ST + s); };     // splitters: lo tiles written
  auto free_bar = [&](int s) { return bar0 + 8u * (2 * ST + s); };  // MMA commit: stage consumed
  auto tfull_bar = [&](int q) { return bar0 + 8u * (3 * ST + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (3 * ST + 2 + q); };
  auto wfull_bar = [&]() { return bar0 + 8u * (3 * ST + 4); };   // TMA: a block's hi weights landed
  auto wsplit_bar = [&]() { return bar0 + 8u * (3 * ST + 5); };  // weight splitters: lo weights written
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * C::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * C::NBAR + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(split_bar(s), C::WR ? 4 : 8);  // four input-splitter (and four weight-splitter) warps
      mbar_init(free_bar(s), 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(tfull_bar(q), 1);
      mbar_init(tempty_bar(q), kEpilogueWarps + (C::WR ? 4 : 0));
    }
    mbar_init(wfull_bar(), 1);
    mbar_init(wsplit_bar(), 4);
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
      uint32_t si = 0, sph = 0, last_si = 0, last_ph = 0;
      int cur_blk = -1;
      (void)last_si; (void)last_ph; (void)cur_blk;
      bool ok = true;
      KSMM_TRACE_DECL;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        const int blk = static_cast<int>(row / P.tiles_n);  // batch-last: (i, l); batch-first: i
        const int n0 = static_cast<int>(row % P.tiles_n) * 128;
        if constexpr (C::WR) {
          if (blk != cur_blk) {
            // new block: once every MMA issued so far has completed (the commit of the last stage
            // covers them all), its weights replace the resident ones
            if (cur_blk >= 0 && !mbar_wait<64>(free_bar(last_si), last_ph, abort_flag, P.status, 39)) {
              ok = false;
              break;
            }
            mbar_expect_tx(wfull_bar(), static_cast<uint32_t>(nchunks) * C::WT_BYTES);
            for (int qc = 0; qc < nchunks; ++qc)
              tma_load_4d(wres0 + qc * 2 * C::WT_BYTES, &tmW, wfull_bar(), 0, qc * kKC, j0 / 32, blk);
            cur_blk = blk;
          }
        }
        for (int qc = 0; qc < nchunks; ++qc) {
          KSMM_TRACE(0, 1);
          if (!mbar_wait<64>(free_bar(si), sph ^ 1u, abort_flag, P.status, 31)) { ok = false; break; }
          KSMM_TRACE(0, 2);
          const uint32_t sb = stage0 + si * C::STAGE_BYTES;
          mbar_expect_tx(full_bar(si), C::XT_BYTES + (C::WR ? 0 : C::WT_BYTES));
          if constexpr (IN_LAST) {
            // (n % 32, k, n / 32, l, i): four atoms of 32 batch entries x 32 k rows
            tma_load_5d(sb, &tmX, full_bar(si), 0, qc * kKC, n0 / 32, blk % P.d, blk / P.d);
          } else {
            tma_load_3d(sb, &tmX, full_bar(si), qc * kKC, blk, n0);
          }
          // (j % 32, k, j / 32, block): NJ / 32 atoms of 32 columns x 32 k rows
          if constexpr (!C::WR) tma_load_4d(sb + C::W_OFF, &tmW, full_bar(si), 0, qc * kKC, j0 / 32, blk);
          KSMM_TRACE(0, 3);
          last_si = si;
          last_ph = sph;
          if (++si == ST) { si = 0; sph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t si = 0, sph = 0, ut = 0, ab = 0, wph = 0;
      int cur_blk = -1;
      (void)wph; (void)cur_blk;
      bool ok = true;
      KSMM_TRACE_DECL;
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
        KSMM_TRACE(1, 10);
        if (!mbar_wait<0>(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 33)) { ok = false; break; }
        KSMM_TRACE(1, 11);
        if constexpr (C::WR) {
          const int blk = static_cast<int>(row / P.tiles_n);
          if (blk != cur_blk) {
            // the block's weights, hi and lo, are in place
            if (!mbar_wait<0>(wsplit_bar(), wph, abort_flag, P.status, 38)) { ok = false; break; }
            wph ^= 1u;
            cur_blk = blk;
          }
        }
        tc_fence_after();
        const uint32_t dcol = tmem_base + buf * C::BUF_COLS, dsmall = dcol + C::NJ;
        for (int qc = 0; qc < nchunks; ++qc) {
          KSMM_TRACE(1, 12);
          if (!mbar_wait<0>(split_bar(si), sph, abort_flag, P.status, 35)) { ok = false; break; }
          KSMM_TRACE(1, 13);
          tc_fence_after();
          const uint32_t xb = stage0 + si * C::STAGE_BYTES;
          const uint32_t wb = C::WR ? wres0 + qc * 2 * C::WT_BYTES : xb + C::W_OFF;
#pragma unroll
          for (int ks = 0; ks < kKC / 8; ++ks) {
            // weights: MN-major, the NJ / 32 hi atoms and then the NJ / 32 lo atoms
            const uint64_t wst = make_desc(wb + ks * 1024, 4096, 512, 1);
            const uint32_t acc = (qc | ks) != 0 ? 1u : 0u;
            if constexpr (C::TS) {
              const uint32_t ahi = tmem_base + C::A_COL0 + ab * C::A_BUF_COLS + ks * 8;
              umma_tf32_ts(dcol, ahi, wst, P.idesc2, acc);
              umma_tf32_ts(dsmall, ahi + kKC, wst, P.idesc, 1u);
              continue;
            }
            uint64_t xhi, xlo;
            if constexpr (IN_LAST) {
              // MN-major, 32-byte atoms: 4 KB between the atoms of 32 batch entries, 512 bytes
              // between groups of 4 k rows; a k step of 8 is two groups
              xhi = make_desc(xb + ks * 1024, 4096, 512, 1);
              xlo = make_desc(xb + C::XT_BYTES + ks * 1024, 4096, 512, 1);
            } else {
              // K-major rows of 32 k with the 128-byte swizzle; a k step is 32 bytes inside the row
              xhi = make_desc(xb + ks * 32, 16, 1024, 2);
              xlo = make_desc(xb + C::XT_BYTES + ks * 32, 16, 1024, 2);
            }
            // hi(x) * [hi(w) | lo(w)]: the leading accumulator and, next to it, the small one
            umma_tf32(dcol, xhi, wst, P.idesc2, acc);
            // lo(x) * hi(w): only the first NJ rows of the same operand
            umma_tf32(dsmall, xlo, wst, P.idesc, 1u);
          }
          KSMM_TRACE(1, 19);
          umma_commit(free_bar(si));
          ab ^= 1u;
          if (++si == ST) { si = 0; sph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));
      }
    }
    __syncwarp();
  } else if (warp < (C::WR ? 6 : 10)) {
    // ===================== splitters =====================
    // warps 2..5: lo tile of the input, warps 6..9: lo tile of the weights; same offsets as the
    // hi tile, so the swizzle does not matter here
    const bool on_w = warp >= 6;
    const int tt = ((warp - 2) & 3) * 32 + lane;
    const uint32_t off0 = on_w ? C::W_OFF : 0u;
    const uint32_t tile_bytes = on_w ? C::WT_BYTES : C::XT_BYTES;
    uint32_t si = 0, sph = 0;
    // TS: the operand buffer written in iteration t is read by the MMAs of iteration t and was
    // last read by those of iteration t - 2, whose commit is the free barrier of stage (t - 2) % ST
    uint32_t iter = 0, s2 = 0, ph2 = 0;
    bool ok = true;
    KSMM_TRACE_DECL;
    const bool tron = warp == 2 && lane == 0;
    const int trole = on_w ? 3 : 2;
    (void)tron; (void)trole;
    for (uint32_t row = row_begin; row < row_end && ok; ++row) {
      for (int qc = 0; qc < nchunks; ++qc) {
        int got = 1;
        if (tron) KSMM_TRACE(trole, 30);
        if (lane == 0) got = mbar_wait<32>(full_bar(si), sph, abort_flag, P.status, 36) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        if (tron) KSMM_TRACE(trole, 33);
        const uint32_t hb = stage0 + si * C::STAGE_BYTES + off0, lb = hb + tile_bytes;
        const int npieces = static_cast<int>(tile_bytes / 16);
        if (C::TS && !on_w) {
          // thread = accumulator row tr (a warp reaches the TMEM lanes of its index mod 4 only):
          // its 32 k values go to tensor memory, as they are and as lo
          const int tr = (warp & 3) * 32 + lane;
          if (iter >= 2) {
            if (lane == 0) got = mbar_wait<32>(free_bar(s2), ph2, abort_flag, P.status, 37) ? 1 : 0;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) { ok = false; break; }
            if (++s2 == ST) { s2 = 0; ph2 ^= 1u; }
          }
          uint32_t v[kKC];
          if constexpr (IN_LAST) {
            // atom tr / 32 (32 batch entries x 32 k rows of 128 bytes), 32-byte piece p at p ^ (k % 4)
            const uint32_t ab0 = hb + (tr >> 5) * 4096 + (lane & 7) * 4;
#pragma unroll
            for (int k = 0; k < kKC; ++k)
              asm volatile("ld.shared.b32 %0, [%1];"
                           : "=r"(v[k])
                           : "r"(ab0 + k * 128 + ((((lane >> 3) ^ (k & 3))) << 5))
                           : "memory");
          } else {
            // row tr of 32 k (128 bytes), 16-byte chunk q at q ^ (row % 8)
            const uint32_t rb = hb + tr * 128;
#pragma unroll
            for (int ch = 0; ch < kKC / 4; ++ch)
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[4 * ch]), "=r"(v[4 * ch + 1]), "=r"(v[4 * ch + 2]), "=r"(v[4 * ch + 3])
                           : "r"(rb + ((ch ^ (tr & 7)) << 4))
                           : "memory");
          }
          tc_fence_after();
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(tr & ~31) << 16) + C::A_COL0 +
                              (iter & 1u) * C::A_BUF_COLS;
          tmem_st32(ta, v);
#pragma unroll
          for (int k = 0; k < kKC; ++k) v[k] = lo_part(v[k]);
          tmem_st32(ta + kKC, v);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(split_bar(si));
          if (tron) KSMM_TRACE(trole, 34);
          ++iter;
          if (++si == ST) { si = 0; sph ^= 1u; }
          continue;
        }
#pragma unroll 4
        for (int pc = tt; pc < npieces; pc += 128) {
          uint32_t v[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                       : "r"(hb + pc * 16)
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(lb + pc * 16),
                       "r"(lo_part(v[0])), "r"(lo_part(v[1])), "r"(lo_part(v[2])), "r"(lo_part(v[3]))
                       : "memory");
        }
        fence_proxy_async();  // the tiles are read by the tensor core through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(split_bar(si));
        if (tron) KSMM_TRACE(trole, 34);
        if (++si == ST) { si = 0; sph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    // A warp owns 32 accumulator rows (batch entries) and every NG-th group of
    // 32 columns (j); one staging tile of 32 x 32 fp32 per TMA store.  With resident weights the
    // four weight warps are a third group: they split a block's weights when the CTA reaches
    // it and store accumulator columns the rest of the time.
    constexpr int NG = C::WR ? 3 : 2;
    const bool helper = warp < 10;
    const int ew = helper ? 0 : warp - 10;  // (helpers store directly and have no staging tile)
    const int q = warp & 3;
    const int grp = helper ? 2 : ew >> 2;
    uint32_t wph = 0;
    int cur_blk = -1;
    (void)wph; (void)cur_blk;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool plain = (P.alpha == 1.f) && (P.bias == nullptr) && (P.act == 0);
    const uint32_t stg = stg0 + ew * C::STG_WARP_BYTES;
    uint32_t ut = 0;
    KSMM_TRACE_DECL;
    const bool etr = warp == 10 && lane == 0;
    (void)etr;
    for (uint32_t row = row_begin; row < row_end; ++row, ++ut) {
      const int blk = static_cast<int>(row / P.tiles_n);
      const int n0 = static_cast<int>(row % P.tiles_n) * 128;
      const uint32_t buf = ut % C::NBUF, bph = (ut / C::NBUF) & 1u;
      int got = 1;
      if constexpr (C::WR) {
        if (helper && blk != cur_blk) {
          // lo tiles of all chunks of the block's weights
          cur_blk = blk;
          if (lane == 0) got = mbar_wait<32>(wfull_bar(), wph, abort_flag, P.status, 41) ? 1 : 0;
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) break;
          wph ^= 1u;
          constexpr int kPieces = C::WT_BYTES / 16;
          for (int pc = (warp - 6) * 32 + lane; pc < nchunks * kPieces; pc += 128) {
            const uint32_t hb = wres0 + (pc / kPieces) * 2 * C::WT_BYTES + (pc % kPieces) * 16;
            uint32_t v[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                         : "r"(hb)
                         : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(hb + C::WT_BYTES),
                         "r"(lo_part(v[0])), "r"(lo_part(v[1])), "r"(lo_part(v[2])), "r"(lo_part(v[3]))
                         : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(wsplit_bar());
        }
      }
      if (etr) KSMM_TRACE(3, 50);
      if (lane == 0) got = mbar_wait<128>(tfull_bar(buf), bph, abort_flag, P.status, 40) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      if (etr) KSMM_TRACE(3, 51);
      tc_fence_after();
      const bool warp_active = n0 + q * 32 < P.batch;
      // direct stores: row (i*b + j0)*d + l of the output, this lane's batch entry
      const int64_t n_row = static_cast<int64_t>(n0) + q * 32 + lane;
      const int64_t jstride = static_cast<int64_t>(P.d) * P.batch;
      float* row_out = P.out + ((static_cast<int64_t>(blk / P.d) * P.b + j0) * P.d + blk % P.d) * P.batch + n_row;
      (void)n_row; (void)jstride; (void)row_out;
      int jlim = P.b - j0;
      if (jlim > C::NJ) jlim = C::NJ;
      const int n_it = warp_active ? ((jlim + 31) / 32 - grp + NG - 1) / NG : 0;
      bool released = false;
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int jj0 = (grp + NG * it) * 32;
        uint32_t r[32], rs[32];
        tmem_ld32(tmem_base + lane_addr + buf * C::BUF_COLS + jj0, r);
        tmem_ld32(tmem_base + lane_addr + buf * C::BUF_COLS + C::NJ + jj0, rs);
        tmem_ld_wait();
        if (etr) KSMM_TRACE(3, 52);
        if (it == n_it - 1) {
          // the accumulator is in registers: the MMA warp may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(buf));
          released = true;
        }
#pragma unroll
        for (int jj = 0; jj < 32; ++jj)
          r[jj] = __float_as_uint(__uint_as_float(r[jj]) + __uint_as_float(rs[jj]));
        if (!plain) {
          // bias of this tile's 32 columns: lane t loads the one of column jj0 + t, shuffles broadcast
          float bl = 0.f;
          if (P.bias != nullptr && j0 + jj0 + lane < P.b) {
            const int j = j0 + jj0 + lane;
            // output feature: batch-last (i*b + j)*d + l with blk = i*d + l; batch-first i*b + j
            const int64_t f = BS_LAST ? (static_cast<int64_t>(blk / P.d) * P.b + j) * P.d + blk % P.d
                                      : static_cast<int64_t>(blk) * P.b + j;
            bl = P.bias[f];
          }
#pragma unroll
          for (int jj = 0; jj < 32; ++jj)
            r[jj] = __float_as_uint(fmaf(P.alpha, __uint_as_float(r[jj]), __shfl_sync(0xffffffffu, bl, jj)));
          if (P.act == KSMM_ACT_GELU) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(apply_activation(__uint_as_float(r[jj]), 1));
          } else if (P.act == KSMM_ACT_RELU) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) r[jj] = __float_as_uint(fmaxf(__uint_as_float(r[jj]), 0.f));
          }
        }
        if constexpr (C::DIRECT) {
          // lane = batch entry n, register jj = output row (i*b + j)*d + l: every store instruction
          // of the warp writes 32 consecutive floats of one row
          if (n_row < P.batch) {
            // few instructions per store: the warps of the epilogue run one dependent stream each,
            // and on short blocks their instruction count sets the time per tile
            float* dst = row_out + jj0 * jstride;
            if (j0 + jj0 + 32 <= P.b) {
#pragma unroll
              for (int jj = 0; jj < 32; ++jj) {
                *dst = __uint_as_float(r[jj]);
                dst += jstride;
              }
            } else {
#pragma unroll
              for (int jj = 0; jj < 32; ++jj)
                if (j0 + jj0 + jj < P.b) dst[jj * jstride] = __uint_as_float(r[jj]);
            }
          }
          if (etr) KSMM_TRACE(3, 53);
        } else {
          if (lane == 0) bulk_wait_read<0>();  // the previous store has read the staging tile
          __syncwarp();
          if constexpr (BS_LAST) {
            // staging tile [32 j][32 n]: lane = n, so every store fills one 128-byte row segment
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(stg + jj * 128 + lane * 4), "r"(r[jj]) : "memory");
          } else {
            // staging tile [32 n][32 j], 128-byte swizzle: lane = n owns one row
            const uint32_t rowaddr = stg + lane * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + ((ch ^ (lane & 7)) << 4)),
                           "r"(r[ch * 4 + 0]), "r"(r[ch * 4 + 1]), "r"(r[ch * 4 + 2]), "r"(r[ch * 4 + 3])
                           : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if constexpr (BS_LAST)
              tma_store_4d(&tmY, stg, n0 + q * 32, blk % P.d, j0 + jj0, blk / P.d);
            else
              tma_store_3d(&tmY, stg, j0 + jj0, blk, n0 + q * 32);
            bulk_commit();
          }
        }
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
      }
    }
    if (!C::DIRECT && lane == 0) bulk_wait<0>();
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

template <bool IN_LAST, bool BS_LAST, int NJ_, int ST_, bool TS_, bool DIRECT_ = false, bool WR_ = false>
static int launch_f(const Problem& p, cudaStream_t stream) {
  using C = CfgF<IN_LAST, BS_LAST, NJ_, ST_, TS_, DIRECT_, WR_>;
  auto kern = ksmm_tc_f32x3_kernel<IN_LAST, BS_LAST, NJ_, ST_, TS_, DIRECT_, WR_>;
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
  if (IN_LAST) {
    // input (a*c*d, batch), row (i*c + k)*d + l, seen as (n % 32, k, n / 32, l, i): one box is the
    // four atoms (32 batch entries x 32 k rows) of an MN-major operand tile
    const uint64_t dims[5] = {32, c, B / 32, d, a};
    const uint64_t str[5] = {1, d * B, 32, B, c * d * B};
    const uint32_t box[5] = {32, kKC, 4, 1, 1};
    if ((st = encode_map(&tmX, KSMM_F32, 5, p.in, dims, str, box, true, true)) != KSMM_OK) return st;
  } else {
    // input (batch, a*c): tile = 128 rows x 32 k of block i, 128-byte swizzle (K-major operand)
    const uint64_t dims[3] = {c, a, B};
    const uint64_t str[3] = {1, c, a * c};
    const uint32_t box[3] = {kKC, 1, 128};
    if ((st = encode_map(&tmX, KSMM_F32, 3, p.in, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // weights (a*d*c, b) row-major seen as (j % 32, k, j / 32, block): NJ / 32 atoms per box
    const uint64_t dims[4] = {32, c, b / 32, a * d};
    const uint64_t str[4] = {1, b, 32, c * b};
    const uint32_t box[4] = {32, kKC, static_cast<uint32_t>(C::NJ / 32), 1};
    if ((st = encode_map(&tmW, KSMM_F32, 4, p.w, dims, str, box, true, true)) != KSMM_OK) return st;
  }
  if (C::DIRECT) {
    tmY = tmW;  // unused: the epilogue stores from registers
  } else if (BS_LAST) {
    // output (a*b*d, batch): row (i*b + j)*d + l; store = 32 j x 32 batch entries
    const uint64_t dims[4] = {B, d, b, a};
    const uint64_t str[4] = {1, B, d * B, b * d * B};
    const uint32_t box[4] = {32, 1, 32, 1};
    if ((st = encode_map(&tmY, KSMM_F32, 4, p.out, dims, str, box, false)) != KSMM_OK) return st;
  } else {
    // output (batch, a*b): store = 32 rows x 32 j of block i, 128-byte swizzle
    const uint64_t dims[3] = {b, a, B};
    const uint64_t str[3] = {1, b, a * b};
    const uint32_t box[3] = {32, 1, 32};
    if ((st = encode_map(&tmY, KSMM_F32, 3, p.out, dims, str, box, true)) != KSMM_OK) return st;
  }
  ParamsF P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + 127) / 128);
  P.tiles_j = static_cast<int>((b + C::NJ - 1) / C::NJ);
  P.nchunks = (p.c + kKC - 1) / kKC;
  P.alpha = p.alpha;
  P.bias = static_cast<const float*>(p.bias);
  P.out = static_cast<float*>(p.out);
  P.act = p.activation;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  // fp32 accumulate, tf32 operands, weights MN-major, batch-last input MN-major when it is read
  // from shared memory (an operand in tensor memory is K-major), M = 128
  const uint32_t common = (1u << 4) | (2u << 7) | (2u << 10) | ((IN_LAST && !C::TS) ? (1u << 15) : 0u) | (1u << 16) |
                          (static_cast<uint32_t>(128 >> 4) << 24);
  P.idesc = common | (static_cast<uint32_t>(C::NJ >> 3) << 17);
  P.idesc2 = common | (static_cast<uint32_t>(2 * C::NJ >> 3) << 17);
  const int sms = num_sms();
  if (sms <= 0) return set_error(KSMM_ERR_NO_DEVICE, "no CUDA device");
  const int64_t rows = static_cast<int64_t>(P.tiles_n) * p.a * p.d;
  if (rows <= 0 || rows > 0x7fffffffLL || P.tiles_j > sms)
    return set_error(KSMM_ERR_UNSUPPORTED, "tensor-core family: work-split limits exceeded");
  P.rows = static_cast<uint32_t>(rows);
  int64_t groups = sms / P.tiles_j;
  if (groups > rows) groups = rows;
  P.row_groups = static_cast<uint32_t>(groups);
  const unsigned grid = static_cast<unsigned>(groups * P.tiles_j);
  cudaError_t err = launch_pdl(kern, grid, kThreadsF, C::SMEM_BYTES, stream, tmX, tmW, tmY, P);
  count_launch();
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace tc

bool tc_f32x3_supported(const Problem& p, bool check_pointers) {
  if (p.in_dtype != KSMM_F32 || p.out_dtype != KSMM_F32) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  // the operand tiles are addressed in atoms of 32 columns; global strides are multiples of 16 bytes
  if (p.b % 32 != 0) return false;
  const bool out_last = p.out_bs_last < 0 ? p.bs_last != 0 : p.out_bs_last != 0;
  if (out_last != (p.bs_last != 0) && (p.d != 1 || p.groups > 1)) return false;  // layout-changing factors
  if (p.bs_last || out_last) {
    if (p.batch % 32 != 0) return false;
  }
  if (!p.bs_last) {
    if (p.d != 1 || p.c % 4 != 0) return false;
  }
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16)
      return false;
  }
  return true;
}

int tc_f32x3_launch(const Problem& p, int config, cudaStream_t stream) {
  // <input batch-last, output batch-last, j tile, stages, input operand in tensor memory, direct
  // stores, resident weights>.  The j tile is the one with the least padded work.  Relative cost
  // of a tile, from tuning runs at 25088 rows over benchmark and reference-list patterns: 1 for
  // 128 columns (input operand from shared memory), 0.72 for 96 columns (input operand in tensor
  // memory; with resident weights on short blocks, batch-last and c <= 32 kMaxResident, where twelve
  // warps store the accumulator) and 0.55 for 64 columns.  E.g. b = 768: eight tiles of 96 (5.76)
  // against six of 128 (6.0), measured level; b = 128, 256, 512: tiles of 128 win by 5 to 27 %.
  const bool can_wr = p.bs_last && p.out_bs_last != 0 && p.c <= 32 * tc::kMaxResident;
  int nj = 96;
  double best = 1e30;
  for (int cand : {128, 96, 64}) {
    const double tile = cand == 128 ? 1.0 : (cand == 96 ? 0.72 : 0.55);
    const double cost = ((p.b + cand - 1) / cand) * tile;
    if (cost < best - 1e-9) { best = cost; nj = cand; }
  }
  if (config == 1) nj = 128;
  if (config == 2) nj = 96;
  if (config == 3) nj = 64;
  const bool out_last = p.out_bs_last < 0 ? p.bs_last != 0 : p.out_bs_last != 0;
  if (out_last != (p.bs_last != 0)) {
    // layout-changing factor (d = 1): the forms with the input operand in tensor memory
    if (nj == 128) nj = 96;
    if (p.bs_last)
      return nj == 96 ? tc::launch_f<true, false, 96, 4, true, false, false>(p, stream)
                      : tc::launch_f<true, false, 64, 6, true, false, false>(p, stream);
    return nj == 96 ? tc::launch_f<false, true, 96, 5, true, true, false>(p, stream)
                    : tc::launch_f<false, true, 64, 6, true, false, false>(p, stream);
  }
  if (p.bs_last) {
    if (nj == 128) return tc::launch_f<true, true, 128, 3, false, true, false>(p, stream);
    if (nj == 96)
      return can_wr ? tc::launch_f<true, true, 96, 5, true, true, true>(p, stream)
                    : tc::launch_f<true, true, 96, 5, true, true, false>(p, stream);
    return tc::launch_f<true, true, 64, 6, true, false, false>(p, stream);
  }
  if (nj == 128) return tc::launch_f<false, false, 128, 3, false, false, false>(p, stream);
  if (nj == 96) return tc::launch_f<false, false, 96, 4, true, false, false>(p, stream);
  return tc::launch_f<false, false, 64, 6, true, false, false>(p, stream);
}

}  // namespace ksmm

#ifdef KSMM_TC_TRACE
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace_f(unsigned long long* host) {
  using namespace ksmm;
  return static_cast<int>(cudaMemcpyFromSymbol(host, tc::g_trace, sizeof(tc::g_trace)));
}
extern "C" __attribute__((visibility("default"))) int ksmm_debug_trace_f_clear() {
  using namespace ksmm;
  static unsigned long long zeros[4][8192];
  return static_cast<int>(cudaMemcpyToSymbol(tc::g_trace, zeros, sizeof(zeros)));
}
#endif
