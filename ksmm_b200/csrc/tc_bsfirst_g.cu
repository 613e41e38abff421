// tcgen05 kernel for batch-first factors whose d is a multiple of 8 (16-bit inputs).
//
// A batch-first row holds, for block row i_a, the c*d values x[n, i_a, k, l] with l fastest; block
// (i_a, l) contracts over k at a stride of d elements.  With d a multiple of 8 the eight values
// l0 .. l0+7 of one (n, k) are 16 contiguous bytes, the smallest piece TMA moves.  A CTA therefore
// takes a group of eight blocks l0 .. l0+7 of one block row:
//   1. TMA fetches, per chunk of 16 k, the pieces (n, k) -> 16 bytes of 128 batch rows through a
//      4-D view (l, n, k, i_a) of the input whose box is (8, 128, 16, 1): shared memory then holds
//      [k][n][8 l], 32 KB;
//   2. four transposer warps (one thread per batch row) turn each 8 k x 8 l square into eight
//      16-byte rows of K-major operand tiles, one tile of 128 x 16 per block (16-byte loads, byte
//      permutes, 16-byte stores; lanes walk consecutive rows, so both sides are conflict-free);
//   3. eight MMAs per chunk (128 batch rows x 64 j x 16 k, one per block) accumulate into eight
//      accumulators side by side in TMEM (8 x 64 = 512 columns);
//   4. the epilogue interleaves them back: for every j the eight l values are one 16-byte piece,
//      staged as [j][n][8 l] and stored through the matching 4-D view of the output.
// The two l groups of d = 16 read and write complementary halves of the same 32-byte sectors; a
// CTA walks the groups of one (block row, batch tile) one after the other, so the second finds
// the sectors in L2.  The reference reads and writes 2 bytes at stride d
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_half.cuh:402-413, 609-618); this library
// used to run such factors as transpose -> batch-last kernel -> transpose.
//
// What bounds it: the 16-byte pieces.  TMA moves about one such piece per two SM cycles (a tile
// of 128 rows x 64 j x 8 l is 8192 pieces in and 8192 out); the same pieces through cp.async and
// plain 16-byte stores (one lane per batch row) measured slower still (73 against 53 us for
// (1,64,64,16) fp16 at 25088 rows; 62 us through the layout conversion, 23 us batch-last).  The
// split tiles are rebuilt for every j tile, so the kernel is used for b <= 64 only; wider
// factors keep the layout conversion.
//
// Warp roles (448 threads): warp 0 TMA producer, warp 1 TMEM owner and MMA issuer, warps 2..5
// transposers, warps 6..13 epilogue (TMEM lane quarter = warp index mod 4).  Waits are bounded
// and report through the device status word as in tc_kernel.cu.
#include <cuda.h>

#include <atomic>

#include "tc_host.h"
#include "tc_kernel.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace tc {

struct ParamsG {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j, lgroups;  // lgroups = d / 8
  uint32_t rows;        // a * tiles_n * lgroups: (block row, batch tile, l group) triples, l group fastest
  uint32_t row_groups;  // CTAs per j tile
  int nchunks;          // ceil(c / 16)
  uint32_t idesc;
  float alpha;
  const void* bias;
  int out_dtype;
  int act;  // ksmm_activation_t
  int* status;
};

constexpr int kThreadsG = (2 + 4 + kEpilogueWarps) * 32;

template <int SR, int SW, int SA>
struct CfgG {
  static constexpr int LG = 8;                        // blocks per CTA
  static constexpr int NJ = 64;                       // j columns per accumulator
  static constexpr int KCL = 16;                      // k values per chunk (one MMA k step)
  static constexpr int RAW_BYTES = KCL * 128 * 16;    // [k][n][8 l]
  // split operand tiles (K-major, no swizzle): [k / 8][n / 8][n % 8][16 bytes] per block
  static constexpr int A_SBO = 128;                   // bytes between groups of 8 rows
  static constexpr int A_LBO = 16 * 128;              // bytes between the two groups of 8 k
  static constexpr int AL_BYTES = (KCL / 8) * A_LBO;  // one block's tile (4 KB)
  static constexpr int A_BYTES = LG * AL_BYTES;
  static constexpr int WL_BYTES = KCL * 128;          // one block's 16 k rows x 64 j (128-byte swizzle)
  static constexpr int WCH_BYTES = LG * WL_BYTES;
  static constexpr int JB = 8;                        // j values per output store
  static constexpr int STG_WARP_BYTES = JB * 32 * 16; // [j][n][8 l]
  static constexpr int STG_BYTES = kEpilogueWarps * STG_WARP_BYTES;
  static constexpr int NBAR = 2 * SR + 2 * SA + 2 * SW + 2;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = STG_BYTES + SW * WCH_BYTES + SR * RAW_BYTES + SA * A_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 512;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(SMEM_BYTES > 116 * 1024, "one CTA per SM, so that the TMEM allocation never waits");
  static_assert(8 * NBAR + 16 <= BAR_BYTES, "barrier area");
};

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

template <int SR, int SW, int SA>
__global__ void __launch_bounds__(kThreadsG, 1)
    ksmm_tc_bsfirst_g_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                             const __grid_constant__ CUtensorMap tmY, const ParamsG P) {
  using C = CfgG<SR, SW, SA>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  // 1024-byte aligned regions first (the swizzled weights), then the rest
  const uint32_t wring0 = sm0;                            // streamed weight chunks
  const uint32_t stg0 = wring0 + SW * C::WCH_BYTES;       // epilogue staging tiles
  const uint32_t rring0 = stg0 + C::STG_BYTES;            // raw input chunks
  const uint32_t aring0 = rring0 + SR * C::RAW_BYTES;     // split operand tiles
  const uint32_t bar0 = aring0 + SA * C::A_BYTES;
  uint8_t* bar_gen = sm_gen + (bar0 - sm0);
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto raw_empty = [&](int s) { return bar0 + 8u * (SR + s); };
  auto a_full = [&](int s) { return bar0 + 8u * (2 * SR + s); };
  auto a_empty = [&](int s) { return bar0 + 8u * (2 * SR + SA + s); };
  auto w_full = [&](int s) { return bar0 + 8u * (2 * SR + 2 * SA + s); };
  auto w_empty = [&](int s) { return bar0 + 8u * (2 * SR + 2 * SA + SW + s); };
  const uint32_t tfull_bar = bar0 + 8u * (2 * SR + 2 * SA + 2 * SW);
  const uint32_t tempty_bar = tfull_bar + 8u;
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
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, kEpilogueWarps);
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
  grid_dep_wait();
  grid_dep_launch();

  const int nchunks = P.nchunks;
  const int tj = static_cast<int>(blockIdx.x % P.tiles_j);
  const uint32_t rc = blockIdx.x / P.tiles_j;
  const uint32_t row_begin = static_cast<uint32_t>(static_cast<uint64_t>(rc) * P.rows / P.row_groups);
  const uint32_t row_end = static_cast<uint32_t>(static_cast<uint64_t>(rc + 1) * P.rows / P.row_groups);
  const int j0 = tj * C::NJ;
  // row -> (block row i, batch tile, l group), l group fastest
  auto decode = [&](uint32_t row, int& i, int& n0, int& l0) {
    l0 = static_cast<int>(row % P.lgroups) * C::LG;
    const uint32_t t = row / P.lgroups;
    n0 = static_cast<int>(t % P.tiles_n) * 128;
    i = static_cast<int>(t / P.tiles_n);
  };

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t ri = 0, rph = 0, wi = 0, wph = 0;
      bool ok = true;
      for (uint32_t row = row_begin; row < row_end && ok; ++row) {
        int i, n0, l0;
        decode(row, i, n0, l0);
        for (int qc = 0; qc < nchunks; ++qc) {
          if (!mbar_wait<64>(raw_empty(ri), rph ^ 1u, abort_flag, P.status, 61)) { ok = false; break; }
          mbar_expect_tx(raw_full(ri), C::RAW_BYTES);
          // (l, n, k, i): 8 l x 128 batch rows x 16 k
          tma_load_4d(rring0 + ri * C::RAW_BYTES, &tmX, raw_full(ri), l0, n0, qc * C::KCL, i);
          if (++ri == SR) { ri = 0; rph ^= 1u; }
          if (!mbar_wait<64>(w_empty(wi), wph ^ 1u, abort_flag, P.status, 62)) { ok = false; break; }
          mbar_expect_tx(w_full(wi), C::WCH_BYTES);
          // (j, k, block): 64 j x 16 k x the 8 blocks of the group
          tma_load_3d(wring0 + wi * C::WCH_BYTES, &tmW, w_full(wi), j0, qc * C::KCL, i * P.d + l0);
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
      for (uint32_t row = row_begin; row < row_end && ok; ++row, ++ut) {
        if (!mbar_wait<0>(tempty_bar, (ut & 1u) ^ 1u, abort_flag, P.status, 63)) { ok = false; break; }
        tc_fence_after();
        for (int qc = 0; qc < nchunks; ++qc) {
          if (!mbar_wait<0>(w_full(wi), wph, abort_flag, P.status, 64)) { ok = false; break; }
          if (!mbar_wait<0>(a_full(ai), aph, abort_flag, P.status, 65)) { ok = false; break; }
          tc_fence_after();
          const uint32_t wbase = wring0 + wi * C::WCH_BYTES;
          const uint32_t abase = aring0 + ai * C::A_BYTES;
#pragma unroll
          for (int l = 0; l < C::LG; ++l) {
            // split tile: K-major, no swizzle (core matrices of 8 rows x 16 bytes)
            const uint64_t adesc = make_desc(abase + l * C::AL_BYTES, C::A_LBO, C::A_SBO, 0);
            // weights: MN-major, 128-byte swizzle, one 64-wide box; SBO = next 8 k rows
            const uint64_t bdesc = make_desc(wbase + l * C::WL_BYTES, C::WL_BYTES, 1024, 2);
            umma<2>(tmem_base + l * C::NJ, adesc, bdesc, P.idesc, qc != 0 ? 1u : 0u);
          }
          umma_commit(a_empty(ai));  // the split tiles and the weight slot are free again
          umma_commit(w_empty(wi));
          if (++ai == SA) { ai = 0; aph ^= 1u; }
          if (++wi == SW) { wi = 0; wph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ===================== transposers =====================
    // thread = batch row n of the tile.  Its 16 pieces (one per k, 8 l each) become, per block l,
    // two 16-byte rows of the K-major tile (k 0..7 and k 8..15); one group of 8 k at a time.
    const int n = (warp - 2) * 32 + lane;
    uint32_t ri = 0, rph = 0, ai = 0, aph = 0;
    bool ok = true;
    for (uint32_t row = row_begin; row < row_end && ok; ++row) {
      for (int qc = 0; qc < nchunks; ++qc) {
        int got = 1;
        if (lane == 0) {
          got = mbar_wait<32>(raw_full(ri), rph, abort_flag, P.status, 66) ? 1 : 0;
          if (got) got = mbar_wait<32>(a_empty(ai), aph ^ 1u, abort_flag, P.status, 67) ? 1 : 0;
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        const uint32_t rbase = rring0 + ri * C::RAW_BYTES + n * 16;
        const uint32_t abase = aring0 + ai * C::A_BYTES + n * 16;
#pragma unroll
        for (int kg = 0; kg < C::KCL / 8; ++kg) {
          uint32_t w[8][4];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[k][0]), "=r"(w[k][1]), "=r"(w[k][2]), "=r"(w[k][3])
                         : "r"(rbase + (kg * 8 + k) * 2048)
                         : "memory");
#pragma unroll
          for (int l = 0; l < C::LG; ++l) {
            // word l / 2 of a piece holds (l even, l odd); pick this block's half of two neighbouring k
            const uint32_t sel = (l & 1) ? 0x7632u : 0x5410u;
            uint32_t o[4];
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) o[kp] = __byte_perm(w[2 * kp][l >> 1], w[2 * kp + 1][l >> 1], sel);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(abase + l * C::AL_BYTES + kg * C::A_LBO),
                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                         : "memory");
          }
        }
        fence_proxy_async();  // the tiles are read by the tensor core through the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(raw_empty(ri));
          mbar_arrive(a_full(ai));
        }
        if (++ri == SR) { ri = 0; rph ^= 1u; }
        if (++ai == SA) { ai = 0; aph ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    // warp = (TMEM lane quarter q, half of the 64 j columns); per store eight j: the eight
    // accumulators' columns j give, for every batch row, one 16-byte piece (l0 .. l0+7) per j
    const int ew = warp - 6;
    const int q = warp & 3;
    const int grp = ew >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const bool plain = (P.alpha == 1.f) && (P.bias == nullptr) && (P.act == 0);
    const uint32_t stg = stg0 + ew * C::STG_WARP_BYTES;
    uint32_t ut = 0;
    for (uint32_t row = row_begin; row < row_end; ++row, ++ut) {
      int i, n0, l0;
      decode(row, i, n0, l0);
      int got = 1;
      if (lane == 0) got = mbar_wait<128>(tfull_bar, ut & 1u, abort_flag, P.status, 68) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      const bool warp_active = n0 + q * 32 < P.batch;
      int jlim = P.b - j0;  // j columns of this tile that exist
      if (jlim > C::NJ) jlim = C::NJ;
      if (warp_active) {
#pragma unroll 1
        for (int it = 0; it < (C::NJ / 2) / C::JB; ++it) {
          const int jj0 = grp * (C::NJ / 2) + it * C::JB;
          if (jj0 >= jlim) break;
          uint32_t r[C::LG][C::JB];
#pragma unroll
          for (int l = 0; l < C::LG; ++l) tmem_ld8(tmem_base + lane_addr + l * C::NJ + jj0, r[l]);
          tmem_ld_wait();
          if (lane == 0) bulk_wait_read<0>();  // the previous store has read the staging tile
          __syncwarp();
#pragma unroll
          for (int jj = 0; jj < C::JB; ++jj) {
            if (!plain) {
              // the eight bias values of (j, l0 .. l0+7): 16 bytes, the same for every lane
              uint32_t bw[4] = {0u, 0u, 0u, 0u};
              if (P.bias != nullptr && jj0 + jj < jlim) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(
                    static_cast<const uint16_t*>(P.bias) + (static_cast<int64_t>(i) * P.b + j0 + jj0 + jj) * P.d + l0));
                bw[0] = bv.x; bw[1] = bv.y; bw[2] = bv.z; bw[3] = bv.w;
              }
#pragma unroll
              for (int l = 0; l < C::LG; ++l) {
                const uint16_t hv = static_cast<uint16_t>((l & 1) ? (bw[l >> 1] >> 16) : (bw[l >> 1] & 0xffffu));
                const float bvf = P.out_dtype == KSMM_BF16 ? __uint_as_float(static_cast<uint32_t>(hv) << 16)
                                                           : __half2float(__ushort_as_half(hv));
                float v = fmaf(P.alpha, __uint_as_float(r[l][jj]), bvf);
                if (P.act == KSMM_ACT_GELU) v = gelu_16bit(v);
                else if (P.act == KSMM_ACT_RELU) v = fmaxf(v, 0.f);
                r[l][jj] = __float_as_uint(v);
              }
            }
            uint32_t wv[4];
#pragma unroll
            for (int m = 0; m < 4; ++m)
              wv[m] = pack2(__uint_as_float(r[2 * m][jj]), __uint_as_float(r[2 * m + 1][jj]), P.out_dtype);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + jj * 512 + lane * 16),
                         "r"(wv[0]), "r"(wv[1]), "r"(wv[2]), "r"(wv[3])
                         : "memory");
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            // (l, n, j, i): 8 l x 32 batch rows x 8 j
            tma_store_4d(&tmY, stg, l0, n0 + q * 32, j0 + jj0, i);
            bulk_commit();
          }
        }
      }
      // this warp's TMEM reads are complete: the next tile's MMAs may overwrite the accumulators
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
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

template <int SR, int SW, int SA>
static int launch_g(const Problem& p, cudaStream_t stream) {
  using C = CfgG<SR, SW, SA>;
  auto kern = ksmm_tc_bsfirst_g_kernel<SR, SW, SA>;
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
  CUtensorMap tmX, tmW, tmY;
  int st;
  {
    // input (batch, a*c*d) seen as (l, n, k, i): the box's pieces land as [k][n][8 l]
    const uint64_t dims[4] = {d, B, c, a};
    const uint64_t str[4] = {1, a * c * d, d, c * d};
    const uint32_t box[4] = {8, 128, static_cast<uint32_t>(C::KCL), 1};
    if ((st = encode_map(&tmX, p.in_dtype, 4, p.in, dims, str, box, false)) != KSMM_OK) return st;
  }
  {
    // weights (a*d*c, b) row-major seen as (b, c, a*d); box = 64 j x 16 k x the 8 blocks of a group
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {64, static_cast<uint32_t>(C::KCL), static_cast<uint32_t>(C::LG)};
    if ((st = encode_map(&tmW, p.in_dtype, 3, p.w, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // output (batch, a*b*d) seen as (l, n, j, i): a store is [8 j][32 n][8 l]
    const uint64_t dims[4] = {d, B, b, a};
    const uint64_t str[4] = {1, a * b * d, d, b * d};
    const uint32_t box[4] = {8, 32, static_cast<uint32_t>(C::JB), 1};
    if ((st = encode_map(&tmY, p.out_dtype, 4, p.out, dims, str, box, false)) != KSMM_OK) return st;
  }
  ParamsG P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + 127) / 128);
  P.tiles_j = static_cast<int>((b + C::NJ - 1) / C::NJ);
  P.lgroups = p.d / C::LG;
  P.nchunks = (p.c + C::KCL - 1) / C::KCL;
  P.alpha = p.alpha;
  P.bias = p.bias;
  P.out_dtype = p.out_dtype;
  P.act = p.activation;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;
  // fp32 accumulate, A K-major, B MN-major, N = 64, M = 128
  P.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(C::NJ >> 3) << 17) |
            (static_cast<uint32_t>(128 >> 4) << 24);
  const int sms = num_sms();
  if (sms <= 0) return set_error(KSMM_ERR_NO_DEVICE, "no CUDA device");
  const int64_t rows = static_cast<int64_t>(P.tiles_n) * p.a * P.lgroups;
  if (rows <= 0 || rows > 0x7fffffffLL || P.tiles_j > sms)
    return set_error(KSMM_ERR_UNSUPPORTED, "tensor-core family: work-split limits exceeded");
  P.rows = static_cast<uint32_t>(rows);
  int64_t groups = sms / P.tiles_j;
  if (groups > rows) groups = rows;
  P.row_groups = static_cast<uint32_t>(groups);
  const unsigned grid = static_cast<unsigned>(groups * P.tiles_j);
  cudaError_t err = launch_pdl(kern, grid, kThreadsG, C::SMEM_BYTES, stream, tmX, tmW, tmY, P);
  count_launch();
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace tc

bool tc_bsfirst_g_supported(const Problem& p, bool check_pointers) {
  if (p.bs_last || p.d < 8 || p.d % 8 != 0) return false;
  if (p.in_dtype != KSMM_F16 && p.in_dtype != KSMM_BF16) return false;
  if (p.out_dtype != p.in_dtype) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  // weight rows are multiples of 16 bytes; one j tile (the split tiles are rebuilt per j tile, and
  // beyond one the layout conversion is faster)
  if (p.b % 8 != 0 || p.b > 64) return false;
  if (p.groups > 1 || p.out_regroup_d || p.in_regrouped || p.out_bs_last >= 0) return false;
  if (static_cast<int64_t>(p.a) * p.d > 0x7fffffffLL) return false;
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16 || (p.bias && reinterpret_cast<uintptr_t>(p.bias) % 16))
      return false;
  }
  return true;
}

int tc_bsfirst_g_launch(const Problem& p, cudaStream_t stream) {
  // <raw stages, weight stages, split-tile buffers>
  return tc::launch_g<2, 3, 2>(p, stream);
}

}  // namespace ksmm
