// tcgen05 / TMEM / TMA KSMM kernel family (KSMM_ALGO_TC) for fp16, bf16 and
// fp8-e4m3 inputs with fp32 accumulation.
//
// One factor with pattern (a,b,c,d) is a*d independent (b x c) blocks, each
// contracted with a (c x batch) slice of the input.  A work unit is one
// 128 x NT tile of one block's output; a persistent CTA (one per SM) walks
// units bid, bid + grid, ... so that the CTAs running at any moment work on
// neighbouring tiles and share their operands in L2.
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
// staging tile, and one thread issues a TMA store of the tile.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator and
// single-thread MMA issuer, warps 2..5 = epilogue (TMEM lane quarter =
// warp index mod 4).  Operand stages form a ring guarded by full/empty
// mbarriers; the accumulator is double-buffered in TMEM (2 x NT columns) so
// the epilogue of unit u overlaps the MMAs of unit u+1.
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

#include <mutex>

#include "tc_kernel.h"

namespace ksmm {
namespace tc {

// one status word per device that loads the module; 0 = no device-side timeout
__device__ int g_tc_status_word = 0;

struct Params {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  int64_t units;
  int nk;
  uint32_t idesc;
  float alpha;
  const void* bias;
  int out_dtype;
  int* status;
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait.  Returns false after the limit, or as soon as another role has
// raised the CTA-wide abort flag; the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code) {
#pragma unroll 1
  for (int q = 0; q < 32; ++q)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int q = 0; q < 64; ++q)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bar_sync_named(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, uint32_t src, int x, int y,
                                             int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(tm)),
      "r"(src), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* tm, uint32_t src, int x, int y,
                                             int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
          "l"(reinterpret_cast<uint64_t>(tm)),
      "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
template <int ES>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                     uint32_t idesc, uint32_t accumulate) {
  if constexpr (ES == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field.
//   MN-major operand: LBO = byte distance between 128-byte-wide groups along
//     M/N, SBO = byte distance between groups of 8 k-rows.
//   K-major operand: SBO = byte distance between groups of 8 M/N rows (LBO unused).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t dsc = 0;
  dsc |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  dsc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  dsc |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  dsc |= static_cast<uint64_t>(1) << 46;  // descriptor version (sm_100)
  dsc |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return dsc;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int out_dtype) {
  if (out_dtype == KSMM_F16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float bias_at(const void* bias, int64_t idx, int out_dtype) {
  if (out_dtype == KSMM_F32) return static_cast<const float*>(bias)[idx];
  if (out_dtype == KSMM_F16) return __half2float(static_cast<const __half*>(bias)[idx]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[idx]);
}

template <bool BS_LAST, int ES, int OS, int NT, int KC, int ST>
struct Cfg {
  static constexpr int NBOX = 128 / ES;        // elements in one 128-byte box row
  static constexpr int UK = 32 / ES;           // k extent of one MMA
  static constexpr int M_BYTES = 128 * KC * ES;
  static constexpr int N_BYTES = NT * KC * ES;
  static constexpr int STAGE_BYTES = M_BYTES + N_BYTES;
  static constexpr int CB = 128 / OS;          // output elements in one staging row
  static constexpr int STG_BYTES = 128 * 128;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = ST * STAGE_BYTES + 2 * STG_BYTES + BAR_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * NT;
  static_assert(NT == 64 || NT == 128 || NT == 256, "TMEM allocation must be a power of two");
  static_assert(KC % UK == 0 && KC % 8 == 0, "k chunk");
  static_assert(BS_LAST || KC == NBOX, "batch-first stages hold one 128-byte k box");
  static_assert(NT % NBOX == 0, "N tile must be whole 128-byte box rows");
  static_assert(2 * ST + 4 <= 24, "barrier area");
};

template <bool BS_LAST, int ES, int OS, int NT, int KC, int ST>
__global__ void __launch_bounds__(192, 1)
    ksmm_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmY, const Params P) {
  using C = Cfg<BS_LAST, ES, OS, NT, KC, ST>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;  // 1024-byte alignment for the 128-byte swizzle
  uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t stg0 = sm0 + ST * C::STAGE_BYTES;
  const uint32_t bar0 = stg0 + 2 * C::STG_BYTES;
  uint8_t* bar_gen = sm_gen + ST * C::STAGE_BYTES + 2 * C::STG_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (ST + s); };
  auto tfull_bar = [&](int q) { return bar0 + 8u * (2 * ST + q); };
  auto tempty_bar = [&](int q) { return bar0 + 8u * (2 * ST + 2 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * ST + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * ST + 4) + 4);
  volatile int* epi_abort = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * ST + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(tfull_bar(q), 1);
      mbar_init(tempty_bar(q), 128);
    }
    *abort_flag = 0;
    *epi_abort = 0;
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

  const int d = P.d;
  const int64_t units = P.units;
  const int nk = P.nk;

  // unit -> (j tile fastest, then batch tile, then block): neighbouring CTAs
  // share the input slice (batch-last) or the input rows (batch-first)
  auto decode = [&](int64_t u, int& tj, int& tn, int& blk) {
    tj = static_cast<int>(u % P.tiles_j);
    const int64_t r = u / P.tiles_j;
    tn = static_cast<int>(r % P.tiles_n);
    blk = static_cast<int>(r / P.tiles_n);
  };

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
        int tj, tn, blk;
        decode(u, tj, tn, blk);
        const int i = blk / d, l = blk % d;
        const int n0 = tn * (BS_LAST ? NT : 128);
        const int j0 = tj * (BS_LAST ? 128 : NT);
        for (int kc = 0; kc < nk; ++kc, ++it) {
          const int s = it % ST;
          const uint32_t ph = (it / ST) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, P.status, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
          const uint32_t mdst = sm0 + s * C::STAGE_BYTES;
          const uint32_t ndst = mdst + C::M_BYTES;
          if constexpr (BS_LAST) {
#pragma unroll
            for (int wb = 0; wb < 128 / C::NBOX; ++wb)
              tma_load_3d(mdst + wb * KC * 128, &tmW, full_bar(s), j0 + wb * C::NBOX, kc * KC, blk);
#pragma unroll
            for (int xb = 0; xb < NT / C::NBOX; ++xb)
              tma_load_4d(ndst + xb * KC * 128, &tmX, full_bar(s), n0 + xb * C::NBOX, l, kc * KC, i);
          } else {
            tma_load_3d(mdst, &tmX, full_bar(s), kc * KC, i, n0);
#pragma unroll
            for (int wb = 0; wb < NT / C::NBOX; ++wb)
              tma_load_3d(ndst + wb * KC * 128, &tmW, full_bar(s), j0 + wb * C::NBOX, kc * KC, blk);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      uint32_t it = 0, ut = 0;
      bool ok = true;
      for (int64_t u = blockIdx.x; u < units && ok; u += gridDim.x, ++ut) {
        const uint32_t buf = ut & 1u, bph = (ut >> 1) & 1u;
        if (!mbar_wait(tempty_bar(buf), bph ^ 1u, abort_flag, P.status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dcol = tmem_base + buf * NT;
        for (int kc = 0; kc < nk; ++kc, ++it) {
          const int s = it % ST;
          const uint32_t ph = (it / ST) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag, P.status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t mdst = sm0 + s * C::STAGE_BYTES;
          const uint32_t ndst = mdst + C::M_BYTES;
#pragma unroll
          for (int k = 0; k < KC / C::UK; ++k) {
            uint64_t adesc, bdesc;
            if constexpr (BS_LAST) {
              adesc = make_desc(mdst + k * C::UK * 128, KC * 128, 1024);
            } else {
              adesc = make_desc(mdst + k * C::UK * ES, 16, 1024);
            }
            bdesc = make_desc(ndst + k * C::UK * 128, KC * 128, 1024);
            umma<ES>(dcol, adesc, bdesc, P.idesc, (kc | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(tfull_bar(buf));  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ===================== epilogue =====================
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    uint32_t ut = 0, stg_count = 0;
    for (int64_t u = blockIdx.x; u < units; u += gridDim.x, ++ut) {
      const uint32_t buf = ut & 1u, bph = (ut >> 1) & 1u;
      int tj, tn, blk;
      decode(u, tj, tn, blk);
      const int i = blk / d, l = blk % d;
      const int n0 = tn * (BS_LAST ? NT : 128);
      const int j0 = tj * (BS_LAST ? 128 : NT);
      if (!mbar_wait(tfull_bar(buf), bph, abort_flag, P.status, 4)) *epi_abort = 1;
      bar_sync_named(1, 128);
      if (*epi_abort) break;
      tc_fence_after();
      // rows of this warp that exist (warp-uniform): j rows (batch-last) or batch rows
      const int64_t row_limit = BS_LAST ? static_cast<int64_t>(P.b) - j0 : P.batch - n0;
      const bool warp_active = (q * 32) < row_limit;
      const int64_t col_limit = BS_LAST ? P.batch - n0 : static_cast<int64_t>(P.b) - j0;
      float bias_row = 0.f;
      if (BS_LAST && P.bias != nullptr && row < row_limit)
        bias_row = bias_at(P.bias, (static_cast<int64_t>(i) * P.b + j0 + row) * d + l, P.out_dtype);
#pragma unroll 1
      for (int cbi = 0; cbi < NT / C::CB; ++cbi) {
        if (static_cast<int64_t>(cbi) * C::CB >= col_limit) break;  // uniform
        const uint32_t sb = stg_count & 1u;
        ++stg_count;
        if (epi_tid == 0) bulk_wait_read<1>();  // the store that last used this buffer has read it
        bar_sync_named(1, 128);
        const uint32_t stg = stg0 + sb * C::STG_BYTES;
        if (warp_active) {
#pragma unroll
          for (int h = 0; h < C::CB / 32; ++h) {
            uint32_t r[32];
            tmem_ld32(tmem_base + lane_addr + buf * NT + cbi * C::CB + h * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              float bv = bias_row;
              if (!BS_LAST && P.bias != nullptr) {
                const int col = cbi * C::CB + h * 32 + e;
                bv = col < col_limit
                         ? bias_at(P.bias, static_cast<int64_t>(i) * P.b + j0 + col, P.out_dtype)
                         : 0.f;
              }
              v[e] = fmaf(P.alpha, __uint_as_float(r[e]), bv);
            }
            const uint32_t rowaddr = stg + row * 128;
            if constexpr (OS == 2) {
#pragma unroll
              for (int ch = 0; ch < 4; ++ch) {
                uint32_t w0 = pack2(v[ch * 8 + 0], v[ch * 8 + 1], P.out_dtype);
                uint32_t w1 = pack2(v[ch * 8 + 2], v[ch * 8 + 3], P.out_dtype);
                uint32_t w2 = pack2(v[ch * 8 + 4], v[ch * 8 + 5], P.out_dtype);
                uint32_t w3 = pack2(v[ch * 8 + 6], v[ch * 8 + 7], P.out_dtype);
                const uint32_t chunk = static_cast<uint32_t>((h * 4 + ch) ^ (row & 7));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + chunk * 16),
                             "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                             : "memory");
              }
            } else {
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) {
                const uint32_t chunk = static_cast<uint32_t>(ch ^ (row & 7));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowaddr + chunk * 16),
                             "r"(__float_as_uint(v[ch * 4 + 0])), "r"(__float_as_uint(v[ch * 4 + 1])),
                             "r"(__float_as_uint(v[ch * 4 + 2])), "r"(__float_as_uint(v[ch * 4 + 3]))
                             : "memory");
              }
            }
          }
        }
        fence_proxy_async();
        bar_sync_named(1, 128);
        if (epi_tid == 0) {
          if constexpr (BS_LAST) {
            tma_store_4d(&tmY, stg, n0 + cbi * C::CB, l, j0, i);
          } else {
            tma_store_3d(&tmY, stg, j0 + cbi * C::CB, i, n0);
          }
          bulk_commit();
        }
      }
      // this thread's TMEM reads of the buffer are complete: hand it back
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
    }
    if (epi_tid == 0) bulk_wait<0>();  // all stores have left shared memory and are visible
    __syncwarp();
  }

  // ===================== teardown =====================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag || *epi_abort) {
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

// rank-R tiled map with 128-byte swizzle; dims/strides innermost first,
// strides in elements (stride of dim 0 is implicitly 1)
static int encode_map(CUtensorMap* tm, int dt, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_elems, const uint32_t* box) {
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
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
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
static constexpr int kNumConfigs = 5;

static int* status_word() {
  // one status word per device, owned by the module image
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tc_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

static int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev];
}

template <bool BS_LAST, int ES, int OS, int NT, int KC, int ST>
static int launch_one(const Problem& p, cudaStream_t stream) {
  using C = Cfg<BS_LAST, ES, OS, NT, KC, ST>;
  auto kern = ksmm_tc_kernel<BS_LAST, ES, OS, NT, KC, ST>;
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
    // weights (a*d*c, b) row-major seen as (b, c, a*d)
    const uint64_t dims[3] = {b, c, a * d};
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
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const uint32_t fmt = p.in_dtype == KSMM_BF16 ? 1u : 0u;  // f16 / e4m3 = 0, bf16 = 1
  uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) |
                   (static_cast<uint32_t>(NT >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
  if (BS_LAST) {
    idesc |= (1u << 15);  // A (weights) is MN-major as well
    const uint64_t xd[4] = {B, d, c, a};
    const uint64_t xs[4] = {1, B, d * B, c * d * B};
    const uint32_t xb[4] = {static_cast<uint32_t>(C::NBOX), 1, static_cast<uint32_t>(KC), 1};
    if ((st = encode_map(&tmX, p.in_dtype, 4, p.in, xd, xs, xb)) != KSMM_OK) return st;
    const uint64_t yd[4] = {B, d, b, a};
    const uint64_t ys[4] = {1, B, d * B, b * d * B};
    const uint32_t yb[4] = {static_cast<uint32_t>(C::CB), 1, 128, 1};
    if ((st = encode_map(&tmY, p.out_dtype, 4, p.out, yd, ys, yb)) != KSMM_OK) return st;
    P.tiles_n = static_cast<int>((B + NT - 1) / NT);
    P.tiles_j = static_cast<int>((b + 127) / 128);
  } else {
    const uint64_t xd[3] = {c, a, B};
    const uint64_t xs[3] = {1, c, a * c};
    const uint32_t xb[3] = {static_cast<uint32_t>(KC), 1, 128};
    if ((st = encode_map(&tmX, p.in_dtype, 3, p.in, xd, xs, xb)) != KSMM_OK) return st;
    const uint64_t yd[3] = {b, a, B};
    const uint64_t ys[3] = {1, b, a * b};
    const uint32_t yb[3] = {static_cast<uint32_t>(C::CB), 1, 128};
    if ((st = encode_map(&tmY, p.out_dtype, 3, p.out, yd, ys, yb)) != KSMM_OK) return st;
    P.tiles_n = static_cast<int>((B + 127) / 128);
    P.tiles_j = static_cast<int>((b + NT - 1) / NT);
  }
  P.idesc = idesc;
  P.units = static_cast<int64_t>(P.tiles_n) * P.tiles_j * p.a * p.d;
  const int sms = num_sms();
  if (sms <= 0) return set_error(KSMM_ERR_NO_DEVICE, "no CUDA device");
  const unsigned grid = static_cast<unsigned>(P.units < sms ? P.units : sms);
  kern<<<grid, 192, C::SMEM_BYTES, stream>>>(tmX, tmW, tmY, P);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "tensor-core kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

template <bool BS_LAST, int ES, int OS>
static int launch_cfg(const Problem& p, int config, cudaStream_t stream) {
  constexpr int R = ES == 2 ? 1 : 2;  // k rows per stage scale with 1 / element size
  if constexpr (BS_LAST) {
    switch (config) {
      case 0: return launch_one<true, ES, OS, 256, 64 * R, 3>(p, stream);
      case 1: return launch_one<true, ES, OS, 128, 64 * R, 4>(p, stream);
      case 2: return launch_one<true, ES, OS, 256, 32 * R, 4>(p, stream);
      case 3: return launch_one<true, ES, OS, 128, 32 * R, 6>(p, stream);
      case 4:
        if constexpr (ES == 2) return launch_one<true, ES, OS, 64, 64 * R, 4>(p, stream);
        break;
    }
  } else {
    switch (config) {
      case 0: return launch_one<false, ES, OS, 256, 64 * R, 3>(p, stream);
      case 1: return launch_one<false, ES, OS, 128, 64 * R, 4>(p, stream);
      case 2: return launch_one<false, ES, OS, 256, 64 * R, 4>(p, stream);
      case 3: return launch_one<false, ES, OS, 128, 64 * R, 6>(p, stream);
      case 4:
        if constexpr (ES == 2) return launch_one<false, ES, OS, 64, 64 * R, 4>(p, stream);
        break;
    }
  }
  return set_error(KSMM_ERR_BAD_ARGUMENT, "tensor-core family: no configuration %d", config);
}

}  // namespace tc

int tc_num_configs() { return tc::kNumConfigs; }

bool tc_config_supported(const Problem& p, int config, bool check_pointers) {
  if (config < 0 || config >= tc::kNumConfigs) return false;
  if (config == 4 && p.in_dtype == KSMM_F8E4M3) return false;
  const int es = dtype_size(p.in_dtype), os = dtype_size(p.out_dtype);
  if (p.in_dtype == KSMM_F32) return false;
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

int tc_default_config(const Problem& p) {
  if (!tc_config_supported(p, 0, true)) return -1;
  // tiny blocks are bandwidth problems that the FFMA family tiles more tightly
  if (p.b < 32 || p.c < 16) return -1;
  if (p.bs_last) return p.batch >= 256 * 148 / 2 || p.batch >= 4096 ? 0 : 1;
  return p.b > 128 ? 0 : (p.b > 64 ? 1 : 4);
}

int tc_launch(const Problem& p, int config, cudaStream_t stream) {
  if (config < 0) config = tc_default_config(p);
  if (config < 0 || !tc_config_supported(p, config, true))
    return set_error(KSMM_ERR_UNSUPPORTED,
                     "tensor-core family cannot run pattern (%d,%d,%d,%d) batch %lld dtype %d "
                     "bs_last %d (alignment or layout rule)",
                     p.a, p.b, p.c, p.d, static_cast<long long>(p.batch), p.in_dtype, p.bs_last);
  const bool last = p.bs_last != 0;
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
                     "a tensor-core kernel gave up waiting (role code %d: 1 producer/empty, "
                     "2 mma/tmem-empty, 3 mma/full, 4 epilogue/tmem-full)",
                     code);
  }
  return KSMM_OK;
}

}  // namespace ksmm
