// fp32 FFMA kernel with TMA-staged operands for the batch-first layout
// (kernel family KSMM_ALGO_SIMT, configuration 8).
//
// In a batch-first row the values x[n, i, k, l] of one block row i are
// contiguous with l fastest.  The kernel lets one CTA compute L = 1, 2 or 4
// neighbouring blocks l at once, so that what it loads and what it stores are
// contiguous runs:
//   d == 1      : L = 1, thread tile 8 j x 8 n, input read as float4 over 4 k
//   d == 2      : L = 2, thread tile 2 l x 4 j x 8 n, float4 = (k,l0)(k,l1)(k+1,l0)(k+1,l1)
//   d == 4      : L = 4, thread tile 4 l x 4 j x 4 n, float4 = (k, l0..l3)
// The input tile is fetched by TMA as rows of 128 bytes (32 floats = 32/L values
// of k for each of the L blocks) with the 128-byte swizzle, which makes the
// per-row float4 reads of the four n lanes of a warp conflict-free; the weights
// of the L blocks come through one box of the (b, c, a*d) view.  Every thread
// ends up with L consecutive outputs per (n, j), stored as 8/16-byte vectors;
// a warp's stores cover whole 128-byte lines.  The reference's batch-first fp32
// kernel reads and writes single floats at stride d
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_float.cuh:156-161, 276-285).
//
// Every TMA box row is exactly one 128-byte swizzle span of contiguous input
// (the (k, l) pairs of a row are contiguous for d = L), which is why d is
// limited to 1, 2 and 4; other d take the register-staged kernel.
//
// Requirements (else the register-staged kernel runs): fp32, batch-first,
// d in {1, 2, 4}, b % 4 == 0, c * d % 4 == 0, 16-byte aligned pointers.
#include <cuda.h>

#include <atomic>

#include "tc_host.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace ffma_first {

using namespace ksmm::tc;

struct Params {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j, lgroups;
  int nk;  // stages of KC values of k
  float alpha;
  const float* bias;
  float* out;
  int64_t out_elems;  // a*b*d*batch, for the store guard
  int* status;
};

template <int L>
struct Cfg {
  static constexpr int KCR = 32 / L;                   // k values in one 128-byte row
  static constexpr int NB = (L == 4) ? 2 : 1;          // row boxes per stage
  static constexpr int KC = KCR * NB;                  // k values per stage
  static constexpr int TJ = 64;                        // j per CTA
  static constexpr int WN = 4;                         // warps along n
  static constexpr int WJ = (L == 1) ? 1 : 2;          // warps along j
  static constexpr int TNW = (L == 4) ? 16 : 32;       // n per warp
  static constexpr int TN = WN * TNW;                  // n per CTA (64 or 128)
  static constexpr int NT = WN * WJ * 32;
  static constexpr int ST = (L == 2) ? 4 : 3;
  static constexpr int RAW_BYTES = NB * TN * 128;
  static constexpr int W_BYTES = L * KC * TJ * 4;
  static constexpr int STAGE_BYTES = RAW_BYTES + W_BYTES;
  static constexpr int SMEM_BYTES = ST * STAGE_BYTES + 1024 + 128;
  static constexpr int MIN_CTAS = (L == 1) ? 3 : 2;
};

// 16-byte store with a guard: an offset outside the output is recorded in the
// device status word (code 25) and skipped instead of being written.
__device__ __forceinline__ void store_checked(const Params& P, int64_t off, const float4& v) {
  if (off < 0 || off + 4 > P.out_elems || (off & 3) != 0) {
    atomicCAS(P.status, 0, 25);
    return;
  }
  *reinterpret_cast<float4*>(P.out + off) = v;
}

template <int L>
__global__ void __launch_bounds__(Cfg<L>::NT, Cfg<L>::MIN_CTAS)
    ksmm_ffma_tma_first_kernel(const __grid_constant__ CUtensorMap tmX,
                               const __grid_constant__ CUtensorMap tmW, const Params P) {
  using C = Cfg<L>;
  constexpr int KC = C::KC, KCR = C::KCR, ST = C::ST, TN = C::TN, TJ = C::TJ;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 1023u) & ~1023u;  // the 128-byte swizzle repeats every 1024 bytes
  const uint8_t* sm_gen = smem_raw + (sm0 - raw);
  const uint32_t bar0 = sm0 + ST * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (ST + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(
      const_cast<uint8_t*>(sm_gen) + ST * C::STAGE_BYTES + 8 * 2 * ST);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int wj = warp % C::WJ, wn = warp / C::WJ;
  const int jl = lane & 7, nl = lane >> 3;

  int64_t bid = blockIdx.x;
  const int tn = static_cast<int>(bid % P.tiles_n);
  bid /= P.tiles_n;
  const int tj = static_cast<int>(bid % P.tiles_j);
  bid /= P.tiles_j;
  const int lg = static_cast<int>(bid % P.lgroups);
  const int i = static_cast<int>(bid / P.lgroups);
  const int l0 = lg * L;
  const int n0 = tn * TN, j0 = tj * TJ;
  const int nk = P.nk;

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), C::NT / 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  auto issue = [&](int kc) {
    const int s = kc % ST;
    const uint32_t dst = sm0 + s * C::STAGE_BYTES;
    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
#pragma unroll
    for (int nb = 0; nb < C::NB; ++nb) {
      // (k, l) merged into one contiguous dimension of c * d elements (d == L)
      tma_load_3d(dst + nb * TN * 128, &tmX, full_bar(s), (kc * KC + nb * KCR) * L, i, n0);
    }
    tma_load_3d(dst + C::RAW_BYTES, &tmW, full_bar(s), j0, kc * KC, i * P.d + l0);
  };
  if (tid == 0) {
    for (int kc = 0; kc < ST - 1 && kc < nk; ++kc) issue(kc);
  }

  float acc[64];
#pragma unroll
  for (int q = 0; q < 64; ++q) acc[q] = 0.f;

  bool ok = true;
  for (int kc = 0; kc < nk; ++kc) {
    const int s = kc % ST;
    if (tid == 0) {
      const int nxt = kc + ST - 1;
      if (nxt < nk) {
        if (kc >= 1) {
          const int ps = (kc - 1) % ST;
          const uint32_t pph = ((kc - 1) / ST) & 1u;
          if (!mbar_wait<0>(empty_bar(ps), pph, abort_flag, P.status, 23)) ok = false;
        }
        if (ok) issue(nxt);
      }
    }
    int got = ok ? 1 : 0;
    if (lane == 0 && ok)
      got = mbar_wait<0>(full_bar(s), (kc / ST) & 1u, abort_flag, P.status, 24) ? 1 : 0;
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) { ok = false; break; }
    const uint8_t* Xs = sm_gen + s * C::STAGE_BYTES;
    const float* Ws = reinterpret_cast<const float*>(Xs + C::RAW_BYTES);  // [l][k][TJ]

    if constexpr (L == 4) {
      // thread: 4 l x 4 j x 4 n; rows n = wn*16 + nl + 4t; acc index (l*4 + j)*4 + t
      const int jt = wj * 32 + jl * 4;
#pragma unroll
      for (int kk = 0; kk < KC; ++kk) {
        float4 x4[4], w4[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int row = wn * 16 + nl + 4 * t;
          const int chunk = (kk % KCR) ^ (row & 7);
          x4[t] = *reinterpret_cast<const float4*>(Xs + (kk / KCR) * TN * 128 + row * 128 + chunk * 16);
        }
#pragma unroll
        for (int l = 0; l < 4; ++l)
          w4[l] = *reinterpret_cast<const float4*>(Ws + (l * KC + kk) * TJ + jt);
#pragma unroll
        for (int l = 0; l < 4; ++l) {
          const float wv[4] = {w4[l].x, w4[l].y, w4[l].z, w4[l].w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float xv = l == 0 ? x4[t].x : (l == 1 ? x4[t].y : (l == 2 ? x4[t].z : x4[t].w));
              acc[(l * 4 + j) * 4 + t] = fmaf(wv[j], xv, acc[(l * 4 + j) * 4 + t]);
            }
        }
      }
    } else if constexpr (L == 2) {
      // thread: 2 l x 4 j x 8 n; rows n = wn*32 + nl + 4t; acc index (l*4 + j)*8 + t
      const int jt = wj * 32 + jl * 4;
#pragma unroll
      for (int k2 = 0; k2 < KC / 2; ++k2) {
        float4 x4[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int row = wn * 32 + nl + 4 * t;
          const int chunk = k2 ^ (row & 7);
          x4[t] = *reinterpret_cast<const float4*>(Xs + row * 128 + chunk * 16);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
          for (int l = 0; l < 2; ++l) {
            const float4 w4 = *reinterpret_cast<const float4*>(Ws + (l * KC + k2 * 2 + kk) * TJ + jt);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int t = 0; t < 8; ++t) {
                const float xv = kk == 0 ? (l == 0 ? x4[t].x : x4[t].y) : (l == 0 ? x4[t].z : x4[t].w);
                acc[(l * 4 + j) * 8 + t] = fmaf(wv[j], xv, acc[(l * 4 + j) * 8 + t]);
              }
          }
        }
      }
    } else {
      // thread: 8 j x 8 n; rows n = wn*32 + nl + 4t; j = h*32 + jl*4 + e; acc index (h*4+e)*8 + t
#pragma unroll
      for (int k4 = 0; k4 < KC / 4; ++k4) {
        float4 x4[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int row = wn * 32 + nl + 4 * t;
          const int chunk = k4 ^ (row & 7);
          x4[t] = *reinterpret_cast<const float4*>(Xs + row * 128 + chunk * 16);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float4 w0 = *reinterpret_cast<const float4*>(Ws + (k4 * 4 + kk) * TJ + jl * 4);
          const float4 w1 = *reinterpret_cast<const float4*>(Ws + (k4 * 4 + kk) * TJ + 32 + jl * 4);
          const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int m = 0; m < 8; ++m)
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              const float xv = kk == 0 ? x4[t].x : (kk == 1 ? x4[t].y : (kk == 2 ? x4[t].z : x4[t].w));
              acc[m * 8 + t] = fmaf(wv[m], xv, acc[m * 8 + t]);
            }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));
  }
  if (!__syncthreads_and(ok ? 1 : 0)) return;  // a bounded wait gave up: leave without storing

  // ---- epilogue: every (n, j) has L consecutive outputs ------------------------
  const int64_t B = P.batch;
  const int64_t abd = static_cast<int64_t>(P.a) * P.b * P.d;
  const float alpha = P.alpha;
  if constexpr (L == 4) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int64_t gn = n0 + wn * 16 + nl + 4 * t;
      if (gn >= B) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gj = j0 + wj * 32 + jl * 4 + j;
        if (gj >= P.b) continue;
        const int64_t col = (static_cast<int64_t>(i) * P.b + gj) * P.d + l0;
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (P.bias) bv = *reinterpret_cast<const float4*>(P.bias + col);
        float4 v;
        v.x = fmaf(alpha, acc[(0 * 4 + j) * 4 + t], bv.x);
        v.y = fmaf(alpha, acc[(1 * 4 + j) * 4 + t], bv.y);
        v.z = fmaf(alpha, acc[(2 * 4 + j) * 4 + t], bv.z);
        v.w = fmaf(alpha, acc[(3 * 4 + j) * 4 + t], bv.w);
        store_checked(P, gn * abd + col, v);
      }
    }
  } else if constexpr (L == 2) {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int64_t gn = n0 + wn * 32 + nl + 4 * t;
      if (gn >= B) continue;
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int gj = j0 + wj * 32 + jl * 4 + jp * 2;  // two consecutive j: 4 consecutive outputs
        if (gj >= P.b) continue;                        // b is a multiple of 4: pairs are whole
        const int64_t col = (static_cast<int64_t>(i) * P.b + gj) * 2;
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (P.bias) bv = *reinterpret_cast<const float4*>(P.bias + col);
        float4 v;
        v.x = fmaf(alpha, acc[(0 * 4 + jp * 2 + 0) * 8 + t], bv.x);
        v.y = fmaf(alpha, acc[(1 * 4 + jp * 2 + 0) * 8 + t], bv.y);
        v.z = fmaf(alpha, acc[(0 * 4 + jp * 2 + 1) * 8 + t], bv.z);
        v.w = fmaf(alpha, acc[(1 * 4 + jp * 2 + 1) * 8 + t], bv.w);
        store_checked(P, gn * abd + col, v);
      }
    }
  } else {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int64_t gn = n0 + wn * 32 + nl + 4 * t;
      if (gn >= B) continue;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int gj = j0 + h * 32 + jl * 4;
        if (gj >= P.b) continue;
        const int64_t col = static_cast<int64_t>(i) * P.b + gj;
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (P.bias) bv = *reinterpret_cast<const float4*>(P.bias + col);
        float4 v;
        v.x = fmaf(alpha, acc[(h * 4 + 0) * 8 + t], bv.x);
        v.y = fmaf(alpha, acc[(h * 4 + 1) * 8 + t], bv.y);
        v.z = fmaf(alpha, acc[(h * 4 + 2) * 8 + t], bv.z);
        v.w = fmaf(alpha, acc[(h * 4 + 3) * 8 + t], bv.w);
        store_checked(P, gn * abd + col, v);
      }
    }
  }
}

template <int L>
static int launch(const Problem& p, cudaStream_t stream) {
  using C = Cfg<L>;
  auto kern = ksmm_ffma_tma_first_kernel<L>;
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
  CUtensorMap tmX, tmW;
  int st;
  {
    // input rows seen as (c*d, a, batch): a box row is 32 contiguous floats = 32/L values of k
    const uint64_t dims[3] = {c * d, a, B};
    const uint64_t str[3] = {1, c * d, a * c * d};
    const uint32_t box[3] = {32, 1, static_cast<uint32_t>(C::TN)};
    if ((st = encode_map(&tmX, KSMM_F32, 3, p.in, dims, str, box, true)) != KSMM_OK) return st;
  }
  {
    // weights (b, c, a*d): TJ columns x KC rows x L consecutive blocks, dense in shared memory
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {static_cast<uint32_t>(C::TJ), static_cast<uint32_t>(C::KC),
                             static_cast<uint32_t>(L)};
    if ((st = encode_map(&tmW, KSMM_F32, 3, p.w, dims, str, box, false)) != KSMM_OK) return st;
  }
  Params P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + C::TN - 1) / C::TN);
  P.tiles_j = static_cast<int>((b + C::TJ - 1) / C::TJ);
  P.lgroups = p.d / L;
  P.nk = (p.c + C::KC - 1) / C::KC;
  P.alpha = p.alpha;
  P.bias = static_cast<const float*>(p.bias);
  P.out = static_cast<float*>(p.out);
  P.out_elems = static_cast<int64_t>(p.a) * p.b * p.d * p.batch;
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const int64_t total = static_cast<int64_t>(P.tiles_n) * P.tiles_j * P.lgroups * p.a;
  if (total <= 0 || total > 0x7fffffffLL)
    return set_error(KSMM_ERR_UNSUPPORTED, "fp32 TMA kernel: %lld tiles exceed the grid limit",
                     static_cast<long long>(total));
  kern<<<static_cast<unsigned>(total), C::NT, C::SMEM_BYTES, stream>>>(tmX, tmW, P);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "fp32 TMA kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

}  // namespace ffma_first

bool ffma_tma_first_supported(const Problem& p, bool check_pointers) {
  if (p.in_dtype != KSMM_F32 || p.out_dtype != KSMM_F32 || p.bs_last) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL) return false;
  if (!(p.d == 1 || p.d == 2 || p.d == 4)) return false;
  if (p.b % 4 != 0 || (static_cast<int64_t>(p.c) * p.d) % 4 != 0) return false;
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16 || reinterpret_cast<uintptr_t>(p.bias) % 16)
      return false;
  }
  return true;
}

int ffma_tma_first_launch(const Problem& p, cudaStream_t stream) {
  if (p.d == 1) return ffma_first::launch<1>(p, stream);
  if (p.d == 2) return ffma_first::launch<2>(p, stream);
  return ffma_first::launch<4>(p, stream);
}

}  // namespace ksmm
