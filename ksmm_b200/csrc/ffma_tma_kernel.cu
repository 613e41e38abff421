// fp32 FFMA kernel with TMA-staged operands (batch-last), kernel family
// KSMM_ALGO_SIMT, configurations 6 and 7.
//
// Same register tiling as simt_kernel.cuh (thread tile 8 x 8, lanes 8 (j) x 4 (n),
// conflict-free 128-bit shared loads), but the operand tiles are brought into a
// four-stage shared-memory ring by TMA: the strided rows of a block's input
// slice through the 4-D tensor map (batch, d, c, a), the weights through
// (b, c, a*d).  The compute warps therefore execute nothing but shared loads
// and FFMAs in the k loop (no global loads, address arithmetic, conversions or
// shared stores, which cost the register-staged kernel a quarter of its issue
// slots), and the warps are decoupled by per-stage mbarriers instead of a
// block-wide barrier per k chunk.  Out-of-range k, j and batch entries are
// zero-filled by TMA; stores are predicated.
//
// Requirements (else the register-staged kernel runs): fp32, batch-last,
// batch % 4 == 0, b % 4 == 0, 16-byte aligned pointers.
//
// Reference counterpart: kernel_bs_last_float
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_float.cuh:301-491).
#include <cuda.h>

#include <atomic>

#include "tc_host.h"
#include "tc_ptx.cuh"

namespace ksmm {
namespace ffma {

using namespace ksmm::tc;

struct Params {
  int a, b, c, d;
  int64_t batch;
  int tiles_n, tiles_j;
  int nk;
  float alpha;
  const float* bias;
  float* out;
  int* status;
};

template <int WJ>
struct Cfg {
  static constexpr int KC = 16;
  static constexpr int ST = 4;
  static constexpr int TN = 128;
  static constexpr int TJ = 64 * WJ;
  static constexpr int NT = WJ * 4 * 32;
  static constexpr int X_BYTES = KC * TN * 4;
  static constexpr int W_BYTES = KC * TJ * 4;
  static constexpr int STAGE_BYTES = X_BYTES + W_BYTES;
  static constexpr int SMEM_BYTES = ST * STAGE_BYTES + 128 + 128;
};

template <int WJ>
__global__ void __launch_bounds__(WJ * 128, 512 / (WJ * 128))
    ksmm_ffma_tma_kernel(const __grid_constant__ CUtensorMap tmX,
                         const __grid_constant__ CUtensorMap tmW, const Params P) {
  using C = Cfg<WJ>;
  constexpr int KC = C::KC, ST = C::ST, TN = C::TN, TJ = C::TJ;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sm0 = (raw + 127u) & ~127u;  // TMA destinations: 128-byte aligned
  const float* sm_gen = reinterpret_cast<const float*>(smem_raw + (sm0 - raw));
  const uint32_t bar0 = sm0 + ST * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (ST + s); };
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_raw + (sm0 - raw) + ST * C::STAGE_BYTES + 8 * 2 * ST);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int wj = warp % WJ, wn = warp / WJ;
  const int jl = lane & 7, nl = lane >> 3;

  int64_t bid = blockIdx.x;
  const int tn = static_cast<int>(bid % P.tiles_n);
  bid /= P.tiles_n;
  const int tj = static_cast<int>(bid % P.tiles_j);
  const int blk = static_cast<int>(bid / P.tiles_j);
  const int i = blk / P.d, l = blk % P.d;
  const int n0 = tn * TN, j0 = tj * TJ;
  const int nk = P.nk;

  if (tid == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), WJ * 4);  // one arrival per warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  auto issue = [&](int kc) {
    const int s = kc % ST;
    const uint32_t dst = sm0 + s * C::STAGE_BYTES;
    mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
    tma_load_4d(dst, &tmX, full_bar(s), n0, l, kc * KC, i);
    tma_load_3d(dst + C::X_BYTES, &tmW, full_bar(s), j0, kc * KC, blk);
  };
  if (tid == 0) {
    for (int kc = 0; kc < ST - 1 && kc < nk; ++kc) issue(kc);
  }

  float acc[8][8];
#pragma unroll
  for (int m = 0; m < 8; ++m)
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[m][t] = 0.f;

  const int xoff = wn * 32 + nl * 4;
  const int woff = wj * 64 + jl * 4;
  bool ok = true;
  for (int kc = 0; kc < nk; ++kc) {
    const int s = kc % ST;
    if (tid == 0) {
      // refill the stage that chunk kc - 1 used, once every warp has released it
      const int nxt = kc + ST - 1;
      if (nxt < nk) {
        if (kc >= 1) {
          const int ps = (kc - 1) % ST;
          const uint32_t pph = ((kc - 1) / ST) & 1u;
          if (!mbar_wait<0>(empty_bar(ps), pph, abort_flag, P.status, 21)) ok = false;
        }
        if (ok) issue(nxt);
      }
    }
    // one lane per warp polls the barrier; the warp-wide shuffle orders the others after it
    int got = ok ? 1 : 0;
    if (lane == 0 && ok) got = mbar_wait<0>(full_bar(s), (kc / ST) & 1u, abort_flag, P.status, 22) ? 1 : 0;
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) { ok = false; break; }
    const float* Xs = sm_gen + s * (C::STAGE_BYTES / 4);
    const float* Ws = Xs + C::X_BYTES / 4;
#pragma unroll
    for (int kk = 0; kk < KC; ++kk) {
      const float4 x0 = *reinterpret_cast<const float4*>(Xs + kk * TN + xoff);
      const float4 x1 = *reinterpret_cast<const float4*>(Xs + kk * TN + xoff + 16);
      const float4 w0 = *reinterpret_cast<const float4*>(Ws + kk * TJ + woff);
      const float4 w1 = *reinterpret_cast<const float4*>(Ws + kk * TJ + woff + 32);
      const float xf[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
      const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int t = 0; t < 8; ++t) acc[m][t] = fmaf(wf[m], xf[t], acc[m][t]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));
  }
  if (!__syncthreads_and(ok ? 1 : 0)) return;  // a bounded wait gave up: leave without storing

  // ---- epilogue: alpha, bias, 128-bit stores --------------------------------
  const int64_t B = P.batch;
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int gj = j0 + wj * 64 + (m >> 2) * 32 + jl * 4 + (m & 3);
    if (gj >= P.b) continue;
    const int64_t row = (static_cast<int64_t>(i) * P.b + gj) * P.d + l;
    const float bv = P.bias ? P.bias[row] : 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int64_t gn = n0 + wn * 32 + half * 16 + nl * 4;
      if (gn < B) {
        float4 v;
        v.x = fmaf(P.alpha, acc[m][half * 4 + 0], bv);
        v.y = fmaf(P.alpha, acc[m][half * 4 + 1], bv);
        v.z = fmaf(P.alpha, acc[m][half * 4 + 2], bv);
        v.w = fmaf(P.alpha, acc[m][half * 4 + 3], bv);
        *reinterpret_cast<float4*>(P.out + row * B + gn) = v;
      }
    }
  }
}

template <int WJ>
static int launch(const Problem& p, cudaStream_t stream) {
  using C = Cfg<WJ>;
  auto kern = ksmm_ffma_tma_kernel<WJ>;
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
    const uint64_t dims[4] = {B, d, c, a};
    const uint64_t str[4] = {1, B, d * B, c * d * B};
    const uint32_t box[4] = {static_cast<uint32_t>(C::TN), 1, static_cast<uint32_t>(C::KC), 1};
    if ((st = encode_map(&tmX, KSMM_F32, 4, p.in, dims, str, box, false)) != KSMM_OK) return st;
  }
  {
    const uint64_t dims[3] = {b, c, a * d};
    const uint64_t str[3] = {1, b, c * b};
    const uint32_t box[3] = {static_cast<uint32_t>(C::TJ), static_cast<uint32_t>(C::KC), 1};
    if ((st = encode_map(&tmW, KSMM_F32, 3, p.w, dims, str, box, false)) != KSMM_OK) return st;
  }
  Params P;
  P.a = p.a; P.b = p.b; P.c = p.c; P.d = p.d;
  P.batch = p.batch;
  P.tiles_n = static_cast<int>((B + C::TN - 1) / C::TN);
  P.tiles_j = static_cast<int>((b + C::TJ - 1) / C::TJ);
  P.nk = (p.c + C::KC - 1) / C::KC;
  P.alpha = p.alpha;
  P.bias = static_cast<const float*>(p.bias);
  P.out = static_cast<float*>(p.out);
  P.status = status_word();
  if (!P.status) return set_error(KSMM_ERR_CUDA, "cannot resolve the device status word");
  const int64_t total = static_cast<int64_t>(P.tiles_n) * P.tiles_j * p.a * p.d;
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

}  // namespace ffma

bool ffma_tma_supported(const Problem& p, bool check_pointers) {
  if (p.in_dtype != KSMM_F32 || p.out_dtype != KSMM_F32 || !p.bs_last) return false;
  if (p.batch <= 0 || p.batch > 0x7fffffffLL || p.batch % 4 != 0 || p.b % 4 != 0) return false;
  if (check_pointers) {
    if (reinterpret_cast<uintptr_t>(p.in) % 16 || reinterpret_cast<uintptr_t>(p.w) % 16 ||
        reinterpret_cast<uintptr_t>(p.out) % 16)
      return false;
  }
  return true;
}

int ffma_tma_launch(const Problem& p, int wide, cudaStream_t stream) {
  return wide ? ffma::launch<2>(p, stream) : ffma::launch<1>(p, stream);
}

}  // namespace ksmm
