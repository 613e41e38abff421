// FFMA register-tiled KSMM kernel (kernel family KSMM_ALGO_SIMT).
//
// One CTA computes a (TJ output rows j) x (TN batch entries) tile of one
// (i_a, i_d) block of one factor: Y4[i,j,l,n] = sum_k W[i,j,k,l] * X4[i,k,l,n].
// The k loop runs over chunks of KC input rows that are staged through shared
// memory as fp32, [k][n] for the input slice and [k][j] for the weights, with
// register-staged double buffering (global loads of chunk kc+1 are in flight
// while chunk kc is consumed; one __syncthreads per chunk).  Each thread
// accumulates a TMJ x 8 register tile by outer products fed by 128-bit shared
// loads; lanes are arranged 8 (j) x 4 (n) so that both operand loads are
// conflict-free broadcasts.
//
// This family handles every shape, alignment, element type and both layouts
// (tails are predicated, vector accesses fall back to scalar ones when the
// alignment rules do not hold); it is the fp32 production path (fp32 KSMM is
// FFMA-bound for b, c >= 48) and the fallback for the tensor-core family.
//
// Reference counterpart: kernel_bs_first_float / kernel_bs_last_float
// (src/ksmm_py/layer/kronecker_sparse/template_kernels_float.cuh:89-286,
// 301-491), which need TILEX | b, TILEK | c, TILEY | batch, 32-bit offsets and
// a hand-tuned table row per pattern.
#pragma once

#include "common.cuh"

namespace ksmm {

struct SimtParams {
  Problem p;
  int tiles_n;
  int tiles_j;
  unsigned flags;  // bit0: input vector loads legal, bit1: weights, bit2: output stores
};

template <typename TIn, typename TOut, bool BS_LAST, int TMJ, int WJ, int WN>
struct SimtCfg {
  static constexpr int KC = 16;
  static constexpr int TN = WN * 32;
  static constexpr int TJ = WJ * 8 * TMJ;
  static constexpr int NT = WJ * WN * 32;
  static constexpr int TNP = TN + 4;
  static constexpr int VJ = TMJ >= 4 ? 4 : TMJ;
  static constexpr int HJ = TMJ / VJ;
  static constexpr int XPT = KC * TN / NT;
  static constexpr int WPT = KC * TJ / NT;
  static constexpr int VW = WPT >= 4 ? 4 : WPT;
  static_assert(XPT % 4 == 0, "input staging must be a whole number of 4-vectors");
  static_assert(WPT >= 1 && WPT % VW == 0, "weight staging");
};

template <typename TIn, typename TOut, bool BS_LAST, int TMJ, int WJ, int WN>
__global__ void __launch_bounds__(WJ* WN * 32, 512 / (WJ * WN * 32))
    ksmm_simt_kernel(const SimtParams sp) {
  using C = SimtCfg<TIn, TOut, BS_LAST, TMJ, WJ, WN>;
  constexpr int KC = C::KC, TN = C::TN, TJ = C::TJ, NT = C::NT, TNP = C::TNP;
  constexpr int VJ = C::VJ, HJ = C::HJ, XPT = C::XPT, WPT = C::WPT, VW = C::VW;

  __shared__ __align__(16) float Xs[2][KC][TNP];
  __shared__ __align__(16) float Ws[2][KC][TJ];

  const Problem& p = sp.p;
  const int a = p.a, b = p.b, c = p.c, d = p.d;
  (void)a;
  const int64_t B = p.batch;
  const bool xvec = sp.flags & 1u, wvec = sp.flags & 2u, yvec = sp.flags & 4u;

  // block -> (batch tile, j tile, block (i,l)); batch tile fastest so that
  // concurrently running CTAs share one weight tile in L2
  int64_t bid = blockIdx.x;
  const int tn = static_cast<int>(bid % sp.tiles_n);
  bid /= sp.tiles_n;
  const int tj = static_cast<int>(bid % sp.tiles_j);
  const int blk = static_cast<int>(bid / sp.tiles_j);
  const int i = blk / d, l = blk % d;
  const int64_t n0 = static_cast<int64_t>(tn) * TN;
  const int j0 = tj * TJ;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int wj = warp % WJ, wn = warp / WJ;
  const int jl = lane & 7, nl = lane >> 3;

  const TIn* __restrict__ X = static_cast<const TIn*>(p.in);
  const TIn* __restrict__ W = static_cast<const TIn*>(p.w);
  const int64_t acd = static_cast<int64_t>(p.a) * c * d;
  const int64_t abd = static_cast<int64_t>(p.a) * b * d;

  float acc[TMJ][8];
#pragma unroll
  for (int m = 0; m < TMJ; ++m)
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[m][t] = 0.f;

  float xr[XPT];
  float wr[WPT];

  auto load_chunk = [&](int k0) {
    // ---- input slice -----------------------------------------------------
    if (xvec) {
#pragma unroll
      for (int r = 0; r < XPT / 4; ++r) {
        const int v = tid + r * NT;
        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (BS_LAST) {
          const int k = v / (TN / 4), n4 = v % (TN / 4);
          const int gk = k0 + k;
          const int64_t gn = n0 + n4 * 4;
          if (gk < c && gn < B) {
            const int64_t row = (static_cast<int64_t>(i) * c + gk) * d + l;
            load_vec<TIn, 4>(X + row * B + gn, tmp);
          }
        } else {
          const int n = v / (KC / 4), k4 = v % (KC / 4);
          const int gk = k0 + k4 * 4;
          const int64_t gn = n0 + n;
          if (gk < c && gn < B) {
            load_vec<TIn, 4>(X + gn * acd + static_cast<int64_t>(i) * c + gk, tmp);
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) xr[r * 4 + e] = tmp[e];
      }
    } else {
#pragma unroll
      for (int r = 0; r < XPT; ++r) {
        const int v = tid + r * NT;
        float val = 0.f;
        if constexpr (BS_LAST) {
          const int k = v / TN, n = v % TN;
          const int gk = k0 + k;
          const int64_t gn = n0 + n;
          if (gk < c && gn < B) {
            const int64_t row = (static_cast<int64_t>(i) * c + gk) * d + l;
            val = ElemTraits<TIn>::to_float(X[row * B + gn]);
          }
        } else {
          const int n = v / KC, k = v % KC;
          const int gk = k0 + k;
          const int64_t gn = n0 + n;
          if (gk < c && gn < B) {
            val = ElemTraits<TIn>::to_float(
                X[gn * acd + (static_cast<int64_t>(i) * c + gk) * d + l]);
          }
        }
        xr[r] = val;
      }
    }
    // ---- weights -----------------------------------------------------------
    const int64_t wbase = static_cast<int64_t>(blk) * c;
    if (wvec) {
#pragma unroll
      for (int r = 0; r < WPT / VW; ++r) {
        const int v = tid + r * NT;
        const int k = v / (TJ / VW), jv = v % (TJ / VW);
        const int gk = k0 + k, gj = j0 + jv * VW;
        float tmp[VW];
#pragma unroll
        for (int e = 0; e < VW; ++e) tmp[e] = 0.f;
        if (gk < c && gj < b) load_vec<TIn, VW>(W + (wbase + gk) * b + gj, tmp);
#pragma unroll
        for (int e = 0; e < VW; ++e) wr[r * VW + e] = tmp[e];
      }
    } else {
#pragma unroll
      for (int r = 0; r < WPT; ++r) {
        const int v = tid + r * NT;
        const int k = v / TJ, j = v % TJ;
        const int gk = k0 + k, gj = j0 + j;
        float val = 0.f;
        if (gk < c && gj < b) val = ElemTraits<TIn>::to_float(W[(wbase + gk) * b + gj]);
        wr[r] = val;
      }
    }
  };

  auto store_chunk = [&](int buf) {
    if (xvec) {
#pragma unroll
      for (int r = 0; r < XPT / 4; ++r) {
        const int v = tid + r * NT;
        if constexpr (BS_LAST) {
          const int k = v / (TN / 4), n4 = v % (TN / 4);
          *reinterpret_cast<float4*>(&Xs[buf][k][n4 * 4]) =
              make_float4(xr[r * 4 + 0], xr[r * 4 + 1], xr[r * 4 + 2], xr[r * 4 + 3]);
        } else {
          const int n = v / (KC / 4), k4 = v % (KC / 4);
#pragma unroll
          for (int e = 0; e < 4; ++e) Xs[buf][k4 * 4 + e][n] = xr[r * 4 + e];
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < XPT; ++r) {
        const int v = tid + r * NT;
        if constexpr (BS_LAST) {
          Xs[buf][v / TN][v % TN] = xr[r];
        } else {
          Xs[buf][v % KC][v / KC] = xr[r];
        }
      }
    }
    if (wvec) {
#pragma unroll
      for (int r = 0; r < WPT / VW; ++r) {
        const int v = tid + r * NT;
        const int k = v / (TJ / VW), jv = v % (TJ / VW);
#pragma unroll
        for (int e = 0; e < VW; ++e) Ws[buf][k][jv * VW + e] = wr[r * VW + e];
      }
    } else {
#pragma unroll
      for (int r = 0; r < WPT; ++r) {
        const int v = tid + r * NT;
        Ws[buf][v / TJ][v % TJ] = wr[r];
      }
    }
  };

  const int nk = (c + KC - 1) / KC;
  load_chunk(0);
  store_chunk(0);
  __syncthreads();

  const int xoff = wn * 32 + nl * 4;
  const int woff = wj * 8 * TMJ + jl * VJ;

  for (int kc = 0; kc < nk; ++kc) {
    const int buf = kc & 1;
    if (kc + 1 < nk) load_chunk((kc + 1) * KC);
#pragma unroll
    for (int kk = 0; kk < KC; ++kk) {
      float xf[8], wf[TMJ];
      const float4 x0 = *reinterpret_cast<const float4*>(&Xs[buf][kk][xoff]);
      const float4 x1 = *reinterpret_cast<const float4*>(&Xs[buf][kk][xoff + 16]);
      xf[0] = x0.x; xf[1] = x0.y; xf[2] = x0.z; xf[3] = x0.w;
      xf[4] = x1.x; xf[5] = x1.y; xf[6] = x1.z; xf[7] = x1.w;
#pragma unroll
      for (int h = 0; h < HJ; ++h) {
        const float* wp = &Ws[buf][kk][woff + h * 8 * VJ];
        if constexpr (VJ == 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(wp);
          wf[h * 4 + 0] = w4.x; wf[h * 4 + 1] = w4.y; wf[h * 4 + 2] = w4.z; wf[h * 4 + 3] = w4.w;
        } else if constexpr (VJ == 2) {
          const float2 w2 = *reinterpret_cast<const float2*>(wp);
          wf[h * 2 + 0] = w2.x; wf[h * 2 + 1] = w2.y;
        } else {
          wf[h] = *wp;
        }
      }
#pragma unroll
      for (int m = 0; m < TMJ; ++m)
#pragma unroll
        for (int t = 0; t < 8; ++t) acc[m][t] = fmaf(wf[m], xf[t], acc[m][t]);
    }
    if (kc + 1 < nk) store_chunk(buf ^ 1);
    __syncthreads();
  }

  // ---- epilogue: alpha, bias, conversion, vector stores ---------------------
  TOut* __restrict__ Y = static_cast<TOut*>(p.out);
  const TOut* __restrict__ bias = static_cast<const TOut*>(p.bias);
  const float alpha = p.alpha;

  if constexpr (BS_LAST) {
#pragma unroll
    for (int m = 0; m < TMJ; ++m) {
      const int h = m / VJ, e = m % VJ;
      const int gj = j0 + wj * 8 * TMJ + h * 8 * VJ + jl * VJ + e;
      if (gj >= b) continue;
      const int64_t row = (static_cast<int64_t>(i) * b + gj) * d + l;
      const float bv = bias ? ElemTraits<TOut>::to_float(bias[row]) : 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t gn = n0 + wn * 32 + half * 16 + nl * 4;
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = fmaf(alpha, acc[m][half * 4 + t], bv);
        if (yvec) {
          if (gn < B) store_vec<TOut, 4>(Y + row * B + gn, v);
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (gn + t < B) Y[row * B + gn + t] = ElemTraits<TOut>::from_float(v[t]);
        }
      }
    }
  } else {
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int64_t gn = n0 + wn * 32 + (t >> 2) * 16 + nl * 4 + (t & 3);
      if (gn >= B) continue;
#pragma unroll
      for (int h = 0; h < HJ; ++h) {
        const int gj = j0 + wj * 8 * TMJ + h * 8 * VJ + jl * VJ;
        if (yvec) {
          if (gj < b) {
            const int64_t col = static_cast<int64_t>(i) * b + gj;  // d == 1 on this path
            float v[VJ];
#pragma unroll
            for (int e = 0; e < VJ; ++e) {
              const float bv = bias ? ElemTraits<TOut>::to_float(bias[col + e]) : 0.f;
              v[e] = fmaf(alpha, acc[h * VJ + e][t], bv);
            }
            store_vec<TOut, VJ>(Y + gn * abd + col, v);
          }
        } else {
#pragma unroll
          for (int e = 0; e < VJ; ++e) {
            if (gj + e < b) {
              const int64_t col = (static_cast<int64_t>(i) * b + gj + e) * d + l;
              const float bv = bias ? ElemTraits<TOut>::to_float(bias[col]) : 0.f;
              Y[gn * abd + col] = ElemTraits<TOut>::from_float(fmaf(alpha, acc[h * VJ + e][t], bv));
            }
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host side: configuration table and launcher
// ---------------------------------------------------------------------------
struct SimtConfigInfo {
  int tmj, wj, wn;
  int tile_j() const { return wj * 8 * tmj; }
  int tile_n() const { return wn * 32; }
};

static constexpr SimtConfigInfo kSimtConfigs[] = {
    {8, 2, 4},  // 0: 128 j x 128 n, 256 threads
    {8, 1, 4},  // 1:  64 j x 128 n, 128 threads
    {4, 1, 4},  // 2:  32 j x 128 n, 128 threads
    {2, 1, 4},  // 3:  16 j x 128 n, 128 threads
    {8, 1, 8},  // 4:  64 j x 256 n, 256 threads
    {1, 1, 4},  // 5:   8 j x 128 n, 128 threads
};
static constexpr int kNumSimtConfigs = sizeof(kSimtConfigs) / sizeof(kSimtConfigs[0]);

template <typename TIn, typename TOut, bool BS_LAST, int TMJ, int WJ, int WN>
int simt_launch_one(const Problem& p, cudaStream_t stream) {
  using C = SimtCfg<TIn, TOut, BS_LAST, TMJ, WJ, WN>;
  SimtParams sp;
  sp.p = p;
  sp.tiles_n = static_cast<int>((p.batch + C::TN - 1) / C::TN);
  sp.tiles_j = (p.b + C::TJ - 1) / C::TJ;
  const int64_t total = static_cast<int64_t>(sp.tiles_n) * sp.tiles_j * p.a * p.d;
  if (total <= 0 || total > 0x7fffffffLL)
    return set_error(KSMM_ERR_UNSUPPORTED, "simt kernel: %lld tiles exceed the grid limit",
                     static_cast<long long>(total));
  const uintptr_t xin = reinterpret_cast<uintptr_t>(p.in);
  const uintptr_t win = reinterpret_cast<uintptr_t>(p.w);
  const uintptr_t yout = reinterpret_cast<uintptr_t>(p.out);
  const uintptr_t bptr = reinterpret_cast<uintptr_t>(p.bias);
  unsigned flags = 0;
  if (BS_LAST) {
    if (p.batch % 4 == 0 && xin % (4 * sizeof(TIn)) == 0) flags |= 1u;
    if (p.batch % 4 == 0 && yout % (4 * sizeof(TOut)) == 0) flags |= 4u;
  } else {
    if (p.d == 1 && p.c % 4 == 0 && xin % (4 * sizeof(TIn)) == 0) flags |= 1u;
    if (p.d == 1 && p.b % C::VJ == 0 && yout % (C::VJ * sizeof(TOut)) == 0 &&
        bptr % (C::VJ * sizeof(TOut)) == 0)
      flags |= 4u;
  }
  if (p.b % C::VW == 0 && win % (C::VW * sizeof(TIn)) == 0) flags |= 2u;
  sp.flags = flags;
  ksmm_simt_kernel<TIn, TOut, BS_LAST, TMJ, WJ, WN>
      <<<static_cast<unsigned>(total), C::NT, 0, stream>>>(sp);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "simt kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

template <typename TIn, typename TOut, bool BS_LAST>
int simt_launch_cfg(const Problem& p, int config, cudaStream_t stream) {
  switch (config) {
    case 0: return simt_launch_one<TIn, TOut, BS_LAST, 8, 2, 4>(p, stream);
    case 1: return simt_launch_one<TIn, TOut, BS_LAST, 8, 1, 4>(p, stream);
    case 2: return simt_launch_one<TIn, TOut, BS_LAST, 4, 1, 4>(p, stream);
    case 3: return simt_launch_one<TIn, TOut, BS_LAST, 2, 1, 4>(p, stream);
    case 4: return simt_launch_one<TIn, TOut, BS_LAST, 8, 1, 8>(p, stream);
    case 5: return simt_launch_one<TIn, TOut, BS_LAST, 1, 1, 4>(p, stream);
    default: return set_error(KSMM_ERR_BAD_ARGUMENT, "simt kernel: no configuration %d", config);
  }
}

template <typename TIn, typename TOut>
int simt_launch_typed(const Problem& p, int config, cudaStream_t stream) {
  return p.bs_last ? simt_launch_cfg<TIn, TOut, true>(p, config, stream)
                   : simt_launch_cfg<TIn, TOut, false>(p, config, stream);
}

// Heuristic default: the j tile with the least padding, larger tiles on ties.
inline int simt_default_config(const Problem& p) {
  int best = 1;
  int64_t best_cost = -1;
  const int order[] = {0, 1, 2, 3, 5};
  for (int ci : order) {
    const int tj = kSimtConfigs[ci].tile_j();
    const int64_t padded = static_cast<int64_t>((p.b + tj - 1) / tj) * tj;
    // small tiles re-read the input slice more often: charge them slightly
    const int64_t cost = padded * 64 + (tj < 64 ? (64 / tj) * 4 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = ci;
    }
  }
  return best;
}

}  // namespace ksmm
