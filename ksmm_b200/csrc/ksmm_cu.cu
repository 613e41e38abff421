// C ABI of libksmm_cu.so: argument checking, kernel-family dispatch, the
// in-process tuner cache, chained factors, and the host-buffer variant.
// Declarations and the reference interfaces they stand in for: include/ksmm_cu.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "tc_kernel.h"

namespace ksmm {

// ---------------------------------------------------------------------------
// error plumbing
// ---------------------------------------------------------------------------
static thread_local char g_last_error[512] = "";
static std::atomic<uint64_t> g_launches{0};
static std::atomic<uint64_t> g_allocs{0};  // device allocations made by the library itself

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return status;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

#define KSMM_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess)                                                             \
      return set_error(KSMM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

// per-dtype instantiations live in their own translation units
int simt_launch_f32(const Problem& p, int config, cudaStream_t stream);
int simt_launch_f16(const Problem& p, int config, cudaStream_t stream);
int simt_launch_bf16(const Problem& p, int config, cudaStream_t stream);
int simt_launch_f8(const Problem& p, int config, cudaStream_t stream);
int simt_default_config_for(const Problem& p);
int simt_num_configs();
// fp32 batch-last kernel with TMA-staged operands (ffma_tma_kernel.cu): configurations
// kFfmaTmaWide (128 x 128 tile) and kFfmaTmaNarrow (64 x 128 tile) of the FFMA family
bool ffma_tma_supported(const Problem& p, bool check_pointers);
int ffma_tma_launch(const Problem& p, int wide, cudaStream_t stream);
// fp32 batch-first kernel with TMA-staged operands (ffma_tma_first.cu): configuration kFfmaTmaFirst
bool ffma_tma_first_supported(const Problem& p, bool check_pointers);
int ffma_tma_first_launch(const Problem& p, cudaStream_t stream);
int launch_transpose(const void* in, void* out, int64_t rows, int64_t cols, int es,
                     cudaStream_t stream);
// backward.cu
int launch_transpose_blocks(const void* in, void* out, int64_t nblk, int c, int b, int es, cudaStream_t stream);
size_t wgrad_workspace_bytes(const Problem& p);
int wgrad_launch(const Problem& p, const void* grad_out, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream);
static constexpr int kFfmaTmaWide = 6, kFfmaTmaNarrow = 7, kFfmaTmaFirst = 8, kNumFfmaConfigs = 9;

static int simt_launch_raw(const Problem& p, int config, cudaStream_t stream) {
  if (config < 0) {
    if (ffma_tma_supported(p, true) && p.b >= 48)
      config = kFfmaTmaNarrow;  // 64 x 128 tiles, four CTAs per SM: fastest in every measured case
    else if (ffma_tma_first_supported(p, true) && p.b >= 48)
      config = kFfmaTmaFirst;
    else
      config = simt_default_config_for(p);
  }
  if (config == kFfmaTmaWide || config == kFfmaTmaNarrow) {
    if (!ffma_tma_supported(p, true))
      return set_error(KSMM_ERR_UNSUPPORTED,
                       "the TMA-staged fp32 kernel needs fp32, batch-last, batch %% 4 == 0, "
                       "b %% 4 == 0 and 16-byte aligned pointers");
    return ffma_tma_launch(p, config == kFfmaTmaWide, stream);
  }
  if (config == kFfmaTmaFirst) {
    if (!ffma_tma_first_supported(p, true))
      return set_error(KSMM_ERR_UNSUPPORTED,
                       "the TMA-staged batch-first fp32 kernel needs fp32, batch-first, d in {1, 2, 4}, "
                       "b %% 4 == 0, c*d %% 4 == 0 and 16-byte aligned pointers");
    return ffma_tma_first_launch(p, stream);
  }
  switch (p.in_dtype) {
    case KSMM_F32:
      if (p.out_dtype != KSMM_F32)
        return set_error(KSMM_ERR_UNSUPPORTED, "fp32 input needs an fp32 output");
      return simt_launch_f32(p, config, stream);
    case KSMM_F16:
      if (p.out_dtype != KSMM_F16)
        return set_error(KSMM_ERR_UNSUPPORTED, "fp16 input needs an fp16 output");
      return simt_launch_f16(p, config, stream);
    case KSMM_BF16:
      if (p.out_dtype != KSMM_BF16)
        return set_error(KSMM_ERR_UNSUPPORTED, "bf16 input needs a bf16 output");
      return simt_launch_bf16(p, config, stream);
    case KSMM_F8E4M3:
      return simt_launch_f8(p, config, stream);
    default:
      return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown input dtype %d", p.in_dtype);
  }
}

// ---------------------------------------------------------------------------
// tuner cache: (batch, a, b, c, d, in_dtype, out_dtype, bs_last) -> (algo, config)
// ---------------------------------------------------------------------------
using ChoiceKey = std::tuple<int64_t, int, int, int, int, int, int, int>;
struct Choice {
  int algo, config;
};
static std::mutex g_choice_mu;
static std::map<ChoiceKey, Choice> g_choices;

// The FFMA family has no activation in its epilogues: an element-wise pass over the output
// follows the kernel (the tensor-core kernels apply it in their epilogue).
template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(T* data, int64_t n, int act) {
  for (int64_t q = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; q < n;
       q += static_cast<int64_t>(gridDim.x) * 256)
    data[q] = ElemTraits<T>::from_float(sizeof(T) == 2 && act == KSMM_ACT_GELU
                                            ? gelu_16bit(ElemTraits<T>::to_float(data[q]))
                                            : apply_activation(ElemTraits<T>::to_float(data[q]), act));
}

// out += residual, for the kernels whose epilogue has no residual input
template <typename T>
__global__ void __launch_bounds__(256) residual_kernel(T* data, const T* __restrict__ res, int64_t n) {
  for (int64_t q = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; q < n;
       q += static_cast<int64_t>(gridDim.x) * 256)
    data[q] = ElemTraits<T>::from_float(ElemTraits<T>::to_float(data[q]) + ElemTraits<T>::to_float(res[q]));
}

static int residual_pass(const Problem& p, cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(p.a) * p.b * p.d * p.batch;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  if (p.out_dtype == KSMM_F32)
    residual_kernel<float><<<grid, 256, 0, stream>>>(static_cast<float*>(p.out), static_cast<const float*>(p.residual), n);
  else if (p.out_dtype == KSMM_F16)
    residual_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<__half*>(p.out), static_cast<const __half*>(p.residual), n);
  else
    residual_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p.out),
                                                             static_cast<const __nv_bfloat16*>(p.residual), n);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "residual kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

static int simt_launch(const Problem& p, int config, cudaStream_t stream) {
  int st = simt_launch_raw(p, config, stream);
  if (st != KSMM_OK || p.activation == 0) return st;
  const int64_t n = static_cast<int64_t>(p.a) * p.b * p.d * p.batch;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  if (p.out_dtype == KSMM_F32)
    activation_kernel<float><<<grid, 256, 0, stream>>>(static_cast<float*>(p.out), n, p.activation);
  else if (p.out_dtype == KSMM_F16)
    activation_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<__half*>(p.out), n, p.activation);
  else
    activation_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p.out), n,
                                                               p.activation);
  count_launch();
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "activation kernel launch failed: %s", cudaGetErrorString(err));
  return KSMM_OK;
}

static ChoiceKey key_of(const Problem& p) {
  return ChoiceKey(p.batch, p.a, p.b, p.c, p.d, p.in_dtype, p.out_dtype, p.bs_last);
}

static bool lookup_choice(const Problem& p, Choice* out) {
  std::lock_guard<std::mutex> g(g_choice_mu);
  auto it = g_choices.find(key_of(p));
  if (it == g_choices.end()) return false;
  *out = it->second;
  return true;
}

static int check_problem(const Problem& p) {
  // an empty batch has empty (possibly null) input and output buffers
  if (p.batch != 0 && (!p.in || !p.w || !p.out))
    return set_error(KSMM_ERR_BAD_ARGUMENT, "null pointer (input=%p values=%p output=%p)", p.in,
                     p.w, p.out);
  if (p.a <= 0 || p.b <= 0 || p.c <= 0 || p.d <= 0)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "pattern (%d,%d,%d,%d) must be positive", p.a, p.b,
                     p.c, p.d);
  if (p.batch < 0) return set_error(KSMM_ERR_BAD_ARGUMENT, "negative batch");
  if (p.in_dtype < KSMM_F32 || p.in_dtype > KSMM_F8E4M3)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown input dtype %d", p.in_dtype);
  if (p.out_dtype < KSMM_F32 || p.out_dtype > KSMM_BF16)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unsupported output dtype %d", p.out_dtype);
  if (p.bs_last != 0 && p.bs_last != 1)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "bs_last must be 0 or 1");
  if (p.activation < 0 || p.activation > 2)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown activation %d", p.activation);
  return KSMM_OK;
}

// ---------------------------------------------------------------------------
// Layout-conversion path for batch-first factors with d > 1 that no direct
// kernel covers (e.g. d = 16): transpose the input to batch-last, run the
// batch-last kernel, transpose the result back.  Three times the minimal HBM
// traffic, but every access is a full line, which beats the strided
// register-staged kernel by a wide margin.  The two transposed buffers come from
// the problem's scratch (chains carve it out of their workspace) or, without
// one, from a library-owned buffer per (device, stream).
// ---------------------------------------------------------------------------
static size_t align_up(size_t v, size_t al) { return (v + al - 1) / al * al; }

struct ConvScratch {
  void* ptr = nullptr;
  size_t cap = 0;
};
static std::mutex g_conv_mu;
static std::map<std::pair<int, cudaStream_t>, ConvScratch> g_conv;

int layout_scratch(const Problem& p, size_t bytes, cudaStream_t stream, void** out) {
  if (p.scratch != nullptr && p.scratch_bytes >= bytes) {
    *out = p.scratch;
    return KSMM_OK;
  }
  if (p.no_alloc)
    return set_error(KSMM_ERR_WORKSPACE,
                     "this factor needs %zu bytes of layout scratch (%zu given) and the call may not "
                     "allocate", bytes, p.scratch ? p.scratch_bytes : static_cast<size_t>(0));
  int dev = 0;
  KSMM_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> g(g_conv_mu);
  ConvScratch& sc = g_conv[std::make_pair(dev, stream)];
  if (sc.cap < bytes) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &cs);
    if (cs != cudaStreamCaptureStatusNone)
      return set_error(KSMM_ERR_WORKSPACE,
                       "the layout scratch must grow to %zu bytes, which cannot happen inside a "
                       "stream capture: pass a scratch, or make one call outside the capture first",
                       bytes);
    if (sc.ptr) {
      // only work on this stream can still be using the old buffer
      KSMM_CUDA_OK(cudaStreamSynchronize(stream));
      KSMM_CUDA_OK(cudaFree(sc.ptr));
      sc.ptr = nullptr;
      sc.cap = 0;
    }
    KSMM_CUDA_OK(cudaMalloc(&sc.ptr, bytes));
    g_allocs.fetch_add(1, std::memory_order_relaxed);
    sc.cap = bytes;
  }
  *out = sc.ptr;
  return KSMM_OK;
}

// a batch-first factor with d > 1 whose batch-last twin has a fast kernel
static bool conversion_possible(const Problem& p) {
  if (p.bs_last || p.d == 1 || p.in_regrouped || p.out_regroup_d) return false;
  return p.batch <= 0x7fffffffLL;
}

// the heuristic: conversion pays when no direct kernel covers the factor and the batch-last
// kernel is a tensor-core (or TMA-staged FFMA) one
static bool conversion_applies(const Problem& p) {
  if (!conversion_possible(p)) return false;
  if (reinterpret_cast<uintptr_t>(p.w) % 16 != 0) return false;
  if (p.in_dtype == KSMM_F32) {
    Problem q = p;
    q.bs_last = 1;
    q.in = q.out = reinterpret_cast<void*>(256);  // alignment is that of the scratch (256 bytes)
    // for compute-heavy blocks the batch-last tensor-core kernel pays for the two transposes;
    // small blocks are bandwidth problems that the direct FFMA kernel (d = 2, 4) serves better
    // (tuned at 25088 rows: (1,256,64,4) 89 us through the conversion against 109 us direct)
    const bool direct = ffma_tma_first_supported(p, true);
    if (tc_default_config(q) >= 0 && (!direct || p.c >= 128 || p.b >= 128)) return true;
    if (direct) return false;
    return q.b >= 48 && ffma_tma_supported(q, false);
  }
  Problem q = p;
  q.bs_last = 1;
  q.in = q.out = reinterpret_cast<void*>(256);
  if (tc_default_config(p) >= 0) return false;  // a direct batch-first kernel covers it
  return q.b >= 32 && q.c >= 16 && tc_config_supported(q, 0, true);
}

static size_t conversion_scratch_bytes(const Problem& p) {
  const int es = dtype_size(p.in_dtype), os = dtype_size(p.out_dtype);
  const size_t n_in = static_cast<size_t>(p.a) * p.c * p.d, n_out = static_cast<size_t>(p.a) * p.b * p.d;
  return align_up(n_in * p.batch * es, 256) + align_up(n_out * p.batch * os, 256);
}

static int run_family(const Problem& p, int algo, int config, cudaStream_t stream);
static int dispatch(const Problem& p, int algo, int config, cudaStream_t stream);

static int forward_via_transpose(const Problem& p, cudaStream_t stream) {
  if (!conversion_possible(p))
    return set_error(KSMM_ERR_UNSUPPORTED, "the layout-conversion path serves batch-first factors with d > 1");
  const int es = dtype_size(p.in_dtype), os = dtype_size(p.out_dtype);
  const int64_t n_in = static_cast<int64_t>(p.a) * p.c * p.d, n_out = static_cast<int64_t>(p.a) * p.b * p.d;
  const size_t in_bytes = align_up(static_cast<size_t>(n_in) * p.batch * es, 256);
  void* base = nullptr;
  int stq = layout_scratch(p, conversion_scratch_bytes(p), stream, &base);
  if (stq != KSMM_OK) return stq;
  void* xt = base;
  void* yt = static_cast<char*>(base) + in_bytes;
  int st = launch_transpose(p.in, xt, p.batch, n_in, es, stream);  // (batch, in) -> (in, batch)
  if (st != KSMM_OK) return st;
  Problem q = p;
  q.in = xt;
  q.out = yt;
  q.bs_last = 1;
  q.scratch = nullptr;
  q.scratch_bytes = 0;
  st = dispatch(q, KSMM_ALGO_AUTO, -1, stream);  // (a batch-last factor never needs scratch)
  if (st != KSMM_OK) return st;
  return launch_transpose(yt, p.out, n_out, p.batch, os, stream);  // (out, batch) -> (batch, out)
}

static int run_family(const Problem& p, int algo, int config, cudaStream_t stream) {
  if (p.residual != nullptr && !(algo == KSMM_ALGO_TC && tc_fuses_residual(p))) {
    // this kernel has no residual input: add it in a pass over the output
    Problem q = p;
    q.residual = nullptr;
    int st = run_family(q, algo, config, stream);
    return st != KSMM_OK ? st : residual_pass(p, stream);
  }
  if (algo == KSMM_ALGO_SIMT) return simt_launch(p, config, stream);
  if (algo == KSMM_ALGO_TC) return tc_launch(p, config, stream);
  if (algo == KSMM_ALGO_CONVERT) return forward_via_transpose(p, stream);
  return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown kernel family %d", algo);
}

// can this (family, configuration) run the problem with the pointers it actually has?
static bool choice_runnable(const Problem& p, const Choice& ch) {
  if (ch.algo == KSMM_ALGO_TC) return tc_config_supported(p, ch.config, true);
  if (ch.algo == KSMM_ALGO_CONVERT) return conversion_possible(p);
  if (ch.algo != KSMM_ALGO_SIMT) return false;
  if (ch.config == kFfmaTmaWide || ch.config == kFfmaTmaNarrow) return ffma_tma_supported(p, true);
  if (ch.config == kFfmaTmaFirst) return ffma_tma_first_supported(p, true);
  return true;  // the register-staged kernels take any alignment
}

// What KSMM_ALGO_AUTO runs: a cached choice when it can run on these pointers (a choice tuned
// on aligned buffers does not bind an unaligned call), else the heuristic.
static Choice auto_choice(const Problem& p) {
  Choice ch;
  if (lookup_choice(p, &ch) && choice_runnable(p, ch)) return ch;
  const int tc_cfg = tc_default_config(p);
  if (tc_cfg >= 0) return Choice{KSMM_ALGO_TC, tc_cfg};
  if (conversion_applies(p)) return Choice{KSMM_ALGO_CONVERT, 0};
  return Choice{KSMM_ALGO_SIMT, -1};
}

// layout scratch the given (family, configuration) needs for this problem
static size_t scratch_need(const Problem& p, const Choice& ch) {
  if (ch.algo == KSMM_ALGO_CONVERT) return conversion_scratch_bytes(p);
  if (ch.algo == KSMM_ALGO_TC && !p.bs_last && p.d != 1 && ch.config == 1 && p.in_dtype != KSMM_F32)
    return tc_bsfirst_dp_scratch_bytes(p);
  return 0;
}

static int dispatch(const Problem& p, int algo, int config, cudaStream_t stream) {
  int st = check_problem(p);
  if (st != KSMM_OK) return st;
  if (p.batch == 0) return KSMM_OK;  // empty batch: nothing to write
  if (algo == KSMM_ALGO_AUTO) {
    const Choice ch = auto_choice(p);
    return run_family(p, ch.algo, ch.config, stream);
  }
  return run_family(p, algo, config, stream);
}

static Problem problem_of(const ksmm_forward_desc_t& dsc) {
  Problem p;
  p.in = dsc.input;
  p.w = dsc.values;
  p.out = dsc.output;
  p.bias = dsc.bias;
  p.batch = dsc.batch;
  p.a = dsc.a; p.b = dsc.b; p.c = dsc.c; p.d = dsc.d;
  p.in_dtype = dsc.in_dtype;
  p.out_dtype = dsc.out_dtype;
  p.bs_last = dsc.bs_last;
  p.alpha = dsc.alpha;
  p.activation = dsc.activation;
  p.scratch = dsc.scratch;
  p.scratch_bytes = dsc.scratch_bytes;
  p.residual = dsc.residual;
  return p;
}

// ---------------------------------------------------------------------------
// FFMA peak probe
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ffma_probe_kernel(float* sink, int iters, float seed) {
  float r[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) r[q] = seed + threadIdx.x * 1e-3f + q;
  const float m = 1.0000001f, add = 1e-7f;
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int q = 0; q < 16; ++q) r[q] = fmaf(r[q], m, add);
  }
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < 16; ++q) s += r[q];
  if (s == 123.456f) sink[0] = s;  // never true; keeps the loop alive
}

// ---------------------------------------------------------------------------
// device buffers owned by the host-memory entry point
// ---------------------------------------------------------------------------
struct HostPathState {
  std::mutex mu;
  int device = -1;
  cudaStream_t stream = nullptr;                   // chains
  cudaStream_t s_in = nullptr, s_out = nullptr;    // host->device and device->host copies
  // indexed by slice parity: input landed, chain done, output copied out
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_cmp[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  // indexed by call parity: weights landed, weights no longer read
  cudaEvent_t ev_w[2] = {nullptr, nullptr}, ev_wfree[2] = {nullptr, nullptr};
  static constexpr int kTickets = 64;
  cudaEvent_t ev_call[kTickets] = {};              // end of a call's last device->host copy
  uint64_t ticket_of[kTickets] = {};               // the call that last recorded the slot (0 = none)
  uint64_t slices = 0, calls = 0;                  // totals since the device was bound
  // input A, output A, weights A, workspace, input B, output B, weights B
  void* buf[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t cap[7] = {0, 0, 0, 0, 0, 0, 0};
};
static HostPathState g_host;

static int host_reserve(int which, size_t bytes) {
  if (bytes <= g_host.cap[which]) return KSMM_OK;
  if (g_host.buf[which]) {
    // (cudaFree waits for the device, so copies and kernels of earlier calls are done with it)
    KSMM_CUDA_OK(cudaFree(g_host.buf[which]));
    g_host.buf[which] = nullptr;
    g_host.cap[which] = 0;
  }
  size_t want = bytes + bytes / 8 + 256;
  KSMM_CUDA_OK(cudaMalloc(&g_host.buf[which], want));
  g_allocs.fetch_add(1, std::memory_order_relaxed);
  g_host.cap[which] = want;
  return KSMM_OK;
}


// ---------------------------------------------------------------------------
// Scratch for ksmm_cu_chain_forward_static: a fixed array inside the module
// image, so that the call never allocates.  In host code the name below is only
// a handle for cudaGetSymbolAddress; kernels must be given the resolved device
// address, never the symbol itself.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_chain_static_scratch[KSMM_CU_STATIC_SCRATCH_BYTES];

static std::mutex g_static_mu;
static void* g_static_scratch_ptr[64] = {nullptr};

// Device address of the scratch array on the current device (resolved once per device).
static int static_scratch_address(void** out) {
  int dev = 0;
  KSMM_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(KSMM_ERR_UNSUPPORTED, "device ordinal %d", dev);
  std::lock_guard<std::mutex> g(g_static_mu);
  if (!g_static_scratch_ptr[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_chain_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(KSMM_ERR_CUDA, "cannot resolve the static scratch array: %s",
                       cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return KSMM_OK;
}

}  // namespace ksmm

using namespace ksmm;

extern "C" {

int ksmm_cu_version(void) { return 100; }

const char* ksmm_cu_last_error(void) { return g_last_error; }

const char* ksmm_cu_status_string(int status) {
  switch (status) {
    case KSMM_OK: return "ok";
    case KSMM_ERR_BAD_ARGUMENT: return "bad argument";
    case KSMM_ERR_UNSUPPORTED: return "unsupported";
    case KSMM_ERR_CUDA: return "CUDA error";
    case KSMM_ERR_WORKSPACE: return "workspace missing or too small";
    case KSMM_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case KSMM_ERR_NO_DEVICE: return "no sm_100 device";
    default: return "unknown status";
  }
}

int ksmm_cu_check_device(void* stream) {
  return tc_check_device(static_cast<cudaStream_t>(stream));
}

uint64_t ksmm_cu_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

uint64_t ksmm_cu_alloc_count(void) { return g_allocs.load(std::memory_order_relaxed); }

int ksmm_cu_debug_wait_probe(int64_t limit_cycles, void* stream) {
  if (limit_cycles < 0 || limit_cycles > 4000000000ll)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "the probe's limit is 0 .. 4e9 cycles");
  return tc_wait_probe(limit_cycles, 99, static_cast<cudaStream_t>(stream));
}

size_t ksmm_cu_layout_scratch_bytes(const ksmm_forward_desc_t* desc) {
  if (!desc) return 0;
  Problem p = problem_of(*desc);
  if (check_problem(p) != KSMM_OK || p.batch == 0) return 0;
  if (desc->algo == KSMM_ALGO_AUTO) return scratch_need(p, auto_choice(p));
  return scratch_need(p, Choice{desc->algo, desc->config});
}

int ksmm_cu_release_scratch(void) {
  // every stream that used a buffer has to be idle before its memory goes away
  KSMM_CUDA_OK(cudaDeviceSynchronize());
  int dev = 0;
  KSMM_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> g(g_conv_mu);
  for (auto it = g_conv.begin(); it != g_conv.end();) {
    if (it->first.first == dev) {
      if (it->second.ptr) cudaFree(it->second.ptr);
      it = g_conv.erase(it);
    } else {
      ++it;
    }
  }
  return KSMM_OK;
}

int ksmm_cu_forward(const void* input, const void* values, void* output, int64_t batch, int a,
                    int b, int c, int d, int dtype, int bs_last, void* stream) {
  Problem p;
  p.in = input; p.w = values; p.out = output; p.bias = nullptr;
  p.batch = batch; p.a = a; p.b = b; p.c = c; p.d = d;
  p.in_dtype = dtype;
  p.out_dtype = dtype;
  p.bs_last = bs_last;
  p.alpha = 1.f;
  if (dtype == KSMM_F8E4M3)
    return set_error(KSMM_ERR_UNSUPPORTED,
                     "fp8 needs an explicit output type and scale: use ksmm_cu_forward_ex");
  return dispatch(p, KSMM_ALGO_AUTO, -1, static_cast<cudaStream_t>(stream));
}

int ksmm_cu_forward_ex(const ksmm_forward_desc_t* desc, void* stream) {
  if (!desc) return set_error(KSMM_ERR_BAD_ARGUMENT, "null descriptor");
  return dispatch(problem_of(*desc), desc->algo, desc->config, static_cast<cudaStream_t>(stream));
}

// bytes of the intermediate activations of a chain (two alternating buffers from three factors on)
static size_t chain_intermediate_bytes(int nfactors, const int32_t* patterns, int64_t batch, int dtype) {
  if (nfactors <= 1 || !patterns || batch <= 0) return 0;
  size_t mx = 0;
  for (int f = 0; f + 1 < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    size_t bytes = static_cast<size_t>(q[0]) * q[1] * q[3] * batch * dtype_size(dtype);
    if (bytes > mx) mx = bytes;
  }
  mx = align_up(mx, 256);
  return nfactors == 2 ? mx : 2 * mx;
}

size_t ksmm_cu_chain_workspace_bytes(int nfactors, const int32_t* patterns, int64_t batch,
                                     int dtype) {
  return chain_intermediate_bytes(nfactors, patterns, batch, dtype);
}

// ---------------------------------------------------------------------------
// Layout plan of a chain.  Batch-last factors are the fast form for every d; batch-first factors
// with d > 1 pay for the interleaved blocks (in-kernel split, or a layout conversion).  A 16-bit
// factor with d = 1 can read one layout and write the other at no extra cost, and a whole tensor
// can be transposed at the chain's ends.  The plan gives every factor its input and output layout
// so that the estimated time of the chain is smallest; the estimates are byte counts weighted by
// how far the kernel of that form runs from the memory roofline (measured on the benchmark
// patterns), which is all this choice needs.
// ---------------------------------------------------------------------------
struct ChainPlan {
  static constexpr int kMax = 16;
  bool pre_transpose = false, post_transpose = false;
  int in_last[kMax], out_last[kMax];
};

static bool can_switch_layout(const int32_t* q, int64_t batch, int dtype) {
  if (q[3] != 1 || q[1] < 32 || q[2] < 16) return false;
  if (dtype == KSMM_F32)  // the fp32 tensor kernel: 32-column atoms, c <= 1024
    return q[1] % 32 == 0 && q[2] % 4 == 0 && q[2] <= 1024 && batch % 32 == 0;
  return (dtype == KSMM_F16 || dtype == KSMM_BF16) && q[1] % 8 == 0 && q[2] % 8 == 0 && batch % 8 == 0;
}

static double step_cost(const int32_t* q, int64_t batch, int dtype, int in_last, int out_last) {
  const double bytes = static_cast<double>(dtype_size(dtype)) * q[0] * q[3] * (static_cast<double>(q[1]) + q[2]) * batch;
  if (dtype == KSMM_F32) {
    // The fp32 tensor kernel is compute-bound from blocks of about 64 x 64 on: its time is the larger
    // of the bytes and the flops at about 35 flop per byte of bandwidth.  A batch-first factor with
    // d > 1 pays a transpose on either side of it.
    const double flops = 2.0 * q[0] * q[3] * static_cast<double>(q[1]) * q[2] * batch;
    const double kernel = bytes > flops / 35.0 ? bytes : flops / 35.0;
    if (in_last != out_last) return can_switch_layout(q, batch, dtype) ? 1.05 * kernel : -1.0;
    if (in_last || q[3] == 1) return kernel;
    return kernel + 1.5 * bytes;
  }
  if (in_last != out_last) return can_switch_layout(q, batch, dtype) ? 1.05 * bytes : -1.0;
  if (in_last || q[3] == 1) return bytes;
  if ((q[3] == 2 || q[3] == 4) && q[1] % 8 == 0 && (static_cast<int64_t>(q[2]) * q[3]) % 8 == 0)
    return 1.9 * bytes;   // in-kernel split of the interleaved blocks
  if (q[3] % 8 == 0 && q[3] <= 16 && q[1] % 8 == 0 && q[1] >= 32 && q[1] <= 64 && q[2] >= 16)
    return 2.3 * bytes;   // groups of eight blocks, 16-byte pieces
  return 2.6 * bytes;     // layout conversion around the batch-last kernel
}

static void plan_chain(int nfactors, const int32_t* patterns, int64_t batch, int dtype, int in_last,
                       int out_last, bool allow_switch, ChainPlan* plan) {
  // default: every factor in the input's layout, a transpose at the end if the output differs
  for (int f = 0; f < nfactors && f < ChainPlan::kMax; ++f) plan->in_last[f] = plan->out_last[f] = in_last;
  plan->pre_transpose = false;
  plan->post_transpose = in_last != out_last;
  const bool planned = dtype == KSMM_F16 || dtype == KSMM_BF16 || dtype == KSMM_F32;
  if (!planned || !allow_switch || nfactors > 8 || batch <= 0) return;
  const double es = dtype_size(dtype);
  const int32_t* p0 = patterns;
  const int32_t* pl = patterns + 4 * (nfactors - 1);
  const double in_bytes = es * p0[0] * p0[2] * p0[3] * batch, out_bytes = es * pl[0] * pl[1] * pl[3] * batch;
  const double kTranspose = 0.75 * 2.0;  // read + write, at a higher fraction of the bandwidth than the kernels
  double best = -1.0;
  // mask bit f = layout of factor f's output; `pre` = transpose the chain input first
  for (int pre = 0; pre < 2; ++pre) {
    for (unsigned mask = 0; mask < (1u << nfactors); ++mask) {
      int state = pre ? !in_last : in_last;
      double cost = pre ? kTranspose * in_bytes : 0.0;
      bool ok = true;
      for (int f = 0; f < nfactors && ok; ++f) {
        const int o = (mask >> f) & 1;
        const double c = step_cost(patterns + 4 * f, batch, dtype, state, o);
        if (c < 0) ok = false;
        cost += c;
        state = o;
      }
      if (!ok) continue;
      if (state != out_last) cost += kTranspose * out_bytes;
      if (best < 0 || cost < best * 0.999) {   // ties keep the earlier (fewer transposes, layout of the input) plan
        best = cost;
        int st2 = pre ? !in_last : in_last;
        for (int f = 0; f < nfactors; ++f) {
          plan->in_last[f] = st2;
          plan->out_last[f] = (mask >> f) & 1;
          st2 = plan->out_last[f];
        }
        plan->pre_transpose = pre != 0;
        plan->post_transpose = st2 != out_last;
      }
    }
  }
}

static int chain_walk(bool run, const void* input, const void* const* values, void* output,
                      const void* bias, void* workspace, size_t inter_bytes, void* scratch,
                      size_t scratch_bytes, int no_alloc, int64_t batch, int nfactors,
                      const int32_t* patterns, int dtype, int bs_last, int out_bs_last, int activation,
                      cudaStream_t stream, size_t* scratch_max, int allow_switch,
                      const void* residual = nullptr);

// One pass over a chain: either plans it (run == false: returns through *scratch_max the layout
// scratch it needs under the current dispatch: transposed copies at the chain's ends plus the
// largest scratch of any factor) or runs it.
static int chain_walk(bool run, const void* input, const void* const* values, void* output,
                      const void* bias, void* workspace, size_t inter_bytes, void* scratch,
                      size_t scratch_bytes, int no_alloc, int64_t batch, int nfactors,
                      const int32_t* patterns, int dtype, int bs_last, int out_bs_last, int activation,
                      cudaStream_t stream, size_t* scratch_max, int allow_switch, const void* residual) {
  if (nfactors > ChainPlan::kMax)
    return set_error(KSMM_ERR_UNSUPPORTED, "chains of more than %d factors", ChainPlan::kMax);
  ChainPlan plan;
  plan_chain(nfactors, patterns, batch, dtype, bs_last, out_bs_last, allow_switch != 0, &plan);
  const size_t es = dtype_size(dtype);
  const int32_t* p0 = patterns;
  const int32_t* pl = patterns + 4 * (nfactors - 1);
  const int64_t in_feats = static_cast<int64_t>(p0[0]) * p0[2] * p0[3];
  const int64_t out_feats = static_cast<int64_t>(pl[0]) * pl[1] * pl[3];
  const size_t pre_bytes = plan.pre_transpose ? align_up(static_cast<size_t>(in_feats) * batch * es, 256) : 0;
  const size_t post_bytes = plan.post_transpose ? align_up(static_cast<size_t>(out_feats) * batch * es, 256) : 0;
  const size_t half = nfactors == 2 ? inter_bytes : inter_bytes / 2;
  const void* cur = input;
  bool cur_regrouped = false;  // the intermediate in `cur` is regrouped by the blocks of factor f
  char* ws = static_cast<char*>(workspace);
  // planning needs plausible (aligned) addresses only
  if (!run) {
    ws = reinterpret_cast<char*>(static_cast<uintptr_t>(1) << 20);
    cur = output = ws;
  }
  // One region holds everything the chain needs beside its intermediates: the transposed copies
  // at the chain's ends first, the factors' layout scratch after them.  It is the caller's
  // scratch when that is large enough, else the library-owned buffer of this stream, taken once
  // for the whole chain (a second request could move it under the first).
  char* t_pre = nullptr;
  char* t_post = nullptr;
  void* f_scratch = nullptr;
  size_t f_scratch_bytes = 0;
  int f_no_alloc = no_alloc;
  if (run && batch > 0) {
    size_t total = 0;
    int stp = chain_walk(false, nullptr, nullptr, nullptr, nullptr, nullptr, inter_bytes, nullptr, 0, 0, batch,
                         nfactors, patterns, dtype, bs_last, out_bs_last, activation, nullptr, &total,
                         allow_switch);
    if (stp != KSMM_OK) return stp;
    if (total > 0) {
      Problem sp;
      sp.scratch = scratch; sp.scratch_bytes = scratch_bytes; sp.no_alloc = no_alloc;
      void* base = nullptr;
      stp = layout_scratch(sp, total, stream, &base);
      if (stp != KSMM_OK) return stp;
      t_pre = static_cast<char*>(base);
      t_post = t_pre + pre_bytes;
      f_scratch = t_post + post_bytes;
      f_scratch_bytes = total - pre_bytes - post_bytes;
      f_no_alloc = 1;  // what the factors need is inside the region by construction
    }
  }
  if (plan.pre_transpose && run && batch > 0) {
    // (batch, features) -> (features, batch) or back
    int st = bs_last ? launch_transpose(input, t_pre, in_feats, batch, static_cast<int>(es), stream)
                     : launch_transpose(input, t_pre, batch, in_feats, static_cast<int>(es), stream);
    if (st != KSMM_OK) return st;
    cur = t_pre;
  }
  size_t factor_scratch_max = 0;
  for (int f = 0; f < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    const bool last = (f + 1 == nfactors);
    void* dst = last ? (plan.post_transpose && run ? static_cast<void*>(t_post) : output) : ws + (f & 1) * half;
    Problem p;
    p.in = cur; p.w = run ? values[f] : ws; p.out = dst; p.bias = last ? bias : nullptr;
    p.batch = batch; p.a = q[0]; p.b = q[1]; p.c = q[2]; p.d = q[3];
    p.in_dtype = dtype; p.out_dtype = dtype; p.alpha = 1.f;
    p.bs_last = plan.in_last[f];
    p.out_bs_last = plan.out_last[f] == plan.in_last[f] ? -1 : plan.out_last[f];
    p.activation = last ? activation : 0;
    // the residual has the chain output's layout: it can join the last factor's epilogue only when
    // that factor writes the final layout itself
    p.residual = (last && !plan.post_transpose) ? residual : nullptr;
    p.scratch = f_scratch; p.scratch_bytes = f_scratch_bytes; p.no_alloc = f_no_alloc;
    const bool same_first = !plan.in_last[f] && !plan.out_last[f];
    // Layout fusion of consecutive batch-first factors: when the next factor has d = 2 or 4 and
    // this one can store its output regrouped by the next factor's blocks, the intermediate is
    // written in that order and the next factor runs the kernel without the transposer stage
    // (and without a regrouping pass).
    bool next_regrouped = false;
    if (!last && same_first && !plan.in_last[f + 1] && !plan.out_last[f + 1]) {
      const int32_t* r = patterns + 4 * (f + 1);
      Problem nx = p;
      // the next factor reads this factor's destination and writes its own one
      nx.in = dst;
      nx.out = (f + 2 == nfactors) ? output : ws + ((f + 1) & 1) * half;
      nx.w = run ? values[f + 1] : ws; nx.bias = nullptr;
      nx.a = r[0]; nx.b = r[1]; nx.c = r[2]; nx.d = r[3];
      p.out_regroup_c = r[2];
      p.out_regroup_d = r[3];
      Choice ch;
      const bool pinned = lookup_choice(p, &ch) || lookup_choice(nx, &ch);  // a tuned choice wins
      if (!pinned && !cur_regrouped && (r[3] == 2 || r[3] == 4) && tc_can_regroup_output(p) &&
          tc_config_supported(nx, 1, true) && tc_default_config(nx) >= 0) {
        next_regrouped = true;
      } else {
        p.out_regroup_c = p.out_regroup_d = 0;
      }
    }
    int st = KSMM_OK;
    if (p.out_bs_last >= 0) {
      // a factor that changes the layout: the 16-bit tensor kernel only (the plan checked its shape
      // rules; pointers are the caller's)
      if (run) st = run_family(p, KSMM_ALGO_TC, -1, stream);
    } else if (cur_regrouped) {
      p.in_regrouped = 1;
      if (run) st = run_family(p, KSMM_ALGO_TC, 1, stream);
    } else if (next_regrouped) {
      if (run) st = run_family(p, KSMM_ALGO_TC, -1, stream);
    } else if (run) {
      st = dispatch(p, KSMM_ALGO_AUTO, -1, stream);
    } else {
      st = check_problem(p);
      if (st == KSMM_OK && batch > 0) {
        const size_t need = scratch_need(p, auto_choice(p));
        if (need > factor_scratch_max) factor_scratch_max = need;
      }
    }
    if (st != KSMM_OK) return st;
    cur = dst;
    cur_regrouped = next_regrouped;
  }
  if (plan.post_transpose && run && batch > 0) {
    // the last factor wrote the other layout into t_post
    const int last_layout = plan.out_last[nfactors - 1];
    int st = last_layout ? launch_transpose(t_post, output, out_feats, batch, static_cast<int>(es), stream)
                         : launch_transpose(t_post, output, batch, out_feats, static_cast<int>(es), stream);
    if (st != KSMM_OK) return st;
    if (residual != nullptr) {
      Problem rp;
      rp.out = output; rp.residual = residual; rp.out_dtype = dtype;
      rp.a = pl[0]; rp.b = pl[1]; rp.d = pl[3]; rp.batch = batch;
      st = residual_pass(rp, stream);
      if (st != KSMM_OK) return st;
    }
  }
  if (scratch_max) *scratch_max = pre_bytes + post_bytes + factor_scratch_max;
  return KSMM_OK;
}

static int check_chain(int nfactors, const int32_t* patterns, const void* const* values, int dtype,
                       int activation) {
  if (activation < 0 || activation > 2)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown activation %d", activation);
  if (nfactors <= 0 || !patterns || !values)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "chain needs at least one factor");
  if (dtype == KSMM_F8E4M3)
    return set_error(KSMM_ERR_UNSUPPORTED, "chains run in fp32, fp16 or bf16");
  if (dtype < KSMM_F32 || dtype > KSMM_F8E4M3)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown dtype %d", dtype);
  for (int f = 0; f < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    if (q[0] <= 0 || q[1] <= 0 || q[2] <= 0 || q[3] <= 0)
      return set_error(KSMM_ERR_BAD_ARGUMENT, "pattern %d (%d,%d,%d,%d) must be positive", f, q[0], q[1],
                       q[2], q[3]);
  }
  for (int f = 0; f + 1 < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    const int32_t* r = patterns + 4 * (f + 1);
    if (static_cast<int64_t>(q[0]) * q[1] * q[3] != static_cast<int64_t>(r[0]) * r[2] * r[3])
      return set_error(KSMM_ERR_BAD_ARGUMENT,
                       "factor %d produces %lld features but factor %d expects %lld", f,
                       static_cast<long long>(q[0]) * q[1] * q[3], f + 1,
                       static_cast<long long>(r[0]) * r[2] * r[3]);
  }
  return KSMM_OK;
}

size_t ksmm_cu_chain_workspace_bytes_ex(int nfactors, const int32_t* patterns, int64_t batch,
                                        int dtype, int bs_last) {
  return ksmm_cu_chain_workspace_bytes_layouts(nfactors, patterns, batch, dtype, bs_last, bs_last);
}

size_t ksmm_cu_chain_workspace_bytes_layouts(int nfactors, const int32_t* patterns, int64_t batch,
                                             int dtype, int bs_last, int out_bs_last) {
  if (nfactors <= 0 || !patterns || batch <= 0) return 0;
  const void* dummy = nullptr;
  if (check_chain(nfactors, patterns, &dummy, dtype, 0) != KSMM_OK) return 0;
  const size_t inter = chain_intermediate_bytes(nfactors, patterns, batch, dtype);
  // the larger of the two plans: with layout-changing factors (every pointer 16-byte aligned) and
  // without them, so that the size holds whatever the pointers of the call turn out to be
  size_t scratch = 0;
  for (int allow = 0; allow < 2; ++allow) {
    size_t need = 0;
    if (chain_walk(false, nullptr, nullptr, nullptr, nullptr, nullptr, inter, nullptr, 0, 0, batch, nfactors,
                   patterns, dtype, bs_last ? 1 : 0, out_bs_last ? 1 : 0, 0, nullptr, &need, allow) != KSMM_OK)
      return 0;
    if (need > scratch) scratch = need;
  }
  return inter + scratch;
}

int ksmm_cu_chain_forward(const void* input, const void* const* values, void* output,
                          const void* bias, void* workspace, size_t workspace_bytes,
                          int64_t batch, int nfactors, const int32_t* patterns, int dtype,
                          int bs_last, void* stream) {
  return ksmm_cu_chain_forward_act(input, values, output, bias, workspace, workspace_bytes, batch,
                                   nfactors, patterns, dtype, bs_last, KSMM_ACT_NONE, stream);
}

// Shared body of the chain entry points.  The workspace holds the intermediates first; whatever
// follows them is handed to the factors as layout scratch.
static int chain_forward_impl(const void* input, const void* const* values, void* output,
                              const void* bias, void* workspace, size_t workspace_bytes, int no_alloc,
                              int64_t batch, int nfactors, const int32_t* patterns, int dtype,
                              int bs_last, int out_bs_last, int activation, cudaStream_t stream,
                              const void* residual = nullptr) {
  int st = check_chain(nfactors, patterns, values, dtype, activation);
  if (st != KSMM_OK) return st;
  if (bs_last != 0 && bs_last != 1) return set_error(KSMM_ERR_BAD_ARGUMENT, "bs_last must be 0 or 1");
  if (out_bs_last != 0 && out_bs_last != 1)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "the output layout must be 0 (batch-first) or 1 (batch-last)");
  if (batch < 0) return set_error(KSMM_ERR_BAD_ARGUMENT, "negative batch");
  const size_t inter = chain_intermediate_bytes(nfactors, patterns, batch, dtype);
  if (inter > 0 && (!workspace || workspace_bytes < inter))
    return set_error(KSMM_ERR_WORKSPACE, "chain workspace: need %zu bytes, got %zu", inter,
                     workspace_bytes);
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  if (workspace && workspace_bytes > inter) {
    scratch = static_cast<char*>(workspace) + inter;
    scratch_bytes = workspace_bytes - inter;
  }
  // layout-changing factors go through TMA on both sides: every buffer has to be 16-byte aligned
  auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  int allow_switch = al16(input) && al16(output) && al16(workspace) && al16(residual) ? 1 : 0;
  for (int f = 0; f < nfactors; ++f) allow_switch &= al16(values[f]) ? 1 : 0;
  if (no_alloc) {
    // refuse before the first launch, not half-way through the chain
    size_t need = 0;
    st = chain_walk(false, nullptr, nullptr, nullptr, nullptr, nullptr, inter, nullptr, 0, 0, batch,
                    nfactors, patterns, dtype, bs_last, out_bs_last, activation, nullptr, &need, allow_switch);
    if (st != KSMM_OK) return st;
    if (need > scratch_bytes)
      return set_error(KSMM_ERR_WORKSPACE,
                       "the chain needs %zu bytes of intermediates and %zu bytes of layout scratch; "
                       "%zu bytes are available and this call may not allocate",
                       inter, need, workspace_bytes);
  }
  return chain_walk(true, input, values, output, bias, workspace, inter, scratch, scratch_bytes, no_alloc,
                    batch, nfactors, patterns, dtype, bs_last, out_bs_last, activation, stream, nullptr,
                    allow_switch, residual);
}

int ksmm_cu_chain_forward_act(const void* input, const void* const* values, void* output,
                              const void* bias, void* workspace, size_t workspace_bytes,
                              int64_t batch, int nfactors, const int32_t* patterns, int dtype,
                              int bs_last, int activation, void* stream) {
  return chain_forward_impl(input, values, output, bias, workspace, workspace_bytes, /*no_alloc=*/0, batch,
                            nfactors, patterns, dtype, bs_last, bs_last, activation,
                            static_cast<cudaStream_t>(stream));
}

int ksmm_cu_chain_forward_desc(const ksmm_chain_desc_t* dsc, void* stream) {
  if (!dsc) return set_error(KSMM_ERR_BAD_ARGUMENT, "null descriptor");
  const int out_last = dsc->out_layout == 0 ? dsc->bs_last : (dsc->out_layout == 2 ? 1 : 0);
  if (dsc->out_layout < 0 || dsc->out_layout > 2)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "out_layout is 0 (as the input), 1 (batch-first) or 2 (batch-last)");
  return chain_forward_impl(dsc->input, dsc->values, dsc->output, dsc->bias, dsc->workspace,
                            dsc->workspace_bytes, /*no_alloc=*/0, dsc->batch, dsc->nfactors, dsc->patterns,
                            dsc->dtype, dsc->bs_last, out_last, dsc->activation,
                            static_cast<cudaStream_t>(stream), dsc->residual);
}

int ksmm_cu_chain_forward_layouts(const void* input, const void* const* values, void* output,
                                  const void* bias, void* workspace, size_t workspace_bytes,
                                  int64_t batch, int nfactors, const int32_t* patterns, int dtype,
                                  int bs_last, int out_bs_last, int activation, void* stream) {
  return chain_forward_impl(input, values, output, bias, workspace, workspace_bytes, /*no_alloc=*/0, batch,
                            nfactors, patterns, dtype, bs_last, out_bs_last, activation,
                            static_cast<cudaStream_t>(stream));
}

// One factor for `groups` stacked problems: one grouped launch where a kernel has that form,
// else one dispatch per group.
static int grouped_factor(Problem p, int groups, int shared_input, cudaStream_t stream) {
  const size_t es = dtype_size(p.in_dtype), os = dtype_size(p.out_dtype);
  const size_t in_elems = static_cast<size_t>(p.a) * p.c * p.d * p.batch;
  const size_t out_elems = static_cast<size_t>(p.a) * p.b * p.d * p.batch;
  const size_t w_elems = static_cast<size_t>(p.a) * p.b * p.c * p.d;
  int st = check_problem(p);
  if (st != KSMM_OK) return st;
  if (p.batch == 0) return KSMM_OK;
  if (groups > 1) {
    Problem g = p;
    g.groups = groups;
    g.group_shared_input = shared_input;
    Choice ch;
    const bool pinned = lookup_choice(p, &ch);  // a tuned choice for the single problem wins
    const int cfg = tc_default_config(g);
    if (!pinned && cfg >= 0) return tc_launch(g, cfg, stream);
  }
  for (int q = 0; q < groups; ++q) {
    Problem g = p;
    g.in = static_cast<const char*>(p.in) + (shared_input ? 0 : q * in_elems * es);
    g.w = static_cast<const char*>(p.w) + q * w_elems * es;
    g.out = static_cast<char*>(p.out) + q * out_elems * os;
    g.bias = p.bias ? static_cast<const char*>(p.bias) + q * static_cast<size_t>(p.a) * p.b * p.d * os : nullptr;
    st = dispatch(g, KSMM_ALGO_AUTO, -1, stream);
    if (st != KSMM_OK) return st;
  }
  return KSMM_OK;
}

int ksmm_cu_grouped_forward(const void* input, const void* values, void* output, const void* bias,
                            int64_t batch, int a, int b, int c, int d, int dtype, int bs_last,
                            int groups, int shared_input, void* stream) {
  if (groups < 1) return set_error(KSMM_ERR_BAD_ARGUMENT, "groups must be at least 1");
  if (dtype == KSMM_F8E4M3)
    return set_error(KSMM_ERR_UNSUPPORTED, "grouped calls run in fp32, fp16 or bf16");
  Problem p;
  p.in = input; p.w = values; p.out = output; p.bias = bias;
  p.batch = batch; p.a = a; p.b = b; p.c = c; p.d = d;
  p.in_dtype = dtype; p.out_dtype = dtype; p.bs_last = bs_last; p.alpha = 1.f;
  return grouped_factor(p, groups, shared_input ? 1 : 0, static_cast<cudaStream_t>(stream));
}

int ksmm_cu_grouped_chain_forward(const void* input, const void* const* values, void* output,
                                  const void* bias, void* workspace, size_t workspace_bytes,
                                  int64_t batch, int nfactors, const int32_t* patterns, int dtype,
                                  int bs_last, int groups, void* stream) {
  if (groups < 1) return set_error(KSMM_ERR_BAD_ARGUMENT, "groups must be at least 1");
  int st = check_chain(nfactors, patterns, values, dtype, 0);
  if (st != KSMM_OK) return st;
  if (bs_last != 0 && bs_last != 1) return set_error(KSMM_ERR_BAD_ARGUMENT, "bs_last must be 0 or 1");
  if (batch < 0) return set_error(KSMM_ERR_BAD_ARGUMENT, "negative batch");
  // per group: the intermediates of one chain; whatever follows the groups' intermediates is
  // layout scratch for the factors that run group by group
  const size_t inter1 = chain_intermediate_bytes(nfactors, patterns, batch, dtype);
  const size_t inter = inter1 * groups;
  if (inter > 0 && (!workspace || workspace_bytes < inter))
    return set_error(KSMM_ERR_WORKSPACE, "grouped chain workspace: need %zu bytes, got %zu", inter,
                     workspace_bytes);
  const size_t half1 = nfactors == 2 ? inter1 : inter1 / 2;  // one buffer of one group
  char* ws = static_cast<char*>(workspace);
  const void* cur = input;
  for (int f = 0; f < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    const bool last = (f + 1 == nfactors);
    // the groups' copies of intermediate buffer (f & 1) are contiguous: a stacked tensor
    void* dst = last ? output : ws + static_cast<size_t>(f & 1) * half1 * groups;
    Problem p;
    p.in = cur; p.w = values[f]; p.out = dst; p.bias = last ? bias : nullptr;
    p.batch = batch; p.a = q[0]; p.b = q[1]; p.c = q[2]; p.d = q[3];
    p.in_dtype = dtype; p.out_dtype = dtype; p.bs_last = bs_last; p.alpha = 1.f;
    if (workspace && workspace_bytes > inter) {
      p.scratch = ws + inter;
      p.scratch_bytes = workspace_bytes - inter;
    }
    st = grouped_factor(p, groups, f == 0 ? 1 : 0, static_cast<cudaStream_t>(stream));
    if (st != KSMM_OK) return st;
    cur = dst;
  }
  return KSMM_OK;
}

// ---- backward of one factor -------------------------------------------------------------------
static Problem backward_problem(const void* in, const void* w, void* out, int64_t batch, int a, int b, int c,
                                int d, int dtype, int bs_last) {
  Problem p;
  p.in = in; p.w = w; p.out = out; p.bias = nullptr;
  p.batch = batch; p.a = a; p.b = b; p.c = c; p.d = d;
  p.in_dtype = dtype; p.out_dtype = dtype; p.bs_last = bs_last; p.alpha = 1.f;
  return p;
}

static int check_backward(const Problem& p) {
  if (p.in_dtype == KSMM_F8E4M3)
    return set_error(KSMM_ERR_UNSUPPORTED, "the backward passes run in fp32, fp16 or bf16");
  return check_problem(p);
}

size_t ksmm_cu_backward_input_workspace_bytes(int64_t batch, int a, int b, int c, int d, int dtype,
                                              int bs_last) {
  if (batch <= 0 || a <= 0 || b <= 0 || c <= 0 || d <= 0) return 0;
  // the transposed blocks, then the layout scratch of the (a, c, b, d) multiplication, if any
  const size_t wt = align_up(static_cast<size_t>(a) * b * c * d * dtype_size(dtype), 256);
  Problem q = backward_problem(reinterpret_cast<void*>(256), reinterpret_cast<void*>(256),
                               reinterpret_cast<void*>(256), batch, a, c, b, d, dtype, bs_last);
  if (check_backward(q) != KSMM_OK) return 0;
  return wt + scratch_need(q, auto_choice(q));
}

int ksmm_cu_backward_input(const void* grad_output, const void* values, void* grad_input, void* workspace,
                           size_t workspace_bytes, int64_t batch, int a, int b, int c, int d, int dtype,
                           int bs_last, void* stream) {
  // dX = K^T dY: pattern (a, c, b, d) with every block transposed
  Problem q = backward_problem(grad_output, nullptr, grad_input, batch, a, c, b, d, dtype, bs_last);
  q.w = workspace;
  int st = check_backward(q);
  if (st != KSMM_OK) return st;
  if (!values) return set_error(KSMM_ERR_BAD_ARGUMENT, "null weights");
  if (batch == 0) return KSMM_OK;
  const size_t wt = align_up(static_cast<size_t>(a) * b * c * d * dtype_size(dtype), 256);
  if (!workspace || workspace_bytes < wt)
    return set_error(KSMM_ERR_WORKSPACE, "backward workspace: need at least %zu bytes, got %zu", wt,
                     workspace_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  st = launch_transpose_blocks(values, workspace, static_cast<int64_t>(a) * d, c, b, dtype_size(dtype), s);
  if (st != KSMM_OK) return st;
  if (workspace_bytes > wt) {
    q.scratch = static_cast<char*>(workspace) + wt;
    q.scratch_bytes = workspace_bytes - wt;
  }
  return dispatch(q, KSMM_ALGO_AUTO, -1, s);
}

size_t ksmm_cu_backward_weights_workspace_bytes(int64_t batch, int a, int b, int c, int d, int dtype,
                                                int bs_last) {
  if (batch <= 0 || a <= 0 || b <= 0 || c <= 0 || d <= 0) return 0;
  Problem p = backward_problem(nullptr, nullptr, nullptr, batch, a, b, c, d, dtype, bs_last);
  return wgrad_workspace_bytes(p);
}

int ksmm_cu_backward_weights(const void* input, const void* grad_output, void* grad_values, void* workspace,
                             size_t workspace_bytes, int64_t batch, int a, int b, int c, int d, int dtype,
                             int bs_last, void* stream) {
  Problem p = backward_problem(input, grad_output, grad_values, batch, a, b, c, d, dtype, bs_last);
  int st = check_backward(p);
  if (st != KSMM_OK) return st;
  return wgrad_launch(p, grad_output, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int ksmm_cu_chain_forward_static(const void* input, const void* const* values, void* output,
                                 const void* bias, int64_t batch, int nfactors,
                                 const int32_t* patterns, int dtype, int bs_last, void* stream) {
  int st = check_chain(nfactors, patterns, values, dtype, 0);
  if (st != KSMM_OK) return st;
  // intermediates and, for batch-first factors that run through a layout conversion, their
  // transposed copies: all of it has to fit into the array
  const size_t need = ksmm_cu_chain_workspace_bytes_ex(nfactors, patterns, batch, dtype, bs_last);
  if (need > static_cast<size_t>(KSMM_CU_STATIC_SCRATCH_BYTES))
    return set_error(KSMM_ERR_WORKSPACE,
                     "the chain needs %zu bytes of scratch but the built-in scratch holds %zu: use "
                     "ksmm_cu_chain_forward with a caller-provided workspace",
                     need, static_cast<size_t>(KSMM_CU_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  if (need > 0) {
    st = static_scratch_address(&scratch);
    if (st != KSMM_OK) return st;
  }
  // every intermediate is fully overwritten by the factor that produces it, so
  // nothing in the scratch has to start at zero
  return chain_forward_impl(input, values, output, bias, scratch,
                            need > 0 ? static_cast<size_t>(KSMM_CU_STATIC_SCRATCH_BYTES) : 0,
                            /*no_alloc=*/1, batch, nfactors, patterns, dtype, bs_last, bs_last, KSMM_ACT_NONE,
                            static_cast<cudaStream_t>(stream));
}

// Enqueues one host-memory chain call on the library's three streams and returns its ticket.
// Caller holds g_host.mu.
static int host_submit(const void* host_input, const void* const* host_values, void* host_output,
                       const void* host_bias, int64_t batch, int nfactors, const int32_t* patterns,
                       int dtype, int bs_last, int device, uint64_t* ticket, bool whole_batch) {
  KSMM_CUDA_OK(cudaSetDevice(device));
  if (g_host.device != device) {
    // buffers, streams and events belong to one device at a time; moving devices drops them
    if (g_host.device >= 0) {
      cudaSetDevice(g_host.device);
      cudaDeviceSynchronize();
      for (int q = 0; q < 7; ++q) {
        if (g_host.buf[q]) cudaFree(g_host.buf[q]);
        g_host.buf[q] = nullptr;
        g_host.cap[q] = 0;
      }
      KSMM_CUDA_OK(cudaSetDevice(device));
    }
    for (cudaStream_t* sp : {&g_host.stream, &g_host.s_in, &g_host.s_out}) {
      if (*sp) cudaStreamDestroy(*sp);
      *sp = nullptr;
      KSMM_CUDA_OK(cudaStreamCreateWithFlags(sp, cudaStreamNonBlocking));
    }
    auto renew = [](cudaEvent_t* ep) -> cudaError_t {
      if (*ep) cudaEventDestroy(*ep);
      *ep = nullptr;
      return cudaEventCreateWithFlags(ep, cudaEventDisableTiming);
    };
    for (int q = 0; q < 2; ++q) {
      KSMM_CUDA_OK(renew(&g_host.ev_in[q]));
      KSMM_CUDA_OK(renew(&g_host.ev_cmp[q]));
      KSMM_CUDA_OK(renew(&g_host.ev_out[q]));
      KSMM_CUDA_OK(renew(&g_host.ev_w[q]));
      KSMM_CUDA_OK(renew(&g_host.ev_wfree[q]));
    }
    for (int q = 0; q < HostPathState::kTickets; ++q) {
      KSMM_CUDA_OK(renew(&g_host.ev_call[q]));
      g_host.ticket_of[q] = 0;
    }
    g_host.slices = 0;
    g_host.calls = 0;
    g_host.device = device;
  }
  const size_t es = dtype_size(dtype);
  const int32_t* p0 = patterns;
  const int32_t* pl = patterns + 4 * (nfactors - 1);
  const size_t in_feats = static_cast<size_t>(p0[0]) * p0[2] * p0[3];
  const size_t out_feats = static_cast<size_t>(pl[0]) * pl[1] * pl[3];
  std::vector<size_t> woff(nfactors + 1, 0);
  for (int f = 0; f < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    woff[f + 1] = woff[f] + align_up(static_cast<size_t>(q[0]) * q[1] * q[2] * q[3] * es, 256);
  }
  const size_t bias_off = woff[nfactors];
  const size_t w_bytes = bias_off + (host_bias ? align_up(out_feats * es, 256) : 0);

  // The batch is cut into slices of `slice` entries that move through a three-stage pipeline
  // (host->device copy, chain, device->host copy) on three streams with two buffers per
  // direction, so that both directions of the link are busy at the same time.  The slice
  // counter runs on across calls: the first copy of one call overlaps the last copies of the
  // call before it.  A synchronous call has only its own slices to overlap, so it cuts the batch
  // in eight; an asynchronous call overlaps with its neighbours and moves its batch in one piece
  // (fewer, larger copies: 6.3 against 5.4 TFLOP/s on the benchmark sweep), up to 1 GiB per buffer.
  int64_t slice = batch;
  static const int forced = [] {
    const char* e = std::getenv("KSMM_HOST_SLICES");  // tuning aid: slices per call for large batches
    return e ? std::atoi(e) : 0;
  }();
  if (forced > 0 && batch >= 8192) {
    slice = ((batch + forced - 1) / forced + 255) / 256 * 256;
  } else if (whole_batch) {
    const size_t per_entry = std::max(in_feats, out_feats) * es;
    const int64_t cap = std::max<int64_t>(256, static_cast<int64_t>((size_t(1) << 30) / per_entry) / 256 * 256);
    if (batch > cap) slice = cap;
  } else if (batch >= 16384) {
    slice = ((batch + 7) / 8 + 255) / 256 * 256;
  } else if (batch >= 8192) {
    slice = ((batch + 3) / 4 + 255) / 256 * 256;
  }
  const int nslices = static_cast<int>((batch + slice - 1) / slice);
  const size_t ws_bytes = ksmm_cu_chain_workspace_bytes_ex(nfactors, patterns, slice, dtype, bs_last);
  const int cp = static_cast<int>(g_host.calls & 1);   // which weight buffer this call uses
  const int wslot = cp ? 6 : 2;
  int st;
  if ((st = host_reserve(0, in_feats * slice * es)) != KSMM_OK) return st;
  if ((st = host_reserve(1, out_feats * slice * es)) != KSMM_OK) return st;
  if ((st = host_reserve(wslot, w_bytes)) != KSMM_OK) return st;
  if ((st = host_reserve(3, ws_bytes)) != KSMM_OK) return st;
  if ((st = host_reserve(4, in_feats * slice * es)) != KSMM_OK) return st;
  if ((st = host_reserve(5, out_feats * slice * es)) != KSMM_OK) return st;
  cudaStream_t sc = g_host.stream, si = g_host.s_in, so = g_host.s_out;
  // weights: wait until the call two back no longer reads this buffer
  if (g_host.calls >= 2) KSMM_CUDA_OK(cudaStreamWaitEvent(si, g_host.ev_wfree[cp], 0));
  std::vector<const void*> dvals(nfactors);
  for (int f = 0; f < nfactors; ++f) {
    const int32_t* q = patterns + 4 * f;
    char* dst = static_cast<char*>(g_host.buf[wslot]) + woff[f];
    KSMM_CUDA_OK(cudaMemcpyAsync(dst, host_values[f],
                                 static_cast<size_t>(q[0]) * q[1] * q[2] * q[3] * es,
                                 cudaMemcpyHostToDevice, si));
    dvals[f] = dst;
  }
  const void* dbias = nullptr;
  if (host_bias) {
    char* dst = static_cast<char*>(g_host.buf[wslot]) + bias_off;
    KSMM_CUDA_OK(cudaMemcpyAsync(dst, host_bias, out_feats * es, cudaMemcpyHostToDevice, si));
    dbias = dst;
  }
  KSMM_CUDA_OK(cudaEventRecord(g_host.ev_w[cp], si));
  KSMM_CUDA_OK(cudaStreamWaitEvent(sc, g_host.ev_w[cp], 0));
  const char* hin = static_cast<const char*>(host_input);
  char* hout = static_cast<char*>(host_output);
  for (int k = 0; k < nslices; ++k) {
    const int64_t n0 = static_cast<int64_t>(k) * slice;
    const int64_t cn = std::min<int64_t>(slice, batch - n0);
    const uint64_t gs = g_host.slices;
    const int sl = static_cast<int>(gs & 1);
    void* din = g_host.buf[sl ? 4 : 0];
    void* dout = g_host.buf[sl ? 5 : 1];
    // host -> device, once the chain of the slice two back has read this input buffer
    if (gs >= 2) KSMM_CUDA_OK(cudaStreamWaitEvent(si, g_host.ev_cmp[sl], 0));
    if (bs_last) {
      // (features, batch) row-major: a slice is a column block
      KSMM_CUDA_OK(cudaMemcpy2DAsync(din, cn * es, hin + n0 * es, batch * es, cn * es, in_feats,
                                     cudaMemcpyHostToDevice, si));
    } else {
      KSMM_CUDA_OK(cudaMemcpyAsync(din, hin + n0 * in_feats * es, cn * in_feats * es,
                                   cudaMemcpyHostToDevice, si));
    }
    KSMM_CUDA_OK(cudaEventRecord(g_host.ev_in[sl], si));
    KSMM_CUDA_OK(cudaStreamWaitEvent(sc, g_host.ev_in[sl], 0));
    // the output buffer is free once the slice two back has left it
    if (gs >= 2) KSMM_CUDA_OK(cudaStreamWaitEvent(sc, g_host.ev_out[sl], 0));
    st = ksmm_cu_chain_forward(din, dvals.data(), dout, dbias, g_host.buf[3], g_host.cap[3], cn,
                               nfactors, patterns, dtype, bs_last, sc);
    if (st != KSMM_OK) {
      cudaDeviceSynchronize();
      return st;
    }
    KSMM_CUDA_OK(cudaEventRecord(g_host.ev_cmp[sl], sc));
    KSMM_CUDA_OK(cudaStreamWaitEvent(so, g_host.ev_cmp[sl], 0));
    if (bs_last) {
      KSMM_CUDA_OK(cudaMemcpy2DAsync(hout + n0 * es, batch * es, dout, cn * es, cn * es, out_feats,
                                     cudaMemcpyDeviceToHost, so));
    } else {
      KSMM_CUDA_OK(cudaMemcpyAsync(hout + n0 * out_feats * es, dout, cn * out_feats * es,
                                   cudaMemcpyDeviceToHost, so));
    }
    KSMM_CUDA_OK(cudaEventRecord(g_host.ev_out[sl], so));
    ++g_host.slices;
  }
  KSMM_CUDA_OK(cudaEventRecord(g_host.ev_wfree[cp], sc));
  ++g_host.calls;
  const uint64_t t = g_host.calls;  // tickets start at 1
  const int slot = static_cast<int>(t % HostPathState::kTickets);
  // a slot is reused every kTickets calls: whoever recorded it last has long been enqueued, and the
  // copy stream is ordered, so the new record can only complete later than the old one
  KSMM_CUDA_OK(cudaEventRecord(g_host.ev_call[slot], so));
  g_host.ticket_of[slot] = t;
  *ticket = t;
  return KSMM_OK;
}

static int host_check_args(const void* host_input, const void* const* host_values, void* host_output,
                           int64_t batch, int nfactors, const int32_t* patterns, int dtype, int bs_last) {
  if (nfactors <= 0 || !patterns || !host_values || !host_input || !host_output)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "null argument to the host-memory chain call");
  if (batch < 0) return set_error(KSMM_ERR_BAD_ARGUMENT, "negative batch");
  if (bs_last != 0 && bs_last != 1) return set_error(KSMM_ERR_BAD_ARGUMENT, "bs_last must be 0 or 1");
  return check_chain(nfactors, patterns, host_values, dtype, 0);
}

int ksmm_cu_chain_forward_host_async(const void* host_input, const void* const* host_values,
                                     void* host_output, const void* host_bias, int64_t batch,
                                     int nfactors, const int32_t* patterns, int dtype, int bs_last,
                                     int device, uint64_t* ticket) {
  if (!ticket) return set_error(KSMM_ERR_BAD_ARGUMENT, "null ticket pointer");
  *ticket = 0;
  int st = host_check_args(host_input, host_values, host_output, batch, nfactors, patterns, dtype, bs_last);
  if (st != KSMM_OK) return st;
  if (batch == 0) return KSMM_OK;  // ticket 0: nothing to wait for
  std::lock_guard<std::mutex> g(g_host.mu);
  return host_submit(host_input, host_values, host_output, host_bias, batch, nfactors, patterns, dtype,
                     bs_last, device, ticket, /*whole_batch=*/true);
}

int ksmm_cu_host_wait(uint64_t ticket) {
  if (ticket == 0) return KSMM_OK;
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> g(g_host.mu);
    if (ticket > g_host.calls) return set_error(KSMM_ERR_BAD_ARGUMENT, "ticket %llu was never issued",
                                                static_cast<unsigned long long>(ticket));
    const int slot = static_cast<int>(ticket % HostPathState::kTickets);
    // a newer call in the same slot completes after this one (one ordered copy stream)
    ev = g_host.ev_call[slot];
  }
  KSMM_CUDA_OK(cudaEventSynchronize(ev));
  return KSMM_OK;
}

int ksmm_cu_chain_forward_host(const void* host_input, const void* const* host_values,
                               void* host_output, const void* host_bias, int64_t batch,
                               int nfactors, const int32_t* patterns, int dtype, int bs_last,
                               int device) {
  uint64_t ticket = 0;
  int st = host_check_args(host_input, host_values, host_output, batch, nfactors, patterns, dtype, bs_last);
  if (st != KSMM_OK) return st;
  if (batch == 0) return KSMM_OK;
  {
    std::lock_guard<std::mutex> g(g_host.mu);
    st = host_submit(host_input, host_values, host_output, host_bias, batch, nfactors, patterns, dtype, bs_last,
                     device, &ticket, /*whole_batch=*/false);
  }
  if (st != KSMM_OK) return st;
  return ksmm_cu_host_wait(ticket);
}

int ksmm_cu_num_configs(int algo) {
  if (algo == KSMM_ALGO_SIMT) return kNumFfmaConfigs;
  if (algo == KSMM_ALGO_TC) return tc_num_configs();
  if (algo == KSMM_ALGO_CONVERT) return 1;
  return 0;
}

int ksmm_cu_config_supported(int algo, int config, int64_t batch, int a, int b, int c, int d,
                             int in_dtype, int out_dtype, int bs_last) {
  Problem p;
  p.in = p.w = nullptr; p.out = nullptr; p.bias = nullptr;
  p.batch = batch; p.a = a; p.b = b; p.c = c; p.d = d;
  p.in_dtype = in_dtype; p.out_dtype = out_dtype; p.bs_last = bs_last; p.alpha = 1.f;
  if (a <= 0 || b <= 0 || c <= 0 || d <= 0 || batch <= 0) return 0;
  if (algo == KSMM_ALGO_SIMT) {
    if (config < 0 || config >= kNumFfmaConfigs) return 0;
    if (config == kFfmaTmaWide || config == kFfmaTmaNarrow) return ffma_tma_supported(p, false);
    if (config == kFfmaTmaFirst) return ffma_tma_first_supported(p, false);
    if (in_dtype == KSMM_F8E4M3) return out_dtype != KSMM_F8E4M3;
    return in_dtype == out_dtype;
  }
  if (algo == KSMM_ALGO_TC) return tc_config_supported(p, config, /*check_pointers=*/false);
  if (algo == KSMM_ALGO_CONVERT) return config == 0 && conversion_possible(p);
  return 0;
}

int ksmm_cu_tune(const ksmm_forward_desc_t* desc, int nrepeats, void* stream, int* best_algo,
                 int* best_config, float* best_ms) {
  if (!desc) return set_error(KSMM_ERR_BAD_ARGUMENT, "null descriptor");
  Problem p = problem_of(*desc);
  int st = check_problem(p);
  if (st != KSMM_OK) return st;
  if (p.batch == 0) return set_error(KSMM_ERR_BAD_ARGUMENT, "cannot tune an empty batch");
  if (nrepeats < 1) nrepeats = 1;
  if (nrepeats > 64) nrepeats = 64;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Every timed launch starts with a cold L2, as it does between the layers of a network: a
  // buffer larger than the cache is overwritten before each one, outside the timed interval.
  // (Timing back-to-back launches on the same operands instead favours whatever re-reads most.)
  int dev = 0, l2_bytes = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&l2_bytes, cudaDevAttrL2CacheSize, dev);
  const size_t flush_bytes = static_cast<size_t>(l2_bytes > 0 ? l2_bytes : (128 << 20)) * 3 / 2;
  void* flush = nullptr;
  KSMM_CUDA_OK(cudaMalloc(&flush, flush_bytes));
  g_allocs.fetch_add(1, std::memory_order_relaxed);
  std::vector<cudaEvent_t> ev(2 * static_cast<size_t>(nrepeats));
  for (auto& e : ev) cudaEventCreate(&e);
  auto cleanup = [&]() {
    for (auto& e : ev) cudaEventDestroy(e);
    cudaFree(flush);
  };
  float best = -1.f;
  Choice win{KSMM_ALGO_SIMT, simt_default_config_for(p)};
  // candidates: every configuration of the two kernel families that can run the problem, and
  // the layout-conversion path (transpose, batch-last kernel, transpose) where it exists
  const int families[3] = {KSMM_ALGO_TC, KSMM_ALGO_SIMT, KSMM_ALGO_CONVERT};
  for (int fam : families) {
    const int ncfg = fam == KSMM_ALGO_CONVERT ? 1 : ksmm_cu_num_configs(fam);
    for (int cfg = 0; cfg < ncfg; ++cfg) {
      if (!choice_runnable(p, Choice{fam, cfg})) continue;
      if (fam == KSMM_ALGO_SIMT &&
          !ksmm_cu_config_supported(fam, cfg, p.batch, p.a, p.b, p.c, p.d, p.in_dtype, p.out_dtype, p.bs_last))
        continue;
      // warm-up (also surfaces launch errors)
      if (run_family(p, fam, cfg, s) != KSMM_OK) continue;
      if (cudaStreamSynchronize(s) != cudaSuccess) {
        cleanup();
        return set_error(KSMM_ERR_CUDA, "tuning candidate (%d,%d) failed on the device", fam, cfg);
      }
      for (int r = 0; r < nrepeats; ++r) {
        cudaMemsetAsync(flush, r & 1, flush_bytes, s);
        cudaEventRecord(ev[2 * r], s);
        run_family(p, fam, cfg, s);
        cudaEventRecord(ev[2 * r + 1], s);
      }
      if (cudaStreamSynchronize(s) != cudaSuccess) {
        cleanup();
        return set_error(KSMM_ERR_CUDA, "tuning candidate (%d,%d) failed on the device", fam, cfg);
      }
      float ms = 0.f;
      for (int r = 0; r < nrepeats; ++r) {
        float one = 0.f;
        cudaEventElapsedTime(&one, ev[2 * r], ev[2 * r + 1]);
        ms += one;
      }
      ms /= nrepeats;
      if (best < 0.f || ms < best) {
        best = ms;
        win = Choice{fam, cfg};
      }
    }
  }
  cleanup();
  if (best < 0.f) return set_error(KSMM_ERR_UNSUPPORTED, "no kernel candidate ran");
  {
    std::lock_guard<std::mutex> g(g_choice_mu);
    g_choices[key_of(p)] = win;
  }
  if (best_algo) *best_algo = win.algo;
  if (best_config) *best_config = win.config;
  if (best_ms) *best_ms = best;
  return KSMM_OK;
}

int ksmm_cu_set_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype,
                       int bs_last, int algo, int config) {
  if (algo != KSMM_ALGO_SIMT && algo != KSMM_ALGO_TC && algo != KSMM_ALGO_CONVERT)
    return set_error(KSMM_ERR_BAD_ARGUMENT, "unknown kernel family %d", algo);
  if (!ksmm_cu_config_supported(algo, config, batch, a, b, c, d, in_dtype, out_dtype, bs_last))
    return set_error(KSMM_ERR_UNSUPPORTED, "configuration (%d,%d) cannot run this problem", algo,
                     config);
  std::lock_guard<std::mutex> g(g_choice_mu);
  g_choices[ChoiceKey(batch, a, b, c, d, in_dtype, out_dtype, bs_last)] = Choice{algo, config};
  return KSMM_OK;
}

int ksmm_cu_clear_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype, int bs_last) {
  std::lock_guard<std::mutex> g(g_choice_mu);
  if (batch < 0) {
    g_choices.clear();  // the whole cache
    return KSMM_OK;
  }
  g_choices.erase(ChoiceKey(batch, a, b, c, d, in_dtype, out_dtype, bs_last));
  return KSMM_OK;
}

int ksmm_cu_get_choice(int64_t batch, int a, int b, int c, int d, int in_dtype, int out_dtype,
                       int bs_last, int* algo, int* config) {
  std::lock_guard<std::mutex> g(g_choice_mu);
  auto it = g_choices.find(ChoiceKey(batch, a, b, c, d, in_dtype, out_dtype, bs_last));
  if (it == g_choices.end()) return set_error(KSMM_ERR_BAD_ARGUMENT, "no cached choice");
  if (algo) *algo = it->second.algo;
  if (config) *config = it->second.config;
  return KSMM_OK;
}

int ksmm_cu_default_choice(const ksmm_forward_desc_t* desc, int* algo, int* config,
                           int* via_transpose) {
  if (!desc) return set_error(KSMM_ERR_BAD_ARGUMENT, "null descriptor");
  Problem p = problem_of(*desc);
  int st = check_problem(p);
  if (st != KSMM_OK) return st;
  int al = KSMM_ALGO_SIMT, cfg = -1, conv = 0;
  Choice ch = auto_choice(p);
  if (ch.algo == KSMM_ALGO_CONVERT) {
    // report the kernel of the batch-last problem that the conversion path dispatches
    conv = 1;
    Problem q = p;
    q.bs_last = 1;
    q.in = q.out = reinterpret_cast<void*>(256);
    ch = auto_choice(q);
  }
  al = ch.algo;
  cfg = ch.config;
  if (algo) *algo = al;
  if (config) *config = cfg;
  if (via_transpose) *via_transpose = conv;
  return KSMM_OK;
}

int ksmm_cu_measure_ffma_peak(float* tflops, void* stream) {
  if (!tflops) return set_error(KSMM_ERR_BAD_ARGUMENT, "null result pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int dev = 0, sms = 0;
  KSMM_CUDA_OK(cudaGetDevice(&dev));
  KSMM_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  float* sink = nullptr;
  KSMM_CUDA_OK(cudaMalloc(&sink, sizeof(float)));
  g_allocs.fetch_add(1, std::memory_order_relaxed);
  const int iters = 4096, blocks = sms * 8;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  ffma_probe_kernel<<<blocks, 256, 0, s>>>(sink, iters, 1.f);  // warm-up
  float best = 1e30f;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(e0, s);
    ffma_probe_kernel<<<blocks, 256, 0, s>>>(sink, iters, 1.f);
    cudaEventRecord(e1, s);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaError_t err = cudaGetLastError();
  cudaFree(sink);
  if (err != cudaSuccess)
    return set_error(KSMM_ERR_CUDA, "ffma probe failed: %s", cudaGetErrorString(err));
  const double fl = 2.0 * 16 * 8 * static_cast<double>(iters) * 256.0 * blocks;
  *tflops = static_cast<float>(fl / (best * 1e-3) / 1e12);
  return KSMM_OK;
}

}  // extern "C"
