// ksmm_cli: standalone driver on top of the C ABI.
//
// Stands in for the reference's `sparse_mm -n <kernel> -d <device> -r <nrepeats>`
// (src/ksmm_cu/src/template_sparse_mm.cu:117-149), whose pattern and batch size
// are compile-time constants substituted by sed: here they are arguments.
//
//   ksmm_cli -n kernel_bs_last_half -p 1,768,192,4 [-b 25088] [-d 0] [-r 100] [-o file.out]
//
// Kernel names as in the reference (template_sparse_mm.cu:194-230):
//   kernel_bs_{first,last}_{float,half,bf16,fp8e4m3}
// The program fills X ~ N(0,1) and the kernel-format weights ~ U(-1/sqrt(c), 1/sqrt(c)),
// warms up, times `nrepeats` launches with one CUDA-event pair each, checks 1 % of the
// batch entries against a CPU loop (the reference does the same,
// template_sparse_mm.cu:806-861) and appends one row in the reference's format
//   "batch a b c d TILEX TILEK TILEY TX TY VSIZE ms std mse"
// (template_sparse_mm.cu:887-890) to <kernel>.out, or to wrong_mse_<kernel>.out if the RMSE
// exceeds the reference's thresholds 1e-5 / 1e-2 / 5e-2.  The tile columns carry the kernel
// family (TILEX: 1 = ffma, 2 = tensor) and configuration (TILEK) the library chose; the
// others are 0.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "../../include/ksmm_cu.h"

#define CK(x)                                                                  \
  do {                                                                         \
    cudaError_t e__ = (x);                                                     \
    if (e__ != cudaSuccess) {                                                  \
      fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e__));                \
      return 2;                                                                \
    }                                                                          \
  } while (0)

static float to_float(const void* p, size_t idx, int dt) {
  switch (dt) {
    case KSMM_F32: return static_cast<const float*>(p)[idx];
    case KSMM_F16: return __half2float(static_cast<const __half*>(p)[idx]);
    case KSMM_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    default: {
      __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<const unsigned char*>(p)[idx], __NV_E4M3);
      return __half2float(__half(h));
    }
  }
}
static void from_float(void* p, size_t idx, int dt, float v) {
  switch (dt) {
    case KSMM_F32: static_cast<float*>(p)[idx] = v; break;
    case KSMM_F16: static_cast<__half*>(p)[idx] = __float2half_rn(v); break;
    case KSMM_BF16: static_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v); break;
    default:
      static_cast<unsigned char*>(p)[idx] =
          static_cast<unsigned char>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
}
static size_t esize(int dt) { return dt == KSMM_F32 ? 4 : (dt == KSMM_F8E4M3 ? 1 : 2); }

int main(int argc, char** argv) {
  std::string kernel = "kernel_bs_last_half", outfile;
  int device = 0, nrepeats = 100, a = 1, b = 48, c = 48, d = 1;
  long long batch = 25088;
  for (int i = 1; i < argc; ++i) {
    std::string f = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (f == "-n" || f == "--kernel") kernel = next();
    else if (f == "-d" || f == "--device") device = atoi(next());
    else if (f == "-r" || f == "--nrepeats") nrepeats = atoi(next());
    else if (f == "-b" || f == "--batch") batch = atoll(next());
    else if (f == "-o" || f == "--out") outfile = next();
    else if (f == "-p" || f == "--pattern") {
      if (sscanf(next(), "%d,%d,%d,%d", &a, &b, &c, &d) != 4) {
        fprintf(stderr, "pattern must be a,b,c,d\n");
        return 1;
      }
    } else {
      fprintf(stderr,
              "usage: %s -n kernel_bs_{first,last}_{float,half,bf16,fp8e4m3} -p a,b,c,d "
              "[-b batch] [-d device] [-r nrepeats] [-o file]\n", argv[0]);
      return 1;
    }
  }
  int bs_last, dt;
  if (kernel.find("_bs_last_") != std::string::npos) bs_last = 1;
  else if (kernel.find("_bs_first_") != std::string::npos) bs_last = 0;
  else { fprintf(stderr, "unknown kernel name %s\n", kernel.c_str()); return 1; }
  if (kernel.find("float") != std::string::npos) dt = KSMM_F32;
  else if (kernel.find("half") != std::string::npos) dt = KSMM_F16;
  else if (kernel.find("bf16") != std::string::npos) dt = KSMM_BF16;
  else if (kernel.find("fp8e4m3") != std::string::npos) dt = KSMM_F8E4M3;
  else { fprintf(stderr, "unknown precision in kernel name %s\n", kernel.c_str()); return 1; }
  const int odt = dt == KSMM_F8E4M3 ? KSMM_BF16 : dt;  // fp8 inputs produce bf16 outputs
  if (outfile.empty()) outfile = kernel + ".out";

  CK(cudaSetDevice(device));
  const size_t n_in = static_cast<size_t>(a) * c * d, n_out = static_cast<size_t>(a) * b * d;
  const size_t nw = static_cast<size_t>(a) * b * c * d;
  std::vector<unsigned char> hx(n_in * batch * esize(dt)), hw(nw * esize(dt)),
      hy(n_out * batch * esize(odt));
  std::mt19937_64 rng(1);
  std::normal_distribution<float> nd(0.f, 1.f);
  std::uniform_real_distribution<float> ud(-1.f / std::sqrt(static_cast<float>(c)),
                                           1.f / std::sqrt(static_cast<float>(c)));
  for (size_t q = 0; q < n_in * batch; ++q) from_float(hx.data(), q, dt, nd(rng));
  for (size_t q = 0; q < nw; ++q) from_float(hw.data(), q, dt, ud(rng));

  void *dx, *dw, *dy;
  CK(cudaMalloc(&dx, hx.size()));
  CK(cudaMalloc(&dw, hw.size()));
  CK(cudaMalloc(&dy, hy.size()));
  CK(cudaMemcpy(dx, hx.data(), hx.size(), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dw, hw.data(), hw.size(), cudaMemcpyHostToDevice));

  ksmm_forward_desc_t desc;
  memset(&desc, 0, sizeof(desc));
  desc.input = dx; desc.values = dw; desc.output = dy; desc.bias = nullptr;
  desc.batch = batch; desc.a = a; desc.b = b; desc.c = c; desc.d = d;
  desc.in_dtype = dt; desc.out_dtype = odt; desc.bs_last = bs_last;
  desc.algo = KSMM_ALGO_AUTO; desc.config = -1; desc.alpha = 1.f;

  // pick the fastest candidate (the reference's tuner does this offline), then time it
  int algo = 0, config = -1;
  float tuned_ms = 0.f;
  int st = ksmm_cu_tune(&desc, 10, nullptr, &algo, &config, &tuned_ms);
  if (st != KSMM_OK) { fprintf(stderr, "tune: %s\n", ksmm_cu_last_error()); return 3; }
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  std::vector<float> times;
  for (int r = 0; r < nrepeats; ++r) {
    CK(cudaEventRecord(e0));
    st = ksmm_cu_forward_ex(&desc, nullptr);
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    if (st != KSMM_OK) { fprintf(stderr, "forward: %s\n", ksmm_cu_last_error()); return 3; }
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    times.push_back(ms);
  }
  if (ksmm_cu_check_device(nullptr) != KSMM_OK) { fprintf(stderr, "%s\n", ksmm_cu_last_error()); return 3; }
  double mean = 0, var = 0;
  for (float t : times) mean += t;
  mean /= times.size();
  for (float t : times) var += (t - mean) * (t - mean);
  const double stdv = std::sqrt(var / times.size());
  CK(cudaMemcpy(hy.data(), dy, hy.size(), cudaMemcpyDeviceToHost));

  // CPU check on every 100th batch entry
  double sq = 0;
  size_t cnt = 0;
  auto xin = [&](long long n, size_t p) { return bs_last ? p * batch + n : n * n_in + p; };
  auto yout = [&](long long n, size_t q) { return bs_last ? q * batch + n : n * n_out + q; };
  for (long long n = 0; n < batch; n += 100) {
    for (int i = 0; i < a; ++i)
      for (int j = 0; j < b; ++j)
        for (int l = 0; l < d; ++l) {
          double acc = 0;
          for (int k = 0; k < c; ++k)
            acc += static_cast<double>(to_float(hw.data(), ((static_cast<size_t>(i) * d + l) * c + k) * b + j, dt)) *
                   to_float(hx.data(), xin(n, (static_cast<size_t>(i) * c + k) * d + l), dt);
          const double got = to_float(hy.data(), yout(n, (static_cast<size_t>(i) * b + j) * d + l), odt);
          sq += (got - acc) * (got - acc);
          ++cnt;
        }
  }
  const double rmse = std::sqrt(sq / cnt);
  const double thr = dt == KSMM_F32 ? 1e-5 : (dt == KSMM_F8E4M3 ? 5e-2 : 1e-2);
  const std::string target = rmse < thr ? outfile : "wrong_mse_" + outfile;
  FILE* f = fopen(target.c_str(), "a");
  if (!f) { perror(target.c_str()); return 4; }
  fprintf(f, "%lld %d %d %d %d %d %d 0 0 0 0 %.6f %.6f %.6e\n", batch, a, b, c, d, algo, config, mean,
          stdv, rmse);
  fclose(f);
  printf("%s pattern (%d,%d,%d,%d) batch %lld: family %d config %d, %.4f +/- %.4f ms, rmse %.3e -> %s\n",
         kernel.c_str(), a, b, c, d, batch, algo, config, mean, stdv, rmse, target.c_str());
  cudaFree(dx); cudaFree(dw); cudaFree(dy);
  return rmse < thr ? 0 : 5;
}
