// Thin PyTorch C++ extension over the C ABI of libksmm_cu.so.
//
// Same module surface as the reference's extension
// (src/ksmm_py/layer/kronecker_sparse/kernel.cpp:25-50): forward(input, factor,
// bs_last, a, b, c, d, dtype, vsize) -> output tensor on the input's device and
// current stream.  `dtype` and `vsize` are accepted for signature compatibility;
// the element type is the input tensor's and vector widths are chosen by the
// library.  chain_forward runs all factors of one KSLinear in one call.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <string>
#include <vector>

#include "../../include/ksmm_cu.h"

namespace {

int dtype_code(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return KSMM_F32;
    case at::kHalf: return KSMM_F16;
    case at::kBFloat16: return KSMM_BF16;
    default: TORCH_CHECK(false, "ksmm: unsupported tensor type ", t.scalar_type());
  }
  return -1;
}

void check_input(const torch::Tensor& x, const char* name) {
  TORCH_CHECK(x.device().is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
}

void check_status(int st) { TORCH_CHECK(st == KSMM_OK, "libksmm_cu: ", ksmm_cu_last_error()); }

torch::Tensor forward(torch::Tensor input, torch::Tensor factor, int64_t bs_last, int64_t a, int64_t b,
                      int64_t c, int64_t d, const std::string& /*dtype*/, int64_t /*vsize*/) {
  check_input(input, "input");
  check_input(factor, "factor");
  TORCH_CHECK(input.dim() == 2 && factor.dim() == 2, "input and factor are 2-D");
  TORCH_CHECK(input.size(bs_last ? 0 : 1) == a * c * d, "input has ", input.size(bs_last ? 0 : 1),
              " features, the pattern expects ", a * c * d);
  TORCH_CHECK(factor.size(0) == a * d * c && factor.size(1) == b, "factor must be (a*d*c, b)");
  TORCH_CHECK(factor.scalar_type() == input.scalar_type() && factor.device() == input.device(),
              "factor and input must share type and device");
  const c10::cuda::CUDAGuard guard(input.device());
  const int64_t batch = input.size(bs_last ? 1 : 0);
  auto out = bs_last ? torch::empty({a * b * d, batch}, input.options())
                     : torch::empty({batch, a * b * d}, input.options());
  check_status(ksmm_cu_forward(input.data_ptr(), factor.data_ptr(), out.data_ptr(), batch,
                               static_cast<int>(a), static_cast<int>(b), static_cast<int>(c),
                               static_cast<int>(d), dtype_code(input), bs_last ? 1 : 0,
                               at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

torch::Tensor chain_forward(torch::Tensor input, std::vector<torch::Tensor> factors,
                            std::vector<std::vector<int64_t>> patterns, int64_t bs_last,
                            c10::optional<torch::Tensor> bias, int64_t activation) {
  check_input(input, "input");
  TORCH_CHECK(input.dim() == 2, "input is 2-D: (features, batch) batch-last, (batch, features) batch-first");
  TORCH_CHECK(!patterns.empty() && patterns.size() == factors.size(), "one factor per pattern");
  std::vector<int32_t> flat;
  std::vector<const void*> vals;
  int64_t feats = input.size(bs_last ? 0 : 1);  // features entering the next factor
  for (size_t f = 0; f < patterns.size(); ++f) {
    TORCH_CHECK(patterns[f].size() == 4, "a pattern is (a, b, c, d)");
    for (int64_t v : patterns[f])
      TORCH_CHECK(v > 0 && v <= 0x7fffffffLL, "pattern values are positive 32-bit integers, got ", v);
    const int64_t a = patterns[f][0], b = patterns[f][1], c = patterns[f][2], d = patterns[f][3];
    TORCH_CHECK(a * c * d == feats, "factor ", f, " expects ", a * c * d, " features but receives ", feats);
    check_input(factors[f], "factor");
    TORCH_CHECK(factors[f].dim() == 2 && factors[f].size(0) == a * d * c && factors[f].size(1) == b,
                "factor ", f, " must have shape (a*d*c, b) = (", a * d * c, ", ", b, ")");
    TORCH_CHECK(factors[f].scalar_type() == input.scalar_type(), "factors share the input's type");
    TORCH_CHECK(factors[f].device() == input.device(), "factors live on the input's device");
    for (int64_t v : patterns[f]) flat.push_back(static_cast<int32_t>(v));
    vals.push_back(factors[f].data_ptr());
    feats = a * b * d;
  }
  const c10::cuda::CUDAGuard guard(input.device());
  const int64_t batch = input.size(bs_last ? 1 : 0);
  const auto& pl = patterns.back();
  const int64_t n_out = pl[0] * pl[1] * pl[3];
  auto out = bs_last ? torch::empty({n_out, batch}, input.options())
                     : torch::empty({batch, n_out}, input.options());
  const int code = dtype_code(input);
  const size_t need = ksmm_cu_chain_workspace_bytes_ex(static_cast<int>(patterns.size()), flat.data(), batch,
                                                       code, bs_last ? 1 : 0);
  torch::Tensor ws;
  if (need > 0) ws = torch::empty({static_cast<int64_t>(need)}, input.options().dtype(at::kByte));
  const void* bptr = nullptr;
  if (bias.has_value()) {
    check_input(*bias, "bias");
    TORCH_CHECK(bias->numel() == n_out && bias->scalar_type() == input.scalar_type() &&
                    bias->device() == input.device(),
                "bias must hold out_size elements of the input's type on the input's device");
    bptr = bias->data_ptr();
  }
  check_status(ksmm_cu_chain_forward_act(input.data_ptr(), vals.data(), out.data_ptr(), bptr,
                                         need > 0 ? ws.data_ptr() : nullptr, need, batch,
                                         static_cast<int>(patterns.size()), flat.data(), code,
                                         bs_last ? 1 : 0, static_cast<int>(activation),
                                         at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("forward", &forward, "One Kronecker-sparse factor (CUDA, libksmm_cu)");
  m.def("chain_forward", &chain_forward, "All factors of a KSLinear in one call (CUDA, libksmm_cu)",
        py::arg("input"), py::arg("factors"), py::arg("patterns"), py::arg("bs_last"),
        py::arg("bias") = py::none(), py::arg("activation") = 0);
}
