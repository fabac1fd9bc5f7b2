// Python bindings of the dense-tower kernels.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "../kernels/rb_dense.h"

namespace py = pybind11;
using torch::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

Tensor& status_word(const torch::Device& dev) {
  static std::map<int, Tensor> words;
  auto it = words.find(dev.index());
  if (it == words.end())
    it = words.emplace(dev.index(), torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt64).device(dev))).first;
  return it->second;
}

// out[MM, NN] = act(A B^T + bias). a: [MM, KK] or (a_mn) [KK, MM]; b: [NN, KK] or (b_mn) [KK, NN]; bf16, inner stride 1.
Tensor gemm_bf16(const Tensor& a, const Tensor& b, OptT bias, bool relu, bool a_mn, bool b_mn, bool out_fp32, OptT accumulate_into) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm_bf16 is a CUDA (sm_100a) kernel");
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16, "bf16 operands expected");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "2-D operands with unit inner stride expected");
  const int64_t MM = a_mn ? a.size(1) : a.size(0), KK = a_mn ? a.size(0) : a.size(1);
  const int64_t NN = b_mn ? b.size(1) : b.size(0), KB = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(KK == KB, "reduction sizes differ: ", KK, " vs ", KB);
  c10::cuda::CUDAGuard g(a.device());
  Tensor out;
  const float* beta = nullptr;
  if (accumulate_into.has_value() && accumulate_into->defined()) {
    out = *accumulate_into;
    TORCH_CHECK(out_fp32 && out.scalar_type() == torch::kFloat32 && out.is_contiguous() && out.size(0) == MM && out.size(1) == NN);
    beta = out.data_ptr<float>();
  } else {
    out = torch::empty({MM, NN}, a.options().dtype(out_fp32 ? torch::kFloat32 : torch::kBFloat16));
  }
  const float* bp = nullptr;
  Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->scalar_type() == torch::kFloat32 ? bias->contiguous() : bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == NN);
    bp = bias_f.data_ptr<float>();
  }
  Tensor& st = status_word(a.device());
  const int rc = rb_gemm_bf16(a.data_ptr(), a.stride(0), a_mn, b.data_ptr(), b.stride(0), b_mn, out.data_ptr(), out.stride(0), out_fp32, bp,
                              beta, (int)MM, (int)NN, (int)KK, relu, st.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "rb_gemm_bf16 failed with code ", rc,
              " (1: operand base/pitch not 16-byte aligned, 2: tensor map encode failed, >2: launch error)");
  return out;
}

int64_t dense_status(const std::string& device) { return status_word(torch::Device(device)).item<int64_t>(); }

}  // namespace

void init_dense(py::module& m) {
  m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("bias") = py::none(), py::arg("relu") = false,
        py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("out_fp32") = false, py::arg("accumulate_into") = py::none());
  m.def("dense_status", &dense_status);
}
