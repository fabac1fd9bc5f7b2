// Functions of one binding file that other binding files call directly (no trip through Python).
#pragma once
#include <cstdlib>
#include <torch/extension.h>
#include <tuple>
#include <vector>
#include "../kernels/rb_kernels.h"

namespace rbx {

// RECIS_DEBUG_BOUNDS=1: the bindings of the row-indexing kernels validate their index tensors on the device before they launch
// (one reduction and one host read per call: a debugging mode) and raise instead of launching a kernel that would leave its
// buffers. Nothing traps on the device.
inline bool debug_bounds() {
  static const bool on = [] { const char* e = std::getenv("RECIS_DEBUG_BOUNDS"); return e != nullptr && e[0] == '1'; }();
  return on;
}
inline void debug_check_range(const char* what, const torch::Tensor& idx, int64_t lo, int64_t hi) {
  if (!debug_bounds() || !idx.defined() || idx.numel() == 0) return;
  auto flat = idx.reshape({-1});
  auto bad = flat.lt(lo).logical_or(flat.ge(hi));
  if (bad.any().item<bool>()) {
    const int64_t pos = bad.nonzero().select(1, 0)[0].item<int64_t>();
    TORCH_CHECK(false, what, ": index ", flat[pos].item<int64_t>(), " at position ", pos, " of ", flat.numel(), " is outside [", lo, ", ", hi, ")");
  }
}
// the first n_dev[0] entries of idx (all of them without n_dev)
inline torch::Tensor debug_prefix(const torch::Tensor& idx, const c10::optional<torch::Tensor>& n_dev) {
  if (!debug_bounds() || !n_dev.has_value() || !n_dev->defined()) return idx;
  const int64_t n = std::min<int64_t>(std::max<int64_t>(n_dev->reshape({-1})[0].item<int64_t>(), 0), idx.numel());
  return idx.reshape({-1}).narrow(0, 0, n);
}

// storage type code (RbRowDType) of a tensor of embedding rows; raises for anything but fp32 / fp16 / bf16 / int8
inline int row_dtype_of(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case torch::kFloat32: return 0;
    case torch::kFloat16: return 1;
    case torch::kBFloat16: return 2;
    case torch::kInt8: return 3;
    default: TORCH_CHECK(false, "embedding rows must be float32, float16, bfloat16 or int8, got ", t.scalar_type()); return 0;
  }
}

// Optimizer description for the kernels: hyper-parameters plus the row slab `w` (fp32 / fp16 / bf16) and its fp32 state slabs.
inline RbOpt make_opt(int64_t kind, double lr, double beta1, double beta2, double eps, double decay, double alpha, double grad_scale,
                      const c10::optional<torch::Tensor>& w, const c10::optional<torch::Tensor>& s1, const c10::optional<torch::Tensor>& s2) {
  RbOpt o;
  o.kind = (int)kind; o.lr = (float)lr; o.beta1 = (float)beta1; o.beta2 = (float)beta2; o.eps = (float)eps; o.decay = (float)decay;
  o.alpha = (float)alpha; o.grad_scale = (float)grad_scale;
  o.w = nullptr; o.w_dtype = 0;
  if (w.has_value() && w->defined()) {
    o.w_dtype = row_dtype_of(*w);
    TORCH_CHECK(o.w_dtype != 3, "int8 tables are read-only: they cannot be updated by an optimizer");
    o.w = w->data_ptr();
  }
  auto f32_ptr = [](const c10::optional<torch::Tensor>& t) -> float* {
    if (!(t.has_value() && t->defined())) return nullptr;
    TORCH_CHECK(t->scalar_type() == torch::kFloat32, "optimizer state slabs are float32");
    return t->data_ptr<float>();
  };
  o.s1 = f32_ptr(s1); o.s2 = f32_ptr(s2);
  return o;
}

// bind_sparse.cpp
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> dedup_partition(
    const torch::Tensor& ids, int64_t world, c10::optional<torch::Tensor> unique_out, c10::optional<torch::Tensor> offsets_out,
    c10::optional<torch::Tensor> status, c10::optional<torch::Tensor> counts_out);
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> build_csr(const torch::Tensor& reverse);

// bind_ragged_fused.cpp: multi-feature sequence truncation on CUDA (three launches and one host read for all features).
// 2-D: values / offsets / drop_nums / pad_nums per feature; 3-D: values / inner offsets (`offsets`) / outer offsets.
struct CutoffResult {
  std::vector<torch::Tensor> values, offsets, outer, drop_nums, pad_nums;
};
CutoffResult fused_cutoff_cuda(const std::vector<torch::Tensor>& values, const std::vector<torch::Tensor>& offsets,
                               const std::vector<torch::Tensor>& outer_offsets, const torch::Tensor& keep_lengths,
                               const torch::Tensor& drop_sides, const torch::Tensor& pad_sides, bool three_d);

}  // namespace rbx
