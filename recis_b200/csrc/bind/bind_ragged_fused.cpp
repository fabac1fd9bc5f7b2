// Host side of the multi-feature sequence truncation on CUDA: builds the feature table, runs the three launches of
// kernels/ragged_fused.cu around the ONE host read that sizes the outputs. Semantics of the reference's
// fused_ragged_cutoff / fused_ragged_cutoff_3D (csrc/ops/fused_ragged_cutoff_kernel.cu:102-258,451-784).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "../kernels/rb_ragged_fused.h"
#include "bind_shared.h"

namespace rbx {

using torch::Tensor;

namespace {
inline bool flag_at(const Tensor& cpu_flags, int t) { return cpu_flags.data_ptr<bool>()[cpu_flags.numel() == 1 ? 0 : t]; }
inline int64_t keep_at(const Tensor& cpu_keep, int t) { return cpu_keep.data_ptr<int64_t>()[cpu_keep.numel() == 1 ? 0 : t]; }
inline Tensor offsets_ready(const Tensor& o) {
  // int32 and int64 offsets are used as they are; anything else is widened
  if (o.scalar_type() == torch::kInt32 || o.scalar_type() == torch::kInt64) return o.contiguous();
  return o.to(torch::kInt64).contiguous();
}
}  // namespace

CutoffResult fused_cutoff_cuda(const std::vector<Tensor>& values, const std::vector<Tensor>& offsets, const std::vector<Tensor>& outer_offsets,
                               const Tensor& keep_lengths, const Tensor& drop_sides, const Tensor& pad_sides, bool three_d) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)offsets.size() == T && (!three_d || (int)outer_offsets.size() == T), "values / offsets length mismatch");
  auto dev = values[0].device();
  c10::cuda::CUDAGuard guard(dev);
  auto st = at::cuda::getCurrentCUDAStream();
  // per-feature settings are tiny host-side tables (a device tensor here would cost a synchronising copy)
  auto keep = keep_lengths.to(torch::kCPU, torch::kInt64).reshape(-1).contiguous();
  auto dl = drop_sides.to(torch::kCPU, torch::kBool).reshape(-1).contiguous();
  auto pl = pad_sides.to(torch::kCPU, torch::kBool).reshape(-1).contiguous();
  TORCH_CHECK(keep.numel() == T || keep.numel() == 1, "keep_lengths: one entry per tensor expected");

  CutoffResult res;
  std::vector<Tensor> vals(T), offs(T), outer(T);
  auto pinned = torch::TensorOptions().dtype(torch::kUInt8).pinned_memory(true);
  auto table_host = torch::empty({(int64_t)(sizeof(RbCutoffFeature) * T)}, pinned);
  auto* feats = reinterpret_cast<RbCutoffFeature*>(table_host.data_ptr());
  int64_t total_rows = 0;
  for (int t = 0; t < T; ++t) {
    vals[t] = values[t].contiguous();
    offs[t] = offsets_ready(offsets[t]);
    RbCutoffFeature& f = feats[t];
    std::memset(&f, 0, sizeof(f));
    f.values = vals[t].data_ptr();
    f.offsets = offs[t].data_ptr();
    f.off_is_i64 = offs[t].scalar_type() == torch::kInt64;
    f.elem_size = (int32_t)vals[t].element_size();
    TORCH_CHECK(f.elem_size == 1 || f.elem_size == 2 || f.elem_size == 4 || f.elem_size == 8, "unsupported value type");
    f.keep = keep_at(keep, t);
    TORCH_CHECK(f.keep >= 0, "keep length must not be negative");
    f.drop_left = flag_at(dl, t); f.pad_left = flag_at(pl, t);
    f.row_prefix = total_rows;
    if (three_d) {
      outer[t] = offsets_ready(outer_offsets[t]).to(offs[t].scalar_type());
      TORCH_CHECK(outer[t].numel() >= 1 && offs[t].numel() >= 1, "empty offsets");
      const int64_t B = outer[t].numel() - 1;
      f.outer_offsets = outer[t].data_ptr();
      f.n_out_rows = B * f.keep;
      res.outer.push_back(torch::zeros({B + 1}, offs[t].options()));        // zeros: a feature with keep == 0 writes nothing
      f.out_outer = res.outer.back().data_ptr();
    } else {
      f.n_out_rows = offs[t].numel() - 1;
    }
    res.offsets.push_back(torch::empty({f.n_out_rows + 1}, offs[t].options()));
    f.out_offsets = res.offsets.back().data_ptr();
    total_rows += f.n_out_rows;
  }
  auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(dev);
  auto scratch = torch::empty({4 * total_rows + T}, i64);
  int64_t* src_beg = scratch.data_ptr<int64_t>();
  int64_t* keep_len = src_beg + total_rows;
  int64_t* drop_n = keep_len + total_rows;
  int64_t* pad_n = drop_n + total_rows;
  int64_t* totals = pad_n + total_rows;
  auto table_dev = torch::empty({table_host.numel() + (int64_t)sizeof(void*) * T}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
  auto* feats_dev = reinterpret_cast<RbCutoffFeature*>(table_dev.data_ptr());
  void** out_ptrs_dev = reinterpret_cast<void**>(static_cast<char*>(table_dev.data_ptr()) + table_host.numel());
  TORCH_CHECK(cudaMemcpyAsync(feats_dev, feats, table_host.numel(), cudaMemcpyHostToDevice, st) == cudaSuccess, "descriptor upload failed");
  rb_cutoff_rows(feats_dev, T, total_rows, three_d ? 1 : 0, src_beg, keep_len, drop_n, pad_n, totals, st);
  // the one host read of the call: how many values every feature keeps
  auto totals_host = torch::empty({T}, torch::TensorOptions().dtype(torch::kInt64).pinned_memory(true));
  TORCH_CHECK(cudaMemcpyAsync(totals_host.data_ptr(), totals, sizeof(int64_t) * T, cudaMemcpyDeviceToHost, st) == cudaSuccess, "totals read failed");
  TORCH_CHECK(cudaStreamSynchronize(st) == cudaSuccess, "stream synchronisation failed");
  auto out_ptrs_host = torch::empty({(int64_t)(sizeof(void*) * T)}, pinned);
  int64_t max_total = 0;
  for (int t = 0; t < T; ++t) {
    const int64_t n = totals_host.data_ptr<int64_t>()[t];
    max_total = std::max(max_total, n);
    res.values.push_back(torch::empty({n}, vals[t].options()));
    reinterpret_cast<void**>(out_ptrs_host.data_ptr())[t] = res.values.back().data_ptr();
  }
  TORCH_CHECK(cudaMemcpyAsync(out_ptrs_dev, out_ptrs_host.data_ptr(), sizeof(void*) * T, cudaMemcpyHostToDevice, st) == cudaSuccess, "pointer upload failed");
  rb_cutoff_copy(feats_dev, T, out_ptrs_dev, totals, src_beg, max_total, st);
  // pinned staging buffers must outlive their asynchronous copies: the copies were issued on `st`, and the buffers are released
  // to torch's pinned-memory cache, which reuses a block only after the stream work recorded at release time has finished
  if (!three_d) {
    for (int t = 0; t < T; ++t) {
      res.drop_nums.push_back(scratch.narrow(0, 2 * total_rows + feats[t].row_prefix, feats[t].n_out_rows));
      res.pad_nums.push_back(scratch.narrow(0, 3 * total_rows + feats[t].row_prefix, feats[t].n_out_rows));
    }
  }
  for (int t = 0; t < T; ++t)
    if (res.offsets[t].scalar_type() != offsets[t].scalar_type()) res.offsets[t] = res.offsets[t].to(offsets[t].scalar_type());
  return res;
}

}  // namespace rbx
