// Ragged-tensor operations: one implementation per op, instantiated for both devices.
//
// Each op is a handful of element-wise passes ("count -> prefix sum -> fill"). A pass is written once as a
// __host__ __device__ lambda and run either as a grid-stride sm_100a kernel on the current stream or as an OpenMP loop on
// the CPU, so the CUDA path and its CPU oracle cannot drift apart. Ops (reference file in parentheses):
//   ragged_to_dense (csrc/ops/ragged_to_dense_kernel.cu:31-153), dense_to_ragged (dense_to_ragged_kernel.cu:10-83),
//   ragged_to_sparse (ragged_to_sparse.cc:8-89: CPU only there), fused_ragged_cutoff 2-D / 3-D
//   (fused_ragged_cutoff_kernel.cu:29-784), calc_ragged_index (calc_ragged_index.cc:15-124: CPU only and one of four
//   drop/pad modes there; all four here), feature_cross_ragged (feature_cross_ragged_kernel.cu:22-418),
//   gen_segment_indices (embedding_segment_reduce_kernel.cu:394-424), and the feature-engine fused ops' bindings.
#include <torch/extension.h>
#include "bind_shared.h"
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "../common/rb_hash.cuh"
#include "../common/rb_launch.h"
#include "../kernels/rb_feature.h"
#include <cub/device/device_segmented_sort.cuh>
#include <algorithm>

namespace py = pybind11;
using torch::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

template <typename F>
__global__ void __launch_bounds__(256) for_each_kernel(int64_t n, F f) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) f(i);
}

template <typename F>
void for_each(const torch::Device& dev, int64_t n, F f) {
  if (n <= 0) return;
  if (dev.is_cuda()) {
    const int64_t blocks = std::min<int64_t>((n + 255) / 256, 148 * 16);
    for_each_kernel<<<(int)blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(n, f);
    rb::note_launch();
  } else {
#pragma omp parallel for schedule(static) if (n > 4096)
    for (int64_t i = 0; i < n; ++i) f(i);
  }
}

// row containing flat position p: offsets[row] <= p < offsets[row + 1]
template <typename T>
__host__ __device__ inline int64_t find_row(const T* off, int64_t n_rows, int64_t p) {
  int64_t lo = 0, hi = n_rows;
  while (hi - lo > 1) { const int64_t mid = (lo + hi) >> 1; if ((int64_t)off[mid] <= p) lo = mid; else hi = mid; }
  return lo;
}

Tensor as_i64(const Tensor& t) { return t.scalar_type() == torch::kInt64 ? t.contiguous() : t.to(torch::kInt64).contiguous(); }

// ---------------------------------------------------------------------------------- ragged <-> dense / sparse
constexpr int kMaxLevels = 5;
struct Levels { const int64_t* off[kMaxLevels]; int64_t rows[kMaxLevels]; int64_t width[kMaxLevels]; int n; };

// values [nnz, ...inner] + offsets (outermost first) -> dense [rows0, max1, ..., maxL, ...inner]
Tensor ragged_to_dense(const Tensor& values, const std::vector<Tensor>& offsets, double default_value) {
  const int L = (int)offsets.size();
  TORCH_CHECK(L >= 1 && L <= kMaxLevels, "1..5 ragged dimensions are supported");
  auto dev = values.device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> off64;
  Levels lv; lv.n = L;
  std::vector<int64_t> shape;
  for (int l = 0; l < L; ++l) {
    off64.push_back(as_i64(offsets[l]));
    lv.off[l] = off64[l].data_ptr<int64_t>();
    lv.rows[l] = off64[l].numel() - 1;
    // widest row of this level: one host read per level, as in the reference (ragged_to_dense.cc:65-70)
    lv.width[l] = lv.rows[l] > 0 ? (off64[l].slice(0, 1) - off64[l].slice(0, 0, lv.rows[l])).max().item<int64_t>() : 0;
  }
  shape.push_back(lv.rows[0]);
  for (int l = 0; l < L; ++l) shape.push_back(lv.width[l]);
  int64_t inner = 1;
  for (int d = 1; d < values.dim(); ++d) { shape.push_back(values.size(d)); inner *= values.size(d); }
  auto out = torch::full(shape, default_value, values.options());
  const int64_t nnz = values.size(0);
  auto vals = values.contiguous();
  AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, values.scalar_type(), "ragged_to_dense", [&] {
    const scalar_t* src = vals.data_ptr<scalar_t>();
    scalar_t* dst = out.data_ptr<scalar_t>();
    for_each(dev, nnz * inner, [=] __host__ __device__(int64_t w) {
      const int64_t i = w / inner, c = w - i * inner;
      // walk from the innermost level outwards collecting the column at each level
      int64_t pos = i, col[kMaxLevels];
      for (int l = lv.n - 1; l >= 0; --l) {
        const int64_t row = find_row(lv.off[l], lv.rows[l], pos);
        col[l] = pos - lv.off[l][row];
        pos = row;
      }
      int64_t idx = pos;                       // outermost row
      for (int l = 0; l < lv.n; ++l) idx = idx * lv.width[l] + col[l];
      dst[idx * inner + c] = src[w];
    });
  });
  return out;
}

// 2-D dense -> (values, offsets int32). check_invalid: trailing entries equal to invalid_value are stripped per row.
std::tuple<Tensor, Tensor> dense_to_ragged(const Tensor& dense, bool check_invalid, double invalid_value) {
  TORCH_CHECK(dense.dim() == 2, "dense_to_ragged expects a 2-D tensor");
  auto dev = dense.device();
  c10::OptionalDeviceGuard guard(dev);
  const int64_t B = dense.size(0), Lm = dense.size(1);
  auto d = dense.contiguous();
  auto lens = torch::empty({B}, d.options().dtype(torch::kInt64));
  int64_t* lp = lens.data_ptr<int64_t>();
  AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, d.scalar_type(), "dense_to_ragged_len", [&] {
    const scalar_t* src = d.data_ptr<scalar_t>();
    const scalar_t inv = static_cast<scalar_t>(invalid_value);
    for_each(dev, B, [=] __host__ __device__(int64_t b) {
      int64_t len = Lm;
      if (check_invalid) { while (len > 0 && src[b * Lm + len - 1] == inv) --len; }
      lp[b] = len;
    });
  });
  auto off64 = torch::zeros({B + 1}, lens.options());
  off64.slice(0, 1).copy_(lens.cumsum(0));
  const int64_t nnz = off64[B].item<int64_t>();
  auto values = torch::empty({nnz}, d.options());
  const int64_t* op = off64.data_ptr<int64_t>();
  AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, d.scalar_type(), "dense_to_ragged_fill", [&] {
    const scalar_t* src = d.data_ptr<scalar_t>();
    scalar_t* dst = values.data_ptr<scalar_t>();
    for_each(dev, nnz, [=] __host__ __device__(int64_t i) {
      const int64_t row = find_row(op, B, i);
      dst[i] = src[row * Lm + (i - op[row])];
    });
  });
  return {values, off64.to(torch::kInt32)};
}

// COO indices [L+1, nnz] of a ragged tensor (outermost row, then the column at every level) + dense shape
std::tuple<Tensor, std::vector<int64_t>> ragged_to_sparse_indices(int64_t nnz, const std::vector<Tensor>& offsets) {
  const int L = (int)offsets.size();
  TORCH_CHECK(L >= 1 && L <= kMaxLevels);
  auto dev = offsets[0].device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> off64;
  Levels lv; lv.n = L;
  for (int l = 0; l < L; ++l) {
    off64.push_back(as_i64(offsets[l]));
    lv.off[l] = off64[l].data_ptr<int64_t>();
    lv.rows[l] = off64[l].numel() - 1;
    lv.width[l] = lv.rows[l] > 0 ? (off64[l].slice(0, 1) - off64[l].slice(0, 0, lv.rows[l])).max().item<int64_t>() : 0;
  }
  auto idx = torch::empty({L + 1, nnz}, off64[0].options());
  int64_t* ip = idx.data_ptr<int64_t>();
  for_each(dev, nnz, [=] __host__ __device__(int64_t i) {
    int64_t pos = i;
    for (int l = lv.n - 1; l >= 0; --l) {
      const int64_t row = find_row(lv.off[l], lv.rows[l], pos);
      ip[(int64_t)(l + 1) * nnz + i] = pos - lv.off[l][row];
      pos = row;
    }
    ip[i] = pos;
  });
  std::vector<int64_t> shape{lv.rows[0]};
  for (int l = 0; l < L; ++l) shape.push_back(lv.width[l]);
  return {idx, shape};
}

// offsets [S+1] -> segment id of every element [nnz]
Tensor gen_segment_indices(const Tensor& offsets, int64_t nnz) {
  auto dev = offsets.device();
  c10::OptionalDeviceGuard guard(dev);
  auto off = as_i64(offsets);
  auto out = torch::empty({nnz}, off.options());
  const int64_t* op = off.data_ptr<int64_t>(); int64_t* o = out.data_ptr<int64_t>();
  const int64_t S = off.numel() - 1;
  for_each(dev, nnz, [=] __host__ __device__(int64_t i) { o[i] = find_row(op, S, i); });
  return out;
}

// ---------------------------------------------------------------------------------- sequence truncate / pad
// 2-D, T tensors fused: rows of tensor t keep at most keep[t] values (dropping from the left when drop_left[t], else
// from the right). No pad values are materialised: pad_nums only reports how many a dense consumer would add.
// Returns (values..., offsets..., drop_nums..., pad_nums...).
std::tuple<std::vector<Tensor>, std::vector<Tensor>, std::vector<Tensor>, std::vector<Tensor>>
fused_ragged_cutoff_2d(const std::vector<Tensor>& values, const std::vector<Tensor>& offsets, const Tensor& keep_lengths,
                       const Tensor& drop_sides, const Tensor& pad_sides) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)offsets.size() == T, "values / offsets length mismatch");
  auto dev = values[0].device();
  if (dev.is_cuda()) {
    // all features in three launches and one host read (kernels/ragged_fused.cu); the code below is the CPU implementation
    auto r = rbx::fused_cutoff_cuda(values, offsets, {}, keep_lengths, drop_sides, pad_sides, false);
    return {r.values, r.offsets, r.drop_nums, r.pad_nums};
  }
  c10::OptionalDeviceGuard guard(dev);
  auto keep = keep_lengths.to(torch::kCPU, torch::kInt64).reshape(-1);
  auto dl = drop_sides.to(torch::kCPU, torch::kBool).reshape(-1);
  TORCH_CHECK(keep.numel() == T || keep.numel() == 1, "keep_lengths: one entry per tensor expected");
  std::vector<Tensor> out_v, out_o, out_d, out_p;
  // concatenated row space: row_prefix[t] rows before tensor t
  std::vector<int64_t> row_prefix(T + 1, 0);
  for (int t = 0; t < T; ++t) row_prefix[t + 1] = row_prefix[t] + offsets[t].numel() - 1;
  const int64_t R = row_prefix[T];
  auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(dev);
  auto new_len = torch::empty({R}, i64), drop_n = torch::empty({R}, i64), pad_n = torch::empty({R}, i64), src_beg = torch::empty({R}, i64);
  std::vector<Tensor> off64(T);
  for (int t = 0; t < T; ++t) {
    off64[t] = as_i64(offsets[t]);
    const int64_t B = off64[t].numel() - 1, k = keep[keep.numel() == 1 ? 0 : t].item<int64_t>();
    const bool left = dl[dl.numel() == 1 ? 0 : t].item<bool>();
    const int64_t* op = off64[t].data_ptr<int64_t>();
    int64_t* nl = new_len.data_ptr<int64_t>() + row_prefix[t]; int64_t* dn = drop_n.data_ptr<int64_t>() + row_prefix[t];
    int64_t* pn = pad_n.data_ptr<int64_t>() + row_prefix[t]; int64_t* sb = src_beg.data_ptr<int64_t>() + row_prefix[t];
    for_each(dev, B, [=] __host__ __device__(int64_t b) {
      const int64_t len = op[b + 1] - op[b];
      const int64_t kept = len < k ? len : k;
      nl[b] = kept; dn[b] = len - kept; pn[b] = k - kept;
      sb[b] = op[b] + (left ? len - kept : 0);
    });
  }
  for (int t = 0; t < T; ++t) {
    const int64_t B = row_prefix[t + 1] - row_prefix[t];
    auto nl = new_len.narrow(0, row_prefix[t], B);
    auto no = torch::zeros({B + 1}, i64);
    no.slice(0, 1).copy_(nl.cumsum(0));
    const int64_t nnz = B > 0 ? no[B].item<int64_t>() : 0;          // output size: one host read per tensor
    auto vals = values[t].contiguous();
    auto nv = torch::empty({nnz}, vals.options());
    const int64_t* nop = no.data_ptr<int64_t>(); const int64_t* sb = src_beg.data_ptr<int64_t>() + row_prefix[t];
    AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, vals.scalar_type(), "cutoff2d_fill", [&] {
      const scalar_t* src = vals.data_ptr<scalar_t>(); scalar_t* dst = nv.data_ptr<scalar_t>();
      for_each(dev, nnz, [=] __host__ __device__(int64_t i) {
        const int64_t row = find_row(nop, B, i);
        dst[i] = src[sb[row] + (i - nop[row])];
      });
    });
    out_v.push_back(nv);
    out_o.push_back(no.to(offsets[t].scalar_type()));
    out_d.push_back(drop_n.narrow(0, row_prefix[t], B));
    out_p.push_back(pad_n.narrow(0, row_prefix[t], B));
  }
  return {out_v, out_o, out_d, out_p};
}

// 3-D: every sample keeps exactly keep[t] inner rows (dropping rows from the left/right, padding with EMPTY rows on the
// left/right). Returns (values..., outer offsets..., inner offsets...).
std::tuple<std::vector<Tensor>, std::vector<Tensor>, std::vector<Tensor>>
fused_ragged_cutoff_3d(const std::vector<Tensor>& values, const std::vector<Tensor>& outer_offsets, const std::vector<Tensor>& inner_offsets,
                       const Tensor& keep_lengths, const Tensor& drop_sides, const Tensor& pad_sides) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)outer_offsets.size() == T && (int)inner_offsets.size() == T);
  auto dev = values[0].device();
  if (dev.is_cuda()) {
    auto r = rbx::fused_cutoff_cuda(values, inner_offsets, outer_offsets, keep_lengths, drop_sides, pad_sides, true);
    for (int t = 0; t < T; ++t)
      if (r.outer[t].scalar_type() != outer_offsets[t].scalar_type()) r.outer[t] = r.outer[t].to(outer_offsets[t].scalar_type());
    return {r.values, r.outer, r.offsets};
  }
  c10::OptionalDeviceGuard guard(dev);
  auto keep = keep_lengths.to(torch::kCPU, torch::kInt64).reshape(-1);
  auto dl = drop_sides.to(torch::kCPU, torch::kBool).reshape(-1);
  auto pl = pad_sides.to(torch::kCPU, torch::kBool).reshape(-1);
  auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(dev);
  std::vector<Tensor> out_v, out_outer, out_inner;
  for (int t = 0; t < T; ++t) {
    auto outer = as_i64(outer_offsets[t]), inner = as_i64(inner_offsets[t]);
    const int64_t B = outer.numel() - 1, k = keep[keep.numel() == 1 ? 0 : t].item<int64_t>();
    const bool drop_left = dl[dl.numel() == 1 ? 0 : t].item<bool>(), pad_left = pl[pl.numel() == 1 ? 0 : t].item<bool>();
    const int64_t* op = outer.data_ptr<int64_t>(); const int64_t* ip = inner.data_ptr<int64_t>();
    // source inner row (or -1 for padding) and length of every output inner row
    auto src_row = torch::empty({B * k}, i64), row_len = torch::empty({B * k}, i64);
    int64_t* sr = src_row.data_ptr<int64_t>(); int64_t* rl = row_len.data_ptr<int64_t>();
    for_each(dev, B * k, [=] __host__ __device__(int64_t w) {
      const int64_t b = w / k, j = w - b * k;
      const int64_t n_rows = op[b + 1] - op[b];
      const int64_t kept = n_rows < k ? n_rows : k, pad = k - kept;
      const int64_t jj = pad_left ? j - pad : j;                 // index among the kept rows
      int64_t src = -1;
      if (jj >= 0 && jj < kept) src = op[b] + (drop_left ? n_rows - kept : 0) + jj;
      sr[w] = src;
      rl[w] = src >= 0 ? ip[src + 1] - ip[src] : 0;
    });
    auto new_inner = torch::zeros({B * k + 1}, i64);
    new_inner.slice(0, 1).copy_(row_len.cumsum(0));
    const int64_t nnz = B * k > 0 ? new_inner[B * k].item<int64_t>() : 0;
    auto vals = values[t].contiguous();
    auto nv = torch::empty({nnz}, vals.options());
    const int64_t* nip = new_inner.data_ptr<int64_t>();
    const int64_t n_out_rows = B * k;
    AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, vals.scalar_type(), "cutoff3d_fill", [&] {
      const scalar_t* src = vals.data_ptr<scalar_t>(); scalar_t* dst = nv.data_ptr<scalar_t>();
      for_each(dev, nnz, [=] __host__ __device__(int64_t i) {
        const int64_t row = find_row(nip, n_out_rows, i);
        dst[i] = src[ip[sr[row]] + (i - nip[row])];
      });
    });
    out_v.push_back(nv);
    out_outer.push_back(torch::arange(0, (B + 1) * k, k, i64).to(outer_offsets[t].scalar_type()));
    out_inner.push_back(new_inner.to(inner_offsets[t].scalar_type()));
  }
  return {out_v, out_outer, out_inner};
}

// Map positions inside truncated / padded rows back to positions of the original values. topk_index [rows, K] holds
// positions in the post-cutoff row of source segment indicator[row]; positions that fall on padding are dropped.
std::tuple<Tensor, Tensor> calc_ragged_index(const Tensor& drop_num, const Tensor& pad_num, bool drop_left, bool pad_left,
                                             const Tensor& offset, const Tensor& topk_index, const Tensor& indicator) {
  auto dev = topk_index.device();
  c10::OptionalDeviceGuard guard(dev);
  auto dn = as_i64(drop_num.to(dev)), pn = as_i64(pad_num.to(dev)), off = as_i64(offset.to(dev)), tk = as_i64(topk_index), ind = as_i64(indicator.to(dev));
  const int64_t rows = tk.size(0), K = tk.size(1);
  auto src = torch::empty({rows * K}, tk.options());
  auto valid = torch::empty({rows * K}, tk.options());
  const int64_t *dp = dn.data_ptr<int64_t>(), *pp = pn.data_ptr<int64_t>(), *op = off.data_ptr<int64_t>(), *tp = tk.data_ptr<int64_t>(),
                *ip = ind.data_ptr<int64_t>();
  int64_t* sp = src.data_ptr<int64_t>(); int64_t* vp = valid.data_ptr<int64_t>();
  for_each(dev, rows * K, [=] __host__ __device__(int64_t w) {
    const int64_t r = w / K;
    const int64_t seg = ip[r], beg = op[seg], end = op[seg + 1];
    const int64_t kept = (end - beg) - dp[seg];
    const int64_t k = tp[w] - (pad_left ? pp[seg] : 0);
    const bool ok = k >= 0 && k < kept;
    sp[w] = beg + (drop_left ? dp[seg] : 0) + k;
    vp[w] = ok ? 1 : 0;
  });
  auto csum = valid.cumsum(0);
  auto out_off = torch::zeros({rows + 1}, tk.options());
  if (rows > 0 && K > 0) out_off.slice(0, 1).copy_(csum.view({rows, K}).select(1, K - 1));
  auto out_idx = src.masked_select(valid.to(torch::kBool));
  return {out_idx.to(topk_index.scalar_type()), out_off.to(offset.scalar_type())};
}

// Per sample: unique(x) x unique(y) -> id = murmur(x, y), weight = wx * wy (first occurrence's weight).
std::tuple<Tensor, Tensor, Tensor> feature_cross_ragged(const Tensor& xv, const Tensor& xo, const Tensor& yv, const Tensor& yo, OptT xw, OptT yw) {
  auto dev = xv.device();
  c10::OptionalDeviceGuard guard(dev);
  auto xoff = as_i64(xo), yoff = as_i64(yo), xval = as_i64(xv), yval = as_i64(yv);
  const int64_t S = xoff.numel() - 1;
  TORCH_CHECK(yoff.numel() - 1 == S, "feature cross: both sides need the same number of rows");
  auto f32 = xval.options().dtype(torch::kFloat32);
  auto xwt = xw.has_value() && xw->defined() ? xw->to(torch::kFloat32).contiguous() : torch::ones({xval.numel()}, f32);
  auto ywt = yw.has_value() && yw->defined() ? yw->to(torch::kFloat32).contiguous() : torch::ones({yval.numel()}, f32);
  // Per-row unique values by a segmented sort (the reference sorts too: DeviceSegmentedRadixSort + block unique,
  // feature_cross_ragged_kernel.cu:22-125): rows come out ascending, a value that repeats keeps the weight of its first
  // occurrence (the sort is stable). Work is O(n log n) whatever the row lengths are.
  auto row_unique = [&](const Tensor& vals, const Tensor& off, const Tensor& w) {
    const int64_t n = vals.numel();
    auto sorted = torch::empty_like(vals);
    auto order = torch::empty({n}, vals.options().dtype(torch::kInt32));
    const int64_t* op = off.data_ptr<int64_t>();
    if (dev.is_cuda()) {
      auto iota = torch::arange(n, order.options());
      auto st = at::cuda::getCurrentCUDAStream();
      size_t bytes = 0;
      cub::DeviceSegmentedSort::StableSortPairs(nullptr, bytes, vals.data_ptr<int64_t>(), sorted.data_ptr<int64_t>(), iota.data_ptr<int32_t>(),
                                                order.data_ptr<int32_t>(), (int)n, (int)S, op, op + 1, st);
      auto temp = torch::empty({(int64_t)bytes + 1}, vals.options().dtype(torch::kUInt8));
      cub::DeviceSegmentedSort::StableSortPairs(temp.data_ptr(), bytes, vals.data_ptr<int64_t>(), sorted.data_ptr<int64_t>(),
                                                iota.data_ptr<int32_t>(), order.data_ptr<int32_t>(), (int)n, (int)S, op, op + 1, st);
      rb::note_launch();
    } else {
      const int64_t* v = vals.data_ptr<int64_t>(); int64_t* so = sorted.data_ptr<int64_t>(); int32_t* od = order.data_ptr<int32_t>();
#pragma omp parallel for schedule(dynamic, 64) if (S > 256)
      for (int64_t r = 0; r < S; ++r) {
        std::vector<int32_t> idx((size_t)(op[r + 1] - op[r]));
        for (size_t k = 0; k < idx.size(); ++k) idx[k] = (int32_t)(op[r] + k);
        std::stable_sort(idx.begin(), idx.end(), [v](int32_t a, int32_t b) { return v[a] < v[b]; });
        for (size_t k = 0; k < idx.size(); ++k) { so[op[r] + k] = v[idx[k]]; od[op[r] + k] = idx[k]; }
      }
    }
    // head of every run of equal values inside a row
    auto head = torch::empty({n}, vals.options());
    {
      const int64_t* so = sorted.data_ptr<int64_t>(); int64_t* h = head.data_ptr<int64_t>();
      for_each(dev, n, [=] __host__ __device__(int64_t i) {
        const int64_t row = find_row(op, S, i);
        h[i] = (i == op[row] || so[i] != so[i - 1]) ? 1 : 0;
      });
    }
    auto rank = head.cumsum(0);                                         // inclusive: rank[i] - 1 = position among the uniques
    auto uoff = torch::zeros({S + 1}, vals.options());
    {
      const int64_t* rk = rank.data_ptr<int64_t>(); int64_t* uo = uoff.data_ptr<int64_t>();
      for_each(dev, S + 1, [=] __host__ __device__(int64_t r) { uo[r] = op[r] > 0 ? rk[op[r] - 1] : 0; });
    }
    return std::make_tuple(sorted, order, head, rank, uoff);
  };
  auto [xs, xord, xh, xrank, xuo] = row_unique(xval, xoff, xwt);
  auto [ys, yord, yh, yrank, yuo] = row_unique(yval, yoff, ywt);
  // output offsets: unique(x) * unique(y) per row
  auto out_off = torch::zeros({S + 1}, xval.options());
  {
    auto per_row = (xuo.slice(0, 1) - xuo.slice(0, 0, S)) * (yuo.slice(0, 1) - yuo.slice(0, 0, S));
    out_off.slice(0, 1).copy_(per_row.cumsum(0));
  }
  const int64_t total = S > 0 ? out_off[S].item<int64_t>() : 0;          // the one host read: the size of the result
  // compact the unique values and their weights
  auto compact = [&](const Tensor& sorted, const Tensor& order, const Tensor& head, const Tensor& rank, const Tensor& w, int64_t n_u) {
    auto uv = torch::empty({n_u}, sorted.options());
    auto uw = torch::empty({n_u}, f32);
    const int64_t* so = sorted.data_ptr<int64_t>(); const int32_t* od = order.data_ptr<int32_t>(); const int64_t* h = head.data_ptr<int64_t>();
    const int64_t* rk = rank.data_ptr<int64_t>(); const float* wp = w.data_ptr<float>();
    int64_t* uvp = uv.data_ptr<int64_t>(); float* uwp = uw.data_ptr<float>();
    for_each(dev, sorted.numel(), [=] __host__ __device__(int64_t i) {
      if (h[i]) { uvp[rk[i] - 1] = so[i]; uwp[rk[i] - 1] = wp[od[i]]; }
    });
    return std::make_pair(uv, uw);
  };
  // sizes of the compacted arrays are bounded by the inputs: no host read needed (the tails stay unused)
  auto [xu, xuw] = compact(xs, xord, xh, xrank, xwt, xval.numel());
  auto [yu, yuw] = compact(ys, yord, yh, yrank, ywt, yval.numel());
  auto out_v = torch::empty({total}, xval.options());
  auto out_w = torch::empty({total}, f32);
  const int64_t *oo = out_off.data_ptr<int64_t>(), *xo_ = xuo.data_ptr<int64_t>(), *yo_ = yuo.data_ptr<int64_t>(), *xp = xu.data_ptr<int64_t>(),
                *yp = yu.data_ptr<int64_t>();
  const float *xwp = xuw.data_ptr<float>(), *ywp = yuw.data_ptr<float>();
  int64_t* ov = out_v.data_ptr<int64_t>(); float* ow = out_w.data_ptr<float>();
  for_each(dev, total, [=] __host__ __device__(int64_t i) {
    const int64_t row = find_row(oo, S, i);
    const int64_t k = i - oo[row], ny = yo_[row + 1] - yo_[row];
    const int64_t a = xo_[row] + k / ny, b = yo_[row] + k % ny;
    ov[i] = (int64_t)rb::hash::murmur_pair((uint64_t)xp[a], (uint64_t)yp[b]);
    ow[i] = xwp[a] * ywp[b];
  });
  return {out_v, out_off.to(xo.scalar_type()), out_w};
}

// ---------------------------------------------------------------------------------- fused feature-engine ops
Tensor to_device_desc(const std::vector<std::vector<int64_t>>& rows, const torch::Device& dev) {
  const int64_t R = (int64_t)rows.size(), C = (int64_t)rows[0].size();
  auto host = torch::empty({R, C}, torch::TensorOptions().dtype(torch::kInt64).pinned_memory(dev.is_cuda()));
  for (int64_t r = 0; r < R; ++r) std::memcpy(host.data_ptr<int64_t>() + r * C, rows[r].data(), sizeof(int64_t) * C);
  return dev.is_cuda() ? host.to(dev, /*non_blocking=*/true) : host;
}

template <typename F>
void cpu_or_cuda(const torch::Device& dev, F&& cuda_fn, std::function<void()> cpu_fn) {
  if (dev.is_cuda()) cuda_fn(); else cpu_fn();
}

// strings: per tensor int8 bytes + int32 offsets -> int64 hashes (kind 0 farm, 1 murmur)
std::vector<Tensor> fused_hash(const std::vector<Tensor>& bytes, const std::vector<Tensor>& offsets, int64_t kind) {
  const int T = (int)bytes.size();
  TORCH_CHECK(T > 0 && (int)offsets.size() == T);
  auto dev = bytes[0].device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> b(T), o(T);
  std::vector<std::vector<int64_t>> rows(3, std::vector<int64_t>(T + 1, 0));
  for (int t = 0; t < T; ++t) {
    TORCH_CHECK(bytes[t].scalar_type() == torch::kInt8 || bytes[t].scalar_type() == torch::kUInt8, "hash input must be a byte tensor");
    b[t] = bytes[t].contiguous(); o[t] = offsets[t].to(torch::kInt32).contiguous();
    rows[0][t] = (int64_t)b[t].data_ptr(); rows[1][t] = (int64_t)o[t].data_ptr();
    rows[2][t + 1] = rows[2][t] + o[t].numel() - 1;
  }
  const int64_t total = rows[2][T];
  auto out = torch::empty({total}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
  if (dev.is_cuda()) {
    auto desc = to_device_desc(rows, dev);
    rb_fused_hash(desc.data_ptr<int64_t>(), T, total, (int)kind, out.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  } else {
    int64_t* op = out.data_ptr<int64_t>();
    for (int t = 0; t < T; ++t) {
      const char* s = reinterpret_cast<const char*>(b[t].data_ptr()); const int32_t* off = o[t].data_ptr<int32_t>();
      const int64_t n = o[t].numel() - 1, base = rows[2][t];
#pragma omp parallel for schedule(static) if (n > 4096)
      for (int64_t k = 0; k < n; ++k) {
        const size_t len = (size_t)(off[k + 1] - off[k]);
        op[base + k] = (int64_t)(kind == 0 ? rb::hash::farm_fingerprint64(s + off[k], len) : rb::hash::murmur64a(s + off[k], len, 0));
      }
    }
  }
  std::vector<Tensor> res;
  for (int t = 0; t < T; ++t) res.push_back(out.narrow(0, rows[2][t], rows[2][t + 1] - rows[2][t]));
  return res;
}

std::vector<Tensor> fused_bucketize(const std::vector<Tensor>& values, const std::vector<Tensor>& boundaries) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)boundaries.size() == T);
  auto dev = values[0].device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> v(T), bd(T);
  std::vector<std::vector<int64_t>> rows(4, std::vector<int64_t>(T + 1, 0));
  for (int t = 0; t < T; ++t) {
    v[t] = values[t].to(torch::kFloat32).contiguous(); bd[t] = boundaries[t].to(dev, torch::kFloat32).contiguous();
    rows[0][t] = (int64_t)v[t].data_ptr(); rows[1][t + 1] = rows[1][t] + v[t].numel();
    rows[2][t] = (int64_t)bd[t].data_ptr(); rows[3][t] = bd[t].numel();
  }
  const int64_t total = rows[1][T];
  auto out = torch::empty({total}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
  if (dev.is_cuda()) {
    auto desc = to_device_desc(rows, dev);
    rb_fused_bucketize(desc.data_ptr<int64_t>(), T, total, out.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  } else {
    int64_t* op = out.data_ptr<int64_t>();
    for (int t = 0; t < T; ++t) {
      const float* x = v[t].data_ptr<float>(); const float* b = bd[t].data_ptr<float>();
      const int64_t n = v[t].numel(), nb = bd[t].numel(), base = rows[1][t];
#pragma omp parallel for schedule(static) if (n > 4096)
      for (int64_t i = 0; i < n; ++i) {
        int64_t lo = 0, hi = nb;
        while (lo < hi) { const int64_t mid = (lo + hi) >> 1; if (!(x[i] < b[mid])) lo = mid + 1; else hi = mid; }
        op[base + i] = lo;
      }
    }
  }
  std::vector<Tensor> res;
  for (int t = 0; t < T; ++t) res.push_back(out.narrow(0, rows[1][t], v[t].numel()).view(values[t].sizes()));
  return res;
}

std::vector<Tensor> fused_mod(const std::vector<Tensor>& values, const std::vector<int64_t>& mods) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)mods.size() == T);
  auto dev = values[0].device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> v(T);
  std::vector<std::vector<int64_t>> rows(4, std::vector<int64_t>(T + 1, 0));
  for (int t = 0; t < T; ++t) {
    TORCH_CHECK(mods[t] > 0, "modulus must be positive");
    v[t] = as_i64(values[t]);
    rows[0][t] = (int64_t)v[t].data_ptr(); rows[1][t + 1] = rows[1][t] + v[t].numel(); rows[2][t] = mods[t];
    // floor(2^64 / m): the kernel replaces the 64-bit division by a multiply-high with this constant
    rows[3][t] = mods[t] == 1 ? 0 : (int64_t)(uint64_t)((((unsigned __int128)1) << 64) / (unsigned __int128)(uint64_t)mods[t]);
  }
  const int64_t total = rows[1][T];
  auto out = torch::empty({total}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
  if (dev.is_cuda()) {
    auto desc = to_device_desc(rows, dev);
    rb_fused_mod(desc.data_ptr<int64_t>(), T, total, out.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  } else {
    int64_t* op = out.data_ptr<int64_t>();
    for (int t = 0; t < T; ++t) {
      const int64_t* x = v[t].data_ptr<int64_t>(); const int64_t n = v[t].numel(), base = rows[1][t]; const uint64_t m = (uint64_t)mods[t];
#pragma omp parallel for schedule(static) if (n > 4096)
      for (int64_t i = 0; i < n; ++i) op[base + i] = (int64_t)((uint64_t)x[i] % m);
    }
  }
  std::vector<Tensor> res;
  for (int t = 0; t < T; ++t) res.push_back(out.narrow(0, rows[1][t], v[t].numel()).view(values[t].sizes()));
  return res;
}

// per tensor: K_t <= 4 (mul, prime, bucket) triples; returns, per tensor, K_t output tensors
std::vector<std::vector<Tensor>> fused_multi_hash(const std::vector<Tensor>& values, const std::vector<std::vector<int64_t>>& muls,
                                                  const std::vector<std::vector<int64_t>>& primes,
                                                  const std::vector<std::vector<int64_t>>& buckets) {
  const int T = (int)values.size();
  TORCH_CHECK(T > 0 && (int)muls.size() == T && (int)primes.size() == T && (int)buckets.size() == T);
  auto dev = values[0].device();
  c10::OptionalDeviceGuard guard(dev);
  std::vector<Tensor> v(T);
  std::vector<std::vector<int64_t>> rows(15, std::vector<int64_t>(T + 1, 1));
  int kmax = 0;
  rows[1][0] = 0;
  for (int t = 0; t < T; ++t) {
    const int K = (int)muls[t].size();
    TORCH_CHECK(K >= 1 && K <= 4 && (int)primes[t].size() == K && (int)buckets[t].size() == K, "1..4 hashes per feature");
    kmax = std::max(kmax, K);
    v[t] = as_i64(values[t]);
    rows[0][t] = (int64_t)v[t].data_ptr(); rows[1][t + 1] = rows[1][t] + v[t].numel(); rows[2][t] = K;
    for (int k = 0; k < K; ++k) { rows[3 + k][t] = muls[t][k]; rows[7 + k][t] = primes[t][k]; rows[11 + k][t] = buckets[t][k]; }
  }
  const int64_t total = rows[1][T];
  auto out = torch::empty({kmax, total}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
  if (dev.is_cuda()) {
    auto desc = to_device_desc(rows, dev);
    rb_fused_multi_hash(desc.data_ptr<int64_t>(), T, total, kmax, out.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  } else {
    int64_t* op = out.data_ptr<int64_t>();
    for (int t = 0; t < T; ++t) {
      const int64_t* x = v[t].data_ptr<int64_t>(); const int64_t n = v[t].numel(), base = rows[1][t];
      for (int k = 0; k < (int)muls[t].size(); ++k) {
        const int64_t mul = muls[t][k], p = primes[t][k], bucket = buckets[t][k];
        for (int64_t i = 0; i < n; ++i) {
          int64_t r = (int64_t)((uint64_t)x[i] * (uint64_t)mul);
          r = ((r % p) + p) % p;
          op[(int64_t)k * total + base + i] = r % bucket;
        }
      }
    }
  }
  std::vector<std::vector<Tensor>> res(T);
  for (int t = 0; t < T; ++t)
    for (int k = 0; k < (int)muls[t].size(); ++k) res[t].push_back(out[k].narrow(0, rows[1][t], v[t].numel()).view(values[t].sizes()));
  return res;
}

}  // namespace

void init_ragged(py::module& m) {
  m.def("ragged_to_dense", &ragged_to_dense);
  m.def("dense_to_ragged", &dense_to_ragged);
  m.def("ragged_to_sparse_indices", &ragged_to_sparse_indices);
  m.def("gen_segment_indices", &gen_segment_indices);
  m.def("fused_ragged_cutoff_2d", &fused_ragged_cutoff_2d);
  m.def("fused_ragged_cutoff_3d", &fused_ragged_cutoff_3d);
  m.def("calc_ragged_index", &calc_ragged_index);
  m.def("feature_cross_ragged", &feature_cross_ragged);
  m.def("fused_hash", &fused_hash);
  m.def("fused_bucketize", &fused_bucketize);
  m.def("fused_mod", &fused_mod);
  m.def("fused_multi_hash", &fused_multi_hash);
}
