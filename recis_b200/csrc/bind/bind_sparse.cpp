// Python bindings of the sparse-path operations. Every function dispatches on the device of its inputs:
// CUDA tensors run the sm_100a kernels on the current stream, CPU tensors run the C++ implementations.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "../cpu/rb_cpu.h"
#include "../kernels/rb_kernels.h"
#include "store.h"
#include "../common/rb_launch.h"
#include "bind_shared.h"

namespace py = pybind11;
using torch::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }
inline const int32_t* opt_i32(const OptT& t) { return t.has_value() && t->defined() ? t->data_ptr<int32_t>() : nullptr; }
inline const float* opt_f32(const OptT& t) { return t.has_value() && t->defined() ? t->data_ptr<float>() : nullptr; }

int64_t pow2_at_least(int64_t x) { int64_t p = 64; while (p < x) p <<= 1; return p; }

}  // namespace

namespace rbx {

// ids -> (unique ids bucketed by owner rank, reverse index, per-owner counts, per-owner offsets)
// unique_out / offsets_out (optional) let the caller place the results in peer-visible memory.
std::tuple<Tensor, Tensor, Tensor, Tensor> dedup_partition(const Tensor& ids, int64_t world, OptT unique_out, OptT offsets_out,
                                                           OptT status, OptT counts_out) {
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous(), "ids: contiguous int64 expected");
  TORCH_CHECK(world >= 1 && world <= 1024, "world size out of range");
  const int64_t n = ids.numel();
  auto o = ids.options();
  const int64_t cap = pow2_at_least(2 * std::max<int64_t>(n, 1));
  auto set_keys = torch::empty({cap}, o);
  auto set_pos = torch::empty({cap + 1}, o.dtype(torch::kInt32));
  auto slot = torch::empty({std::max<int64_t>(n, 1)}, o.dtype(torch::kInt32));
  Tensor counts = counts_out.has_value() && counts_out->defined() ? *counts_out : torch::empty({world}, o.dtype(torch::kInt32));
  TORCH_CHECK(counts.numel() >= world && counts.scalar_type() == torch::kInt32, "dedup_partition: counts_out: int32 [world]");
  Tensor offsets = offsets_out.has_value() && offsets_out->defined() ? *offsets_out : torch::empty({world + 1}, o.dtype(torch::kInt32));
  Tensor unique_ids = unique_out.has_value() && unique_out->defined() ? *unique_out : torch::empty({n}, o);
  const bool guarded = status.has_value() && status->defined();   // a smaller unique buffer needs the status word
  TORCH_CHECK(offsets.numel() >= world + 1 && offsets.scalar_type() == torch::kInt32 && (guarded || unique_ids.numel() >= n) &&
              unique_ids.scalar_type() == torch::kInt64, "dedup_partition: output buffers too small or of the wrong type");
  auto reverse = torch::empty({n}, o.dtype(torch::kInt32));
  if (ids.is_cuda()) {
    c10::cuda::CUDAGuard g(ids.device());
    rb_dedup_partition(ids.data_ptr<int64_t>(), n, (int)world, reinterpret_cast<uint64_t*>(set_keys.data_ptr<int64_t>()),
                       set_pos.data_ptr<int32_t>(), cap, slot.data_ptr<int32_t>(), counts.data_ptr<int32_t>(),
                       offsets.data_ptr<int32_t>(), unique_ids.data_ptr<int64_t>(), reverse.data_ptr<int32_t>(), unique_ids.numel(),
                       guarded ? status->data_ptr<int64_t>() : nullptr, cur_stream());
  } else {
    rbc_dedup_partition(ids.data_ptr<int64_t>(), n, (int)world, reinterpret_cast<uint64_t*>(set_keys.data_ptr<int64_t>()),
                        set_pos.data_ptr<int32_t>(), cap, slot.data_ptr<int32_t>(), counts.data_ptr<int32_t>(),
                        offsets.data_ptr<int32_t>(), unique_ids.data_ptr<int64_t>(), reverse.data_ptr<int32_t>(), unique_ids.numel(),
                        guarded ? status->data_ptr<int64_t>() : nullptr);
  }
  return {unique_ids, reverse, counts, offsets};
}

}  // namespace rbx

namespace {
using rbx::dedup_partition;

// desc: int64 [4, F+1] (id pointers, nnz prefix, offsets pointers, segment prefix) on the target device.
std::tuple<Tensor, Tensor> encode_merge(const Tensor& desc, const Tensor& table_idx, int64_t F, int64_t total_nnz, int64_t total_seg,
                                        bool with_offsets) {
  auto o = desc.options();
  auto ids = torch::empty({total_nnz}, o.dtype(torch::kInt64));
  Tensor offs = with_offsets ? torch::empty({total_seg + 1}, o.dtype(torch::kInt32)) : Tensor();
  int32_t* op = with_offsets ? offs.data_ptr<int32_t>() : nullptr;
  if (desc.is_cuda()) {
    c10::cuda::CUDAGuard g(desc.device());
    rb_encode_merge(desc.data_ptr<int64_t>(), table_idx.data_ptr<int64_t>(), (int)F, total_nnz, total_seg, ids.data_ptr<int64_t>(), op,
                    cur_stream());
  } else {
    rbc_encode_merge(desc.data_ptr<int64_t>(), table_idx.data_ptr<int64_t>(), (int)F, total_nnz, total_seg, ids.data_ptr<int64_t>(), op);
  }
  return {ids, offs};
}

// out[i] = src[rows[i]] (zeros where rows[i] < 0); rows of any element type, the result has the type of src
// encode_merge for several feature lists at once (the lanes of one runtime group): the descriptor tables of all lists are
// written into one pinned staging buffer (a small ring, reused once its copy has completed) and travel to the device in ONE
// asynchronous copy, then one kernel per list prefixes ids with the 12-bit child index and rebases offsets. Everything a
// Python implementation would spend on building small tensors per list happens here instead.
struct DescRing {
  static constexpr int kSlots = 8;
  Tensor buf[kSlots];
  cudaEvent_t ev[kSlots] = {};
  bool used[kSlots] = {};
  int head = 0;
};

std::vector<std::tuple<Tensor, Tensor>> coalesce_lanes(const std::vector<std::vector<Tensor>>& ids, const std::vector<std::vector<Tensor>>& offsets,
                                                       const std::vector<std::vector<int64_t>>& children) {
  const size_t L = ids.size();
  TORCH_CHECK(L > 0 && offsets.size() == L && children.size() == L, "coalesce_lanes: one list of ids / offsets / children per lane");
  const auto dev = ids[0][0].device();
  int64_t words = 0;
  for (size_t l = 0; l < L; ++l) {
    TORCH_CHECK(!ids[l].empty() && offsets[l].size() == ids[l].size() && children[l].size() == ids[l].size(), "coalesce_lanes: ragged lists");
    words += 5 * ((int64_t)ids[l].size() + 1);
  }
  int64_t* host = nullptr;
  Tensor host_t;
  static DescRing rings[64];
  DescRing* ring = nullptr;
  int slot = 0;
  if (dev.is_cuda()) {
    ring = &rings[dev.index() % 64];
    slot = ring->head++ % DescRing::kSlots;
    if (ring->used[slot]) cudaEventSynchronize(ring->ev[slot]);          // issued eight uses ago: long finished
    if (!ring->buf[slot].defined() || ring->buf[slot].numel() < words) {
      ring->buf[slot] = torch::empty({std::max<int64_t>(words, 1024)}, torch::TensorOptions().dtype(torch::kInt64).pinned_memory(true));
      if (!ring->used[slot]) cudaEventCreateWithFlags(&ring->ev[slot], cudaEventDisableTiming);
    }
    host = ring->buf[slot].data_ptr<int64_t>();
  } else {
    host_t = torch::empty({words}, torch::TensorOptions().dtype(torch::kInt64));
    host = host_t.data_ptr<int64_t>();
  }
  struct Meta { int64_t F, nnz, segs, pos; };
  std::vector<Meta> meta(L);
  int64_t pos = 0;
  for (size_t l = 0; l < L; ++l) {
    const int64_t F = (int64_t)ids[l].size();
    int64_t* d = host + pos;                                   // [5][F + 1]: id pointers, nnz prefix, offset pointers, segment prefix, child
    int64_t nnz = 0, segs = 0;
    for (int64_t f = 0; f < F; ++f) {
      const Tensor& v = ids[l][f]; const Tensor& o = offsets[l][f];
      TORCH_CHECK(v.scalar_type() == torch::kInt64 && v.is_contiguous() && o.scalar_type() == torch::kInt32 && o.is_contiguous() &&
                  v.device() == dev && o.device() == dev, "coalesce_lanes: ids int64, offsets int32, contiguous, on one device");
      d[f] = reinterpret_cast<int64_t>(v.data_ptr());
      d[(F + 1) + f] = nnz;
      d[2 * (F + 1) + f] = reinterpret_cast<int64_t>(o.data_ptr());
      d[3 * (F + 1) + f] = segs;
      d[4 * (F + 1) + f] = children[l][f];
      nnz += v.numel(); segs += o.numel() - 1;
    }
    d[F] = 0; d[(F + 1) + F] = nnz; d[2 * (F + 1) + F] = 0; d[3 * (F + 1) + F] = segs; d[4 * (F + 1) + F] = 0;
    meta[l] = {F, nnz, segs, pos};
    pos += 5 * (F + 1);
  }
  std::vector<std::tuple<Tensor, Tensor>> out;
  auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(dev);
  if (dev.is_cuda()) {
    c10::cuda::CUDAGuard g(dev);
    auto st = cur_stream();
    auto desc = torch::empty({words}, i64);
    TORCH_CHECK(cudaMemcpyAsync(desc.data_ptr(), host, sizeof(int64_t) * words, cudaMemcpyHostToDevice, st) == cudaSuccess, "descriptor upload failed");
    cudaEventRecord(ring->ev[slot], st);
    ring->used[slot] = true;
    for (size_t l = 0; l < L; ++l) {
      const Meta& m = meta[l];
      auto o_ids = torch::empty({m.nnz}, i64);
      auto o_off = torch::empty({m.segs + 1}, i64.dtype(torch::kInt32));
      const int64_t* d = desc.data_ptr<int64_t>() + m.pos;
      rb_encode_merge(d, d + 4 * (m.F + 1), (int)m.F, m.nnz, m.segs, o_ids.data_ptr<int64_t>(), o_off.data_ptr<int32_t>(), st);
      out.emplace_back(o_ids, o_off);
    }
  } else {
    for (size_t l = 0; l < L; ++l) {
      const Meta& m = meta[l];
      auto o_ids = torch::empty({m.nnz}, i64);
      auto o_off = torch::empty({m.segs + 1}, i64.dtype(torch::kInt32));
      const int64_t* d = host + m.pos;
      rbc_encode_merge(d, d + 4 * (m.F + 1), (int)m.F, m.nnz, m.segs, o_ids.data_ptr<int64_t>(), o_off.data_ptr<int32_t>());
      out.emplace_back(o_ids, o_off);
    }
  }
  return out;
}

Tensor gather_rows(const Tensor& src, const Tensor& rows, OptT n_dev) {
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous() && rows.scalar_type() == torch::kInt32);
  const int64_t n = rows.numel(); const int64_t D = src.size(1);
  auto out = n_dev.has_value() ? torch::zeros({n, D}, src.options()) : torch::empty({n, D}, src.options());
  if (n == 0) return out;
  rbx::debug_check_range("gather_rows: rows", rbx::debug_prefix(rows, n_dev), -1, src.size(0));
  const int64_t row_bytes = D * src.element_size();
  if (src.is_cuda()) {
    c10::cuda::CUDAGuard g(src.device());
    rb_gather_rows(src.data_ptr(), rows.data_ptr<int32_t>(), n, opt_i32(n_dev), row_bytes, out.data_ptr(), cur_stream());
  } else {
    rbc_gather_rows(src.data_ptr(), rows.data_ptr<int32_t>(), n, opt_i32(n_dev), row_bytes, out.data_ptr());
  }
  return out;
}

// dst[rows[i]] = src[i] (or src[0] when broadcast); src must have the element type of dst
void scatter_rows(Tensor dst, const Tensor& rows, const Tensor& src, bool broadcast) {
  TORCH_CHECK(dst.dim() == 2 && dst.is_contiguous() && src.is_contiguous() && rows.scalar_type() == torch::kInt32);
  TORCH_CHECK(src.scalar_type() == dst.scalar_type(), "scatter_rows: source rows are ", src.scalar_type(), ", the table stores ", dst.scalar_type());
  const int64_t n = rows.numel(); const int64_t row_bytes = dst.size(1) * dst.element_size();
  if (n == 0) return;
  rbx::debug_check_range("scatter_rows: rows", rows, -1, dst.size(0));
  TORCH_CHECK(!rbx::debug_bounds() || broadcast || src.numel() >= n * dst.size(1), "scatter_rows: ", src.numel() / std::max<int64_t>(dst.size(1), 1),
              " source rows for ", n, " indices");
  if (dst.is_cuda()) {
    c10::cuda::CUDAGuard g(dst.device());
    rb_scatter_rows(dst.data_ptr(), rows.data_ptr<int32_t>(), n, row_bytes, src.data_ptr(), broadcast, cur_stream());
  } else {
    rbc_scatter_rows(dst.data_ptr(), rows.data_ptr<int32_t>(), n, row_bytes, src.data_ptr(), broadcast);
  }
}

void fill_rows_i64(Tensor dst, const Tensor& rows, int64_t value) {
  const int64_t n = rows.numel();
  if (n == 0) return;
  rbx::debug_check_range("fill_rows_i64: rows", rows, -1, dst.numel());
  if (dst.is_cuda()) {
    c10::cuda::CUDAGuard g(dst.device());
    rb_fill_rows_i64(dst.data_ptr<int64_t>(), rows.data_ptr<int32_t>(), n, value, cur_stream());
  } else {
    rbc_fill_rows_i64(dst.data_ptr<int64_t>(), rows.data_ptr<int32_t>(), n, value);
  }
}

// Pooling forward. Returns (out, gsrc, gscale); gsrc/gscale are empty tensors unless need_grad. With `out` given (a
// [batch * perm_total, D] tensor shared by several calls) the call fills features perm_off .. perm_off + perm_f - 1 of it.
std::tuple<Tensor, Tensor, Tensor> pool_forward(const Tensor& base, OptT rows, const Tensor& rev, const Tensor& offsets, OptT weights,
                                                int64_t mode, int64_t perm_b, int64_t perm_f, bool need_grad, OptT out_opt,
                                                int64_t perm_off, int64_t perm_total) {
  TORCH_CHECK(base.dim() == 2 && base.is_contiguous());
  const int base_dtype = rbx::row_dtype_of(base);
  TORCH_CHECK(rev.scalar_type() == torch::kInt32 && offsets.scalar_type() == torch::kInt32);
  const int64_t n_seg = offsets.numel() - 1, n = rev.numel(); const int D = (int)base.size(1);
  if (perm_f > 0) TORCH_CHECK(perm_b * perm_f == n_seg, "permuted pooling output needs n_seg == batch * features");
  Tensor out;
  if (out_opt.has_value() && out_opt->defined()) {
    out = *out_opt;
    TORCH_CHECK(out.is_contiguous() && out.scalar_type() == torch::kFloat32 && out.device() == base.device() && perm_off >= 0,
                "pool_forward: out must be contiguous fp32 on the same device");
    if (perm_f > 0) {
      TORCH_CHECK(perm_total >= perm_off + perm_f && out.numel() == perm_b * perm_total * D, "pool_forward: out must be [batch * perm_total, D]");
    } else {
      TORCH_CHECK(out.numel() >= (perm_off + n_seg) * D, "pool_forward: out is too small for rows perm_off .. perm_off + n_seg");
    }
  } else {
    perm_off = 0; perm_total = perm_f;
    out = torch::empty({n_seg, D}, base.options().dtype(torch::kFloat32));
  }
  Tensor gsrc, gscale;
  if (need_grad) {
    gsrc = torch::empty({n}, rev.options());
    gscale = torch::empty({n}, base.options().dtype(torch::kFloat32));
  }
  int32_t* gp = need_grad ? gsrc.data_ptr<int32_t>() : nullptr;
  float* gs = need_grad ? gscale.data_ptr<float>() : nullptr;
  if (rbx::debug_bounds() && n > 0) {
    const bool via = rows.has_value() && rows->defined();
    rbx::debug_check_range("pool_forward: reverse index", rev, 0, via ? rows->numel() : base.size(0));
    if (via) rbx::debug_check_range("pool_forward: table rows of the referenced unique ids", rows->index_select(0, rev.to(torch::kInt64)), -1, base.size(0));
    rbx::debug_check_range("pool_forward: offsets", offsets, 0, n + 1);
  }
  if (base.is_cuda()) {
    c10::cuda::CUDAGuard g(base.device());
    rb_pool_forward(base.data_ptr(), base_dtype, opt_i32(rows), rev.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(), opt_f32(weights), n_seg, D,
                    (int)mode, (int)perm_b, (int)perm_f, (int)perm_off, (int)perm_total, out.data_ptr<float>(), gp, gs, cur_stream());
  } else {
    rbc_pool_forward(base.data_ptr(), base_dtype, opt_i32(rows), rev.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(), opt_f32(weights), n_seg,
                     D, (int)mode, (int)perm_b, (int)perm_f, (int)perm_off, (int)perm_total, out.data_ptr<float>(), gp, gs);
  }
  return {out, gsrc, gscale};
}

std::tuple<Tensor, Tensor, Tensor> tile_forward(const Tensor& base, OptT rows, const Tensor& rev, const Tensor& offsets, OptT weights,
                                                int64_t tile_len, bool need_grad) {
  TORCH_CHECK(base.dim() == 2 && base.is_contiguous());
  const int base_dtype = rbx::row_dtype_of(base);
  const int64_t n_seg = offsets.numel() - 1, n = rev.numel(); const int D = (int)base.size(1);
  auto f32 = base.options().dtype(torch::kFloat32);
  auto out = torch::empty({n_seg, tile_len * D}, f32);
  Tensor gsrc, gscale;
  if (need_grad) { gsrc = torch::empty({n}, rev.options()); gscale = torch::empty({n}, f32); }
  int32_t* gp = need_grad ? gsrc.data_ptr<int32_t>() : nullptr;
  float* gs = need_grad ? gscale.data_ptr<float>() : nullptr;
  if (base.is_cuda()) {
    c10::cuda::CUDAGuard g(base.device());
    rb_tile_forward(base.data_ptr(), base_dtype, opt_i32(rows), rev.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(), opt_f32(weights), n_seg, D,
                    (int)tile_len, out.data_ptr<float>(), gp, gs, cur_stream());
  } else {
    rbc_tile_forward(base.data_ptr(), base_dtype, opt_i32(rows), rev.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(), opt_f32(weights), n_seg,
                     D, (int)tile_len, out.data_ptr<float>(), gp, gs);
  }
  return {out, gsrc, gscale};
}

}  // namespace

namespace rbx {
// reverse index -> (csr_u, csr_elem, start): elements grouped by unique index, stable in element order.
std::tuple<Tensor, Tensor, Tensor> build_csr(const Tensor& reverse) {
  TORCH_CHECK(reverse.scalar_type() == torch::kInt32 && reverse.is_contiguous());
  const int64_t n = reverse.numel();
  auto o = reverse.options();
  auto csr_u = torch::empty({n}, o), csr_elem = torch::empty({n}, o), start = torch::empty({n + 1}, o);
  if (n == 0) return {csr_u, csr_elem, start};
  if (reverse.is_cuda()) {
    c10::cuda::CUDAGuard g(reverse.device());
    int bits = 1; while ((1ll << bits) < n && bits < 31) ++bits;  // unique indices are < n
    const size_t tb = rb_sort_temp_bytes(n);
    auto temp = torch::empty({(int64_t)tb}, o.dtype(torch::kUInt8));
    auto iota = torch::empty({n}, o);
    rb_build_csr(reverse.data_ptr<int32_t>(), n, bits, temp.data_ptr(), tb, iota.data_ptr<int32_t>(), csr_u.data_ptr<int32_t>(),
                 csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), cur_stream());
  } else {
    rbc_build_csr(reverse.data_ptr<int32_t>(), n, csr_u.data_ptr<int32_t>(), csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>());
  }
  return {csr_u, csr_elem, start};
}
}  // namespace rbx

namespace {
using rbx::build_csr;

using rbx::make_opt;

// Per-unique gradient reduction. apply=false: returns gu [n_unique_max, D] (rows beyond the unique count are undefined).
// apply=true: runs the optimizer on row rows[u] of (w, s1, s2) in the same kernel and returns an empty tensor.
Tensor grad_reduce(const Tensor& grad_out, const Tensor& gsrc, const Tensor& gscale, const Tensor& csr_u, const Tensor& csr_elem,
                   const Tensor& start, int64_t D, OptT rows, bool apply, int64_t kind, double lr, double beta1, double beta2, double eps,
                   double decay, double alpha, double grad_scale, OptT w, OptT s1, OptT s2, int64_t n_unique_max, OptT gu_out) {
  TORCH_CHECK(grad_out.is_contiguous() && grad_out.scalar_type() == torch::kFloat32, "grad_out must be contiguous fp32");
  const int64_t n = csr_u.numel();
  RbOpt opt = make_opt(kind, lr, beta1, beta2, eps, decay, alpha, grad_scale, w, s1, s2);
  if (apply) TORCH_CHECK(opt.w != nullptr, "apply needs the weight slab");
  Tensor gu = apply ? Tensor() : (gu_out.has_value() && gu_out->defined() ? *gu_out : torch::zeros({n_unique_max, D}, grad_out.options()));
  float* gup = apply ? nullptr : gu.data_ptr<float>();
  if (n == 0) return gu;
  if (grad_out.is_cuda()) {
    c10::cuda::CUDAGuard g(grad_out.device());
    const int64_t n_chunks = (n + rb_grad_reduce_chunk() - 1) / rb_grad_reduce_chunk();
    auto span = torch::zeros({n_chunks, D}, grad_out.options());
    rb_grad_reduce(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                   csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), n, (int)D, span.data_ptr<float>(), opt_i32(rows), gup,
                   apply ? 1 : 0, opt, cur_stream());
  } else {
    rbc_grad_reduce(grad_out.data_ptr<float>(), gsrc.data_ptr<int32_t>(), gscale.data_ptr<float>(), csr_u.data_ptr<int32_t>(),
                    csr_elem.data_ptr<int32_t>(), start.data_ptr<int32_t>(), n, (int)D, opt_i32(rows), gup, apply ? 1 : 0, opt);
  }
  return gu;
}

void sparse_apply(const Tensor& rows, const Tensor& grads, OptT n_dev, int64_t kind, double lr, double beta1, double beta2, double eps,
                  double decay, double alpha, double grad_scale, Tensor w, OptT s1, OptT s2) {
  TORCH_CHECK(rows.scalar_type() == torch::kInt32 && grads.is_contiguous() && grads.scalar_type() == torch::kFloat32);
  const int64_t n = rows.numel(); const int D = (int)w.size(1);
  if (n == 0) return;
  rbx::debug_check_range("sparse_apply: rows", rbx::debug_prefix(rows, n_dev), -1, w.size(0));
  RbOpt opt = make_opt(kind, lr, beta1, beta2, eps, decay, alpha, grad_scale, w, s1, s2);
  if (w.is_cuda()) {
    c10::cuda::CUDAGuard g(w.device());
    rb_sparse_apply(rows.data_ptr<int32_t>(), grads.data_ptr<float>(), n, opt_i32(n_dev), D, opt, cur_stream());
  } else {
    rbc_sparse_apply(rows.data_ptr<int32_t>(), grads.data_ptr<float>(), n, opt_i32(n_dev), D, opt);
  }
}

}  // namespace

void init_sparse(py::module& m) {
  using rbx::EmbeddingStore;
  py::class_<EmbeddingStore, std::shared_ptr<EmbeddingStore>>(m, "EmbeddingStore")
      .def(py::init([](int64_t dim, int64_t capacity, const std::string& device, int init_kind, double a, double b, double lo, double hi,
                       int64_t seed, bool track_last_seen, bool growable, OptT emb_storage, py::object emb_dtype) {
             const torch::ScalarType dt = emb_dtype.is_none() ? torch::kFloat32 : torch::python::detail::py_object_to_dtype(emb_dtype);
             return std::make_shared<EmbeddingStore>(dim, capacity, torch::Device(device), init_kind, a, b, lo, hi, seed, track_last_seen,
                                                     growable, emb_storage, dt);
           }),
           py::arg("dim"), py::arg("capacity"), py::arg("device"), py::arg("init_kind"), py::arg("a"), py::arg("b"), py::arg("lo"),
           py::arg("hi"), py::arg("seed"), py::arg("track_last_seen") = true, py::arg("growable") = true,
           py::arg("emb_storage") = py::none(), py::arg("emb_dtype") = py::none())
      .def("lookup_or_insert", &EmbeddingStore::lookup_or_insert, py::arg("ids"), py::arg("n_dev") = py::none(),
           py::arg("step") = py::none(), py::arg("admit_threshold") = 1, py::arg("ids_unique") = false)
      .def("find", &EmbeddingStore::find, py::arg("ids"), py::arg("n_dev") = py::none())
      .def("erase", &EmbeddingStore::erase)
      .def("snapshot", &EmbeddingStore::snapshot, py::arg("expired_only") = false, py::arg("threshold") = 0)
      .def("add_slot", &EmbeddingStore::add_slot, py::arg("name"), py::arg("fill") = 0.0)
      .def("slot", &EmbeddingStore::slot)
      .def("has_slot", &EmbeddingStore::has_slot)
      .def("slot_names", &EmbeddingStore::slot_names)
      .def("emb", &EmbeddingStore::emb)
      .def("last_seen", &EmbeddingStore::last_seen)
      .def("keys", &EmbeddingStore::keys)
      .def("index_rows", &EmbeddingStore::index_rows)
      .def("ctr", &EmbeddingStore::ctr)
      .def("free_list", &EmbeddingStore::free_list)
      .def("counters", &EmbeddingStore::counters)
      .def("reserve", &EmbeddingStore::reserve)
      .def("grows_in_place", &EmbeddingStore::grows_in_place)
      .def("rebuild_index", &EmbeddingStore::rebuild_index)
      .def("clear", &EmbeddingStore::clear)
      .def("size", &EmbeddingStore::size)
      .def("capacity", &EmbeddingStore::capacity)
      .def("dim", &EmbeddingStore::dim)
      .def("set_name", &EmbeddingStore::set_name);

  m.def("dedup_partition", &dedup_partition, py::arg("ids"), py::arg("world"), py::arg("unique_out") = py::none(),
        py::arg("offsets_out") = py::none(), py::arg("status") = py::none(), py::arg("counts_out") = py::none());
  m.def("encode_merge", &encode_merge);
  m.def("coalesce_lanes", &coalesce_lanes);
  m.def("gather_rows", &gather_rows, py::arg("src"), py::arg("rows"), py::arg("n_dev") = py::none());
  m.def("scatter_rows", &scatter_rows);
  m.def("fill_rows_i64", &fill_rows_i64);
  m.def("pool_forward", &pool_forward, py::arg("base"), py::arg("rows"), py::arg("rev"), py::arg("offsets"), py::arg("weights"),
        py::arg("mode"), py::arg("perm_b"), py::arg("perm_f"), py::arg("need_grad"), py::arg("out") = py::none(),
        py::arg("perm_off") = 0, py::arg("perm_total") = 0);
  m.def("tile_forward", &tile_forward);
  m.def("build_csr", &build_csr);
  m.def("grad_reduce", &grad_reduce, py::arg("grad_out"), py::arg("gsrc"), py::arg("gscale"), py::arg("csr_u"), py::arg("csr_elem"), py::arg("start"),
        py::arg("D"), py::arg("rows"), py::arg("apply"), py::arg("kind"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"),
        py::arg("decay"), py::arg("alpha"), py::arg("grad_scale"), py::arg("w"), py::arg("s1"), py::arg("s2"), py::arg("n_unique_max"),
        py::arg("gu_out") = py::none());
  m.def("sparse_apply", &sparse_apply);
  m.def("grad_reduce_chunk", []() { return rb_grad_reduce_chunk(); });
  m.def("launch_count", []() { return rb_launch_count(); });
}
