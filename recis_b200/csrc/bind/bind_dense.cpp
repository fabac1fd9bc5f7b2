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
  }
  int splits = 1;
  if (out_fp32 && !relu && !(bias.has_value() && bias->defined())) splits = rb_gemm_splits((int)MM, (int)NN, (int)KK);
  if (!out.defined())
    out = splits > 1 ? torch::zeros({MM, NN}, a.options().dtype(torch::kFloat32))
                     : torch::empty({MM, NN}, a.options().dtype(out_fp32 ? torch::kFloat32 : torch::kBFloat16));
  if (splits > 1) beta = nullptr;   // accumulate_into + split-K: the reductions land directly on the existing values
  const float* bp = nullptr;
  Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->scalar_type() == torch::kFloat32 ? bias->contiguous() : bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == NN);
    bp = bias_f.data_ptr<float>();
  }
  Tensor& st = status_word(a.device());
  const int rc = rb_gemm_bf16(a.data_ptr(), a.stride(0), a_mn, b.data_ptr(), b.stride(0), b_mn, out.data_ptr(), out.stride(0), out_fp32, bp,
                              beta, (int)MM, (int)NN, (int)KK, relu, splits, st.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "rb_gemm_bf16 failed with code ", rc,
              " (1: operand base/pitch not 16-byte aligned, 2: tensor map encode failed, >2: launch error)");
  return out;
}

// [x | strict lower triangle of Z Z^T | 0 pad]; Z = [x; cube]. out_cols = padded width (multiple of 8).
Tensor dot_interaction_fwd(const Tensor& x, const Tensor& cube, int64_t out_cols) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && cube.scalar_type() == torch::kFloat32 &&
              cube.is_contiguous() && cube.dim() == 3);
  const int B = (int)cube.size(0), F = (int)cube.size(1), D = (int)cube.size(2);
  TORCH_CHECK(x.size(0) == B && x.size(1) == D && out_cols >= D + (F + 1) * F / 2);
  c10::cuda::CUDAGuard g(x.device());
  auto out = torch::empty({B, out_cols}, x.options());
  // tensor-core kernel when the shape allows (at most 31 fields, width 64 or 128), SIMT kernel otherwise
  int rc = rb_dot_interaction_tc_fwd(x.data_ptr(), cube.data_ptr<float>(), B, F, D, (int)out_cols, out.data_ptr(),
                                     status_word(x.device()).data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  if (rc == 1)
    rc = rb_dot_interaction_fwd(x.data_ptr(), cube.data_ptr<float>(), B, F, D, (int)out_cols, out.data_ptr(),
                                at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "dot_interaction: too many fields or too wide for shared memory (code ", rc, ")");
  return out;
}

std::tuple<Tensor, Tensor> dot_interaction_bwd(const Tensor& x, const Tensor& cube, const Tensor& dout) {
  const int B = (int)cube.size(0), F = (int)cube.size(1), D = (int)cube.size(2);
  TORCH_CHECK(dout.scalar_type() == torch::kBFloat16 && dout.is_contiguous() && dout.size(0) == B);
  c10::cuda::CUDAGuard g(x.device());
  auto dx = torch::empty({B, D}, cube.options());
  auto dcube = torch::empty_like(cube);
  int rc = rb_dot_interaction_tc_bwd(x.data_ptr(), cube.data_ptr<float>(), dout.data_ptr(), B, F, D, (int)dout.size(1),
                                     dx.data_ptr<float>(), dcube.data_ptr<float>(), status_word(x.device()).data_ptr<int64_t>(),
                                     at::cuda::getCurrentCUDAStream());
  if (rc == 1)
    rc = rb_dot_interaction_bwd(x.data_ptr(), cube.data_ptr<float>(), dout.data_ptr(), B, F, D, (int)dout.size(1),
                                dx.data_ptr<float>(), dcube.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "dot_interaction backward failed (code ", rc, ")");
  return {dx, dcube};
}

Tensor fm_fwd(const Tensor& cube) {
  TORCH_CHECK(cube.is_cuda() && cube.scalar_type() == torch::kFloat32 && cube.is_contiguous() && cube.dim() == 3);
  c10::cuda::CUDAGuard g(cube.device());
  auto out = torch::empty({cube.size(0), 1}, cube.options());
  rb_fm_fwd(cube.data_ptr<float>(), (int)cube.size(0), (int)cube.size(1), (int)cube.size(2), out.data_ptr<float>(),
            at::cuda::getCurrentCUDAStream());
  return out;
}

Tensor fm_bwd(const Tensor& cube, const Tensor& gout) {
  c10::cuda::CUDAGuard g(cube.device());
  auto go = gout.contiguous().to(torch::kFloat32);
  auto dcube = torch::empty_like(cube);
  rb_fm_bwd(cube.data_ptr<float>(), go.data_ptr<float>(), (int)cube.size(0), (int)cube.size(1), (int)cube.size(2), dcube.data_ptr<float>(),
            at::cuda::getCurrentCUDAStream());
  return dcube;
}

// returns (dy bf16 [M, N], db fp32 [N])
std::tuple<Tensor, Tensor> relu_bwd_bias(const Tensor& y, const Tensor& dout, bool relu, OptT db_out = c10::nullopt) {
  TORCH_CHECK(dout.is_cuda() && dout.scalar_type() == torch::kBFloat16 && dout.is_contiguous() && dout.dim() == 2);
  TORCH_CHECK(!relu || (y.scalar_type() == torch::kBFloat16 && y.is_contiguous() && y.sizes() == dout.sizes()));
  c10::cuda::CUDAGuard g(dout.device());
  const int M = (int)dout.size(0), N = (int)dout.size(1);
  Tensor dy = relu ? torch::empty_like(dout) : dout;
  // db_out: a zeroed fp32 [N] to add the column sums to (a caller that batches its zero-fills); else a fresh one
  auto db = db_out.has_value() && db_out->defined() ? *db_out : torch::zeros({N}, dout.options().dtype(torch::kFloat32));
  if (rb_relu_bwd_bias_vec(relu ? y.data_ptr() : nullptr, dout.data_ptr(), M, N, relu, relu ? dy.data_ptr() : nullptr, db.data_ptr<float>(),
                           at::cuda::getCurrentCUDAStream()) == 1)
    rb_relu_bwd_bias(relu ? y.data_ptr() : nullptr, dout.data_ptr(), M, N, relu, relu ? dy.data_ptr() : nullptr, db.data_ptr<float>(),
                     at::cuda::getCurrentCUDAStream());
  return {dy, db};
}

Tensor cast_pad_bf16(const Tensor& src, int64_t rows_p, int64_t cols_p) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1);
  c10::cuda::CUDAGuard g(src.device());
  auto dst = torch::empty({rows_p, cols_p}, src.options().dtype(torch::kBFloat16));
  rb_cast_pad_bf16(src.data_ptr<float>(), (int)src.size(0), (int)src.size(1), (int)src.stride(0), dst.data_ptr(), (int)rows_p, (int)cols_p,
                   at::cuda::getCurrentCUDAStream());
  return dst;
}

inline int64_t pad8(int64_t n) { return (n + 7) / 8 * 8; }

// Whole MLP forward in one call: per layer cast+pad the fp32 master weight to bf16, then GEMM with fused bias (+ReLU).
// x: [M, K0] any float dtype (cast / zero-padded to bf16 [M, pad8(K0)] here). Returns (padded bf16 input, layer outputs, bf16 weights).
// wb_cached: empty, or per layer an up-to-date bf16 copy [pad8(N), pad8(K)] of the weight (kept by the caller across steps and
// rewritten by the dense optimizer) that replaces the cast.
std::tuple<Tensor, std::vector<Tensor>, std::vector<Tensor>> mlp_forward(const Tensor& x_in, const std::vector<Tensor>& weights,
                                                                         const std::vector<Tensor>& biases, const std::vector<bool>& relu,
                                                                         const std::vector<c10::optional<Tensor>>& wb_cached) {
  TORCH_CHECK(x_in.is_cuda() && x_in.dim() == 2 && weights.size() == biases.size() && weights.size() == relu.size());
  TORCH_CHECK(wb_cached.empty() || wb_cached.size() == weights.size(), "wb_cached must be empty or hold one entry per layer");
  c10::cuda::CUDAGuard g(x_in.device());
  const int64_t K0p = pad8(weights[0].size(1));
  Tensor x = x_in.scalar_type() == torch::kBFloat16 ? x_in : x_in.to(torch::kBFloat16);
  if (x.size(1) != K0p) x = torch::constant_pad_nd(x, {0, K0p - x.size(1)});
  x = x.contiguous();
  std::vector<Tensor> ys, wbs;
  Tensor h = x;
  for (size_t l = 0; l < weights.size(); ++l) {
    const int64_t N = weights[l].size(0), K = weights[l].size(1), Np = pad8(N), Kp = pad8(K);
    TORCH_CHECK(h.size(1) == Kp, "layer ", l, ": input width ", h.size(1), " does not match the padded weight width ", Kp);
    Tensor wb;
    if (!wb_cached.empty() && wb_cached[l].has_value() && wb_cached[l]->defined()) {
      wb = *wb_cached[l];
      TORCH_CHECK(wb.scalar_type() == torch::kBFloat16 && wb.is_contiguous() && wb.dim() == 2 && wb.size(0) == Np && wb.size(1) == Kp &&
                      wb.device() == x.device(), "layer ", l, ": the cached bf16 weight must be contiguous [", Np, ", ", Kp, "]");
    } else {
      wb = cast_pad_bf16(weights[l], Np, Kp);
    }
    Tensor bp = Np == N ? biases[l] : torch::constant_pad_nd(biases[l], {0, Np - N});
    h = gemm_bf16(h, wb, bp, relu[l], false, false, false, c10::nullopt);
    ys.push_back(h); wbs.push_back(wb);
  }
  return {x, ys, wbs};
}

// (dx bf16 [M, K], column sums of dx fp32 [K]) with dx = (dy [M, N] . W [N, K]) set to zero where mask [M, K] <= 0: the input gradient
// of a layer, already passed through the ReLU of the layer below, and that layer's bias gradient, all in the GEMM's epilogue.
std::tuple<Tensor, Tensor> gemm_dgrad_fused(const Tensor& dy, const Tensor& w, OptT mask, OptT db_out = c10::nullopt) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16 && dy.dim() == 2 && w.dim() == 2 &&
              dy.stride(1) == 1 && w.stride(1) == 1 && dy.size(1) == w.size(0), "bf16 dy [M, N] and W [N, K] expected");
  const int64_t MM = dy.size(0), KK = dy.size(1), NN = w.size(1);
  c10::cuda::CUDAGuard g(dy.device());
  auto out = torch::empty({MM, NN}, dy.options());
  auto db = db_out.has_value() && db_out->defined() ? *db_out : torch::zeros({NN}, dy.options().dtype(torch::kFloat32));
  TORCH_CHECK(db.scalar_type() == torch::kFloat32 && db.is_contiguous() && db.numel() == NN, "db_out: contiguous fp32 [K]");
  RbGemmEpilogue epi{nullptr, 0, db.data_ptr<float>()};
  if (mask.has_value() && mask->defined()) {
    TORCH_CHECK(mask->scalar_type() == torch::kBFloat16 && mask->dim() == 2 && mask->stride(1) == 1 && mask->size(0) == MM && mask->size(1) == NN,
                "mask: bf16 [M, K]");
    epi.mask_src = mask->data_ptr();
    epi.mask_ld = mask->stride(0);
  }
  Tensor& st = status_word(dy.device());
  const int rc = rb_gemm_bf16_ex(dy.data_ptr(), dy.stride(0), 0, w.data_ptr(), w.stride(0), 1, out.data_ptr(), out.stride(0), 0, nullptr, nullptr,
                                 &epi, (int)MM, (int)NN, (int)KK, 0, 1, st.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "rb_gemm_bf16_ex failed with code ", rc);
  return {out, db};
}

// Whole MLP backward in one call. dout: bf16 [M, pad8(N_last)]. Returns (dx or undefined, weight grads fp32 [N, K], bias grads fp32 [N]).
std::tuple<Tensor, std::vector<Tensor>, std::vector<Tensor>> mlp_backward(const Tensor& dout_in, const Tensor& x, const std::vector<Tensor>& ys,
                                                                          const std::vector<Tensor>& wbs, const std::vector<bool>& relu,
                                                                          const std::vector<std::vector<int64_t>>& shapes, bool need_dx) {
  c10::cuda::CUDAGuard g(x.device());
  const int L = (int)ys.size();
  std::vector<Tensor> dws(L), dbs(L);
  Tensor dout = dout_in.contiguous();
  Tensor dx;
  // The last layer's pre-activation gradient comes from one element-wise kernel; below it, every layer's comes out of the GEMM
  // above it: dy_{l-1} = (dy_l W_l) with the ReLU mask of y_{l-1} applied and its column sums (the bias gradient) taken in the
  // epilogue, so a layer costs two GEMMs and nothing else.
  // Weight gradients (split reductions add into their output) and bias gradients (column sums are added) all start from zero:
  // one buffer, one fill for the whole call, instead of two per layer.
  std::vector<int64_t> w_off(L), b_off(L);
  int64_t total = 0;
  auto up64 = [](int64_t n) { return (n + 63) / 64 * 64; };          // every piece starts 256-byte aligned
  for (int l = 0; l < L; ++l) {
    w_off[l] = total; total += up64(wbs[l].size(0) * wbs[l].size(1));
    b_off[l] = total; total += up64(wbs[l].size(0));
  }
  Tensor zero = torch::zeros({total}, x.options().dtype(torch::kFloat32));
  auto dw_view = [&](int l) { return zero.narrow(0, w_off[l], wbs[l].size(0) * wbs[l].size(1)).view({wbs[l].size(0), wbs[l].size(1)}); };
  auto db_view = [&](int l) { return zero.narrow(0, b_off[l], wbs[l].size(0)); };
  Tensor dy, db;
  std::tie(dy, db) = relu_bwd_bias(ys[L - 1], dout, relu[L - 1], db_view(L - 1));
  for (int l = L - 1; l >= 0; --l) {
    const Tensor& h_in = l == 0 ? x : ys[l - 1];
    Tensor dw = gemm_bf16(dy, h_in, c10::nullopt, false, true, true, true, dw_view(l));   // dy^T . h  (both MN-major, split-K)
    dws[l] = dw.narrow(0, 0, shapes[l][0]).narrow(1, 0, shapes[l][1]);
    dbs[l] = db.narrow(0, 0, shapes[l][0]);
    if (l > 0) {
      std::tie(dy, db) = gemm_dgrad_fused(dy, wbs[l], relu[l - 1] ? c10::optional<Tensor>(ys[l - 1]) : c10::nullopt, db_view(l - 1));
    } else if (need_dx) {
      dx = gemm_bf16(dy, wbs[0], c10::nullopt, false, false, true, false, c10::nullopt);    // dy . W  (W read MN-major)
    }
  }
  return {dx, dws, dbs};
}

// out (fp32) = a b^T + bias + residual: a projection added onto the fp32 residual stream in the GEMM's epilogue
Tensor gemm_bf16_residual(const Tensor& a, const Tensor& b, OptT bias, const Tensor& residual) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16 && a.dim() == 2 && b.dim() == 2 &&
              a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1), "bf16 [M, K] and [N, K] operands expected");
  const int64_t MM = a.size(0), NN = b.size(0), KK = a.size(1);
  TORCH_CHECK(residual.scalar_type() == torch::kFloat32 && residual.is_contiguous() && residual.dim() == 2 && residual.size(0) == MM &&
              residual.size(1) == NN, "residual: contiguous fp32 [M, N]");
  c10::cuda::CUDAGuard g(a.device());
  auto out = torch::empty({MM, NN}, a.options().dtype(torch::kFloat32));
  const float* bp = nullptr;
  Tensor bias_f;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->scalar_type() == torch::kFloat32 ? bias->contiguous() : bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == NN);
    bp = bias_f.data_ptr<float>();
  }
  Tensor& st = status_word(a.device());
  const int rc = rb_gemm_bf16(a.data_ptr(), a.stride(0), 0, b.data_ptr(), b.stride(0), 0, out.data_ptr(), out.stride(0), 1, bp,
                              residual.data_ptr<float>(), (int)MM, (int)NN, (int)KK, 0, 1, st.data_ptr<int64_t>(),
                              at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "rb_gemm_bf16 failed with code ", rc);
  return out;
}

// (y [rows, H] bf16 or fp32, stats [rows, 2] = mean and rstd)
std::tuple<Tensor, Tensor> layer_norm_fwd(const Tensor& x, const Tensor& gamma, const Tensor& beta, double eps, bool out_bf16) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.is_contiguous() && x.dim() == 2, "x: contiguous fp32 [rows, hidden] on CUDA");
  const int64_t rows = x.size(0), H = x.size(1);
  TORCH_CHECK(gamma.scalar_type() == torch::kFloat32 && beta.scalar_type() == torch::kFloat32 && gamma.is_contiguous() && beta.is_contiguous() &&
              gamma.numel() == H && beta.numel() == H, "gamma, beta: contiguous fp32 [hidden]");
  c10::cuda::CUDAGuard g(x.device());
  auto y = torch::empty({rows, H}, x.options().dtype(out_bf16 ? torch::kBFloat16 : torch::kFloat32));
  auto stats = torch::empty({rows, 2}, x.options());
  const int rc = rb_layer_norm_fwd(x.data_ptr<float>(), gamma.data_ptr<float>(), beta.data_ptr<float>(), rows, (int)H, (float)eps, y.data_ptr(),
                                   out_bf16, stats.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "layer_norm: hidden width must be a multiple of 4 and at most 1024");
  return {y, stats};
}

// (dx fp32 [rows, H], dgamma [H], dbeta [H])
std::tuple<Tensor, Tensor, Tensor> layer_norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& stats, const Tensor& gamma) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.sizes() == x.sizes() &&
              (dy.scalar_type() == torch::kFloat32 || dy.scalar_type() == torch::kBFloat16), "dy: contiguous fp32 or bf16, shaped like x");
  c10::cuda::CUDAGuard g(x.device());
  const int64_t rows = x.size(0), H = x.size(1);
  auto dx = torch::empty_like(x);
  auto dgb = torch::zeros({2, H}, x.options());
  const int rc = rb_layer_norm_bwd(dy.data_ptr(), dy.scalar_type() == torch::kBFloat16, x.data_ptr<float>(), stats.data_ptr<float>(),
                                   gamma.data_ptr<float>(), rows, (int)H, dx.data_ptr<float>(), dgb.data_ptr<float>(),
                                   dgb.data_ptr<float>() + H, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "layer_norm backward: hidden width must be a multiple of 4 and at most 1024");
  return {dx, dgb.select(0, 0), dgb.select(0, 1)};
}

// (interest [B, H], lse [B]) of the target attention over packed sequences
std::tuple<Tensor, Tensor> target_attention_fwd(const Tensor& x, const Tensor& q, const Tensor& offsets, double scale) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.is_contiguous() && x.dim() == 2, "x: contiguous fp32 [tokens, hidden] on CUDA");
  TORCH_CHECK(q.scalar_type() == torch::kFloat32 && q.is_contiguous() && q.dim() == 2 && q.size(1) == x.size(1), "q: contiguous fp32 [batch, hidden]");
  TORCH_CHECK(offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous() && offsets.numel() == q.size(0) + 1, "offsets: int32 [batch + 1]");
  c10::cuda::CUDAGuard g(x.device());
  const int B = (int)q.size(0), H = (int)q.size(1);
  auto interest = torch::empty({B, H}, x.options());
  auto lse = torch::empty({B}, x.options());
  const int rc = rb_target_attention_fwd(x.data_ptr<float>(), q.data_ptr<float>(), offsets.data_ptr<int32_t>(), B, H, (float)scale,
                                         interest.data_ptr<float>(), lse.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "target_attention: hidden width must be a multiple of 4 and at most 1024");
  return {interest, lse};
}

// (dx [T, H], dq [B, H])
std::tuple<Tensor, Tensor> target_attention_bwd(const Tensor& x, const Tensor& q, const Tensor& offsets, const Tensor& interest, const Tensor& lse,
                                                const Tensor& d_interest, double scale) {
  TORCH_CHECK(d_interest.scalar_type() == torch::kFloat32 && d_interest.is_contiguous() && d_interest.sizes() == interest.sizes());
  c10::cuda::CUDAGuard g(x.device());
  const int B = (int)q.size(0), H = (int)q.size(1);
  auto dx = torch::zeros_like(x);          // tokens outside every sequence (none in a well-formed batch) keep a zero gradient
  auto dq = torch::empty_like(q);
  const int rc = rb_target_attention_bwd(x.data_ptr<float>(), q.data_ptr<float>(), offsets.data_ptr<int32_t>(), interest.data_ptr<float>(),
                                         lse.data_ptr<float>(), d_interest.data_ptr<float>(), B, H, (float)scale, dx.data_ptr<float>(),
                                         dq.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(rc == 0, "target_attention backward: hidden width must be a multiple of 4 and at most 1024");
  return {dx, dq};
}

int64_t dense_status(const std::string& device) { return status_word(torch::Device(device)).item<int64_t>(); }

}  // namespace

void init_dense(py::module& m) {
  m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("bias") = py::none(), py::arg("relu") = false,
        py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("out_fp32") = false, py::arg("accumulate_into") = py::none());
  m.def("dense_status", &dense_status);
  m.def("gemm_bf16_residual", &gemm_bf16_residual);
  m.def("gemm_dgrad_fused", &gemm_dgrad_fused, py::arg("dy"), py::arg("w"), py::arg("mask"), py::arg("db_out") = c10::nullopt);
  m.def("layer_norm_fwd", &layer_norm_fwd);
  m.def("layer_norm_bwd", &layer_norm_bwd);
  m.def("target_attention_fwd", &target_attention_fwd);
  m.def("target_attention_bwd", &target_attention_bwd);
  m.def("mlp_forward", &mlp_forward, py::arg("x"), py::arg("weights"), py::arg("biases"), py::arg("relu"),
        py::arg("wb_cached") = std::vector<c10::optional<Tensor>>());
  m.def("mlp_backward", &mlp_backward);
  m.def("dot_interaction_fwd", &dot_interaction_fwd);
  m.def("dot_interaction_bwd", &dot_interaction_bwd);
  m.def("fm_fwd", &fm_fwd);
  m.def("fm_bwd", &fm_bwd);
  m.def("relu_bwd_bias", &relu_bwd_bias, py::arg("y"), py::arg("dout"), py::arg("relu"), py::arg("db_out") = c10::nullopt);
  m.def("cast_pad_bf16", &cast_pad_bf16);
  // Ragged self-attention forward on the tensor cores (head width 64): returns (out bf16 [T, H * 64], lse2 fp32 [T, H]).
  m.def("ragged_attention_fwd", [](const Tensor& qkv, const Tensor& offsets, int64_t H, int64_t max_len, double scale) {
    TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.is_contiguous() && qkv.dim() == 2 &&
                    qkv.size(1) == 3 * H * 64, "qkv: contiguous bf16 [T, 3 * H * 64] on CUDA");
    TORCH_CHECK(offsets.is_cuda() && offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous() && offsets.numel() >= 2);
    c10::cuda::CUDAGuard g(qkv.device());
    const int64_t T = qkv.size(0), B = offsets.numel() - 1;
    auto out = torch::zeros({T, H * 64}, qkv.options());
    auto lse = torch::zeros({T, H}, qkv.options().dtype(torch::kFloat32));
    const int rc = rb_ragged_attention_fwd(qkv.data_ptr(), offsets.data_ptr<int32_t>(), T, (int)B, (int)H, (int)max_len, (float)scale,
                                           out.data_ptr(), lse.data_ptr<float>(), status_word(qkv.device()).data_ptr<int64_t>(),
                                           at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "ragged_attention_fwd failed (code ", rc, ")");
    return std::make_tuple(out, lse);
  });
  // Backward of the above: returns dqkv fp32 [T, 3 * H * 64].
  m.def("ragged_attention_bwd", [](const Tensor& qkv, const Tensor& out, const Tensor& d_out, const Tensor& lse, const Tensor& offsets,
                                   int64_t H, int64_t max_len, double scale) {
    TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == torch::kBFloat16 && qkv.is_contiguous() && qkv.size(1) == 3 * H * 64);
    TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && d_out.scalar_type() == torch::kBFloat16 &&
                d_out.is_contiguous() && out.sizes() == d_out.sizes() && out.size(0) == qkv.size(0) && out.size(1) == H * 64);
    TORCH_CHECK(lse.scalar_type() == torch::kFloat32 && lse.is_contiguous() && lse.numel() == qkv.size(0) * H);
    c10::cuda::CUDAGuard g(qkv.device());
    const int64_t T = qkv.size(0), B = offsets.numel() - 1;
    auto dqkv = torch::zeros({T, 3 * H * 64}, qkv.options().dtype(torch::kFloat32));
    auto delta = torch::empty({T, H}, dqkv.options());
    const int rc = rb_ragged_attention_bwd(qkv.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                                           offsets.data_ptr<int32_t>(), T, (int)B, (int)H, (int)max_len, (float)scale,
                                           dqkv.data_ptr<float>(), status_word(qkv.device()).data_ptr<int64_t>(),
                                           at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "ragged_attention_bwd failed (code ", rc, ")");
    return dqkv;
  });
  // Multi-tensor dense Adam (see rb_dense.h for the update rule); ws/gs/ms/vs are parallel lists of fp32 CUDA tensors,
  // w_bf16 an optional parallel list (entries may be undefined) of bf16 shadows that receive the rounded weights.
  m.def("dense_adam", [](std::vector<Tensor> ws, std::vector<Tensor> gs, std::vector<Tensor> ms, std::vector<Tensor> vs,
                         std::vector<c10::optional<Tensor>> w_bf16, double beta1, double beta2, double eps, double decay,
                         double step_size, double inv_sqrt_bc2, double l2) {
    TORCH_CHECK(ws.size() == gs.size() && ws.size() == ms.size() && ws.size() == vs.size(), "parallel lists differ in length");
    TORCH_CHECK(w_bf16.empty() || w_bf16.size() == ws.size(), "w_bf16 must be empty or parallel to the weights");
    if (ws.empty()) return;
    c10::cuda::CUDAGuard guard(ws[0].device());
    for (size_t i0 = 0; i0 < ws.size(); i0 += RB_DENSE_ADAM_MAX) {
      RbDenseAdamArgs a{};
      a.count = (int)std::min<size_t>(RB_DENSE_ADAM_MAX, ws.size() - i0);
      for (int k = 0; k < a.count; ++k) {
        const Tensor &w = ws[i0 + k], &g = gs[i0 + k], &mm = ms[i0 + k], &vv = vs[i0 + k];
        TORCH_CHECK(w.is_cuda() && w.scalar_type() == torch::kFloat32 && w.is_contiguous() && g.is_contiguous() && mm.is_contiguous() &&
                        vv.is_contiguous() && g.scalar_type() == torch::kFloat32 && g.numel() == w.numel() && mm.numel() == w.numel() &&
                        vv.numel() == w.numel(),
                    "dense_adam wants contiguous fp32 CUDA tensors of equal size");
        a.w[k] = w.data_ptr<float>(); a.g[k] = g.data_ptr<float>(); a.m[k] = mm.data_ptr<float>(); a.v[k] = vv.data_ptr<float>();
        a.n[k] = w.numel();
        a.w_bf16[k] = nullptr;
        a.cols[k] = 0; a.bf16_ld[k] = 0;
        if (!w_bf16.empty() && w_bf16[i0 + k].has_value() && w_bf16[i0 + k]->defined()) {
          const Tensor& wb = *w_bf16[i0 + k];
          TORCH_CHECK(wb.scalar_type() == torch::kBFloat16 && wb.is_contiguous(), "the bf16 copy must be contiguous bf16");
          if (wb.numel() != w.numel()) {
            // a copy padded for the GEMM: [rows_padded, cols_padded] of a 2-D weight [rows, cols]; the padding stays zero
            TORCH_CHECK(w.dim() == 2 && wb.dim() == 2 && wb.size(0) >= w.size(0) && wb.size(1) >= w.size(1), "bf16 copy: shape ", wb.sizes(),
                        " cannot hold the weight ", w.sizes());
            a.cols[k] = (int32_t)w.size(1);
            a.bf16_ld[k] = (int32_t)wb.size(1);
          }
          a.w_bf16[k] = wb.data_ptr();
        }
      }
      rb_dense_adam(&a, (float)beta1, (float)beta2, (float)eps, (float)decay, (float)step_size, (float)inv_sqrt_bc2, (float)l2,
                    at::cuda::getCurrentCUDAStream());
    }
  });
}
