// Grouped AUC on the host (role of the reference's csrc/ops/gauc.cc:16-123).
// Samples arrive sorted by group (`indicators`); every maximal run of equal indicators is one group. A group contributes
// its AUC (trapezoid over the prediction-sorted samples, ties in arrival order) weighted by its size when it contains both
// classes. Unlike the reference loop, the first and the last group are evaluated too.
#include <torch/extension.h>
#include <algorithm>
#include <numeric>
#include <vector>

namespace py = pybind11;
using torch::Tensor;

namespace {

// labels / predictions: [n] (probability of the positive class) or [n, 2] (negative, positive); indicators: [n] integers.
std::tuple<Tensor, Tensor> gauc_calc(const Tensor& labels_in, const Tensor& preds_in, const Tensor& indicators_in) {
  auto labels = labels_in.to(torch::kCPU, torch::kFloat64).contiguous();
  auto preds = preds_in.to(torch::kCPU, torch::kFloat64).contiguous();
  auto ind = indicators_in.to(torch::kCPU, torch::kInt64).contiguous();
  TORCH_CHECK(ind.dim() == 1 && (labels.dim() == 1 || (labels.dim() == 2 && labels.size(1) == 2)) && labels.sizes() == preds.sizes());
  const int64_t n = labels.size(0);
  const int dim = (int)labels.dim();
  const double* pl = labels.data_ptr<double>(); const double* pp = preds.data_ptr<double>(); const int64_t* pi = ind.data_ptr<int64_t>();
  auto click = [&](const double* p, int64_t k) { return dim == 1 ? p[k] : p[2 * k + 1]; };
  auto nonclick = [&](const double* p, int64_t k) { return dim == 1 ? 1.0 - p[k] : p[2 * k]; };
  std::vector<int64_t> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  std::vector<double> aucs;
  std::vector<int64_t> counts;
  for (int64_t begin = 0; begin < n;) {
    int64_t end = begin + 1;
    while (end < n && pi[end] == pi[begin]) ++end;
    std::stable_sort(idx.begin() + begin, idx.begin() + end, [&](int64_t a, int64_t b) { return click(pp, a) < click(pp, b); });
    double fp1 = 0, tp1 = 0, fp2 = 0, tp2 = 0, auc = 0;
    for (int64_t k = begin; k < end; ++k) {
      const int64_t i = idx[k];
      fp2 += nonclick(pl, i); tp2 += click(pl, i);
      auc += (fp2 - fp1) * (tp2 + tp1);
      fp1 = fp2; tp1 = tp2;
    }
    if (tp2 * fp2 > 0) { aucs.push_back(1.0 - auc / (2.0 * tp2 * fp2)); counts.push_back(end - begin); }
    begin = end;
  }
  auto a = torch::empty({(int64_t)aucs.size()}, torch::kFloat64);
  auto c = torch::empty({(int64_t)aucs.size()}, torch::kInt64);
  std::copy(aucs.begin(), aucs.end(), a.data_ptr<double>());
  std::copy(counts.begin(), counts.end(), c.data_ptr<int64_t>());
  return {a, c};
}

}  // namespace

void init_metrics(py::module& m) { m.def("gauc_calc", &gauc_calc); }
