// Native input pipeline pieces: a multi-threaded, checkpointable synthetic batch source and a ragged batch packer.
//
// The reference's input path is the column-io C++ dataset graph (third_party/column-io/cc/column-io/dataset:
// parallel_dataset.cc, packer.cc, prefetch_dataset.cc) reading ORC / ODPS. The open part of that is rebuilt here as:
//   * SyntheticSource: worker threads generate whole batches (dense features, labels, power-law ids with Poisson /
//     geometric / uniform / fixed bag lengths) straight into pinned tensors and park them in a bounded reorder buffer;
//     batch k is a pure function of (seed, k), so the iterator state is a single integer.
//   * pack_ragged: concatenates per-row id lists (as delivered by a columnar reader) into values + offsets.
#include <torch/extension.h>
#include <cmath>
#include <condition_variable>
#include <map>
#include <mutex>
#include <thread>

namespace py = pybind11;
using torch::Tensor;

namespace {

struct Rng {                       // splitmix64 stream
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed) {}
  uint64_t next() { uint64_t z = (s += 0x9e3779b97f4a7c15ull); z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull; z = (z ^ (z >> 27)) * 0x94d049bb133111ebull; return z ^ (z >> 31); }
  double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }   // [0, 1)
  double normal() { const double u1 = 1.0 - uniform(), u2 = uniform(); return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2); }
};

inline uint64_t mix64(uint64_t x) { x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull; x ^= x >> 27; x *= 0x94d049bb133111ebull; x ^= x >> 31; return x; }

struct FieldSpec { double zipf_a; int id_bits; int64_t universe; int len_kind; double mean_len; int64_t min_len, max_len; double geo_p; };

struct Batch { Tensor dense, label; std::vector<Tensor> ids, offsets; };

class SyntheticSource {
 public:
  SyntheticSource(int64_t batch, int64_t dense_dim, std::vector<std::tuple<double, int64_t, int64_t, int64_t, double, int64_t, int64_t, double>> fields,
                  double label_rate, int64_t seed, int64_t threads, int64_t depth, bool pin)
      : batch_(batch), dense_dim_(dense_dim), label_rate_(label_rate), seed_((uint64_t)seed), depth_(std::max<int64_t>(depth, 1)), pin_(pin) {
    for (auto& f : fields)
      fields_.push_back(FieldSpec{std::get<0>(f), (int)std::get<1>(f), std::get<2>(f), (int)std::get<3>(f), std::get<4>(f), std::get<5>(f),
                                  std::get<6>(f), std::get<7>(f)});
    n_threads_ = std::max<int64_t>(threads, 1);
    start();
  }
  ~SyntheticSource() { stop(); }

  py::tuple next() {
    Batch b;
    {
      py::gil_scoped_release nogil;
      std::unique_lock<std::mutex> lk(mu_);
      cv_ready_.wait(lk, [&] { return ready_.count(cursor_) > 0; });
      b = std::move(ready_[cursor_]);
      ready_.erase(cursor_);
      ++cursor_;
      cv_space_.notify_all();
    }
    py::list fields;
    for (size_t i = 0; i < b.ids.size(); ++i) fields.append(py::make_tuple(b.ids[i], b.offsets[i]));
    return py::make_tuple(b.dense, b.label, fields);
  }

  int64_t state() const { return cursor_; }

  void set_state(int64_t step) {
    stop();
    cursor_ = next_to_make_ = step;
    ready_.clear();
    start();
  }

 private:
  void start() {
    stopping_ = false;
    next_to_make_ = cursor_;
    for (int64_t t = 0; t < n_threads_; ++t) workers_.emplace_back([this] { work(); });
  }
  void stop() {
    { std::lock_guard<std::mutex> lk(mu_); stopping_ = true; }
    cv_space_.notify_all(); cv_ready_.notify_all();
    for (auto& w : workers_) w.join();
    workers_.clear();
  }
  void work() {
    for (;;) {
      int64_t step;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_space_.wait(lk, [&] { return stopping_ || next_to_make_ < cursor_ + depth_; });
        if (stopping_) return;
        step = next_to_make_++;
      }
      Batch b = make(step);
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (stopping_) return;
        ready_[step] = std::move(b);
      }
      cv_ready_.notify_all();
    }
  }
  Tensor alloc(std::vector<int64_t> shape, torch::ScalarType dt) { return torch::empty(shape, torch::TensorOptions().dtype(dt).pinned_memory(pin_)); }

  int64_t bag_len(Rng& r, const FieldSpec& f) {
    double v;
    switch (f.len_kind) {
      case 1: {  // Poisson: Knuth for small means, normal approximation above
        if (f.mean_len < 30) { const double L = std::exp(-f.mean_len); double p = 1.0; int64_t k = 0; do { ++k; p *= r.uniform(); } while (p > L); v = (double)(k - 1); }
        else v = std::floor(f.mean_len + std::sqrt(f.mean_len) * r.normal() + 0.5);
        break;
      }
      case 2: v = std::floor(std::log(1.0 - r.uniform()) / std::log(1.0 - f.geo_p)) + 1.0; break;
      case 3: return f.min_len + (int64_t)(r.uniform() * (double)(f.max_len - f.min_len + 1));
      default: return (int64_t)f.mean_len;
    }
    return std::min(std::max((int64_t)v, f.min_len), f.max_len);
  }

  Batch make(int64_t step) {
    Batch b;
    Rng r(mix64(seed_ * 0x9E3779B97F4A7C15ull + (uint64_t)step));
    if (dense_dim_ > 0) {
      b.dense = alloc({batch_, dense_dim_}, torch::kFloat32);
      float* d = b.dense.data_ptr<float>();
      for (int64_t i = 0; i < batch_ * dense_dim_; ++i) d[i] = (float)std::log1p(std::exp(r.normal()));
    }
    b.label = alloc({batch_, 1}, torch::kFloat32);
    float* l = b.label.data_ptr<float>();
    for (int64_t i = 0; i < batch_; ++i) l[i] = r.uniform() < label_rate_ ? 1.f : 0.f;
    for (size_t k = 0; k < fields_.size(); ++k) {
      const FieldSpec& f = fields_[k];
      Tensor off = alloc({batch_ + 1}, torch::kInt32);
      int32_t* op = off.data_ptr<int32_t>();
      op[0] = 0;
      for (int64_t i = 0; i < batch_; ++i) op[i + 1] = op[i] + (int32_t)bag_len(r, f);
      const int64_t nnz = op[batch_];
      Tensor ids = alloc({nnz}, torch::kInt64);
      int64_t* ip = ids.data_ptr<int64_t>();
      const double N = std::pow(2.0, f.id_bits), e = 1.0 - f.zipf_a, base = std::pow(N, e) - 1.0;
      const uint64_t mask = f.id_bits >= 64 ? ~0ull : ((1ull << f.id_bits) - 1), salt = (uint64_t)(k + 1) * 0x9E3779B97F4A7C15ull;
      for (int64_t i = 0; i < nnz; ++i) {
        double x = std::floor(std::pow(base * r.uniform() + 1.0, 1.0 / e));
        uint64_t rank = (uint64_t)std::min(x, N);
        if (f.universe > 0) rank %= (uint64_t)f.universe;
        ip[i] = (int64_t)(mix64(rank + salt) & mask);
      }
      b.ids.push_back(ids); b.offsets.push_back(off);
    }
    return b;
  }

  int64_t batch_, dense_dim_;
  double label_rate_;
  uint64_t seed_;
  int64_t depth_, n_threads_;
  bool pin_;
  std::vector<FieldSpec> fields_;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_ready_, cv_space_;
  std::map<int64_t, Batch> ready_;
  int64_t cursor_ = 0, next_to_make_ = 0;
  bool stopping_ = false;
};

// rows: list of 1-D int64 tensors (one per sample) -> (values, offsets int32), optionally pinned
std::tuple<Tensor, Tensor> pack_ragged(const std::vector<Tensor>& rows, bool pin) {
  const int64_t B = (int64_t)rows.size();
  auto off = torch::empty({B + 1}, torch::TensorOptions().dtype(torch::kInt32).pinned_memory(pin));
  int32_t* op = off.data_ptr<int32_t>();
  op[0] = 0;
  for (int64_t i = 0; i < B; ++i) op[i + 1] = op[i] + (int32_t)rows[i].numel();
  auto dt = B > 0 ? rows[0].scalar_type() : torch::kInt64;
  auto vals = torch::empty({op[B]}, torch::TensorOptions().dtype(dt).pinned_memory(pin));
  const int64_t esz = vals.element_size();
  char* vp = reinterpret_cast<char*>(vals.data_ptr());
  for (int64_t i = 0; i < B; ++i) {
    auto r = rows[i].contiguous();
    TORCH_CHECK(r.scalar_type() == dt, "pack_ragged: mixed dtypes");
    std::memcpy(vp + (int64_t)op[i] * esz, r.data_ptr(), (size_t)r.numel() * esz);
  }
  return {vals, off};
}

}  // namespace

void init_io(py::module& m) {
  py::class_<SyntheticSource>(m, "SyntheticSource")
      .def(py::init<int64_t, int64_t, std::vector<std::tuple<double, int64_t, int64_t, int64_t, double, int64_t, int64_t, double>>, double,
                    int64_t, int64_t, int64_t, bool>())
      .def("next", &SyntheticSource::next)
      .def("state", &SyntheticSource::state)
      .def("set_state", &SyntheticSource::set_state);
  m.def("pack_ragged", &pack_ragged);
}
