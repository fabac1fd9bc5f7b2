#pragma once
#include <torch/extension.h>
#include <map>
#include <string>
#include <vector>
#include "../kernels/rb_kernels.h"
#include "vmm_slab.h"

namespace rbx {

class EmbeddingStore {
 public:
  EmbeddingStore(int64_t dim, int64_t capacity, torch::Device device, int init_kind, double a, double b, double lo, double hi,
                 int64_t seed, bool track_last_seen, bool growable, c10::optional<torch::Tensor> emb_storage,
                 torch::ScalarType emb_dtype = torch::kFloat32);
  ~EmbeddingStore();
  EmbeddingStore(const EmbeddingStore&) = delete;
  EmbeddingStore& operator=(const EmbeddingStore&) = delete;
  // ids_unique: no id occurs twice in `ids` (new ids may then reuse erased index slots)
  torch::Tensor lookup_or_insert(const torch::Tensor& ids, c10::optional<torch::Tensor> n_dev, c10::optional<torch::Tensor> step,
                                 int64_t admit_threshold, bool ids_unique = false);
  torch::Tensor find(const torch::Tensor& ids, c10::optional<torch::Tensor> n_dev);
  torch::Tensor erase(const torch::Tensor& ids);
  std::tuple<torch::Tensor, torch::Tensor> snapshot(bool expired_only, int64_t threshold);
  void add_slot(const std::string& name, double fill);
  torch::Tensor slot(const std::string& name) const;
  bool has_slot(const std::string& name) const { return slots_.count(name) > 0; }
  std::vector<std::string> slot_names() const { return slot_order_; }
  torch::Tensor emb() const { return emb_; }
  torch::Tensor last_seen() const { return last_seen_; }
  torch::Tensor keys() const { return keys_; }
  torch::Tensor index_rows() const { return rows_; }
  torch::Tensor ctr() const { return ctr_; }
  torch::Tensor free_list() const { return free_list_; }
  std::vector<int64_t> counters() const;
  void reserve(int64_t new_cap);
  int64_t fit_growth(int64_t wanted, int64_t needed);   // `wanted` rows, or fewer (but at least `needed`) when the device's free memory says so
  bool grows_in_place() const { return use_vmm_ && !vmm_.empty(); }
  void rebuild_index(int64_t nslots);
  void ensure_room(int64_t n_incoming);
  void clear();
  int64_t size() const;
  int64_t capacity() const { return cap_rows_; }
  int64_t dim() const { return dim_; }
  RbTable view() const;
  RbInit init() const { return init_; }
  void set_name(const std::string& n) { name_ = n; }

 private:
  void alloc_index(int64_t nslots);
  void refresh_bounds();
  // one per-row array [rows, ...]: backed by a growable virtual range on CUDA (grows in place), else a plain tensor
  torch::Tensor alloc_slab(const std::string& key, int64_t rows, int64_t width, torch::ScalarType dtype);
  bool grow_slab_in_place(const std::string& key, torch::Tensor& t, int64_t new_rows);
  std::map<std::string, std::shared_ptr<VmmSlab>> vmm_;
  bool use_vmm_ = false;
  int64_t max_rows_ = 0;
  int64_t dim_, cap_rows_;
  torch::Device device_;
  bool growable_;
  RbInit init_;
  std::string name_ = "store";
  torch::Tensor keys_, rows_, ctr_, free_list_, emb_, last_seen_;
  std::map<std::string, torch::Tensor> slots_;
  std::map<std::string, double> slot_fill_;
  std::vector<std::string> slot_order_;
  int64_t rows_upper_ = 0, bump_upper_ = 0, index_upper_ = 0;
  int64_t tomb_seen_ = 0;           // erased index slots as of the newest counters the host has seen
  // asynchronous counter mirror (pinned host copies of the device counters, see store.cpp)
  static constexpr int kMirror = 8;
  static constexpr int kMirrorStride = RB_CTR_COUNT + 1;
  void post_mirror(int64_t n_issued, const int32_t* n_dev = nullptr);
  int64_t seen_n_dev_ = 0;          // recent maximum of the device-side id counts of lookup_or_insert calls
  int64_t est_new_ = -1;            // recent maximum of rows (or index entries) one call really added; -1 = no history yet
  int64_t rows_prev_ = -1, index_prev_ = 0, calls_prev_ = 0, calls_total_ = 0;
  int64_t mirror_calls_[kMirror];
  void absorb_mirror();
  int64_t* mirror_host_ = nullptr;
  cudaEvent_t mirror_ev_[kMirror];
  int64_t mirror_issued_[kMirror];
  int64_t mirror_head_ = 0, issued_total_ = 0, absorbed_issued_ = 0;
};

}  // namespace rbx
