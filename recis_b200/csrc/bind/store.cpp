// EmbeddingStore: the native dynamic-embedding table (index + row arena + named per-row slots).
//
// Plays the role of the reference's Hashtable / IdMap / IdAllocator / SlotGroup stack
// (csrc/embedding/hashtable.cc:82-313, slot_group.cc:39-174, id_allocator.cc:17-62) with a different layout:
// one open-addressing index, one contiguous [capacity, dim] slab per slot (no vector of blocks, hence no
// per-call pointer tables and no per-op stream synchronisation), rows initialised on admission as a pure
// function of (seed, id). The host keeps pessimistic upper bounds of the allocator counters so that the hot
// path never reads device memory; it synchronises only when a bound says that growth may be needed.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "../kernels/rb_kernels.h"
#include "../cpu/rb_cpu.h"
#include "store.h"
#include <c10/cuda/CUDACachingAllocator.h>
#include <climits>
#include <cstdlib>
#include "bind_shared.h"

namespace rbx {

static int64_t pow2_at_least(int64_t x) { int64_t p = 1024; while (p < x) p <<= 1; return p; }

EmbeddingStore::EmbeddingStore(int64_t dim, int64_t capacity, torch::Device device, int init_kind, double a, double b,
                               double lo, double hi, int64_t seed, bool track_last_seen, bool growable,
                               c10::optional<torch::Tensor> emb_storage, torch::ScalarType emb_dtype)
    : dim_(dim), cap_rows_(std::max<int64_t>(capacity, 16)), device_(device), growable_(growable) {
  init_.kind = init_kind; init_.a = (float)a; init_.b = (float)b; init_.lo = (float)lo; init_.hi = (float)hi;
  init_.seed = (uint64_t)seed;
  auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(device_);
  TORCH_CHECK(emb_dtype == torch::kFloat32 || emb_dtype == torch::kFloat16 || emb_dtype == torch::kBFloat16 || emb_dtype == torch::kInt8,
              "embedding rows are stored as float32, float16, bfloat16 or int8");
  if (emb_storage.has_value()) {
    TORCH_CHECK(emb_storage->numel() >= cap_rows_ * dim_ && emb_storage->scalar_type() == emb_dtype, "emb_storage too small or of the wrong type");
    emb_ = emb_storage->view({-1}).narrow(0, 0, cap_rows_ * dim_).view({cap_rows_, dim_});
    growable_ = false;  // externally owned (peer-mapped) storage cannot move
  }
  // Growable tables on a GPU keep their per-row arrays in reserved virtual ranges that grow in place (vmm_slab.h): room is
  // reserved for max_rows_ rows (RECIS_TABLE_MAX_ROWS, default 16 x the initial capacity, at least 64 Mi rows), physical
  // memory is only mapped for the current capacity. RECIS_TABLE_VMM=0 switches back to allocate + copy.
  const char* vmm_env = std::getenv("RECIS_TABLE_VMM");
  use_vmm_ = device_.is_cuda() && growable_ && !(vmm_env && std::string(vmm_env) == "0");
  const char* max_env = std::getenv("RECIS_TABLE_MAX_ROWS");
  max_rows_ = max_env ? std::atoll(max_env) : std::max<int64_t>(cap_rows_ * 16, (int64_t)1 << 26);
  max_rows_ = std::min<int64_t>(std::max<int64_t>(max_rows_, cap_rows_), (int64_t)INT32_MAX - 1024);
  if (!emb_storage.has_value()) emb_ = alloc_slab("embedding", cap_rows_, dim_, emb_dtype);   // rows in their storage type; slots stay fp32
  if (track_last_seen) { last_seen_ = alloc_slab("last_seen", cap_rows_, 0, torch::kInt64); last_seen_.zero_(); }
  alloc_index(pow2_at_least(cap_rows_ * 2));
  ctr_ = torch::zeros({RB_CTR_COUNT}, f32.dtype(torch::kInt64));
  free_list_ = alloc_slab("free_list", cap_rows_, 0, torch::kInt32);
}

// width == 0: a 1-D array [rows]; else [rows, width]
torch::Tensor EmbeddingStore::alloc_slab(const std::string& key, int64_t rows, int64_t width, torch::ScalarType dtype) {
  std::vector<int64_t> shape = width > 0 ? std::vector<int64_t>{rows, width} : std::vector<int64_t>{rows};
  if (use_vmm_) {
    const size_t row_bytes = (size_t)std::max<int64_t>(width, 1) * c10::elementSize(dtype);
    auto slab = VmmSlab::create(device_.index(), (size_t)max_rows_ * row_bytes);
    if (slab && slab->ensure((size_t)rows * row_bytes)) {
      vmm_[key] = slab;
      return slab->view(shape, dtype);
    }
    use_vmm_ = !vmm_.empty();          // the first failure switches the whole table to plain tensors; later ones fall back singly
  }
  return torch::empty(shape, torch::TensorOptions().dtype(dtype).device(device_));
}

// more rows for a slab that lives in a virtual range: map pages, re-create the view; false when the slab is a plain tensor
bool EmbeddingStore::grow_slab_in_place(const std::string& key, torch::Tensor& t, int64_t new_rows) {
  auto it = vmm_.find(key);
  if (it == vmm_.end()) return false;
  std::vector<int64_t> shape = t.sizes().vec();
  int64_t per_row = 1;
  for (size_t i = 1; i < shape.size(); ++i) per_row *= shape[i];
  if (!it->second->ensure((size_t)new_rows * per_row * t.element_size())) return false;
  shape[0] = new_rows;
  t = it->second->view(shape, t.scalar_type());
  return true;
}

void EmbeddingStore::alloc_index(int64_t nslots) {
  auto o = torch::TensorOptions().device(device_);
  keys_ = torch::full({nslots}, -1, o.dtype(torch::kInt64));
  rows_ = torch::full({nslots}, -1, o.dtype(torch::kInt32));
}

RbTable EmbeddingStore::view() const {
  RbTable t;
  t.keys = reinterpret_cast<uint64_t*>(keys_.data_ptr<int64_t>());
  t.rows = rows_.data_ptr<int32_t>();
  t.mask = (uint64_t)keys_.numel() - 1;
  t.ctr = ctr_.data_ptr<int64_t>();
  t.free_list = free_list_.data_ptr<int32_t>();
  t.cap_rows = cap_rows_;
  return t;
}

void EmbeddingStore::add_slot(const std::string& name, double fill) {
  if (slots_.count(name)) return;
  slots_[name] = alloc_slab("slot:" + name, cap_rows_, dim_, torch::kFloat32);
  slots_[name].fill_(fill);
  slot_fill_[name] = fill;
  slot_order_.push_back(name);
}

torch::Tensor EmbeddingStore::slot(const std::string& name) const {
  auto it = slots_.find(name);
  TORCH_CHECK(it != slots_.end(), "no slot named ", name);
  return it->second;
}

std::vector<int64_t> EmbeddingStore::counters() const {
  auto c = ctr_.cpu();
  std::vector<int64_t> v(c.data_ptr<int64_t>(), c.data_ptr<int64_t>() + RB_CTR_COUNT);
  return v;
}

void EmbeddingStore::refresh_bounds() {
  auto c = counters();
  rows_upper_ = c[RB_CTR_BUMP] - c[RB_CTR_FREE_TOP];
  if (rows_upper_ < 0) rows_upper_ = 0;
  bump_upper_ = c[RB_CTR_BUMP];
  index_upper_ = c[RB_CTR_LIVE] + c[RB_CTR_TOMBSTONES] + c[RB_CTR_PROBATION];
  tomb_seen_ = c[RB_CTR_TOMBSTONES];
  absorbed_issued_ = issued_total_;
  TORCH_CHECK((c[RB_CTR_STATUS] & 3) == 0, "embedding store reported status ", c[RB_CTR_STATUS],
              " (1 = row arena exhausted, 2 = index full); raise the capacity");
}

// Asynchronous counter mirror: after every lookup-or-insert the 64-byte counter block is copied to pinned host memory on the
// same stream. ensure_room() takes the newest copy that has already landed (cudaEventQuery, never a wait) as the truth and
// only adds the ids issued since then, so the pessimistic bound is at most a step or two ahead of reality.
void EmbeddingStore::post_mirror(int64_t n_issued, const int32_t* n_dev) {
  issued_total_ += n_issued;
  if (!device_.is_cuda()) return;
  if (mirror_host_ == nullptr) {
    // per slot: the counter block, then one more word that receives the device-side id count of the call (int32 in its low half)
    if (cudaHostAlloc(reinterpret_cast<void**>(&mirror_host_), sizeof(int64_t) * kMirrorStride * kMirror, cudaHostAllocDefault) != cudaSuccess) {
      mirror_host_ = nullptr;
      return;
    }
    for (int i = 0; i < kMirror; ++i) { cudaEventCreateWithFlags(&mirror_ev_[i], cudaEventDisableTiming); mirror_issued_[i] = -1; }
  }
  const int slot = (int)(mirror_head_++ % kMirror);
  auto st = at::cuda::getCurrentCUDAStream();
  int64_t* dst = mirror_host_ + slot * kMirrorStride;
  dst[RB_CTR_COUNT] = -1;                                   // "no device-side count in this slot"
  bool posted = cudaMemcpyAsync(dst, ctr_.data_ptr<int64_t>(), sizeof(int64_t) * RB_CTR_COUNT, cudaMemcpyDeviceToHost, st) == cudaSuccess;
  if (posted && n_dev != nullptr) {
    dst[RB_CTR_COUNT] = 0;
    posted = cudaMemcpyAsync(dst + RB_CTR_COUNT, n_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, st) == cudaSuccess;
  }
  posted = posted && cudaEventRecord(mirror_ev_[slot], st) == cudaSuccess;
  // a slot whose copy could not be posted is never absorbed: the bounds then stay pessimistic until a later mirror lands
  mirror_issued_[slot] = posted ? issued_total_ : -1;
  mirror_calls_[slot] = calls_total_;
}

EmbeddingStore::~EmbeddingStore() {
  if (mirror_host_ != nullptr) {
    for (int i = 0; i < kMirror; ++i) cudaEventDestroy(mirror_ev_[i]);
    cudaFreeHost(mirror_host_);
    mirror_host_ = nullptr;
  }
}

void EmbeddingStore::absorb_mirror() {
  if (mirror_host_ == nullptr) return;
  for (int back = 1; back <= kMirror && back <= (int)mirror_head_; ++back) {
    const int slot = (int)((mirror_head_ - back) % kMirror);
    if (mirror_issued_[slot] < 0 || mirror_issued_[slot] <= absorbed_issued_) break;
    if (cudaEventQuery(mirror_ev_[slot]) != cudaSuccess) continue;
    const int64_t* c = mirror_host_ + slot * kMirrorStride;
    TORCH_CHECK((c[RB_CTR_STATUS] & 3) == 0, "embedding store '", name_, "' reported status ", c[RB_CTR_STATUS],
                " (1 = row arena exhausted, 2 = index full) in an earlier step; raise the capacity");
    if (c[RB_CTR_COUNT] >= 0) seen_n_dev_ = std::max<int64_t>(seen_n_dev_ * 7 / 8, c[RB_CTR_COUNT] & 0xFFFFFFFFll);   // decaying maximum
    const int64_t pending = issued_total_ - mirror_issued_[slot];
    const int64_t rows_now = std::max<int64_t>(c[RB_CTR_BUMP] - c[RB_CTR_FREE_TOP], 0);
    const int64_t index_now = c[RB_CTR_LIVE] + c[RB_CTR_TOMBSTONES] + c[RB_CTR_PROBATION];
    // how many rows / index entries one call really adds (decaying maximum over the calls seen so far)
    if (rows_prev_ >= 0 && mirror_calls_[slot] > calls_prev_) {
      const int64_t calls = mirror_calls_[slot] - calls_prev_;
      const int64_t grown = std::max<int64_t>(std::max(rows_now - rows_prev_, index_now - index_prev_), 0);
      const int64_t per_call = (grown + calls - 1) / calls;
      est_new_ = std::max<int64_t>(est_new_ < 0 ? 0 : est_new_ * 7 / 8, per_call);
    }
    rows_prev_ = rows_now; index_prev_ = index_now; calls_prev_ = mirror_calls_[slot];
    rows_upper_ = rows_now + pending;
    index_upper_ = index_now + pending;
    tomb_seen_ = c[RB_CTR_TOMBSTONES];
    absorbed_issued_ = mirror_issued_[slot];
    break;
  }
}

void EmbeddingStore::ensure_room(int64_t n_incoming) {
  // rows_upper_ / index_upper_ = the newest counters that came back through the mirror + what was set aside for the calls issued
  // since. Without history (first calls, CPU stores) a bound that crosses the capacity makes us read the true counters, which
  // synchronises; with history we act on the bounds as they are: growing a little early costs memory, never a stall.
  absorb_mirror();
  const bool lagged_ok = device_.is_cuda() && est_new_ >= 0;
  if (rows_upper_ + n_incoming > cap_rows_ || index_upper_ + n_incoming > (int64_t)(0.65 * keys_.numel())) {
    if (!lagged_ok) refresh_bounds();
    if (rows_upper_ + n_incoming > cap_rows_) {
      if (!growable_) {
        if (lagged_ok) refresh_bounds();          // fixed storage: make sure before failing
        TORCH_CHECK(rows_upper_ + n_incoming <= cap_rows_, "embedding store '", name_, "' is full (", rows_upper_, " rows of ", cap_rows_,
                    ") and cannot grow: it was created with fixed (peer-mapped) storage");
      } else {
        int64_t nc = cap_rows_;
        while (rows_upper_ + n_incoming > nc) nc = nc + nc / 2 + 1024;
        reserve(fit_growth(nc, rows_upper_ + n_incoming));
      }
    }
    if (index_upper_ + n_incoming > (int64_t)(0.65 * keys_.numel())) {
      // Erased slots do not survive a rebuild: size the new index for what is live (and on probation) only, never smaller than
      // the old one. A table whose eviction keeps pace with its inserts is rebuilt at the same size - a clean-up - instead of
      // doubling every time the tombstones pile up.
      const int64_t need = pow2_at_least((std::max<int64_t>(index_upper_ - tomb_seen_, 0) + n_incoming) * 2);
      rebuild_index(std::max<int64_t>(need, keys_.numel()));
      index_upper_ = std::max<int64_t>(index_upper_ - tomb_seen_, 0);
      tomb_seen_ = 0;
    }
  }
  rows_upper_ += n_incoming; index_upper_ += n_incoming;
}

void EmbeddingStore::rebuild_index(int64_t nslots) {
  RbTable src = view();
  auto old_keys = keys_, old_rows = rows_;
  alloc_index(nslots);
  RbTable dst = view();
  if (device_.is_cuda()) {
    c10::cuda::CUDAGuard g(device_);
    rb_table_rehash(src, dst, at::cuda::getCurrentCUDAStream());
  } else {
    rbc_table_rehash(src, dst);
  }
  ctr_.select(0, RB_CTR_TOMBSTONES).zero_();
  // the tombstones are gone; with mirrored history the (pessimistic) bounds stay as they are until the next mirror lands
  if (!(device_.is_cuda() && est_new_ >= 0)) refresh_bounds();
}

// Growth by half is the policy while memory is plentiful. Close to the device's limit (a table that is most of the GPU's memory)
// the step shrinks to what the free memory can hold, down to just the rows that are needed: a table must not fail at 1.5 x its
// size when 1.1 x would have fitted.
int64_t EmbeddingStore::fit_growth(int64_t wanted, int64_t needed) {
  if (!device_.is_cuda() || !use_vmm_) return wanted;
  int64_t row_bytes = 0;
  auto add = [&](const torch::Tensor& t) { if (t.defined() && t.size(0) > 0) row_bytes += t.numel() / t.size(0) * (int64_t)t.element_size(); };
  add(emb_);
  for (auto& kv : slots_) add(kv.second);
  add(last_seen_);
  add(free_list_);
  if (row_bytes <= 0) return wanted;
  c10::cuda::CUDAGuard g(device_);
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return wanted;
  // kept free: 2 GiB for an index rebuild and odd allocations, and what the tensor allocator holds now (the step's activations
  // and workspaces will be asked for again after its cache has been emptied below)
  const int64_t held = (int64_t)c10::cuda::CUDACachingAllocator::getDeviceStats(device_.index()).reserved_bytes[0].current;
  int64_t margin = (int64_t)2 << 30;
  auto rows_that_fit = [&](size_t fb) { return std::max<int64_t>(((int64_t)fb - margin) / row_bytes, 0); };
  if (cap_rows_ + rows_that_fit(free_b) < wanted) {
    c10::cuda::CUDACachingAllocator::emptyCache();                // blocks the tensor allocator caches cannot back a mapped range
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return wanted;
    margin += held;
  }
  const int64_t fits = cap_rows_ + rows_that_fit(free_b);
  if (fits >= wanted) return wanted;
  return std::max<int64_t>(needed + needed / 64 + 1024, std::min(fits, wanted));   // below `needed` the reservation itself reports the failure
}

void EmbeddingStore::reserve(int64_t new_cap) {
  if (new_cap <= cap_rows_) return;
  TORCH_CHECK(growable_, "store has fixed storage");
  // in place where the slab lives in a virtual range (pages are mapped behind the old end, nothing moves), else a new tensor
  // and a copy of the old rows
  auto grow = [&](const std::string& key, torch::Tensor& t, double fill, bool do_fill) {
    if (!grow_slab_in_place(key, t, new_cap)) {
      TORCH_CHECK(vmm_.find(key) == vmm_.end(), "embedding store '", name_, "': cannot grow to ", new_cap, " rows in place (the reserved range "
                  "holds ", max_rows_, " rows or the device is out of memory); raise RECIS_TABLE_MAX_ROWS or set RECIS_TABLE_VMM=0");
      std::vector<int64_t> shape = t.sizes().vec();
      shape[0] = new_cap;
      auto nt = torch::empty(shape, t.options());
      nt.narrow(0, 0, cap_rows_).copy_(t);
      t = nt;
    }
    if (do_fill) t.narrow(0, cap_rows_, new_cap - cap_rows_).fill_(fill);
  };
  grow("embedding", emb_, 0.0, false);
  for (auto& kv : slots_) grow("slot:" + kv.first, kv.second, slot_fill_[kv.first], true);
  if (last_seen_.defined()) grow("last_seen", last_seen_, 0.0, true);
  grow("free_list", free_list_, 0.0, false);
  cap_rows_ = new_cap;
  if (keys_.numel() < 2 * new_cap) rebuild_index(pow2_at_least(2 * new_cap));
}

torch::Tensor EmbeddingStore::lookup_or_insert(const torch::Tensor& ids, c10::optional<torch::Tensor> n_dev,
                                               c10::optional<torch::Tensor> step, int64_t admit_threshold, bool ids_unique) {
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && ids.device() == device_, "ids must be contiguous int64 on the store's device");
  const int64_t n = ids.numel();
  auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(device_);
  auto rows_out = torch::empty({n}, i32);
  if (n == 0) return rows_out;
  // How many ids may be new? With a device-side count the buffer length n is only the window capacity, often many times
  // the real count; making room for all of it would force a (synchronising) look at the true counters, or a growth,
  // on every call. The counts of earlier calls come back through the asynchronous mirror: make room for their recent maximum
  // plus a quarter. Should a call exceed that AND the arena be full, the kernel's bounds guard sets the status word
  // (no row is written out of range) and a later call reports it.
  int64_t n_room = n;
  if (n_dev.has_value() && device_.is_cuda()) {
    absorb_mirror();
    if (seen_n_dev_ == 0) {
      // no count has come back yet (first calls only): read this call's count directly, which synchronises once
      int32_t now = 0;
      c10::cuda::CUDAGuard g(device_);
      auto st = at::cuda::getCurrentCUDAStream();
      if (cudaMemcpyAsync(&now, n_dev->data_ptr<int32_t>(), sizeof(int32_t), cudaMemcpyDeviceToHost, st) == cudaSuccess &&
          cudaStreamSynchronize(st) == cudaSuccess && now > 0)
        seen_n_dev_ = now;
    }
    if (seen_n_dev_ > 0) n_room = std::min<int64_t>(n, seen_n_dev_ + seen_n_dev_ / 4 + 65536);
  }
  // ... and of those ids only some are new: twice the recent maximum of rows actually added per call, once that is known
  if (device_.is_cuda()) {
    absorb_mirror();
    if (est_new_ >= 0) n_room = std::min<int64_t>(n_room, 2 * est_new_ + 65536);
  }
  ++calls_total_;
  ensure_room(n_room);
  auto slot_scratch = torch::empty({n}, i32);
  auto new_rows = torch::empty({n}, i32);
  auto new_keys = torch::empty({n}, i32.dtype(torch::kInt64));
  const int32_t* nd = n_dev.has_value() ? n_dev->data_ptr<int32_t>() : nullptr;
  const int64_t* sd = (step.has_value() && last_seen_.defined()) ? step->data_ptr<int64_t>() : nullptr;
  int64_t* ls = last_seen_.defined() && sd ? last_seen_.data_ptr<int64_t>() : nullptr;
  if (device_.is_cuda()) {
    c10::cuda::CUDAGuard g(device_);
    rb_table_lookup_or_insert(view(), ids.data_ptr<int64_t>(), n, nd, slot_scratch.data_ptr<int32_t>(), new_rows.data_ptr<int32_t>(),
                              new_keys.data_ptr<int64_t>(), rows_out.data_ptr<int32_t>(), emb_.data_ptr(), rbx::row_dtype_of(emb_), (int)dim_, init_, ls,
                              sd, (int)admit_threshold, ids_unique ? 1 : 0, at::cuda::getCurrentCUDAStream());
  } else {
    rbc_table_lookup_or_insert(view(), ids.data_ptr<int64_t>(), n, nd, slot_scratch.data_ptr<int32_t>(), new_rows.data_ptr<int32_t>(),
                               new_keys.data_ptr<int64_t>(), rows_out.data_ptr<int32_t>(), emb_.data_ptr(), rbx::row_dtype_of(emb_), (int)dim_, init_, ls,
                               sd, (int)admit_threshold, ids_unique ? 1 : 0);
  }
  post_mirror(n_room, nd);
  return rows_out;
}

torch::Tensor EmbeddingStore::find(const torch::Tensor& ids, c10::optional<torch::Tensor> n_dev) {
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && ids.device() == device_);
  const int64_t n = ids.numel();
  auto rows_out = torch::empty({n}, torch::TensorOptions().dtype(torch::kInt32).device(device_));
  const int32_t* nd = n_dev.has_value() ? n_dev->data_ptr<int32_t>() : nullptr;
  if (n == 0) return rows_out;
  if (device_.is_cuda()) {
    c10::cuda::CUDAGuard g(device_);
    rb_table_find(view(), ids.data_ptr<int64_t>(), n, nd, rows_out.data_ptr<int32_t>(), at::cuda::getCurrentCUDAStream());
  } else {
    rbc_table_find(view(), ids.data_ptr<int64_t>(), n, nd, rows_out.data_ptr<int32_t>());
  }
  return rows_out;
}

torch::Tensor EmbeddingStore::erase(const torch::Tensor& ids) {
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && ids.device() == device_);
  const int64_t n = ids.numel();
  auto erased = torch::empty({n}, torch::TensorOptions().dtype(torch::kInt32).device(device_));
  if (n == 0) return erased;
  if (device_.is_cuda()) {
    c10::cuda::CUDAGuard g(device_);
    auto st = at::cuda::getCurrentCUDAStream();
    rb_table_erase(view(), ids.data_ptr<int64_t>(), n, nullptr, erased.data_ptr<int32_t>(), st);
    for (auto& kv : slots_) {
      auto fillv = torch::full({dim_}, slot_fill_[kv.first], kv.second.options());
      rb_scatter_rows(kv.second.data_ptr(), erased.data_ptr<int32_t>(), n, dim_ * (int64_t)sizeof(float), fillv.data_ptr(), 1, st);
    }
  } else {
    rbc_table_erase(view(), ids.data_ptr<int64_t>(), n, nullptr, erased.data_ptr<int32_t>());
    for (auto& kv : slots_) {
      auto fillv = torch::full({dim_}, slot_fill_[kv.first], kv.second.options());
      rbc_scatter_rows(kv.second.data_ptr(), erased.data_ptr<int32_t>(), n, dim_ * (int64_t)sizeof(float), fillv.data_ptr(), 1);
    }
  }
  return erased;
}

std::tuple<torch::Tensor, torch::Tensor> EmbeddingStore::snapshot(bool expired_only, int64_t threshold) {
  // Size of the result is data dependent: this is a checkpoint / eviction-time call, one host read is fine.
  auto c = counters();
  const int64_t cap = std::max<int64_t>(c[RB_CTR_LIVE], 1);
  auto o = torch::TensorOptions().device(device_);
  auto ids = torch::empty({cap}, o.dtype(torch::kInt64));
  auto rows = torch::empty({cap}, o.dtype(torch::kInt32));
  auto counter = torch::zeros({1}, o.dtype(torch::kInt64));
  const bool use_filter = expired_only && last_seen_.defined();
  const int64_t* ls = use_filter ? last_seen_.data_ptr<int64_t>() : nullptr;
  if (device_.is_cuda()) {
    c10::cuda::CUDAGuard g(device_);
    rb_table_snapshot(view(), ids.data_ptr<int64_t>(), rows.data_ptr<int32_t>(), cap, counter.data_ptr<int64_t>(), ls, threshold,
                      use_filter ? 1 : 0, at::cuda::getCurrentCUDAStream());
  } else {
    rbc_table_snapshot(view(), ids.data_ptr<int64_t>(), rows.data_ptr<int32_t>(), cap, counter.data_ptr<int64_t>(), ls, threshold,
                       use_filter ? 1 : 0);
  }
  const int64_t n = std::min<int64_t>(counter.item<int64_t>(), cap);
  return {ids.narrow(0, 0, n), rows.narrow(0, 0, n)};
}

void EmbeddingStore::clear() {
  keys_.fill_(-1); rows_.fill_(-1); ctr_.zero_();
  for (auto& kv : slots_) kv.second.fill_(slot_fill_[kv.first]);
  if (last_seen_.defined()) last_seen_.zero_();
  rows_upper_ = bump_upper_ = index_upper_ = 0;
  est_new_ = -1; rows_prev_ = -1; index_prev_ = 0; seen_n_dev_ = 0;
  absorbed_issued_ = issued_total_;
}

int64_t EmbeddingStore::size() const { return counters()[RB_CTR_LIVE]; }

}  // namespace rbx
