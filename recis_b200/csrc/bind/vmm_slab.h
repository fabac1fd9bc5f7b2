// Device memory that grows in place: a reserved virtual address range with physical pages mapped on demand.
//
// A table's row slabs (embedding rows, optimizer state, last-seen steps, free list) used to grow by allocating a larger
// tensor and copying everything: a transient 2x of memory and a copy proportional to the table. Here a slab reserves
// virtual addresses for its largest size up front (cuMemAddressReserve) and maps physical memory chunk by chunk
// (cuMemCreate / cuMemMap / cuMemSetAccess) as the capacity grows: the base address never changes, nothing is copied, and
// growing costs the same whatever the table holds. The reference grows by appending fixed-size blocks to a vector
// (csrc/embedding/hashtable.cc:255-261, slot_group.cc:169-174), which avoids the copy at the price of a pointer table per
// kernel call; the virtual range keeps one flat [capacity, dim] array instead.
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint), so the library has no link-time dependency on
// the driver and loads on machines without one; where the calls are unavailable or fail, callers fall back to allocate + copy.
#pragma once
#include <torch/extension.h>
#include <memory>
#include <vector>

namespace rbx {

class VmmSlab : public std::enable_shared_from_this<VmmSlab> {
 public:
  // reserve `max_bytes` of address space on `device`; nullptr when virtual memory management is unavailable
  static std::shared_ptr<VmmSlab> create(int device, size_t max_bytes);
  ~VmmSlab();
  VmmSlab(const VmmSlab&) = delete;
  VmmSlab& operator=(const VmmSlab&) = delete;
  // make at least `bytes` usable (maps more physical memory; never moves or copies); false on failure or beyond the reservation
  bool ensure(size_t bytes);
  void* data() const { return reinterpret_cast<void*>(base_); }
  size_t mapped() const { return mapped_; }
  size_t reserved() const { return reserved_; }
  // tensor over the first sizes.numel() elements; keeps this slab alive for as long as the tensor lives
  torch::Tensor view(at::IntArrayRef sizes, torch::ScalarType dtype);

 private:
  VmmSlab() = default;
  int device_ = 0;
  unsigned long long base_ = 0;
  size_t reserved_ = 0, mapped_ = 0, granularity_ = 0;
  std::vector<std::pair<unsigned long long, size_t>> handles_;   // (allocation handle, bytes)
};

}  // namespace rbx
