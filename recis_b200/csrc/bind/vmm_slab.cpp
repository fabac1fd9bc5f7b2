// See vmm_slab.h.
#include "vmm_slab.h"
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

namespace rbx {

namespace {

struct DriverFns {
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  bool ok = false;
};

const DriverFns& driver() {
  static DriverFns fns;
  static std::once_flag once;
  std::call_once(once, [] {
    auto get = [](const char* name, void** out) {
      cudaDriverEntryPointQueryResult st;
      return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &st) == cudaSuccess && st == cudaDriverEntryPointSuccess && *out != nullptr;
    };
    bool ok = true;
    ok &= get("cuMemAddressReserve", reinterpret_cast<void**>(&fns.reserve));
    ok &= get("cuMemAddressFree", reinterpret_cast<void**>(&fns.addr_free));
    ok &= get("cuMemCreate", reinterpret_cast<void**>(&fns.create));
    ok &= get("cuMemRelease", reinterpret_cast<void**>(&fns.release));
    ok &= get("cuMemMap", reinterpret_cast<void**>(&fns.map));
    ok &= get("cuMemUnmap", reinterpret_cast<void**>(&fns.unmap));
    ok &= get("cuMemSetAccess", reinterpret_cast<void**>(&fns.set_access));
    ok &= get("cuMemGetAllocationGranularity", reinterpret_cast<void**>(&fns.granularity));
    (void)cudaGetLastError();                 // a failed lookup must not leave a sticky runtime error behind
    fns.ok = ok;
  });
  return fns;
}

CUmemAllocationProp props_for(int device) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

}  // namespace

std::shared_ptr<VmmSlab> VmmSlab::create(int device, size_t max_bytes) {
  const DriverFns& d = driver();
  if (!d.ok || max_bytes == 0) return nullptr;
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  if (cudaFree(nullptr) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }      // make sure the device's context exists
  auto prop = props_for(device);
  size_t gran = 0;
  if (d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return nullptr;
  std::shared_ptr<VmmSlab> s(new VmmSlab());
  s->device_ = device;
  s->granularity_ = gran;
  s->reserved_ = (max_bytes + gran - 1) / gran * gran;
  CUdeviceptr base = 0;
  if (d.reserve(&base, s->reserved_, gran, 0, 0) != CUDA_SUCCESS) return nullptr;
  s->base_ = (unsigned long long)base;
  return s;
}

bool VmmSlab::ensure(size_t bytes) {
  if (bytes <= mapped_) return true;
  if (bytes > reserved_) return false;
  const DriverFns& d = driver();
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_);
  // map one more physical allocation behind what is mapped; at least 64 MiB at a time so that a table that grows row by row
  // does not end up with thousands of mappings
  size_t want = bytes - mapped_;
  const size_t min_chunk = std::max<size_t>(granularity_, (size_t)64 << 20);
  if (want < min_chunk) want = std::min(min_chunk, reserved_ - mapped_);
  want = (want + granularity_ - 1) / granularity_ * granularity_;
  auto prop = props_for(device_);
  CUmemGenericAllocationHandle h = 0;
  if (d.create(&h, want, &prop, 0) != CUDA_SUCCESS) return false;
  if (d.map((CUdeviceptr)(base_ + mapped_), want, 0, h, 0) != CUDA_SUCCESS) { d.release(h); return false; }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.set_access((CUdeviceptr)(base_ + mapped_), want, &acc, 1) != CUDA_SUCCESS) {
    d.unmap((CUdeviceptr)(base_ + mapped_), want);
    d.release(h);
    return false;
  }
  handles_.emplace_back((unsigned long long)h, want);
  mapped_ += want;
  return true;
}

VmmSlab::~VmmSlab() {
  const DriverFns& d = driver();
  if (!d.ok || base_ == 0) return;
  // the memory may still be in use by queued kernels: wait for the device before unmapping (tables die rarely)
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  size_t off = 0;
  for (auto& hb : handles_) {
    d.unmap((CUdeviceptr)(base_ + off), hb.second);
    d.release((CUmemGenericAllocationHandle)hb.first);
    off += hb.second;
  }
  d.addr_free((CUdeviceptr)base_, reserved_);
  cudaSetDevice(prev);
}

torch::Tensor VmmSlab::view(at::IntArrayRef sizes, torch::ScalarType dtype) {
  auto self = shared_from_this();
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, (c10::DeviceIndex)device_);
  return torch::from_blob(data(), sizes, [self](void*) mutable { self.reset(); }, opts);
}

}  // namespace rbx
