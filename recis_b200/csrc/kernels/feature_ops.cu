// Feature-engine kernels (sm_100a): every op processes ALL features of an execution step in one launch.
//
// A launch walks the concatenated element space of its input tensors; a small descriptor table (device resident,
// copied asynchronously from pinned memory by the caller) maps a flat index to (tensor, element). This is what the
// reference does with its fused launcher (csrc/cuda/element_wise_kernel.cuh:15-91), minus the stream synchronisation and
// raw allocation it performs on every call.
//   fused_hash        csrc/ops/fused_hash_kernel.cu:47-459        byte strings -> FarmHash Fingerprint64 / MurmurHash64A
//   fused_bucketize   csrc/ops/fused_bucketized_kernel.cu:11-60   value -> number of boundaries <= value
//   fused_mod         csrc/ops/fused_uint64_mod_kernel.cu:12-39   uint64(x) % m
//   fused_multi_hash  csrc/ops/multi_hash_kernel.cu:11-75         (((x*mul) % p + p) % p) % bucket, up to 4 per feature
#include "../common/rb_common.cuh"
#include "../common/rb_hash.cuh"
#include "../common/rb_launch.h"
#include "rb_feature.h"

namespace {

constexpr int kThreads = 256;

inline int blocks_for(int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  return (int)std::min<int64_t>(std::max<int64_t>(b, 1), 148 * 16);
}

__device__ __forceinline__ int find_tensor(const int64_t* prefix, int T, int64_t i) {
  int lo = 0, hi = T;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (prefix[mid] <= i) lo = mid; else hi = mid; }
  return lo;
}

// desc rows: [0] string-byte pointers (int8), [1] string offsets pointers (int32), [2] prefix over strings (T+1)
__global__ void __launch_bounds__(kThreads)
fused_hash_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int kind, int64_t* __restrict__ out) {
  const int64_t* bytes_ptr = desc; const int64_t* off_ptr = desc + (T + 1); const int64_t* prefix = desc + 2 * (T + 1);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = find_tensor(prefix, T, i);
    const int64_t k = i - prefix[t];
    const int32_t* off = reinterpret_cast<const int32_t*>(off_ptr[t]);
    const char* s = reinterpret_cast<const char*>(bytes_ptr[t]) + off[k];
    const size_t len = (size_t)(off[k + 1] - off[k]);
    out[i] = (int64_t)(kind == 0 ? rb::hash::farm_fingerprint64(s, len) : rb::hash::murmur64a(s, len, 0));
  }
}

// desc rows: [0] value pointers (float), [1] prefix (T+1), [2] boundary pointers (float), [3] boundary counts
__global__ void __launch_bounds__(kThreads)
fused_bucketize_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int64_t* __restrict__ out) {
  const int64_t* val_ptr = desc; const int64_t* prefix = desc + (T + 1); const int64_t* bnd_ptr = desc + 2 * (T + 1);
  const int64_t* bnd_len = desc + 3 * (T + 1);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = find_tensor(prefix, T, i);
    const float v = reinterpret_cast<const float*>(val_ptr[t])[i - prefix[t]];
    const float* b = reinterpret_cast<const float*>(bnd_ptr[t]);
    int lo = 0, hi = (int)bnd_len[t];            // first boundary > v  ==  count of boundaries <= v
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (!(v < b[mid])) lo = mid + 1; else hi = mid; }
    out[i] = lo;
  }
}

// desc rows: [0] value pointers (int64), [1] prefix (T+1), [2] modulus
__global__ void __launch_bounds__(kThreads)
fused_mod_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int64_t* __restrict__ out) {
  const int64_t* val_ptr = desc; const int64_t* prefix = desc + (T + 1); const int64_t* mod = desc + 2 * (T + 1);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = find_tensor(prefix, T, i);
    const uint64_t x = (uint64_t) reinterpret_cast<const int64_t*>(val_ptr[t])[i - prefix[t]];
    out[i] = (int64_t)(x % (uint64_t)mod[t]);
  }
}

// desc rows: [0] value pointers, [1] prefix, [2] hash count K_t, [3..6] muls, [7..10] primes, [11..14] buckets
// out: K_max planes of `total` elements; plane k holds hash k of every element (unused planes of a tensor are 0).
__global__ void __launch_bounds__(kThreads)
fused_multi_hash_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int kmax, int64_t* __restrict__ out) {
  const int64_t* val_ptr = desc; const int64_t* prefix = desc + (T + 1); const int64_t* kcnt = desc + 2 * (T + 1);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = find_tensor(prefix, T, i);
    const int64_t x = reinterpret_cast<const int64_t*>(val_ptr[t])[i - prefix[t]];
    for (int k = 0; k < kmax; ++k) {
      int64_t r = 0;
      if (k < kcnt[t]) {
        const int64_t mul = desc[(3 + k) * (T + 1) + t], p = desc[(7 + k) * (T + 1) + t], bucket = desc[(11 + k) * (T + 1) + t];
        r = (int64_t)((uint64_t)x * (uint64_t)mul);     // wrapping multiply, as int64 overflow does in the reference
        r = ((r % p) + p) % p;
        r = r % bucket;
      }
      out[(int64_t)k * total + i] = r;
    }
  }
}

}  // namespace

extern "C" {

void rb_fused_hash(const int64_t* desc, int T, int64_t total, int kind, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_hash_kernel<<<blocks_for(total), kThreads, 0, st>>>(desc, T, total, kind, out);
  rb::note_launch();
}
void rb_fused_bucketize(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_bucketize_kernel<<<blocks_for(total), kThreads, 0, st>>>(desc, T, total, out);
  rb::note_launch();
}
void rb_fused_mod(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_mod_kernel<<<blocks_for(total), kThreads, 0, st>>>(desc, T, total, out);
  rb::note_launch();
}
void rb_fused_multi_hash(const int64_t* desc, int T, int64_t total, int kmax, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_multi_hash_kernel<<<blocks_for(total), kThreads, 0, st>>>(desc, T, total, kmax, out);
  rb::note_launch();
}

}  // extern "C"
