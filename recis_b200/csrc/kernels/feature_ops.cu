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

inline int chunk_blocks(int64_t n) {
  int64_t b = (n + 4095) / 4096;
  return (int)std::min<int64_t>(std::max<int64_t>(b, 1), 148 * 8);
}

__device__ __forceinline__ int find_tensor(const int64_t* prefix, int T, int64_t i) {
  int lo = 0, hi = T;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (prefix[mid] <= i) lo = mid; else hi = mid; }
  return lo;
}

// Work is handed out in chunks of kChunk consecutive elements of the concatenated element space. Almost every chunk lies
// inside one tensor (features have far more than kChunk elements): the block looks the tensor up ONCE (two binary searches by
// thread 0), fetches that tensor's parameters once and streams the chunk with coalesced loads. Only a chunk that straddles a
// tensor boundary walks the prefix table per element.
constexpr int kChunk = 4096;

struct ChunkRange { int64_t c0, c1; int t_first, t_last; };

__device__ __forceinline__ ChunkRange chunk_range(const int64_t* prefix, int T, int64_t chunk, int64_t total, int* s_t) {
  ChunkRange r;
  r.c0 = chunk * kChunk;
  r.c1 = min(r.c0 + (int64_t)kChunk, total);
  __syncthreads();                                  // the previous chunk is done with s_t
  if (threadIdx.x == 0) { s_t[0] = find_tensor(prefix, T, r.c0); s_t[1] = find_tensor(prefix, T, r.c1 - 1); }
  __syncthreads();
  r.t_first = s_t[0]; r.t_last = s_t[1];
  return r;
}

__device__ __forceinline__ int advance_tensor(const int64_t* prefix, int t, int64_t i) {
  while (i >= prefix[t + 1]) ++t;
  return t;
}

// desc rows: [0] string-byte pointers (int8), [1] string offsets pointers (int32), [2] prefix over strings (T+1)
__global__ void __launch_bounds__(kThreads)
fused_hash_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int kind, int64_t* __restrict__ out) {
  __shared__ int s_t[2];
  const int64_t* bytes_ptr = desc; const int64_t* off_ptr = desc + (T + 1); const int64_t* prefix = desc + 2 * (T + 1);
  const int64_t n_chunks = (total + kChunk - 1) / kChunk;
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const ChunkRange r = chunk_range(prefix, T, chunk, total, s_t);
    int t = r.t_first;
    const int32_t* off = reinterpret_cast<const int32_t*>(off_ptr[t]);
    const char* bytes = reinterpret_cast<const char*>(bytes_ptr[t]);
    int64_t base = prefix[t];
    for (int64_t i = r.c0 + threadIdx.x; i < r.c1; i += kThreads) {
      if (r.t_first != r.t_last) {
        const int t2 = advance_tensor(prefix, t, i);
        if (t2 != t) { t = t2; off = reinterpret_cast<const int32_t*>(off_ptr[t]); bytes = reinterpret_cast<const char*>(bytes_ptr[t]); base = prefix[t]; }
      }
      const int64_t k = i - base;
      const int32_t o0 = off[k], o1 = off[k + 1];
      const char* sp = bytes + o0;
      const size_t len = (size_t)(o1 - o0);
      out[i] = (int64_t)(kind == 0 ? rb::hash::farm_fingerprint64(sp, len) : rb::hash::murmur64a(sp, len, 0));
    }
  }
}

// desc rows: [0] value pointers (float), [1] prefix (T+1), [2] boundary pointers (float), [3] boundary counts
constexpr int kMaxSmemBounds = 2048;
__global__ void __launch_bounds__(kThreads)
fused_bucketize_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int64_t* __restrict__ out) {
  __shared__ int s_t[2];
  __shared__ float s_bnd[kMaxSmemBounds];
  const int64_t* val_ptr = desc; const int64_t* prefix = desc + (T + 1); const int64_t* bnd_ptr = desc + 2 * (T + 1);
  const int64_t* bnd_len = desc + 3 * (T + 1);
  const int64_t n_chunks = (total + kChunk - 1) / kChunk;
  int cached_t = -1;                                 // tensor whose boundaries sit in s_bnd
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const ChunkRange r = chunk_range(prefix, T, chunk, total, s_t);
    if (r.t_first == r.t_last && bnd_len[r.t_first] <= kMaxSmemBounds) {
      const int t = r.t_first;
      const int nb = (int)bnd_len[t];
      if (cached_t != t) {                           // uniform for the block: every thread tracks the same cached_t
        const float* b = reinterpret_cast<const float*>(bnd_ptr[t]);
        for (int j = threadIdx.x; j < nb; j += kThreads) s_bnd[j] = b[j];
        cached_t = t;
        __syncthreads();
      }
      const float* v = reinterpret_cast<const float*>(val_ptr[t]) + (r.c0 - prefix[t]);
      const int n = (int)(r.c1 - r.c0);
      for (int i = threadIdx.x; i < n; i += kThreads) {
        const float x = v[i];
        int lo = 0, hi = nb;                         // first boundary > x  ==  count of boundaries <= x
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (!(x < s_bnd[mid])) lo = mid + 1; else hi = mid; }
        out[r.c0 + i] = lo;
      }
    } else {
      int t = r.t_first;
      for (int64_t i = r.c0 + threadIdx.x; i < r.c1; i += kThreads) {
        t = advance_tensor(prefix, t, i);
        const float x = reinterpret_cast<const float*>(val_ptr[t])[i - prefix[t]];
        const float* b = reinterpret_cast<const float*>(bnd_ptr[t]);
        int lo = 0, hi = (int)bnd_len[t];
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (!(x < b[mid])) lo = mid + 1; else hi = mid; }
        out[i] = lo;
      }
    }
  }
}

// x mod m without a 64-bit division: q = hi64(x * magic) with magic = floor(2^64 / m) is floor(x / m) or one less.
__device__ __forceinline__ uint64_t mod_by_magic(uint64_t x, uint64_t m, uint64_t magic) {
  uint64_t r = x - __umul64hi(x, magic) * m;
  if (r >= m) r -= m;
  if (r >= m) r -= m;
  return r;
}

// desc rows: [0] value pointers (int64), [1] prefix (T+1), [2] modulus, [3] floor(2^64 / modulus) (0 for modulus 1)
__global__ void __launch_bounds__(kThreads)
fused_mod_kernel(const int64_t* __restrict__ desc, int T, int64_t total, int64_t* __restrict__ out) {
  __shared__ int s_t[2];
  const int64_t* val_ptr = desc; const int64_t* prefix = desc + (T + 1); const int64_t* mod = desc + 2 * (T + 1);
  const int64_t* magic = desc + 3 * (T + 1);
  const int64_t n_chunks = (total + kChunk - 1) / kChunk;
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const ChunkRange r = chunk_range(prefix, T, chunk, total, s_t);
    if (r.t_first == r.t_last) {
      const int t = r.t_first;
      const uint64_t m = (uint64_t)mod[t], mg = (uint64_t)magic[t];
      const int64_t* v = reinterpret_cast<const int64_t*>(val_ptr[t]) + (r.c0 - prefix[t]);
      const int n = (int)(r.c1 - r.c0);
      if (m == 1) { for (int i = threadIdx.x; i < n; i += kThreads) out[r.c0 + i] = 0; continue; }
#pragma unroll 4
      for (int i = threadIdx.x; i < n; i += kThreads) out[r.c0 + i] = (int64_t)mod_by_magic((uint64_t)v[i], m, mg);
    } else {
      int t = r.t_first;
      for (int64_t i = r.c0 + threadIdx.x; i < r.c1; i += kThreads) {
        t = advance_tensor(prefix, t, i);
        const uint64_t x = (uint64_t) reinterpret_cast<const int64_t*>(val_ptr[t])[i - prefix[t]];
        out[i] = (int64_t)(x % (uint64_t)mod[t]);
      }
    }
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
  fused_hash_kernel<<<chunk_blocks(total), kThreads, 0, st>>>(desc, T, total, kind, out);
  rb::note_launch();
}
void rb_fused_bucketize(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_bucketize_kernel<<<chunk_blocks(total), kThreads, 0, st>>>(desc, T, total, out);
  rb::note_launch();
}
void rb_fused_mod(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_mod_kernel<<<chunk_blocks(total), kThreads, 0, st>>>(desc, T, total, out);
  rb::note_launch();
}
void rb_fused_multi_hash(const int64_t* desc, int T, int64_t total, int kmax, int64_t* out, cudaStream_t st) {
  if (total <= 0) return;
  fused_multi_hash_kernel<<<blocks_for(total), kThreads, 0, st>>>(desc, T, total, kmax, out);
  rb::note_launch();
}

}  // extern "C"
