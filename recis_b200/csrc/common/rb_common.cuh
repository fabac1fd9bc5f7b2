// Shared device helpers for every sm_100a kernel of this library.
//
// Conventions:
//  * kernels never trap or assert; a failure sets a bit in a device status word
//    that the host reads at a step boundary.
//  * every spin wait is bounded (see rb_comm.cuh).
//  * row payloads are moved with 16-byte vector accesses whenever the row
//    length allows it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

namespace rb {

constexpr uint64_t kEmptyKey = 0xFFFFFFFFFFFFFFFFull;   // id -1 : never a legal id
constexpr uint64_t kErasedKey = 0xFFFFFFFFFFFFFFFEull;  // id -2 : tombstone
constexpr int32_t kRowPending = -1;

// status bits (device status word, int64)
enum StatusBits : int64_t {
  kStatusOk = 0,
  kStatusRowsExhausted = 1,    // row arena full
  kStatusIndexFull = 2,        // probe sequence wrapped without an empty slot
  kStatusWaitTimeout = 4,      // a bounded peer wait gave up
  kStatusWindowOverflow = 8,   // a communication window was too small
  kStatusBadIndex = 16,        // an index failed a bounds check and was skipped
};

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x) {
  // splitmix64 finaliser: full avalanche, cheap.
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

// Owner rank of an id: the low 16 bits select one of 65536 slices; rank r owns a
// contiguous run of slices, the first (65536 % W) ranks owning one slice more.
__host__ __device__ __forceinline__ int owner_of(uint64_t key, int world) {
  const uint32_t slice = (uint32_t)(key & 0xFFFFu);
  const uint32_t q = 65536u / (uint32_t)world, r = 65536u % (uint32_t)world;
  const uint32_t big = r * (q + 1);
  return slice < big ? (int)(slice / (q + 1)) : (int)(r + (slice - big) / q);
}

// ---------------------------------------------------------------- Philox4x32-10
struct Philox {
  uint32_t k0, k1;
  __host__ __device__ static inline void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
    uint64_t p = (uint64_t)a * b; hi = (uint32_t)(p >> 32); lo = (uint32_t)p;
  }
  __host__ __device__ inline void gen(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t out[4]) const {
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      uint32_t h0, l0, h1, l1;
      mulhilo(0xD2511F53u, c0, h0, l0);
      mulhilo(0xCD9E8D57u, c2, h1, l1);
      c0 = h1 ^ c1 ^ a; c1 = l1; c2 = h0 ^ c3 ^ b; c3 = l0;
      a += 0x9E3779B9u; b += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
  }
};

__host__ __device__ __forceinline__ float u32_to_unit(uint32_t x) {
  // (0,1]: never returns 0 so log() is safe.
  return ((float)(x >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

// Row initialiser description. The value of element d of the row of id `key`
// is a pure function of (seed, key, d): independent of insertion order, of the
// shard count and of the device, so seeded runs reproduce on CPU and GPU.
enum InitKind : int { kInitConstant = 0, kInitUniform = 1, kInitNormal = 2, kInitTruncNormal = 3 };
struct InitSpec {
  int kind;
  float a;   // constant value | uniform low  | normal mean
  float b;   //                | uniform high | normal std
  float lo;  // trunc normal lower bound (absolute)
  float hi;  // trunc normal upper bound (absolute)
  uint64_t seed;
};

// Four values for columns [4*q, 4*q+4) of the row of `key`.
__host__ __device__ inline void init_quad(const InitSpec& s, uint64_t key, uint32_t q, float out[4]) {
  if (s.kind == kInitConstant) { out[0] = out[1] = out[2] = out[3] = s.a; return; }
  Philox ph{(uint32_t)s.seed, (uint32_t)(s.seed >> 32)};
  uint32_t r[4];
  ph.gen((uint32_t)key, (uint32_t)(key >> 32), q, 0u, r);
  if (s.kind == kInitUniform) {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = s.a + (s.b - s.a) * u32_to_unit(r[i]);
    return;
  }
  // Box-Muller on two pairs
  float n[4];
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    float u1 = u32_to_unit(r[2 * p]), u2 = u32_to_unit(r[2 * p + 1]);
    float rad = sqrtf(-2.0f * logf(u1));
    float sn, cs;
#ifdef __CUDA_ARCH__
    sincospif(2.0f * u2, &sn, &cs);
#else
    sn = sinf(6.283185307179586f * u2); cs = cosf(6.283185307179586f * u2);
#endif
    n[2 * p] = rad * cs; n[2 * p + 1] = rad * sn;
  }
  if (s.kind == kInitNormal) {
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = s.a + s.b * n[i];
    return;
  }
  // truncated normal: resample (bounded) with fresh counters, clamp as a last resort
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float v = s.a + s.b * n[i];
    uint32_t tries = 1;
    while ((v < s.lo || v > s.hi) && tries < 16) {
      uint32_t rr[4];
      ph.gen((uint32_t)key, (uint32_t)(key >> 32), q, tries * 4u + (uint32_t)i + 1u, rr);
      float u1 = u32_to_unit(rr[0]), u2 = u32_to_unit(rr[1]);
      v = s.a + s.b * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
      ++tries;
    }
    out[i] = fminf(fmaxf(v, s.lo), s.hi);
  }
}

#ifdef __CUDACC__
__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
// vector reduction to global memory (sm_90+): one 16-byte red instead of four scalar atomics.
__device__ __forceinline__ void red_add_f4(float* p, float4 v) {
  atomicAdd(reinterpret_cast<float4*>(p), v);
}
__device__ __forceinline__ float4 f4_fma(float w, float4 a, float4 acc) {
  acc.x = fmaf(w, a.x, acc.x); acc.y = fmaf(w, a.y, acc.y); acc.z = fmaf(w, a.z, acc.z); acc.w = fmaf(w, a.w, acc.w);
  return acc;
}
__device__ __forceinline__ void set_status(int64_t* status, int64_t bit) {
  if (status) atomicOr(reinterpret_cast<unsigned long long*>(status), (unsigned long long)bit);
}
#endif

inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

}  // namespace rb
