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

// Storage type of embedding rows. Rows may be kept in 32- or 16-bit floating point, or (read-only tables) as 8-bit integers;
// optimizer state and every accumulation stay fp32. Codes are shared by the CUDA kernels, their CPU twins and the bindings.
enum RowDType : int { kRowF32 = 0, kRowF16 = 1, kRowBF16 = 2, kRowI8 = 3 };
__host__ __device__ __forceinline__ int row_elem_size(int dtype) { return dtype == kRowF32 ? 4 : (dtype == kRowI8 ? 1 : 2); }

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

#ifdef __CUDACC__
}  // namespace rb
#include <cuda_bf16.h>
#include <cuda_fp16.h>
namespace rb {
// Four consecutive row elements <-> float4 (the address is aligned to four elements), and single elements.
template <typename T> struct RowIO;
template <> struct RowIO<float> {
  static __device__ __forceinline__ float4 ld4(const float* p) { return ld_f4(p); }
  static __device__ __forceinline__ void st4(float* p, float4 v) { st_f4(p, v); }
  static __device__ __forceinline__ float ld1(const float* p) { return *p; }
  static __device__ __forceinline__ void st1(float* p, float v) { *p = v; }
};
template <> struct RowIO<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct RowIO<__half> {
  static __device__ __forceinline__ float4 ld4(const __half* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st4(__half* p, float4 v) {
    uint2 raw;
    *reinterpret_cast<__half2*>(&raw.x) = __floats2half2_rn(v.x, v.y);
    *reinterpret_cast<__half2*>(&raw.y) = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
  }
  static __device__ __forceinline__ float ld1(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st1(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct RowIO<int8_t> {
  static __device__ __forceinline__ float4 ld4(const int8_t* p) {
    const char4 c = *reinterpret_cast<const char4*>(p);
    return make_float4((float)c.x, (float)c.y, (float)c.z, (float)c.w);
  }
  static __device__ __forceinline__ int8_t q(float v) { return (int8_t)max(-128, min(127, __float2int_rn(v))); }
  static __device__ __forceinline__ void st4(int8_t* p, float4 v) {
    char4 c; c.x = q(v.x); c.y = q(v.y); c.z = q(v.z); c.w = q(v.w);
    *reinterpret_cast<char4*>(p) = c;
  }
  static __device__ __forceinline__ float ld1(const int8_t* p) { return (float)*p; }
  static __device__ __forceinline__ void st1(int8_t* p, float v) { *p = q(v); }
};
#endif

// Calls f(T{}) with T the row type of `dtype`. int8 rows are read-only: kernels that update rows pass with_i8 = false.
#define RB_DISPATCH_ROW(dtype, with_i8, ...)                                             \
  do {                                                                                   \
    switch (dtype) {                                                                     \
      case rb::kRowF32: { using T = float; __VA_ARGS__; } break;                         \
      case rb::kRowF16: { using T = __half; __VA_ARGS__; } break;                        \
      case rb::kRowBF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;                \
      case rb::kRowI8: if (with_i8) { using T = int8_t; __VA_ARGS__; } break;            \
      default: break;                                                                    \
    }                                                                                    \
  } while (0)

inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

}  // namespace rb
