// Epilogue helpers shared by the tcgen05 GEMM kernels: 32 consecutive fp32 values of one output row become bf16 or fp32 and go
// either straight to global memory (row32 / red32) or into a shared-memory slab laid out as boxes of 32 rows x 128 bytes in the
// 128-byte swizzle, which is what a TMA store (or add-reduction) of such a box expects (stage32).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace rb {
namespace gemm {

template <typename OutT> struct Store;
template <> struct Store<__nv_bfloat16> {
  static __device__ __forceinline__ void row32(__nv_bfloat16* dst, const float (&v)[32], int valid, bool vec_ok) {
    if (vec_ok && valid == 32) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]), p1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]), p3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
        u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
        d4[q] = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
  }
  static __device__ __forceinline__ void red32(__nv_bfloat16*, const float (&)[32], int, bool) {}   // split-K needs fp32 output
  // 32 consecutive columns of one row into the swizzled staging slab: box of 64 columns, four 16-byte chunks
  static constexpr int kBoxCols = 64;
  static __device__ __forceinline__ void stage32(uint8_t* slab, int lane, int c0, const float (&v)[32]) {
    uint8_t* row = slab + (c0 >> 6) * 4096 + lane * 128;
    const int jbase = (c0 & 63) >> 3;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]), p1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]), p3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
      u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(row + (((jbase + q) ^ (lane & 7)) << 4)) = u;
    }
  }
};
template <> struct Store<float> {
  static __device__ __forceinline__ void row32(float* dst, const float (&v)[32], int valid, bool vec_ok) {
    if (vec_ok && valid == 32) {
      float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
      for (int q = 0; q < 8; ++q) d4[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (j < valid) dst[j] = v[j];
    }
  }
  static __device__ __forceinline__ void red32(float* dst, const float (&v)[32], int valid, bool vec_ok) {
    if (vec_ok && valid == 32) {
#pragma unroll
      for (int q = 0; q < 8; ++q) atomicAdd(reinterpret_cast<float4*>(dst) + q, make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (j < valid) atomicAdd(dst + j, v[j]);
    }
  }
  // 32 consecutive columns of one row = one full 128-byte row of a 32-column box: eight 16-byte chunks
  static constexpr int kBoxCols = 32;
  static __device__ __forceinline__ void stage32(uint8_t* slab, int lane, int c0, const float (&v)[32]) {
    uint8_t* row = slab + (c0 >> 5) * 4096 + lane * 128;
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<float4*>(row + ((q ^ (lane & 7)) << 4)) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
  }
};

// v[j] = 0 where the mask row (32 bf16 starting at mrow) is not positive; a row outside the matrix becomes all zeros
__device__ __forceinline__ void apply_mask32(float (&v)[32], const __nv_bfloat16* mrow, int valid, bool row_ok) {
  if (!row_ok) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = 0.f;
    return;
  }
  if (valid == 32 && (reinterpret_cast<uintptr_t>(mrow) & 15) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 u = reinterpret_cast<const uint4*>(mrow)[q];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 y = __bfloat1622float2(h[e]);
        if (!(y.x > 0.f)) v[q * 8 + 2 * e] = 0.f;
        if (!(y.y > 0.f)) v[q * 8 + 2 * e + 1] = 0.f;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid && !(__bfloat162float(mrow[j]) > 0.f)) v[j] = 0.f;
  }
}

// Column sums of a 32 x 32 block held one row per lane: after five exchange steps lane l holds the sum of column l over the warp's
// 32 rows (each step keeps half of the columns and adds the other lane's copy of them), which it adds to dst[l]. Destroys v.
__device__ __forceinline__ void column_sums32(float (&v)[32], int lane, int valid, float* dst) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < off; ++j) {
      const float keep = up ? v[j + off] : v[j];
      const float give = up ? v[j] : v[j + off];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, give, off);
    }
  }
  if (lane < valid) atomicAdd(dst + lane, v[0]);
}

}  // namespace gemm
}  // namespace rb
