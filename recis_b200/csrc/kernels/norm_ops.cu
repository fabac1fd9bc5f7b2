// LayerNorm over the last dimension of a [rows, H] fp32 matrix, forward and backward, one warp per row.
//
// forward:  y = (x - mean) * rstd * gamma + beta, written as bf16 (to feed a GEMM without a separate cast) or fp32;
//           mean and rstd are kept per row for the backward pass.
// backward: dx = rstd * (g - mean_H(g) - xhat * mean_H(g * xhat)) with g = dy * gamma and xhat = (x - mean) * rstd;
//           dgamma = sum_rows dy * xhat and dbeta = sum_rows dy are accumulated in registers over the rows a warp visits,
//           reduced over the warps of a block in shared memory and added to the (zeroed) outputs with one atomic per block
//           and column. One pass over x and dy; torch's layer norm backward makes three (input gradient, then the two
//           weight gradients through a separate column reduction), see the reference's use of nn.LayerNorm in
//           examples/seq2seq/transformer.py.
//
// H must be a multiple of 4 and at most 1024; a row is held in registers as NV float4 per lane (NV = ceil(H / 128)).
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "rb_dense.h"
#include <cuda_bf16.h>
#include <algorithm>

namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T> struct Io;
template <> struct Io<float> {
  static __device__ __forceinline__ float4 ld(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void st(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Io<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <int NV, typename OutT>
__global__ void __launch_bounds__(kWarps * 32)
layer_norm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta, int64_t rows, int H,
                      float eps, OutT* __restrict__ y, float* __restrict__ stats) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), n_warps = (int64_t)gridDim.x * kWarps;
  float4 g[NV], b[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    g[i] = c < H ? *reinterpret_cast<const float4*>(gamma + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    b[i] = c < H ? *reinterpret_cast<const float4*>(beta + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_h = 1.f / (float)H;
  for (int64_t r = warp; r < rows; r += n_warps) {
    const float* xr = x + r * H;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 4;
      v[i] = c < H ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      s += v[i].x + v[i].y + v[i].z + v[i].w;
    }
    const float mean = warp_sum(s) * inv_h;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 4;
      if (c < H) {
        const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
        q += a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3;
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_h + eps);
    OutT* yr = y + r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 4;
      if (c < H)
        Io<OutT>::st(yr + c, make_float4((v[i].x - mean) * rstd * g[i].x + b[i].x, (v[i].y - mean) * rstd * g[i].y + b[i].y,
                                         (v[i].z - mean) * rstd * g[i].z + b[i].z, (v[i].w - mean) * rstd * g[i].w + b[i].w));
    }
    if (lane == 0) { stats[2 * r] = mean; stats[2 * r + 1] = rstd; }
  }
}

template <int NV, typename InT>
__global__ void __launch_bounds__(kWarps * 32)
layer_norm_bwd_kernel(const InT* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ stats,
                      const float* __restrict__ gamma, int64_t rows, int H, float* __restrict__ dx, float* __restrict__ dgamma,
                      float* __restrict__ dbeta) {
  extern __shared__ float red[];                 // [kWarps][2][NV * 128]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * kWarps + w, n_warps = (int64_t)gridDim.x * kWarps;
  float4 g[NV], ag[NV], ab[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    g[i] = c < H ? *reinterpret_cast<const float4*>(gamma + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    ag[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float inv_h = 1.f / (float)H;
  for (int64_t r = warp; r < rows; r += n_warps) {
    const float mean = stats[2 * r], rstd = stats[2 * r + 1];
    const float* xr = x + r * H;
    const InT* dr = dy + r * H;
    float4 xh[NV], gd[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 4;
      if (c < H) {
        const float4 xv = *reinterpret_cast<const float4*>(xr + c);
        const float4 d = Io<InT>::ld(dr + c);
        xh[i] = make_float4((xv.x - mean) * rstd, (xv.y - mean) * rstd, (xv.z - mean) * rstd, (xv.w - mean) * rstd);
        gd[i] = make_float4(d.x * g[i].x, d.y * g[i].y, d.z * g[i].z, d.w * g[i].w);
        s1 += gd[i].x + gd[i].y + gd[i].z + gd[i].w;
        s2 += gd[i].x * xh[i].x + gd[i].y * xh[i].y + gd[i].z * xh[i].z + gd[i].w * xh[i].w;
        ag[i].x += d.x * xh[i].x; ag[i].y += d.y * xh[i].y; ag[i].z += d.z * xh[i].z; ag[i].w += d.w * xh[i].w;
        ab[i].x += d.x; ab[i].y += d.y; ab[i].z += d.z; ab[i].w += d.w;
      } else {
        xh[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        gd[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const float m1 = warp_sum(s1) * inv_h, m2 = warp_sum(s2) * inv_h;
    float* dxr = dx + r * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 4;
      if (c < H)
        *reinterpret_cast<float4*>(dxr + c) = make_float4(rstd * (gd[i].x - m1 - xh[i].x * m2), rstd * (gd[i].y - m1 - xh[i].y * m2),
                                                          rstd * (gd[i].z - m1 - xh[i].z * m2), rstd * (gd[i].w - m1 - xh[i].w * m2));
    }
  }
  // weight gradients: warps of the block -> shared memory -> one atomic per column and block
  constexpr int W = NV * 128;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    *reinterpret_cast<float4*>(&red[(w * 2 + 0) * W + c]) = ag[i];
    *reinterpret_cast<float4*>(&red[(w * 2 + 1) * W + c]) = ab[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * W; c += kWarps * 32) {
    const int which = c / W, col = c - which * W;
    if (col >= H) continue;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kWarps; ++k) s += red[(k * 2 + which) * W + col];
    atomicAdd((which == 0 ? dgamma : dbeta) + col, s);
  }
}

// dy[m, n] = (relu && y[m, n] <= 0) ? 0 : dout[m, n]; db[n] += sum_m dy[m, n]. A thread owns 8 consecutive columns (one 16-byte
// load per operand and row); the block's threads tile (rows per pass) x (column groups); column sums stay in registers over the
// block's rows and meet in shared memory at the end.
template <bool WRITE>
__global__ void __launch_bounds__(256)
relu_bwd_bias_vec_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dout, int64_t M, int N, int relu,
                         __nv_bfloat16* __restrict__ dy, float* __restrict__ db, int groups_per_block) {
  __shared__ float part[256 * 8];
  const int grp = threadIdx.x % groups_per_block;                 // column group inside the block's column window
  const int rlane = threadIdx.x / groups_per_block, rlanes = 256 / groups_per_block;
  const int col = (blockIdx.x * groups_per_block + grp) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (col < N) {
    for (int64_t m = (int64_t)blockIdx.y * rlanes + rlane; m < M; m += (int64_t)gridDim.y * rlanes) {
      const int64_t o = m * N + col;
      uint4 d = *reinterpret_cast<const uint4*>(dout + o);
      __nv_bfloat162* dp = reinterpret_cast<__nv_bfloat162*>(&d);
      if (relu) {
        const uint4 yv = *reinterpret_cast<const uint4*>(y + o);
        const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 yy = __bfloat1622float2(yp[j]);
          float2 dd = __bfloat1622float2(dp[j]);
          if (!(yy.x > 0.f)) dd.x = 0.f;
          if (!(yy.y > 0.f)) dd.y = 0.f;
          dp[j] = __floats2bfloat162_rn(dd.x, dd.y);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 dd = __bfloat1622float2(dp[j]);
        acc[2 * j] += dd.x; acc[2 * j + 1] += dd.y;
      }
      if (WRITE) *reinterpret_cast<uint4*>(dy + o) = d;
    }
  }
  if (db == nullptr) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) part[(rlane * groups_per_block + grp) * 8 + j] = acc[j];
  __syncthreads();
  for (int c = threadIdx.x; c < groups_per_block * 8; c += 256) {
    const int gcol = blockIdx.x * groups_per_block * 8 + c;
    if (gcol >= N) continue;
    float s = 0.f;
    for (int k = 0; k < rlanes; ++k) s += part[(k * groups_per_block) * 8 + c];
    atomicAdd(db + gcol, s);
  }
}

int grid_rows(int64_t rows) { return (int)std::min<int64_t>(std::max<int64_t>((rows + kWarps - 1) / kWarps, 1), 148 * 8); }

}  // namespace

extern "C" {

int rb_layer_norm_fwd(const float* x, const float* gamma, const float* beta, int64_t rows, int H, float eps, void* y, int y_bf16,
                      float* stats, cudaStream_t st) {
  if (H % 4 != 0 || H > 1024 || H <= 0) return 1;
  if (rows <= 0) return 0;
  const int nv = (H + 127) / 128;
  const int grid = grid_rows(rows);
#define RB_LN_FWD(NV)                                                                                                             \
  if (y_bf16) layer_norm_fwd_kernel<NV, __nv_bfloat16><<<grid, kWarps * 32, 0, st>>>(x, gamma, beta, rows, H, eps,                 \
                                                                                      reinterpret_cast<__nv_bfloat16*>(y), stats); \
  else layer_norm_fwd_kernel<NV, float><<<grid, kWarps * 32, 0, st>>>(x, gamma, beta, rows, H, eps, reinterpret_cast<float*>(y), stats);
  if (nv <= 1) { RB_LN_FWD(1) } else if (nv <= 2) { RB_LN_FWD(2) } else if (nv <= 4) { RB_LN_FWD(4) } else { RB_LN_FWD(8) }
#undef RB_LN_FWD
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// dgamma and dbeta must be zero (or hold the value to accumulate onto) on entry
int rb_layer_norm_bwd(const void* dy, int dy_bf16, const float* x, const float* stats, const float* gamma, int64_t rows, int H, float* dx,
                      float* dgamma, float* dbeta, cudaStream_t st) {
  if (H % 4 != 0 || H > 1024 || H <= 0) return 1;
  if (rows <= 0) return 0;
  const int nv = (H + 127) / 128;
  const int grid = (int)std::min<int64_t>(std::max<int64_t>((rows + kWarps - 1) / kWarps, 1), 148 * 4);
#define RB_LN_BWD(NV)                                                                                                              \
  {                                                                                                                                \
    const size_t smem = (size_t)kWarps * 2 * NV * 128 * sizeof(float);                                                             \
    if (dy_bf16) {                                                                                                                 \
      auto k = layer_norm_bwd_kernel<NV, __nv_bfloat16>;                                                                           \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
      k<<<grid, kWarps * 32, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy), x, stats, gamma, rows, H, dx, dgamma, dbeta);  \
    } else {                                                                                                                       \
      auto k = layer_norm_bwd_kernel<NV, float>;                                                                                   \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                       \
      k<<<grid, kWarps * 32, smem, st>>>(reinterpret_cast<const float*>(dy), x, stats, gamma, rows, H, dx, dgamma, dbeta);          \
    }                                                                                                                              \
  }
  if (nv <= 1) RB_LN_BWD(1) else if (nv <= 2) RB_LN_BWD(2) else if (nv <= 4) RB_LN_BWD(4) else RB_LN_BWD(8)
#undef RB_LN_BWD
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Returns 1 when the shape does not suit the vectorised kernel (the caller then uses the column-per-thread kernel).
int rb_relu_bwd_bias_vec(const void* y, const void* dout, int64_t M, int N, int relu, void* dy, float* db, cudaStream_t st) {
  if (N % 8 != 0 || M <= 0) return 1;
  const int groups = N / 8;
  int gpb;                                                     // column groups per block: a divisor of 256
  if (groups >= 32) { if (groups % 32 != 0) return 1; gpb = 32; }
  else { gpb = 1; while (gpb < groups) gpb <<= 1; if (gpb != groups) return 1; }
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dy)) & 15) return 1;
  const int rlanes = 256 / gpb;
  const int gx = groups / gpb;
  const int gy = (int)std::min<int64_t>(std::max<int64_t>(M / (rlanes * 4), 1), std::max(1, 148 * 8 / gx));
  dim3 grid(gx, gy);
  if (dy)
    relu_bwd_bias_vec_kernel<true><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(y), reinterpret_cast<const __nv_bfloat16*>(dout),
                                                         M, N, relu, reinterpret_cast<__nv_bfloat16*>(dy), db, gpb);
  else
    relu_bwd_bias_vec_kernel<false><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(y), reinterpret_cast<const __nv_bfloat16*>(dout),
                                                          M, N, relu, nullptr, db, gpb);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
