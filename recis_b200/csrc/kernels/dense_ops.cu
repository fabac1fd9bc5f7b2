// Dense-tower helper kernels (sm_100a): pairwise dot interaction and FM second-order interaction (forward + backward),
// ReLU-backward fused with the bias gradient, and the fp32 -> padded bf16 weight cast that feeds the tcgen05 GEMM.
//
// In the reference these are chains of PyTorch ops inside the example models (examples/deepfm/deepfm_model.py:88-93
// computes the FM term with sum/pow/sub; a DLRM-style dot interaction would be bmm + tril-index gather, whose backward
// is an index_put with accumulation). Here each is one kernel per direction.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "rb_dense.h"
#include <cuda_bf16.h>
#include <type_traits>

namespace {

constexpr int kMaxVec = 64;   // at most 63 embedding fields + the dense vector per sample

// ---------------------------------------------------------------------------------- dot interaction
// z_0 = x[b] (bf16), z_k = cube[b][k-1] (fp32). out[b] = [x (D values), z_i . z_j for i > j (row-major lower triangle), 0 pad]
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
dot_interaction_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cube, int B, int F, int D, int out_ld,
                           __nv_bfloat16* __restrict__ out) {
  extern __shared__ float z[];                    // [(F+1)][D+1]
  const int b = blockIdx.x;
  const int V = F + 1, ld = D + 1;
  for (int i = threadIdx.x; i < V * D; i += THREADS) {
    const int v = i / D, d = i - v * D;
    z[v * ld + d] = v == 0 ? __bfloat162float(x[(int64_t)b * D + d]) : cube[((int64_t)b * F + (v - 1)) * D + d];
  }
  __syncthreads();
  __nv_bfloat16* o = out + (int64_t)b * out_ld;
  for (int d = threadIdx.x; d < D; d += THREADS) o[d] = x[(int64_t)b * D + d];
  const int P = V * (V - 1) / 2;
  for (int p = threadIdx.x; p < P; p += THREADS) {
    // p -> (i, j), i > j, row-major over the strict lower triangle
    int i = (int)((1.f + sqrtf(1.f + 8.f * (float)p)) * 0.5f);
    while (i * (i - 1) / 2 > p) --i;
    while ((i + 1) * i / 2 <= p) ++i;
    const int j = p - i * (i - 1) / 2;
    const float* zi = z + i * ld; const float* zj = z + j * ld;
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; ++d) acc = fmaf(zi[d], zj[d], acc);
    o[D + p] = __float2bfloat16_rn(acc);
  }
  for (int c = D + P + threadIdx.x; c < out_ld; c += THREADS) o[c] = __float2bfloat16_rn(0.f);
}

// dz_i = sum_{j != i} g_ij z_j with g the symmetric matrix built from the lower-triangle gradients; dx also gets dout[:, :D].
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
dot_interaction_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cube, const __nv_bfloat16* __restrict__ dout,
                           int B, int F, int D, int out_ld, float* __restrict__ dx, float* __restrict__ dcube) {
  extern __shared__ float sm[];
  const int V = F + 1, ld = D + 1;
  float* z = sm;                  // [V][D+1]
  float* g = sm + V * ld;         // [V][V]
  const int b = blockIdx.x;
  for (int i = threadIdx.x; i < V * D; i += THREADS) {
    const int v = i / D, d = i - v * D;
    z[v * ld + d] = v == 0 ? __bfloat162float(x[(int64_t)b * D + d]) : cube[((int64_t)b * F + (v - 1)) * D + d];
  }
  const __nv_bfloat16* go = dout + (int64_t)b * out_ld;
  for (int e = threadIdx.x; e < V * V; e += THREADS) {
    const int i = e / V, j = e - i * V;
    float v = 0.f;
    if (i > j) v = __bfloat162float(go[D + i * (i - 1) / 2 + j]);
    else if (j > i) v = __bfloat162float(go[D + j * (j - 1) / 2 + i]);
    g[e] = v;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += THREADS) {
    float col[kMaxVec];
#pragma unroll 1
    for (int j = 0; j < V; ++j) col[j] = z[j * ld + d];
    for (int i = 0; i < V; ++i) {
      float acc = 0.f;
      const float* gi = g + i * V;
      for (int j = 0; j < V; ++j) acc = fmaf(gi[j], col[j], acc);
      if (i == 0) dx[(int64_t)b * D + d] = acc + __bfloat162float(go[d]);
      else dcube[((int64_t)b * F + (i - 1)) * D + d] = acc;
    }
  }
}

// ---------------------------------------------------------------------------------- FM second-order term
// out[b] = 0.5 * sum_d ((sum_f v_fd)^2 - sum_f v_fd^2); cube [B, F, D] fp32 (weights already applied by the caller).
// One thread owns one float4 column group of one sample, so a warp covers 32 / (D/4) samples and every 32-byte sector it
// touches is used in full (narrow embeddings, D = 8 .. 32, are the common case for FM); the D/4 partial results of a sample
// are combined with shuffles. Q = D/4 must be a power of two <= 32; other widths take the generic kernel below.
template <int Q>
__global__ void __launch_bounds__(256)
fm_fwd_vec_kernel(const float* __restrict__ cube, int B, int F, float* __restrict__ out) {
  constexpr int D = Q * 4;
  const int64_t total = (int64_t)B * Q;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // the loop bound is rounded up to a whole warp so that the shuffles below always have all lanes present
  const int64_t total_pad = (total + 31) / 32 * 32;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total_pad; t += stride) {
    const bool live = t < total;
    const int64_t b = t / Q; const int q = (int)(t - b * Q);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float s2 = 0.f;
    if (live) {
      const float* p = cube + b * F * D + q * 4;
#pragma unroll 4
      for (int f = 0; f < F; ++f) {
        const float4 v = *reinterpret_cast<const float4*>(p + (int64_t)f * D);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        s2 = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s2))));
      }
    }
    float part = s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w - s2;
#pragma unroll
    for (int o = Q / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (live && q == 0) out[b] = 0.5f * part;
  }
}

// dcube[b,f,d] = g[b] * (S_d - v_fd), same thread mapping
template <int Q>
__global__ void __launch_bounds__(256)
fm_bwd_vec_kernel(const float* __restrict__ cube, const float* __restrict__ gout, int B, int F, float* __restrict__ dcube) {
  constexpr int D = Q * 4;
  const int64_t total = (int64_t)B * Q;
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = t / Q; const int q = (int)(t - b * Q);
    const float* p = cube + b * F * D + q * 4;
    float* o = dcube + b * F * D + q * 4;
    const float g = gout[b];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int f = 0; f < F; ++f) {
      const float4 v = *reinterpret_cast<const float4*>(p + (int64_t)f * D);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
#pragma unroll 4
    for (int f = 0; f < F; ++f) {
      const float4 v = *reinterpret_cast<const float4*>(p + (int64_t)f * D);      // second pass hits L1/L2
      *reinterpret_cast<float4*>(o + (int64_t)f * D) = make_float4(g * (s.x - v.x), g * (s.y - v.y), g * (s.z - v.z), g * (s.w - v.w));
    }
  }
}

// generic widths: one block per sample
__global__ void __launch_bounds__(128)
fm_fwd_kernel(const float* __restrict__ cube, int B, int F, int D, float* __restrict__ out) {
  __shared__ float red[4];
  const int b = blockIdx.x;
  float part = 0.f;
  for (int d = threadIdx.x; d < D; d += 128) {
    float s = 0.f, s2 = 0.f;
    for (int f = 0; f < F; ++f) { const float v = cube[((int64_t)b * F + f) * D + d]; s += v; s2 = fmaf(v, v, s2); }
    part += s * s - s2;
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  if (threadIdx.x == 0) out[b] = 0.5f * (red[0] + red[1] + red[2] + red[3]);
}

__global__ void __launch_bounds__(128)
fm_bwd_kernel(const float* __restrict__ cube, const float* __restrict__ gout, int B, int F, int D, float* __restrict__ dcube) {
  const int b = blockIdx.x;
  const float g = gout[b];
  for (int d = threadIdx.x; d < D; d += 128) {
    float s = 0.f;
    for (int f = 0; f < F; ++f) s += cube[((int64_t)b * F + f) * D + d];
    for (int f = 0; f < F; ++f) {
      const int64_t o = ((int64_t)b * F + f) * D + d;
      dcube[o] = g * (s - cube[o]);
    }
  }
}

template <typename Fn>
inline bool fm_dispatch_q(int D, const void* p0, const void* p1, Fn&& fn) {
  if (D % 4 != 0 || (reinterpret_cast<uintptr_t>(p0) & 15) || (reinterpret_cast<uintptr_t>(p1) & 15)) return false;
  switch (D / 4) {
    case 1: fn(std::integral_constant<int, 1>{}); return true;
    case 2: fn(std::integral_constant<int, 2>{}); return true;
    case 4: fn(std::integral_constant<int, 4>{}); return true;
    case 8: fn(std::integral_constant<int, 8>{}); return true;
    case 16: fn(std::integral_constant<int, 16>{}); return true;
    case 32: fn(std::integral_constant<int, 32>{}); return true;
    default: return false;
  }
}

// ---------------------------------------------------------------------------------- ReLU backward + bias gradient
// dy[m, n] = y[m, n] > 0 ? dout[m, n] : 0 (relu != 0), db[n] += sum_m dy[m, n]. One block handles 32 columns x 256-row slabs.
__global__ void __launch_bounds__(256)
relu_bwd_bias_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dout, int M, int N, int relu,
                     __nv_bfloat16* __restrict__ dy, float* __restrict__ db) {
  __shared__ float part[8][33];
  const int col = blockIdx.x * 32 + (threadIdx.x & 31);
  const int rlane = threadIdx.x >> 5;                       // 8 row lanes
  float acc = 0.f;
  if (col < N) {
    for (int m = blockIdx.y * 8 + rlane; m < M; m += gridDim.y * 8) {
      const int64_t o = (int64_t)m * N + col;
      float v = __bfloat162float(dout[o]);
      if (relu && !(__bfloat162float(y[o]) > 0.f)) v = 0.f;
      if (dy) dy[o] = __float2bfloat16_rn(v);
      acc += v;
    }
  }
  part[rlane][threadIdx.x & 31] = acc;
  __syncthreads();
  if (rlane == 0 && col < N && db) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) s += part[r][threadIdx.x & 31];
    atomicAdd(db + col, s);
  }
}

// fp32 [rows, cols] (row pitch src_ld) -> bf16 [rows_p, cols_p], zero padded
__global__ void __launch_bounds__(256)
cast_pad_bf16_kernel(const float* __restrict__ src, int rows, int cols, int src_ld, __nv_bfloat16* __restrict__ dst, int rows_p, int cols_p) {
  const int64_t total = (int64_t)rows_p * cols_p;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols_p), c = (int)(i - (int64_t)r * cols_p);
    dst[i] = __float2bfloat16_rn((r < rows && c < cols) ? src[(int64_t)r * src_ld + c] : 0.f);
  }
}

inline int blocks_for(int64_t n) { int64_t b = (n + 255) / 256; return (int)std::min<int64_t>(std::max<int64_t>(b, 1), 148 * 16); }

}  // namespace

extern "C" {

int rb_dot_interaction_fwd(const void* x, const float* cube, int B, int F, int D, int out_ld, void* out, cudaStream_t st) {
  if (F + 1 > kMaxVec) return 1;
  const size_t smem = (size_t)(F + 1) * (D + 1) * sizeof(float);
  if (smem > 200 * 1024) return 2;
  auto kern = dot_interaction_fwd_kernel<128>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kern<<<B, 128, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), cube, B, F, D, out_ld, reinterpret_cast<__nv_bfloat16*>(out));
  rb::note_launch();
  return 0;
}

int rb_dot_interaction_bwd(const void* x, const float* cube, const void* dout, int B, int F, int D, int out_ld, float* dx, float* dcube,
                           cudaStream_t st) {
  if (F + 1 > kMaxVec) return 1;
  const size_t smem = ((size_t)(F + 1) * (D + 1) + (size_t)(F + 1) * (F + 1)) * sizeof(float);
  if (smem > 200 * 1024) return 2;
  auto kern = dot_interaction_bwd_kernel<128>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  kern<<<B, 128, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), cube, reinterpret_cast<const __nv_bfloat16*>(dout), B, F, D, out_ld,
                             dx, dcube);
  rb::note_launch();
  return 0;
}

void rb_fm_fwd(const float* cube, int B, int F, int D, float* out, cudaStream_t st) {
  if (B <= 0) return;
  const bool vec = fm_dispatch_q(D, cube, cube, [&](auto q) {
    constexpr int Q = decltype(q)::value;
    const int64_t blocks = ((int64_t)B * Q + 255) / 256;
    fm_fwd_vec_kernel<Q><<<(int)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(cube, B, F, out);
  });
  if (!vec) fm_fwd_kernel<<<B, 128, 0, st>>>(cube, B, F, D, out);
  rb::note_launch();
}

void rb_fm_bwd(const float* cube, const float* gout, int B, int F, int D, float* dcube, cudaStream_t st) {
  if (B <= 0) return;
  const bool vec = fm_dispatch_q(D, cube, dcube, [&](auto q) {
    constexpr int Q = decltype(q)::value;
    const int64_t blocks = ((int64_t)B * Q + 255) / 256;
    fm_bwd_vec_kernel<Q><<<(int)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(cube, gout, B, F, dcube);
  });
  if (!vec) fm_bwd_kernel<<<B, 128, 0, st>>>(cube, gout, B, F, D, dcube);
  rb::note_launch();
}

void rb_relu_bwd_bias(const void* y, const void* dout, int M, int N, int relu, void* dy, float* db, cudaStream_t st) {
  if (M <= 0 || N <= 0) return;
  dim3 grid((N + 31) / 32, std::min(std::max(M / 256, 1), 64));
  relu_bwd_bias_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(y), reinterpret_cast<const __nv_bfloat16*>(dout), M, N,
                                             relu, reinterpret_cast<__nv_bfloat16*>(dy), db);
  rb::note_launch();
}

void rb_cast_pad_bf16(const float* src, int rows, int cols, int src_ld, void* dst, int rows_p, int cols_p, cudaStream_t st) {
  cast_pad_bf16_kernel<<<blocks_for((int64_t)rows_p * cols_p), 256, 0, st>>>(src, rows, cols, src_ld, reinterpret_cast<__nv_bfloat16*>(dst),
                                                                             rows_p, cols_p);
  rb::note_launch();
}

}  // extern "C"

// ------------------------------------------------------------------ multi-tensor dense Adam (TF-style and PyTorch-style)
namespace {
__global__ void __launch_bounds__(256)
dense_adam_kernel(const __grid_constant__ RbDenseAdamArgs a, float b1, float b2, float eps, float decay, float step_size,
                  float inv_sqrt_bc2, float l2) {
  const int t = blockIdx.y;
  float* __restrict__ w = a.w[t];
  const float* __restrict__ g = a.g[t];
  float* __restrict__ m = a.m[t];
  float* __restrict__ v = a.v[t];
  __nv_bfloat16* __restrict__ wb = reinterpret_cast<__nv_bfloat16*>(a.w_bf16[t]);
  const int64_t n = a.n[t];
  const int cols = a.cols[t], ld = a.bf16_ld[t];
  const bool padded = wb != nullptr && ld > 0 && ld != cols;          // the bf16 copy has a wider row pitch than the weight
  const float c1 = 1.f - b1, c2 = 1.f - b2;
  auto upd = [&](float& wi, float gi, float& mi, float& vi) {
    gi += l2 * wi;
    mi = b1 * mi + c1 * gi;
    vi = b2 * vi + c2 * gi * gi;
    wi = wi * decay - step_size * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
  };
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15) == 0 && (wb == nullptr || (reinterpret_cast<uintptr_t>(wb) & 7) == 0) &&
                   (!padded || ((cols & 3) == 0 && (ld & 3) == 0));    // four consecutive elements stay in one row of the copy
  auto bf16_index = [&](int64_t i) { return padded ? (i / cols) * (int64_t)ld + (i % cols) : i; };
  const int64_t n4 = vec ? n >> 2 : 0;
  for (int64_t i = tid; i < n4; i += stride) {
    float4 wi = reinterpret_cast<float4*>(w)[i], mi = reinterpret_cast<float4*>(m)[i], vi = reinterpret_cast<float4*>(v)[i];
    const float4 gi = reinterpret_cast<const float4*>(g)[i];
    upd(wi.x, gi.x, mi.x, vi.x); upd(wi.y, gi.y, mi.y, vi.y); upd(wi.z, gi.z, mi.z, vi.z); upd(wi.w, gi.w, mi.w, vi.w);
    reinterpret_cast<float4*>(w)[i] = wi; reinterpret_cast<float4*>(m)[i] = mi; reinterpret_cast<float4*>(v)[i] = vi;
    if (wb) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(wi.x, wi.y), hi = __floats2bfloat162_rn(wi.z, wi.w);
      uint2 pk; pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(wb + bf16_index(i << 2)) = pk;
    }
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
    float wi = w[i], mi = m[i], vi = v[i];
    upd(wi, g[i], mi, vi);
    w[i] = wi; m[i] = mi; v[i] = vi;
    if (wb) wb[bf16_index(i)] = __float2bfloat16_rn(wi);
  }
}
}  // namespace

extern "C" void rb_dense_adam(const RbDenseAdamArgs* args, float beta1, float beta2, float eps, float decay, float step_size,
                              float inv_sqrt_bc2, float l2, cudaStream_t st) {
  if (args->count <= 0) return;
  int64_t max_n = 0;
  for (int i = 0; i < args->count; ++i) max_n = args->n[i] > max_n ? args->n[i] : max_n;
  if (max_n == 0) return;
  int64_t bx = (max_n / 4 + 255) / 256;
  bx = bx < 1 ? 1 : (bx > 148 * 4 ? 148 * 4 : bx);
  dense_adam_kernel<<<dim3((unsigned)bx, (unsigned)args->count), 256, 0, st>>>(*args, beta1, beta2, eps, decay, step_size, inv_sqrt_bc2, l2);
  rb::note_launch();
}
