// Pairwise dot interaction (DLRM) on the 5th-generation tensor cores, forward and backward.
//
// Per sample the op is a tiny GEMM: Z = [x; e_1 .. e_F] is (F+1) x D, the output is the strict lower triangle of Z Z^T and the
// backward is dZ = (G + G^T) Z with G the gradient of that triangle. A SIMT version of it is bound by shared-memory bandwidth
// (every product reads two operands from shared memory). Here four samples share one 128-row tensor-core tile:
//
//   forward   rows (s, i) = sample s, vector i (32 rows per sample, zero padded) are staged once as bf16 in the 128-byte
//             swizzled layout; ONE tcgen05.mma chain computes S = Zt Zt^T (128 x 128 x D, fp32 in tensor memory) with the same
//             shared-memory tile as both operands; each warp reads back the 32 x 32 diagonal block of its sample with
//             tcgen05.ld and writes [x, triangle, zero pad] as one contiguous bf16 row.
//   backward  A = block-diagonal symmetric gradient matrix (128 x 128, K-major), B = the same Z tile read as an MN-major
//             operand (N = embedding column, K = tile row), dZ = A B (128 x D) in tensor memory; each thread owns one row
//             (s, i) and stores it to dx (i = 0, plus the pass-through gradient of x) or dcube (1 <= i <= F).
//
// The off-diagonal 32 x 32 blocks are computed and thrown away: at these sizes the tensor core has >10x headroom and the
// kernel is bound by reading the fp32 embeddings from HBM once. Operands are rounded to bf16 (the output is bf16 anyway).
// The reference has no fused interaction; a PyTorch model would use bmm + tril index gather (examples/deepfm/deepfm_model.py
// shows the FM analogue). Waits are bounded; a timeout sets the status word and the CTA returns after freeing tensor memory.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "../common/rb_tcgen05.cuh"
#include "rb_dense.h"
#include <cuda_bf16.h>

namespace {

using namespace rb::tc;

constexpr int kRows = 128;        // tile rows = 4 samples x 32 vectors
constexpr int kVP = 32;           // padded vectors per sample
constexpr int kSamples = 4;
constexpr int kTileChunk = kRows * 128;   // bytes of one [128 rows x 64 bf16] swizzled block

// Stage Z of sample b (warp-wide): row 0 = x (bf16), rows 1..F = cube rows (fp32 -> bf16), other rows zero.
__device__ __forceinline__ void stage_sample(uint8_t* tile, int w, int lane, const __nv_bfloat16* __restrict__ x,
                                             const float* __restrict__ cube, int b, int B, int F, int D) {
  const int c = lane * 4;                         // 4 consecutive columns per lane, D <= 128
  if (c >= D) return;
  uint8_t* base = tile + (c >> 6) * kTileChunk;
  const int cc = c & 63;
  const bool live = b < B;
#pragma unroll 8
  for (int i = 0; i < kVP; ++i) {
    uint2 v = make_uint2(0u, 0u);
    if (live && i == 0) {
      v = *reinterpret_cast<const uint2*>(x + (int64_t)b * D + c);
    } else if (live && i <= F) {
      const float4 f = *reinterpret_cast<const float4*>(cube + ((int64_t)b * F + (i - 1)) * D + c);
      __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
      v.x = *reinterpret_cast<uint32_t*>(&lo); v.y = *reinterpret_cast<uint32_t*>(&hi);
    }
    *reinterpret_cast<uint2*>(base + swizzle128_offset(w * kVP + i, cc)) = v;
  }
}

__global__ void __launch_bounds__(128, 4)
dot_interaction_tc_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cube, int B, int F, int D, int out_ld,
                              __nv_bfloat16* __restrict__ out, int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* tile = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(tile + 2 * kTileChunk);       // [4][out_ld]
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kSamples + w;
  if (threadIdx.x == 0) { abort_flag = 0; mbar_init(&done_bar, 1); mbar_fence_init(); }
  if (w == 0) tmem_alloc(&tmem_slot, 128);
  stage_sample(tile, w, lane, x, cube, b, B, F, D);
  fence_smem_to_async();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(128, 128, false, false);
    const uint32_t sa = smem_u32(tile);
    for (int k = 0; k < D / 16; ++k) {
      const uint64_t d = make_desc(sa + (k >> 2) * kTileChunk + (k & 3) * 32, 16, 1024);
      umma_bf16(tmem, d, d, idesc, k > 0 ? 1u : 0u);
    }
    umma_commit(&done_bar);
  }
  // x part and zero tail of the output row while the tensor core works
  const int V = F + 1, P = V * (V - 1) / 2;
  __nv_bfloat16* mine = orow + w * out_ld;
  if (b < B) {
    for (int d = lane; d < D; d += 32) mine[d] = x[(int64_t)b * D + d];
    for (int c = D + P + lane; c < out_ld; c += 32) mine[c] = __float2bfloat16_rn(0.f);
  }
  const bool ok = mbar_wait(&done_bar, 0, &abort_flag);
  fence_after_sync();
  if (ok) {
    uint32_t r[32];
    tmem_ld32(tmem + ((uint32_t)(w * 32) << 16) + (uint32_t)(w * 32), r);
    tmem_ld_wait();
    if (b < B && lane < V) {
      __nv_bfloat16* t = mine + D + lane * (lane - 1) / 2;
#pragma unroll
      for (int j = 0; j < 31; ++j)
        if (j < lane) t[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
    __syncwarp();
    if (b < B) {
      __nv_bfloat16* o = out + (int64_t)b * out_ld;
      if ((out_ld & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        for (int q = lane; q < out_ld / 8; q += 32) reinterpret_cast<uint4*>(o)[q] = reinterpret_cast<const uint4*>(mine)[q];
      } else {
        for (int c = lane; c < out_ld; c += 32) o[c] = mine[c];
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (w == 0) { fence_after_sync(); tmem_dealloc(tmem, 128); }
  if (threadIdx.x == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

__global__ void __launch_bounds__(128, 3)
dot_interaction_tc_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cube, const __nv_bfloat16* __restrict__ dout,
                              int B, int F, int D, int out_ld, float* __restrict__ dx, float* __restrict__ dcube,
                              int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  uint8_t* ztile = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* gtile = ztile + 2 * kTileChunk;
  __nv_bfloat16* grow = reinterpret_cast<__nv_bfloat16*>(gtile + 2 * kTileChunk);      // [4][out_ld] staged dout rows
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kSamples + w;
  const int V = F + 1;
  if (threadIdx.x == 0) { abort_flag = 0; mbar_init(&done_bar, 1); mbar_fence_init(); }
  if (w == 0) tmem_alloc(&tmem_slot, 128);
  stage_sample(ztile, w, lane, x, cube, b, B, F, D);
  __nv_bfloat16* mine = grow + w * out_ld;
  if (b < B) {
    const __nv_bfloat16* go = dout + (int64_t)b * out_ld;
    if ((out_ld & 7) == 0 && (reinterpret_cast<uintptr_t>(dout) & 15) == 0) {
      for (int q = lane; q < out_ld / 8; q += 32) reinterpret_cast<uint4*>(mine)[q] = reinterpret_cast<const uint4*>(go)[q];
    } else {
      for (int c = lane; c < out_ld; c += 32) mine[c] = go[c];
    }
  }
  __syncwarp();
  {
    // row (w, i = lane) of the block-diagonal symmetric gradient matrix: 128 bf16, non-zero only in columns [32 w, 32 w + 32)
    const int i = lane, R = w * kVP + i;
    uint32_t pk[16];
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) {
      float g2[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = jj * 2 + h;
        float v = 0.f;
        if (b < B && i < V && j < V && i != j) {
          const int hi = i > j ? i : j, lo = i > j ? j : i;
          v = __bfloat162float(mine[D + hi * (hi - 1) / 2 + lo]);
        }
        g2[h] = v;
      }
      __nv_bfloat162 p = __floats2bfloat162_rn(g2[0], g2[1]);
      pk[jj] = *reinterpret_cast<uint32_t*>(&p);
    }
#pragma unroll
    for (int q = 0; q < 16; ++q) {                 // sixteen 16-byte chunks = 128 columns; chunks 4w .. 4w+3 carry the data
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      const int rel = q - 4 * w;
      if (rel >= 0 && rel < 4) v = make_uint4(pk[rel * 4], pk[rel * 4 + 1], pk[rel * 4 + 2], pk[rel * 4 + 3]);
      *reinterpret_cast<uint4*>(gtile + (q >> 3) * kTileChunk + swizzle128_offset(R, (q & 7) * 8)) = v;
    }
  }
  fence_smem_to_async();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_bf16(128, D, false, true);
    const uint32_t sg = smem_u32(gtile), sz = smem_u32(ztile);
#pragma unroll
    for (int k = 0; k < 8; ++k) {                  // K = 128 tile rows
      const uint64_t da = make_desc(sg + (k >> 2) * kTileChunk + (k & 3) * 32, 16, 1024);
      const uint64_t db = make_desc(sz + k * 2048, kTileChunk, 1024);
      umma_bf16(tmem, da, db, idesc, k > 0 ? 1u : 0u);
    }
    umma_commit(&done_bar);
  }
  const bool ok = mbar_wait(&done_bar, 0, &abort_flag);
  fence_after_sync();
  if (ok) {
    const int i = lane;
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + ((uint32_t)(w * 32) << 16) + (uint32_t)c0, r);
      tmem_ld_wait();
      if (b < B && i < V) {
        float* dst = i == 0 ? dx + (int64_t)b * D + c0 : dcube + ((int64_t)b * F + (i - 1)) * D + c0;
        const int valid = min(32, D - c0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (q * 4 >= valid) break;
          float4 v = make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                                 __uint_as_float(r[q * 4 + 3]));
          if (i == 0) {
            v.x += __bfloat162float(mine[c0 + q * 4]); v.y += __bfloat162float(mine[c0 + q * 4 + 1]);
            v.z += __bfloat162float(mine[c0 + q * 4 + 2]); v.w += __bfloat162float(mine[c0 + q * 4 + 3]);
          }
          *reinterpret_cast<float4*>(dst + q * 4) = v;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (w == 0) { fence_after_sync(); tmem_dealloc(tmem, 128); }
  if (threadIdx.x == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

inline bool tc_shape_ok(int F, int D, const void* x, const void* cube) {
  return F + 1 <= kVP && (D == 64 || D == 128) && (reinterpret_cast<uintptr_t>(x) & 7) == 0 &&
         (reinterpret_cast<uintptr_t>(cube) & 15) == 0;
}

}  // namespace

// Return 0 when the tensor-core kernel ran, 1 when the shape is outside its range (caller falls back), >1 on a launch error.
extern "C" int rb_dot_interaction_tc_fwd(const void* x, const float* cube, int B, int F, int D, int out_ld, void* out, int64_t* status,
                                         cudaStream_t st) {
  if (!tc_shape_ok(F, D, x, cube)) return 1;
  const size_t smem = 1024 + 2 * kTileChunk + (size_t)kSamples * out_ld * 2 + 16;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(dot_interaction_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) return 3;
    attr = true;
  }
  if (smem > 100 * 1024) return 1;
  dot_interaction_tc_fwd_kernel<<<(B + kSamples - 1) / kSamples, 128, smem, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), cube, B, F, D, out_ld, reinterpret_cast<__nv_bfloat16*>(out), status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

extern "C" int rb_dot_interaction_tc_bwd(const void* x, const float* cube, const void* dout, int B, int F, int D, int out_ld, float* dx,
                                         float* dcube, int64_t* status, cudaStream_t st) {
  if (!tc_shape_ok(F, D, x, cube) || (reinterpret_cast<uintptr_t>(dx) & 15) || (reinterpret_cast<uintptr_t>(dcube) & 15) || D % 4) return 1;
  const size_t smem = 1024 + 4 * kTileChunk + (size_t)kSamples * out_ld * 2 + 16;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(dot_interaction_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess) return 3;
    attr = true;
  }
  if (smem > 100 * 1024) return 1;
  dot_interaction_tc_bwd_kernel<<<(B + kSamples - 1) / kSamples, 128, smem, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), cube, reinterpret_cast<const __nv_bfloat16*>(dout), B, F, D, out_ld, dx, dcube, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
