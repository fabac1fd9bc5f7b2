// Ragged (unpadded) multi-head self-attention forward on the 5th-generation tensor cores, head width 64.
//
// Input is the packed projection output qkv [T, 3 * H * 64] (bf16) of all sequences of a batch back to back, plus the
// sequence boundaries offsets [B + 1]; no padding exists anywhere. One CTA (128 threads) owns one (sequence, head, 128-query
// tile) and walks the sequence's keys in tiles of 128 with the usual online softmax:
//
//   S  = Q K^T        tcgen05.mma, A = Q tile, B = K tile, both K-major, staged in shared memory in the 128-byte swizzle by
//                     ordinary 16-byte stores (rows past the end of the sequence are zero); fp32 result in tensor memory
//   P  = exp2(S * scale * log2 e - m)   each thread owns one query row: it reads its row of S back with tcgen05.ld, keeps the
//                     running maximum m and sum l in registers and writes P (bf16) into shared memory as the next A operand
//   PV = P V          tcgen05.mma, B = the V tile read as an MN-major operand (N = head column, K = key row)
//   O  = O * alpha + PV   in registers (64 fp32 per thread), so no tensor-memory store is needed for the rescale
//
// and finally writes O / l (bf16) and the log-sum-exp (base 2) of the row. Keys past the end of the sequence are masked in
// the softmax; query rows past the end are computed on zeros and not stored. Two CTAs fit on an SM (80 KB shared memory,
// 256 tensor-memory columns each), which overlaps one CTA's softmax with the other's tensor-core work.
//
// The reference has no attention kernel; its sequence example pads to the longest sequence and calls the library SDPA
// (examples/seq2seq/transformer.py:36-38). Waits are bounded; a timeout sets the status word and the CTA frees its tensor
// memory and returns. This kernel is opt-in (RECIS_ATTENTION=tcgen05) until it has been validated on hardware.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "../common/rb_tcgen05.cuh"
#include "rb_dense.h"
#include <cuda_bf16.h>

namespace {

using namespace rb::tc;

constexpr int kTile = 128;                 // queries per CTA = keys per step = tensor-memory lanes
constexpr int kHead = 64;                  // head width (one 128-byte swizzle row)
constexpr int kBlk = kTile * 128;          // bytes of one [128 rows x 64 bf16] swizzled block
constexpr uint32_t kTmemCols = 256;        // S: columns 0..127, PV: columns 128..191

// Copy one row of 64 bf16 (128 bytes) from global memory (or zeros) into row r of a swizzled block.
__device__ __forceinline__ void stage_row(uint8_t* blk, int r, const __nv_bfloat16* src) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 v = src ? reinterpret_cast<const uint4*>(src)[c] : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(blk + swizzle128_offset(r, c * 8)) = v;
  }
}

__global__ void __launch_bounds__(128, 2)
ragged_attention_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const int32_t* __restrict__ offsets, int H, float scale_log2,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ lse2, int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int b = blockIdx.y, h = blockIdx.z, qt = blockIdx.x;
  const int s0 = offsets[b], L = offsets[b + 1] - s0;
  if (qt * kTile >= L) return;                                   // uniform for the CTA, before any barrier or allocation

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* qtile = smem;                  // [128 q][64 d]      K-major A of S = Q K^T
  uint8_t* ktile = smem + kBlk;           // [128 keys][64 d]   K-major B of S
  uint8_t* vtile = smem + 2 * kBlk;       // [128 keys][64 d]   MN-major B of PV (N = d, K = key)
  uint8_t* ptile = smem + 3 * kBlk;       // 2 x [128 q][64 keys] K-major A of PV
  const int t = threadIdx.x, warp = t >> 5;
  const int64_t ld = (int64_t)3 * H * kHead;
  if (t == 0) { abort_flag = 0; mbar_init(&bar_s, 1); mbar_init(&bar_o, 1); mbar_fence_init(); }
  if (warp == 0) tmem_alloc(&tmem_slot, kTmemCols);

  const int q = qt * kTile + t;
  const bool q_ok = q < L;
  stage_row(qtile, t, q_ok ? qkv + (int64_t)(s0 + q) * ld + h * kHead : nullptr);

  float o[kHead];
#pragma unroll
  for (int d = 0; d < kHead; ++d) o[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t idesc_s = make_idesc_bf16(kTile, kTile, false, false);
  const uint32_t idesc_o = make_idesc_bf16(kTile, kHead, false, true);
  bool ok = true;

  const int n_kv = (L + kTile - 1) / kTile;
  for (int j = 0; j < n_kv && ok; ++j) {
    const int key = j * kTile + t;
    const __nv_bfloat16* krow = key < L ? qkv + (int64_t)(s0 + key) * ld + (H + h) * kHead : nullptr;
    stage_row(ktile, t, krow);
    stage_row(vtile, t, krow ? krow + H * kHead : nullptr);
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (t == 0) {
      const uint32_t sq = smem_u32(qtile), sk = smem_u32(ktile);
#pragma unroll
      for (int k = 0; k < kHead / 16; ++k)
        umma_bf16(tmem, make_desc(sq + k * 32, 16, 1024), make_desc(sk + k * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
      umma_commit(&bar_s);
    }
    // the outcome of a bounded wait is made uniform for the CTA: every thread takes the same path through the barriers below
    ok = __syncthreads_and(mbar_wait(&bar_s, (uint32_t)(j & 1), &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;

    // ---- online softmax on this thread's row of S
    const int valid = min(kTile, L - j * kTile);                 // key columns of this tile that exist
    float mx = -INFINITY;
    for (int c0 = 0; c0 < kTile; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + (uint32_t)c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (c0 + i < valid) mx = fmaxf(mx, __uint_as_float(r[i]) * scale_log2);
    }
    const float m_new = fmaxf(m, mx);
    const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
    float rowsum = 0.f;
    for (int c0 = 0; c0 < kTile; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + (uint32_t)c0, r);
      tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = (c0 + 2 * i < valid) ? exp2f(__uint_as_float(r[2 * i]) * scale_log2 - m_new) : 0.f;
        const float p1 = (c0 + 2 * i + 1 < valid) ? exp2f(__uint_as_float(r[2 * i + 1]) * scale_log2 - m_new) : 0.f;
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        // the sum uses the rounded values, so that l matches what the tensor core multiplies with
        rowsum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
        pk[i] = *reinterpret_cast<const uint32_t*>(&pb);
      }
      uint8_t* blk = ptile + (c0 >> 6) * kBlk;
#pragma unroll
      for (int cq = 0; cq < 4; ++cq)
        *reinterpret_cast<uint4*>(blk + swizzle128_offset(t, (c0 & 63) + cq * 8)) =
            make_uint4(pk[cq * 4], pk[cq * 4 + 1], pk[cq * 4 + 2], pk[cq * 4 + 3]);
    }
    l = l * alpha + rowsum;
    m = m_new;
#pragma unroll
    for (int d = 0; d < kHead; ++d) o[d] *= alpha;

    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (t == 0) {
      const uint32_t sp = smem_u32(ptile), sv = smem_u32(vtile);
#pragma unroll
      for (int k = 0; k < kTile / 16; ++k)
        umma_bf16(tmem + 128u, make_desc(sp + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024), make_desc(sv + k * 2048, kBlk, 1024), idesc_o,
                  k > 0 ? 1u : 0u);
      umma_commit(&bar_o);
    }
    ok = __syncthreads_and(mbar_wait(&bar_o, (uint32_t)(j & 1), &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;
    for (int c0 = 0; c0 < kHead; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + 128u + (uint32_t)c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[c0 + i] += __uint_as_float(r[i]);
    }
  }

  if (ok && q_ok) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = out + (int64_t)(s0 + q) * H * kHead + h * kHead;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
        w[i] = *reinterpret_cast<const uint32_t*>(&v);
      }
      reinterpret_cast<uint4*>(dst)[c] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (lse2) lse2[(int64_t)(s0 + q) * H + h] = m + log2f(l);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, kTmemCols); }
  if (t == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

}  // namespace

// qkv: bf16 [T, 3 * H * 64] packed (q | k | v, each H heads of 64), offsets: int32 [B + 1] on the device, max_len: an upper bound
// of the sequence lengths (sizes the grid), out: bf16 [T, H * 64], lse2: fp32 [T, H] or null (log2-domain log-sum-exp).
// Returns 0 on launch, 1 when the arguments are outside the kernel's range (alignment), > 1 on a launch error.
extern "C" int rb_ragged_attention_fwd(const void* qkv, const int32_t* offsets, int B, int H, int max_len, float scale, void* out, float* lse2,
                                       int64_t* status, cudaStream_t st) {
  if (B <= 0 || H <= 0 || max_len <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return 1;
  const size_t smem = 1024 + 5 * (size_t)kBlk;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ragged_attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
    attr = true;
  }
  dim3 grid((max_len + kTile - 1) / kTile, B, H);
  ragged_attention_fwd_kernel<<<grid, 128, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(qkv), offsets, H, scale * 1.4426950408889634f,
                                                       reinterpret_cast<__nv_bfloat16*>(out), lse2, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
