// Ragged (unpadded) multi-head self-attention forward on the 5th-generation tensor cores, head width 64.
//
// Input is the packed projection output qkv [T, 3 * H * 64] (bf16) of all sequences of a batch back to back, plus the
// sequence boundaries offsets [B + 1]; no padding exists anywhere. One CTA (128 threads) owns one (sequence, head, 128-query
// tile) and walks the sequence's keys in tiles of 128 with the usual online softmax:
//
//   S  = Q K^T        tcgen05.mma, A = Q tile, B = K tile, both K-major; the tiles arrive by TMA straight from the packed matrix
//                     in the 128-byte swizzle (the next K tile as soon as S is complete, the next V tile as soon as P V is);
//                     fp32 result in tensor memory
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
// memory and returns. These kernels are what ops/attention.py runs on CUDA for head width 64 (RECIS_ATTENTION=padded selects
// the padded library path).
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "../common/rb_tcgen05.cuh"
#include "rb_dense.h"
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstring>

namespace {

using namespace rb::tc;

constexpr int kTile = 128;                 // queries per CTA = keys per step = tensor-memory lanes
constexpr int kHead = 64;                  // head width (one 128-byte swizzle row)
constexpr int kBlk = kTile * 128;          // bytes of one [128 rows x 64 bf16] swizzled block
constexpr uint32_t kTmemCols = 256;        // S: columns 0..127, PV: columns 128..191

// 2^x on the special-function unit: one instruction, flushes denormals, 2^-inf = 0 (which is how masked entries become zero)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two floats -> packed bf16x2 (round to nearest even), first argument in the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One thread's row of a 128-key tile of S (tensor memory at `trow`): new running maximum and sum, P = 2^(S * scale_log2 - m)
// written as bf16 into the two K-major blocks of `ptile`. Returns the factor by which what was accumulated under the old
// maximum shrinks. kMask selects whether key columns >= valid are masked: a full tile pays for no compare or select.
// The row is read from tensor memory once (four 32-column reads in flight) and stays in registers for both passes; the
// maximum and the sum run as four independent chains each, since one warp per scheduler hides no dependent latency.
template <bool kMask>
__device__ __forceinline__ float softmax_row(uint32_t trow, int valid, float scale_log2, int t, uint8_t* ptile, float& m, float& l) {
  uint32_t s0[32], s1[32], s2[32], s3[32];
  tmem_ld32(trow, s0);
  tmem_ld32(trow + 32u, s1);
  tmem_ld32(trow + 64u, s2);
  tmem_ld32(trow + 96u, s3);
  tmem_ld_wait();
  // masking is a select on the value (no branch per element): a masked key becomes -inf here and an exact zero after the
  // exponential; scale_log2 > 0, so the maximum can be taken before scaling
  if (kMask) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i >= valid) s0[i] = 0xff800000u;
      if (32 + i >= valid) s1[i] = 0xff800000u;
      if (64 + i >= valid) s2[i] = 0xff800000u;
      if (96 + i >= valid) s3[i] = 0xff800000u;
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    mx0 = fmaxf(mx0, __uint_as_float(s0[i]));
    mx1 = fmaxf(mx1, __uint_as_float(s1[i]));
    mx2 = fmaxf(mx2, __uint_as_float(s2[i]));
    mx3 = fmaxf(mx3, __uint_as_float(s3[i]));
  }
  const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
  const float m_new = fmaxf(m, mx * scale_log2);
  const float alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
  float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) {                 // 32 key columns per quarter; two quarters per 64-wide K-major block
    uint8_t* blk = ptile + (q4 >> 1) * kBlk;
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t ua = q4 == 0 ? s0[2 * i] : q4 == 1 ? s1[2 * i] : q4 == 2 ? s2[2 * i] : s3[2 * i];
      const uint32_t ub = q4 == 0 ? s0[2 * i + 1] : q4 == 1 ? s1[2 * i + 1] : q4 == 2 ? s2[2 * i + 1] : s3[2 * i + 1];
      // -inf * scale_log2 - m_new = -inf (m_new is finite whenever the tile has one existing key): 2^-inf = 0
      const float p0 = fast_exp2(fmaf(__uint_as_float(ua), scale_log2, -m_new));
      const float p1 = fast_exp2(fmaf(__uint_as_float(ub), scale_log2, -m_new));
      if (i & 1) { sum1 += p0; sum3 += p1; } else { sum0 += p0; sum2 += p1; }
      pk[i] = pack_bf16x2(p0, p1);
    }
#pragma unroll
    for (int cq = 0; cq < 4; ++cq)
      *reinterpret_cast<uint4*>(blk + swizzle128_offset(t, (q4 & 1) * 32 + cq * 8)) =
          make_uint4(pk[cq * 4], pk[cq * 4 + 1], pk[cq * 4 + 2], pk[cq * 4 + 3]);
  }
  l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
  m = m_new;
  return alpha;
}

__global__ void __launch_bounds__(128, 2)
ragged_attention_fwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const int32_t* __restrict__ offsets, int H, float scale_log2,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ lse2, int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_q, bar_k, bar_v, bar_s, bar_o;
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
  // Q, K and V tiles arrive by TMA straight from the packed [T, 3 * H * 64] matrix (box of 128 rows x 64 columns, 128-byte
  // swizzle). Rows past the end of the sequence belong to the next sequence (or read as zeros past the end of the matrix):
  // surplus query rows are computed and never stored, surplus keys are masked in the softmax, and the surplus rows of the V
  // tile are zeroed in shared memory, so that a zero probability never meets a non-finite value.
  const int xq = h * kHead, xk = (H + h) * kHead, xv = (2 * H + h) * kHead;
  if (t == 0) {
    abort_flag = 0;
    mbar_init(&bar_q, 1); mbar_init(&bar_k, 1); mbar_init(&bar_v, 1); mbar_init(&bar_s, 1); mbar_init(&bar_o, 1);
    mbar_fence_init();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_qkv) : "memory");
    mbar_expect_tx(&bar_q, kBlk); tma_load_2d(qtile, &map_qkv, xq, s0 + qt * kTile, &bar_q);
    mbar_expect_tx(&bar_k, kBlk); tma_load_2d(ktile, &map_qkv, xk, s0, &bar_k);
    mbar_expect_tx(&bar_v, kBlk); tma_load_2d(vtile, &map_qkv, xv, s0, &bar_v);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, kTmemCols);

  const int q = qt * kTile + t;
  const bool q_ok = q < L;
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
    const uint32_t ph = (uint32_t)(j & 1);
    if (t == 0) {
      bool got = (j > 0 || mbar_wait(&bar_q, 0, &abort_flag)) && mbar_wait(&bar_k, ph, &abort_flag);
      if (got) {
        fence_after_sync();
        const uint32_t sq = smem_u32(qtile), sk = smem_u32(ktile);
#pragma unroll
        for (int k = 0; k < kHead / 16; ++k)
          umma_bf16(tmem, make_desc(sq + k * 32, 16, 1024), make_desc(sk + k * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(&bar_s);
      }
    }
    // the outcome of a bounded wait is made uniform for the CTA: every thread takes the same path through the barriers below
    ok = __syncthreads_and(mbar_wait(&bar_s, ph, &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;
    // S is complete, so the K tile is free: the next one travels while this tile's softmax and P V run
    if (t == 0 && j + 1 < n_kv) { mbar_expect_tx(&bar_k, kBlk); tma_load_2d(ktile, &map_qkv, xk, s0 + (j + 1) * kTile, &bar_k); }

    // ---- online softmax on this thread's row of S; only the sequence's last key tile can hold keys that do not exist
    const int valid = min(kTile, L - j * kTile);                 // key columns of this tile that exist
    float alpha;
    if (valid == kTile) alpha = softmax_row<false>(tmem + lane_base, kTile, scale_log2, t, ptile, m, l);
    else alpha = softmax_row<true>(tmem + lane_base, valid, scale_log2, t, ptile, m, l);

    if (valid < kTile) {
      // last, partial tile: the V rows past the end of the sequence become zeros (this thread's row, once V has landed)
      ok = mbar_wait(&bar_v, ph, &abort_flag);
      if (ok && t >= valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(vtile + swizzle128_offset(t, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    fence_smem_to_async();
    fence_before_sync();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;
    if (t == 0) {
      if (mbar_wait(&bar_v, ph, &abort_flag)) {
        fence_after_sync();
        const uint32_t sp = smem_u32(ptile), sv = smem_u32(vtile);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)
          umma_bf16(tmem + 128u, make_desc(sp + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024), make_desc(sv + k * 2048, kBlk, 1024), idesc_o,
                    k > 0 ? 1u : 0u);
        umma_commit(&bar_o);
      }
    }
    ok = __syncthreads_and(mbar_wait(&bar_o, ph, &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;
    // P V is complete, so the V tile is free
    if (t == 0 && j + 1 < n_kv) { mbar_expect_tx(&bar_v, kBlk); tma_load_2d(vtile, &map_qkv, xv, s0 + (j + 1) * kTile, &bar_v); }
    {
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem + lane_base + 128u, r0);
      tmem_ld32(tmem + lane_base + 160u, r1);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {           // O = O * alpha + P V, one multiply-add per element
        o[i] = fmaf(o[i], alpha, __uint_as_float(r0[i]));
        o[32 + i] = fmaf(o[32 + i], alpha, __uint_as_float(r1[i]));
      }
    }
  }

  if (ok && q_ok) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = out + (int64_t)(s0 + q) * H * kHead + h * kHead;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      reinterpret_cast<uint4*>(dst)[c] = make_uint4(pack_bf16x2(o[c * 8] * inv, o[c * 8 + 1] * inv), pack_bf16x2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv),
                                                    pack_bf16x2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv), pack_bf16x2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv));
    if (lse2) lse2[(int64_t)(s0 + q) * H + h] = m + log2f(l);
  }
  if (abort_flag) {
    // a wait ran out: a copy may still be on its way into shared memory; give it time before the memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, kTmemCols); }
  if (t == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

// ---------------------------------------------------------------------------------------------- backward
// delta[t, h] = sum_d dO[t, h, d] * O[t, h, d] (the row-wise correction term of the softmax backward); one warp per (t, h).
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, int64_t rows, float* __restrict__ delta) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162*>(o + r * kHead)[lane];
    const __nv_bfloat162 b = reinterpret_cast<const __nv_bfloat162*>(d_o + r * kHead)[lane];
    float v = __bfloat162float(a.x) * __bfloat162float(b.x) + __bfloat162float(a.y) * __bfloat162float(b.y);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) delta[r] = v;
  }
}

// One CTA owns one (sequence, head, 128-key tile) and walks the sequence's queries in tiles of 128. Per query tile:
//   S  = Q K^T, dP = dO V^T                          (two MMA chains, 128 x 128 x 64 each, results in tensor memory)
//   P  = exp2(S * scale * log2 e - lse2[q]),  dS = P * (dP - delta[q]) * scale        (thread = query row; written to shared
//                                                     memory as bf16 tiles [q][key])
//   dV += P^T dO, dK += dS^T Q                       (the [q][key] tiles read as MN-major A operands, dO / Q as MN-major B;
//                                                     accumulated in tensor memory over all query tiles)
//   dQ  = dS K                                       (the dS tile read as a K-major A operand, K as an MN-major B) and added to
//                                                     the global dQ with fp32 reductions (other key tiles add theirs)
// dK and dV of the tile's keys are stored once at the end. Gradients go to dqkv [T, 3 * H * 64] in fp32 (the q part must be
// zero on entry).
constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 320, kColDQ = 384;

// One thread's query row of a [128 q x 128 keys] tile in the backward: P = 2^(S * scale_log2 - lse) and
// dS = P * (dP - delta) * scale, written as bf16 into the [q][key] tiles. kMask selects whether key columns >= valid are
// masked (a masked entry enters the exponential as -inf, so P and dS are exact zeros there; dP and delta are finite).
template <bool kMask>
__device__ __forceinline__ void p_ds_chunk(const uint32_t (&rs)[32], const uint32_t (&rp)[32], int c0, int valid, float scale, float scale_log2,
                                           float lse_q, float nds, int t, uint8_t* ptile, uint8_t* dstile) {
  uint32_t pk[16], dk[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    float p[2], ds[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int c = c0 + 2 * e + u;
      const float x = (!kMask || c < valid) ? fmaf(__uint_as_float(rs[2 * e + u]), scale_log2, -lse_q) : -INFINITY;
      p[u] = fast_exp2(x);
      ds[u] = p[u] * fmaf(__uint_as_float(rp[2 * e + u]), scale, nds);
    }
    pk[e] = pack_bf16x2(p[0], p[1]);
    dk[e] = pack_bf16x2(ds[0], ds[1]);
  }
  const uint32_t boff = (uint32_t)(c0 >> 6) * kBlk;
#pragma unroll
  for (int cq = 0; cq < 4; ++cq) {
    const uint32_t off = boff + swizzle128_offset(t, (c0 & 63) + cq * 8);
    *reinterpret_cast<uint4*>(ptile + off) = make_uint4(pk[cq * 4], pk[cq * 4 + 1], pk[cq * 4 + 2], pk[cq * 4 + 3]);
    *reinterpret_cast<uint4*>(dstile + off) = make_uint4(dk[cq * 4], dk[cq * 4 + 1], dk[cq * 4 + 2], dk[cq * 4 + 3]);
  }
}

// The row is walked in four chunks of 32 key columns with two register sets: the next chunk's S and dP travel from tensor
// memory while the current chunk is computed.
template <bool kMask>
__device__ __forceinline__ void p_ds_row(uint32_t trow, int valid, float scale, float scale_log2, float lse_q, float delta_q, int t,
                                         uint8_t* ptile, uint8_t* dstile) {
  const float nds = -delta_q * scale;                              // (dP - delta) * scale = dP * scale + nds
  uint32_t sa[32], pa[32], sb[32], pb[32];
  tmem_ld32(trow + kColS, sa);
  tmem_ld32(trow + kColDP, pa);
  tmem_ld_wait();
  tmem_ld32(trow + kColS + 32u, sb);
  tmem_ld32(trow + kColDP + 32u, pb);
  p_ds_chunk<kMask>(sa, pa, 0, valid, scale, scale_log2, lse_q, nds, t, ptile, dstile);
  tmem_ld_wait();
  tmem_ld32(trow + kColS + 64u, sa);
  tmem_ld32(trow + kColDP + 64u, pa);
  p_ds_chunk<kMask>(sb, pb, 32, valid, scale, scale_log2, lse_q, nds, t, ptile, dstile);
  tmem_ld_wait();
  tmem_ld32(trow + kColS + 96u, sb);
  tmem_ld32(trow + kColDP + 96u, pb);
  p_ds_chunk<kMask>(sa, pa, 64, valid, scale, scale_log2, lse_q, nds, t, ptile, dstile);
  tmem_ld_wait();
  p_ds_chunk<kMask>(sb, pb, 96, valid, scale, scale_log2, lse_q, nds, t, ptile, dstile);
}

__global__ void __launch_bounds__(128, 1)
ragged_attention_bwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                            const float* __restrict__ lse2, const float* __restrict__ delta, const int32_t* __restrict__ offsets, int H,
                            float scale, float scale_log2, float* __restrict__ dqkv, const __grid_constant__ CUtensorMap map_dq, int dq_tma,
                            int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar1, bar2, bar_kv, bar_in[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int b = blockIdx.y, h = blockIdx.z, kt = blockIdx.x;
  const int s0 = offsets[b], L = offsets[b + 1] - s0;
  if (kt * kTile >= L) return;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* ktile = smem;                   // [128 keys][64 d]
  uint8_t* vtile = smem + kBlk;            // [128 keys][64 d]
  uint8_t* qtiles = smem + 2 * kBlk;       // 2 x [128 q][64 d]: this step's tile and the next one's, arriving
  uint8_t* dotiles = smem + 4 * kBlk;      // 2 x [128 q][64 d]
  uint8_t* ptile = smem + 6 * kBlk;        // 2 x [128 q][64 keys]
  uint8_t* dstile = smem + 8 * kBlk;       // 2 x [128 q][64 keys]
  uint8_t* dqstage = smem + 10 * kBlk;     // 2 x [128 q][32 d] fp32: the dQ tile on its way out (two 128-byte-wide boxes)
  const int t = threadIdx.x, warp = t >> 5;
  const int64_t ld = (int64_t)3 * H * kHead;
  // All tiles arrive by TMA (boxes of 128 rows x 64 columns of the packed matrices, 128-byte swizzle). Rows past the end of the
  // sequence belong to the next sequence: every such key and query is masked in P and dS below, and the surplus rows of the
  // tiles are zeroed in shared memory, so that the zeros of P and dS never meet a non-finite value.
  const int xq = h * kHead, xk = (H + h) * kHead, xv = (2 * H + h) * kHead;
  if (t == 0) {
    abort_flag = 0;
    mbar_init(&bar1, 1); mbar_init(&bar2, 1); mbar_init(&bar_kv, 1); mbar_init(&bar_in[0], 1); mbar_init(&bar_in[1], 1);
    mbar_fence_init();
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_qkv) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_do) : "memory");
    mbar_expect_tx(&bar_kv, 2 * kBlk);
    tma_load_2d(ktile, &map_qkv, xk, s0 + kt * kTile, &bar_kv);
    tma_load_2d(vtile, &map_qkv, xv, s0 + kt * kTile, &bar_kv);
    mbar_expect_tx(&bar_in[0], 2 * kBlk);
    tma_load_2d(qtiles, &map_qkv, xq, s0, &bar_in[0]);
    tma_load_2d(dotiles, &map_do, xq, s0, &bar_in[0]);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 512);

  const int key = kt * kTile + t;
  const bool key_ok = key < L;
  const int valid_keys = min(kTile, L - kt * kTile);
  // the first query tile's softmax statistics and correction terms
  float lse_next = t < L ? lse2[(int64_t)(s0 + t) * H + h] : 0.f;
  float delta_next = t < L ? delta[(int64_t)(s0 + t) * H + h] : 0.f;
  bool ok = mbar_wait(&bar_kv, 0, &abort_flag);
  if (ok && !key_ok) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      *reinterpret_cast<uint4*>(ktile + swizzle128_offset(t, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(vtile + swizzle128_offset(t, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  fence_smem_to_async();
  fence_before_sync();
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t idesc_kk = make_idesc_bf16(kTile, kTile, false, false);    // S, dP: both operands K-major
  const uint32_t idesc_mm = make_idesc_bf16(kTile, kHead, true, true);      // dV, dK: both operands MN-major
  const uint32_t idesc_km = make_idesc_bf16(kTile, kHead, false, true);     // dQ: A K-major, B MN-major

  const int n_q = (L + kTile - 1) / kTile;
  for (int i = 0; i < n_q && ok; ++i) {
    const int q = i * kTile + t;
    const bool q_ok = q < L;
    const int64_t tok = s0 + q;
    const int buf = i & 1;
    const uint32_t ph_in = (uint32_t)(i >> 1) & 1u;
    uint8_t* qtile = qtiles + buf * kBlk;
    uint8_t* dotile = dotiles + buf * kBlk;
    const float lse_q = lse_next, delta_q = delta_next;
    if (i + 1 < n_q) {
      // the next query tile travels while this one is computed; its buffer was last read by the MMAs of step i - 1 (bar2)
      const int64_t row0 = s0 + (i + 1) * kTile;
      const int left = L - (i + 1) * kTile;
      if (t == 0) {
        mbar_expect_tx(&bar_in[buf ^ 1], 2 * kBlk);
        tma_load_2d(qtiles + (buf ^ 1) * kBlk, &map_qkv, xq, (int)row0, &bar_in[buf ^ 1]);
        tma_load_2d(dotiles + (buf ^ 1) * kBlk, &map_do, xq, (int)row0, &bar_in[buf ^ 1]);
      }
      lse_next = t < left ? lse2[(row0 + t) * H + h] : 0.f;
      delta_next = t < left ? delta[(row0 + t) * H + h] : 0.f;
    }
    if (L - i * kTile < kTile) {
      // last, partial query tile: its surplus rows become zeros (this thread's row, once the tile has landed)
      ok = mbar_wait(&bar_in[buf], ph_in, &abort_flag);
      if (ok && !q_ok) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          *reinterpret_cast<uint4*>(qtile + swizzle128_offset(t, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(dotile + swizzle128_offset(t, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      fence_smem_to_async();
      fence_before_sync();
      ok = __syncthreads_and(ok ? 1 : 0) != 0;
      fence_after_sync();
      if (!ok) break;
    }
    if (t == 0) {
      if (mbar_wait(&bar_in[buf], ph_in, &abort_flag)) {
        fence_after_sync();
        const uint32_t sq = smem_u32(qtile), sk = smem_u32(ktile), sdo = smem_u32(dotile), sv = smem_u32(vtile);
#pragma unroll
        for (int k = 0; k < kHead / 16; ++k)
          umma_bf16(tmem + kColS, make_desc(sq + k * 32, 16, 1024), make_desc(sk + k * 32, 16, 1024), idesc_kk, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < kHead / 16; ++k)
          umma_bf16(tmem + kColDP, make_desc(sdo + k * 32, 16, 1024), make_desc(sv + k * 32, 16, 1024), idesc_kk, k > 0 ? 1u : 0u);
        umma_commit(&bar1);
      }
    }
    ok = __syncthreads_and(mbar_wait(&bar1, (uint32_t)(i & 1), &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;

    // masking is needed only where the tile holds a key or a query that does not exist (the sequence's last tiles)
    const int vk = q_ok ? valid_keys : 0;                          // key columns of this thread's row that count
    if (valid_keys == kTile && L - i * kTile >= kTile)
      p_ds_row<false>(tmem + lane_base, kTile, scale, scale_log2, lse_q, delta_q, t, ptile, dstile);
    else
      p_ds_row<true>(tmem + lane_base, vk, scale, scale_log2, lse_q, delta_q, t, ptile, dstile);
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (t == 0) {
      const uint32_t sp = smem_u32(ptile), sds = smem_u32(dstile), sq = smem_u32(qtile), sdo = smem_u32(dotile), sk = smem_u32(ktile);
      const uint32_t acc0 = i > 0 ? 1u : 0u;
#pragma unroll
      for (int k = 0; k < kTile / 16; ++k) {        // reduction over the 128 queries of this tile, 16 rows per step
        // A = P^T / dS^T: [q][key] tiles read MN-major (M = key: two 64-wide blocks kBlk apart, 16 q rows = 2048 bytes per step)
        // B = dO / Q:     [q][d] tiles read MN-major (N = d, one 64-wide block)
        umma_bf16(tmem + kColDV, make_desc(sp + k * 2048, kBlk, 1024), make_desc(sdo + k * 2048, kBlk, 1024), idesc_mm, (acc0 | (k > 0 ? 1u : 0u)));
        umma_bf16(tmem + kColDK, make_desc(sds + k * 2048, kBlk, 1024), make_desc(sq + k * 2048, kBlk, 1024), idesc_mm, (acc0 | (k > 0 ? 1u : 0u)));
      }
#pragma unroll
      for (int k = 0; k < kTile / 16; ++k)          // reduction over the 128 keys: dS read K-major, K read MN-major
        umma_bf16(tmem + kColDQ, make_desc(sds + (k >> 2) * kBlk + (k & 3) * 32, 16, 1024), make_desc(sk + k * 2048, kBlk, 1024), idesc_km,
                  k > 0 ? 1u : 0u);
      umma_commit(&bar2);
      // the previous step's dQ tile must have been read before this step's is written over it (after the barrier below)
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    ok = __syncthreads_and(mbar_wait(&bar2, (uint32_t)(i & 1), &abort_flag) ? 1 : 0) != 0;
    fence_after_sync();
    if (!ok) break;
    for (int c0 = 0; c0 < kHead; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + kColDQ + (uint32_t)c0, r);
      tmem_ld_wait();
      if (dq_tma) {
        // row t of a 32-column fp32 box: eight 16-byte chunks in the 128-byte swizzle
        uint8_t* row = dqstage + (c0 >> 5) * kBlk + t * 128;
#pragma unroll
        for (int e = 0; e < 8; ++e)
          *reinterpret_cast<float4*>(row + ((e ^ (t & 7)) << 4)) = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                                                               __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3]));
      } else if (q_ok) {
        float* dst = dqkv + tok * ld + h * kHead + c0;
#pragma unroll
        for (int e = 0; e < 8; ++e)
          atomicAdd(reinterpret_cast<float4*>(dst) + e, make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]),
                                                                    __uint_as_float(r[4 * e + 2]), __uint_as_float(r[4 * e + 3])));
      }
    }
    if (dq_tma) {
      // The tile leaves as two add-reductions of [128 rows x 32 columns]. Rows past the end of this sequence hold exact zeros
      // (their P and dS were masked), so adding them onto the next sequence's rows changes nothing; rows past the end of the
      // matrix are clipped by the copy.
      fence_smem_to_async();
      __syncthreads();
      if (t == 0) {
#pragma unroll
        for (int bx = 0; bx < 2; ++bx)
          asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                       ::"l"(&map_dq), "r"(smem_u32(dqstage + bx * kBlk)), "r"(h * kHead + bx * 32), "r"(s0 + i * kTile) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
  }
  if (t == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the copies that read it
  if (abort_flag) {
    // a wait ran out: a tile may still be on its way into shared memory; give it time before the memory goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }

  if (ok) {
    for (int c0 = 0; c0 < kHead; c0 += 32) {
      uint32_t rv[32], rk[32];
      tmem_ld32(tmem + lane_base + kColDV + (uint32_t)c0, rv);
      tmem_ld32(tmem + lane_base + kColDK + (uint32_t)c0, rk);
      tmem_ld_wait();
      if (key_ok) {
        float* dk_dst = dqkv + (int64_t)(s0 + key) * ld + (H + h) * kHead + c0;
        float* dv_dst = dk_dst + H * kHead;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          reinterpret_cast<float4*>(dk_dst)[e] = make_float4(__uint_as_float(rk[4 * e]), __uint_as_float(rk[4 * e + 1]),
                                                             __uint_as_float(rk[4 * e + 2]), __uint_as_float(rk[4 * e + 3]));
          reinterpret_cast<float4*>(dv_dst)[e] = make_float4(__uint_as_float(rv[4 * e]), __uint_as_float(rv[4 * e + 1]),
                                                             __uint_as_float(rv[4 * e + 2]), __uint_as_float(rv[4 * e + 3]));
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) { fence_after_sync(); tmem_dealloc(tmem, 512); }
  if (t == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

}  // namespace

// qkv: bf16 [T, 3 * H * 64] packed (q | k | v, each H heads of 64), T tokens, offsets: int32 [B + 1] on the device, max_len: an upper bound
// of the sequence lengths (sizes the grid), out: bf16 [T, H * 64], lse2: fp32 [T, H] or null (log2-domain log-sum-exp).
// Returns 0 on launch, 1 when the arguments are outside the kernel's range (alignment), > 1 on a launch error.
extern "C" int rb_ragged_attention_fwd(const void* qkv, const int32_t* offsets, int64_t T, int B, int H, int max_len, float scale, void* out,
                                       float* lse2, int64_t* status, cudaStream_t st) {
  if (B <= 0 || H <= 0 || max_len <= 0 || T <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return 1;
  CUtensorMap map_qkv;
  if (rb_tensor_map_2d(&map_qkv, qkv, T, (int64_t)3 * H * kHead, (int64_t)3 * H * kHead, kHead, kTile, 0) != 0) return 1;
  const size_t smem = 1024 + 5 * (size_t)kBlk;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ragged_attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
    attr = true;
  }
  dim3 grid((max_len + kTile - 1) / kTile, B, H);
  ragged_attention_fwd_kernel<<<grid, 128, smem, st>>>(map_qkv, offsets, H, scale * 1.4426950408889634f,
                                                       reinterpret_cast<__nv_bfloat16*>(out), lse2, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// Backward of rb_ragged_attention_fwd. out / d_out: bf16 [T, H * 64]; lse2: fp32 [T, H] from the forward; delta: fp32 [T, H]
// scratch; dqkv: fp32 [T, 3 * H * 64], zero on entry (dQ is accumulated with reductions). Same return codes as the forward.
extern "C" int rb_ragged_attention_bwd(const void* qkv, const void* out, const void* d_out, const float* lse2, float* delta,
                                       const int32_t* offsets, int64_t T, int B, int H, int max_len, float scale, float* dqkv,
                                       int64_t* status, cudaStream_t st) {
  if (B <= 0 || H <= 0 || max_len <= 0 || T <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(d_out) & 15) || (reinterpret_cast<uintptr_t>(dqkv) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 3))
    return 1;
  const int64_t rows = T * H;
  const int64_t blocks = (rows + 7) / 8;
  attention_delta_kernel<<<(int)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                                                   reinterpret_cast<const __nv_bfloat16*>(d_out), rows, delta);
  rb::note_launch();
  const size_t smem = 1024 + 12 * (size_t)kBlk;
  CUtensorMap map_qkv, map_do;
  if (rb_tensor_map_2d(&map_qkv, qkv, T, (int64_t)3 * H * kHead, (int64_t)3 * H * kHead, kHead, kTile, 0) != 0 ||
      rb_tensor_map_2d(&map_do, d_out, T, (int64_t)H * kHead, (int64_t)H * kHead, kHead, kTile, 0) != 0)
    return 1;
  // dQ leaves as TMA add-reductions of [128 x 32] fp32 boxes when a tensor map can be made; otherwise as per-row reductions
  CUtensorMap map_dq;
  const int dq_tma = rb_tensor_map_2d(&map_dq, dqkv, T, (int64_t)3 * H * kHead, (int64_t)3 * H * kHead, 32, kTile, 1) == 0 ? 1 : 0;
  if (!dq_tma) memset(&map_dq, 0, sizeof(map_dq));
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ragged_attention_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
    attr = true;
  }
  dim3 grid((max_len + kTile - 1) / kTile, B, H);
  ragged_attention_bwd_kernel<<<grid, 128, smem, st>>>(map_qkv, map_do, lse2, delta, offsets, H, scale, scale * 1.4426950408889634f, dqkv,
                                                       map_dq, dq_tma, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
