// bf16 GEMM for the dense towers on the 5th-generation tensor cores (sm_100a):
//   D[MM, NN] = act( A[MM, KK] * B[NN, KK]^T + bias[NN] )            fp32 accumulation in tensor memory
//
// * operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no cluster multicast),
// * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x BN x 16 per instruction),
// * the accumulator lives in TMEM and is read back with tcgen05.ld for a fused bias + ReLU + convert epilogue; the converted
//   tile is staged in the (by then idle) operand stages in the 128-byte swizzled layout and leaves with TMA stores, one
//   32-row slab per epilogue warp (split-K partial tiles leave with TMA fp32 add-reductions),
// * warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer (owns the TMEM allocation), warps 2..5 = epilogue,
// * a ring of kStages shared-memory stages with full/empty mbarriers overlaps copies with math.
//
// Either operand may be "K-major" (reduction dimension contiguous in memory: x[MM][KK]) or "MN-major" (output
// dimension contiguous: x[KK][MM]); the second form is what the backward GEMMs need (dgrad reads W[N][K] as its
// B operand, wgrad reads dY[M][N] and X[M][K] with the batch as the reduction), so no transposed copies are made.
//
// The reference has no GEMM kernel of its own: its dense layers are nn.Linear (cuBLAS), see
// examples/deepfm/deepfm_model.py:49-52 in the reference project.
//
// Every mbarrier wait is bounded; on a timeout the kernel records kStatusWaitTimeout in the status word, drains its
// outstanding copies (bounded), frees its tensor memory and returns.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "../common/rb_tcgen05.cuh"
#include "rb_dense.h"
#include "rb_gemm_store.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace {

using namespace rb::tc;      // mbarrier / TMA / tcgen05 wrappers and descriptor builders

constexpr int BM = 128;       // rows of D per CTA (= UMMA M, = TMEM lanes)
constexpr int BN = 128;       // columns of D per CTA (= UMMA N, = TMEM fp32 columns)
constexpr int BK = 64;        // reduction elements per stage (64 bf16 = one 128-byte swizzle row)
constexpr int UK = 16;        // reduction elements per tcgen05.mma (bf16)
constexpr int kStages = 3;     // 3 x 32 KB: two CTAs fit on one SM, so one CTA's epilogue overlaps the other's main loop
constexpr int kThreads = 192;
constexpr uint32_t kTileBytes = BM * BK * 2;                    // 16 KB per operand per stage
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;   // + slack for 1024-byte alignment

using rb::gemm::Store;

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kThreads, 2)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_o, int tma_out, OutT* __restrict__ out,
                         const float* __restrict__ bias, const float* __restrict__ beta_src, const RbGemmEpilogue epi,
                         int MM, int NN, int KK, int ldo, int relu, int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float bias_s[BN];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // split-K: blockIdx.z owns a contiguous range of reduction blocks and accumulates its partial tile with fp32 reductions
  const int total_kb = (KK + BK - 1) / BK;
  const int kb_per = (total_kb + (int)gridDim.z - 1) / (int)gridDim.z;
  const int kb_begin = (int)blockIdx.z * kb_per;
  const int num_kb = max(0, min(total_kb, kb_begin + kb_per) - kb_begin);
  const bool split = gridDim.z > 1;
  if (split && num_kb == 0) return;           // uniform for the whole CTA, before any barrier or allocation

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&tmem_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (warp >= 2) {
    // the tile's bias, fetched while the main loop has not even started (of a split reduction only the first part adds it)
    const int t = (int)threadIdx.x - 64;
    bias_s[t] = (bias != nullptr && n0 + t < NN && (!split || blockIdx.z == 0)) ? bias[n0 + t] : 0.f;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    int issued = 0;
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % kStages;
      const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
      ok = mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag);
      if (!ok) break;
      uint8_t* sa = smem + s * kStageBytes;
      uint8_t* sb = sa + kTileBytes;
      mbar_expect_tx(&full_bar[s], kStageBytes);
      const int k0 = (kb_begin + kb) * BK;
      if (!A_MN) tma_load_2d(sa, &map_a, k0, m0, &full_bar[s]);                      // box {BK, BM}
      else { tma_load_2d(sa, &map_a, m0, k0, &full_bar[s]); tma_load_2d(sa + kTileBytes / 2, &map_a, m0 + 64, k0, &full_bar[s]); }  // 2 x box {64, BK}
      if (!B_MN) tma_load_2d(sb, &map_b, k0, n0, &full_bar[s]);
      else { tma_load_2d(sb, &map_b, n0, k0, &full_bar[s]); tma_load_2d(sb + kTileBytes / 2, &map_b, n0 + 64, k0, &full_bar[s]); }
      ++issued;
    }
    if (!ok) {
      // drain: the copies already issued must land before this CTA's shared memory goes away
      for (int j = max(0, issued - kStages); j < issued; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (uint32_t)(j / kStages) & 1u;
        for (uint32_t it = 0; it < kSpinLimit; ++it) if (mbar_try_wait(&full_bar[s], ph)) break;
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer
    // instruction descriptor: D = f32, A = B = bf16, majors, N >> 3, M >> 4
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % kStages;
      const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
      ok = mbar_wait(&full_bar[s], ph, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sa = smem_u32(smem + s * kStageBytes), sb = sa + kTileBytes;
#pragma unroll
      for (int k = 0; k < BK / UK; ++k) {
        // K-major: 16 elements = 32 bytes further along the swizzled 128-byte row; 8-row groups are 1024 bytes apart.
        // MN-major: 16 reduction rows = two 8-row (1024-byte) groups; 64-wide MN blocks are BK*128 bytes apart.
        const uint64_t da = A_MN ? make_desc(sa + k * 2048, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
        const uint64_t db = B_MN ? make_desc(sb + k * 2048, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
        umma_bf16(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&empty_bar[s]);     // stage reusable once these MMAs have read it
    }
    if (ok) umma_commit(&tmem_full_bar);
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue (4 warps, one TMEM lane quarter each)
    const bool ok = num_kb > 0 ? mbar_wait(&tmem_full_bar, 0, &abort_flag) : true;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
      const bool add_beta = beta_src != nullptr && (!split || blockIdx.z == 0);
      const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
      // every MMA has completed (tmem_full), so nothing reads the operand stages any more: they become the staging area.
      // One slab of 32 rows per warp, made of boxes of 32 rows x 128 bytes in the layout the TMA store expects.
      constexpr int kBoxes = BN / Store<OutT>::kBoxCols;
      uint8_t* slab = smem + q * kBoxes * 4096;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= NN) break;
        uint32_t r[32];
        if (num_kb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        float v[32];
        const int valid = min(32, NN - (n0 + c0));
        const float* brow = beta_src + (int64_t)row * ldo + n0 + c0;
        const bool beta_here = add_beta && row < MM;
        const bool beta_vec = beta_here && valid == 32 && (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(beta_src) & 15) == 0);
#pragma unroll
        for (int j4 = 0; j4 < 32; j4 += 4) {
          float4 bt = make_float4(0.f, 0.f, 0.f, 0.f);
          if (beta_vec) bt = *reinterpret_cast<const float4*>(brow + j4);
          else if (beta_here) {
            if (j4 + 0 < valid) bt.x = brow[j4 + 0];
            if (j4 + 1 < valid) bt.y = brow[j4 + 1];
            if (j4 + 2 < valid) bt.z = brow[j4 + 2];
            if (j4 + 3 < valid) bt.w = brow[j4 + 3];
          }
          const float4 bs = *reinterpret_cast<const float4*>(&bias_s[c0 + j4]);
          const float x0 = __uint_as_float(r[j4 + 0]) + bs.x + bt.x, x1 = __uint_as_float(r[j4 + 1]) + bs.y + bt.y;
          const float x2 = __uint_as_float(r[j4 + 2]) + bs.z + bt.z, x3 = __uint_as_float(r[j4 + 3]) + bs.w + bt.w;
          v[j4 + 0] = relu ? fmaxf(x0, 0.f) : x0; v[j4 + 1] = relu ? fmaxf(x1, 0.f) : x1;
          v[j4 + 2] = relu ? fmaxf(x2, 0.f) : x2; v[j4 + 3] = relu ? fmaxf(x3, 0.f) : x3;
        }
        if (epi.mask_src != nullptr)
          rb::gemm::apply_mask32(v, reinterpret_cast<const __nv_bfloat16*>(epi.mask_src) + (int64_t)row * epi.mask_ld + n0 + c0, valid, row < MM);
        if (tma_out) Store<OutT>::stage32(slab, lane, c0, v);
        else if (row < MM) {
          if (split) Store<OutT>::red32(out + (int64_t)row * ldo + n0 + c0, v, valid, vec_ok);
          else Store<OutT>::row32(out + (int64_t)row * ldo + n0 + c0, v, valid, vec_ok);
        }
        if (epi.colsum != nullptr) {
          if (row >= MM) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          rb::gemm::column_sums32(v, lane, valid, epi.colsum + n0 + c0);
        }
      }
      if (tma_out) {
        // the slab leaves through the async proxy: order this warp's shared-memory writes before it, then one lane stores
        // (or add-reduces, for a split reduction) each box; rows and columns beyond the matrix are clipped by the copy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && m0 + q * 32 < MM) {
#pragma unroll
          for (int bx = 0; bx < kBoxes; ++bx) {
            const int col = n0 + bx * Store<OutT>::kBoxCols;
            if (col >= NN) break;
            if (split)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(slab + bx * 4096)), "r"(col), "r"(m0 + q * 32) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(slab + bx * 4096)), "r"(col), "r"(m0 + q * 32) : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the slab must stay until the copies have read it
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

// ---------------------------------------------------------------------- persistent variant
// One CTA per SM walks a strided list of output tiles. Two accumulator stages live in tensor memory (2 x BN columns): while the
// epilogue warps drain the accumulator of tile i (tcgen05.ld, bias / residual / ReLU, staging, TMA store), the MMA warp already
// fills the other accumulator with tile i+1, and the TMA warp runs ahead through the shared-memory ring across tile
// boundaries. With the whole SM to itself the CTA has a deeper ring (six stages for bf16 output, five for fp32) and a
// staging area of its own, so a tile's prologue and epilogue cost nothing after the first tile - which is what the short
// reductions (K = 512 .. 1024) of recommendation MLPs were expected to need. Measured, it is slower than two co-resident
// one-tile CTAs (8192^3: 0.90 against 1.16 PFLOP/s; 8192 x 1024 x 1024: 36 against 31 microseconds): with 128 x 128 tiles the
// tensor core's operand reads and the TMA fills together ask for twice the shared-memory bandwidth of an SM, and two independent
// producer / consumer chains use what there is better than one deep ring. Opt-in (RECIS_GEMM_PERSISTENT=1), kept for
// comparison; it needs an output that can leave through TMA stores, and split reductions keep the kernel above.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename OutT> struct PersistentCfg;
template <> struct PersistentCfg<__nv_bfloat16> { static constexpr int kStagesP = 6; static constexpr uint32_t kStagingBytes = BM * BN * 2; };
template <> struct PersistentCfg<float> { static constexpr int kStagesP = 5; static constexpr uint32_t kStagingBytes = BM * BN * 4; };
template <typename OutT> constexpr uint32_t persistent_smem_bytes() {
  return PersistentCfg<OutT>::kStagesP * kStageBytes + PersistentCfg<OutT>::kStagingBytes + 1024;
}

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                    const __grid_constant__ CUtensorMap map_o, const float* __restrict__ bias,
                                    const float* __restrict__ beta_src, int MM, int NN, int KK, int ldo, int relu,
                                    int64_t* __restrict__ status) {
  constexpr int S = PersistentCfg<OutT>::kStagesP;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[S];
  __shared__ __align__(8) uint64_t empty_bar[S];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + S * kStageBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (NN + BN - 1) / BN, tiles_m = (MM + BM - 1) / BM;
  const int num_tiles = tiles_n * tiles_m;
  const int total_kb = (KK + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full_bar[a], 1); mbar_init(&acc_empty_bar[a], 4); }   // 4 epilogue warps release a stage
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)(2 * BN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer: runs ahead across tiles
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    uint32_t it = 0;
    uint32_t issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        ok = mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag);
        if (!ok) break;
        uint8_t* sa = smem + s * kStageBytes;
        uint8_t* sb = sa + kTileBytes;
        mbar_expect_tx(&full_bar[s], kStageBytes);
        const int k0 = kb * BK;
        if (!A_MN) tma_load_2d(sa, &map_a, k0, m0, &full_bar[s]);
        else { tma_load_2d(sa, &map_a, m0, k0, &full_bar[s]); tma_load_2d(sa + kTileBytes / 2, &map_a, m0 + 64, k0, &full_bar[s]); }
        if (!B_MN) tma_load_2d(sb, &map_b, k0, n0, &full_bar[s]);
        else { tma_load_2d(sb, &map_b, n0, k0, &full_bar[s]); tma_load_2d(sb + kTileBytes / 2, &map_b, n0 + 64, k0, &full_bar[s]); }
        ++issued;
      }
    }
    if (!ok) {
      // drain: copies already issued must land before this CTA's shared memory goes away
      const uint32_t first = issued > (uint32_t)S ? issued - S : 0u;
      for (uint32_t j = first; j < issued; ++j) {
        const int s = j % S;
        const uint32_t ph = (j / S) & 1u;
        for (uint32_t spin = 0; spin < kSpinLimit; ++spin) if (mbar_try_wait(&full_bar[s], ph)) break;
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------ MMA issuer: alternates between the two accumulators
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    uint32_t it = 0, j = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++j) {
      const uint32_t acc = j & 1u, acc_ph = (j >> 1) & 1u;
      ok = mbar_wait(&acc_empty_bar[acc], acc_ph ^ 1u, &abort_flag);      // the epilogue has drained this accumulator
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + acc * (uint32_t)BN;
      for (int kb = 0; kb < total_kb; ++kb, ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        ok = mbar_wait(&full_bar[s], ph, &abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(smem + s * kStageBytes), sb = sa + kTileBytes;
#pragma unroll
        for (int k = 0; k < BK / UK; ++k) {
          const uint64_t da = A_MN ? make_desc(sa + k * 2048, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
          const uint64_t db = B_MN ? make_desc(sb + k * 2048, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
          umma_bf16(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&acc_full_bar[acc]);
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue: drains accumulator j & 1 of every tile
    const int q = warp & 3;
    constexpr int kBoxes = BN / Store<OutT>::kBoxCols;
    uint8_t* slab = staging + q * kBoxes * 4096;          // this warp's 32 rows, as boxes of 32 rows x 128 bytes
    uint32_t j = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++j) {
      const uint32_t acc = j & 1u, acc_ph = (j >> 1) & 1u;
      const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
      const int row = m0 + q * 32 + lane;
      // this tile's bias for the lane's four column chunks, fetched before the accumulator is waited for
      float bias_r[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) bias_r[c] = (bias != nullptr && n0 + c * 32 + lane < NN) ? bias[n0 + c * 32 + lane] : 0.f;
      if (!mbar_wait(&acc_full_bar[acc], acc_ph, &abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // the previous tile's stores must have read the slab before it is written again
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int c0 = c * 32;
        if (n0 + c0 < NN) {                                  // uniform for the warp
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * (uint32_t)BN + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          float v[32];
          const int valid = min(32, NN - (n0 + c0));
          const float* brow = beta_src + (int64_t)row * ldo + n0 + c0;
          const bool beta_here = beta_src != nullptr && row < MM;
          const bool beta_vec = beta_here && valid == 32 && (ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(beta_src) & 15) == 0);
#pragma unroll
          for (int j4 = 0; j4 < 32; j4 += 4) {
            float4 bt = make_float4(0.f, 0.f, 0.f, 0.f);
            if (beta_vec) bt = *reinterpret_cast<const float4*>(brow + j4);
            else if (beta_here) {
              if (j4 + 0 < valid) bt.x = brow[j4 + 0];
              if (j4 + 1 < valid) bt.y = brow[j4 + 1];
              if (j4 + 2 < valid) bt.z = brow[j4 + 2];
              if (j4 + 3 < valid) bt.w = brow[j4 + 3];
            }
            // column c0 + j's bias sits in lane j's register
            const float x0 = __uint_as_float(r[j4 + 0]) + __shfl_sync(0xffffffffu, bias_r[c], j4 + 0) + bt.x;
            const float x1 = __uint_as_float(r[j4 + 1]) + __shfl_sync(0xffffffffu, bias_r[c], j4 + 1) + bt.y;
            const float x2 = __uint_as_float(r[j4 + 2]) + __shfl_sync(0xffffffffu, bias_r[c], j4 + 2) + bt.z;
            const float x3 = __uint_as_float(r[j4 + 3]) + __shfl_sync(0xffffffffu, bias_r[c], j4 + 3) + bt.w;
            v[j4 + 0] = relu ? fmaxf(x0, 0.f) : x0; v[j4 + 1] = relu ? fmaxf(x1, 0.f) : x1;
            v[j4 + 2] = relu ? fmaxf(x2, 0.f) : x2; v[j4 + 3] = relu ? fmaxf(x3, 0.f) : x3;
          }
          Store<OutT>::stage32(slab, lane, c0, v);
        }
      }
      // every lane's tcgen05.ld has completed (wait::ld above): the accumulator goes back to the MMA warp before the stores
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty_bar[acc]);
        if (m0 + q * 32 < MM) {
#pragma unroll
          for (int bx = 0; bx < kBoxes; ++bx) {
            const int col = n0 + bx * Store<OutT>::kBoxCols;
            if (col >= NN) break;
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_o), "r"(smem_u32(slab + bx * 4096)), "r"(col), "r"(m0 + q * 32) : "memory");
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the stores' reads
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                             CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// 2-D tensor [rows][cols] (cols contiguous, row pitch ld elements) of bf16 (fp32 = false) or fp32, box {box_cols, box_rows},
// 128-byte swizzle. Encoding costs a microsecond or two of host time and the same few operands come back every step (the
// weights always, the activations whenever the caching allocator hands the same block out again), so encoded maps are kept
// per thread, keyed by everything that goes into them.
struct MapKey {
  const void* base; int64_t rows, cols, ld; int box_cols, box_rows, fp32;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols && box_rows == o.box_rows && fp32 == o.fp32;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    for (uint64_t v : {(uint64_t)k.rows, (uint64_t)k.cols, (uint64_t)k.ld, (uint64_t)((k.box_cols << 12) ^ (k.box_rows << 1) ^ k.fp32)})
      h = (h ^ v) * 0x100000001B3ull + (h >> 29);
    return (size_t)h;
  }
};

bool get_map(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows, bool fp32) {
  thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, cols, ld, box_cols, box_rows, fp32 ? 1 : 0};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (fp32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() >= 512) cache.clear();          // bounded: a map is 128 bytes and cheap to make again
  cache.emplace(key, map);
  *out = map;
  return true;
}

template <bool A_MN, bool B_MN, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, int tma_out, void* out, const float* bias, const float* beta_src,
           const RbGemmEpilogue& epi, int MM, int NN, int KK, int ldo, int relu, int splits, int64_t* status, cudaStream_t st) {
  auto kern = gemm_bf16_tcgen05_kernel<A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess) return 3;
    attr_set = true;
  }
  dim3 grid((NN + BN - 1) / BN, (MM + BM - 1) / BM, splits);
  kern<<<grid, kThreads, kSmemBytes, st>>>(ma, mb, mo, tma_out, reinterpret_cast<OutT*>(out), bias, beta_src, epi, MM, NN, KK, ldo, relu, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

template <bool A_MN, bool B_MN, typename OutT>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const float* bias, const float* beta_src, int MM,
                      int NN, int KK, int ldo, int relu, int64_t* status, cudaStream_t st) {
  auto kern = gemm_bf16_tcgen05_persistent_kernel<A_MN, B_MN, OutT>;
  constexpr uint32_t smem = persistent_smem_bytes<OutT>();
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 3;
    attr_set = true;
  }
  const int tiles = ((NN + BN - 1) / BN) * ((MM + BM - 1) / BM);
  const int grid = std::min(tiles, 148);               // one CTA per SM (2 x 128 tensor-memory columns, about 225 KB shared memory)
  kern<<<grid, kThreads, smem, st>>>(ma, mb, mo, bias, beta_src, MM, NN, KK, ldo, relu, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

// RECIS_GEMM_2CTA: unset = the kernel that pairs two SMs on a 256 x 256 tile takes the problems that fill the GPU with such
// tiles, 1 = every problem of at least 192 x 192, 0 = never
int pair_mode() {
  static const int mode = [] { const char* e = std::getenv("RECIS_GEMM_2CTA"); return e == nullptr ? -1 : (e[0] == '1' ? 1 : 0); }();
  return mode;
}

bool persistent_enabled() {
  static const bool on = [] { const char* e = std::getenv("RECIS_GEMM_PERSISTENT"); return e != nullptr && e[0] == '1'; }();
  return on;
}

}  // namespace

extern "C" int rb_tensor_map_2d(void* out_map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows, int fp32) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld * (fp32 ? 4 : 2)) % 16) return 1;
  return get_map(reinterpret_cast<CUtensorMap*>(out_map), base, rows, cols, ld, box_cols, box_rows, fp32 != 0) ? 0 : 2;
}

extern "C" int rb_gemm_splits(int MM, int NN, int KK) {
  // few output tiles and a long reduction (weight gradients): spread the reduction over about two waves of CTAs
  const int tiles = ((NN + BN - 1) / BN) * ((MM + BM - 1) / BM);
  const int total_kb = (KK + BK - 1) / BK;
  int splits = (2 * 148 + tiles - 1) / tiles;
  splits = std::min(splits, total_kb / 4);
  return std::max(splits, 1);
}

extern "C" int rb_gemm_bf16(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo,
                            int out_fp32, const float* bias, const float* beta_src, int MM, int NN, int KK, int relu, int splits,
                            int64_t* status, cudaStream_t st) {
  return rb_gemm_bf16_ex(a, lda, a_mn, b, ldb, b_mn, out, ldo, out_fp32, bias, beta_src, nullptr, MM, NN, KK, relu, splits, status, st);
}

extern "C" int rb_gemm_bf16_ex(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo,
                               int out_fp32, const float* bias, const float* beta_src, const RbGemmEpilogue* epi_in, int MM, int NN, int KK,
                               int relu, int splits, int64_t* status, cudaStream_t st) {
  RbGemmEpilogue epi{nullptr, 0, nullptr};
  if (epi_in != nullptr) epi = *epi_in;
  const bool extra = epi.mask_src != nullptr || epi.colsum != nullptr;
  if (extra && splits > 1) return 6;                 // a mask or column sums need the whole reduction in one CTA
  if (MM <= 0 || NN <= 0) return 0;
  // TMA constraints: 16-byte aligned base, row pitch a multiple of 16 bytes
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (lda % 8) || (ldb % 8)) return 1;
  // Pairs of SMs on 256 x 256 tiles when that fills the GPU: at least 192 CTAs (a split reduction is cut finer to get there)
  const int pmode = pair_mode();
  if (pmode != 0 && MM >= 192 && NN >= 192) {
    const int pairs = ((MM + 255) / 256) * ((NN + 255) / 256);
    int psplits = 1;
    if (splits > 1) {
      const int total_kb = (KK + BK - 1) / BK;
      psplits = std::max(1, std::min((256 + 2 * pairs - 1) / (2 * pairs), total_kb / 4));
    }
    if (pmode == 1 || 2 * pairs * psplits >= 192) {
      const int rc = rb_gemm_bf16_pair(a, lda, a_mn, b, ldb, b_mn, out, ldo, out_fp32, bias, beta_src, &epi, MM, NN, KK, relu, psplits, status, st);
      if (rc != 7) return rc;
    }
  }
  CUtensorMap ma, mb, mo;
  const bool oka = a_mn ? get_map(&ma, a, KK, MM, lda, 64, BK, false) : get_map(&ma, a, MM, KK, lda, BK, BM, false);
  const bool okb = b_mn ? get_map(&mb, b, KK, NN, ldb, 64, BK, false) : get_map(&mb, b, NN, KK, ldb, BK, BN, false);
  if (!oka || !okb) return 2;
  // the output leaves through TMA stores when its base and row pitch are 16-byte aligned; otherwise rows are stored directly
  const int es = out_fp32 ? 4 : 2;
  int tma_out = 0;
  if ((reinterpret_cast<uintptr_t>(out) & 15) == 0 && (ldo * es) % 16 == 0 && get_map(&mo, out, MM, NN, ldo, out_fp32 ? 32 : 64, 32, out_fp32 != 0))
    tma_out = 1;
  else
    mo = ma;
  if (splits > 1 && (!out_fp32 || relu)) return 6;   // partial tiles are accumulated with fp32 reductions into a zeroed output
  if (persistent_enabled() && tma_out && splits <= 1 && KK > 0 && !extra) {
#define RB_GEMM_PCASE(AM, BMJ)                                                                                                  \
  if ((a_mn != 0) == AM && (b_mn != 0) == BMJ)                                                                                  \
    return out_fp32 ? launch_persistent<AM, BMJ, float>(ma, mb, mo, bias, beta_src, MM, NN, KK, (int)ldo, relu, status, st)             \
                    : launch_persistent<AM, BMJ, __nv_bfloat16>(ma, mb, mo, bias, beta_src, MM, NN, KK, (int)ldo, relu, status, st);
    RB_GEMM_PCASE(false, false)
    RB_GEMM_PCASE(false, true)
    RB_GEMM_PCASE(true, false)
    RB_GEMM_PCASE(true, true)
#undef RB_GEMM_PCASE
  }
#define RB_GEMM_CASE(AM, BMJ)                                                                                                   \
  if ((a_mn != 0) == AM && (b_mn != 0) == BMJ)                                                                                  \
    return out_fp32 ? launch<AM, BMJ, float>(ma, mb, mo, tma_out, out, bias, beta_src, epi, MM, NN, KK, (int)ldo, relu, splits, status, st)  \
                    : launch<AM, BMJ, __nv_bfloat16>(ma, mb, mo, tma_out, out, bias, beta_src, epi, MM, NN, KK, (int)ldo, relu, 1, status, st);
  RB_GEMM_CASE(false, false)
  RB_GEMM_CASE(false, true)
  RB_GEMM_CASE(true, false)
  RB_GEMM_CASE(true, true)
#undef RB_GEMM_CASE
  return 5;
}
