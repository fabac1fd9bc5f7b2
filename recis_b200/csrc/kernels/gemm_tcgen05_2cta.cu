// bf16 GEMM on pairs of SMs (tcgen05 cta_group::2): D[MM, NN] = act( A[MM, KK] * B[NN, KK]^T + bias + residual ).
//
// Two CTAs of a cluster, on the two SMs of one pair, compute one 256 x 256 tile of D together. Each CTA stages ITS half of the
// operands - 128 rows of A and 128 rows of B per 64-wide reduction step, 32 KB - with plain TMA loads of its own, and keeps its
// 128 rows of the fp32 accumulator (256 columns) in its own tensor memory; one thread of the leader CTA (cluster rank 0) issues
// tcgen05.mma.cta_group::2 for both, the hardware reading each CTA's A half from that CTA's shared memory and sharing the two
// B halves between the pair. A 128 x 128 tile per SM (the one-CTA kernel in gemm_tcgen05.cu) needs 256 bytes of shared-memory
// traffic per clock at full tensor rate - operand reads plus the TMA fill of the next stage - against the 128 an SM has; the
// pair needs half of that per SM for the same math, which is what lifts the ceiling of the one-CTA kernel.
//
// Protocol per reduction step s (ring of kStages, the barriers live at the same shared-memory offsets in both CTAs):
//   * both producers (warp 0) wait for their own empty[s]; the leader arms ITS full[s] with the bytes of both CTAs;
//     both issue their loads with the leader's full[s] as the completion barrier (no load is multicast);
//   * the leader's MMA thread (warp 1) waits for full[s], issues four 256 x 256 x 16 MMAs and commits them to empty[s] of
//     both CTAs (tcgen05.commit with a two-CTA mask), and after the last step to accumulator_full of both CTAs;
//   * the epilogue warps (2..9) of each CTA drain their own accumulator, two warps per lane quarter with 128 columns each:
//     tcgen05.ld, bias / residual / ReLU, conversion, staging in the by then idle operand stages in the 128-byte-swizzled box
//     layout, TMA stores (add-reductions for a split reduction) of 32-row slabs.
// Operands may be K-major or MN-major as in the one-CTA kernel. Every wait is bounded: on a timeout the CTA records
// kStatusWaitTimeout, gives outstanding copies time to land, joins the cluster barrier, frees its tensor memory and returns.
//
// The reference has no GEMM kernel of its own: its dense layers are nn.Linear (cuBLAS), examples/deepfm/deepfm_model.py:49-52.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "../common/rb_tcgen05.cuh"
#include "rb_dense.h"
#include "rb_gemm_store.cuh"
#include <cuda.h>
#include <cuda_bf16.h>
#include <algorithm>
#include <cstdlib>

namespace {

using namespace rb::tc;
using rb::gemm::Store;

constexpr int TM = 128;        // rows of D per CTA (the pair covers 256)
constexpr int TN = 256;        // columns of D per pair; each CTA stages 128 rows of B
constexpr int BK = 64;
constexpr int UK = 16;
constexpr int kStages = 3;     // 3 x 32 KB per CTA: two CTAs (of different pairs) share an SM
constexpr int kThreads = 320;     // producer warp, MMA warp, 8 epilogue warps (two per tensor-memory lane quarter)
constexpr uint32_t kHalfBytes = 128 * BK * 2;                   // 16 KB: one operand half of one stage
constexpr uint32_t kStageBytes = 2 * kHalfBytes;                // this CTA's A half + B half
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;                     // clears the CTA-rank bit of a shared::cluster address: rank 0's copy

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load into this CTA's shared memory that reports its bytes to the barrier at `bar_cluster_addr` (the leader's full barrier)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// completion of all MMAs issued so far arrives once on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 2)
gemm_bf16_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              const __grid_constant__ CUtensorMap map_o, const float* __restrict__ bias,
                              const float* __restrict__ beta_src, const RbGemmEpilogue epi, int MM, int NN, int KK, int ldo, int relu,
                              int64_t* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float bias_s[TN];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                        // 0 = leader
  const int m0 = (int)(blockIdx.x >> 1) * 2 * TM + (int)rank * TM;      // this CTA's rows of D (and of A)
  const int n0 = (int)blockIdx.y * TN;                                   // the pair's columns of D
  const int nb0 = n0 + (int)rank * 128;                                  // this CTA's rows of B
  const int total_kb = (KK + BK - 1) / BK;
  const int kb_per = (total_kb + (int)gridDim.z - 1) / (int)gridDim.z;
  const int kb_begin = (int)blockIdx.z * kb_per;
  const int num_kb = max(0, min(total_kb, kb_begin + kb_per) - kb_begin);
  const bool split = gridDim.z > 1;
  if (split && num_kb == 0) return;          // uniform for the whole cluster (same blockIdx.z), before any barrier or allocation

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&tmem_full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)TN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  } else if (warp >= 2) {
    const int c = (int)threadIdx.x - 64;                 // 256 epilogue threads, one column of the tile's bias each
    bias_s[c] = (bias != nullptr && n0 + c < NN && (!split || blockIdx.z == 0)) ? bias[n0 + c] : 0.f;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  __syncwarp();
  cluster_sync();                            // the peer's barriers exist before anything of ours signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % kStages;
      const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
      ok = mbar_wait(&empty_bar[s], ph ^ 1u, &abort_flag);
      if (!ok) break;
      uint8_t* sa = smem + s * kStageBytes;
      uint8_t* sb = sa + kHalfBytes;
      if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);        // both CTAs' loads complete on the leader's barrier
      const uint32_t bar = smem_u32(&full_bar[s]) & kPeerMask;
      const int k0 = (kb_begin + kb) * BK;
      if (!A_MN) tma_load_2d_pair(sa, &map_a, k0, m0, bar);                                   // box {BK, 128}
      else { tma_load_2d_pair(sa, &map_a, m0, k0, bar); tma_load_2d_pair(sa + kHalfBytes / 2, &map_a, m0 + 64, k0, bar); }   // 2 x box {64, BK}
      if (!B_MN) tma_load_2d_pair(sb, &map_b, k0, nb0, bar);
      else { tma_load_2d_pair(sb, &map_b, nb0, k0, bar); tma_load_2d_pair(sb + kHalfBytes / 2, &map_b, nb0 + 64, k0, bar); }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    // instruction descriptor: D = f32, A = B = bf16, majors, N >> 3, M >> 4 with M = 256 (both CTAs' rows)
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                           ((uint32_t)(TN >> 3) << 17) | ((uint32_t)((2 * TM) >> 4) << 24);
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % kStages;
      const uint32_t ph = (uint32_t)(kb / kStages) & 1u;
      ok = mbar_wait(&full_bar[s], ph, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sa = smem_u32(smem + s * kStageBytes), sb = sa + kHalfBytes;
#pragma unroll
      for (int k = 0; k < BK / UK; ++k) {
        const uint64_t da = A_MN ? make_desc(sa + k * 2048, BK * 128, 1024) : make_desc(sa + k * 32, 16, 1024);
        const uint64_t db = B_MN ? make_desc(sb + k * 2048, BK * 128, 1024) : make_desc(sb + k * 32, 16, 1024);
        umma_bf16_pair(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit_pair(&empty_bar[s]);
    }
    if (ok) umma_commit_pair(&tmem_full_bar);
  } else if (warp >= 2) {
    // ------------------------------------------------------------------ epilogue (8 warps: lane quarter warp & 3, column half (warp - 2) / 4)
    const bool ok = num_kb > 0 ? mbar_wait(&tmem_full_bar, 0, &abort_flag) : true;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const int q = warp & 3, half = (warp - 2) >> 2;
      const int row = m0 + q * 32 + lane;
      const bool add_beta = beta_src != nullptr && (!split || blockIdx.z == 0);
      // every MMA of the pair has completed, so neither CTA's operand stages are read any more: they become the staging area.
      // A warp stages kPass columns at a time into its own 8 KB slab: boxes of 32 rows x 128 bytes.
      constexpr int kPass = 256 / (int)sizeof(OutT);                   // 128 columns of bf16, 64 of fp32: 8 KB per 32 rows
      constexpr int kBoxes = kPass / Store<OutT>::kBoxCols;            // 2
      uint8_t* slab = smem + (half * 4 + q) * 8192;
#pragma unroll 1
      for (int p0 = half * 128; p0 < half * 128 + 128; p0 += kPass) {
        if (n0 + p0 >= NN) break;
        if (p0 > half * 128) {
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous pass's boxes have been read
          __syncwarp();
        }
#pragma unroll 1
        for (int c0 = p0; c0 < p0 + kPass; c0 += 32) {
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
          Store<OutT>::stage32(slab, lane, c0 - p0, v);
          if (epi.colsum != nullptr) {
            if (row >= MM) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
            rb::gemm::column_sums32(v, lane, valid, epi.colsum + n0 + c0);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && m0 + q * 32 < MM) {
#pragma unroll
          for (int bx = 0; bx < kBoxes; ++bx) {
            const int col = n0 + p0 + bx * Store<OutT>::kBoxCols;
            if (col >= NN) break;
            if (split)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(slab + bx * 4096)), "r"(col), "r"(m0 + q * 32) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"(&map_o), "r"(smem_u32(slab + bx * 4096)), "r"(col), "r"(m0 + q * 32) : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");       // the slab must stay until the copies have read it
    }
  }
  if (abort_flag) {
    // a wait ran out: copies of this pair may still be on their way into shared memory; give them time before it goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  __syncwarp();
  cluster_sync();                            // both epilogues are done and nothing of the peer's is in flight towards this CTA
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TN) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag) rb::set_status(status, rb::kStatusWaitTimeout);
}

template <bool A_MN, bool B_MN, typename OutT>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const float* bias, const float* beta_src,
                const RbGemmEpilogue& epi, int MM, int NN, int KK, int ldo, int relu, int splits, int64_t* status, cudaStream_t st) {
  auto kern = gemm_bf16_tcgen05_2cta_kernel<A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess) return 3;
    attr_set = true;
  }
  dim3 grid(2 * ((MM + 2 * TM - 1) / (2 * TM)), (NN + TN - 1) / TN, splits);
  kern<<<grid, kThreads, kSmemBytes, st>>>(ma, mb, mo, bias, beta_src, epi, MM, NN, KK, ldo, relu, status);
  rb::note_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}

}  // namespace

// Same contract as rb_gemm_bf16 (rb_dense.h), for outputs that can leave through TMA stores (base and row pitch 16-byte aligned).
// Returns 7 when the problem does not suit the pair kernel (the caller then uses the one-CTA kernel).
extern "C" int rb_gemm_bf16_pair(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo,
                                 int out_fp32, const float* bias, const float* beta_src, const RbGemmEpilogue* epi_in, int MM, int NN, int KK,
                                 int relu, int splits, int64_t* status, cudaStream_t st) {
  RbGemmEpilogue epi{nullptr, 0, nullptr};
  if (epi_in != nullptr) epi = *epi_in;
  if ((epi.mask_src != nullptr || epi.colsum != nullptr) && splits > 1) return 6;
  if (MM < 192 || NN < 192 || KK <= 0) return 7;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (lda % 8) || (ldb % 8)) return 1;
  const int es = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (ldo * es) % 16) return 7;
  if (splits > 1 && (!out_fp32 || relu)) return 6;
  CUtensorMap ma, mb, mo;
  // boxes: K-major operands {BK, 128 rows}; MN-major operands {64, BK}; output {32 or 64 columns, 32 rows}
  const int ra = a_mn ? rb_tensor_map_2d(&ma, a, KK, MM, lda, 64, BK, 0) : rb_tensor_map_2d(&ma, a, MM, KK, lda, BK, 128, 0);
  const int rbm = b_mn ? rb_tensor_map_2d(&mb, b, KK, NN, ldb, 64, BK, 0) : rb_tensor_map_2d(&mb, b, NN, KK, ldb, BK, 128, 0);
  const int ro = rb_tensor_map_2d(&mo, out, MM, NN, ldo, out_fp32 ? 32 : 64, 32, out_fp32);
  if (ra || rbm || ro) return 2;
#define RB_PAIR_CASE(AM, BMJ)                                                                                                    \
  if ((a_mn != 0) == AM && (b_mn != 0) == BMJ)                                                                                   \
    return out_fp32 ? launch_pair<AM, BMJ, float>(ma, mb, mo, bias, beta_src, epi, MM, NN, KK, (int)ldo, relu, splits, status, st)    \
                    : launch_pair<AM, BMJ, __nv_bfloat16>(ma, mb, mo, bias, beta_src, epi, MM, NN, KK, (int)ldo, relu, 1, status, st);
  RB_PAIR_CASE(false, false)
  RB_PAIR_CASE(false, true)
  RB_PAIR_CASE(true, false)
  RB_PAIR_CASE(true, true)
#undef RB_PAIR_CASE
  return 5;
}
