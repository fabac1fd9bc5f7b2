// Sparse-path kernels (sm_100a): id dedup + owner bucketing, multi-tensor id encode / offset merge,
// row gather / scatter, ragged pooling (sum / mean / tile), and the chunked segmented gradient
// reduction that can apply the row-wise optimizer in the same pass.
//
// Reference behaviour covered (by path inside the reference project):
//   csrc/ops/ids_partition_kernel.cu:23-165        dedup + shard routing (there: rotate + radix sort + unique)
//   csrc/ops/ids_encode_kernel.cu:16-59             12-bit table prefix
//   csrc/ops/embedding_segment_reduce_kernel.cu     merge_offsets :352-392, pooling fwd/bwd :21-350
//   csrc/ops/segment_ops_kernel.cu:10-290           "sparse mode" pooling with weight normalisation
//   csrc/ops/ragged_tile_kernel.cu:25-280           tile combiner
//   csrc/ops/block_ops_kernel.cu:15-392             gather / insert
// The structure is different: dedup is a scratch hash set (no 64-bit sort, no host read of the
// unique count), pooling reads the row arena directly, and the backward pass is a segmented reduction
// over a (unique, element) sorted list that updates each touched row exactly once, so there is no
// per-element atomic traffic and no intermediate gradient tensor on the single-GPU path.
#include "../common/rb_common.cuh"
#include "rb_kernels.h"
#include "../common/rb_opt.cuh"
#include "rb_comm.h"
#include "../common/rb_launch.h"
#include <cub/device/device_radix_sort.cuh>
#include <cooperative_groups.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "rb_noalloc.h"

namespace cg = cooperative_groups;

using namespace rb;

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 32;  // CSR positions per work item of the gradient reduction

inline int grid_stride_blocks(int64_t work_items, int threads = kThreads) {
  int64_t b = (work_items + threads - 1) / threads;
  if (b < 1) b = 1;
  const int64_t cap = 148 * 16;
  return (int)(b < cap ? b : cap);
}

// ------------------------------------------------------------------ dedup + owner bucketing
__global__ void __launch_bounds__(kThreads)
dedup_claim_kernel(const int64_t* __restrict__ ids, int64_t n, int world, uint64_t* __restrict__ set_keys,
                   int32_t* __restrict__ set_pos, uint64_t mask, int32_t* __restrict__ slot_out, int32_t* __restrict__ counts) {
  extern __shared__ int32_t sm[];  // [world] block histogram, [world] block base
  int32_t* hist = sm; int32_t* base = sm + world;
  for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x; i0 < n; i0 += (int64_t)gridDim.x * blockDim.x) {
    for (int w = threadIdx.x; w < world; w += blockDim.x) hist[w] = 0;
    __syncthreads();
    const int64_t i = i0 + threadIdx.x;
    int32_t slot = -1, local = 0, owner = 0; bool won = false;
    if (i < n) {
      const uint64_t key = (uint64_t)ids[i];
      uint64_t h = mix64(key) & mask;
      for (uint64_t probe = 0; probe <= mask; ++probe, h = (h + 1) & mask) {
        uint64_t k = *reinterpret_cast<volatile uint64_t*>(&set_keys[h]);
        if (k == kEmptyKey && key != kEmptyKey) {
          k = atomicCAS(reinterpret_cast<unsigned long long*>(&set_keys[h]), (unsigned long long)kEmptyKey, (unsigned long long)key);
          if (k == kEmptyKey) { won = true; k = key; }
        }
        if (k == key) { slot = (int32_t)h; break; }
      }
      if (key == kEmptyKey) {  // the sentinel itself cannot live in the set: treat every occurrence as the same id in slot 0's shadow
        slot = (int32_t)(mask + 1);                    // one spare cell past the end
        won = atomicCAS(&set_pos[mask + 1], -1, -2) == -1;
      }
      if (won) { owner = owner_of(key, world); local = atomicAdd(&hist[owner], 1); }
    }
    __syncthreads();
    for (int w = threadIdx.x; w < world; w += blockDim.x) base[w] = hist[w] ? atomicAdd(&counts[w], hist[w]) : 0;
    __syncthreads();
    if (i < n) {
      if (won) set_pos[slot] = base[owner] + local;
      slot_out[i] = slot | (won ? (int32_t)0x80000000 : 0);
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kThreads)
dedup_assign_kernel(const int64_t* __restrict__ ids, int64_t n, int world, const int32_t* __restrict__ set_pos,
                    const int32_t* __restrict__ slot_in, const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                    int64_t* __restrict__ unique_ids, int32_t* __restrict__ reverse, int64_t unique_cap, int64_t* status) {
  extern __shared__ int32_t off[];  // [world+1]
  if (threadIdx.x == 0) {
    int32_t run = 0;
    for (int w = 0; w < world; ++w) { off[w] = run; run += counts[w]; }
    off[world] = run;
    // more unique ids than the output buffer holds: flag it; positions beyond the buffer are dropped below (memory safe)
    if (run > unique_cap && blockIdx.x == 0 && status) set_status(status, kStatusWindowOverflow);
  }
  __syncthreads();
  // published boundaries are clamped to the buffer, so that nobody downstream reads or writes past it after an overflow
  if (blockIdx.x == 0)
    for (int w = threadIdx.x; w <= world; w += blockDim.x) offsets[w] = (int32_t)min((int64_t)off[w], unique_cap);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t s = slot_in[i];
    const uint64_t key = (uint64_t)ids[i];
    const int32_t u = off[owner_of(key, world)] + set_pos[s & 0x7FFFFFFF];
    reverse[i] = u < unique_cap ? u : 0;
    if (s < 0 && u < unique_cap) unique_ids[u] = (int64_t)key;
  }
}

// ------------------------------------------------------------------ multi-tensor encode + offset merge
__device__ __forceinline__ int find_tensor(const int64_t* prefix, int F, int64_t i) {
  int lo = 0, hi = F;  // prefix[lo] <= i < prefix[hi]
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (prefix[mid] <= i) lo = mid; else hi = mid; }
  return lo;
}

__global__ void __launch_bounds__(kThreads)
encode_merge_kernel(const int64_t* __restrict__ desc, const int64_t* __restrict__ table_idx, int F, int64_t total_nnz,
                    int64_t total_seg, int64_t* __restrict__ ids_out, int32_t* __restrict__ offsets_out) {
  const int64_t* id_ptr = desc; const int64_t* nnz_prefix = desc + (F + 1);
  const int64_t* off_ptr = desc + 2 * (F + 1); const int64_t* seg_prefix = desc + 3 * (F + 1);
  const int64_t total = total_nnz + total_seg + 1;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    if (w < total_nnz) {
      const int f = find_tensor(nnz_prefix, F, w);
      const int64_t v = reinterpret_cast<const int64_t*>(id_ptr[f])[w - nnz_prefix[f]];
      ids_out[w] = (int64_t)(((uint64_t)v & 0x000FFFFFFFFFFFFFull) | ((uint64_t)table_idx[f] << 52));
    } else if (offsets_out) {
      const int64_t j = w - total_nnz;
      if (j == total_seg) { offsets_out[j] = (int32_t)total_nnz; continue; }
      const int f = find_tensor(seg_prefix, F, j);
      offsets_out[j] = reinterpret_cast<const int32_t*>(off_ptr[f])[j - seg_prefix[f]] + (int32_t)nnz_prefix[f];
    }
  }
}

// ------------------------------------------------------------------ row gather / scatter
// Rows are copied as bytes, V bytes per thread and access (V = the largest of 16, 8, 4, 2, 1 that divides the row size), so
// that one pair of kernels serves rows of every element type.
template <typename V>
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const V* __restrict__ src, const int32_t* __restrict__ rows, int64_t n_max, const int32_t* __restrict__ n_dev,
                   int q, V* __restrict__ out) {
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  const int64_t total = n * q;
  V zero; memset(&zero, 0, sizeof(V));
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = w / q; const int c = (int)(w - r * q);
    const int32_t row = rows[r];
    out[r * q + c] = row >= 0 ? src[(int64_t)row * q + c] : zero;
  }
}

template <typename V>
__global__ void __launch_bounds__(kThreads)
scatter_rows_kernel(V* __restrict__ dst, const int32_t* __restrict__ rows, int64_t n, int q, const V* __restrict__ src,
                    int src_broadcast) {
  const int64_t total = n * q;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = w / q; const int c = (int)(w - r * q);
    const int32_t row = rows[r];
    if (row >= 0) dst[(int64_t)row * q + c] = src_broadcast ? src[c] : src[w];
  }
}

// f(V{}, q) with V the widest vector type that divides row_bytes and keeps both base pointers aligned
template <typename F>
inline void dispatch_row_bytes(int64_t row_bytes, const void* a, const void* b, F&& f) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | (uintptr_t)row_bytes;
  if ((al & 15) == 0) f(uint4{}, (int)(row_bytes / 16));
  else if ((al & 7) == 0) f(uint2{}, (int)(row_bytes / 8));
  else if ((al & 3) == 0) f(uint32_t{}, (int)(row_bytes / 4));
  else if ((al & 1) == 0) f(uint16_t{}, (int)(row_bytes / 2));
  else f(uint8_t{}, (int)row_bytes);
}

__global__ void __launch_bounds__(kThreads)
fill_rows_i64_kernel(int64_t* __restrict__ dst, const int32_t* __restrict__ rows, int64_t n, int64_t value) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    if (rows[i] >= 0) dst[rows[i]] = value;
}

// ------------------------------------------------------------------ pooling forward
// perm_f > 0: segment s = f * perm_b + b goes to row b * perm_total + perm_off + f of the output (perm_total features per
// sample in the output, this call fills features perm_off .. perm_off + perm_f - 1)
// perm_f <= 0: plain layout, segment s goes to row perm_off + s.
__device__ __forceinline__ int64_t out_row_of(int64_t s, int perm_b, int perm_f, int perm_off, int perm_total) {
  if (perm_f <= 0) return s + perm_off;
  const int64_t f = s / perm_b, b = s - f * perm_b;
  return b * perm_total + perm_off + f;
}

// One group of G lanes per segment; each lane owns NACC float4 column slots (columns lane + a*G).
template <int G, int NACC, typename T>
__global__ void __launch_bounds__(kThreads)
pool_forward_kernel(const T* __restrict__ base, const int32_t* __restrict__ rows, const int32_t* __restrict__ rev,
                    const int32_t* __restrict__ offsets, const float* __restrict__ weights, int64_t n_seg, int D, int mode,
                    int perm_b, int perm_f, int perm_off, int perm_total, float* __restrict__ out, int32_t* __restrict__ gsrc,
                    float* __restrict__ gscale) {
  const int lane = threadIdx.x % G;
  const int cols = D >> 2;
  const int64_t n_groups = (int64_t)gridDim.x * (kThreads / G);
  for (int64_t s = blockIdx.x * (int64_t)(kThreads / G) + threadIdx.x / G; s < n_seg; s += n_groups) {
    const int32_t beg = offsets[s], end = offsets[s + 1];
    float4 acc[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int32_t i = beg; i < end; i += 4) {
      int32_t r[4]; float w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r[j] = -1; w[j] = 0.f;
        if (i + j < end) {
          const int32_t u = rev[i + j];
          r[j] = rows ? rows[u] : u;
          w[j] = weights ? weights[i + j] : 1.f;
          wsum += w[j];
        }
      }
      float4 v[4][NACC];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          const int c = lane + a * G;
          v[j][a] = (r[j] >= 0 && c < cols) ? RowIO<T>::ld4(base + (int64_t)r[j] * D + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int a = 0; a < NACC; ++a) acc[a] = f4_fma(w[j], v[j][a], acc[a]);
    }
    float scale = 1.f;
    if (mode == 1) scale = end > beg ? 1.f / (float)(end - beg) : 0.f;
    else if (mode == 2) scale = wsum != 0.f ? 1.f / wsum : 0.f;
    const int64_t orow = out_row_of(s, perm_b, perm_f, perm_off, perm_total);
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int c = lane + a * G;
      if (c < cols) st_f4(out + orow * D + c * 4, make_float4(acc[a].x * scale, acc[a].y * scale, acc[a].z * scale, acc[a].w * scale));
    }
    if (gsrc) {
      for (int32_t i = beg + lane; i < end; i += G) {
        gsrc[i] = (int32_t)orow;
        gscale[i] = (weights ? weights[i] : 1.f) * scale;
      }
    }
  }
}

// Any D (not a multiple of 4, or wider than 512): one thread per (segment, column).
template <typename T>
__global__ void __launch_bounds__(kThreads)
pool_forward_scalar_kernel(const T* __restrict__ base, const int32_t* __restrict__ rows, const int32_t* __restrict__ rev,
                           const int32_t* __restrict__ offsets, const float* __restrict__ weights, int64_t n_seg, int D, int mode,
                           int perm_b, int perm_f, int perm_off, int perm_total, float* __restrict__ out, int32_t* __restrict__ gsrc,
                           float* __restrict__ gscale) {
  const int64_t total = n_seg * D;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = w / D; const int c = (int)(w - s * D);
    const int32_t beg = offsets[s], end = offsets[s + 1];
    float acc = 0.f, wsum = 0.f;
    for (int32_t i = beg; i < end; ++i) {
      const int32_t u = rev[i]; const int32_t r = rows ? rows[u] : u;
      const float wt = weights ? weights[i] : 1.f;
      wsum += wt;
      if (r >= 0) acc = fmaf(wt, RowIO<T>::ld1(base + (int64_t)r * D + c), acc);
    }
    float scale = 1.f;
    if (mode == 1) scale = end > beg ? 1.f / (float)(end - beg) : 0.f;
    else if (mode == 2) scale = wsum != 0.f ? 1.f / wsum : 0.f;
    const int64_t orow = out_row_of(s, perm_b, perm_f, perm_off, perm_total);
    out[orow * D + c] = acc * scale;
    if (gsrc && c == 0)
      for (int32_t i = beg; i < end; ++i) { gsrc[i] = (int32_t)orow; gscale[i] = (weights ? weights[i] : 1.f) * scale; }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
tile_forward_kernel(const T* __restrict__ base, const int32_t* __restrict__ rows, const int32_t* __restrict__ rev,
                    const int32_t* __restrict__ offsets, const float* __restrict__ weights, int64_t n_seg, int D, int tile_len,
                    float* __restrict__ out, int32_t* __restrict__ gsrc, float* __restrict__ gscale) {
  const int64_t total = n_seg * tile_len * (int64_t)D;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t st = w / D; const int c = (int)(w - st * D);
    const int64_t s = st / tile_len; const int t = (int)(st - s * tile_len);
    const int32_t beg = offsets[s], end = offsets[s + 1];
    float v = 0.f;
    if (beg + t < end) {
      const int32_t u = rev[beg + t]; const int32_t r = rows ? rows[u] : u;
      const float wt = weights ? weights[beg + t] : 1.f;
      if (r >= 0) v = wt * RowIO<T>::ld1(base + (int64_t)r * D + c);
      if (gsrc && c == 0) { gsrc[beg + t] = (int32_t)st; gscale[beg + t] = wt; }
    }
    out[w] = v;
    // elements beyond tile_len contribute nothing: mark them once (by the thread of the last tile slot)
    if (gsrc && c == 0 && t == tile_len - 1)
      for (int32_t i = beg + tile_len; i < end; ++i) { gsrc[i] = -1; gscale[i] = 0.f; }
  }
}

// ------------------------------------------------------------------ backward structure
__global__ void __launch_bounds__(kThreads) iota_kernel(int32_t* out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) out[i] = (int32_t)i;
}

__global__ void __launch_bounds__(kThreads) csr_heads_kernel(const int32_t* __restrict__ csr_u, int64_t n, int32_t* __restrict__ start) {
  for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
    const int32_t u = csr_u[p];
    if (p == 0 || csr_u[p - 1] != u) start[u] = (int32_t)p;
    if (p == n - 1) start[u + 1] = (int32_t)n;
  }
}

// ------------------------------------------------------------------ chunked segmented gradient reduction
// VEC = 4: float4 columns, G lanes x NACC slots per group. Work item = kChunk consecutive CSR positions.
// Shared-memory copy of a push descriptor: row_ptr(u) is where the gradient of unique index u is stored (nullptr = dropped).
struct PushTable {
  int32_t off[17];
  int32_t dst[16];
  float* base[16];
  __device__ __forceinline__ void load(const RbGuPush& p) {
    if (threadIdx.x <= p.world) off[threadIdx.x] = p.off[threadIdx.x];
    if (threadIdx.x < p.world) { dst[threadIdx.x] = p.dst_base[threadIdx.x]; base[threadIdx.x] = static_cast<float*>(p.base[threadIdx.x]); }
    __syncthreads();
  }
  __device__ __forceinline__ float* row_ptr(int32_t u, int world, int64_t cap_rows, int D) const {
    int o = 0;
    while (o + 1 < world && off[o + 1] <= u) ++o;
    const int64_t r = (int64_t)dst[o] + (u - off[o]);
    return r < cap_rows ? base[o] + r * D : nullptr;
  }
};

template <int G, int NACC, bool PUSH, typename T>
__global__ void __launch_bounds__(kThreads)
grad_reduce_kernel(const float* __restrict__ grad_out, const int32_t* __restrict__ gsrc, const float* __restrict__ gscale,
                   const int32_t* __restrict__ csr_u, const int32_t* __restrict__ csr_elem, const int32_t* __restrict__ start,
                   int64_t n, int D, float* __restrict__ span_acc, const int32_t* __restrict__ rows, float* __restrict__ gu,
                   int apply, RbOpt opt, RbGuPush push) {
  __shared__ PushTable ptab;
  if (PUSH) ptab.load(push);
  // Phase 1 (per chunk): the lanes of the group fetch the metadata of all positions of the chunk in parallel (one
  // dependent chain for the whole chunk instead of one per position) and park it in shared memory.
  // Phase 2: walk the segments of the chunk; the optimizer state of a row is requested when its segment starts, so
  // those loads are in flight together with the gradient gathers of the segment.
  __shared__ int32_t meta[(kThreads / G) * kChunk * 5];
  auto tile = cg::tiled_partition<G>(cg::this_thread_block());
  const int lane = threadIdx.x % G;
  const int gid = threadIdx.x / G;
  int32_t* m_u = meta + gid * kChunk * 5;
  int32_t* m_gs = m_u + kChunk;
  int32_t* m_row = m_u + 2 * kChunk;      // >= 0 row to update / unique index to store, -1 skip, -2 segment crosses the chunk
  int32_t* m_dst = m_u + 3 * kChunk;      // chunk that owns a crossing segment
  float* m_sc = reinterpret_cast<float*>(m_u + 4 * kChunk);
  const int cols = D >> 2;
  const int64_t n_chunks = (n + kChunk - 1) / kChunk;
  const int64_t n_groups = (int64_t)gridDim.x * (kThreads / G);
  // The sorted positions are bucketed by owner rank, so chunks in their natural order would make every rank write to owner 0
  // first, then to owner 1, ...: all ranks' stores would converge on one GPU's links at a time (measured on 4 GPUs: 0.38 TB/s
  // per rank against 0.60 for the row push, which serves all peers at once). When pushing, the chunks are therefore visited in
  // a transposed order - virtual index v = (column, lane) of a [kSpread x ceil(n_chunks / kSpread)] grid read lane-first - so the
  // chunks in flight at any moment are spread over the whole sequence and every owner receives from every rank all the time.
  constexpr int64_t kSpread = 64;
  const int64_t spread_cols = (n_chunks + kSpread - 1) / kSpread;
  const int64_t n_virtual = PUSH ? spread_cols * kSpread : n_chunks;
  for (int64_t v = blockIdx.x * (int64_t)(kThreads / G) + gid; v < n_virtual; v += n_groups) {
    const int64_t c = PUSH ? (v % kSpread) * spread_cols + v / kSpread : v;
    if (c >= n_chunks) continue;              // uniform for the group (c depends on v and the group id only)
    const int64_t p0 = c * kChunk, p1 = min(p0 + (int64_t)kChunk, n);
    const int cnt = (int)(p1 - p0);
    for (int j = lane; j < cnt; j += G) {
      const int32_t u = csr_u[p0 + j];
      const int32_t e = csr_elem[p0 + j];
      const int32_t s0 = start[u], s1 = start[u + 1];
      const bool complete = s0 >= p0 && s1 <= p1;
      m_u[j] = u;
      m_gs[j] = gsrc[e];
      m_sc[j] = gscale[e];
      m_row[j] = complete ? (apply ? (rows ? rows[u] : u) : u) : -2;
      m_dst[j] = s0 / kChunk;
    }
    tile.sync();
    int j = 0;
    while (j < cnt) {
      const int32_t u = m_u[j];
      const int32_t row = m_row[j];
      int jend = j + 1;
      while (jend < cnt && m_u[jend] == u) ++jend;
      float4 sw[NACC], s1v[NACC], s2v[NACC];
      const bool upd = apply && row >= 0;
      if (upd) {
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          const int col = lane + a * G;
          if (col < cols) {
            const int64_t off = (int64_t)row * D + col * 4;
            sw[a] = RowIO<T>::ld4(static_cast<const T*>(opt.w) + off);
            if (opt.kind != RB_OPT_SGD) s1v[a] = ld_f4(opt.s1 + off);
            if (opt.kind == RB_OPT_ADAM) s2v[a] = ld_f4(opt.s2 + off);
          }
        }
      }
      float4 acc[NACC];
#pragma unroll
      for (int a = 0; a < NACC; ++a) acc[a] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = j; k < jend; k += 4) {
        float4 v[4][NACC];
        float sc[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int32_t gs = (k + t < jend) ? m_gs[k + t] : -1;
          sc[t] = (k + t < jend) ? m_sc[k + t] : 0.f;
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            const int col = lane + a * G;
            v[t][a] = (gs >= 0 && col < cols) ? ld_f4(grad_out + (int64_t)gs * D + col * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
          for (int a = 0; a < NACC; ++a) acc[a] = f4_fma(sc[t], v[t][a], acc[a]);
      }
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        const int col = lane + a * G;
        if (col >= cols) continue;
        if (row == -2) red_add_f4(span_acc + (int64_t)m_dst[j] * D + col * 4, acc[a]);
        else if (upd) opt_update_pre_f4<T>(opt, (int64_t)row * D + col * 4, acc[a], sw[a], s1v[a], s2v[a]);
        else if (!apply) {
          if (PUSH) {
            float* dstp = ptab.row_ptr(row, push.world, push.cap_rows, D);
            if (dstp) st_f4(dstp + col * 4, acc[a]);
          } else {
            st_f4(gu + (int64_t)row * D + col * 4, acc[a]);
          }
        }
      }
      j = jend;
    }
    tile.sync();
  }
}

// Rows whose occurrences cross a chunk boundary were accumulated in span_acc[chunk of their first
// occurrence]; finish them here and leave span_acc zeroed for the next step.
template <int G, int NACC, bool PUSH, typename T>
__global__ void __launch_bounds__(kThreads)
grad_span_finish_kernel(const int32_t* __restrict__ csr_u, const int32_t* __restrict__ start, int64_t n, int D,
                        float* __restrict__ span_acc, const int32_t* __restrict__ rows, float* __restrict__ gu, int apply, RbOpt opt,
                        RbGuPush push) {
  __shared__ PushTable ptab;
  if (PUSH) ptab.load(push);
  const int lane = threadIdx.x % G;
  const int cols = D >> 2;
  const int64_t n_chunks = (n + kChunk - 1) / kChunk;
  const int64_t n_groups = (int64_t)gridDim.x * (kThreads / G);
  for (int64_t c = blockIdx.x * (int64_t)(kThreads / G) + threadIdx.x / G; c < n_chunks; c += n_groups) {
    const int64_t p0 = c * kChunk, p1 = min(p0 + (int64_t)kChunk, n);
    const int32_t u = csr_u[p1 - 1];
    const int32_t s0 = start[u], s1 = start[u + 1];
    if (!(s0 >= p0 && s1 > p1)) continue;
    const int32_t row = rows ? rows[u] : u;
    float* src = span_acc + c * D;
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      const int col = lane + a * G;
      if (col < cols) {
        const float4 g = ld_f4(src + col * 4);
        st_f4(src + col * 4, make_float4(0.f, 0.f, 0.f, 0.f));
        if (apply) { if (row >= 0) opt_update_f4<T>(opt, (int64_t)row * D + col * 4, g); }
        else if (PUSH) {
          float* dstp = ptab.row_ptr(u, push.world, push.cap_rows, D);
          if (dstp) st_f4(dstp + col * 4, g);
        } else st_f4(gu + (int64_t)u * D + col * 4, g);
      }
    }
  }
}

// Scalar variant for D not a multiple of 4: one thread per (unique row, column) walking its CSR range.
template <typename T>
__global__ void __launch_bounds__(kThreads)
grad_reduce_scalar_kernel(const float* __restrict__ grad_out, const int32_t* __restrict__ gsrc, const float* __restrict__ gscale,
                          const int32_t* __restrict__ csr_u, const int32_t* __restrict__ csr_elem, const int32_t* __restrict__ start,
                          int64_t n, int D, const int32_t* __restrict__ rows, float* __restrict__ gu, int apply, RbOpt opt) {
  const int32_t n_unique = csr_u[n - 1] + 1;
  const int64_t total = (int64_t)n_unique * D;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int32_t u = (int32_t)(w / D); const int c = (int)(w - (int64_t)u * D);
    float acc = 0.f;
    for (int32_t p = start[u]; p < start[u + 1]; ++p) {
      const int32_t e = csr_elem[p]; const int32_t gs = gsrc[e];
      if (gs >= 0) acc = fmaf(gscale[e], grad_out[(int64_t)gs * D + c], acc);
    }
    if (apply) { const int32_t row = rows ? rows[u] : u; if (row >= 0) opt_update_f1<T>(opt, (int64_t)row * D + c, acc); }
    else gu[w] = acc;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sparse_apply_kernel(const int32_t* __restrict__ rows, const float* __restrict__ grads, int64_t n_max, const int32_t* __restrict__ n_dev,
                    int D, RbOpt opt) {
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  if ((D & 3) == 0) {
    const int q = D >> 2; const int64_t total = n * q;
    for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
      const int64_t r = w / q; const int c = (int)(w - r * q);
      const int32_t row = rows[r];
      if (row >= 0) opt_update_f4<T>(opt, (int64_t)row * D + c * 4, ld_f4(grads + r * D + c * 4));
    }
  } else {
    const int64_t total = n * D;
    for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
      const int64_t r = w / D; const int c = (int)(w - r * D);
      const int32_t row = rows[r];
      if (row >= 0) opt_update_f1<T>(opt, (int64_t)row * D + c, grads[w]);
    }
  }
}

template <typename F>
inline bool dispatch_cols(int D, F&& f) {
  if ((D & 3) != 0 || D > 512) return false;
  const int cols = D >> 2;
  // narrow rows share the 4-lane variant (lanes beyond the row width idle): keeps per-group shared-memory staging small
  if (cols <= 4) f(std::integral_constant<int, 4>{}, std::integral_constant<int, 1>{});
  else if (cols <= 8) f(std::integral_constant<int, 8>{}, std::integral_constant<int, 1>{});
  else if (cols <= 16) f(std::integral_constant<int, 16>{}, std::integral_constant<int, 1>{});
  else if (cols <= 32) f(std::integral_constant<int, 32>{}, std::integral_constant<int, 1>{});
  else if (cols <= 64) f(std::integral_constant<int, 32>{}, std::integral_constant<int, 2>{});
  else f(std::integral_constant<int, 32>{}, std::integral_constant<int, 4>{});
  return true;
}

}  // namespace

extern "C" {

void rb_dedup_partition(const int64_t* ids, int64_t n, int world, uint64_t* set_keys, int32_t* set_pos, int64_t set_cap,
                        int32_t* slot_scratch, int32_t* counts, int32_t* offsets, int64_t* unique_ids, int32_t* reverse,
                        int64_t unique_cap, int64_t* status, cudaStream_t st) {
  cudaMemsetAsync(counts, 0, sizeof(int32_t) * world, st);
  if (n <= 0) { cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (world + 1), st); return; }
  cudaMemsetAsync(set_keys, 0xFF, sizeof(uint64_t) * set_cap, st);
  cudaMemsetAsync(set_pos + set_cap, 0xFF, sizeof(int32_t), st);  // spare cell for the sentinel id (-1)
  const int g = grid_stride_blocks(n);
  dedup_claim_kernel<<<g, kThreads, 2 * world * sizeof(int32_t), st>>>(ids, n, world, set_keys, set_pos, (uint64_t)set_cap - 1,
                                                                      slot_scratch, counts);
  rb::note_launch();
  dedup_assign_kernel<<<g, kThreads, (world + 1) * sizeof(int32_t), st>>>(ids, n, world, set_pos, slot_scratch, counts, offsets,
                                                                         unique_ids, reverse, unique_cap, status);
  rb::note_launch();
}

void rb_encode_merge(const int64_t* desc, const int64_t* table_idx, int F, int64_t total_nnz, int64_t total_seg,
                     int64_t* ids_out, int32_t* offsets_out, cudaStream_t st) {
  encode_merge_kernel<<<grid_stride_blocks(total_nnz + total_seg + 1), kThreads, 0, st>>>(desc, table_idx, F, total_nnz, total_seg,
                                                                                         ids_out, offsets_out);
  rb::note_launch();
}

void rb_gather_rows(const void* src, const int32_t* rows, int64_t n_max, const int32_t* n_dev, int64_t row_bytes, void* out, cudaStream_t st) {
  if (n_max <= 0 || row_bytes <= 0) return;
  dispatch_row_bytes(row_bytes, src, out, [&](auto v, int q) {
    using V = decltype(v);
    gather_rows_kernel<V><<<grid_stride_blocks(n_max * q), kThreads, 0, st>>>(static_cast<const V*>(src), rows, n_max, n_dev, q, static_cast<V*>(out));
  });
  rb::note_launch();
}

void rb_scatter_rows(void* dst, const int32_t* rows, int64_t n, int64_t row_bytes, const void* src, int src_broadcast, cudaStream_t st) {
  if (n <= 0 || row_bytes <= 0) return;
  dispatch_row_bytes(row_bytes, src, dst, [&](auto v, int q) {
    using V = decltype(v);
    scatter_rows_kernel<V><<<grid_stride_blocks(n * q), kThreads, 0, st>>>(static_cast<V*>(dst), rows, n, q, static_cast<const V*>(src), src_broadcast);
  });
  rb::note_launch();
}

void rb_fill_rows_i64(int64_t* dst, const int32_t* rows, int64_t n, int64_t value, cudaStream_t st) {
  if (n <= 0) return;
  fill_rows_i64_kernel<<<grid_stride_blocks(n), kThreads, 0, st>>>(dst, rows, n, value);
  rb::note_launch();
}

void rb_pool_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                     int64_t n_seg, int D, int mode, int perm_b, int perm_f, int perm_off, int perm_total, float* out, int32_t* gsrc,
                     float* gscale, cudaStream_t st) {
  if (n_seg <= 0) return;
  if (perm_f > 0 && perm_total <= 0) { perm_total = perm_f; perm_off = 0; }
  RB_DISPATCH_ROW(base_dtype, true, {
    const T* b = static_cast<const T*>(base);
    const bool ok = dispatch_cols(D, [&](auto g, auto nacc) {
      constexpr int G = decltype(g)::value, NACC = decltype(nacc)::value;
      const int64_t blocks = (n_seg + (kThreads / G) - 1) / (kThreads / G);
      pool_forward_kernel<G, NACC, T><<<(int)std::min<int64_t>(blocks, 148 * 64), kThreads, 0, st>>>(
          b, rows, rev, offsets, weights, n_seg, D, mode, perm_b, perm_f, perm_off, perm_total, out, gsrc, gscale);
    });
    if (!ok)
      pool_forward_scalar_kernel<T><<<grid_stride_blocks(n_seg * D), kThreads, 0, st>>>(b, rows, rev, offsets, weights, n_seg, D, mode,
                                                                                       perm_b, perm_f, perm_off, perm_total, out, gsrc, gscale);
  });
  rb::note_launch();
}

void rb_tile_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                     int64_t n_seg, int D, int tile_len, float* out, int32_t* gsrc, float* gscale, cudaStream_t st) {
  if (n_seg <= 0) return;
  RB_DISPATCH_ROW(base_dtype, true,
                  (tile_forward_kernel<T><<<grid_stride_blocks(n_seg * tile_len * D), kThreads, 0, st>>>(
                      static_cast<const T*>(base), rows, rev, offsets, weights, n_seg, D, tile_len, out, gsrc, gscale)));
  rb::note_launch();
}

size_t rb_sort_temp_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int32_t*)nullptr, (int32_t*)nullptr, (const int32_t*)nullptr,
                                  (int32_t*)nullptr, (int)n, 0, 32, (cudaStream_t)0);
  return bytes;
}

void rb_build_csr(const int32_t* reverse, int64_t n, int key_bits, void* temp, size_t temp_bytes, int32_t* iota_scratch,
                  int32_t* csr_u, int32_t* csr_elem, int32_t* start, cudaStream_t st) {
  if (n <= 0) return;
  iota_kernel<<<grid_stride_blocks(n), kThreads, 0, st>>>(iota_scratch, n);
  rb::note_launch();
  cub::DeviceRadixSort::SortPairs(temp, temp_bytes, reverse, csr_u, (const int32_t*)iota_scratch, csr_elem, (int)n, 0, key_bits, st);
  csr_heads_kernel<<<grid_stride_blocks(n), kThreads, 0, st>>>(csr_u, n, start);
  rb::note_launch();
}

void rb_sort_pairs_i32(const int32_t* keys_in, int32_t* keys_out, const int32_t* vals_in, int32_t* vals_out, int64_t n, int key_bits,
                       void* temp, size_t temp_bytes, cudaStream_t st) {
  if (n <= 0) return;
  cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys_in, keys_out, vals_in, vals_out, (int)n, 0, key_bits, st);
  rb::note_launch();
}

void rb_iota_i32(int32_t* out, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  iota_kernel<<<grid_stride_blocks(n), kThreads, 0, st>>>(out, n);
  rb::note_launch();
}

int rb_grad_reduce_chunk() { return kChunk; }

void rb_grad_reduce(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                    const int32_t* start, int64_t n, int D, float* span_acc, const int32_t* rows, float* gu, int apply, RbOpt opt,
                    cudaStream_t st) {
  if (n <= 0) return;
  const int64_t n_chunks = (n + kChunk - 1) / kChunk;
  const int dtype = apply ? opt.w_dtype : (int)rb::kRowF32;      // without an update no row is touched: one instantiation serves
  RB_DISPATCH_ROW(dtype, false, {
    const bool ok = dispatch_cols(D, [&](auto g, auto nacc) {
      constexpr int G = decltype(g)::value, NACC = decltype(nacc)::value;
      const int64_t blocks = (n_chunks + (kThreads / G) - 1) / (kThreads / G);
      const int grid = (int)std::min<int64_t>(blocks, 148 * 64);
      grad_reduce_kernel<G, NACC, false, T><<<grid, kThreads, 0, st>>>(grad_out, gsrc, gscale, csr_u, csr_elem, start, n, D, span_acc, rows,
                                                                       gu, apply, opt, RbGuPush{});
      rb::note_launch();
      grad_span_finish_kernel<G, NACC, false, T><<<grid, kThreads, 0, st>>>(csr_u, start, n, D, span_acc, rows, gu, apply, opt, RbGuPush{});
      rb::note_launch();
    });
    if (!ok) {
      grad_reduce_scalar_kernel<T><<<grid_stride_blocks(n * D), kThreads, 0, st>>>(grad_out, gsrc, gscale, csr_u, csr_elem, start, n, D, rows,
                                                                                  gu, apply, opt);
      rb::note_launch();
    }
  });
}

void rb_grad_reduce_push(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                         const int32_t* start, int64_t n, int D, float* span_acc, RbGuPush push, int max_blocks, cudaStream_t st) {
  if (n <= 0) return;
  const int64_t n_chunks = (n + kChunk - 1) / kChunk;
  RbOpt opt{};
  dispatch_cols(D, [&](auto g, auto nacc) {
    constexpr int G = decltype(g)::value, NACC = decltype(nacc)::value;
    const int64_t blocks = (n_chunks + (kThreads / G) - 1) / (kThreads / G);
    // max_blocks > 0 caps the grid (NVLink-bound kernel: a small grid leaves SMs to kernels of other streams)
    const int grid = (int)std::min<int64_t>(blocks, max_blocks > 0 ? max_blocks : 148 * 64);
    grad_reduce_kernel<G, NACC, true, float><<<grid, kThreads, 0, st>>>(grad_out, gsrc, gscale, csr_u, csr_elem, start, n, D, span_acc, nullptr,
                                                                        nullptr, 0, opt, push);
    rb::note_launch();
    grad_span_finish_kernel<G, NACC, true, float><<<grid, kThreads, 0, st>>>(csr_u, start, n, D, span_acc, nullptr, nullptr, 0, opt, push);
    rb::note_launch();
  });
}

void rb_sparse_apply(const int32_t* rows, const float* grads, int64_t n_max, const int32_t* n_dev, int D, RbOpt opt, cudaStream_t st) {
  if (n_max <= 0) return;
  RB_DISPATCH_ROW(opt.w_dtype, false,
                  (sparse_apply_kernel<T><<<grid_stride_blocks(n_max * ((D + 3) / 4)), kThreads, 0, st>>>(rows, grads, n_max, n_dev, D, opt)));
  rb::note_launch();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------------
// Allocation-free dedup + owner bucketing (declared in rb_noalloc.h).
//
// rb_dedup_partition above needs three scratch buffers (the hash set's keys and positions, and one slot index per id) which
// its callers obtain from an allocator. Some callers cannot do that: code that runs while a CUDA graph is being captured, a
// serving loop that must not touch cudaMalloc / the framework's caching allocator on its latency path, or a C host
// program that links this library without any tensor framework. For them the same two kernels run on a scratch area that
// lives in the library image itself: a file-scope __device__ array, present on every GPU that loads the library, for as long
// as the process lives. The price is a fixed ceiling on the number of ids per call and no concurrency between calls.
namespace {

constexpr int64_t kNoAllocMaxIds = RB_NOALLOC_MAX_IDS;                 // ids per call
constexpr int64_t kNoAllocMaxSlots = 2 * kNoAllocMaxIds;               // hash-set slots (power of two, load <= 0.5)
constexpr size_t kNoAllocKeysBytes = sizeof(uint64_t) * kNoAllocMaxSlots;
constexpr size_t kNoAllocPosBytes = ((sizeof(int32_t) * (kNoAllocMaxSlots + 1) + 255) / 256) * 256;
constexpr size_t kNoAllocSlotBytes = sizeof(int32_t) * kNoAllocMaxIds;
constexpr size_t kNoAllocBytes = kNoAllocKeysBytes + kNoAllocPosBytes + kNoAllocSlotBytes;   // about 7.3 MB

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kNoAllocMaxDevices = 64;
void* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

void noalloc_fail(char* err, size_t err_len, const char* msg) {
  if (err && err_len) { std::strncpy(err, msg, err_len - 1); err[err_len - 1] = '\0'; }
}

}  // namespace

extern "C" int rb_dedup_partition_noalloc(const int64_t* ids, int64_t n, int world, int32_t* counts, int32_t* offsets, int64_t* unique_ids,
                                          int32_t* reverse, cudaStream_t st, char* err, size_t err_len) {
  if (n < 0 || world < 1 || world > 1024) { noalloc_fail(err, err_len, "rb_dedup_partition_noalloc: n must be >= 0 and world in [1, 1024]"); return 1; }
  if (n > kNoAllocMaxIds) {
    char msg[192];
    std::snprintf(msg, sizeof(msg), "rb_dedup_partition_noalloc: %lld ids exceed the built-in scratch limit of %lld ids per call",
                  (long long)n, (long long)kNoAllocMaxIds);
    noalloc_fail(err, err_len, msg);
    return 2;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    noalloc_fail(err, err_len, "rb_dedup_partition_noalloc: no current CUDA device (or device index >= 64)");
    return 3;
  }
  void* base = nullptr;
  {
    // Set-up, once per device, with that device current: the array's name is only a host-side handle; the device address that
    // a kernel may dereference comes from cudaGetSymbolAddress.
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr) {
        noalloc_fail(err, err_len, cudaGetErrorString(e));
        return 4;
      }
      g_noalloc_ptr[dev] = p;
    }
    base = g_noalloc_ptr[dev];
  }
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * world, st) != cudaSuccess) { noalloc_fail(err, err_len, "memset of counts failed"); return 5; }
  if (n == 0) {
    if (cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (world + 1), st) != cudaSuccess) { noalloc_fail(err, err_len, "memset of offsets failed"); return 5; }
    return 0;
  }
  int64_t cap = 64;
  while (cap < 2 * n) cap <<= 1;                                        // <= kNoAllocMaxSlots because n <= kNoAllocMaxIds
  uint64_t* set_keys = reinterpret_cast<uint64_t*>(base);
  int32_t* set_pos = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(base) + kNoAllocKeysBytes);
  int32_t* slot = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(base) + kNoAllocKeysBytes + kNoAllocPosBytes);
  // the array keeps whatever the previous call left behind: everything that must start "empty" is reset here
  if (cudaMemsetAsync(set_keys, 0xFF, sizeof(uint64_t) * cap, st) != cudaSuccess ||
      cudaMemsetAsync(set_pos + cap, 0xFF, sizeof(int32_t), st) != cudaSuccess) {     // spare cell of the id -1; it moves with cap
    noalloc_fail(err, err_len, "memset of the built-in scratch failed");
    return 5;
  }
  const int g = grid_stride_blocks(n);
  dedup_claim_kernel<<<g, kThreads, 2 * world * sizeof(int32_t), st>>>(ids, n, world, set_keys, set_pos, (uint64_t)cap - 1, slot, counts);
  dedup_assign_kernel<<<g, kThreads, (world + 1) * sizeof(int32_t), st>>>(ids, n, world, set_pos, slot, counts, offsets, unique_ids, reverse, n, nullptr);
  rb::note_launch(2);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { noalloc_fail(err, err_len, cudaGetErrorString(e)); return 6; }
  return 0;
}
