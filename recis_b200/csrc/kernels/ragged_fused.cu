// Multi-feature sequence truncation ("ragged cutoff") for sm_100a: ALL features of a call in three launches.
//
// The reference fuses the truncation of many ragged features into one kernel set (csrc/ops/fused_ragged_cutoff_kernel.cu:
// per-feature look-back scan on a (tiles, features) grid :102-258, 2-D / 3-D copy kernels over all features :451-784); a model
// with a thousand sparse fields cannot afford a launch set and a host read per field. Here a call is
//   1. one kernel over the concatenated rows of all features: per output row, where its values start in the source and how many
//      are kept (2-D: a row keeps at most `keep` values; 3-D: a sample keeps exactly `keep` inner rows, padded with empty ones),
//   2. one kernel with one block per feature: exclusive scan of the kept lengths -> the feature's new offsets and its total,
//   3. (after ONE host read of the per-feature totals, which sizes the outputs) one copy kernel on a (tiles, features) grid.
// Values are moved as bytes (element size 1, 2, 4 or 8), offsets may be int32 or int64 per feature.
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "rb_ragged_fused.h"
#include <cub/block/block_scan.cuh>

namespace {

constexpr int kThreads = 256;
constexpr int kScanThreads = 1024;

__device__ __forceinline__ int64_t ld_off(const void* p, int is_i64, int64_t i) {
  return is_i64 ? static_cast<const int64_t*>(p)[i] : (int64_t)static_cast<const int32_t*>(p)[i];
}
__device__ __forceinline__ void st_off(void* p, int is_i64, int64_t i, int64_t v) {
  if (is_i64) static_cast<int64_t*>(p)[i] = v; else static_cast<int32_t*>(p)[i] = (int32_t)v;
}

// the feature whose concatenated-row range contains r: prefix[t] <= r < prefix[t + 1]
__device__ __forceinline__ int find_feature(const RbCutoffFeature* f, int T, int64_t r) {
  int lo = 0, hi = T;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (f[mid].row_prefix <= r) lo = mid; else hi = mid; }
  return lo;
}

// 2-D: output row b of feature t keeps min(len, keep) values, from the right end when drop_left
__global__ void __launch_bounds__(kThreads)
cutoff2d_rows_kernel(const RbCutoffFeature* __restrict__ feats, int T, int64_t total_rows, int64_t* __restrict__ src_beg,
                     int64_t* __restrict__ keep_len, int64_t* __restrict__ drop_n, int64_t* __restrict__ pad_n) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < total_rows; r += (int64_t)gridDim.x * blockDim.x) {
    const RbCutoffFeature f = feats[find_feature(feats, T, r)];
    const int64_t b = r - f.row_prefix;
    const int64_t beg = ld_off(f.offsets, f.off_is_i64, b), len = ld_off(f.offsets, f.off_is_i64, b + 1) - beg;
    const int64_t kept = len < f.keep ? len : f.keep;
    src_beg[r] = beg + (f.drop_left ? len - kept : 0);
    keep_len[r] = kept; drop_n[r] = len - kept; pad_n[r] = f.keep - kept;
  }
}

// 3-D: sample b of feature t keeps exactly `keep` inner rows; output inner row w = b * keep + j is source inner row src (or an
// empty padding row). Also writes the new outer offsets (b * keep).
__global__ void __launch_bounds__(kThreads)
cutoff3d_rows_kernel(const RbCutoffFeature* __restrict__ feats, int T, int64_t total_rows, int64_t* __restrict__ src_beg,
                     int64_t* __restrict__ keep_len) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < total_rows; r += (int64_t)gridDim.x * blockDim.x) {
    const RbCutoffFeature f = feats[find_feature(feats, T, r)];
    const int64_t w = r - f.row_prefix, k = f.keep;
    const int64_t b = w / k, j = w - b * k;
    const int64_t o0 = ld_off(f.outer_offsets, f.off_is_i64, b), n_rows = ld_off(f.outer_offsets, f.off_is_i64, b + 1) - o0;
    const int64_t kept = n_rows < k ? n_rows : k, pad = k - kept;
    const int64_t jj = f.pad_left ? j - pad : j;                  // index among the kept rows
    int64_t beg = 0, len = 0;
    if (jj >= 0 && jj < kept) {
      const int64_t src = o0 + (f.drop_left ? n_rows - kept : 0) + jj;
      beg = ld_off(f.offsets, f.off_is_i64, src);
      len = ld_off(f.offsets, f.off_is_i64, src + 1) - beg;
    }
    src_beg[r] = beg; keep_len[r] = len;
    if (j == 0) st_off(f.out_outer, f.off_is_i64, b, b * k);
    if (w == f.n_out_rows - 1) st_off(f.out_outer, f.off_is_i64, b + 1, (b + 1) * k);
  }
}

// One block per feature: exclusive scan of its rows' kept lengths -> new offsets [n_out_rows + 1] and the feature's total.
__global__ void __launch_bounds__(kScanThreads)
cutoff_scan_kernel(const RbCutoffFeature* __restrict__ feats, const int64_t* __restrict__ keep_len, int64_t* __restrict__ totals) {
  using Scan = cub::BlockScan<int64_t, kScanThreads>;
  __shared__ typename Scan::TempStorage tmp;
  __shared__ int64_t carry;
  const RbCutoffFeature f = feats[blockIdx.x];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < f.n_out_rows; base += kScanThreads) {
    const int64_t i = base + threadIdx.x;
    const int64_t v = i < f.n_out_rows ? keep_len[f.row_prefix + i] : 0;
    int64_t excl, sum;
    Scan(tmp).ExclusiveSum(v, excl, sum);
    const int64_t c = carry;
    if (i < f.n_out_rows) st_off(f.out_offsets, f.off_is_i64, i, c + excl);
    __syncthreads();
    if (threadIdx.x == 0) carry = c + sum;
    __syncthreads();
  }
  if (threadIdx.x == 0) { st_off(f.out_offsets, f.off_is_i64, f.n_out_rows, carry); totals[blockIdx.x] = carry; }
}

// (row tiles, features) grid: eight lanes copy one output row, from src_beg[row] to new_offsets[row]. No search: a row knows where
// it starts on both sides (a lookup of the row by element position, as a flat loop over the elements needs, costs a binary search
// of 13 dependent loads per element at 8192 rows).
template <typename V>
__device__ __forceinline__ void copy_feature(const RbCutoffFeature& f, void* out_values, const int64_t* __restrict__ src_beg, int64_t total) {
  const V* src = static_cast<const V*>(f.values); V* dst = static_cast<V*>(out_values);
  const int sub = threadIdx.x & 7;
  const int64_t groups = ((int64_t)gridDim.x * blockDim.x) >> 3;
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3; r < f.n_out_rows; r += groups) {
    const int64_t o0 = ld_off(f.out_offsets, f.off_is_i64, r), len = ld_off(f.out_offsets, f.off_is_i64, r + 1) - o0;
    const int64_t s0 = src_beg[f.row_prefix + r];
    for (int64_t j = sub; j < len; j += 8) dst[o0 + j] = src[s0 + j];
  }
  (void)total;
}

__global__ void __launch_bounds__(kThreads)
cutoff_copy_kernel(const RbCutoffFeature* __restrict__ feats, void* const* __restrict__ out_values, const int64_t* __restrict__ totals,
                   const int64_t* __restrict__ src_beg) {
  const RbCutoffFeature f = feats[blockIdx.y];
  const int64_t total = totals[blockIdx.y];
  void* out = out_values[blockIdx.y];
  switch (f.elem_size) {
    case 8: copy_feature<uint64_t>(f, out, src_beg, total); break;
    case 4: copy_feature<uint32_t>(f, out, src_beg, total); break;
    case 2: copy_feature<uint16_t>(f, out, src_beg, total); break;
    default: copy_feature<uint8_t>(f, out, src_beg, total); break;
  }
}

inline int blocks_for(int64_t n) {
  int64_t b = (n + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  const int64_t cap = 148 * 16;
  return (int)(b < cap ? b : cap);
}

}  // namespace

extern "C" {

void rb_cutoff_rows(const RbCutoffFeature* feats, int T, int64_t total_rows, int three_d, int64_t* src_beg, int64_t* keep_len,
                    int64_t* drop_n, int64_t* pad_n, int64_t* totals, cudaStream_t st) {
  if (T <= 0) return;
  if (total_rows > 0) {
    if (three_d) cutoff3d_rows_kernel<<<blocks_for(total_rows), kThreads, 0, st>>>(feats, T, total_rows, src_beg, keep_len);
    else cutoff2d_rows_kernel<<<blocks_for(total_rows), kThreads, 0, st>>>(feats, T, total_rows, src_beg, keep_len, drop_n, pad_n);
    rb::note_launch();
  }
  cutoff_scan_kernel<<<T, kScanThreads, 0, st>>>(feats, keep_len, totals);
  rb::note_launch();
}

void rb_cutoff_copy(const RbCutoffFeature* feats, int T, void* const* out_values, const int64_t* totals, const int64_t* src_beg,
                    int64_t max_total, cudaStream_t st) {
  if (T <= 0 || max_total <= 0) return;
  int64_t tiles = (max_total + kThreads - 1) / kThreads;
  const int64_t cap = std::max<int64_t>(1, (148 * 16) / T);      // the grid's y dimension carries the features
  if (tiles > cap) tiles = cap;
  dim3 grid((unsigned)tiles, (unsigned)T);
  cutoff_copy_kernel<<<grid, kThreads, 0, st>>>(feats, out_values, totals, src_beg);
  rb::note_launch();
}

}  // extern "C"
