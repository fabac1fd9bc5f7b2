// C launch API of the multi-feature sequence truncation kernels (ragged_fused.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// One feature of a fused truncation call (an array of these lives in device memory).
typedef struct RbCutoffFeature {
  const void* values;         // source values, elem_size bytes each
  const void* offsets;        // 2-D: row offsets [n_rows + 1]; 3-D: inner-row offsets
  const void* outer_offsets;  // 3-D only: sample offsets [n_samples + 1] into the inner rows
  void* out_offsets;          // new (inner) offsets [n_out_rows + 1], same integer type as `offsets`
  void* out_outer;            // 3-D only: new sample offsets [n_samples + 1]
  int64_t n_out_rows;         // 2-D: rows; 3-D: samples * keep
  int64_t keep;               // 2-D: values kept per row at most; 3-D: inner rows per sample exactly
  int64_t row_prefix;         // output rows of the features before this one (position in the concatenated row space)
  int32_t elem_size;          // 1, 2, 4 or 8
  int32_t off_is_i64;         // offsets are int64 (else int32)
  int32_t drop_left;          // drop from the left end (keep the newest) instead of the right end
  int32_t pad_left;           // 3-D: empty padding rows go in front
} RbCutoffFeature;

// Launches 1 and 2: per output row its source position and kept length (plus drop / pad counts for 2-D), then per feature
// the scan of the kept lengths into out_offsets and totals[t]. src_beg / keep_len (and drop_n / pad_n for 2-D): int64 [total_rows].
void rb_cutoff_rows(const RbCutoffFeature* feats, int T, int64_t total_rows, int three_d, int64_t* src_beg, int64_t* keep_len,
                    int64_t* drop_n, int64_t* pad_n, int64_t* totals, cudaStream_t st);
// Launch 3: the copy, on a (tiles, features) grid. out_values: device array of T pointers; max_total: largest totals[t] (host).
void rb_cutoff_copy(const RbCutoffFeature* feats, int T, void* const* out_values, const int64_t* totals, const int64_t* src_beg,
                    int64_t max_total, cudaStream_t st);

#ifdef __cplusplus
}
#endif
