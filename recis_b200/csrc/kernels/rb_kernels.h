// C launch API of the sm_100a kernels. Every function enqueues work on `st` and
// returns without synchronising. Sizes that are only known on the device are
// passed as `n_dev` (int32 in device memory) together with a host upper bound
// `n_max` that sizes the grid and the buffers; `n_dev == nullptr` means n_max is exact.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- table counters (int64 each, device memory)
enum RbCounter {
  RB_CTR_BUMP = 0,        // rows ever bump-allocated
  RB_CTR_FREE_TOP = 1,    // height of the free-row stack
  RB_CTR_NEW = 2,         // tickets handed out by the running lookup-or-insert
  RB_CTR_STATUS = 3,      // sticky error bits (rb::StatusBits)
  RB_CTR_LIVE = 4,        // admitted ids
  RB_CTR_TOMBSTONES = 5,  // erased slots not yet reclaimed by a rehash
  RB_CTR_PROBATION = 6,   // ids seen but not yet admitted
  RB_CTR_LAST_NEW = 7,    // rows admitted by the last lookup-or-insert
  RB_CTR_COUNT = 8
};

typedef struct RbTable {
  uint64_t* keys;      // [mask+1], 0xFF..FF empty, 0xFF..FE erased
  int32_t* rows;       // [mask+1], >=0 row, -1 none/pending, <=-2 probation count
  uint64_t mask;
  int64_t* ctr;        // [RB_CTR_COUNT]
  int32_t* free_list;  // [cap_rows]
  int64_t cap_rows;
} RbTable;

typedef struct RbInit {
  int kind;  // 0 constant, 1 uniform, 2 normal, 3 truncated normal
  float a, b, lo, hi;
  uint64_t seed;
} RbInit;

// row-wise sparse optimizers
enum RbOptKind { RB_OPT_ADAM = 0, RB_OPT_ADAGRAD = 1, RB_OPT_SGD = 2 };
// storage types of embedding rows (rb::RowDType): 0 fp32, 1 fp16, 2 bf16, 3 int8 (read-only tables)
enum RbRowDType { RB_ROW_F32 = 0, RB_ROW_F16 = 1, RB_ROW_BF16 = 2, RB_ROW_I8 = 3 };
typedef struct RbOpt {
  int kind;
  float lr;
  float beta1, beta2, eps;
  float decay;      // multiplicative weight decay factor applied to touched rows (1 = none)
  float alpha;      // Adam: -lr*sqrt(1-beta2^t)/(1-beta1^t)
  float grad_scale; // 1/(world * accumulation steps) etc.
  void* w;          // [cap, D] embedding slab, elements of type w_dtype (fp32 / fp16 / bf16)
  int w_dtype;      // RbRowDType of w; the state below and all arithmetic are fp32
  float* s1;        // Adam exp_avg    | Adagrad accumulator
  float* s2;        // Adam exp_avg_sq | unused
} RbOpt;

// Where per-unique gradients go when they are pushed to the ranks that own the rows instead of being stored locally:
// unique index u in [off[o], off[o+1]) is written to row dst_base[o] + (u - off[o]) of base[o], a (peer-mapped) window
// of cap_rows rows on rank o. off and dst_base are device arrays; rows that would fall beyond cap_rows are dropped.
typedef struct RbGuPush {
  const int32_t* off;        // [world+1] bucket boundaries of this rank's unique ids
  const int32_t* dst_base;   // [world]   first row of this rank's bucket inside owner o's window
  void* base[16];
  int world;
  int64_t cap_rows;
} RbGuPush;

// ---- table.cu
void rb_table_lookup_or_insert(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* slot_scratch,
                               int32_t* new_rows, int64_t* new_keys, int32_t* rows_out, void* emb, int emb_dtype, int D, RbInit init,
                               int64_t* last_seen, const int64_t* step_dev, int admit_threshold, int ids_unique, cudaStream_t st);
// ids_unique != 0: the caller guarantees that no id occurs twice in `ids`; new ids may then take erased slots (tombstones)
// met on their probe path instead of lengthening the chain, which keeps a table with steady eviction from filling its index.
void rb_table_find(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* rows_out, cudaStream_t st);
void rb_table_erase(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* erased_rows, cudaStream_t st);
void rb_table_snapshot(RbTable t, int64_t* ids_out, int32_t* rows_out, int64_t out_cap, int64_t* counter,
                       const int64_t* last_seen, int64_t threshold, int use_filter, cudaStream_t st);
void rb_table_rehash(RbTable src, RbTable dst, cudaStream_t st);

// ---- sparse_ops.cu
// Dedup ids and bucket the unique ids by owner rank. unique_ids holds unique_cap entries: when the batch has more unique ids
// the overflow bit is set in *status (nullable), the surplus ids are dropped and their reverse indices point at entry 0.
void rb_dedup_partition(const int64_t* ids, int64_t n, int world, uint64_t* set_keys, int32_t* set_pos, int64_t set_cap,
                        int32_t* slot_scratch, int32_t* counts, int32_t* offsets /*[world+1]*/, int64_t* unique_ids,
                        int32_t* reverse, int64_t unique_cap, int64_t* status, cudaStream_t st);
// Multi-tensor concat: ids get the 12-bit table prefix, offsets get the running nnz prefix.
// desc = int64[4][F+1] on the device: id pointers, nnz prefix, offsets pointers (int32 offsets), segment prefix;
// table_idx = int64[F].
void rb_encode_merge(const int64_t* desc, const int64_t* table_idx, int F, int64_t total_nnz, int64_t total_seg,
                     int64_t* ids_out, int32_t* offsets_out, cudaStream_t st);
// Row copies work on bytes: row_bytes = D * element size, any element type (source and destination have the same).
void rb_gather_rows(const void* src, const int32_t* rows, int64_t n_max, const int32_t* n_dev, int64_t row_bytes, void* out, cudaStream_t st);
void rb_scatter_rows(void* dst, const int32_t* rows, int64_t n, int64_t row_bytes, const void* src, int src_broadcast, cudaStream_t st);
void rb_fill_rows_i64(int64_t* dst, const int32_t* rows, int64_t n, int64_t value, cudaStream_t st);
// Pooling: out[orow(s)] = sum_i scale_i * base[row_i]; row_i = rows ? rows[rev[i]] : rev[i].
// mode 0 sum, 1 mean over length, 2 mean over weight sum. perm_f > 0 writes segment s=(f*perm_b+b) to row
// b*perm_total + perm_off + f (perm_total <= 0 means perm_total = perm_f, perm_off = 0): several calls can fill disjoint
// feature ranges of one [batch, perm_total, D] output. perm_f <= 0: segment s goes to row perm_off + s.
// gsrc/gscale (nullable) record, per element, the output row and the scale for the backward pass.
// base holds rows of type base_dtype (RbRowDType); sums and the output are fp32.
void rb_pool_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                     int64_t n_seg, int D, int mode, int perm_b, int perm_f, int perm_off, int perm_total, float* out, int32_t* gsrc,
                     float* gscale, cudaStream_t st);
// Tile combiner: out[s, t*D:(t+1)*D] = base[row of element t of segment s], t < tile_len, zero padded.
void rb_tile_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                     int64_t n_seg, int D, int tile_len, float* out, int32_t* gsrc, float* gscale, cudaStream_t st);
// Backward structure: stable radix sort of (reverse, element) pairs and per-unique start positions.
size_t rb_sort_temp_bytes(int64_t n);
void rb_build_csr(const int32_t* reverse, int64_t n, int key_bits, void* temp, size_t temp_bytes, int32_t* iota_scratch,
                  int32_t* csr_u, int32_t* csr_elem, int32_t* start /*[n+1]*/, cudaStream_t st);
// Segmented reduction of output gradients to unique rows, chunked so that one hot id cannot serialise the kernel.
// apply != 0: the optimizer update runs in the same kernel on row rows[u] (fused backward + update);
// apply == 0: the per-unique gradient is stored to gu[u].
void rb_grad_reduce(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                    const int32_t* start, int64_t n, int D, float* span_acc /*[ceil(n/chunk), D] zeros*/, const int32_t* rows,
                    float* gu, int apply, RbOpt opt, cudaStream_t st);
// Same reduction with apply == 0 semantics, the result rows stored through `push` (float4 rows only: D % 4 == 0, D <= 512).
void rb_grad_reduce_push(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                         const int32_t* start, int64_t n, int D, float* span_acc, RbGuPush push, int max_blocks, cudaStream_t st);
int rb_grad_reduce_chunk();
void rb_sparse_apply(const int32_t* rows, const float* grads, int64_t n_max, const int32_t* n_dev, int D, RbOpt opt, cudaStream_t st);

#ifdef __cplusplus
}
#endif
