// CPU counterparts of the launchers in kernels/rb_kernels.h (same arguments minus the stream).
#pragma once
#include "../kernels/rb_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

void rbc_table_lookup_or_insert(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* slot_scratch,
                                int32_t* new_rows, int64_t* new_keys, int32_t* rows_out, void* emb, int emb_dtype, int D, RbInit init,
                                int64_t* last_seen, const int64_t* step_dev, int admit_threshold, int ids_unique);
void rbc_table_find(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* rows_out);
void rbc_table_erase(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* erased_rows);
void rbc_table_snapshot(RbTable t, int64_t* ids_out, int32_t* rows_out, int64_t out_cap, int64_t* counter,
                        const int64_t* last_seen, int64_t threshold, int use_filter);
void rbc_table_rehash(RbTable src, RbTable dst);
void rbc_dedup_partition(const int64_t* ids, int64_t n, int world, uint64_t* set_keys, int32_t* set_pos, int64_t set_cap,
                         int32_t* slot_scratch, int32_t* counts, int32_t* offsets, int64_t* unique_ids, int32_t* reverse,
                         int64_t unique_cap, int64_t* status);
void rbc_encode_merge(const int64_t* desc, const int64_t* table_idx, int F, int64_t total_nnz, int64_t total_seg,
                      int64_t* ids_out, int32_t* offsets_out);
void rbc_gather_rows(const void* src, const int32_t* rows, int64_t n_max, const int32_t* n_dev, int64_t row_bytes, void* out);
void rbc_scatter_rows(void* dst, const int32_t* rows, int64_t n, int64_t row_bytes, const void* src, int src_broadcast);
void rbc_fill_rows_i64(int64_t* dst, const int32_t* rows, int64_t n, int64_t value);
void rbc_pool_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                      int64_t n_seg, int D, int mode, int perm_b, int perm_f, int perm_off, int perm_total, float* out, int32_t* gsrc,
                      float* gscale);
void rbc_tile_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                      int64_t n_seg, int D, int tile_len, float* out, int32_t* gsrc, float* gscale);
void rbc_build_csr(const int32_t* reverse, int64_t n, int32_t* csr_u, int32_t* csr_elem, int32_t* start);
void rbc_grad_reduce(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                     const int32_t* start, int64_t n, int D, const int32_t* rows, float* gu, int apply, RbOpt opt);
void rbc_sparse_apply(const int32_t* rows, const float* grads, int64_t n_max, const int32_t* n_dev, int D, RbOpt opt);

#ifdef __cplusplus
}
#endif
