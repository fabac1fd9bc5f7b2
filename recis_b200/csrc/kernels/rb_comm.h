// C launch API of the peer-memory exchange kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "rb_kernels.h"

#define RB_MAX_PEERS 16

#ifdef __cplusplus
extern "C" {
#endif

// One pointer per rank (this rank's own buffer at index `me`), passed by value to kernels.
typedef struct RbPeers { void* p[RB_MAX_PEERS]; } RbPeers;

enum RbChannel { RB_CH_IDS = 0, RB_CH_EMB = 1, RB_CH_GRAD = 2, RB_CH_AR0 = 3, RB_CH_AR1 = 4, RB_CH_COUNT = 8 };

void rb_comm_signal(RbPeers flag_pads, int channel, int me, int world, int64_t epoch, cudaStream_t st);
void rb_comm_wait(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status, cudaStream_t st);
// Same as rb_comm_wait, and adds the time spent per peer to stats: int64 [RB_CH_COUNT * world + RB_CH_COUNT] (nanoseconds per
// (channel, peer), then the number of waits per channel).
void rb_comm_wait_timed(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status, int64_t* stats,
                        cudaStream_t st);
// peer_counts (entries may be null) and demand (nullable, int32[2]): see pull_ids_kernel; prefix_out is clamped to in_cap
void rb_comm_pull_ids(RbPeers peer_ids, RbPeers peer_offsets, RbPeers peer_counts, int me, int world, int64_t* ids_in, int64_t in_cap,
                      int32_t* prefix_out, int32_t* n_in_dev, int32_t* demand, int64_t* status, cudaStream_t st);
// prefix: int32[4*world+2] written by rb_comm_pull_ids = per-source prefix sums [world+1], per-source window offsets
// [world], for every owner o the first row of this rank's bucket inside o's incoming order [world], and a copy of this
// rank's own bucket boundaries [world+1]
// blocks > 0 caps the grid size (the kernel is NVLink-bound; a small grid leaves SMs to concurrent kernels)
// rows travel as bytes: row_bytes = D * element size of the table's rows, a multiple of 16
void rb_comm_push_emb(const void* emb, const int32_t* rows_in, const int32_t* prefix, RbPeers peer_uemb, int me, int world,
                      int64_t row_bytes, int64_t n_in_max, int blocks, cudaStream_t st);
// head: int32[table capacity], all -1 between calls; next: int32[n_in_max] scratch; g_in: this rank's gradient window
// [n_in_max, D] filled by the requesters (rb_grad_reduce_push); unroll: 1, 2 or 4 work items in flight per thread.
void rb_comm_owner_reduce(const int32_t* rows_in, int32_t* head, int32_t* next, const int32_t* prefix, const float* g_in, int world,
                          int D, int mean_by_id, int apply, RbOpt opt, int32_t* out_rows, float* out_grads, int64_t n_in_max,
                          int unroll, cudaStream_t st);
void rb_comm_allreduce_slice(RbPeers bufs, int me, int world, int64_t n_padded, float scale, cudaStream_t st);
// generic key/value radix sort of int32 pairs (keys need `key_bits` low bits); temp sized by rb_sort_temp_bytes
void rb_sort_pairs_i32(const int32_t* keys_in, int32_t* keys_out, const int32_t* vals_in, int32_t* vals_out, int64_t n, int key_bits,
                       void* temp, size_t temp_bytes, cudaStream_t st);
void rb_iota_i32(int32_t* out, int64_t n, cudaStream_t st);
void rb_comm_copy(void* dst, const void* src, int64_t nbytes, int blocks, cudaStream_t st);

#ifdef __cplusplus
}
#endif
