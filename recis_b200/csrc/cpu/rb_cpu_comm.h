// CPU counterparts of the exchange launchers in kernels/rb_comm.h (same arguments minus the stream). The "peer" pointers are
// addresses of shared-memory mappings of the other ranks' windows.
#pragma once
#include <algorithm>
#include <cmath>
#include <vector>
#include "../kernels/rb_comm.h"

#ifdef __cplusplus
extern "C" {
#endif

void rbc_comm_signal(RbPeers flag_pads, int channel, int me, int world, int64_t epoch);
void rbc_comm_wait(const int64_t* flags, int channel, int world, int64_t epoch, int64_t limit_us, int64_t* status);
void rbc_comm_wait_timed(const int64_t* flags, int channel, int world, int64_t epoch, int64_t limit_us, int64_t* status, int64_t* stats);
void rbc_comm_pull_ids(RbPeers peer_ids, RbPeers peer_offsets, RbPeers peer_counts, int me, int world, int64_t* ids_in, int64_t in_cap,
                       int32_t* prefix_out, int32_t* n_in_out, int32_t* demand, int64_t* status);
void rbc_comm_push_emb(const void* emb, const int32_t* rows_in, const int32_t* prefix, RbPeers peer_uemb, int me, int world,
                       int64_t row_bytes, int64_t in_cap);
// gu: [n_unique, D] per-unique gradients in this rank's bucketed order; off / dst_base as in RbGuPush
void rbc_comm_push_grads(const float* gu, int D, const int32_t* off, const int32_t* dst_base, RbPeers peer_gin, int world, int64_t cap_rows);
void rbc_comm_owner_reduce(const int32_t* rows_in, int32_t* head, int32_t* next, const int32_t* prefix, const float* g_in, int world,
                           int D, int mean_by_id, int apply, RbOpt opt, int32_t* out_rows, float* out_grads);
void rbc_comm_allreduce_slice(RbPeers bufs, int me, int world, int64_t n_padded, float scale);

#ifdef __cplusplus
}
#endif
