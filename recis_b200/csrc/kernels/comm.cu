// Multi-GPU exchange kernels over peer-mapped memory (NVLink 5 / NVSwitch), sm_100a.
//
// One process per GPU; every rank maps the other ranks' symmetric buffers (cudaIpc handles) and these kernels issue
// ordinary ld/st/red to peer addresses. No NCCL call is involved and the host never learns the split sizes.
// They replace the reference's four torch.distributed all_to_all_single calls per table group and step
// (recis/nn/modules/embedding.py:498-624: counts C1, ids C2, embeddings C3, gradients C4) and DDP's bucketed
// all-reduce (recis/framework/trainer.py:170-184):
//
//   forward   requester: dedup + bucket ids by owner into its own window            -> signal(IDS)
//             owner:     wait(IDS), pull ids from every requester's window, table lookup-or-insert,
//                        push the embedding row of every incoming id straight into the requester's
//                        unique-embedding buffer (peer stores)                       -> signal(EMB)
//             requester: wait(EMB), pool from its local unique-embedding buffer
//   backward  requester: reduce pooled gradients to one gradient per unique id and store each of them straight into
//                        the gradient window of the rank that owns the id (peer stores)  -> signal(GRAD)
//             owner:     wait(GRAD), for every touched row: add the contributions of all requesters (they sit in this
//                        rank's own window: local loads only), apply the row-wise optimizer   (one kernel)
//   dense     two-shot all-reduce: each rank reduces 1/W of the flat gradient buffer from all peers and writes the
//             averaged slice back to all peers.
//
// Synchronisation is a per-(channel, source rank) epoch word in each rank's flag pad, written with st.release.sys
// after a system-scope fence and polled with ld.acquire.sys. Every poll loop is bounded: on a timeout the kernel sets
// kStatusWaitTimeout in the status word and returns, so a missing peer can never hang a GPU.
// No TMA multicast is used anywhere; peer memory is only touched by plain loads and stores.
#include "../common/rb_common.cuh"
#include "../common/rb_opt.cuh"
#include "../common/rb_launch.h"
#include "rb_comm.h"

using namespace rb;

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void st_release_sys(int64_t* p, int64_t v) {
  asm volatile("st.release.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int64_t ld_acquire_sys(const int64_t* p) {
  int64_t v;
  asm volatile("ld.acquire.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

inline int grid_stride_blocks(int64_t work_items) {
  int64_t b = (work_items + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  const int64_t cap = 148 * 16;
  return (int)(b < cap ? b : cap);
}

// flags layout per rank: [channel][source rank] int64 epochs
__global__ void comm_signal_kernel(RbPeers flag_pads, int channel, int me, int world, int64_t epoch) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int64_t*>(flag_pads.p[p]) + (int64_t)channel * world + me, epoch);
  }
}

__global__ void comm_wait_kernel(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status) {
  const int p = threadIdx.x;
  if (p < world) {
    const int64_t* f = flags + (int64_t)channel * world + p;
    // spin_limit is a time limit in microseconds (measured with the global nanosecond timer), doubly bounded by an
    // iteration count so that a stuck timer cannot turn this into an endless loop.
    bool ok = false;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    const uint64_t limit_ns = (uint64_t)spin_limit * 1000ull;
    for (int64_t it = 0; it < (int64_t)1 << 34; ++it) {
      if (ld_acquire_sys(f) >= epoch) { ok = true; break; }
      __nanosleep(100);
      if ((it & 63) == 63) {
        uint64_t t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) break;
      }
    }
    if (!ok) set_status(status, kStatusWaitTimeout);
    __threadfence_system();
  }
}

// The same wait with accounting: thread p adds the nanoseconds it spent until peer p's flag arrived to
// stats[channel * world + p] (and the number of waits to stats[RB_CH_COUNT * world + channel]; RB_CH_COUNT * (world + 1) words). The time of a wait as a
// whole is the maximum over p, i.e. the time until the last peer arrived: what a step pays for being ahead of its peers.
// Kept apart from comm_wait_kernel so that the default path carries no extra work.
__global__ void comm_wait_timed_kernel(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status,
                                       unsigned long long* stats) {
  const int p = threadIdx.x;
  if (p < world) {
    const int64_t* f = flags + (int64_t)channel * world + p;
    bool ok = false;
    uint64_t t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    t1 = t0;
    const uint64_t limit_ns = (uint64_t)spin_limit * 1000ull;
    for (int64_t it = 0; it < (int64_t)1 << 34; ++it) {
      if (ld_acquire_sys(f) >= epoch) { ok = true; break; }
      __nanosleep(100);
      if ((it & 63) == 63) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) break;
      }
    }
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (!ok) set_status(status, kStatusWaitTimeout);
    atomicAdd(stats + (int64_t)channel * world + p, (unsigned long long)(t1 - t0));
    if (p == 0) atomicAdd(stats + (int64_t)RB_CH_COUNT * world + channel, 1ull);
    __threadfence_system();
  }
}

__device__ __forceinline__ int find_src(const int32_t* prefix, int world, int64_t j) {
  int r = 0;
  while (r + 1 < world && prefix[r + 1] <= j) ++r;
  return r;
}

// Owner: gather the ids every requester bucketed for me. peer_offsets[r] -> int32[world+1] of requester r (boundaries
// clamped to its window), peer_ids[r] -> its bucketed unique ids, peer_counts[r] -> int32[world] unclamped per-owner unique
// counts of requester r (what it wanted to send). Writes ids_in, prefix[4*world+2] and n_in. Everything published in prefix is
// clamped to in_cap: a window that is too small drops ids (and sets the overflow bit), it never makes a later kernel index
// past a buffer. demand[0..1] (nullable) keep running maxima over ALL ranks of (unique ids one requester wanted to send,
// ids one owner was asked for): every rank computes the same two numbers from the same W x W counts, which is what lets the
// hosts agree on growing the windows without a collective.
__global__ void __launch_bounds__(kThreads)
pull_ids_kernel(RbPeers peer_ids, RbPeers peer_offsets, RbPeers peer_counts, int me, int world, int64_t* __restrict__ ids_in,
                int64_t in_cap, int32_t* __restrict__ prefix_out, int32_t* __restrict__ n_in_dev, int32_t* __restrict__ demand,
                int64_t* status) {
  __shared__ int32_t prefix[RB_MAX_PEERS + 1];
  __shared__ int32_t src_off[RB_MAX_PEERS];
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int r = 0; r < world; ++r) {
      const int32_t* off = reinterpret_cast<const int32_t*>(peer_offsets.p[r]);
      const int32_t b = off[me], e = off[me + 1];
      prefix[r] = (int32_t)min(run, in_cap); src_off[r] = b; run += (e - b);
    }
    prefix[world] = (int32_t)min(run, in_cap);
    if (run > in_cap) set_status(status, kStatusWindowOverflow);
  }
  __syncthreads();
  const int64_t n_in = prefix[world];
  if (blockIdx.x == 0) {
    // prefix_out = [prefix[0..world], src_off[0..world-1]]: kept by the owner for the rest of the step, because the
    // requesters' offset windows are rewritten by their next forward pass.
    for (int r = threadIdx.x; r <= world; r += blockDim.x) prefix_out[r] = prefix[r];
    for (int r = threadIdx.x; r < world; r += blockDim.x) prefix_out[world + 1 + r] = src_off[r];
    // prefix_out[2*world+1 + o]: where THIS rank's bucket for owner o starts inside o's incoming order (the sum of what the
    // lower ranks send to o); the backward pass pushes its per-unique gradients to exactly those rows of o's window.
    for (int o = threadIdx.x; o < world; o += blockDim.x) {
      int32_t base = 0;
      for (int r = 0; r < me; ++r) {
        const int32_t* off = reinterpret_cast<const int32_t*>(peer_offsets.p[r]);
        base += off[o + 1] - off[o];
      }
      prefix_out[2 * world + 1 + o] = base;
    }
    // prefix_out[3*world+1 ..]: a copy of THIS rank's own bucket boundaries [world+1] (its offsets window is rewritten by its
    // next forward pass; the backward pass needs this step's)
    {
      const int32_t* own = reinterpret_cast<const int32_t*>(peer_offsets.p[me]);
      for (int w = threadIdx.x; w <= world; w += blockDim.x) prefix_out[3 * world + 1 + w] = own[w];
    }
    if (threadIdx.x == 0) *n_in_dev = (int32_t)n_in;
    if (demand != nullptr && peer_counts.p[0] != nullptr && threadIdx.x < world) {
      // thread t: what requester t wanted to send in total, and what owner t was asked for in total
      int64_t out_t = 0, in_t = 0;
      const int32_t* mine = reinterpret_cast<const int32_t*>(peer_counts.p[threadIdx.x]);
      for (int o = 0; o < world; ++o) out_t += mine[o];
      for (int r = 0; r < world; ++r) in_t += reinterpret_cast<const int32_t*>(peer_counts.p[r])[threadIdx.x];
      atomicMax(&demand[0], (int32_t)min(out_t, (int64_t)0x7FFFFFFF));
      atomicMax(&demand[1], (int32_t)min(in_t, (int64_t)0x7FFFFFFF));
    }
  }
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < n_in; j += (int64_t)gridDim.x * blockDim.x) {
    const int r = find_src(prefix, world, j);
    const int64_t* src = reinterpret_cast<const int64_t*>(peer_ids.p[r]);
    ids_in[j] = src[src_off[r] + (j - prefix[r])];
  }
}

// Owner: store the embedding row of incoming id j into its requester's unique-embedding buffer. Rows travel as bytes (q
// 16-byte pieces per row), so one kernel serves fp32, fp16 and bf16 rows: the wire format is the storage format.
// A work item is (k, piece): it serves the k-th id of EVERY requester, so all peer links carry traffic for the whole
// kernel (instead of one requester after the other) and each thread has up to `world` independent load/store pairs in flight.
__global__ void __launch_bounds__(kThreads)
push_emb_kernel(const uint4* __restrict__ emb, const int32_t* __restrict__ rows_in, const int32_t* __restrict__ prefix_in,
                RbPeers peer_uemb, int me, int world, int q) {
  __shared__ int32_t prefix[RB_MAX_PEERS + 1];
  __shared__ int32_t dst_off[RB_MAX_PEERS];
  __shared__ int32_t max_cnt;
  if (threadIdx.x <= world) prefix[threadIdx.x] = prefix_in[threadIdx.x];
  if (threadIdx.x < world) dst_off[threadIdx.x] = prefix_in[world + 1 + threadIdx.x];
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t m = 0;
    for (int r = 0; r < world; ++r) m = max(m, prefix[r + 1] - prefix[r]);
    max_cnt = m;
  }
  __syncthreads();
  const int64_t total = (int64_t)max_cnt * q;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  constexpr int U = 4;                       // rows in flight per thread and requester
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int64_t w0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w0 < total; w0 += stride * U) {
    for (int r0 = 0; r0 < world; ++r0) {
      const int r = (r0 + me + 1) % world;    // start with the right neighbour: ranks do not all hammer rank 0 first
      const int32_t cnt = prefix[r + 1] - prefix[r];
      int32_t row[U]; int64_t k[U]; int c[U]; uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t w = w0 + u * stride;
        k[u] = w / q; c[u] = (int)(w - k[u] * q);
        row[u] = (w < total && k[u] < cnt) ? rows_in[prefix[r] + k[u]] : -2;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = row[u] >= 0 ? emb[(int64_t)row[u] * q + c[u]] : zero;
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (row[u] != -2) reinterpret_cast<uint4*>(peer_uemb.p[r])[((int64_t)dst_off[r] + k[u]) * q + c[u]] = v[u];
    }
  }
}

// Owner: chain together the incoming ids that resolved to the same table row (different requesters may ask for the
// same id). head[row] holds the last linked incoming index (-1 when idle), next[j] the one linked before j.
__global__ void __launch_bounds__(kThreads)
owner_link_kernel(const int32_t* __restrict__ rows_in, const int32_t* __restrict__ prefix_in, int world, int32_t* __restrict__ head,
                  int32_t* __restrict__ next) {
  const int64_t n_in = prefix_in[world];
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < n_in; j += (int64_t)gridDim.x * blockDim.x) {
    const int32_t row = rows_in[j];
    next[j] = row >= 0 ? atomicExch(&head[row], (int32_t)j) : -1;
  }
}

__global__ void __launch_bounds__(kThreads)
owner_unlink_kernel(const int32_t* __restrict__ rows_in, const int32_t* __restrict__ prefix_in, int world, int32_t* __restrict__ head) {
  const int64_t n_in = prefix_in[world];
  for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < n_in; j += (int64_t)gridDim.x * blockDim.x)
    if (rows_in[j] >= 0) head[rows_in[j]] = -1;
}

// Owner: one work item per (incoming id j, float4 column); the gradients of all requesters already sit in this rank's
// window g_in (row j = the j-th incoming id), pushed there by the requesters' backward kernels. The item whose j heads its
// row's chain sums the chain (at most one entry per requester; a + b is order independent, three or more are summed in
// ascending j order so the result does not depend on scheduling), then updates the row (apply) or stores (row, gradient)
// at position j (apply == 0; non-head positions get row -1). U independent items are in flight per thread: their index
// reads, optimizer-state loads and gradient loads are all issued before any of them is consumed.
template <int U, typename T>
__global__ void __launch_bounds__(kThreads)
owner_reduce_kernel(const int32_t* __restrict__ rows_in, const int32_t* __restrict__ head, const int32_t* __restrict__ next,
                    const int32_t* __restrict__ prefix_in, const float* __restrict__ g_in, int world, int D,
                    int mean_by_id, int apply, RbOpt opt, int32_t* __restrict__ out_rows, float* __restrict__ out_grads) {
  const int64_t n_in = prefix_in[world];
  const int q = D >> 2;
  const int64_t total = n_in * q;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t w0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w0 < total; w0 += stride * U) {
    int64_t j0[U]; int c[U]; int32_t row[U]; int32_t nx[U]; bool is_head[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t w = w0 + u * stride;
      j0[u] = w / q; c[u] = (int)(w - j0[u] * q);
      row[u] = w < total ? rows_in[j0[u]] : -1;
      if (w >= total) j0[u] = -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      is_head[u] = row[u] >= 0 && head[row[u]] == (int32_t)j0[u];
      nx[u] = is_head[u] ? next[j0[u]] : -1;
      if (!apply && c[u] == 0 && j0[u] >= 0 && !is_head[u]) out_rows[j0[u]] = -1;
    }
    float4 sw[U], s1v[U], s2v[U], acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      acc[u] = make_float4(0.f, 0.f, 0.f, 0.f); sw[u] = acc[u]; s1v[u] = acc[u]; s2v[u] = acc[u];
      if (!is_head[u]) continue;
      const int64_t off = (int64_t)row[u] * D + c[u] * 4;
      if (apply) {
        sw[u] = RowIO<T>::ld4(static_cast<const T*>(opt.w) + off);
        if (opt.kind != RB_OPT_SGD) s1v[u] = ld_f4(opt.s1 + off);
        if (opt.kind == RB_OPT_ADAM) s2v[u] = ld_f4(opt.s2 + off);
      }
      acc[u] = ld_f4(g_in + j0[u] * D + c[u] * 4);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!is_head[u]) continue;
      int cnt = 1;
      if (nx[u] >= 0) {                                   // several requesters asked for this id
        int32_t chain[RB_MAX_PEERS];
        chain[0] = (int32_t)j0[u];
        for (int32_t j = nx[u]; j >= 0 && cnt < RB_MAX_PEERS; j = next[j]) chain[cnt++] = j;
        if (cnt > 2) {
          for (int a = 1; a < cnt; ++a) {
            const int32_t v = chain[a]; int b = a - 1;
            while (b >= 0 && chain[b] > v) { chain[b + 1] = chain[b]; --b; }
            chain[b + 1] = v;
          }
          acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int a = (cnt > 2 ? 0 : 1); a < cnt; ++a) {
          const float4 g = ld_f4(g_in + (int64_t)chain[a] * D + c[u] * 4);
          acc[u].x += g.x; acc[u].y += g.y; acc[u].z += g.z; acc[u].w += g.w;
        }
      }
      if (mean_by_id && cnt > 1) { const float sc = 1.f / (float)cnt; acc[u].x *= sc; acc[u].y *= sc; acc[u].z *= sc; acc[u].w *= sc; }
      const int64_t off = (int64_t)row[u] * D + c[u] * 4;
      if (apply) {
        opt_update_pre_f4<T>(opt, off, acc[u], sw[u], s1v[u], s2v[u]);
      } else {
        if (c[u] == 0) out_rows[j0[u]] = row[u];
        const float gs = opt.grad_scale;
        st_f4(out_grads + j0[u] * D + c[u] * 4, make_float4(acc[u].x * gs, acc[u].y * gs, acc[u].z * gs, acc[u].w * gs));
      }
    }
  }
}

// Two-shot all-reduce (mean) over peer-mapped flat fp32 buffers. Phase 0: reduce my slice from all peers into
// registers and write the averaged values back into every peer's buffer. Caller brackets it with signal / wait.
__global__ void __launch_bounds__(kThreads)
allreduce_slice_kernel(RbPeers bufs, int me, int world, int64_t n, float scale) {
  const int64_t n4 = n >> 2;                                  // n is padded to a multiple of 4 * world by the host
  const int64_t per = n4 / world;
  const int64_t beg = per * me, end = beg + per;
  for (int64_t i = beg + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < end; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(bufs.p[r])[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(bufs.p[r])[i] = acc;
  }
}

}  // namespace

extern "C" {

void rb_comm_signal(RbPeers flag_pads, int channel, int me, int world, int64_t epoch, cudaStream_t st) {
  comm_signal_kernel<<<1, 32, 0, st>>>(flag_pads, channel, me, world, epoch);
  rb::note_launch();
}

void rb_comm_wait_timed(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status, int64_t* stats,
                        cudaStream_t st) {
  comm_wait_timed_kernel<<<1, 32, 0, st>>>(flags, channel, world, epoch, spin_limit, status, reinterpret_cast<unsigned long long*>(stats));
  rb::note_launch();
}

void rb_comm_wait(const int64_t* flags, int channel, int world, int64_t epoch, int64_t spin_limit, int64_t* status, cudaStream_t st) {
  comm_wait_kernel<<<1, 32, 0, st>>>(flags, channel, world, epoch, spin_limit, status);
  rb::note_launch();
}

void rb_comm_pull_ids(RbPeers peer_ids, RbPeers peer_offsets, RbPeers peer_counts, int me, int world, int64_t* ids_in, int64_t in_cap,
                      int32_t* prefix_out, int32_t* n_in_dev, int32_t* demand, int64_t* status, cudaStream_t st) {
  pull_ids_kernel<<<grid_stride_blocks(in_cap / 4 + 1), kThreads, 0, st>>>(peer_ids, peer_offsets, peer_counts, me, world, ids_in, in_cap,
                                                                        prefix_out, n_in_dev, demand, status);
  rb::note_launch();
}

void rb_comm_push_emb(const void* emb, const int32_t* rows_in, const int32_t* prefix, RbPeers peer_uemb, int me, int world,
                      int64_t row_bytes, int64_t n_in_max, int blocks, cudaStream_t st) {
  // blocks > 0 caps the grid: the kernel is bound by NVLink, not by the SMs, and a small grid leaves the SMs to kernels of
  // other streams that run at the same time
  const int q = (int)(row_bytes / 16);         // callers guarantee row_bytes % 16 == 0
  int g = grid_stride_blocks(n_in_max * q);
  if (blocks > 0 && blocks < g) g = blocks;
  push_emb_kernel<<<g, kThreads, 0, st>>>(static_cast<const uint4*>(emb), rows_in, prefix, peer_uemb, me, world, q);
  rb::note_launch();
}

void rb_comm_owner_reduce(const int32_t* rows_in, int32_t* head, int32_t* next, const int32_t* prefix, const float* g_in, int world,
                          int D, int mean_by_id, int apply, RbOpt opt, int32_t* out_rows, float* out_grads, int64_t n_in_max,
                          int unroll, cudaStream_t st) {
  const int g1 = grid_stride_blocks(n_in_max / 4 + 1);
  owner_link_kernel<<<g1, kThreads, 0, st>>>(rows_in, prefix, world, head, next);
  rb::note_launch();
  const int g2 = grid_stride_blocks(n_in_max * (D / 4) / 4 + 1);
  const int dtype = apply ? opt.w_dtype : (int)rb::kRowF32;      // without an update no row is touched
  RB_DISPATCH_ROW(dtype, false, {
    if (unroll >= 4)
      owner_reduce_kernel<4, T><<<g2, kThreads, 0, st>>>(rows_in, head, next, prefix, g_in, world, D, mean_by_id, apply, opt, out_rows, out_grads);
    else if (unroll >= 2)
      owner_reduce_kernel<2, T><<<g2, kThreads, 0, st>>>(rows_in, head, next, prefix, g_in, world, D, mean_by_id, apply, opt, out_rows, out_grads);
    else
      owner_reduce_kernel<1, T><<<g2, kThreads, 0, st>>>(rows_in, head, next, prefix, g_in, world, D, mean_by_id, apply, opt, out_rows, out_grads);
  });
  rb::note_launch();
  owner_unlink_kernel<<<g1, kThreads, 0, st>>>(rows_in, prefix, world, head);
  rb::note_launch();
}

void rb_comm_allreduce_slice(RbPeers bufs, int me, int world, int64_t n_padded, float scale, cudaStream_t st) {
  const int64_t per = (n_padded / 4) / world;
  allreduce_slice_kernel<<<grid_stride_blocks(per), kThreads, 0, st>>>(bufs, me, world, n_padded, scale);
  rb::note_launch();
}

}  // extern "C"

// Plain streaming copy between two device pointers (either may be a peer mapping): the microbenchmark that measures what
// NVLink delivers to ordinary loads / stores issued from a kernel.
namespace {
__global__ void __launch_bounds__(256) peer_copy_kernel(float4* __restrict__ dst, const float4* __restrict__ src, int64_t n4) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
}
}  // namespace

extern "C" void rb_comm_copy(void* dst, const void* src, int64_t nbytes, int blocks, cudaStream_t st) {
  peer_copy_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), nbytes / 16);
  rb::note_launch();
}
