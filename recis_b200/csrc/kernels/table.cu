// GPU dynamic-embedding index: one open-addressing hash table (u64 key -> row) with
// in-kernel row allocation, written for sm_100a.
//
// It provides what the reference's IdMap + IdAllocator pair provides
// (csrc/embedding/gpu_id_map.cu:19-116, csrc/embedding/id_allocator.cc:17-62,
// csrc/ops/hashtable_ops_kernel.cu:9-172) with a different structure: the reference
// chains find -> cumsum -> .item() -> GenIds -> compaction -> insert with several
// host synchronisations; here lookup-or-insert is three stream-ordered launches
// (claim, init, resolve) that never return to the host.
//
// Row allocation: inside one call every newly admitted key takes a dense ticket;
// tickets below the free-stack height reuse freed rows, the rest bump-allocate.
// The free-stack height and the bump pointer are constant during the claim kernel
// and are advanced by the resolve kernel, so no thread ever waits for another.
#include "../common/rb_common.cuh"
#include "rb_kernels.h"
#include "../common/rb_launch.h"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;
using namespace rb;

namespace {

constexpr int kThreads = 256;
constexpr uint32_t kMaxProbe = 1u << 22;

__device__ __forceinline__ int32_t alloc_row(const RbTable& t, uint64_t key, int32_t* new_rows, int64_t* new_keys) {
  auto g = cg::coalesced_threads();
  unsigned long long base = 0;
  if (g.thread_rank() == 0) base = atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_NEW]), (unsigned long long)g.size());
  const int64_t ticket = (int64_t)g.shfl(base, 0) + g.thread_rank();
  const int64_t free_top = t.ctr[RB_CTR_FREE_TOP], bump = t.ctr[RB_CTR_BUMP];
  int64_t row = ticket < free_top ? (int64_t)t.free_list[free_top - 1 - ticket] : bump + (ticket - free_top);
  if (row >= t.cap_rows) { set_status(&t.ctr[RB_CTR_STATUS], kStatusRowsExhausted); row = -1; }
  new_rows[ticket] = (int32_t)row; new_keys[ticket] = (int64_t)key;  // ticket < ids in this call <= buffer length
  return (int32_t)row;
}

// Find `key`, or claim an empty slot for it. Returns the slot, or -1.
// Row tickets for newly claimed keys are handed out once per block (ballot + one global atomic per block): a step that
// inserts a million new ids would otherwise serialise tens of thousands of atomics on the single ticket counter.
__global__ void __launch_bounds__(kThreads)
table_claim_kernel(RbTable t, const int64_t* __restrict__ ids, int64_t n_max, const int32_t* __restrict__ n_dev,
                   int32_t* __restrict__ slot_out, int32_t* __restrict__ new_rows, int64_t* __restrict__ new_keys,
                   int admit_threshold, int insert, int reuse_tombstones) {
  __shared__ int32_t warp_cnt[kThreads / 32];
  __shared__ unsigned long long block_base;
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x; i0 < n; i0 += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = i0 + threadIdx.x;
    int32_t slot = -1;
    bool need_row = false;
    int prob_delta = 0;                          // change of the probation counter caused by this thread (added once per warp below)
    uint64_t key = kEmptyKey;
    uint64_t h = 0;
    if (i < n) {
      key = (uint64_t)ids[i];
      if (key < kErasedKey) {
        h = mix64(key) & t.mask;
        int64_t tomb = -1;                      // first erased slot on the probe path (only looked at when reuse is allowed)
        for (uint32_t probe = 0; probe < kMaxProbe; ++probe, h = (h + 1) & t.mask) {
          uint64_t k = *reinterpret_cast<volatile uint64_t*>(&t.keys[h]);
          bool won = false;
          if (reuse_tombstones && k == kErasedKey && tomb < 0) tomb = (int64_t)h;
          if (k == kEmptyKey) {
            if (!insert) break;
            if (tomb >= 0) {
              // The key is not in the table (the chain ends here). Take the erased slot met on the way instead of making the
              // chain longer. Safe only because the ids of this call are distinct: no other thread can be inserting this key
              // into a different slot at the same time.
              const uint64_t prev = atomicCAS(reinterpret_cast<unsigned long long*>(&t.keys[tomb]), (unsigned long long)kErasedKey,
                                              (unsigned long long)key);
              if (prev == kErasedKey) {
                won = true; k = key; h = (uint64_t)tomb;
                atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_TOMBSTONES]), (unsigned long long)(-1ll));
              }
              tomb = -1;                        // taken by another key's thread: fall through to the empty slot
            }
            if (!won) {
              k = atomicCAS(reinterpret_cast<unsigned long long*>(&t.keys[h]), (unsigned long long)kEmptyKey, (unsigned long long)key);
              won = (k == kEmptyKey);
              if (won) k = key;
            }
          }
          if (k != key) {
            if (probe + 1 == kMaxProbe || probe >= t.mask) { set_status(&t.ctr[RB_CTR_STATUS], kStatusIndexFull); break; }
            continue;
          }
          slot = (int32_t)h;
          if (won) {
            if (admit_threshold <= 1) {
              need_row = true;                                       // ticket comes from the block-wide hand-out below
            } else {
              *reinterpret_cast<volatile int32_t*>(&t.rows[h]) = -2;  // probation, seen once
              prob_delta = 1;
            }
          } else if (insert && admit_threshold > 1) {
            // key exists; if it is on probation, count this occurrence and admit at the threshold.
            for (int spin = 0; spin < 64; ++spin) {
              const int32_t v = *reinterpret_cast<volatile int32_t*>(&t.rows[h]);
              if (v >= -1) break;            // admitted, or another thread is admitting it right now
              const int32_t seen = -1 - v;   // occurrences so far
              if (seen + 1 >= admit_threshold) {
                if (atomicCAS(&t.rows[h], v, kRowPending) == v) {
                  const int32_t row = alloc_row(t, key, new_rows, new_keys);
                  *reinterpret_cast<volatile int32_t*>(&t.rows[h]) = row >= 0 ? row : -1;
                  prob_delta = -1;
                  break;
                }
              } else if (atomicCAS(&t.rows[h], v, v - 1) == v) {
                break;
              }
            }
          }
          break;
        }
      }
      slot_out[i] = slot;
    }
    // ---- the probation counter moves once per warp: with an admission threshold most ids of a step are new to the table, and one
    // atomic per id on a single counter serialises tens of millions of them
    {
      const int wsum = __reduce_add_sync(0xffffffffu, prob_delta);
      if (lane == 0 && wsum != 0) atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_PROBATION]), (unsigned long long)(long long)wsum);
    }
    // ---- block-wide ticket hand-out
    const unsigned ballot = __ballot_sync(0xffffffffu, need_row);
    if (lane == 0) warp_cnt[warp] = __popc(ballot);
    __syncthreads();
    if (threadIdx.x == 0) {
      int total = 0;
      for (int wv = 0; wv < kThreads / 32; ++wv) { const int cnt = warp_cnt[wv]; warp_cnt[wv] = total; total += cnt; }
      block_base = total ? atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_NEW]), (unsigned long long)total) : 0ull;
    }
    __syncthreads();
    if (need_row) {
      const int64_t ticket = (int64_t)block_base + warp_cnt[warp] + __popc(ballot & ((1u << lane) - 1u));
      const int64_t free_top = t.ctr[RB_CTR_FREE_TOP], bump = t.ctr[RB_CTR_BUMP];
      int64_t row = ticket < free_top ? (int64_t)t.free_list[free_top - 1 - ticket] : bump + (ticket - free_top);
      if (row >= t.cap_rows) { set_status(&t.ctr[RB_CTR_STATUS], kStatusRowsExhausted); row = -1; }
      new_rows[ticket] = (int32_t)row; new_keys[ticket] = (int64_t)key;
      *reinterpret_cast<volatile int32_t*>(&t.rows[h]) = (int32_t)row;
    }
    __syncthreads();
  }
}

// Initialise the embedding of every row admitted by the preceding claim kernel.
// Values are a function of (seed, id, column), see rb_common.cuh.
template <typename T>
__global__ void __launch_bounds__(kThreads)
table_init_rows_kernel(RbTable t, const int32_t* __restrict__ new_rows, const int64_t* __restrict__ new_keys,
                       T* __restrict__ emb, int D, InitSpec spec) {
  const int64_t n_new = t.ctr[RB_CTR_NEW];
  const int quads = (D + 3) / 4;
  const int64_t total = n_new * quads;
  for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = w / quads; const int q = (int)(w - r * quads);
    const int32_t row = new_rows[r];
    if (row < 0) continue;
    float v[4];
    init_quad(spec, (uint64_t)new_keys[r], (uint32_t)q, v);
    T* dst = emb + (int64_t)row * D + q * 4;
    if ((D & 3) == 0) RowIO<T>::st4(dst, make_float4(v[0], v[1], v[2], v[3]));
    else for (int j = 0; j < 4 && q * 4 + j < D; ++j) RowIO<T>::st1(dst + j, v[j]);
  }
}

// slot -> row for every looked-up id; stamps the last-seen step; block 0 advances the allocator.
__global__ void __launch_bounds__(kThreads)
table_resolve_kernel(RbTable t, const int32_t* __restrict__ slots, int64_t n_max, const int32_t* __restrict__ n_dev,
                     int32_t* __restrict__ rows_out, int64_t* __restrict__ last_seen, const int64_t* __restrict__ step_dev,
                     int finalize) {
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  const int64_t step = step_dev ? *step_dev : 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_max; i += (int64_t)gridDim.x * blockDim.x) {
    if (i >= n) { rows_out[i] = -1; continue; }  // entries past the device-side count read as "no row"
    const int32_t s = slots[i];
    int32_t row = -1;
    if (s >= 0) { row = t.rows[s]; if (row < 0) row = -1; }
    rows_out[i] = row;
    if (last_seen && row >= 0) last_seen[row] = step;
  }
  if (finalize && blockIdx.x == 0 && threadIdx.x == 0) {
    const int64_t n_new = t.ctr[RB_CTR_NEW];
    const int64_t free_top = t.ctr[RB_CTR_FREE_TOP];
    const int64_t reused = n_new < free_top ? n_new : free_top;
    int64_t bump = t.ctr[RB_CTR_BUMP] + (n_new - reused);
    if (bump > t.cap_rows) bump = t.cap_rows;
    t.ctr[RB_CTR_FREE_TOP] = free_top - reused;
    t.ctr[RB_CTR_BUMP] = bump;
    t.ctr[RB_CTR_LIVE] += n_new;
    t.ctr[RB_CTR_LAST_NEW] = n_new;
    t.ctr[RB_CTR_NEW] = 0;
  }
}

__global__ void __launch_bounds__(kThreads)
table_find_kernel(RbTable t, const int64_t* __restrict__ ids, int64_t n_max, const int32_t* __restrict__ n_dev,
                  int32_t* __restrict__ rows_out) {
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_max; i += (int64_t)gridDim.x * blockDim.x) {
    if (i >= n) { rows_out[i] = -1; continue; }
    const uint64_t key = (uint64_t)ids[i];
    int32_t row = -1;
    if (key < kErasedKey) {
      uint64_t h = mix64(key) & t.mask;
      for (uint32_t probe = 0; probe < kMaxProbe && probe <= t.mask; ++probe, h = (h + 1) & t.mask) {
        const uint64_t k = t.keys[h];
        if (k == key) { row = t.rows[h]; if (row < 0) row = -1; break; }
        if (k == kEmptyKey) break;
      }
    }
    rows_out[i] = row;
  }
}

// Erase ids: tombstone the slot and push the row on the free stack. Ids must be unique within a call.
__global__ void __launch_bounds__(kThreads)
table_erase_kernel(RbTable t, const int64_t* __restrict__ ids, int64_t n_max, const int32_t* __restrict__ n_dev,
                   int32_t* __restrict__ erased_rows) {
  const int64_t n = n_dev ? min((int64_t)*n_dev, n_max) : n_max;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t key = (uint64_t)ids[i];
    int32_t row = -1;
    if (key < kErasedKey) {
      uint64_t h = mix64(key) & t.mask;
      for (uint32_t probe = 0; probe < kMaxProbe && probe <= t.mask; ++probe, h = (h + 1) & t.mask) {
        const uint64_t k = t.keys[h];
        if (k == key) {
          // exactly one thread turns the key into a tombstone
          if (atomicCAS(reinterpret_cast<unsigned long long*>(&t.keys[h]), (unsigned long long)key, (unsigned long long)kErasedKey) == key) {
            row = t.rows[h];
            t.rows[h] = -1;
            atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_TOMBSTONES]), 1ull);
            if (row >= 0) {
              const unsigned long long pos = atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_FREE_TOP]), 1ull);
              if ((int64_t)pos < t.cap_rows) t.free_list[pos] = row;
              atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_LIVE]), (unsigned long long)(-1ll));
            } else {
              if (row < -1) atomicAdd(reinterpret_cast<unsigned long long*>(&t.ctr[RB_CTR_PROBATION]), (unsigned long long)(-1ll));
              row = -1;
            }
          }
          break;
        }
        if (k == kEmptyKey) break;
      }
    }
    erased_rows[i] = row;
  }
}

// Compact (id,row) of every admitted entry; optionally only those whose last-seen step is below a threshold.
__global__ void __launch_bounds__(kThreads)
table_snapshot_kernel(RbTable t, int64_t* __restrict__ ids_out, int32_t* __restrict__ rows_out, int64_t out_cap,
                      int64_t* __restrict__ counter, const int64_t* __restrict__ last_seen, int64_t threshold, int use_filter) {
  const int64_t nslots = (int64_t)t.mask + 1;
  for (int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; s < nslots; s += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t k = t.keys[s];
    if (k >= kErasedKey) continue;
    const int32_t row = t.rows[s];
    if (row < 0) continue;
    if (use_filter && !(last_seen[row] < threshold)) continue;
    auto g = cg::coalesced_threads();
    unsigned long long base = 0;
    if (g.thread_rank() == 0) base = atomicAdd(reinterpret_cast<unsigned long long*>(counter), (unsigned long long)g.size());
    const int64_t pos = (int64_t)g.shfl(base, 0) + g.thread_rank();
    if (pos < out_cap) { ids_out[pos] = (int64_t)k; if (rows_out) rows_out[pos] = row; }
  }
}

// Re-insert every entry (admitted or on probation) of `src` into the empty index `dst`.
__global__ void __launch_bounds__(kThreads)
table_rehash_kernel(RbTable src, RbTable dst) {
  const int64_t nslots = (int64_t)src.mask + 1;
  for (int64_t s = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; s < nslots; s += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t k = src.keys[s];
    if (k >= kErasedKey) continue;
    const int32_t row = src.rows[s];
    if (row == -1) continue;
    uint64_t h = mix64(k) & dst.mask;
    for (uint32_t probe = 0; probe < kMaxProbe && probe <= dst.mask; ++probe, h = (h + 1) & dst.mask) {
      if (atomicCAS(reinterpret_cast<unsigned long long*>(&dst.keys[h]), (unsigned long long)kEmptyKey, (unsigned long long)k) == kEmptyKey) {
        dst.rows[h] = row;
        break;
      }
    }
  }
}

inline int grid_for(int64_t n, int per_thread = 1) {
  int64_t b = (n + (int64_t)kThreads * per_thread - 1) / ((int64_t)kThreads * per_thread);
  if (b < 1) b = 1;
  const int64_t cap = 148 * 16;  // grid-stride kernels: a few waves of resident CTAs per SM
  return (int)(b < cap ? b : cap);
}

}  // namespace

extern "C" {

void rb_table_lookup_or_insert(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* slot_scratch,
                               int32_t* new_rows, int64_t* new_keys, int32_t* rows_out, void* emb, int emb_dtype, int D, RbInit init,
                               int64_t* last_seen, const int64_t* step_dev, int admit_threshold, int ids_unique, cudaStream_t st) {
  if (n_max <= 0) return;
  const int g = grid_for(n_max);
  InitSpec spec{init.kind, init.a, init.b, init.lo, init.hi, init.seed};
  table_claim_kernel<<<g, kThreads, 0, st>>>(t, ids, n_max, n_dev, slot_scratch, new_rows, new_keys, admit_threshold, 1, ids_unique);
  rb::note_launch();
  RB_DISPATCH_ROW(emb_dtype, true,
                  (table_init_rows_kernel<T><<<grid_for(n_max * ((D + 3) / 4), 4), kThreads, 0, st>>>(t, new_rows, new_keys,
                                                                                                  static_cast<T*>(emb), D, spec)));
  rb::note_launch();
  table_resolve_kernel<<<g, kThreads, 0, st>>>(t, slot_scratch, n_max, n_dev, rows_out, last_seen, step_dev, 1);
  rb::note_launch();
}

void rb_table_find(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* rows_out, cudaStream_t st) {
  if (n_max <= 0) return;
  table_find_kernel<<<grid_for(n_max), kThreads, 0, st>>>(t, ids, n_max, n_dev, rows_out);
  rb::note_launch();
}

void rb_table_erase(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* erased_rows, cudaStream_t st) {
  if (n_max <= 0) return;
  table_erase_kernel<<<grid_for(n_max), kThreads, 0, st>>>(t, ids, n_max, n_dev, erased_rows);
  rb::note_launch();
}

void rb_table_snapshot(RbTable t, int64_t* ids_out, int32_t* rows_out, int64_t out_cap, int64_t* counter,
                       const int64_t* last_seen, int64_t threshold, int use_filter, cudaStream_t st) {
  table_snapshot_kernel<<<grid_for((int64_t)t.mask + 1), kThreads, 0, st>>>(t, ids_out, rows_out, out_cap, counter, last_seen,
                                                                           threshold, use_filter);
  rb::note_launch();
}

void rb_table_rehash(RbTable src, RbTable dst, cudaStream_t st) {
  table_rehash_kernel<<<grid_for((int64_t)src.mask + 1), kThreads, 0, st>>>(src, dst);
  rb::note_launch();
}

}  // extern "C"
