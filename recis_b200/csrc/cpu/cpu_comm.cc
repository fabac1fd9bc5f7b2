// CPU twin of the peer-memory exchange kernels (kernels/comm.cu): the same window arithmetic, flag protocol and duplicate
// chaining, executed by one process per rank on buffers that live in shared memory mapped by every rank. It is the oracle of the
// exchange logic on machines without GPUs (the multi-rank tests run the whole fused path of parallel/fused_exchange.py through
// it) and a shared-memory exchange for CPU multi-process runs. Flags are 64-bit epochs written with release stores and polled
// with acquire loads; every wait is bounded by wall-clock time and reports through the status word, like its device version.
#include <chrono>
#include <cstring>
#include <thread>
#include "rb_cpu.h"
#include "rb_cpu_comm.h"
#include "rb_cpu_row.h"

namespace {

constexpr int64_t kStatusWaitTimeout = 4, kStatusWindowOverflow = 8;      // same bits as rb_common.cuh

inline void set_status(int64_t* status, int64_t bit) { __atomic_fetch_or(status, bit, __ATOMIC_RELAXED); }

inline void opt_update(const RbOpt& o, int64_t off, float g) {
  g *= o.grad_scale;
  float w = rbcpu::row_ld(o.w, o.w_dtype, off);
  if (o.kind == RB_OPT_ADAM) {
    const float m = o.beta1 * o.s1[off] + (1.f - o.beta1) * g;
    const float v = o.beta2 * o.s2[off] + (1.f - o.beta2) * g * g;
    o.s1[off] = m; o.s2[off] = v;
    w = w * o.decay + o.alpha * m / (std::sqrt(v) + o.eps);
  } else if (o.kind == RB_OPT_ADAGRAD) {
    const float a = o.s1[off] + g * g;
    o.s1[off] = a;
    w = w * o.decay - o.lr * g / (std::sqrt(a) + o.eps);
  } else {
    w = w * o.decay - o.lr * g;
  }
  rbcpu::row_st(o.w, o.w_dtype, off, w);
}

}  // namespace

extern "C" {

void rbc_comm_signal(RbPeers flag_pads, int channel, int me, int world, int64_t epoch) {
  for (int p = 0; p < world; ++p)
    __atomic_store_n(reinterpret_cast<int64_t*>(flag_pads.p[p]) + (int64_t)channel * world + me, epoch, __ATOMIC_RELEASE);
}

void rbc_comm_wait(const int64_t* flags, int channel, int world, int64_t epoch, int64_t limit_us, int64_t* status) {
  const auto t0 = std::chrono::steady_clock::now();
  for (int p = 0; p < world; ++p) {
    const int64_t* f = flags + (int64_t)channel * world + p;
    int64_t spins = 0;
    while (__atomic_load_n(f, __ATOMIC_ACQUIRE) < epoch) {
      if ((++spins & 1023) == 0) {
        if (std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() > limit_us) {
          set_status(status, kStatusWaitTimeout);
          return;
        }
        std::this_thread::yield();
      }
    }
  }
}

// The same wait with accounting (layout of stats as in rb_comm_wait_timed): nanoseconds until each peer's flag arrived, per
// (channel, peer), and the number of waits per channel.
void rbc_comm_wait_timed(const int64_t* flags, int channel, int world, int64_t epoch, int64_t limit_us, int64_t* status, int64_t* stats) {
  const auto t0 = std::chrono::steady_clock::now();
  bool timed_out = false;
  for (int p = 0; p < world; ++p) {
    const int64_t* f = flags + (int64_t)channel * world + p;
    int64_t spins = 0;
    while (!timed_out && __atomic_load_n(f, __ATOMIC_ACQUIRE) < epoch) {
      if ((++spins & 1023) == 0) {
        if (std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() > limit_us) timed_out = true;
        std::this_thread::yield();
      }
    }
    stats[(int64_t)channel * world + p] += std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
  }
  stats[(int64_t)RB_CH_COUNT * world + channel] += 1;
  if (timed_out) set_status(status, kStatusWaitTimeout);
}

void rbc_comm_pull_ids(RbPeers peer_ids, RbPeers peer_offsets, RbPeers peer_counts, int me, int world, int64_t* ids_in, int64_t in_cap,
                       int32_t* prefix_out, int32_t* n_in_out, int32_t* demand, int64_t* status) {
  // everything published in prefix_out is clamped to in_cap (see pull_ids_kernel): an overflow drops ids, nothing downstream
  // indexes past a buffer
  int64_t run = 0;
  for (int r = 0; r < world; ++r) {
    const int32_t* off = reinterpret_cast<const int32_t*>(peer_offsets.p[r]);
    const int32_t b = off[me], e = off[me + 1];
    prefix_out[r] = (int32_t)std::min<int64_t>(run, in_cap);
    prefix_out[world + 1 + r] = b;
    run += e - b;
  }
  prefix_out[world] = (int32_t)std::min<int64_t>(run, in_cap);
  if (run > in_cap) set_status(status, kStatusWindowOverflow);
  for (int o = 0; o < world; ++o) {          // where this rank's bucket for owner o starts inside o's incoming order
    int32_t base = 0;
    for (int r = 0; r < me; ++r) {
      const int32_t* off = reinterpret_cast<const int32_t*>(peer_offsets.p[r]);
      base += off[o + 1] - off[o];
    }
    prefix_out[2 * world + 1 + o] = base;
  }
  {
    const int32_t* own = reinterpret_cast<const int32_t*>(peer_offsets.p[me]);       // this rank's own boundaries, kept for the backward
    for (int w = 0; w <= world; ++w) prefix_out[3 * world + 1 + w] = own[w];
  }
  const int64_t n_in = prefix_out[world];
  *n_in_out = (int32_t)n_in;
  if (demand != nullptr && peer_counts.p[0] != nullptr) {
    for (int t = 0; t < world; ++t) {
      int64_t out_t = 0, in_t = 0;
      for (int o = 0; o < world; ++o) out_t += reinterpret_cast<const int32_t*>(peer_counts.p[t])[o];
      for (int r = 0; r < world; ++r) in_t += reinterpret_cast<const int32_t*>(peer_counts.p[r])[t];
      demand[0] = std::max<int32_t>(demand[0], (int32_t)std::min<int64_t>(out_t, 0x7FFFFFFF));
      demand[1] = std::max<int32_t>(demand[1], (int32_t)std::min<int64_t>(in_t, 0x7FFFFFFF));
    }
  }
  for (int r = 0; r < world; ++r) {
    const int64_t* src = reinterpret_cast<const int64_t*>(peer_ids.p[r]) + prefix_out[world + 1 + r];
    const int64_t beg = prefix_out[r];
    const int64_t cnt = (int64_t)prefix_out[r + 1] - beg;
    if (cnt > 0) std::memcpy(ids_in + beg, src, sizeof(int64_t) * (size_t)cnt);
  }
}

void rbc_comm_push_emb(const void* emb, const int32_t* rows_in, const int32_t* prefix, RbPeers peer_uemb, int me, int world,
                       int64_t row_bytes, int64_t in_cap) {
  (void)me;
  const char* src = static_cast<const char*>(emb);
  for (int r = 0; r < world; ++r) {
    char* dst = reinterpret_cast<char*>(peer_uemb.p[r]) + (int64_t)prefix[world + 1 + r] * row_bytes;
    const int64_t beg = prefix[r], end = std::min<int64_t>(prefix[r + 1], in_cap);
    for (int64_t j = beg; j < end; ++j) {
      const int32_t row = rows_in[j];
      if (row >= 0) std::memcpy(dst + (j - beg) * row_bytes, src + (int64_t)row * row_bytes, (size_t)row_bytes);
      else std::memset(dst + (j - beg) * row_bytes, 0, (size_t)row_bytes);
    }
  }
}

void rbc_comm_push_grads(const float* gu, int D, const int32_t* off, const int32_t* dst_base, RbPeers peer_gin, int world, int64_t cap_rows) {
  for (int o = 0; o < world; ++o) {
    float* base = reinterpret_cast<float*>(peer_gin.p[o]);
    for (int64_t u = off[o]; u < off[o + 1]; ++u) {
      const int64_t r = (int64_t)dst_base[o] + (u - off[o]);
      if (r < cap_rows) std::memcpy(base + r * D, gu + u * D, sizeof(float) * D);
    }
  }
}

void rbc_comm_owner_reduce(const int32_t* rows_in, int32_t* head, int32_t* next, const int32_t* prefix, const float* g_in, int world,
                           int D, int mean_by_id, int apply, RbOpt opt, int32_t* out_rows, float* out_grads) {
  const int64_t n_in = prefix[world];
  for (int64_t j = 0; j < n_in; ++j) {                       // link: head[row] = last incoming index, next[j] = the one before
    const int32_t row = rows_in[j];
    if (row >= 0) { next[j] = head[row]; head[row] = (int32_t)j; } else next[j] = -1;
  }
  std::vector<float> acc((size_t)D);
  for (int64_t j = 0; j < n_in; ++j) {
    const int32_t row = rows_in[j];
    const bool is_head = row >= 0 && head[row] == (int32_t)j;
    if (!is_head) { if (!apply) out_rows[j] = -1; continue; }
    int32_t chain[RB_MAX_PEERS];
    int cnt = 0;
    for (int32_t k = (int32_t)j; k >= 0 && cnt < RB_MAX_PEERS; k = next[k]) chain[cnt++] = k;
    std::sort(chain, chain + cnt);                           // ascending incoming order: the sum does not depend on arrival order
    std::fill(acc.begin(), acc.end(), 0.f);
    for (int a = 0; a < cnt; ++a) {
      const float* g = g_in + (int64_t)chain[a] * D;
      for (int d = 0; d < D; ++d) acc[d] += g[d];
    }
    if (mean_by_id && cnt > 1) { const float sc = 1.f / (float)cnt; for (int d = 0; d < D; ++d) acc[d] *= sc; }
    if (apply) {
      for (int d = 0; d < D; ++d) opt_update(opt, (int64_t)row * D + d, acc[d]);
    } else {
      out_rows[j] = row;
      for (int d = 0; d < D; ++d) out_grads[j * D + d] = acc[d] * opt.grad_scale;
    }
  }
  for (int64_t j = 0; j < n_in; ++j) if (rows_in[j] >= 0) head[rows_in[j]] = -1;      // unlink
}

void rbc_comm_allreduce_slice(RbPeers bufs, int me, int world, int64_t n_padded, float scale) {
  const int64_t per = n_padded / world, beg = per * me, end = beg + per;
  for (int64_t i = beg; i < end; ++i) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += reinterpret_cast<const float*>(bufs.p[r])[i];
    acc *= scale;
    for (int r = 0; r < world; ++r) reinterpret_cast<float*>(bufs.p[r])[i] = acc;
  }
}

}  // extern "C"
