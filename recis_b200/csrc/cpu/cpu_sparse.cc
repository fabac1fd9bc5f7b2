// CPU implementations of the table and sparse-path operations, with the semantics of the CUDA kernels
// in kernels/table.cu and kernels/sparse_ops.cu. They are (a) the oracle the GPU tests compare against,
// (b) the implementation used when a model runs on CPU (gloo ranks), and (c) the timed CPU baseline.
//
// The reference's CPU counterparts are csrc/embedding/cpu_id_map.cc:73-184 (flat_hash_map under a mutex),
// csrc/ops/hashtable_ops.cc:5-59, csrc/ops/block_ops.cc:6-272, csrc/ops/block_apply_adamw_op.cc:8-85 and
// csrc/ops/ids_partition.cc:6-38; its pooling kernels have no CPU version at all. Here every operation has one.
#include "../common/rb_common.cuh"
#include "../kernels/rb_kernels.h"
#include "rb_cpu.h"
#include "rb_cpu_row.h"
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

using namespace rb;

namespace {
inline int64_t eff_n(int64_t n_max, const int32_t* n_dev) { return n_dev ? std::min<int64_t>(*n_dev, n_max) : n_max; }

inline int32_t cpu_alloc_row(RbTable& t, uint64_t key, int32_t* new_rows, int64_t* new_keys) {
  const int64_t ticket = t.ctr[RB_CTR_NEW]++;
  const int64_t free_top = t.ctr[RB_CTR_FREE_TOP], bump = t.ctr[RB_CTR_BUMP];
  int64_t row = ticket < free_top ? (int64_t)t.free_list[free_top - 1 - ticket] : bump + (ticket - free_top);
  if (row >= t.cap_rows) { t.ctr[RB_CTR_STATUS] |= kStatusRowsExhausted; row = -1; }
  new_rows[ticket] = (int32_t)row; new_keys[ticket] = (int64_t)key;
  return (int32_t)row;
}

inline void cpu_opt_update(const RbOpt& o, int64_t off, float g) {
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
inline int64_t out_row_of(int64_t s, int perm_b, int perm_f, int perm_off, int perm_total) {
  if (perm_f <= 0) return s + perm_off;
  const int64_t f = s / perm_b, b = s - f * perm_b;
  return b * perm_total + perm_off + f;
}
}  // namespace

extern "C" {

void rbc_table_lookup_or_insert(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* slot_scratch,
                                int32_t* new_rows, int64_t* new_keys, int32_t* rows_out, void* emb, int emb_dtype, int D, RbInit init,
                                int64_t* last_seen, const int64_t* step_dev, int admit_threshold, int ids_unique) {
  (void)ids_unique;        // inserts run one after the other here: an erased slot on the probe path can always be taken
  const int64_t n = eff_n(n_max, n_dev);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t key = (uint64_t)ids[i];
    int32_t slot = -1;
    if (key < kErasedKey) {
      uint64_t h = mix64(key) & t.mask;
      int64_t tomb = -1;
      for (uint64_t probe = 0; probe <= t.mask; ++probe, h = (h + 1) & t.mask) {
        const uint64_t k = t.keys[h];
        if (k == kErasedKey && tomb < 0) tomb = (int64_t)h;
        if (k == kEmptyKey) {
          if (tomb >= 0) { h = (uint64_t)tomb; t.ctr[RB_CTR_TOMBSTONES]--; }
          t.keys[h] = key; slot = (int32_t)h;
          if (admit_threshold <= 1) t.rows[h] = cpu_alloc_row(t, key, new_rows, new_keys);
          else { t.rows[h] = -2; t.ctr[RB_CTR_PROBATION]++; }
          break;
        }
        if (k == key) {
          slot = (int32_t)h;
          const int32_t v = t.rows[h];
          if (admit_threshold > 1 && v < -1) {
            const int32_t seen = -1 - v;
            if (seen + 1 >= admit_threshold) { t.rows[h] = cpu_alloc_row(t, key, new_rows, new_keys); t.ctr[RB_CTR_PROBATION]--; }
            else t.rows[h] = v - 1;
          }
          break;
        }
        if (probe == t.mask) t.ctr[RB_CTR_STATUS] |= kStatusIndexFull;
      }
    }
    slot_scratch[i] = slot;
  }
  const int64_t n_new = t.ctr[RB_CTR_NEW];
  InitSpec spec{init.kind, init.a, init.b, init.lo, init.hi, init.seed};
  const int quads = (D + 3) / 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n_new; ++r) {
    const int32_t row = new_rows[r];
    if (row < 0) continue;
    for (int q = 0; q < quads; ++q) {
      float v[4];
      init_quad(spec, (uint64_t)new_keys[r], (uint32_t)q, v);
      for (int j = 0; j < 4 && q * 4 + j < D; ++j) rbcpu::row_st(emb, emb_dtype, (int64_t)row * D + q * 4 + j, v[j]);
    }
  }
  const int64_t step = step_dev ? *step_dev : 0;
  for (int64_t i = n; i < n_max; ++i) rows_out[i] = -1;
  for (int64_t i = 0; i < n; ++i) {
    const int32_t s = slot_scratch[i];
    int32_t row = -1;
    if (s >= 0) { row = t.rows[s]; if (row < 0) row = -1; }
    rows_out[i] = row;
    if (last_seen && row >= 0) last_seen[row] = step;
  }
  const int64_t free_top = t.ctr[RB_CTR_FREE_TOP];
  const int64_t reused = std::min(n_new, free_top);
  t.ctr[RB_CTR_FREE_TOP] = free_top - reused;
  t.ctr[RB_CTR_BUMP] = std::min(t.ctr[RB_CTR_BUMP] + (n_new - reused), t.cap_rows);
  t.ctr[RB_CTR_LIVE] += n_new;
  t.ctr[RB_CTR_LAST_NEW] = n_new;
  t.ctr[RB_CTR_NEW] = 0;
}

void rbc_table_find(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* rows_out) {
  const int64_t n = eff_n(n_max, n_dev);
  for (int64_t i = n; i < n_max; ++i) rows_out[i] = -1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t key = (uint64_t)ids[i];
    int32_t row = -1;
    if (key < kErasedKey) {
      uint64_t h = mix64(key) & t.mask;
      for (uint64_t probe = 0; probe <= t.mask; ++probe, h = (h + 1) & t.mask) {
        const uint64_t k = t.keys[h];
        if (k == key) { row = t.rows[h]; if (row < 0) row = -1; break; }
        if (k == kEmptyKey) break;
      }
    }
    rows_out[i] = row;
  }
}

void rbc_table_erase(RbTable t, const int64_t* ids, int64_t n_max, const int32_t* n_dev, int32_t* erased_rows) {
  const int64_t n = eff_n(n_max, n_dev);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t key = (uint64_t)ids[i];
    int32_t row = -1;
    if (key < kErasedKey) {
      uint64_t h = mix64(key) & t.mask;
      for (uint64_t probe = 0; probe <= t.mask; ++probe, h = (h + 1) & t.mask) {
        const uint64_t k = t.keys[h];
        if (k == key) {
          row = t.rows[h]; t.keys[h] = kErasedKey; t.rows[h] = -1; t.ctr[RB_CTR_TOMBSTONES]++;
          if (row >= 0) { t.free_list[t.ctr[RB_CTR_FREE_TOP]++] = row; t.ctr[RB_CTR_LIVE]--; }
          else { if (row < -1) t.ctr[RB_CTR_PROBATION]--; row = -1; }
          break;
        }
        if (k == kEmptyKey) break;
      }
    }
    erased_rows[i] = row;
  }
}

void rbc_table_snapshot(RbTable t, int64_t* ids_out, int32_t* rows_out, int64_t out_cap, int64_t* counter,
                        const int64_t* last_seen, int64_t threshold, int use_filter) {
  const int64_t nslots = (int64_t)t.mask + 1;
  for (int64_t s = 0; s < nslots; ++s) {
    const uint64_t k = t.keys[s];
    if (k >= kErasedKey) continue;
    const int32_t row = t.rows[s];
    if (row < 0) continue;
    if (use_filter && !(last_seen[row] < threshold)) continue;
    const int64_t pos = (*counter)++;
    if (pos < out_cap) { ids_out[pos] = (int64_t)k; if (rows_out) rows_out[pos] = row; }
  }
}

void rbc_table_rehash(RbTable src, RbTable dst) {
  const int64_t nslots = (int64_t)src.mask + 1;
  for (int64_t s = 0; s < nslots; ++s) {
    const uint64_t k = src.keys[s];
    if (k >= kErasedKey) continue;
    const int32_t row = src.rows[s];
    if (row == -1) continue;
    uint64_t h = mix64(k) & dst.mask;
    for (uint64_t probe = 0; probe <= dst.mask; ++probe, h = (h + 1) & dst.mask)
      if (dst.keys[h] == kEmptyKey) { dst.keys[h] = k; dst.rows[h] = row; break; }
  }
}

void rbc_dedup_partition(const int64_t* ids, int64_t n, int world, uint64_t* set_keys, int32_t* set_pos, int64_t set_cap,
                         int32_t* slot_scratch, int32_t* counts, int32_t* offsets, int64_t* unique_ids, int32_t* reverse,
                         int64_t unique_cap, int64_t* status) {
  std::memset(counts, 0, sizeof(int32_t) * world);
  std::memset(offsets, 0, sizeof(int32_t) * (world + 1));
  if (n <= 0) return;
  std::memset(set_keys, 0xFF, sizeof(uint64_t) * set_cap);
  set_pos[set_cap] = -1;
  const uint64_t mask = (uint64_t)set_cap - 1;
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t key = (uint64_t)ids[i];
    int32_t slot = -1; bool won = false;
    if (key == kEmptyKey) { slot = (int32_t)set_cap; won = set_pos[set_cap] == -1; if (won) set_pos[set_cap] = -2; }
    else {
      uint64_t h = mix64(key) & mask;
      for (uint64_t probe = 0; probe <= mask; ++probe, h = (h + 1) & mask) {
        if (set_keys[h] == kEmptyKey) { set_keys[h] = key; won = true; }
        if (set_keys[h] == key) { slot = (int32_t)h; break; }
      }
    }
    if (won) set_pos[slot] = counts[owner_of(key, world)]++;
    slot_scratch[i] = slot | (won ? (int32_t)0x80000000 : 0);
  }
  // More unique ids than the output holds (an exchange window): flagged in the status word, boundaries clamped to the buffer,
  // the ids beyond it dropped (their reverse index points at entry 0) - the device version does the same.
  std::vector<int32_t> off((size_t)world + 1);
  int32_t run = 0;
  for (int w = 0; w < world; ++w) { off[w] = run; run += counts[w]; }
  off[world] = run;
  if (run > unique_cap && status) __atomic_fetch_or(status, (int64_t)8, __ATOMIC_RELAXED);
  for (int w = 0; w <= world; ++w) offsets[w] = (int32_t)std::min<int64_t>(off[w], unique_cap);
  for (int64_t i = 0; i < n; ++i) {
    const int32_t s = slot_scratch[i];
    const uint64_t key = (uint64_t)ids[i];
    const int32_t u = off[owner_of(key, world)] + set_pos[s & 0x7FFFFFFF];
    reverse[i] = u < unique_cap ? u : 0;
    if (s < 0 && u < unique_cap) unique_ids[u] = (int64_t)key;
  }
}

void rbc_encode_merge(const int64_t* desc, const int64_t* table_idx, int F, int64_t total_nnz, int64_t total_seg,
                      int64_t* ids_out, int32_t* offsets_out) {
  const int64_t* id_ptr = desc; const int64_t* nnz_prefix = desc + (F + 1);
  const int64_t* off_ptr = desc + 2 * (F + 1); const int64_t* seg_prefix = desc + 3 * (F + 1);
  for (int f = 0; f < F; ++f) {
    const int64_t* src = reinterpret_cast<const int64_t*>(id_ptr[f]);
    const int64_t n = nnz_prefix[f + 1] - nnz_prefix[f];
    for (int64_t i = 0; i < n; ++i)
      ids_out[nnz_prefix[f] + i] = (int64_t)(((uint64_t)src[i] & 0x000FFFFFFFFFFFFFull) | ((uint64_t)table_idx[f] << 52));
    if (offsets_out) {
      const int32_t* so = reinterpret_cast<const int32_t*>(off_ptr[f]);
      const int64_t ns = seg_prefix[f + 1] - seg_prefix[f];
      for (int64_t j = 0; j < ns; ++j) offsets_out[seg_prefix[f] + j] = so[j] + (int32_t)nnz_prefix[f];
    }
  }
  if (offsets_out) offsets_out[total_seg] = (int32_t)total_nnz;
}

void rbc_gather_rows(const void* src, const int32_t* rows, int64_t n_max, const int32_t* n_dev, int64_t row_bytes, void* out) {
  const int64_t n = eff_n(n_max, n_dev);
  const char* s = static_cast<const char*>(src); char* o = static_cast<char*>(out);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    if (rows[r] >= 0) std::memcpy(o + r * row_bytes, s + (int64_t)rows[r] * row_bytes, (size_t)row_bytes);
    else std::memset(o + r * row_bytes, 0, (size_t)row_bytes);
  }
}

void rbc_scatter_rows(void* dst, const int32_t* rows, int64_t n, int64_t row_bytes, const void* src, int src_broadcast) {
  const char* s = static_cast<const char*>(src); char* d = static_cast<char*>(dst);
  for (int64_t r = 0; r < n; ++r)
    if (rows[r] >= 0) std::memcpy(d + (int64_t)rows[r] * row_bytes, src_broadcast ? s : s + r * row_bytes, (size_t)row_bytes);
}

void rbc_fill_rows_i64(int64_t* dst, const int32_t* rows, int64_t n, int64_t value) {
  for (int64_t i = 0; i < n; ++i) if (rows[i] >= 0) dst[rows[i]] = value;
}

void rbc_pool_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                      int64_t n_seg, int D, int mode, int perm_b, int perm_f, int perm_off, int perm_total, float* out, int32_t* gsrc,
                      float* gscale) {
  if (perm_f > 0 && perm_total <= 0) { perm_total = perm_f; perm_off = 0; }
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < n_seg; ++s) {
    const int32_t beg = offsets[s], end = offsets[s + 1];
    const int64_t orow = out_row_of(s, perm_b, perm_f, perm_off, perm_total);
    float* o = out + orow * D;
    std::memset(o, 0, sizeof(float) * D);
    float wsum = 0.f;
    for (int32_t i = beg; i < end; ++i) {
      const int32_t u = rev[i]; const int32_t r = rows ? rows[u] : u;
      const float wt = weights ? weights[i] : 1.f;
      wsum += wt;
      if (r >= 0) {
        if (base_dtype == kRowF32) { const float* e = static_cast<const float*>(base) + (int64_t)r * D; for (int c = 0; c < D; ++c) o[c] += wt * e[c]; }
        else for (int c = 0; c < D; ++c) o[c] += wt * rbcpu::row_ld(base, base_dtype, (int64_t)r * D + c);
      }
    }
    float scale = 1.f;
    if (mode == 1) scale = end > beg ? 1.f / (float)(end - beg) : 0.f;
    else if (mode == 2) scale = wsum != 0.f ? 1.f / wsum : 0.f;
    if (scale != 1.f) for (int c = 0; c < D; ++c) o[c] *= scale;
    if (gsrc) for (int32_t i = beg; i < end; ++i) { gsrc[i] = (int32_t)orow; gscale[i] = (weights ? weights[i] : 1.f) * scale; }
  }
}

void rbc_tile_forward(const void* base, int base_dtype, const int32_t* rows, const int32_t* rev, const int32_t* offsets, const float* weights,
                      int64_t n_seg, int D, int tile_len, float* out, int32_t* gsrc, float* gscale) {
#pragma omp parallel for schedule(static)
  for (int64_t s = 0; s < n_seg; ++s) {
    const int32_t beg = offsets[s], end = offsets[s + 1];
    for (int t = 0; t < tile_len; ++t) {
      float* o = out + (s * tile_len + t) * D;
      std::memset(o, 0, sizeof(float) * D);
      if (beg + t < end) {
        const int32_t u = rev[beg + t]; const int32_t r = rows ? rows[u] : u;
        const float wt = weights ? weights[beg + t] : 1.f;
        if (r >= 0) for (int c = 0; c < D; ++c) o[c] = wt * rbcpu::row_ld(base, base_dtype, (int64_t)r * D + c);
        if (gsrc) { gsrc[beg + t] = (int32_t)(s * tile_len + t); gscale[beg + t] = wt; }
      }
    }
    if (gsrc) for (int32_t i = beg + tile_len; i < end; ++i) { gsrc[i] = -1; gscale[i] = 0.f; }
  }
}

void rbc_build_csr(const int32_t* reverse, int64_t n, int32_t* csr_u, int32_t* csr_elem, int32_t* start) {
  if (n <= 0) return;
  int32_t n_unique = 0;
  for (int64_t i = 0; i < n; ++i) n_unique = std::max(n_unique, reverse[i] + 1);
  std::vector<int32_t> cnt(n_unique + 1, 0);
  for (int64_t i = 0; i < n; ++i) cnt[reverse[i] + 1]++;
  for (int32_t u = 0; u < n_unique; ++u) cnt[u + 1] += cnt[u];
  for (int32_t u = 0; u <= n_unique; ++u) start[u] = cnt[u];
  for (int64_t i = 0; i < n; ++i) { const int32_t p = cnt[reverse[i]]++; csr_u[p] = reverse[i]; csr_elem[p] = (int32_t)i; }
}

void rbc_grad_reduce(const float* grad_out, const int32_t* gsrc, const float* gscale, const int32_t* csr_u, const int32_t* csr_elem,
                     const int32_t* start, int64_t n, int D, const int32_t* rows, float* gu, int apply, RbOpt opt) {
  if (n <= 0) return;
  const int32_t n_unique = csr_u[n - 1] + 1;
#pragma omp parallel
  {
    std::vector<float> acc(D);
#pragma omp for schedule(dynamic, 64)
    for (int32_t u = 0; u < n_unique; ++u) {
      std::fill(acc.begin(), acc.end(), 0.f);
      for (int32_t p = start[u]; p < start[u + 1]; ++p) {
        const int32_t e = csr_elem[p]; const int32_t gs = gsrc[e];
        if (gs < 0) continue;
        const float sc = gscale[e]; const float* g = grad_out + (int64_t)gs * D;
        for (int c = 0; c < D; ++c) acc[c] += sc * g[c];
      }
      if (apply) {
        const int32_t row = rows ? rows[u] : u;
        if (row >= 0) for (int c = 0; c < D; ++c) cpu_opt_update(opt, (int64_t)row * D + c, acc[c]);
      } else {
        std::memcpy(gu + (int64_t)u * D, acc.data(), sizeof(float) * D);
      }
    }
  }
}

void rbc_sparse_apply(const int32_t* rows, const float* grads, int64_t n_max, const int32_t* n_dev, int D, RbOpt opt) {
  const int64_t n = eff_n(n_max, n_dev);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    if (rows[r] < 0) continue;
    for (int c = 0; c < D; ++c) cpu_opt_update(opt, (int64_t)rows[r] * D + c, grads[r * D + c]);
  }
}

}  // extern "C"
