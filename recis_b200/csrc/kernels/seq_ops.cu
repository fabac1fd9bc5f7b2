// Target attention over packed (ragged) sequences, sm_100a: one query per sequence, softmax over the sequence's tokens,
// weighted sum of the tokens - forward and backward, each ONE pass over the tokens.
//
//   s_t = scale * <x_t, q_b>,  a = softmax_t(s),  interest_b = sum_t a_t x_t            (t over the tokens of sequence b)
//
// The DIN-style interest extraction of a user-behaviour model. Written with tensor ops it is a chain of gather / multiply /
// segment-max / exp / segment-sum / divide / scatter-add passes, each of which re-reads the [tokens, hidden] activations;
// here one CTA walks a sequence once with an online softmax (running maximum, running sum, rescaled accumulator), so the
// activations cross HBM once in the forward pass and twice (read x, write dx) in the backward pass.
// Layout: a warp owns tokens w, w + W, ... of its sequence; lane l owns columns l*4 + k*128 (float4 per 128 columns), so a
// token row is read with fully coalesced 16-byte loads; hidden must be a multiple of 4 and at most 1024.
// The reference has no such op (its sequence example pools with padded tensor ops, examples/seq2seq/seq2seq_model.py).
#include "../common/rb_common.cuh"
#include "../common/rb_launch.h"
#include "rb_dense.h"

namespace {

constexpr int kWarps = 8;
constexpr int kMaxQuads = 8;      // float4 slots per lane: hidden <= 8 * 128

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int NQ>
__global__ void __launch_bounds__(kWarps * 32)
target_attention_fwd_kernel(const float* __restrict__ x, const float* __restrict__ q, const int32_t* __restrict__ offsets, int H, float scale,
                            float* __restrict__ interest, float* __restrict__ lse) {
  __shared__ float sm_m[kWarps], sm_l[kWarps];
  __shared__ float sm_acc[kWarps][NQ * 128];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int beg = offsets[b], end = offsets[b + 1];
  float4 qv[NQ], acc[NQ];
#pragma unroll
  for (int k = 0; k < NQ; ++k) {
    const int c = lane * 4 + k * 128;
    qv[k] = c < H ? rb::ld_f4(q + (int64_t)b * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -INFINITY, l = 0.f;
  for (int t = beg + warp; t < end; t += kWarps) {
    float4 xv[NQ];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NQ; ++k) {
      const int c = lane * 4 + k * 128;
      xv[k] = c < H ? rb::ld_f4(x + (int64_t)t * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      dot += xv[k].x * qv[k].x + xv[k].y * qv[k].y + xv[k].z * qv[k].z + xv[k].w * qv[k].w;
    }
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float alpha = m == -INFINITY ? 0.f : __expf(m - m_new);
    const float p = __expf(s - m_new);
    l = l * alpha + p;
#pragma unroll
    for (int k = 0; k < NQ; ++k) {
      acc[k].x = acc[k].x * alpha + p * xv[k].x; acc[k].y = acc[k].y * alpha + p * xv[k].y;
      acc[k].z = acc[k].z * alpha + p * xv[k].z; acc[k].w = acc[k].w * alpha + p * xv[k].w;
    }
    m = m_new;
  }
  // combine the warps' partial softmaxes
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int k = 0; k < NQ; ++k) rb::st_f4(&sm_acc[warp][lane * 4 + k * 128], acc[k]);
  __syncthreads();
  float gm = -INFINITY;
  for (int w = 0; w < kWarps; ++w) gm = fmaxf(gm, sm_m[w]);
  float gl = 0.f;
  for (int w = 0; w < kWarps; ++w) gl += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * __expf(sm_m[w] - gm);
  const float inv = gl > 0.f ? 1.f / gl : 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < kWarps; ++w) if (sm_m[w] != -INFINITY) v += sm_acc[w][c] * __expf(sm_m[w] - gm);
    interest[(int64_t)b * H + c] = v * inv;
  }
  if (threadIdx.x == 0) lse[b] = gl > 0.f ? gm + __logf(gl) : 0.f;
}

// d a_t = <dI_b, x_t>;  d s_t = a_t (d a_t - <dI_b, interest_b>);  dx_t = a_t dI_b + scale d s_t q_b;  dq_b = scale sum_t d s_t x_t
template <int NQ>
__global__ void __launch_bounds__(kWarps * 32)
target_attention_bwd_kernel(const float* __restrict__ x, const float* __restrict__ q, const int32_t* __restrict__ offsets,
                            const float* __restrict__ interest, const float* __restrict__ lse, const float* __restrict__ d_interest, int H,
                            float scale, float* __restrict__ dx, float* __restrict__ dq) {
  __shared__ float sm_dq[kWarps][NQ * 128];
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int beg = offsets[b], end = offsets[b + 1];
  float4 qv[NQ], gv[NQ], dqa[NQ];
  float delta = 0.f;
#pragma unroll
  for (int k = 0; k < NQ; ++k) {
    const int c = lane * 4 + k * 128;
    const bool on = c < H;
    qv[k] = on ? rb::ld_f4(q + (int64_t)b * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    gv[k] = on ? rb::ld_f4(d_interest + (int64_t)b * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 iv = on ? rb::ld_f4(interest + (int64_t)b * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    delta += gv[k].x * iv.x + gv[k].y * iv.y + gv[k].z * iv.z + gv[k].w * iv.w;
    dqa[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  delta = warp_sum(delta);
  const float lse_b = lse[b];
  for (int t = beg + warp; t < end; t += kWarps) {
    float4 xv[NQ];
    float dot_q = 0.f, dot_g = 0.f;
#pragma unroll
    for (int k = 0; k < NQ; ++k) {
      const int c = lane * 4 + k * 128;
      xv[k] = c < H ? rb::ld_f4(x + (int64_t)t * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
      dot_q += xv[k].x * qv[k].x + xv[k].y * qv[k].y + xv[k].z * qv[k].z + xv[k].w * qv[k].w;
      dot_g += xv[k].x * gv[k].x + xv[k].y * gv[k].y + xv[k].z * gv[k].z + xv[k].w * gv[k].w;
    }
    dot_q = warp_sum(dot_q); dot_g = warp_sum(dot_g);
    const float a = __expf(dot_q * scale - lse_b);
    const float ds = a * (dot_g - delta) * scale;
#pragma unroll
    for (int k = 0; k < NQ; ++k) {
      const int c = lane * 4 + k * 128;
      if (c < H)
        rb::st_f4(dx + (int64_t)t * H + c, make_float4(a * gv[k].x + ds * qv[k].x, a * gv[k].y + ds * qv[k].y, a * gv[k].z + ds * qv[k].z,
                                                      a * gv[k].w + ds * qv[k].w));
      dqa[k].x += ds * xv[k].x; dqa[k].y += ds * xv[k].y; dqa[k].z += ds * xv[k].z; dqa[k].w += ds * xv[k].w;
    }
  }
#pragma unroll
  for (int k = 0; k < NQ; ++k) rb::st_f4(&sm_dq[warp][lane * 4 + k * 128], dqa[k]);
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < kWarps; ++w) v += sm_dq[w][c];
    dq[(int64_t)b * H + c] = v;
  }
}

template <typename F>
bool dispatch_quads(int H, F&& f) {
  if (H % 4 != 0 || H > kMaxQuads * 128) return false;
  const int nq = (H + 127) / 128;
  if (nq <= 1) f(std::integral_constant<int, 1>{});
  else if (nq <= 2) f(std::integral_constant<int, 2>{});
  else if (nq <= 4) f(std::integral_constant<int, 4>{});
  else f(std::integral_constant<int, 8>{});
  return true;
}

}  // namespace

// x: fp32 [T, H] packed tokens, q: fp32 [B, H], offsets: int32 [B + 1]; interest: fp32 [B, H], lse: fp32 [B]. Returns 1 when H
// is outside the kernel's range (not a multiple of 4 or above 1024).
extern "C" int rb_target_attention_fwd(const float* x, const float* q, const int32_t* offsets, int B, int H, float scale, float* interest,
                                       float* lse, cudaStream_t st) {
  if (B <= 0) return 0;
  const bool ok = dispatch_quads(H, [&](auto nq) {
    constexpr int NQ = decltype(nq)::value;
    target_attention_fwd_kernel<NQ><<<B, kWarps * 32, 0, st>>>(x, q, offsets, H, scale, interest, lse);
  });
  if (ok) rb::note_launch();
  return ok ? 0 : 1;
}

extern "C" int rb_target_attention_bwd(const float* x, const float* q, const int32_t* offsets, const float* interest, const float* lse,
                                       const float* d_interest, int B, int H, float scale, float* dx, float* dq, cudaStream_t st) {
  if (B <= 0) return 0;
  const bool ok = dispatch_quads(H, [&](auto nq) {
    constexpr int NQ = decltype(nq)::value;
    target_attention_bwd_kernel<NQ><<<B, kWarps * 32, 0, st>>>(x, q, offsets, interest, lse, d_interest, H, scale, dx, dq);
  });
  if (ok) rb::note_launch();
  return ok ? 0 : 1;
}
