// Row-wise sparse optimizer updates (Adam / AdamW family, Adagrad, SGD) on one float4 (or one element) of a row.
// Math of the reference's csrc/ops/block_apply_adamw_op_kernel.cu:11-22,109-120; shared by the fused backward kernels
// (kernels/sparse_ops.cu) and the owner-side update of the peer-memory exchange (kernels/comm.cu).
#pragma once
#include "rb_common.cuh"
#include "../kernels/rb_kernels.h"

namespace rb {

// The row (o.w, elements of type T) is read and written in its storage type; moments and arithmetic are fp32.
template <typename T>
__device__ __forceinline__ void opt_update_pre_f4(const RbOpt& o, int64_t off, float4 g, float4 w, float4 m, float4 v);

template <typename T>
__device__ __forceinline__ void opt_update_f4(const RbOpt& o, int64_t off, float4 g) {
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 w = RowIO<T>::ld4(static_cast<const T*>(o.w) + off);
  const float4 m = o.kind != RB_OPT_SGD ? ld_f4(o.s1 + off) : zero;
  const float4 v = o.kind == RB_OPT_ADAM ? ld_f4(o.s2 + off) : zero;
  opt_update_pre_f4<T>(o, off, g, w, m, v);
}

// Same update with the row's state already in registers (requested when the row's segment started).
template <typename T>
__device__ __forceinline__ void opt_update_pre_f4(const RbOpt& o, int64_t off, float4 g, float4 w, float4 m, float4 v) {
  const float gs = o.grad_scale;
  g.x *= gs; g.y *= gs; g.z *= gs; g.w *= gs;
  if (o.kind == RB_OPT_ADAM) {
    const float b1 = o.beta1, b2 = o.beta2, c1 = 1.f - o.beta1, c2 = 1.f - o.beta2;
    m.x = b1 * m.x + c1 * g.x; m.y = b1 * m.y + c1 * g.y; m.z = b1 * m.z + c1 * g.z; m.w = b1 * m.w + c1 * g.w;
    v.x = b2 * v.x + c2 * g.x * g.x; v.y = b2 * v.y + c2 * g.y * g.y; v.z = b2 * v.z + c2 * g.z * g.z; v.w = b2 * v.w + c2 * g.w * g.w;
    w.x = w.x * o.decay + o.alpha * m.x / (sqrtf(v.x) + o.eps);
    w.y = w.y * o.decay + o.alpha * m.y / (sqrtf(v.y) + o.eps);
    w.z = w.z * o.decay + o.alpha * m.z / (sqrtf(v.z) + o.eps);
    w.w = w.w * o.decay + o.alpha * m.w / (sqrtf(v.w) + o.eps);
    st_f4(o.s1 + off, m); st_f4(o.s2 + off, v);
  } else if (o.kind == RB_OPT_ADAGRAD) {
    m.x += g.x * g.x; m.y += g.y * g.y; m.z += g.z * g.z; m.w += g.w * g.w;
    w.x = w.x * o.decay - o.lr * g.x / (sqrtf(m.x) + o.eps);
    w.y = w.y * o.decay - o.lr * g.y / (sqrtf(m.y) + o.eps);
    w.z = w.z * o.decay - o.lr * g.z / (sqrtf(m.z) + o.eps);
    w.w = w.w * o.decay - o.lr * g.w / (sqrtf(m.w) + o.eps);
    st_f4(o.s1 + off, m);
  } else {
    w.x = w.x * o.decay - o.lr * g.x; w.y = w.y * o.decay - o.lr * g.y;
    w.z = w.z * o.decay - o.lr * g.z; w.w = w.w * o.decay - o.lr * g.w;
  }
  RowIO<T>::st4(static_cast<T*>(o.w) + off, w);
}

template <typename T>
__device__ __forceinline__ void opt_update_f1(const RbOpt& o, int64_t off, float g) {
  g *= o.grad_scale;
  T* wp = static_cast<T*>(o.w) + off;
  float w = RowIO<T>::ld1(wp);
  if (o.kind == RB_OPT_ADAM) {
    const float m = o.beta1 * o.s1[off] + (1.f - o.beta1) * g;
    const float v = o.beta2 * o.s2[off] + (1.f - o.beta2) * g * g;
    o.s1[off] = m; o.s2[off] = v;
    w = w * o.decay + o.alpha * m / (sqrtf(v) + o.eps);
  } else if (o.kind == RB_OPT_ADAGRAD) {
    const float a = o.s1[off] + g * g;
    o.s1[off] = a;
    w = w * o.decay - o.lr * g / (sqrtf(a) + o.eps);
  } else {
    w = w * o.decay - o.lr * g;
  }
  RowIO<T>::st1(wp, w);
}

}  // namespace rb
