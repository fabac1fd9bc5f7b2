// Element access to embedding rows of any storage type on the CPU (see rb::RowDType): loads widen to float, stores round.
#pragma once
#include <c10/util/BFloat16.h>
#include <c10/util/Half.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include "../common/rb_common.cuh"

namespace rbcpu {

inline float row_ld(const void* base, int dtype, int64_t i) {
  switch (dtype) {
    case rb::kRowF16: return static_cast<float>(static_cast<const c10::Half*>(base)[i]);
    case rb::kRowBF16: return static_cast<float>(static_cast<const c10::BFloat16*>(base)[i]);
    case rb::kRowI8: return static_cast<float>(static_cast<const int8_t*>(base)[i]);
    default: return static_cast<const float*>(base)[i];
  }
}

inline void row_st(void* base, int dtype, int64_t i, float v) {
  switch (dtype) {
    case rb::kRowF16: static_cast<c10::Half*>(base)[i] = c10::Half(v); break;
    case rb::kRowBF16: static_cast<c10::BFloat16*>(base)[i] = c10::BFloat16(v); break;
    case rb::kRowI8: static_cast<int8_t*>(base)[i] = (int8_t)std::max(-128.f, std::min(127.f, std::nearbyint(v))); break;
    default: static_cast<float*>(base)[i] = v; break;
  }
}

}  // namespace rbcpu
