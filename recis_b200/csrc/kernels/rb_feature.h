// C launch API of the fused feature-engine kernels (feature_ops.cu). `desc` is a device-resident int64 table with
// T+1 columns per row; the row meaning is documented next to each kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
void rb_fused_hash(const int64_t* desc, int T, int64_t total, int kind, int64_t* out, cudaStream_t st);
void rb_fused_bucketize(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st);
void rb_fused_mod(const int64_t* desc, int T, int64_t total, int64_t* out, cudaStream_t st);
void rb_fused_multi_hash(const int64_t* desc, int T, int64_t total, int kmax, int64_t* out, cudaStream_t st);
#ifdef __cplusplus
}
#endif
