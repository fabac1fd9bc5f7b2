// C launch API of the dense-tower kernels (tensor-core GEMM, interactions, element-wise helpers).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// D[MM, NN] = act(A * B^T + bias (+ beta_src)); A is [MM][KK] (a_mn = 0, pitch lda) or [KK][MM] (a_mn = 1); B is [NN][KK]
// (b_mn = 0) or [KK][NN] (b_mn = 1); bf16 operands, fp32 accumulation, bf16 or fp32 output with row pitch ldo.
// beta_src (nullable, fp32, same layout as the output) is added before the activation (gradient accumulation).
// Returns 0 on success; 1 = operand alignment unsuitable for TMA, 2 = tensor-map encode failed, >2 = launch error.
// splits > 1 (fp32 output without activation only): the reduction is split over gridDim.z CTAs that accumulate into `out`
// with fp32 reductions; `out` must then be zero (or hold the value to accumulate onto) on entry.
int rb_gemm_bf16(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo, int out_fp32,
                 const float* bias, const float* beta_src, int MM, int NN, int KK, int relu, int splits, int64_t* status,
                 cudaStream_t st);
// Optional extra epilogue work, applied after bias / residual / ReLU:
//   mask_src  bf16 [MM, mask_ld]: D[m, n] is set to zero where mask_src[m, n] <= 0 (the ReLU backward of the layer below, when D
//             is the gradient of that layer's output);
//   colsum    fp32 [NN]: the column sums of the final D are ADDED to it (the bias gradient of the layer below); zero it first.
typedef struct {
  const void* mask_src;
  int64_t mask_ld;
  float* colsum;
} RbGemmEpilogue;
int rb_gemm_bf16_ex(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo, int out_fp32,
                    const float* bias, const float* beta_src, const RbGemmEpilogue* epi, int MM, int NN, int KK, int relu, int splits,
                    int64_t* status, cudaStream_t st);
// The same GEMM on pairs of SMs (256 x 256 tiles, tcgen05 cta_group::2; gemm_tcgen05_2cta.cu). Returns 7 when the problem does not
// suit it (fewer than 192 rows or columns, output not TMA-storable); rb_gemm_bf16 tries it first when RECIS_GEMM_2CTA allows.
int rb_gemm_bf16_pair(const void* a, int64_t lda, int a_mn, const void* b, int64_t ldb, int b_mn, void* out, int64_t ldo, int out_fp32,
                      const float* bias, const float* beta_src, const RbGemmEpilogue* epi, int MM, int NN, int KK, int relu, int splits,
                      int64_t* status, cudaStream_t st);
int rb_gemm_splits(int MM, int NN, int KK);
// A (cached) TMA descriptor of a 2-D bf16 or fp32 matrix [rows][cols] with row pitch ld elements, box {box_cols, box_rows}, 128-byte
// swizzle, written to out_map (a CUtensorMap, 128 bytes). 0 on success, 1 = base or pitch not 16-byte aligned, 2 = encode failed.
int rb_tensor_map_2d(void* out_map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows, int fp32);   // heuristic split count for a weight-gradient shaped problem

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
extern "C" {
#endif
// x: bf16 [B, D]; cube: fp32 [B, F, D]; out: bf16 [B, out_ld] = [x, lower triangle of Z Z^T, zero pad]. Returns 0 on success.
int rb_dot_interaction_fwd(const void* x, const float* cube, int B, int F, int D, int out_ld, void* out, cudaStream_t st);
int rb_dot_interaction_bwd(const void* x, const float* cube, const void* dout, int B, int F, int D, int out_ld, float* dx, float* dcube,
                           cudaStream_t st);
// Tensor-core (tcgen05) versions for at most 31 fields and D in {64, 128}. Return 0 = ran, 1 = shape outside their range
// (call the SIMT version instead), > 1 = launch error. A bounded wait that ran out sets the timeout bit in *status.
int rb_dot_interaction_tc_fwd(const void* x, const float* cube, int B, int F, int D, int out_ld, void* out, int64_t* status,
                              cudaStream_t st);
int rb_dot_interaction_tc_bwd(const void* x, const float* cube, const void* dout, int B, int F, int D, int out_ld, float* dx,
                              float* dcube, int64_t* status, cudaStream_t st);
// Ragged multi-head self-attention forward, head width 64 (attention_tcgen05.cu). qkv: bf16 [T, 3 * H * 64] packed, offsets:
// int32 [B + 1] (device), out: bf16 [T, H * 64], lse2: fp32 [T, H] or null. 0 = launched, 1 = unsuitable arguments, > 1 = error.
int rb_ragged_attention_fwd(const void* qkv, const int32_t* offsets, int64_t T, int B, int H, int max_len, float scale, void* out,
                            float* lse2, int64_t* status, cudaStream_t st);
// Backward: out / d_out bf16 [T, H * 64], lse2 from the forward, delta fp32 [T, H] scratch, dqkv fp32 [T, 3 * H * 64] zeroed.
int rb_ragged_attention_bwd(const void* qkv, const void* out, const void* d_out, const float* lse2, float* delta, const int32_t* offsets,
                            int64_t T, int B, int H, int max_len, float scale, float* dqkv, int64_t* status, cudaStream_t st);
void rb_fm_fwd(const float* cube, int B, int F, int D, float* out, cudaStream_t st);
void rb_fm_bwd(const float* cube, const float* gout, int B, int F, int D, float* dcube, cudaStream_t st);
// dy = relu ? dout * (y > 0) : dout (bf16, may be null to skip the store); db[n] += column sums of dy (fp32, may be null)
void rb_relu_bwd_bias(const void* y, const void* dout, int M, int N, int relu, void* dy, float* db, cudaStream_t st);
void rb_cast_pad_bf16(const float* src, int rows, int cols, int src_ld, void* dst, int rows_p, int cols_p, cudaStream_t st);

// Multi-tensor dense Adam: one launch updates up to RB_DENSE_ADAM_MAX fp32 tensors (gridDim.y = tensor).
//   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  w = w * decay - step_size * m / (sqrt(v) * inv_sqrt_bc2 + eps)
// TensorFlow-style AdamW (epsilon outside the bias correction): step_size = lr sqrt(1-b2^t)/(1-b1^t), inv_sqrt_bc2 = 1,
// decay = 1 - wd. PyTorch Adam/AdamW: step_size = lr/(1-b1^t), inv_sqrt_bc2 = 1/sqrt(1-b2^t), decay = 1 (Adam, whose L2
// term is `l2` added to g) or 1 - lr wd (AdamW). Also writes the updated weights as bf16 when w_bf16[i] is not null.
#define RB_DENSE_ADAM_MAX 24
typedef struct RbDenseAdamArgs {
  float* w[RB_DENSE_ADAM_MAX];
  const float* g[RB_DENSE_ADAM_MAX];
  float* m[RB_DENSE_ADAM_MAX];
  float* v[RB_DENSE_ADAM_MAX];
  void* w_bf16[RB_DENSE_ADAM_MAX];
  int32_t cols[RB_DENSE_ADAM_MAX];       // columns of the weight (its last dimension); used with bf16_ld
  int32_t bf16_ld[RB_DENSE_ADAM_MAX];    // row pitch of the bf16 copy in elements (a copy padded for TMA); 0 or == cols: same layout as w
  int64_t n[RB_DENSE_ADAM_MAX];
  int count;
} RbDenseAdamArgs;
void rb_dense_adam(const RbDenseAdamArgs* args, float beta1, float beta2, float eps, float decay, float step_size, float inv_sqrt_bc2,
                   float l2, cudaStream_t st);
// ---- seq_ops.cu: target attention over packed sequences (one query per sequence), forward and backward, one pass each.
// x: fp32 [T, H] packed tokens, q: fp32 [B, H], offsets: int32 [B + 1]; interest: fp32 [B, H]; lse: fp32 [B] (log-sum-exp of the
// scaled scores, kept for the backward pass). Return 1 when H is outside the kernels' range (multiple of 4, at most 1024).
int rb_target_attention_fwd(const float* x, const float* q, const int32_t* offsets, int B, int H, float scale, float* interest,
                            float* lse, cudaStream_t st);
int rb_target_attention_bwd(const float* x, const float* q, const int32_t* offsets, const float* interest, const float* lse,
                            const float* d_interest, int B, int H, float scale, float* dx, float* dq, cudaStream_t st);

// ---- norm_ops.cu: LayerNorm over the last dimension of fp32 [rows, H] (H a multiple of 4, at most 1024; otherwise 1 is returned).
// forward writes y as bf16 (y_bf16 != 0) or fp32 and stats[rows][2] = (mean, rstd); backward takes dy as bf16 or fp32 and ADDS the
// weight gradients to dgamma / dbeta (zero them first).
int rb_layer_norm_fwd(const float* x, const float* gamma, const float* beta, int64_t rows, int H, float eps, void* y, int y_bf16,
                      float* stats, cudaStream_t st);
int rb_layer_norm_bwd(const void* dy, int dy_bf16, const float* x, const float* stats, const float* gamma, int64_t rows, int H, float* dx,
                      float* dgamma, float* dbeta, cudaStream_t st);
// ReLU backward + bias gradient with 16-byte accesses; returns 1 when the width does not suit it (not a multiple of 8, or neither
// a power of two below 256 nor a multiple of 256), and the caller falls back to rb_relu_bwd_bias.
int rb_relu_bwd_bias_vec(const void* y, const void* dout, int64_t M, int N, int relu, void* dy, float* db, cudaStream_t st);

#ifdef __cplusplus
}
#endif
