/*
 * tt_fused.h - C ABI of the operators that sit either side of attention in a
 * transformer block, exported by libtt_attn.so for NVIDIA B200 (sm_100a): the two
 * fused element-wise / row operators (HBM-bound streaming kernels) and the
 * projection y = x w^T + bias (tensor cores).
 *
 *   tt_fused_add_rms_norm  replaces fusedAddRmsNormOpCudaImpl
 *                          (src/Operation/OpFusedCuda.cuh:103-142; CPU form
 *                          src/Operation/OpFusedCpu.h:42-72)
 *   tt_silu_mul            replaces siluMulOpCudaImpl
 *                          (src/Operation/OpFusedCuda.cuh:16-101; CPU form
 *                          src/Operation/OpFusedCpu.h:14-39)
 *   tt_linear              replaces the library gemm behind function::linear =
 *                          op::matmul(input, weight, false, true, bias) for 16-bit
 *                          tensors (src/Function/FuncNNLayer.h:14-19,
 *                          src/Operation/OpLinalg.cpp:243-269,
 *                          src/Operation/OpLinalgCuda.cuh:141-215; CPU form
 *                          src/Operation/OpLinalgCpu.h:118-151)
 *
 * dtype uses the reference's enum values (src/Tensor/DType.h:20-24): 0 = Float32,
 * 1 = Float16, 2 = BFloat16.  Arithmetic is fp32 with one rounding to the tensor
 * dtype per stored value, as in the reference's CUDA kernels.  Tensors are dense and
 * row-major with the normalised / gated dimension innermost.  Work is enqueued on
 * `stream` of `device`; nothing synchronises the host or allocates.  Return value: 0
 * or a negative tt_attn_status (tt_attn.h).
 */
#ifndef TT_FUSED_H_
#define TT_FUSED_H_

#include "tt_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* In place, exactly as op::fusedAddRmsNorm(input, residual, weight, eps):
 *   residual <- T(input + residual)                         (fp32 add, rounded to T)
 *   input    <- T(residual * rsqrt(mean(r^2) + eps) * weight)
 * where the mean runs over the unrounded fp32 sums r and the product uses the
 * rounded residual (src/Operation/OpFusedCuda.cuh:110-127). */
typedef struct tt_fused_add_rms_norm_params {
  uint32_t struct_size;
  int32_t dtype;
  int64_t rows, dim;
  void* input;        /* [rows, dim], read and overwritten */
  void* residual;     /* [rows, dim], read and overwritten */
  const void* weight; /* [dim] */
  float eps;
  int32_t device;
  void* stream;
} tt_fused_add_rms_norm_params;

/* out[r, j] = silu(x[r, j]) * x[r, d + j] for x [rows, 2d], silu(g) = g / (1 + exp(-g))
 * (src/Operation/OpFusedCuda.cuh:38-42). */
typedef struct tt_silu_mul_params {
  uint32_t struct_size;
  int32_t dtype;
  int64_t rows, d; /* d = half of x's last dimension */
  const void* x;   /* [rows, 2d] */
  void* out;       /* [rows, d] */
  int32_t device;
  void* stream;
} tt_silu_mul_params;

/* y[M,N] = x[M,K] w[N,K]^T + bias[N] (bias may be NULL), Float16 / BFloat16 only (Float32
 * stays on the library gemm: TT_ATTN_ERR_DTYPE).  fp32 accumulation, the bias is added in
 * fp32 before the single rounding to the tensor dtype.  ldx / ldw / ldy are the row strides
 * in elements (0 = dense); K, N and the strides must be multiples of 8 and the pointers
 * 16-byte aligned (TT_ATTN_ERR_ALIGN otherwise).  `status` (optional device word) receives a
 * non-zero value if a bounded device-side wait expired. */
typedef struct tt_linear_params {
  uint32_t struct_size;
  int32_t dtype;
  int64_t M, N, K;
  const void* x;    /* [M, K] */
  const void* w;    /* [N, K] */
  const void* bias; /* [N] or NULL */
  void* y;          /* [M, N] */
  int64_t ldx, ldw, ldy;
  int32_t device;
  void* stream;
  int32_t* status;
} tt_linear_params;

TT_ATTN_API int tt_linear(const tt_linear_params* p);
TT_ATTN_API int tt_fused_add_rms_norm(const tt_fused_add_rms_norm_params* p);
TT_ATTN_API int tt_silu_mul(const tt_silu_mul_params* p);

#ifdef __cplusplus
}
#endif
#endif /* TT_FUSED_H_ */
