/*
 * TinyTorchFusedOps.h - binds libtt_attn.so's B200 versions of the reference's two
 * hand-fused transformer-block operators into TinyTorch's dispatch tables.
 *
 * The reference registers siluMulOpCudaImpl / fusedAddRmsNormOpCudaImpl for
 * CUDA x {Float32, Float16, BFloat16} from registerFusedCuda()
 * (src/Operation/OpFused.h:28-31, src/Operation/OpFusedCuda.cuh:59-101,129-142).
 * registerFusedOpsB200() stores the implementations below into the same table
 * slots (a dispatch table entry is a plain function pointer, src/Tensor/Dispatch.h:32-45),
 * so op::siluMul, op::fusedAddRmsNorm and the function:: wrappers
 * (src/Function/FuncFused.h:31-35) reach the new kernels without any change at the
 * call sites.  Call it once after static initialisation (e.g. first thing in main),
 * because the order of STATIC_CALL initialisers across translation units is not
 * defined.
 *
 * Error convention: a non-zero status is logged with LOGE and then ASSERT(false)
 * fires, like every reference op (src/Utils/Macros.h:34-43).
 */
#pragma once

#include "Operation/OpFused.h"
#include "TinyTorch.h"
#include "Utils/CUDAUtils.h"
#include "tt_fused.h"

namespace tinytorch {
namespace op {

inline void fusedB200Check(int rc) {
  if (rc != TT_ATTN_OK) {
    LOGE("tt_fused: %s %s", tt_attn_strerror(rc), rc == TT_ATTN_ERR_LAUNCH ? tt_attn_last_cuda_error() : "");
    ASSERT(false && "tt_fused call failed");
  }
}

inline Tensor siluMulOpB200Impl(const Tensor& self) {
  ASSERT(self.size(-1) % 2 == 0);
  SizeVector retShape = self.shape();
  retShape.back() /= 2;
  auto ret = Tensor::empty(retShape, self.options().noGrad());
  tt_silu_mul_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(self.dtype());  // enum values are the ABI (src/Tensor/DType.h:20-24)
  p.d = self.size(-1) / 2;
  p.rows = ret.numel() / (p.d > 0 ? p.d : 1);
  p.x = self.dataPtr<>();
  p.out = ret.dataPtr<>();
  p.device = self.device().index;
  p.stream = cuda::getCurrentCUDAStream(self.device().index).stream();
  fusedB200Check(tt_silu_mul(&p));
  return ret;
}

inline void fusedAddRmsNormOpB200Impl(Tensor& input, Tensor& residual, const Tensor& weight, float eps) {
  ASSERT(input.shape() == residual.shape());
  tt_fused_add_rms_norm_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(input.dtype());
  p.dim = input.size(-1);
  p.rows = input.numel() / (p.dim > 0 ? p.dim : 1);
  p.input = input.dataPtr<>();
  p.residual = residual.dataPtr<>();
  p.weight = weight.dataPtr<>();
  p.eps = eps;
  p.device = input.device().index;
  p.stream = cuda::getCurrentCUDAStream(input.device().index).stream();
  fusedB200Check(tt_fused_add_rms_norm(&p));
}

// y = input w^T + bias for CUDA Float16 / BFloat16 tensors whose last dimension is contiguous and whose sizes
// and row strides are multiples of 8: what FuncLinear::forward (src/Function/FuncNNLayer.h:16-18) gets from
// op::matmul(input, weight, false, true, bias).  Returns an undefined Tensor when the kernel does not apply, so
// that the caller falls back to op::matmul.
inline Tensor linearOpB200(const Tensor& input, const Tensor& weight, const Tensor& bias) {
  if (!input.device().isCuda() || (input.dtype() != DType::Float16 && input.dtype() != DType::BFloat16)) return {};
  if (weight.dim() != 2 || weight.dtype() != input.dtype() || input.dim() < 1) return {};
  const int64_t K = input.size(-1), N = weight.size(0);
  if (weight.size(1) != K || K % 8 != 0 || N % 8 != 0) return {};
  if (bias.defined() && (bias.dim() != 1 || bias.size(0) != N || bias.dtype() != input.dtype())) return {};
  SizeVector retShape = input.shape();
  retShape.back() = N;
  auto ret = Tensor::empty(retShape, input.options().noGrad());
  tt_linear_params p{};
  p.struct_size = sizeof(p);
  p.dtype = static_cast<int32_t>(input.dtype());
  p.K = K, p.N = N, p.M = input.numel() / K;  // tensors are dense: leading dimensions flatten into rows
  p.x = input.dataPtr<>(), p.w = weight.dataPtr<>(), p.y = ret.dataPtr<>();
  p.bias = bias.defined() ? bias.dataPtr<>() : nullptr;
  p.device = input.device().index;
  p.stream = cuda::getCurrentCUDAStream(input.device().index).stream();
  fusedB200Check(tt_linear(&p));
  return ret;
}

inline void registerFusedOpsB200() {
  const std::vector<DispatchDType> floats = {DispatchDType::Float32, DispatchDType::Float16, DispatchDType::BFloat16};
  REGISTER_OP_IMPL_MULTI(siluMul, {DispatchDevice::CUDA}, floats, &siluMulOpB200Impl);
  REGISTER_OP_IMPL_MULTI(fusedAddRmsNorm, {DispatchDevice::CUDA}, floats, &fusedAddRmsNormOpB200Impl);
}

}  // namespace op
}  // namespace tinytorch
