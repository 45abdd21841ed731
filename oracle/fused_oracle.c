/*
 * TEST INFRASTRUCTURE ONLY - never linked or loaded by the product path.
 *
 * Plain-C restatement of the reference's CPU fp32 implementations of its two fused
 * transformer-block operators, same loop order and the same float operations:
 *   oracle_silu_mul            siluMulOpCpuImpl          src/Operation/OpFusedCpu.h:14-39
 *                              with OpCpuSilu::apply      src/Operation/OpElemWiseCpu.h:123-128
 *   oracle_fused_add_rms_norm  fusedAddRmsNormOpCpuImpl  src/Operation/OpFusedCpu.h:42-72
 *   oracle_linear              function::linear = op::matmul(input, weight, false, true, bias)
 *                              src/Function/FuncNNLayer.h:14-19 -> gemmCpuImpl (no BLAS build)
 *                              src/Operation/OpLinalgCpu.h:118-151; pinned by the reference's
 *                              own known answer test/test_function.cpp:234-248
 * Pinned against the reference's own code (oracle/_ref, ref_silu_mul /
 * ref_fused_add_rms_norm) and the committed fixture tests/golden/ref_seeded_fused.npz;
 * the reference's test suite holds no vector for these two operators.
 */
#include <math.h>
#include <stdint.h>

/* x [rows, last] -> out [rows, last/2]: silu(gate) * up, gate = first half of a row. */
void oracle_silu_mul(const float* x, int64_t rows, int64_t last, float* out) {
  const int64_t half = last / 2;
  for (int64_t i = 0; i < rows; i++) {
    const float* in = x + i * last;
    float* o = out + i * half;
    for (int64_t j = 0; j < half; j++) {
      const float g = in[j];
      const float s = g / (1.0f + expf(-g));
      o[j] = s * in[j + half];
    }
  }
}

/* In place: residual <- input + residual; input <- residual * invRms * weight. */
void oracle_fused_add_rms_norm(float* input, float* residual, const float* weight, int64_t rows, int64_t dim,
                               float eps) {
  for (int64_t row = 0; row < rows; row++) {
    float* in = input + row * dim;
    float* res = residual + row * dim;
    float sum_sq = 0.f;
    for (int64_t i = 0; i < dim; i++) {
      const float r = in[i] + res[i];
      res[i] = r;
      sum_sq += r * r;
    }
    const float inv_rms = 1.f / sqrtf(sum_sq / (float)dim + eps);
    for (int64_t i = 0; i < dim; i++) in[i] = res[i] * inv_rms * weight[i];
  }
}

/* y[M,N] = x[M,K] w[N,K]^T + bias[N]: C is pre-filled with the bias (or zero), then
 * accumulated in the reference's i-p-j order, one float multiply-add at a time. */
void oracle_linear(const float* x, const float* w, const float* bias, int64_t M, int64_t N, int64_t K, float* y) {
  for (int64_t i = 0; i < M; i++)
    for (int64_t j = 0; j < N; j++) y[i * N + j] = bias ? bias[j] : 0.f;
  for (int64_t i = 0; i < M; i++) {
    for (int64_t p = 0; p < K; p++) {
      const float a = x[i * K + p];
      for (int64_t j = 0; j < N; j++) y[i * N + j] += a * w[j * K + p];
    }
  }
}
