// GELU (tanh form) and its derivative, shared by the elementwise kernels and the GEMM epilogue.
//
//   gelu(x)  = 0.5 x (1 + tanh(u)) = x * sigmoid(2u),   u = k (x + c x^3),  k = sqrt(2/pi), c = 0.044715
//   gelu'(x) = s + x s (1 - s) * 2 du/dx,               s = sigmoid(2u),    du/dx = k (1 + 3 c x^2)
//
// The forward form uses the hardware tanh (relative error about 2^-11, far inside one bf16
// rounding of the result).  The derivative multiplies (1 - s) by a factor that grows with x,
// so it takes the sigmoid from ex2 and rcp (a few ulp each) instead: about a dozen FMA-pipe
// instructions and two special-function ones per element.
#pragma once

namespace pccl {

__device__ __forceinline__ float tanh_hw(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_hw(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_hw(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * x * (1.f + 0.044715f * x * x);
  return 0.5f * x * (1.f + tanh_hw(u));
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
  x = fminf(fmaxf(x, -20.f), 20.f);                          // beyond that the derivative is 0 or 1 to fp32 precision
  constexpr float k2 = 2.f * 0.7978845608028654f;            // 2k
  constexpr float log2e = 1.4426950408889634f;
  const float x2 = x * x;
  // exp(-2u) = 2^(x * (A + B x^2)); overflow gives s = 0, underflow s = 1
  const float e = ex2_hw(x * fmaf(x2, -k2 * 0.044715f * log2e, -k2 * log2e));
  const float s = rcp_hw(1.f + e);
  const float q = fmaf(x2, 3.f * 0.044715f * k2, k2);        // 2 du/dx
  return s * fmaf(x * (1.f - s), q, 1.f);
}

}  // namespace pccl
