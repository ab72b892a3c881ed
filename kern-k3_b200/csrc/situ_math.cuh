// SiTU activation of the shared-expert landing, act = (4 tanh(g / 4) sigmoid(g)) * (25 tanh(u / 25)), in two
// forms: the reference's formula written out operation for operation, and the cheaper value-identical form
// the kernels of this library use.  A header of its own so that a test-only probe can evaluate both forms on
// every bf16 input without being part of the shipped library.
#pragma once

namespace k3g {

__device__ __forceinline__ float mufu_tanh(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// The reference's formula, operation for operation (source/k3_land_fused.cu:88-92).
__device__ __forceinline__ float situ_reference_form(float g, float u) {
  const float a = 4.0f * mufu_tanh(g * 0.25f);
  const float s = __frcp_rn(1.0f + __expf(-g));
  const float c = 25.0f * mufu_tanh(u * 0.04f);
  return (a * s) * c;
}
// The same function with fewer instructions; every step below is value-preserving:
//  - __expf(-g) is ex2.approx(-g * log2 e); flushing a subnormal exponential to zero cannot change 1 + e;
//  - x = 1 + e >= 1, where one Newton step on rcp.approx is the correctly rounded reciprocal as long as the
//    result is a normal number (x <= 2^126); larger x (g < -87) takes the full-range reciprocal;
//  - scaling by 4 is exact and commutes with rounding, so (4 t s) c = (t s)(4 c) and 4 (25 th) = 100 th.
// The probe built from tests/native/situ_probe.cu compares the two on every bf16 value of g and of u.
__device__ __forceinline__ float situ_value(float g, float u) {
  const float t = mufu_tanh(g * 0.25f);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(g, -1.4426950408889634f)));
  const float x = 1.0f + e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  r = __fmaf_rn(r, __fmaf_rn(-x, r, 1.0f), r);
  if (x > 0x1p126f) r = __frcp_rn(x);
  const float c4 = 100.0f * mufu_tanh(u * 0.04f);
  return (t * r) * c4;
}
}  // namespace k3g
