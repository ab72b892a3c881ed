// TEST INFRASTRUCTURE — CPU oracle numerics.  Nothing under oracle/ is part of the
// shipped library; only the test-suite, the smoke check and the benchmark's CPU
// baseline may build or call it.
//
// Software restatement of the device primitives the K3 prefill glue kernels of
// xiaguan/kern-k3 rely on, written independently of the CUDA intrinsics so that a
// disagreement between this file and the GPU path is a real finding:
//
//   * bf16 <-> f32: round-to-nearest-even, the meaning of __float2bfloat16 /
//     __floats2bfloat162_rn used at every landing point of the reference
//     (e.g. source/k3_residual_v2.cu:84, source/k3_mla_prep_v2.cu:76-79).
//   * E4M3 encode: round-to-nearest-even with saturation to +-448 and NaN -> 0x7f,
//     the meaning of __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)
//     (source/k3_moe_prefill_v4.cu:136, source/k3_quant_fp8_pair_v2.cu:76-83).
//   * UE8M0 exponent: e = ceil(log2(amax / 448)) clamped to [-127, 127]
//     (source/k3_moe_prefill_v4.cu:130-131), evaluated with exact integer
//     arithmetic on the bits of amax (see k3o_ue8m0_exp).
//   * reciprocal square root: correctly rounded (the reference calls the
//     approximate rsqrtf, source/k3_residual_v2.cu:242; its last-ulp behaviour is a
//     hardware table a CPU cannot reproduce, so both sides of the parity check use
//     the correctly rounded value).
//   * a deterministic exp / sigmoid built only from IEEE-754 fma/mul/add/div, used
//     where an index decision depends on a transcendental (router top-k,
//     source/k3_router_argmax.cu:100-104).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace k3o {

static inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

static inline float bf2f(uint16_t h) { return bits_f32((uint32_t)h << 16); }

// f32 -> bf16, round to nearest even; NaN -> 0x7fff (the canonical NaN CUDA returns).
static inline uint16_t f2bf(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
static inline float land(float f) { return bf2f(f2bf(f)); }

// bf16 x bf16 -> bf16 product (__hmul2 on bf16): the f32 product of two bf16 values is
// exact (8 + 8 significand bits), so one RNE rounding of it is the whole operation.
static inline uint16_t bfmul(uint16_t a, uint16_t b) { return f2bf(bf2f(a) * bf2f(b)); }

// E4M3 (1-4-3, bias 7, max 448, 0x7f/0xff = NaN, no infinity), RNE, saturating.
static inline uint8_t e4m3_encode(float x) {
  const uint32_t u = f32_bits(x);
  const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fu;   // NaN
  const double a = std::fabs((double)x);
  if (a >= 448.0) return sign | 0x7eu;                 // includes +-inf
  if (a < 0.015625) {                                  // below 2^-6: subnormal step 2^-9
    const int q = (int)std::nearbyint(a * 512.0);      // 0..8, ties to even
    return sign | (uint8_t)q;                          // q == 8 is the smallest normal 0x08
  }
  int e; const double m = std::frexp(a, &e);           // a = m * 2^e, m in [0.5, 1)
  int ex = e - 1;                                      // a = (2m) * 2^ex, 2m in [1, 2)
  int q = (int)std::nearbyint((2.0 * m - 1.0) * 8.0);  // 0..8, ties to even
  if (q == 8) { q = 0; ++ex; }
  int code = ((ex + 7) << 3) | q;
  if (code > 0x7e) code = 0x7e;
  return sign | (uint8_t)code;
}

static inline float e4m3_decode(uint8_t c) {
  const int s = c >> 7, ex = (c >> 3) & 0xf, m = c & 7;
  if (ex == 0xf && m == 7) return std::nanf("");
  const float v = ex == 0 ? std::ldexp((float)m, -9) : std::ldexp(1.0f + (float)m / 8.0f, ex - 7);
  return s ? -v : v;
}

// Smallest integer e with 448 * 2^e >= amax, clamped to [-127, 127]; 0 for amax == 0.
// amax = m * 2^(E-127) with m in [1, 2) and 448 = 1.75 * 2^8, so
// ceil(log2(amax / 448)) = E - 135 + (m > 1.75).  The reference evaluates
// (int)ceilf(log2f(amax / 448.f)) (source/k3_moe_prefill_v4.cu:130); amax is a bf16
// magnitude, so amax / 448 is either exactly a power of two (amax = 7 * 2^k) or at least
// 0.4 % away from one, and no f32 rounding of the quotient or the logarithm can move the
// ceiling across an integer: the two formulations agree on every bf16 input.
static inline int ue8m0_exp(float amax) {
  if (!(amax > 0.0f)) return 0;
  const uint32_t u = f32_bits(amax);
  const int E = (int)((u >> 23) & 0xffu);
  const uint32_t man = u & 0x7fffffu;
  int e;
  if (E == 0) e = -127;                                 // f32 subnormal: far below 448 * 2^-127
  else e = E - 135 + (man > 0x600000u ? 1 : 0);         // 0x600000 = the fraction of 1.75
  if (e < -127) e = -127;
  if (e > 127) e = 127;
  return e;
}

// 2^(-e) for e in [-127, 127], exact.
static inline float pow2_neg(int e) { return std::ldexp(1.0f, -e); }

// Round-to-nearest 1/sqrt(x) for positive finite x.  Evaluated in the x87 64-bit-significand
// format and rounded once to f32: the two-step rounding can differ from the IEEE
// round-to-nearest value only when the extended result lies within ~2^-40 (relative) of a
// float midpoint.  The device side uses the correctly rounded __frsqrt_rn.
static inline float rsqrt_rn(float x) { return (float)(1.0L / sqrtl((long double)x)); }

// Deterministic exp: IEEE operations only, identical sequence on the device
// (explicit __fmaf_rn / __fmul_rn there).  |x| is clamped to 80 so 2^n stays normal.
static inline float det_exp(float x) {
  x = std::fmin(std::fmax(x, -80.0f), 80.0f);
  const float t = x * 1.44269502162933349609375f;            // log2(e) rounded to f32
  const float n = std::nearbyintf(t);                        // ties to even
  float f = std::fmaf(n, -0.693145751953125f, x);            // ln2 high part (exact product)
  f = std::fmaf(n, -1.42860676533018704503775e-06f, f);      // ln2 low part
  float p = 1.98756915e-4f;                                  // degree-7 Taylor-like minimax
  p = std::fmaf(p, f, 1.39819995e-3f);
  p = std::fmaf(p, f, 8.33345205e-3f);
  p = std::fmaf(p, f, 4.16657962e-2f);
  p = std::fmaf(p, f, 1.66666657e-1f);
  p = std::fmaf(p, f, 5.00000000e-1f);
  p = std::fmaf(p, f, 1.0f);
  p = std::fmaf(p, f, 1.0f);
  const int32_t ni = (int32_t)n;
  return bits_f32(f32_bits(p) + ((uint32_t)ni << 23));       // p * 2^n, p in [0.70, 1.42]
}

static inline float det_sigmoid(float s) { return 1.0f / (1.0f + det_exp(-s)); }

}  // namespace k3o
