// Device-side primitives shared by the sm_100a kernels of this library.
//
// Everything here is register-level: 16-byte global accesses with cache hints, bf16 pair
// packing, the E4M3 / UE8M0 (MXFP8) conversions, fixed-order warp reductions and the
// IEEE-only exp used where an integer decision depends on a transcendental.  No kernel in
// this library is a dense contraction, so there is no tensor-core code.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace k3g {

struct V8 { unsigned w[4]; };   // eight bf16 = one 16-byte vector

// ---- global memory, 16 bytes at a time -------------------------------------------------
// Streaming loads: read once through the non-coherent path, not allocated in L1.
__device__ __forceinline__ V8 ld_stream(const void* p) {
  V8 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
  return v;
}
// Plain (possibly remote / coherent) load: used for peer memory that another GPU wrote.
__device__ __forceinline__ V8 ld_plain(const void* p) {
  V8 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
  return v;
}
// Cached read-only load (small tables reused by every row: gamma, taps).
__device__ __forceinline__ V8 ld_keep(const void* p) {
  const uint4 t = __ldg((const uint4*)p);
  V8 v; v.w[0] = t.x; v.w[1] = t.y; v.w[2] = t.z; v.w[3] = t.w;
  return v;
}
__device__ __forceinline__ void st_stream(void* p, const V8& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}
__device__ __forceinline__ void st_stream8(void* p, unsigned a, unsigned b) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" :: "l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void st_plain(void* p, const V8& v) {
  *(uint4*)p = make_uint4(v.w[0], v.w[1], v.w[2], v.w[3]);
}

// 32 bytes at a time (sm_100: 256-bit global loads and stores), for kernels that only move bytes.
struct V16 { unsigned w[8]; };
template <int BYTES> struct VecOf;
template <> struct VecOf<16> { typedef V8 type; };
template <> struct VecOf<32> { typedef V16 type; };
__device__ __forceinline__ V16 ld_stream32(const void* p) {
  V16 v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
  return v;
}
__device__ __forceinline__ V16 ld_plain32(const void* p) {      // plain (possibly remote / coherent) load
  V16 v;
  asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
  return v;
}
__device__ __forceinline__ V16 ld_keep32(const void* p) {       // read-only path, allocated in the caches
  V16 v;
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream32(void* p, const V16& v) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :: "l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7]) : "memory");
}
template <int BYTES> __device__ __forceinline__ typename VecOf<BYTES>::type ld_stream_vec(const void* p);
template <> __device__ __forceinline__ V8 ld_stream_vec<16>(const void* p) { return ld_stream(p); }
template <> __device__ __forceinline__ V16 ld_stream_vec<32>(const void* p) { return ld_stream32(p); }
template <int BYTES> __device__ __forceinline__ typename VecOf<BYTES>::type ld_keep_vec(const void* p);
template <> __device__ __forceinline__ V8 ld_keep_vec<16>(const void* p) { return ld_keep(p); }
template <> __device__ __forceinline__ V16 ld_keep_vec<32>(const void* p) { return ld_keep32(p); }
template <int BYTES> __device__ __forceinline__ void st_stream_vec(void* p, const typename VecOf<BYTES>::type& v);
template <> __device__ __forceinline__ void st_stream_vec<16>(void* p, const V8& v) { st_stream(p, v); }
template <> __device__ __forceinline__ void st_stream_vec<32>(void* p, const V16& v) { st_stream32(p, v); }

// ---- bf16 pairs ---------------------------------------------------------------------------
__device__ __forceinline__ float bf_lo(unsigned u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(unsigned u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ unsigned pack_bf2(float lo, float hi) {   // one cvt.rn.bf16x2.f32
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&h);
}
__device__ __forceinline__ __nv_bfloat162 as_bf2(unsigned u) { return *reinterpret_cast<const __nv_bfloat162*>(&u); }
__device__ __forceinline__ unsigned from_bf2(__nv_bfloat162 h) { return *reinterpret_cast<const unsigned*>(&h); }
// bf16x2 product / sum with one round-to-nearest-even per element (mul.rn / add.rn .bf16x2).
__device__ __forceinline__ unsigned mul_bf2(unsigned a, unsigned b) { return from_bf2(__hmul2(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ unsigned add_bf2(unsigned a, unsigned b) { return from_bf2(__hadd2(as_bf2(a), as_bf2(b))); }
__device__ __forceinline__ unsigned absmax_bf2(unsigned m, unsigned x) {
  return from_bf2(__hmax2(as_bf2(m), __habs2(as_bf2(x))));
}
__device__ __forceinline__ float land_bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---- packed f32x2 arithmetic (sm_100: one instruction for two IEEE round-to-nearest results) ----
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 f2_splat(float a) { return f2_pack(a, a); }
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) { f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) { f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) { f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
// a bf16 pair widened to an f32 pair, and an f32 pair rounded (RNE) to a bf16 pair
__device__ __forceinline__ f32x2 f2_from_bf2(unsigned u) { return f2_pack(bf_lo(u), bf_hi(u)); }
__device__ __forceinline__ unsigned f2_to_bf2(f32x2 v) { float lo, hi; f2_unpack(v, lo, hi); return pack_bf2(lo, hi); }
// sigmoid of a pair: packed scale and add, one ex2.approx and one rcp.approx per element
__device__ __forceinline__ f32x2 f2_fast_sigmoid(f32x2 x) {
  float a, b, ea, eb, ra, rb;
  f2_unpack(f2_mul(x, f2_splat(-1.4426950408889634f)), a, b);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ea) : "f"(a));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(eb) : "f"(b));
  f2_unpack(f2_add(f2_pack(ea, eb), f2_splat(1.0f)), a, b);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(ra) : "f"(a));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rb) : "f"(b));
  return f2_pack(ra, rb);
}

// ---- fixed-order reductions --------------------------------------------------------------
template <int LANES>
__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- MXFP8: E4M3 codes with one UE8M0 exponent per 32 elements ---------------------------
// e = smallest integer with 448 * 2^e >= amax (0 when amax == 0), clamped to [-127, 127];
// amax arrives as the bf16 bit pattern of a non-negative value.
__device__ __forceinline__ int ue8m0_exp_from_bf16(unsigned amax_bf16) {
  const unsigned E = (amax_bf16 >> 7) & 0xffu, man = amax_bf16 & 0x7fu;
  int e = (int)E - 135 + (man > 0x60u ? 1 : 0);       // 448 = 1.75 * 2^8; 0x60 = fraction of 1.75
  if (E == 0) e = -127;
  e = max(e, -127);
  if ((amax_bf16 & 0x7fffu) == 0) e = 0;
  return e;                                           // bf16 magnitudes never reach e > 120
}
__device__ __forceinline__ float pow2_neg(int e) { return __uint_as_float((unsigned)(127 - e) << 23); }

// two / four floats -> packed E4M3, round-to-nearest-even, saturating (cvt.rn.satfinite.e4m3x2.f32)
__device__ __forceinline__ unsigned e4m3x2(float lo, float hi) {
  return (unsigned)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ unsigned e4m3x4(float a, float b, float c, float d) {
  return e4m3x2(a, b) | (e4m3x2(c, d) << 16);
}
// Eight bf16 (one V8) scaled by s (a power of two) -> eight E4M3 codes in two words.
__device__ __forceinline__ void quant8(const V8& x, float s, unsigned& q0, unsigned& q1) {
  q0 = e4m3x4(__fmul_rn(bf_lo(x.w[0]), s), __fmul_rn(bf_hi(x.w[0]), s),
              __fmul_rn(bf_lo(x.w[1]), s), __fmul_rn(bf_hi(x.w[1]), s));
  q1 = e4m3x4(__fmul_rn(bf_lo(x.w[2]), s), __fmul_rn(bf_hi(x.w[2]), s),
              __fmul_rn(bf_lo(x.w[3]), s), __fmul_rn(bf_hi(x.w[3]), s));
}
// |max| over the eight bf16 of a vector, as a bf16 bit pattern.
__device__ __forceinline__ unsigned absmax8(const V8& x) {
  unsigned m = from_bf2(__habs2(as_bf2(x.w[0])));
  m = absmax_bf2(m, x.w[1]);
  m = absmax_bf2(m, x.w[2]);
  m = absmax_bf2(m, x.w[3]);
  const __nv_bfloat162 h = as_bf2(m);
  const __nv_bfloat16 r = __hmax(__low2bfloat16(h), __high2bfloat16(h));
  return (unsigned)__bfloat16_as_ushort(r);
}
__device__ __forceinline__ unsigned max_bf16_bits(unsigned a, unsigned b) { return a > b ? a : b; }  // non-negative bf16: bit order = value order

// ---- deterministic exp / sigmoid (IEEE operations only) ---------------------------------
// Same operation sequence as the host-side check uses; no approximate instruction, so the
// top-k selection that depends on it is reproducible bit for bit on any IEEE machine.
__device__ __forceinline__ float det_exp(float x) {
  x = fminf(fmaxf(x, -80.0f), 80.0f);
  const float t = __fmul_rn(x, 1.44269502162933349609375f);
  const float n = rintf(t);
  float f = __fmaf_rn(n, -0.693145751953125f, x);
  f = __fmaf_rn(n, -1.42860676533018704503775e-06f, f);
  float p = 1.98756915e-4f;
  p = __fmaf_rn(p, f, 1.39819995e-3f);
  p = __fmaf_rn(p, f, 8.33345205e-3f);
  p = __fmaf_rn(p, f, 4.16657962e-2f);
  p = __fmaf_rn(p, f, 1.66666657e-1f);
  p = __fmaf_rn(p, f, 5.00000000e-1f);
  p = __fmaf_rn(p, f, 1.0f);
  p = __fmaf_rn(p, f, 1.0f);
  return __uint_as_float(__float_as_uint(p) + ((unsigned)(int)n << 23));
}
__device__ __forceinline__ float det_sigmoid(float s) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, det_exp(-s))); }

// Fast sigmoid for bf16-landed results: one ex2.approx and one rcp.approx.
__device__ __forceinline__ float fast_sigmoid(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}

// ---- ring-order reduction chain over the ranks' partial buffers (pull reduce-scatter) ------------
// Chain position k reads base[k]; first hop unrounded, every later hop lands one bf16 rounding:
// a = f32(bf16(a + f32(v_k))).  bf16x2 add.rn is that operation on a pair.
template <int NR, int OWNPOS, int DESCEND>
__device__ __forceinline__ void rs_bases(const __nv_bfloat16* src, const unsigned long long* src_peer, long long off, int rank,
                                         const uint4* (&base)[NR]) {
#pragma unroll
  for (int k = 0; k < NR; ++k) {
    if (k == OWNPOS) {
      base[k] = reinterpret_cast<const uint4*>(src + off);
    } else {
      const int pi = (k < OWNPOS) ? k : k - 1;
      const int o = DESCEND ? (NR - 1 - pi) : (1 + pi);
      base[k] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src_peer[(rank + o) & (NR - 1)]) + off);
    }
  }
}

template <int NR>
__device__ __forceinline__ V8 rs_chain(const uint4* const (&base)[NR], long long i) {
  V8 x[NR];
#pragma unroll
  for (int k = 0; k < NR; ++k) x[k] = ld_plain(base[k] + i);     // all hops' loads issued back to back
  V8 a = x[0];
#pragma unroll
  for (int k = 1; k < NR; ++k) {
#pragma unroll
    for (int j = 0; j < 4; ++j) a.w[j] = add_bf2(a.w[j], x[k].w[j]);
  }
  return a;
}

// The same chain for one row in the 128-thread team layout (thread t owns the 16-byte vectors t + 128 v, v < VPT),
// pulled with 32-BYTE loads: over NVLink the wider access moves measurably more (32-byte peer stores reached 666 GB/s
// where 16-byte ones reached 590).  Vectors are taken in pairs (2p, 2p + 1): the even lane of a lane pair loads the
// pair's two neighbouring vectors of chunk 2p, the odd lane those of chunk 2p + 1; the chain is added on all eight
// words (it is element-wise, so it does not care whose element it is), and the two lanes then swap the halves that
// belong to each other -- four shuffles per pair.  An odd last vector is loaded as 16 bytes.  PIF pairs are in flight
// at a time (NR x 32 bytes each).  row_vec = index of the row's first 16-byte vector from each base; it must be even
// and every base 32-byte aligned.
template <int VPT, int NR, int PIF>
__device__ __forceinline__ void rs_chain_team_row(const uint4* const (&base)[NR], long long row_vec, int t, V8 (&x)[VPT]) {
  constexpr int kTeamThreads = 128;
  const bool odd = (t & 1) != 0;
#pragma unroll
  for (int p0 = 0; p0 < VPT / 2; p0 += PIF) {
    V16 a[PIF][NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) {
#pragma unroll
      for (int c = 0; c < PIF; ++c) {
        if (p0 + c < VPT / 2) {
          const int va = 2 * (p0 + c), vb = va + 1;
          a[c][k] = ld_plain32(base[k] + row_vec + (t & ~1) + kTeamThreads * (odd ? vb : va));
        }
      }
    }
#pragma unroll
    for (int c = 0; c < PIF; ++c) {
      if (p0 + c < VPT / 2) {
        const int va = 2 * (p0 + c), vb = va + 1;
        V16 s = a[c][0];
#pragma unroll
        for (int k = 1; k < NR; ++k) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s.w[j] = add_bf2(s.w[j], a[c][k].w[j]);
        }
        V8 got;
#pragma unroll
        for (int j = 0; j < 4; ++j) got.w[j] = __shfl_xor_sync(0xffffffffu, odd ? s.w[j] : s.w[4 + j], 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          x[va].w[j] = odd ? got.w[j] : s.w[j];
          x[vb].w[j] = odd ? s.w[4 + j] : got.w[j];
        }
      }
    }
  }
  if (VPT & 1) {
    const long long vi = row_vec + t + kTeamThreads * (VPT - 1);
    V8 q[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) q[k] = ld_plain(base[k] + vi);
    x[VPT - 1] = q[0];
#pragma unroll
    for (int k = 1; k < NR; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) x[VPT - 1].w[j] = add_bf2(x[VPT - 1].w[j], q[k].w[j]);
    }
  }
}

}  // namespace k3g
