// MLA prep: RMSNorm of the q / kv low-rank rows, latent-cache append, gate-band landing, and the
// config-level variant with RoPE and FMHA packing.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   kern_k3_mla_prep_head  source/k3_mla_prep_v2.cu:130-211 (f32 partial) and
//                          source/k3_mla_prep_bf16.cu (bf16 partial, -DK3G_MLA_BF16)
//   kern_k3_mla_prep_gate  source/k3_mla_prep_v2.cu:91-118
//
// Row layout (MLA_FUSED columns): q_a [0,1536) | kv_a [1536,2048) | rope [2048,2112) | gate band.
// Reduction order kept from the reference: a unit is 4 consecutive columns, a group is 32 units;
// lane partial = fma chain over the unit's 4 landed values from 0, xor-butterfly over the group's
// 32 lanes, groups summed in ascending order (12 q groups, 4 kv groups).
//
// Layout for B200: ONE WARP PER ROW.  Lane l owns unit 32 G + l of every group G, so each group
// is one coalesced 512 B (f32) / 256 B (bf16) load, the whole head of the row (2112 values)
// stays in registers between the reduction and the scaled stores -- the row is read once, not
// twice -- and there is no shared memory and no block barrier.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {

constexpr int kQ = 1536, kKV = 512, kRope = 64, kKVA = kKV + kRope, kHead = kQ + kKV + kRope;   // 2112
constexpr int kQG = kQ / 128, kKG = kKV / 128;                                                  // 12, 4

// Four landed (bf16-rounded) values of one unit, as two packed words.
template <bool PB>
__device__ __forceinline__ uint2 load_unit(const void* row, int unit) {
  if (PB) {
    return __ldcs(reinterpret_cast<const uint2*>(row) + unit);
  } else {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(row) + unit);
    return make_uint2(pack_bf2(v.x, v.y), pack_bf2(v.z, v.w));
  }
}
__device__ __forceinline__ float unit_sumsq(uint2 u) {
  float p = 0.f;
  p = __fmaf_rn(bf_lo(u.x), bf_lo(u.x), p);
  p = __fmaf_rn(bf_hi(u.x), bf_hi(u.x), p);
  p = __fmaf_rn(bf_lo(u.y), bf_lo(u.y), p);
  p = __fmaf_rn(bf_hi(u.y), bf_hi(u.y), p);
  return p;
}
// bf16(bf16(x * sc) * gamma) on a unit
__device__ __forceinline__ uint2 unit_norm(uint2 u, float sc, uint2 g) {
  return make_uint2(mul_bf2(pack_bf2(__fmul_rn(bf_lo(u.x), sc), __fmul_rn(bf_hi(u.x), sc)), g.x),
                    mul_bf2(pack_bf2(__fmul_rn(bf_lo(u.y), sc), __fmul_rn(bf_hi(u.y), sc)), g.y));
}

template <bool PB>
__device__ __forceinline__ void mla_head_body(const void* __restrict__ partial, int fused, const __nv_bfloat16* __restrict__ gamma_q,
                                              const __nv_bfloat16* __restrict__ gamma_kv, const long long* __restrict__ slot_mapping,
                                              __nv_bfloat16* __restrict__ slab, long long layer_off, long long page_stride,
                                              __nv_bfloat16* __restrict__ q_norm, int B, float eps) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int b = blockIdx.x * wpb + (threadIdx.x >> 5); b < B; b += gridDim.x * wpb) {
    const char* row = reinterpret_cast<const char*>(partial) + (size_t)b * fused * (PB ? 2 : 4);
    uint2 uq[kQG], uk[kKG], ur = make_uint2(0u, 0u);
#pragma unroll
    for (int g = 0; g < kQG; ++g) uq[g] = load_unit<PB>(row, 32 * g + lane);
#pragma unroll
    for (int g = 0; g < kKG; ++g) uk[g] = load_unit<PB>(row, kQ / 4 + 32 * g + lane);
    if (lane < kRope / 4) ur = load_unit<PB>(row, (kQ + kKV) / 4 + lane);
    float tq = 0.f, tk = 0.f;
#pragma unroll
    for (int g = 0; g < kQG; ++g) tq = __fadd_rn(tq, butterfly_sum<32>(unit_sumsq(uq[g])));
#pragma unroll
    for (int g = 0; g < kKG; ++g) tk = __fadd_rn(tk, butterfly_sum<32>(unit_sumsq(uk[g])));
    const float scq = __frsqrt_rn(__fmaf_rn(tq, 1.f / (float)kQ, eps));
    const float sck = __frsqrt_rn(__fmaf_rn(tk, 1.f / (float)kKV, eps));
#pragma unroll
    for (int g = 0; g < kQG; ++g) {
      const int u = 32 * g + lane;
      const uint2 gm = __ldg(reinterpret_cast<const uint2*>(gamma_q) + u);
      __stcs(reinterpret_cast<uint2*>(q_norm + (size_t)b * kQ) + u, unit_norm(uq[g], scq, gm));
    }
    const long long slot = slot_mapping[b];
    if (slot < 0) continue;                       // "no slot": nothing is appended
    __nv_bfloat16* rowp = slab + (slot / 64) * page_stride + layer_off + (slot % 64) * kKVA;
#pragma unroll
    for (int g = 0; g < kKG; ++g) {
      const int u = 32 * g + lane;
      const uint2 gm = __ldg(reinterpret_cast<const uint2*>(gamma_kv) + u);
      *(reinterpret_cast<uint2*>(rowp) + u) = unit_norm(uk[g], sck, gm);
    }
    if (lane < kRope / 4) *(reinterpret_cast<uint2*>(rowp + kKV) + lane) = ur;
  }
}

// gate band: mla_gate[b, c] = bf16(P[b, 2112 + c]), eight columns per thread
template <bool PB>
__device__ __forceinline__ void mla_gate_body(const void* __restrict__ partial, int fused, int inner, __nv_bfloat16* __restrict__ mla_gate,
                                              int B) {
  const int vpr = inner >> 3;
  const long long total = (long long)B * vpr;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / vpr;
    const int c = (int)(i - b * vpr) * 8;
    V8 o;
    if (PB) {
      o = ld_stream(reinterpret_cast<const __nv_bfloat16*>(partial) + b * fused + kHead + c);
    } else {
      const float* p = reinterpret_cast<const float*>(partial) + b * fused + kHead + c;
      const V8 f0 = ld_stream(p), f1 = ld_stream(p + 4);
      o.w[0] = pack_bf2(__uint_as_float(f0.w[0]), __uint_as_float(f0.w[1]));
      o.w[1] = pack_bf2(__uint_as_float(f0.w[2]), __uint_as_float(f0.w[3]));
      o.w[2] = pack_bf2(__uint_as_float(f1.w[0]), __uint_as_float(f1.w[1]));
      o.w[3] = pack_bf2(__uint_as_float(f1.w[2]), __uint_as_float(f1.w[3]));
    }
    st_stream(mla_gate + b * inner + c, o);
  }
}

// rotate eight (x1, x2) pairs: o1 = bf16(fma(-x2, sin, x1 * cos)), o2 = bf16(fma(x1, sin, x2 * cos))
__device__ __forceinline__ void rope8(const V8& x1, const V8& x2, const V8& cs, const V8& sn, V8& o1, V8& o2) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a0 = bf_lo(x1.w[j]), a1 = bf_hi(x1.w[j]), b0 = bf_lo(x2.w[j]), b1 = bf_hi(x2.w[j]);
    const float c0 = bf_lo(cs.w[j]), c1 = bf_hi(cs.w[j]), s0 = bf_lo(sn.w[j]), s1 = bf_hi(sn.w[j]);
    o1.w[j] = pack_bf2(__fmaf_rn(-b0, s0, __fmul_rn(a0, c0)), __fmaf_rn(-b1, s1, __fmul_rn(a1, c1)));
    o2.w[j] = pack_bf2(__fmaf_rn(a0, s0, __fmul_rn(b0, c0)), __fmaf_rn(a1, s1, __fmul_rn(b1, c1)));
  }
}

// Config-level prep.  kv [T,576], q [T,heads,192], rope_tab [T,64] = cos|sin.  Flat thread mapping:
// item = (token, head, c) with c = 0..3 one 8-pair chunk of the rope slice; the thread rotates that
// chunk of q, writes the rotated k_rope chunk into the head's k slots and copies four of the head's
// sixteen nope vectors -- six independent 16-byte loads in flight, no shared memory.  The latent
// RMSNorm needs a whole warp per token: global warp w also normalises token w (there are at least as
// many warps as tokens when heads >= 8; otherwise warps stride over tokens).
__global__ void __launch_bounds__(128) mla_rope_pack_kernel(const __nv_bfloat16* __restrict__ kv, const __nv_bfloat16* __restrict__ q,
                                                            const __nv_bfloat16* __restrict__ gamma_kv, const __nv_bfloat16* __restrict__ rope_tab,
                                                            __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                                            __nv_bfloat16* __restrict__ latent_out, int T, int heads, float eps) {
  const int lane = threadIdx.x & 31;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long items = (long long)T * heads * 4;
  for (long long it = gtid; it < items; it += nthreads) {
    const int c = (int)(it & 3);
    const long long th = it >> 2;                      // token * heads + head
    const int t = (int)(th / heads);
    const size_t o = (size_t)th * 192;
    const __nv_bfloat16* kvr = kv + (size_t)t * kKVA + kKV;
    const __nv_bfloat16* tab = rope_tab + (size_t)t * 64;
    const V8 a1 = ld_stream(q + o + 128 + 8 * c), a2 = ld_stream(q + o + 160 + 8 * c);
    V8 n4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) n4[j] = ld_stream(q + o + 8 * (4 * j + c));
    const V8 cs = ld_keep(tab + 8 * c), sn = ld_keep(tab + 32 + 8 * c);
    const V8 b1 = ld_keep(kvr + 8 * c), b2 = ld_keep(kvr + 32 + 8 * c);
    V8 o1, o2, k1, k2;
    rope8(a1, a2, cs, sn, o1, o2);
    rope8(b1, b2, cs, sn, k1, k2);
    st_stream(q_out + o + 128 + 8 * c, o1);
    st_stream(q_out + o + 160 + 8 * c, o2);
    st_stream(k_out + o + 128 + 8 * c, k1);
    st_stream(k_out + o + 160 + 8 * c, k2);
#pragma unroll
    for (int j = 0; j < 4; ++j) st_stream(q_out + o + 8 * (4 * j + c), n4[j]);
  }
  // latent RMSNorm (kv groups' reduction order), one warp per token
  const long long nwarps = nthreads >> 5;
  for (long long t = gtid >> 5; t < T; t += nwarps) {
    const __nv_bfloat16* kvr = kv + (size_t)t * kKVA;
    uint2 uk[kKG];
#pragma unroll
    for (int g = 0; g < kKG; ++g) uk[g] = __ldg(reinterpret_cast<const uint2*>(kvr) + 32 * g + lane);
    float tk = 0.f;
#pragma unroll
    for (int g = 0; g < kKG; ++g) tk = __fadd_rn(tk, butterfly_sum<32>(unit_sumsq(uk[g])));
    const float sck = __frsqrt_rn(__fmaf_rn(tk, 1.f / (float)kKV, eps));
#pragma unroll
    for (int g = 0; g < kKG; ++g) {
      const int u = 32 * g + lane;
      __stcs(reinterpret_cast<uint2*>(latent_out + (size_t)t * kKV) + u, unit_norm(uk[g], sck, __ldg(reinterpret_cast<const uint2*>(gamma_kv) + u)));
    }
  }
}

template <bool PB>
__global__ void __launch_bounds__(128) mla_head_kernel(const void* partial, int fused, const __nv_bfloat16* gq, const __nv_bfloat16* gkv,
                                                       const long long* slot_mapping, __nv_bfloat16* slab, long long layer_off,
                                                       long long page_stride, __nv_bfloat16* q_norm, int B, float eps) {
  mla_head_body<PB>(partial, fused, gq, gkv, slot_mapping, slab, layer_off, page_stride, q_norm, B, eps);
}
template <bool PB>
__global__ void __launch_bounds__(256) mla_gate_kernel(const void* partial, int fused, int inner, __nv_bfloat16* mla_gate, int B) {
  mla_gate_body<PB>(partial, fused, inner, mla_gate, B);
}

}  // namespace

// ---- manifest entry points (INNER / MLA_FUSED / eps are build constants there) -----------------
#ifndef INNER
#define INNER 3072
#endif
#ifndef MLA_FUSED
#define MLA_FUSED (2112 + INNER)
#endif
#ifdef K3G_MLA_BF16
typedef __nv_bfloat16 k3g_mla_partial_t;
#define K3G_MLA_PB true
#else
typedef float k3g_mla_partial_t;
#define K3G_MLA_PB false
#endif

extern "C" __global__ void __launch_bounds__(512) kern_k3_mla_prep_head(
    const k3g_mla_partial_t* __restrict__ partial, const __nv_bfloat16* __restrict__ gamma_q_a, const __nv_bfloat16* __restrict__ gamma_kv_a,
    const long long* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ slab, long long layer_off, long long page_stride,
    __nv_bfloat16* __restrict__ q_norm, int B) {
  mla_head_body<K3G_MLA_PB>(partial, MLA_FUSED, gamma_q_a, gamma_kv_a, slot_mapping, slab, layer_off, page_stride, q_norm, B, 1e-5f);
}
extern "C" __global__ void __launch_bounds__(384) kern_k3_mla_prep_gate(const k3g_mla_partial_t* __restrict__ partial,
                                                                       __nv_bfloat16* __restrict__ mla_gate, int B) {
  mla_gate_body<K3G_MLA_PB>(partial, MLA_FUSED, INNER, mla_gate, B);
}

#ifndef K3G_CUBIN_ONLY
K3G_API int k3g_mla_prep(const void* partial, int partial_is_bf16, const void* gamma_q, const void* gamma_kv, const void* slot_mapping,
                         void* slab, long long layer_off, long long page_stride, void* q_norm, void* mla_gate, int B, int inner,
                         float eps, void* stream) {
  K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(gamma_q); K3G_REQUIRE_PTR(gamma_kv); K3G_REQUIRE_PTR(slot_mapping);
  K3G_REQUIRE_PTR(slab); K3G_REQUIRE_PTR(q_norm);
  K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(q_norm); K3G_REQUIRE_ALIGNED(mla_gate);
  K3G_REQUIRE(((uintptr_t)slab & 7) == 0 && layer_off % 4 == 0 && page_stride % 4 == 0, K3G_EALIGN);
  K3G_REQUIRE(B >= 0 && inner >= 0 && inner % 8 == 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  const int fused = kHead + inner;
  cudaStream_t st = k3g_stream(stream);
  const int hgrid = (B + 3) / 4;
  if (partial_is_bf16)
    mla_head_kernel<true><<<hgrid, 128, 0, st>>>(partial, fused, (const __nv_bfloat16*)gamma_q, (const __nv_bfloat16*)gamma_kv,
                                                 (const long long*)slot_mapping, (__nv_bfloat16*)slab, layer_off, page_stride,
                                                 (__nv_bfloat16*)q_norm, B, eps);
  else
    mla_head_kernel<false><<<hgrid, 128, 0, st>>>(partial, fused, (const __nv_bfloat16*)gamma_q, (const __nv_bfloat16*)gamma_kv,
                                                  (const long long*)slot_mapping, (__nv_bfloat16*)slab, layer_off, page_stride,
                                                  (__nv_bfloat16*)q_norm, B, eps);
  if (mla_gate && inner > 0) {
    const long long total = (long long)B * (inner / 8);
    const int ggrid = (int)((total + 255) / 256);
    if (partial_is_bf16) mla_gate_kernel<true><<<ggrid, 256, 0, st>>>(partial, fused, inner, (__nv_bfloat16*)mla_gate, B);
    else mla_gate_kernel<false><<<ggrid, 256, 0, st>>>(partial, fused, inner, (__nv_bfloat16*)mla_gate, B);
  }
  return k3g_launch_status();
}

K3G_API int k3g_mla_prep_rope_pack(const void* kv, const void* q, const void* gamma_kv, const void* rope_tab, void* q_out, void* k_out,
                                   void* latent_out, int T, int heads, float eps, void* stream) {
  K3G_REQUIRE_PTR(kv); K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(gamma_kv); K3G_REQUIRE_PTR(rope_tab); K3G_REQUIRE_PTR(q_out);
  K3G_REQUIRE_PTR(k_out); K3G_REQUIRE_PTR(latent_out);
  K3G_REQUIRE_ALIGNED(kv); K3G_REQUIRE_ALIGNED(q); K3G_REQUIRE_ALIGNED(rope_tab); K3G_REQUIRE_ALIGNED(q_out); K3G_REQUIRE_ALIGNED(k_out);
  K3G_REQUIRE_ALIGNED(latent_out); K3G_REQUIRE_ALIGNED(gamma_kv);
  K3G_REQUIRE(T >= 0 && heads > 0 && heads <= 128, K3G_ESHAPE);
  if (T == 0) return K3G_OK;
  const long long items = (long long)T * heads * 4;
  long long grid = (items + 127) / 128;
  if (grid < (T + 3) / 4) grid = (T + 3) / 4;      // at least one warp per token for the latent norm
  K3G_REQUIRE(grid <= 0x7fffffffLL, K3G_ELIMIT);
  mla_rope_pack_kernel<<<(unsigned)grid, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)kv, (const __nv_bfloat16*)q,
                                                                   (const __nv_bfloat16*)gamma_kv, (const __nv_bfloat16*)rope_tab,
                                                                   (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, (__nv_bfloat16*)latent_out,
                                                                   T, heads, eps);
  return k3g_launch_status();
}
#endif
