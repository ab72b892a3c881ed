// bf16 -> FP8 quantisation kernels.
//
//   kern_k3_moe_quant        MXFP8: E4M3 codes + one UE8M0 exponent per 32 consecutive elements
//                            (replaces xiaguan/kern-k3 source/k3_moe_prefill_v4.cu:111-140)
//   kern_quant_fp8_amax_v2   per-tensor pair: partial |max| per block            (replaces
//   kern_quant_fp8_apply_v2  scale = amax / 448, y = e4m3(x / scale)              source/k3_quant_fp8_pair_v2.cu:42-95)
//
// MXFP8 layout: a thread owns one 32-element group (64 contiguous input bytes): four 16-byte
// loads in flight, the amax taken in registers, 32 code bytes out as two 16-byte stores.  The
// exponent is computed on the bf16 bits of amax (exact integer arithmetic, no log2).
//
// Per-tensor pair: the amax pass walks the tensor forwards with ordinary (L2-allocating)
// loads and the apply pass walks it backwards, so the tail the first pass left in the 126 MB
// L2 is what the second pass reads first.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

extern "C" __global__ void __launch_bounds__(256) kern_k3_moe_quant(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                                   uint8_t* __restrict__ sf, int rows, int cols) {
  // One thread per 32-element group: four 16-byte loads in flight, amax in registers (no
  // shuffles), two 16-byte code stores and one scale byte (a warp's 32 scale bytes are contiguous).
  const long long ngroups = (long long)rows * cols / 32;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += (long long)gridDim.x * blockDim.x) {
    const __nv_bfloat16* src = x + g * 32;
    V8 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = ld_plain(src + 8 * j);   // through L1: the warp's four loads share their sectors
    unsigned am = absmax8(v[0]);
#pragma unroll
    for (int j = 1; j < 4; ++j) am = max_bf16_bits(am, absmax8(v[j]));
    const int e = ue8m0_exp_from_bf16(am);
    const float sc = pow2_neg(e);
    V8 o0, o1;
    quant8(v[0], sc, o0.w[0], o0.w[1]);
    quant8(v[1], sc, o0.w[2], o0.w[3]);
    quant8(v[2], sc, o1.w[0], o1.w[1]);
    quant8(v[3], sc, o1.w[2], o1.w[3]);
    st_stream(q + g * 32, o0);
    st_stream(q + g * 32 + 16, o1);
    sf[g] = (uint8_t)(e + 127);
  }
}

#define K3G_QT 256

__device__ __forceinline__ unsigned block_max_u32(unsigned m) {
  __shared__ unsigned s[K3G_QT / 32];
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
  __syncthreads();
  unsigned r = 0;
#pragma unroll
  for (int w = 0; w < K3G_QT / 32; ++w) r = max(r, s[w]);
  __syncthreads();
  return r;
}

// partials[b] = max |x| over block b's slice, as f32.  |bf16| ordering = unsigned ordering of
// the low 15 bits, so the maximum is taken on bit patterns (exact, order-free).
// VB bytes per access (32 when x allows it), four accesses in flight per thread: the pass is a pure read stream and
// one 16-byte load per thread at a time leaves HBM half idle.  Loads allocate in L2 on purpose (see the apply pass).
template <int VB>
__device__ __forceinline__ unsigned amax_words(const unsigned char* p) {
  unsigned m2 = 0;
  if (VB == 32) {
    unsigned w[8];
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(p));
#pragma unroll
    for (int j = 0; j < 8; ++j) m2 = __vmaxu2(m2, w[j] & 0x7fff7fffu);
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    m2 = __vmaxu2(__vmaxu2(v.x & 0x7fff7fffu, v.y & 0x7fff7fffu), __vmaxu2(v.z & 0x7fff7fffu, v.w & 0x7fff7fffu));
  }
  return m2;
}

template <int VB>
__device__ __forceinline__ void amax_body(const __nv_bfloat16* __restrict__ x, int n, float* __restrict__ partials) {
  constexpr int EPV = VB / 2;                                      // elements per access
  const unsigned char* p = reinterpret_cast<const unsigned char*>(x);
  const long long nv = n / EPV;
  const long long stride = (long long)gridDim.x * K3G_QT;
  unsigned m2 = 0;   // two 15-bit maxima, packed like the data
  long long i = (long long)blockIdx.x * K3G_QT + threadIdx.x;
  for (; i + 3 * stride < nv; i += 4 * stride) {
    const unsigned a = amax_words<VB>(p + i * VB), b = amax_words<VB>(p + (i + stride) * VB);
    const unsigned c = amax_words<VB>(p + (i + 2 * stride) * VB), d = amax_words<VB>(p + (i + 3 * stride) * VB);
    m2 = __vmaxu2(m2, __vmaxu2(__vmaxu2(a, b), __vmaxu2(c, d)));
  }
  for (; i < nv; i += stride) m2 = __vmaxu2(m2, amax_words<VB>(p + i * VB));
  unsigned m = max(m2 & 0xffffu, m2 >> 16);
  if (blockIdx.x == 0 && threadIdx.x < (n % EPV))
    m = max(m, (unsigned)__bfloat16_as_ushort(x[nv * EPV + threadIdx.x]) & 0x7fffu);
  m = block_max_u32(m);
  if (threadIdx.x == 0) partials[blockIdx.x] = __uint_as_float(m << 16);
}

extern "C" __global__ void __launch_bounds__(K3G_QT) kern_quant_fp8_amax_v2(const __nv_bfloat16* __restrict__ x, int n,
                                                                           float* __restrict__ partials) {
  if ((reinterpret_cast<unsigned long long>(x) & 31ull) == 0) amax_body<32>(x, n, partials);
  else amax_body<16>(x, n, partials);
}

// y = e4m3(x * (1 / scale)), scale = max(partials) / 448.  The tensor is walked BACKWARDS: the amax pass went forwards
// with L2-allocating loads, so what it touched last is what this pass reads first, out of the 126 MB L2.  VB = 32:
// a thread converts sixteen elements per access (one 32-byte load, one 16-byte store), two accesses in flight.
template <int VB>
__device__ __forceinline__ void apply_vec(const unsigned char* xp, uint8_t* yp, float inv) {
  if (VB == 32) {
    const V16 v = ld_stream32(xp);
    V8 lo, hi, o;
#pragma unroll
    for (int j = 0; j < 4; ++j) { lo.w[j] = v.w[j]; hi.w[j] = v.w[4 + j]; }
    quant8(lo, inv, o.w[0], o.w[1]);
    quant8(hi, inv, o.w[2], o.w[3]);
    st_stream(yp, o);
  } else {
    const V8 v = ld_stream(xp);
    unsigned q0, q1;
    quant8(v, inv, q0, q1);
    st_stream8(yp, q0, q1);
  }
}

template <int VB>
__device__ __forceinline__ void apply_body(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, int n, float inv) {
  constexpr int EPV = VB / 2;
  const unsigned char* xp = reinterpret_cast<const unsigned char*>(x);
  const long long nv = n / EPV;
  const long long total = (long long)gridDim.x * K3G_QT;
  // backwards: start with the part of x the amax pass touched last
  for (long long i = nv - 1 - ((long long)blockIdx.x * K3G_QT + threadIdx.x); i >= 0; i -= 2 * total) {
    const long long i1 = i - total;
    if (i1 >= 0) {
      // both loads issued before the first conversion
      if (VB == 32) {
        const V16 a = ld_stream32(xp + i * VB), b = ld_stream32(xp + i1 * VB);
        V8 lo, hi, o;
#pragma unroll
        for (int j = 0; j < 4; ++j) { lo.w[j] = a.w[j]; hi.w[j] = a.w[4 + j]; }
        quant8(lo, inv, o.w[0], o.w[1]); quant8(hi, inv, o.w[2], o.w[3]);
        st_stream(y + i * EPV, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) { lo.w[j] = b.w[j]; hi.w[j] = b.w[4 + j]; }
        quant8(lo, inv, o.w[0], o.w[1]); quant8(hi, inv, o.w[2], o.w[3]);
        st_stream(y + i1 * EPV, o);
      } else {
        const V8 a = ld_stream(xp + i * VB), b = ld_stream(xp + i1 * VB);
        unsigned q0, q1;
        quant8(a, inv, q0, q1);
        st_stream8(y + i * EPV, q0, q1);
        quant8(b, inv, q0, q1);
        st_stream8(y + i1 * EPV, q0, q1);
      }
    } else {
      apply_vec<VB>(xp + i * VB, y + i * EPV, inv);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n % EPV)) {
    const long long i = nv * EPV + threadIdx.x;
    y[i] = (uint8_t)(e4m3x2(__fmul_rn(__bfloat162float(x[i]), inv), 0.f) & 0xffu);
  }
}

extern "C" __global__ void __launch_bounds__(K3G_QT) kern_quant_fp8_apply_v2(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, int n,
                                                                            const float* __restrict__ partials, int nb,
                                                                            float* __restrict__ scale_out) {
  // partials are non-negative floats: bit order = value order.  Every block takes the maximum of all of them, so the
  // reads are 16 bytes wide and eight per thread are in flight (a producer may leave one partial per row: 16384 words).
  unsigned m = 0;
  int b = 0;
  if ((reinterpret_cast<unsigned long long>(partials) & 15ull) == 0) {
    const uint4* p4 = reinterpret_cast<const uint4*>(partials);
    const int n4 = nb >> 2;
    int i = threadIdx.x;
    for (; i + 7 * K3G_QT < n4; i += 8 * K3G_QT) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = __ldg(p4 + i + k * K3G_QT);
#pragma unroll
      for (int k = 0; k < 8; ++k) m = max(max(m, max(v[k].x, v[k].y)), max(v[k].z, v[k].w));
    }
    for (; i < n4; i += K3G_QT) {
      const uint4 v = __ldg(p4 + i);
      m = max(max(m, max(v.x, v.y)), max(v.z, v.w));
    }
    b = n4 << 2;
  }
  for (b += threadIdx.x; b < nb; b += K3G_QT) m = max(m, __float_as_uint(partials[b]));
  const float amax = __uint_as_float(block_max_u32(m));
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = scale;
  const float inv = __fdiv_rn(1.f, scale);
  if ((reinterpret_cast<unsigned long long>(x) & 31ull) == 0 && (reinterpret_cast<unsigned long long>(y) & 15ull) == 0) apply_body<32>(x, y, n, inv);
  else apply_body<16>(x, y, n, inv);
}

#ifndef K3G_CUBIN_ONLY
K3G_API int k3g_moe_quant(const void* x, void* q, void* sf, int rows, int cols, int grid_hint, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(sf);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE_ALIGNED(q);
  K3G_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0, K3G_ESHAPE);
  const long long nvec = (long long)rows * cols / 32;
  if (nvec == 0) return K3G_OK;
  long long grid = (nvec + 255) / 256;       // one group per thread
  if (grid_hint > 0 && grid_hint < grid) grid = grid_hint;
  K3G_REQUIRE(grid <= 0x7fffffffLL, K3G_ELIMIT);
  kern_k3_moe_quant<<<(unsigned)grid, 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)sf, rows, cols);
  return k3g_launch_status();
}

// op `quant_fp8_tensor` of the reference manifest: both launches share one grid width, and
// partials must hold that many floats.
K3G_API int k3g_quant_fp8_tensor(const void* x, void* y, void* scale_out, void* partials, int n, int grid, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(y); K3G_REQUIRE_PTR(partials);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE(((uintptr_t)y & 7) == 0, K3G_EALIGN);
  K3G_REQUIRE(n >= 0 && grid > 0, K3G_ESHAPE);
  kern_quant_fp8_amax_v2<<<grid, K3G_QT, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, n, (float*)partials);
  kern_quant_fp8_apply_v2<<<grid, K3G_QT, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)y, n, (const float*)partials,
                                                                  grid, (float*)scale_out);
  return k3g_launch_status();
}
// The apply launch alone, for tensors whose producer already left partial maxima (k3g_attnres_rms_push_amax,
// k3g_land_add_attnres_rms_stats_amax, k3g_situ_rms_amax): partials [nparts] f32 non-negative, any partition
// of the tensor; the result is bit-identical to k3g_quant_fp8_tensor because the maximum is exact and order-free.
K3G_API int k3g_quant_fp8_apply(const void* x, void* y, void* scale_out, const void* partials, int nparts, int n, int grid, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(y); K3G_REQUIRE_PTR(partials);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE(((uintptr_t)y & 7) == 0, K3G_EALIGN);
  K3G_REQUIRE(n >= 0 && grid > 0 && nparts > 0, K3G_ESHAPE);
  kern_quant_fp8_apply_v2<<<grid, K3G_QT, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)y, n, (const float*)partials, nparts,
                                                                  (float*)scale_out);
  return k3g_launch_status();
}
#endif
