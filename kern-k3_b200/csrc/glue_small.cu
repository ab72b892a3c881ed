// The remaining per-layer glue of the prefill program: shared-expert SiTU landing + MoE latent
// RMSNorm, the MLA output gate, and the two state/cache staging copies.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   kern_k3_situ_rms_bf16   source/k3_land_fused.cu:123-202   (op land_situ_rms)
//   kern_sigmoid_mul_bf16   source/sigmoid_mul.cu:15-44        (op mla_gate)
//   kern_k3_span_state      source/k3_span_state.cu:19-29      (ops span_state_load / span_state_store)
//   kern_k3_latent_gather   source/k3_mla_v2.cu:22-33          (op latent_gather)
//   kern_k3_land_situ       source/k3_land.cu:211-237          (op land_situ_n33792: SiTU on an f32 partial)
//   kern_k3_land            source/k3_land.cu:166-188          (f32 -> bf16 landing of a column band)
//   kern_k3_rms             source/k3_land.cu:107-160          (stand-alone latent RMSNorm)
//
// SiTU: act = bf16((4 tanh(g/4) * sigmoid(g)) * 25 tanh(u/25)), g = sp[row, i], u = sp[row, n + i].
// The activation uses the same hardware approximations as the reference (tanh.approx, ex2.approx in
// __expf, a round-to-nearest reciprocal), so it is the same function of the same bf16 inputs.
// Latent RMSNorm: ln = bf16(lat * rs) (x) gamma with rs = rsqrt_rn(sum / h + 1e-5); the sum keeps the
// reference's order -- a per-vector fma chain over 8 elements, an xor-butterfly over each group of 32
// consecutive vectors, then one butterfly over the (up to 32) group sums.
//
// Layout for B200: one launch of short 128-thread blocks, one in four of which normalises latent rows
// (2 rows per item, all 8 vector loads of a thread issued up front) while the others run SiTU items (512
// consecutive vectors of the flat activation, 8 loads per thread up front); 64 registers per thread keep 8
// blocks resident per SM, so the latency-bound norm hides under the MUFU-bound activation as in the
// reference's 1:2 job split.
#include "k3g_device.cuh"
#include "k3g_host.h"
#include "situ_math.cuh"

using namespace k3g;

namespace {

__device__ __forceinline__ V8 situ_vec(const V8& g, const V8& u) {
  V8 o;
#pragma unroll
  for (int j = 0; j < 4; ++j) o.w[j] = pack_bf2(situ_value(bf_lo(g.w[j]), bf_lo(u.w[j])), situ_value(bf_hi(g.w[j]), bf_hi(u.w[j])));
  return o;
}

constexpr int kRmsRows = 2;      // rows per norm item

// sums[r] = sum of squares of row r in the reference's order.  v[r][k] is vector (t + 128 k) of row r.
template <int ROWS, int VPT>
__device__ __forceinline__ void rms_rows(const V8 (&v)[ROWS][VPT], int nvec, float* sm, float* sums) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      float p = 0.f;
      if (t + 128 * k < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = bf_lo(v[r][k].w[j]), hi = bf_hi(v[r][k].w[j]);
          p = __fmaf_rn(lo, lo, p);
          p = __fmaf_rn(hi, hi, p);
        }
      }
      p = butterfly_sum<32>(p);                           // group (warp + 4 k) of 32 consecutive vectors
      if (lane == 0) sm[r * 32 + warp + 4 * k] = p;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const float x = lane < 4 * VPT ? sm[r * 32 + lane] : 0.f;   // groups past the row's end hold 0, like the reference's idle warps
    sums[r] = butterfly_sum<32>(x);
  }
  __syncthreads();
}

template <int ROWS, int VPT>
__device__ __forceinline__ void rms_item(const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                         __nv_bfloat16* __restrict__ ln, int h, int L, int r0, float* sm) {
  const int t = threadIdx.x, nvec = h >> 3;
  V8 v[ROWS][VPT];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      v[r][k] = V8{{0u, 0u, 0u, 0u}};
      if (r0 + r < L && t + 128 * k < nvec) v[r][k] = ld_stream(lat + (size_t)(r0 + r) * h + (t + 128 * k) * 8);
    }
  }
  float sums[ROWS];
  rms_rows<ROWS, VPT>(v, nvec, sm, sums);
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (r0 + r >= L) continue;
    const float rs = __frsqrt_rn(__fadd_rn(__fdiv_rn(sums[r], (float)h), 1e-5f));
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (t + 128 * k >= nvec) continue;
      const V8 g = ld_keep(gam + (t + 128 * k) * 8);
      V8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(v[r][k].w[j]), rs), __fmul_rn(bf_hi(v[r][k].w[j]), rs)), g.w[j]);
      st_stream(ln + (size_t)(r0 + r) * h + (t + 128 * k) * 8, o);
    }
  }
}

// Rows wider than 4 x 128 vectors (h > 4096, not a shape of the reference deployment): one row at a time,
// vectors read once for the sum and again (from L2) for the output, so no vector stays in a register.
__device__ __noinline__ void rms_row_wide(const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                          __nv_bfloat16* __restrict__ ln, int h, int row, float* sm) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nvec = h >> 3;
  const int vpt = (nvec + 127) >> 7;
  const __nv_bfloat16* src = lat + (size_t)row * h;
  for (int k = 0; k < vpt; ++k) {
    float p = 0.f;
    if (t + 128 * k < nvec) {
      const V8 v = ld_plain(src + (t + 128 * k) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf_lo(v.w[j]), hi = bf_hi(v.w[j]);
        p = __fmaf_rn(lo, lo, p);
        p = __fmaf_rn(hi, hi, p);
      }
    }
    p = butterfly_sum<32>(p);
    if (lane == 0) sm[warp + 4 * k] = p;
  }
  __syncthreads();
  const float sum = butterfly_sum<32>(lane < 4 * vpt ? sm[lane] : 0.f);
  __syncthreads();
  const float rs = __frsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)h), 1e-5f));
  for (int k = 0; k < vpt; ++k) {
    if (t + 128 * k >= nvec) continue;
    const V8 v = ld_plain(src + (t + 128 * k) * 8), g = ld_keep(gam + (t + 128 * k) * 8);
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(v.w[j]), rs), __fmul_rn(bf_hi(v.w[j]), rs)), g.w[j]);
    st_stream(ln + (size_t)row * h + (t + 128 * k) * 8, o);
  }
}

// One SiTU item: kSituVec x 128 consecutive 16-byte vectors of the flat [B][n / 8] activation; every load
// of the item is issued before the first store.
#ifndef K3G_SITU_VEC
#define K3G_SITU_VEC 4
#endif
constexpr int kSituVec = K3G_SITU_VEC;
// item_max != nullptr: item_max[chunk] = max |act| over the item (bit-pattern maximum, as the per-tensor FP8
// amax pass takes it), so a following quantisation of act can skip its own pass over the tensor.
__device__ __forceinline__ void situ_item(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act, unsigned nv, unsigned total,
                                          unsigned chunk, float* __restrict__ item_max = nullptr, unsigned* s_max = nullptr) {
  const unsigned base = chunk * (kSituVec * 128u) + threadIdx.x;
  V8 g[kSituVec], u[kSituVec];
  size_t off[kSituVec];
#pragma unroll
  for (int k = 0; k < kSituVec; ++k) {
    const unsigned idx = base + 128u * k;
    if (idx < total) {
      const unsigned row = idx / nv, col = idx - row * nv;
      const __nv_bfloat16* p = sp + ((size_t)row * 2 * nv + col) * 8;
      g[k] = ld_stream(p);
      u[k] = ld_stream(p + (size_t)nv * 8);
      off[k] = (size_t)idx * 8;
    }
  }
  unsigned m2 = 0u;
#pragma unroll
  for (int k = 0; k < kSituVec; ++k)
    if (base + 128u * k < total) {
      const V8 o = situ_vec(g[k], u[k]);
#pragma unroll
      for (int j = 0; j < 4; ++j) m2 = __vmaxu2(m2, o.w[j] & 0x7fff7fffu);
      st_stream(act + off[k], o);
    }
  if (item_max != nullptr) {
    unsigned m = __reduce_max_sync(0xffffffffu, max(m2 & 0xffffu, m2 >> 16));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) item_max[chunk] = __uint_as_float(max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3])) << 16);
    __syncthreads();
  }
}

}  // namespace

// One latent row whose source is the ring-order reduce-scatter chain over NR ranks' partial buffers (k3g::rs_chain):
// the pull reduce-scatter folded into the norm that consumes it.  Two vectors (2 NR loads) in flight per thread.
template <int NR>
__device__ __forceinline__ void rms_row_pull(const uint4* const (&ring)[NR], const __nv_bfloat16* __restrict__ gam, __nv_bfloat16* __restrict__ ln,
                                             int h, int row, float* sm) {
  const int t = threadIdx.x, nvec = h >> 3;
  V8 v[1][4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    v[0][k] = V8{{0u, 0u, 0u, 0u}};
    if (t + 128 * k < nvec) v[0][k] = rs_chain<NR>(ring, (long long)row * nvec + t + 128 * k);
  }
  float sums[1];
  rms_rows<1, 4>(v, nvec, sm, sums);
  const float rs = __frsqrt_rn(__fadd_rn(__fdiv_rn(sums[0], (float)h), 1e-5f));
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (t + 128 * k >= nvec) continue;
    const V8 g = ld_keep(gam + (t + 128 * k) * 8);
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(v[0][k].w[j]), rs), __fmul_rn(bf_hi(v[0][k].w[j]), rs)), g.w[j]);
    st_stream(ln + (size_t)row * h + (t + 128 * k) * 8, o);
  }
}

// Work items: ceil(L / 2) norm items (2 latent rows each) and ceil(B * n / 4096) SiTU items (512 vectors
// each).  Blocks with blockIdx.x % K3G_SITU_MOD == 0 stride over the norm items, the others over the SiTU
// items, so that the hardware block scheduler keeps both kinds resident on every SM and the latency-bound
// norm hides under the MUFU-bound activation.  Any grid of at least K3G_SITU_MOD blocks and any block of at
// least 128 threads is valid (the reference launches 3 * ceil(tokens / 16) blocks of 512): a block is one
// team of 128 threads, further threads exit.  Requires n % 8 == 0, h % 8 == 0, h <= 8192, B * n / 8 < 2^31.
#ifndef K3G_SITU_MOD
#define K3G_SITU_MOD 5
#endif
#ifndef K3G_SITU_IPB
#define K3G_SITU_IPB 1
#endif
__device__ __forceinline__ void situ_rms_blocks(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                                __nv_bfloat16* __restrict__ ln, int n, int B, int h, int L, float* __restrict__ item_max) {
  __shared__ float sm[kRmsRows * 32];
  if (threadIdx.x >= 128) return;
  const unsigned nv = (unsigned)n >> 3, total = (unsigned)B * nv;
  const unsigned RG = (unsigned)(L + kRmsRows - 1) / kRmsRows, SC = (total + kSituVec * 128u - 1) / (kSituVec * 128u);
  const unsigned q = blockIdx.x / K3G_SITU_MOD, job = blockIdx.x - q * K3G_SITU_MOD;
  const unsigned norm_blocks = (gridDim.x + K3G_SITU_MOD - 1) / K3G_SITU_MOD;
  if (job == 0) {
    const int vpt = ((h >> 3) + 127) >> 7;
    for (unsigned r = q; r < RG; r += norm_blocks) {
      const int r0 = (int)r * kRmsRows;
      if (vpt <= 4) {
        rms_item<kRmsRows, 4>(lat, gam, ln, h, L, r0, sm);
      } else {
        for (int w = 0; w < kRmsRows && r0 + w < L; ++w) rms_row_wide(lat, gam, ln, h, r0 + w, sm);
      }
    }
  } else {
    const unsigned situ_blocks = gridDim.x - norm_blocks;
    for (unsigned c = blockIdx.x - q - 1; c < SC; c += situ_blocks) situ_item(sp, act, nv, total, c, item_max, reinterpret_cast<unsigned*>(sm));
  }
}
extern "C" __global__ void __launch_bounds__(512) kern_k3_situ_rms_bf16(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                                       const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                                                       __nv_bfloat16* __restrict__ ln, int n, int B, int h, int L) {
  situ_rms_blocks(sp, act, lat, gam, ln, n, B, h, L, nullptr);
}
// The same launch, with item_max [ceil(B * n / 4096)] f32 = max |act| per SiTU item.
__global__ void __launch_bounds__(512) situ_rms_amax_kernel(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                            const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                                            __nv_bfloat16* __restrict__ ln, int n, int B, int h, int L, float* __restrict__ item_max) {
  situ_rms_blocks(sp, act, lat, gam, ln, n, B, h, L, item_max);
}

// SiTU landing + latent RMSNorm with the latent rows pulled from every rank's partial buffer [NR * L, h] (row
// rank * L + r, ring order, one bf16 rounding per hop): every other block pulls and normalises one row per item,
// the others run SiTU items, so the activation hides under the NVLink transfer.  h <= 4096.
template <int NR>
__global__ void __launch_bounds__(128) rs_situ_rms_kernel(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                          const __nv_bfloat16* __restrict__ partial, const unsigned long long* __restrict__ partial_peer,
                                                          int rank, const __nv_bfloat16* __restrict__ gam, __nv_bfloat16* __restrict__ ln, int n, int B,
                                                          int h, int L, float* __restrict__ item_max) {
  __shared__ float sm[kRmsRows * 32];
  const unsigned nv = (unsigned)n >> 3, total = (unsigned)B * nv;
  const unsigned SC = (total + kSituVec * 128u - 1) / (kSituVec * 128u);
  const unsigned q = blockIdx.x >> 1, pull_blocks = (gridDim.x + 1) >> 1;
  if ((blockIdx.x & 1) == 0) {
    const uint4* ring[NR];
    rs_bases<NR, NR - 1, 0>(partial, partial_peer, (long long)rank * L * h, rank, ring);
    for (unsigned r = q; r < (unsigned)L; r += pull_blocks) rms_row_pull<NR>(ring, gam, ln, h, (int)r, sm);
  } else {
    const unsigned situ_blocks = gridDim.x - pull_blocks;
    for (unsigned c = q; c < SC; c += situ_blocks) situ_item(sp, act, nv, total, c, item_max, reinterpret_cast<unsigned*>(sm));
  }
}

#if defined(K3G_CUBIN_ONLY) && defined(K3G_FUSED_ENTRIES)
// Module k3g_fused_situ, op rs_situ_rms (second launch; the first is the arrive barrier) of a manifest rewritten by
// `patch_manifest.py --fuse`: kern_k3_situ_rms_bf16 with the latent rows pulled from every rank's partial buffer and
// the item maxima for the following quantisation.  The tensor-parallel width is a build constant (K3G_NR).
#ifndef K3G_NR
#define K3G_NR 4
#endif
extern "C" __global__ void __launch_bounds__(128) kern_k3g_rs_situ_rms(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                                      const __nv_bfloat16* __restrict__ partial,
                                                                      const unsigned long long* __restrict__ partial_peer, int rank, int nranks,
                                                                      const __nv_bfloat16* __restrict__ gam, __nv_bfloat16* __restrict__ ln, int n,
                                                                      int B, int h, int L, float* __restrict__ item_max) {
  if (nranks != K3G_NR) return;
  __shared__ float sm[kRmsRows * 32];
  const unsigned nv = (unsigned)n >> 3, total = (unsigned)B * nv;
  const unsigned SC = (total + kSituVec * 128u - 1) / (kSituVec * 128u);
  const unsigned q = blockIdx.x >> 1, pull_blocks = (gridDim.x + 1) >> 1;
  if ((blockIdx.x & 1) == 0) {
    const uint4* ring[K3G_NR];
    rs_bases<K3G_NR, K3G_NR - 1, 0>(partial, partial_peer, (long long)rank * L * h, rank, ring);
    for (unsigned r = q; r < (unsigned)L; r += pull_blocks) rms_row_pull<K3G_NR>(ring, gam, ln, h, (int)r, sm);
  } else {
    const unsigned situ_blocks = gridDim.x - pull_blocks;
    for (unsigned c = q; c < SC; c += situ_blocks) situ_item(sp, act, nv, total, c, item_max, reinterpret_cast<unsigned*>(sm));
  }
}
#endif

// ---- f32 landings (module k3_land) -----------------------------------------------------------------
// row / column of flat index i over rows of `width` items: 32-bit division whenever the index fits
__device__ __forceinline__ void split_index(long long i, int width, long long& row, int& col) {
  if (i < (1ll << 32)) {
    const unsigned r = (unsigned)i / (unsigned)width;
    row = r; col = (int)((unsigned)i - r * (unsigned)width);
  } else {
    row = i / width; col = (int)(i - row * width);
  }
}

__device__ __forceinline__ float land_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// act[b, i] = bf16(SiTU(bf16(p[b, i]), bf16(p[b, n + i]))): both operands land to bf16 before the activation.
// Flat over the B * n / 4 groups of four elements, any 1-D or 2-D grid (the reference launches (B, ceil(n / 1024))
// blocks of 1024); n % 4 != 0 takes the element-wise path.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_land_situ(const float* __restrict__ p, __nv_bfloat16* __restrict__ act, int n, int B) {
  const long long nthreads = (long long)gridDim.x * gridDim.y * blockDim.x;
  const long long tid = ((long long)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
  if ((n & 3) == 0) {
    const int nq = n >> 2;
    const long long items = (long long)B * nq;
    for (long long i0 = tid; i0 < items; i0 += 2 * nthreads) {       // two groups (four 16-byte loads) in flight per thread
      const long long i1 = i0 + nthreads;
      long long r0, r1;
      int c0, c1;
      split_index(i0, nq, r0, c0);
      split_index(i1, nq, r1, c1);
      const float4 g0 = __ldcs(reinterpret_cast<const float4*>(p + r0 * 2 * n) + c0), u0 = __ldcs(reinterpret_cast<const float4*>(p + r0 * 2 * n + n) + c0);
      float4 g1 = g0, u1 = u0;
      if (i1 < items) { g1 = __ldcs(reinterpret_cast<const float4*>(p + r1 * 2 * n) + c1); u1 = __ldcs(reinterpret_cast<const float4*>(p + r1 * 2 * n + n) + c1); }
      st_stream8(act + r0 * n + 4 * c0, pack_bf2(situ_value(land_bf16(g0.x), land_bf16(u0.x)), situ_value(land_bf16(g0.y), land_bf16(u0.y))),
                 pack_bf2(situ_value(land_bf16(g0.z), land_bf16(u0.z)), situ_value(land_bf16(g0.w), land_bf16(u0.w))));
      if (i1 < items)
        st_stream8(act + r1 * n + 4 * c1, pack_bf2(situ_value(land_bf16(g1.x), land_bf16(u1.x)), situ_value(land_bf16(g1.y), land_bf16(u1.y))),
                   pack_bf2(situ_value(land_bf16(g1.z), land_bf16(u1.z)), situ_value(land_bf16(g1.w), land_bf16(u1.w))));
    }
  } else {
    const long long items = (long long)B * n;
    for (long long i = tid; i < items; i += nthreads) {
      long long r;
      int c;
      split_index(i, n, r, c);
      act[i] = __float2bfloat16_rn(situ_value(land_bf16(p[r * 2 * n + c]), land_bf16(p[r * 2 * n + n + c])));
    }
  }
}

// o[b, i] = bf16(p[b * ldc + off + i]), i < n.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_land(const float* __restrict__ p, __nv_bfloat16* __restrict__ o, int n, int off, int ldc, int B) {
  const long long nthreads = (long long)gridDim.x * gridDim.y * blockDim.x;
  const long long tid = ((long long)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
  if (((n | off | ldc) & 3) == 0) {
    const int nq = n >> 2;
    const long long items = (long long)B * nq;
    for (long long i = tid; i < items; i += nthreads) {
      long long r;
      int c;
      split_index(i, nq, r, c);
      const float4 v = __ldcs(reinterpret_cast<const float4*>(p + r * ldc + off) + c);
      st_stream8(o + r * n + 4 * c, pack_bf2(v.x, v.y), pack_bf2(v.z, v.w));
    }
  } else {
    const long long items = (long long)B * n;
    for (long long i = tid; i < items; i += nthreads) {
      long long r;
      int c;
      split_index(i, n, r, c);
      o[i] = __float2bfloat16_rn(p[r * ldc + off + c]);
    }
  }
}

// o [B, h] = bf16(x * rs) (x) gamma, rs = rsqrt_rn(sum x^2 / h + 1e-5): the norm items of kern_k3_situ_rms_bf16 alone.
// The sum's order is the one a 1024-thread block of the reference produces for h <= 8192 (one vector per
// thread): warp w sums vectors 32 w .. 32 w + 31 by butterfly, warp 0 sums the warp totals.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_rms(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                                              __nv_bfloat16* __restrict__ o, int h, int B) {
  __shared__ float sm[kRmsRows * 32];
  if (threadIdx.x >= 128) return;
  const int vpt = ((h >> 3) + 127) >> 7;
  const int groups = (B + kRmsRows - 1) / kRmsRows;
  for (int q = blockIdx.x; q < groups; q += gridDim.x) {
    const int r0 = q * kRmsRows;
    if (vpt <= 4) {
      rms_item<kRmsRows, 4>(x, gamma, o, h, B, r0, sm);
    } else {
      for (int w = 0; w < kRmsRows && r0 + w < B; ++w) rms_row_wide(x, gamma, o, h, r0 + w, sm);
    }
  }
}


// out = bf16(attn * bf16(sigmoid(gate))), gate a strided per-head view: gate(t, h, d) = gate + t * tstride + h * hstride + d.
extern "C" __global__ void __launch_bounds__(256) kern_sigmoid_mul_bf16(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ attn,
                                                                       const __nv_bfloat16* __restrict__ gate, int heads, int head_dim,
                                                                       int gate_tstride, int gate_hstride) {
  // programmatic dependent launch, as in the reference: nothing produced by the previous kernel is
  // touched before the wait, and the next launch may start its prologue right after it
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int n = heads * head_dim;
  const int j = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (j >= n) return;
  const int h = j / head_dim, d = j - h * head_dim;
  const long long t = blockIdx.x;                             // one token row per block in x
  const V8 gv = ld_stream(gate + t * gate_tstride + (long long)h * gate_hstride + d);
  const V8 av = ld_stream(attn + t * n + j);
  V8 o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.w[i] = mul_bf2(av.w[i], f2_to_bf2(f2_fast_sigmoid(f2_from_bf2(gv.w[i]))));
  st_stream(out + t * n + j, o);
}

#ifndef HEADS
#define HEADS 24
#endif
// rec <-> buf copy of the sequence's KDA recurrent state ([HEADS][128][128] f32): grid (HEADS, 32), block 128.
extern "C" __global__ void __launch_bounds__(128) kern_k3_span_state(void* __restrict__ kda_base, const int* __restrict__ line_index,
                                                                    long long line_bytes, const int* __restrict__ span_at,
                                                                    float* __restrict__ buf, int to_line) {
  float4* rec = reinterpret_cast<float4*>(reinterpret_cast<char*>(kda_base) + (long long)line_index[span_at[0]] * line_bytes) + (size_t)blockIdx.x * 4096;
  float4* b = reinterpret_cast<float4*>(buf) + (size_t)blockIdx.x * 4096;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < 4096; j += gridDim.y * blockDim.x) {
    if (to_line) rec[j] = __ldcs(b + j);
    else __stcs(b + j, rec[j]);
  }
}

// The sequence's cached latent rows laid contiguous: out[t] = page row t for t < lens[0], zero after.
extern "C" __global__ void __launch_bounds__(576) kern_k3_latent_gather(const __nv_bfloat16* __restrict__ slab, const int* __restrict__ block_table,
                                                                       long long page_stride, const int* __restrict__ lens,
                                                                       __nv_bfloat16* __restrict__ out, int n) {
  const int lanes = 72;                                      // a 576-element row is 72 x 16 bytes
  const int rows_per_block = blockDim.x / lanes;
  const int lane = threadIdx.x % lanes, sub = threadIdx.x / lanes;
  if (sub >= rows_per_block) return;
  const int len = lens[0];
  for (int t = blockIdx.x * rows_per_block + sub; t < n; t += gridDim.x * rows_per_block) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t < len) v = __ldg(reinterpret_cast<const uint4*>(slab + block_table[t / 64] * page_stride + (long long)(t % 64) * 576) + lane);
    __stcs(reinterpret_cast<uint4*>(out + (long long)t * 576) + lane, v);
  }
}

#ifndef K3G_CUBIN_ONLY
static int situ_rms_impl(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* item_max,
                         void* stream) {
  K3G_REQUIRE_PTR(sp); K3G_REQUIRE_PTR(act); K3G_REQUIRE_PTR(lat); K3G_REQUIRE_PTR(gam); K3G_REQUIRE_PTR(ln);
  K3G_REQUIRE_ALIGNED(sp); K3G_REQUIRE_ALIGNED(act); K3G_REQUIRE_ALIGNED(lat); K3G_REQUIRE_ALIGNED(gam); K3G_REQUIRE_ALIGNED(ln);
  K3G_REQUIRE(n > 0 && n % 8 == 0 && h > 0 && h % 8 == 0 && h <= 8192 && B >= 0 && L >= 0, K3G_ESHAPE);
  if (B == 0 && L == 0) return K3G_OK;
  K3G_REQUIRE((long long)B * (n / 8) < (1ll << 31), K3G_ESHAPE);
  // K3G_SITU_IPB items per block: short blocks, so the block scheduler balances the two kinds of work
  const long long rg = (L + kRmsRows - 1) / kRmsRows, sc = ((long long)B * (n / 8) + kSituVec * 128 - 1) / (kSituVec * 128);
  const long long nb = (rg + K3G_SITU_IPB - 1) / K3G_SITU_IPB, sb = (sc + K3G_SITU_IPB * (K3G_SITU_MOD - 1) - 1) / (K3G_SITU_IPB * (K3G_SITU_MOD - 1));
  long long q = K3G_SITU_MOD * (nb > sb ? nb : sb);
  if (q < K3G_SITU_MOD) q = K3G_SITU_MOD;
  K3G_REQUIRE(q < (1ll << 31), K3G_ESHAPE);
  if (item_max)
    situ_rms_amax_kernel<<<(unsigned)q, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)sp, (__nv_bfloat16*)act, (const __nv_bfloat16*)lat,
                                                                     (const __nv_bfloat16*)gam, (__nv_bfloat16*)ln, n, B, h, L, (float*)item_max);
  else
    kern_k3_situ_rms_bf16<<<(unsigned)q, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)sp, (__nv_bfloat16*)act, (const __nv_bfloat16*)lat,
                                                                      (const __nv_bfloat16*)gam, (__nv_bfloat16*)ln, n, B, h, L);
  return k3g_launch_status();
}

K3G_API int k3g_situ_rms(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* stream) {
  return situ_rms_impl(sp, act, lat, gam, ln, n, B, h, L, nullptr, stream);
}

// The same call with item_max [ceil(B * n / 4096)] f32 = max |act| over each run of 4096 consecutive elements of
// act: the partials a following k3g_quant_fp8_apply of act takes instead of a pass over the tensor.
K3G_API int k3g_situ_rms_amax(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* item_max,
                              void* stream) {
  K3G_REQUIRE_PTR(item_max);
  return situ_rms_impl(sp, act, lat, gam, ln, n, B, h, L, item_max, stream);
}

// Pull reduce-scatter folded into the latent norm (no counterpart in the reference, which runs kern_k3_rs_pull and then
// kern_k3_situ_rms_bf16): partial = this rank's [nranks * L, h] bf16 partial sums, partial_peer = u64 table of every
// rank's buffer; ln [L, h] is the norm of the ring-order chain of rows rank * L + r, bit-identical to the two calls in
// sequence.  Bracket with k3g_rs_arrive as for k3g_rs_pull.  h <= 4096; nranks 1, 2, 4 or 8; item_max may be null.
K3G_API int k3g_rs_situ_rms(const void* sp, void* act, const void* partial, const void* partial_peer, int rank, int nranks, const void* gam,
                            void* ln, int n, int B, int h, int L, void* item_max, void* stream) {
  K3G_REQUIRE_PTR(sp); K3G_REQUIRE_PTR(act); K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(partial_peer); K3G_REQUIRE_PTR(gam); K3G_REQUIRE_PTR(ln);
  K3G_REQUIRE_ALIGNED(sp); K3G_REQUIRE_ALIGNED(act); K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(gam); K3G_REQUIRE_ALIGNED(ln);
  K3G_REQUIRE(n > 0 && n % 8 == 0 && h > 0 && h % 8 == 0 && h <= 4096 && B >= 0 && L >= 0, K3G_ESHAPE);
  K3G_REQUIRE(nranks == 1 || nranks == 2 || nranks == 4 || nranks == 8, K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks, K3G_ERANGE);
  if (B == 0 && L == 0) return K3G_OK;
  K3G_REQUIRE((long long)B * (n / 8) < (1ll << 31), K3G_ESHAPE);
  const long long sc = ((long long)B * (n / 8) + kSituVec * 128 - 1) / (kSituVec * 128);
  long long q = 2 * (L > sc ? L : sc);
  if (q < 2) q = 2;
  K3G_REQUIRE(q < (1ll << 31), K3G_ESHAPE);
#define K3G_RS_SITU(NR)                                                                                                                      \
  rs_situ_rms_kernel<NR><<<(unsigned)q, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)sp, (__nv_bfloat16*)act, (const __nv_bfloat16*)partial, \
                                                                     (const unsigned long long*)partial_peer, rank, (const __nv_bfloat16*)gam,   \
                                                                     (__nv_bfloat16*)ln, n, B, h, L, (float*)item_max)
  switch (nranks) {
    case 1: K3G_RS_SITU(1); break;
    case 2: K3G_RS_SITU(2); break;
    case 4: K3G_RS_SITU(4); break;
    default: K3G_RS_SITU(8); break;
  }
#undef K3G_RS_SITU
  return k3g_launch_status();
}

K3G_API int k3g_land_situ(const void* p, void* act, int n, int B, void* stream) {
  K3G_REQUIRE_PTR(p); K3G_REQUIRE_PTR(act);
  K3G_REQUIRE_ALIGNED(p); K3G_REQUIRE_ALIGNED(act);
  K3G_REQUIRE(n > 0 && B >= 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  const long long items = (n & 3) ? (long long)B * n : (long long)B * (n >> 2);
  long long blocks = (items + 511) / 512;                 // 256 threads, two groups each
  if (blocks > (1ll << 30)) blocks = 1ll << 30;
  kern_k3_land_situ<<<(unsigned)blocks, 256, 0, k3g_stream(stream)>>>((const float*)p, (__nv_bfloat16*)act, n, B);
  return k3g_launch_status();
}

K3G_API int k3g_land(const void* p, void* o, int n, int off, int ldc, int B, void* stream) {
  K3G_REQUIRE_PTR(p); K3G_REQUIRE_PTR(o);
  K3G_REQUIRE_ALIGNED(p); K3G_REQUIRE_ALIGNED(o);
  K3G_REQUIRE(n > 0 && off >= 0 && ldc >= off + n && B >= 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  const long long items = ((n | off | ldc) & 3) ? (long long)B * n : (long long)B * (n >> 2);
  long long blocks = (items + 255) / 256;
  if (blocks > (1ll << 30)) blocks = 1ll << 30;
  kern_k3_land<<<(unsigned)blocks, 256, 0, k3g_stream(stream)>>>((const float*)p, (__nv_bfloat16*)o, n, off, ldc, B);
  return k3g_launch_status();
}

K3G_API int k3g_rms(const void* x, const void* gamma, void* o, int h, int B, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(o);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(o);
  K3G_REQUIRE(h > 0 && h % 8 == 0 && h <= 8192 && B >= 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  kern_k3_rms<<<(unsigned)((B + kRmsRows - 1) / kRmsRows), 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma,
                                                                                        (__nv_bfloat16*)o, h, B);
  return k3g_launch_status();
}

K3G_API int k3g_sigmoid_mul(void* out, const void* attn, const void* gate, int tokens, int heads, int head_dim, int gate_tstride,
                            int gate_hstride, void* stream) {
  K3G_REQUIRE_PTR(out); K3G_REQUIRE_PTR(attn); K3G_REQUIRE_PTR(gate);
  K3G_REQUIRE_ALIGNED(out); K3G_REQUIRE_ALIGNED(attn); K3G_REQUIRE_ALIGNED(gate);
  K3G_REQUIRE(tokens >= 0 && heads > 0 && head_dim > 0 && head_dim % 8 == 0 && gate_tstride % 8 == 0 && gate_hstride % 8 == 0, K3G_ESHAPE);
  if (tokens == 0) return K3G_OK;
  const dim3 grid((unsigned)tokens, (unsigned)((heads * head_dim + 2047) / 2048), 1);
  kern_sigmoid_mul_bf16<<<grid, 256, 0, k3g_stream(stream)>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, heads,
                                                             head_dim, gate_tstride, gate_hstride);
  return k3g_launch_status();
}

// The reference fixes the head count when the module is built (HEADS, = gridDim.x of its launch); the kernel here takes it
// from the grid, so the library entry serves any count: `heads` heads of [128][128] f32 = heads * 64 KB per direction.
K3G_API int k3g_span_state(void* kda_base, const void* line_index, long long line_bytes, const void* span_at, void* buf, int to_line,
                           int heads, void* stream) {
  K3G_REQUIRE_PTR(kda_base); K3G_REQUIRE_PTR(line_index); K3G_REQUIRE_PTR(span_at); K3G_REQUIRE_PTR(buf);
  K3G_REQUIRE_ALIGNED(kda_base); K3G_REQUIRE_ALIGNED(buf); K3G_REQUIRE(line_bytes % 16 == 0, K3G_EALIGN);
  K3G_REQUIRE(heads > 0 && heads <= 65535 && (long long)heads * 65536 <= line_bytes, K3G_ESHAPE);
  kern_k3_span_state<<<dim3((unsigned)heads, 32, 1), 128, 0, k3g_stream(stream)>>>(kda_base, (const int*)line_index, line_bytes, (const int*)span_at,
                                                                                 (float*)buf, to_line);
  return k3g_launch_status();
}

K3G_API int k3g_latent_gather(const void* slab, const void* block_table, long long page_stride, const void* lens, void* out, int n,
                              void* stream) {
  K3G_REQUIRE_PTR(slab); K3G_REQUIRE_PTR(block_table); K3G_REQUIRE_PTR(lens); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE_ALIGNED(slab); K3G_REQUIRE_ALIGNED(out); K3G_REQUIRE(page_stride % 8 == 0, K3G_EALIGN);
  K3G_REQUIRE(n >= 0, K3G_ESHAPE);
  if (n == 0) return K3G_OK;
  kern_k3_latent_gather<<<(n + 7) / 8, 576, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)slab, (const int*)block_table, page_stride,
                                                                    (const int*)lens, (__nv_bfloat16*)out, n);
  return k3g_launch_status();
}
#endif
