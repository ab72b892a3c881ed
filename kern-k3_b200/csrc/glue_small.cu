// The remaining per-layer glue of the prefill program: shared-expert SiTU landing + MoE latent
// RMSNorm, the MLA output gate, and the two state/cache staging copies.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   kern_k3_situ_rms_bf16   source/k3_land_fused.cu:123-202   (op land_situ_rms)
//   kern_sigmoid_mul_bf16   source/sigmoid_mul.cu:15-44        (op mla_gate)
//   kern_k3_span_state      source/k3_span_state.cu:19-29      (ops span_state_load / span_state_store)
//   kern_k3_latent_gather   source/k3_mla_v2.cu:22-33          (op latent_gather)
//
// SiTU: act = bf16((4 tanh(g/4) * sigmoid(g)) * 25 tanh(u/25)), g = sp[row, i], u = sp[row, n + i].
// The activation uses the same hardware approximations as the reference (tanh.approx, ex2.approx in
// __expf, a round-to-nearest reciprocal), so it is the same function of the same bf16 inputs.
// Latent RMSNorm: ln = bf16(lat * rs) (x) gamma with rs = rsqrt_rn(sum / h + 1e-5); the sum keeps the
// reference's order -- a per-vector fma chain over 8 elements, an xor-butterfly over each group of 32
// consecutive vectors, then one butterfly over the (up to 32) group sums.
//
// Layout for B200: one launch, every block is a team of 128 threads; blocks with blockIdx.x % 3 == 0
// normalise latent rows (4 per pass, all 4 x 4 vector loads of the team's threads issued up front),
// the others run the SiTU stream (2 rows per pass), so the latency-bound norm hides under the
// MUFU/HBM-bound activation exactly as in the reference's job split, with grid-stride passes.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {

__device__ __forceinline__ float tanh_approx(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float situ1(float g, float u) {
  const float a = 4.0f * tanh_approx(g * 0.25f);
  const float s = __frcp_rn(1.0f + __expf(-g));
  const float c = 25.0f * tanh_approx(u * 0.04f);
  return (a * s) * c;
}
__device__ __forceinline__ V8 situ8(const V8& g, const V8& u) {
  V8 o;
#pragma unroll
  for (int j = 0; j < 4; ++j) o.w[j] = pack_bf2(situ1(bf_lo(g.w[j]), bf_lo(u.w[j])), situ1(bf_hi(g.w[j]), bf_hi(u.w[j])));
  return o;
}

constexpr int kRmsRows = 4;      // rows per norm pass (= the reference's RMS_R, so its grid maps one block to one pass)
constexpr int kSituRows = 2;     // rows per SiTU pass
constexpr int kMaxVpt = 8;       // vectors per thread of a 128-thread team: h <= 8192

// sums[r] = sum of squares of row r in the reference's order.  v[r][k] is vector (t + 128 k) of row r.
template <int VPT>
__device__ __forceinline__ void rms_rows(const V8 (&v)[kRmsRows][VPT], int nvec, float* sm, float* sums) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll
  for (int r = 0; r < kRmsRows; ++r) {
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
  for (int r = 0; r < kRmsRows; ++r) {
    const float x = lane < 4 * VPT ? sm[r * 32 + lane] : 0.f;   // groups past the row's end hold 0, like the reference's idle warps
    sums[r] = butterfly_sum<32>(x);
  }
  __syncthreads();
}

template <int VPT>
__device__ __forceinline__ void rms_job(const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                        __nv_bfloat16* __restrict__ ln, int h, int L, int pass, int npass_stride, float* sm) {
  const int t = threadIdx.x, nvec = h >> 3;
  const int groups = (L + kRmsRows - 1) / kRmsRows;
  for (int q = pass; q < groups; q += npass_stride) {
    const int r0 = q * kRmsRows;
    V8 v[kRmsRows][VPT];
#pragma unroll
    for (int r = 0; r < kRmsRows; ++r) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        v[r][k] = V8{{0u, 0u, 0u, 0u}};
        if (r0 + r < L && t + 128 * k < nvec) v[r][k] = ld_stream(lat + (size_t)(r0 + r) * h + (t + 128 * k) * 8);
      }
    }
    float sums[kRmsRows];
    rms_rows<VPT>(v, nvec, sm, sums);
#pragma unroll
    for (int r = 0; r < kRmsRows; ++r) {
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
}

__device__ __forceinline__ void situ_job(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act, int n, int B, int pass,
                                         int npass_stride) {
  const int nv = n >> 3;
  const int groups = (B + kSituRows - 1) / kSituRows;
  for (int j0 = pass; j0 < groups; j0 += npass_stride) {
#pragma unroll
    for (int r = 0; r < kSituRows; ++r) {
      const int row = kSituRows * j0 + r;
      if (row >= B) break;
      const __nv_bfloat16* grow = sp + (size_t)row * 2 * n;
      __nv_bfloat16* orow = act + (size_t)row * n;
      for (int v0 = threadIdx.x; v0 < nv; v0 += 2 * blockDim.x) {       // two vectors (four loads) in flight per thread
        const int v1 = v0 + blockDim.x;
        const V8 g0 = ld_stream(grow + v0 * 8), u0 = ld_stream(grow + n + v0 * 8);
        V8 g1, u1;
        if (v1 < nv) { g1 = ld_stream(grow + v1 * 8); u1 = ld_stream(grow + n + v1 * 8); }
        st_stream(orow + v0 * 8, situ8(g0, u0));
        if (v1 < nv) st_stream(orow + v1 * 8, situ8(g1, u1));
      }
    }
  }
}

}  // namespace

// grid: any multiple of 3 blocks (the reference launches 3 * ceil(tokens / 16) blocks of 512 threads; a
// team here is 128 threads, so a 512-thread block simply idles its upper warps' vector slots -- the
// vector ownership t + 128 k only uses threadIdx.x < 128).  Requires n % 8 == 0, h % 8 == 0, h <= 8192.
extern "C" __global__ void __launch_bounds__(512) kern_k3_situ_rms_bf16(const __nv_bfloat16* __restrict__ sp, __nv_bfloat16* __restrict__ act,
                                                                       const __nv_bfloat16* __restrict__ lat, const __nv_bfloat16* __restrict__ gam,
                                                                       __nv_bfloat16* __restrict__ ln, int n, int B, int h, int L) {
  __shared__ float sm[kRmsRows * 32];
  const int q = blockIdx.x / 3, job = blockIdx.x - 3 * q, stride = gridDim.x / 3;
  if (job == 0) {
    if (threadIdx.x >= 128) return;                        // one 128-thread team per norm block
    const int vpt = ((h >> 3) + 127) >> 7;
    if (vpt <= 4) rms_job<4>(lat, gam, ln, h, L, q, stride, sm);
    else rms_job<kMaxVpt>(lat, gam, ln, h, L, q, stride, sm);
  } else {
    situ_job(sp, act, n, B, 2 * q + (job - 1), 2 * stride);
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
K3G_API int k3g_situ_rms(const void* sp, void* act, const void* lat, const void* gam, void* ln, int n, int B, int h, int L, void* stream) {
  K3G_REQUIRE_PTR(sp); K3G_REQUIRE_PTR(act); K3G_REQUIRE_PTR(lat); K3G_REQUIRE_PTR(gam); K3G_REQUIRE_PTR(ln);
  K3G_REQUIRE_ALIGNED(sp); K3G_REQUIRE_ALIGNED(act); K3G_REQUIRE_ALIGNED(lat); K3G_REQUIRE_ALIGNED(gam); K3G_REQUIRE_ALIGNED(ln);
  K3G_REQUIRE(n > 0 && n % 8 == 0 && h > 0 && h % 8 == 0 && h <= 8192 && B >= 0 && L >= 0, K3G_ESHAPE);
  if (B == 0 && L == 0) return K3G_OK;
  const int rg = (L + kRmsRows - 1) / kRmsRows, sg = (B + kSituRows - 1) / kSituRows;
  int q = rg > (sg + 1) / 2 ? rg : (sg + 1) / 2;
  if (q < 1) q = 1;
  kern_k3_situ_rms_bf16<<<3 * q, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)sp, (__nv_bfloat16*)act, (const __nv_bfloat16*)lat,
                                                              (const __nv_bfloat16*)gam, (__nv_bfloat16*)ln, n, B, h, L);
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

// heads is a build constant of the reference module (HEADS); the library entry serves the 24-head build.
K3G_API int k3g_span_state(void* kda_base, const void* line_index, long long line_bytes, const void* span_at, void* buf, int to_line,
                           void* stream) {
  K3G_REQUIRE_PTR(kda_base); K3G_REQUIRE_PTR(line_index); K3G_REQUIRE_PTR(span_at); K3G_REQUIRE_PTR(buf);
  K3G_REQUIRE_ALIGNED(kda_base); K3G_REQUIRE_ALIGNED(buf); K3G_REQUIRE(line_bytes % 16 == 0, K3G_EALIGN);
  kern_k3_span_state<<<dim3(HEADS, 32, 1), 128, 0, k3g_stream(stream)>>>(kda_base, (const int*)line_index, line_bytes, (const int*)span_at,
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
