// KDA glue: causal depthwise conv (width 4) + SiLU on the q/k/v streams, and the output gate
// (per-head RMSNorm x sigmoid(gate)) with an optional fused MXFP8 epilogue.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   kern_k3_span_gather    source/k3_span_gather_v3.cu:251-293 (row math :131-142, window :236-248)
//   kern_k3_kda_out_gate   source/k3_kda_out_gate_v3.cu:36-118
//
// span conv.  Stream s in {q,k,v}; x_i[c] = partial[(at + i) * row_stride + s * inner + c], rows
// i < 0 come from the stored 3-row window; y = fma(x_i, w3, fma(x_{i-1}, w2, fma(x_{i-3}, w0,
// x_{i-2} * w1))) (the reference build's contraction of its four-term sum); sb = bf16(y); out = bf16(sb * sigmoid(sb)); the new window is the last three
// INPUT rows.  A thread owns 4 consecutive columns (8 bytes) and walks a run of rows with the three
// previous inputs sliding in registers, the next four row loads issued before the current four rows are computed
// and stored, seven blocks per SM;
// rows per block = max(3, ceil(span / gridDim.z)), so the reference launch (16 rows) and a coarser one
// (fewer halo re-reads) are both valid.  Three is the floor because only the block that starts at row 0
// may read the stored window: it also overwrites it, and a block starting at row 1 or 2 would race with
// that store.  The sigmoid is ex2.approx + rcp.approx, as in the
// reference: two MUFU ops per element is what a 6.5 TB/s stream leaves room for.
//
// output gate.  16 lanes per head, 8 consecutive d per lane: ss = fma chain, xor-butterfly over
// the 16 lanes, r = rsqrt(fma(ss, 1/128, eps)); o = bf16((a * r) * gamma_o); gt = bf16(sigmoid(g));
// gated = bf16(o * gt).  A 32-element MXFP8 group is four lanes of one head.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {

// A thread owns kVec = 4 consecutive columns (8 bytes): small register footprint (the three sliding
// taps, one chunk of rows, the next chunk's raw loads and 16 tap weights), so seven 128-thread blocks stay
// resident per SM (eight would spill the prefetched chunk with f32 taps; measured slower).
#ifndef K3G_SPAN_MINB
#define K3G_SPAN_MINB 7
#endif
constexpr int kVec = 4;
constexpr int kChunk = 4;

__device__ __forceinline__ uint2 ld8_stream(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ void unpack4(uint2 v, float* x) {
  x[0] = bf_lo(v.x); x[1] = bf_hi(v.x); x[2] = bf_lo(v.y); x[3] = bf_hi(v.y);
}

template <bool TAPS_BF16>
__device__ __forceinline__ void load_taps(const void* cw, size_t off, float* w) {
  if (TAPS_BF16) {
    unpack4(__ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(cw) + off)), w);
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(cw) + off));
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
  }
}

// One output row of 4 columns: y = fma(x, w3, fma(t2, w2, fma(t0, w0, t1 * w1))), sb = bf16(y),
// out = bf16(sb * sigmoid(sb)).
__device__ __forceinline__ uint2 conv_silu_row(const float* t0, const float* t1, const float* t2, const float* x, const float (*w)[kVec]) {
  unsigned o[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float y[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = 2 * j + h;
      float a = __fmul_rn(t1[k], w[1][k]);
      a = __fmaf_rn(t0[k], w[0][k], a);
      a = __fmaf_rn(t2[k], w[2][k], a);
      y[h] = __fmaf_rn(x[k], w[3][k], a);
    }
    const unsigned sbp = pack_bf2(y[0], y[1]);
    const float s0 = bf_lo(sbp), s1 = bf_hi(sbp);
    o[j] = pack_bf2(s0 * fast_sigmoid(s0), s1 * fast_sigmoid(s1));
  }
  return make_uint2(o[0], o[1]);
}

template <bool TAPS_BF16>
__device__ __forceinline__ void span_stream(const __nv_bfloat16* __restrict__ partial, long long row_stride, const void* __restrict__ cw,
                                            __nv_bfloat16* win, __nv_bfloat16* __restrict__ out, int inner, int s, int c, int row0,
                                            int row1, int span) {
  float w[4][kVec];
#pragma unroll
  for (int t = 0; t < 4; ++t) load_taps<TAPS_BF16>(cw, ((size_t)s * 4 + t) * inner + c, w[t]);
  const __nv_bfloat16* col = partial + (size_t)s * inner + c;
  float x[kChunk + 3][kVec];
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    const int i = row0 - 3 + t;
    unpack4(i < 0 ? *reinterpret_cast<const uint2*>(win + (size_t)(i + 3) * inner + c) : ld8_stream(col + (size_t)i * row_stride), x[t]);
  }
  // full chunks: no per-row predicates, pointers advance by constant strides.  The loads of chunk n + 1 are issued
  // before chunk n is computed and stored, so a thread always has a chunk of rows on its way from HBM.
  const __nv_bfloat16* pin = col + (size_t)row0 * row_stride;
  __nv_bfloat16* pout = out + (size_t)row0 * inner + c;
  int r = row0;
  uint2 raw[kChunk];
  if (r + kChunk <= row1) {
#pragma unroll
    for (int k = 0; k < kChunk; ++k) raw[k] = ld8_stream(pin + k * row_stride);
  }
  for (; r + kChunk <= row1; r += kChunk) {
#pragma unroll
    for (int k = 0; k < kChunk; ++k) unpack4(raw[k], x[3 + k]);
    pin += kChunk * row_stride;
    if (r + 2 * kChunk <= row1) {
#pragma unroll
      for (int k = 0; k < kChunk; ++k) raw[k] = ld8_stream(pin + k * row_stride);
    }
#pragma unroll
    for (int k = 0; k < kChunk; ++k) __stcs(reinterpret_cast<uint2*>(pout + (size_t)k * inner), conv_silu_row(x[k], x[k + 1], x[k + 2], x[k + 3], w));
#pragma unroll
    for (int t = 0; t < 3; ++t)
#pragma unroll
      for (int k = 0; k < kVec; ++k) x[t][k] = x[kChunk + t][k];
    pout += (size_t)kChunk * inner;
  }
  for (; r < row1; ++r) {                                   // ragged tail, one row at a time
    unpack4(ld8_stream(pin), x[3]);
    __stcs(reinterpret_cast<uint2*>(pout), conv_silu_row(x[0], x[1], x[2], x[3], w));
#pragma unroll
    for (int t = 0; t < 3; ++t)
#pragma unroll
      for (int k = 0; k < kVec; ++k) x[t][k] = x[t + 1][k];
    pin += row_stride;
    pout += inner;
  }
  if (row0 == 0) {
    // new window = inputs span-3 .. span-1 (old window rows when span < 3); this thread has
    // already read every old tap it needs, and no other thread reads these columns of the window
    // (blocks that start later begin at row >= 3: see the rows-per-block floor in span_gather_body)
    uint2 nw[3];
#pragma unroll
    for (int t = 0; t < 3; ++t) {
      const int i = span - 3 + t;
      nw[t] = i < 0 ? *reinterpret_cast<const uint2*>(win + (size_t)(i + 3) * inner + c) : ld8_stream(col + (size_t)i * row_stride);
    }
#pragma unroll
    for (int t = 0; t < 3; ++t) *reinterpret_cast<uint2*>(win + (size_t)t * inner + c) = nw[t];
  }
}

// beta transpose + flow landing for one z-chunk of rows, shared by the chunk's x-blocks: block x takes
// the heads h = x, x + gridDim.x, ... (stores along i stay contiguous) and the rows i = x mod gridDim.x
// of the flow band (256 contiguous bytes per row).
__device__ __forceinline__ void span_beta_flow(const float* __restrict__ wsm, int heads, __nv_bfloat16* __restrict__ span_beta,
                                               __nv_bfloat16* __restrict__ span_flow, int row0, int row1, int span) {
  const int R = row1 - row0, gx = (int)gridDim.x, bx = (int)blockIdx.x;
  const int nh = (heads - bx + gx - 1) / gx;
  for (int idx = threadIdx.x; idx < R * nh; idx += blockDim.x) {
    const int h = bx + (idx / R) * gx, i = row0 + idx % R;
    span_beta[(size_t)h * span + i] = __float2bfloat16_rn(__ldg(wsm + (size_t)i * 256 + h));
  }
  const int nr = (R - bx + gx - 1) / gx;
  for (int idx = threadIdx.x; idx < nr * 32; idx += blockDim.x) {
    const int i = row0 + bx + (idx / 32) * gx, c4 = (idx % 32) * 4;
    const float4 v = __ldcs(reinterpret_cast<const float4*>(wsm + (size_t)i * 256 + 96 + c4));
    *reinterpret_cast<uint2*>(span_flow + (size_t)i * 128 + c4) = make_uint2(pack_bf2(v.x, v.y), pack_bf2(v.z, v.w));
  }
}

// grid (ceil(inner / 512), 4, row chunks), block 128: y < 3 = stream, y == 3 = beta/flow (optional)
template <bool TAPS_BF16>
__device__ __forceinline__ void span_gather_body(const __nv_bfloat16* __restrict__ partial, long long row_stride, const void* __restrict__ cw,
                                                 __nv_bfloat16* win_base, const float* __restrict__ wsm_partial, __nv_bfloat16* span_q,
                                                 __nv_bfloat16* span_k, __nv_bfloat16* span_v, __nv_bfloat16* span_beta,
                                                 __nv_bfloat16* span_flow, int heads, int at, int span) {
  const int inner = heads * 128;
  // at least three rows per block: blocks z >= 1 then start at row >= 3 and never read the window that the
  // row-0 block of the same launch overwrites (a short span under a wide grid leaves the extra blocks idle)
  const int rpb = max(3, (span + (int)gridDim.z - 1) / (int)gridDim.z);
  const int row0 = blockIdx.z * rpb, row1 = min(span, row0 + rpb);
  if (row0 >= span) return;
  if (blockIdx.y == 3) {
    if (wsm_partial) span_beta_flow(wsm_partial + (size_t)at * 256, heads, span_beta, span_flow, row0, row1, span);
    return;
  }
  const int s = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * kVec;
  if (c >= inner) return;
  __nv_bfloat16* out = s == 0 ? span_q : s == 1 ? span_k : span_v;
  span_stream<TAPS_BF16>(partial + (size_t)at * row_stride, row_stride, cw, win_base + (size_t)s * 3 * inner, out, inner, s, c, row0, row1,
                         span);
}

template <bool TAPS_BF16>
__global__ void __launch_bounds__(128, K3G_SPAN_MINB) span_conv_kernel(const __nv_bfloat16* partial, long long row_stride, const void* cw, __nv_bfloat16* win,
                                                        const float* wsm_partial, __nv_bfloat16* span_q, __nv_bfloat16* span_k,
                                                        __nv_bfloat16* span_v, __nv_bfloat16* span_beta, __nv_bfloat16* span_flow,
                                                        int heads, int at, int span) {
  span_gather_body<TAPS_BF16>(partial, row_stride, cw, win, wsm_partial, span_q, span_k, span_v, span_beta, span_flow, heads, at, span);
}

// ---- output gate -----------------------------------------------------------------------------------
// grid (rows, ceil(heads * 16 / blockDim.x)): blockIdx.x walks rows (grid-stride), blockIdx.y * blockDim.x
// + threadIdx.x is the thread's 8-column vector inside the row -- no integer division anywhere.
template <bool STORE_GATED, bool QUANT>
__device__ __forceinline__ void out_gate_body(const __nv_bfloat16* __restrict__ attn, const __nv_bfloat16* __restrict__ gate,
                                              long long gate_stride, long long gate_off, const float* __restrict__ gamma_o,
                                              __nv_bfloat16* __restrict__ gated, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                              int heads, int at, int span, float eps) {
  const int inner = heads * 128;
  const int vec = blockIdx.y * blockDim.x + threadIdx.x;
  const int col = vec * 8;
  const bool live = col < inner;                               // heads * 16 is a multiple of 16: half-warps are live or dead whole
  const int lane = threadIdx.x & 31;
  const int d0 = col & 127;
  f32x2 gm[4];
  {
    const float4 m0 = __ldg(reinterpret_cast<const float4*>(gamma_o + d0)), m1 = __ldg(reinterpret_cast<const float4*>(gamma_o + d0 + 4));
    gm[0] = f2_pack(m0.x, m0.y); gm[1] = f2_pack(m0.z, m0.w); gm[2] = f2_pack(m1.x, m1.y); gm[3] = f2_pack(m1.z, m1.w);
  }
  // two rows per pass: four 16-byte loads in flight per thread before the first dependent instruction
  for (int i0 = 2 * blockIdx.x; i0 < span; i0 += 2 * gridDim.x) {
    V8 av[2], gv[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      av[k] = V8{{0u, 0u, 0u, 0u}}; gv[k] = V8{{0u, 0u, 0u, 0u}};
      if (live && i0 + k < span) {
        av[k] = ld_stream(attn + (size_t)(i0 + k) * inner + col);
        gv[k] = ld_stream(gate + (size_t)(at + i0 + k) * gate_stride + gate_off + col);
      }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const bool on = live && i0 + k < span;
      const long long b = at + i0 + k;
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf_lo(av[k].w[j]), hi = bf_hi(av[k].w[j]);
        ss = __fmaf_rn(lo, lo, ss);
        ss = __fmaf_rn(hi, hi, ss);
      }
      ss = butterfly_sum<16>(ss);
      const f32x2 r2 = f2_splat(__frsqrt_rn(__fmaf_rn(ss, 1.0f / 128.0f, eps)));
      V8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned ov = f2_to_bf2(f2_mul(f2_mul(f2_from_bf2(av[k].w[j]), r2), gm[j]));
        const unsigned gt = f2_to_bf2(f2_fast_sigmoid(f2_from_bf2(gv[k].w[j])));
        o.w[j] = mul_bf2(ov, gt);
      }
      if (STORE_GATED && on) st_stream(gated + (size_t)b * inner + col, o);
      if (QUANT) {
        unsigned am = absmax8(o);
        am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 2));
        const int e = ue8m0_exp_from_bf16(am);
        unsigned q0, q1;
        quant8(o, pow2_neg(e), q0, q1);
        unsigned sfb = (unsigned)(e + 127);
        sfb |= __shfl_down_sync(0xffffffffu, sfb, 4) << 8;
        sfb |= __shfl_down_sync(0xffffffffu, sfb, 8) << 16;
        if (on) {
          st_stream8(q + (size_t)b * inner + col, q0, q1);
          if ((lane & 15) == 0) *reinterpret_cast<unsigned*>(sf + (((size_t)b * inner + col) >> 5)) = sfb;
        }
      }
    }
  }
}

template <bool STORE_GATED, bool QUANT>
__global__ void __launch_bounds__(128) out_gate_kernel(const __nv_bfloat16* attn, const __nv_bfloat16* gate, long long gate_stride,
                                                       long long gate_off, const float* gamma_o, __nv_bfloat16* gated, uint8_t* q,
                                                       uint8_t* sf, int heads, int at, int span, float eps) {
  out_gate_body<STORE_GATED, QUANT>(attn, gate, gate_stride, gate_off, gamma_o, gated, q, sf, heads, at, span, eps);
}

}  // namespace

// ---- manifest entry points (HEADS is a build constant there) -------------------------------------
#ifndef HEADS
#define HEADS 24
#endif
#define K3G_KDA_INNER (HEADS * 128)
#define K3G_KDA_REC_BYTES ((long long)HEADS * 128 * 128 * 4)

extern "C" __global__ void __launch_bounds__(128, K3G_SPAN_MINB) kern_k3_span_gather(
    const __nv_bfloat16* __restrict__ partial, const float* __restrict__ cw, void* __restrict__ kda_base, const int* __restrict__ line_index,
    long long line_bytes, const float* __restrict__ wsm_partial, __nv_bfloat16* __restrict__ span_q, __nv_bfloat16* __restrict__ span_k,
    __nv_bfloat16* __restrict__ span_v, __nv_bfloat16* __restrict__ span_beta, __nv_bfloat16* __restrict__ span_flow,
    const int* __restrict__ span_at, int span) {
  const int at = span_at[0];
  // the window rows live in the sequence's KDA state line, after the recurrent state
  __nv_bfloat16* win = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(kda_base) + (long long)line_index[at] * line_bytes + K3G_KDA_REC_BYTES);
  span_gather_body<false>(partial, 4LL * K3G_KDA_INNER, cw, win, wsm_partial, span_q, span_k, span_v, span_beta, span_flow, HEADS, at, span);
}

extern "C" __global__ void __launch_bounds__(128) kern_k3_kda_out_gate(const __nv_bfloat16* __restrict__ attn, const __nv_bfloat16* __restrict__ gate_partial,
                                                                      const float* __restrict__ gamma_o, __nv_bfloat16* __restrict__ gated,
                                                                      const int* __restrict__ span_at, int span) {
  out_gate_body<true, false>(attn, gate_partial, 4LL * K3G_KDA_INNER, 3LL * K3G_KDA_INNER, gamma_o, gated, nullptr, nullptr, HEADS, span_at[0],
                             span, 1e-5f);
}

#ifndef K3G_CUBIN_ONLY
// Conv + SiLU on the three streams.  win: [3 streams][3 rows][inner] bf16, read as the initial
// state and overwritten with the final one (zero-fill it for a zero initial state).  cw:
// [3][4][inner] taps, f32 or bf16.  wsm_partial (f32 [rows, 256]) may be null: then span_beta /
// span_flow are not produced.  rows_per_block <= 0 selects 64; values below 3 are raised to 3 (the
// window hand-over needs every block but the first to start at row >= 3).
K3G_API int k3g_span_gather(const void* partial, long long row_stride, const void* cw, int taps_bf16, void* win, const void* wsm_partial,
                            void* span_q, void* span_k, void* span_v, void* span_beta, void* span_flow, int heads, int at, int span,
                            int rows_per_block, void* stream) {
  K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(cw); K3G_REQUIRE_PTR(win); K3G_REQUIRE_PTR(span_q); K3G_REQUIRE_PTR(span_k); K3G_REQUIRE_PTR(span_v);
  if (wsm_partial) { K3G_REQUIRE_PTR(span_beta); K3G_REQUIRE_PTR(span_flow); K3G_REQUIRE_ALIGNED(wsm_partial); }
  K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(cw); K3G_REQUIRE_ALIGNED(win); K3G_REQUIRE_ALIGNED(span_q); K3G_REQUIRE_ALIGNED(span_k);
  K3G_REQUIRE_ALIGNED(span_v);
  K3G_REQUIRE(heads > 0 && heads <= 512 && span >= 0 && at >= 0 && row_stride >= 3LL * heads * 128 && row_stride % 8 == 0, K3G_ESHAPE);
  if (span == 0) return K3G_OK;
  const int rpb = rows_per_block > 0 ? (rows_per_block < 3 ? 3 : rows_per_block) : 64;
  const int inner = heads * 128;
  const dim3 grid((inner + 511) / 512, wsm_partial ? 4 : 3, (span + rpb - 1) / rpb);
  K3G_REQUIRE(grid.z <= 65535, K3G_ELIMIT);
  if (taps_bf16)
    span_conv_kernel<true><<<grid, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)partial, row_stride, cw, (__nv_bfloat16*)win,
                                                                (const float*)wsm_partial, (__nv_bfloat16*)span_q, (__nv_bfloat16*)span_k,
                                                                (__nv_bfloat16*)span_v, (__nv_bfloat16*)span_beta, (__nv_bfloat16*)span_flow,
                                                                heads, at, span);
  else
    span_conv_kernel<false><<<grid, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)partial, row_stride, cw, (__nv_bfloat16*)win,
                                                                 (const float*)wsm_partial, (__nv_bfloat16*)span_q, (__nv_bfloat16*)span_k,
                                                                 (__nv_bfloat16*)span_v, (__nv_bfloat16*)span_beta, (__nv_bfloat16*)span_flow,
                                                                 heads, at, span);
  return k3g_launch_status();
}

// Output gate.  gate element (row b, column c) = gate[b * gate_stride + gate_off + c].  gated may be
// null when only the MXFP8 form is wanted; q / sf may be null when only bf16 is wanted.
K3G_API int k3g_kda_out_gate(const void* attn, const void* gate, long long gate_stride, long long gate_off, const void* gamma_o,
                             void* gated, void* q, void* sf, int heads, int at, int span, float eps, void* stream) {
  K3G_REQUIRE_PTR(attn); K3G_REQUIRE_PTR(gate); K3G_REQUIRE_PTR(gamma_o);
  K3G_REQUIRE(gated != nullptr || (q != nullptr && sf != nullptr), K3G_ENULL);
  K3G_REQUIRE((q == nullptr) == (sf == nullptr), K3G_ENULL);
  K3G_REQUIRE_ALIGNED(attn); K3G_REQUIRE_ALIGNED(gate); K3G_REQUIRE_ALIGNED(gamma_o); K3G_REQUIRE_ALIGNED(gated);
  K3G_REQUIRE(((uintptr_t)q & 7) == 0 && ((uintptr_t)sf & 3) == 0, K3G_EALIGN);
  K3G_REQUIRE(heads > 0 && heads % 2 == 0 && span >= 0 && at >= 0 && gate_stride % 8 == 0 && gate_off % 8 == 0, K3G_ESHAPE);
  if (span == 0) return K3G_OK;
  const dim3 grid((unsigned)((span + 1) / 2), (unsigned)((heads * 16 + 127) / 128), 1);
  cudaStream_t st = k3g_stream(stream);
#define K3G_OG_ARGS (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, gate_stride, gate_off, (const float*)gamma_o, \
    (__nv_bfloat16*)gated, (uint8_t*)q, (uint8_t*)sf, heads, at, span, eps
  if (gated && q) out_gate_kernel<true, true><<<grid, 128, 0, st>>>(K3G_OG_ARGS);
  else if (gated) out_gate_kernel<true, false><<<grid, 128, 0, st>>>(K3G_OG_ARGS);
  else out_gate_kernel<false, true><<<grid, 128, 0, st>>>(K3G_OG_ARGS);
#undef K3G_OG_ARGS
  return k3g_launch_status();
}
#endif
