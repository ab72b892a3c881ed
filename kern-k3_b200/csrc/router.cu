// Router top-k: sigmoid scores, bias-corrected selection, renormalised weights.
//
// Replaces kern_k3_router_topk of xiaguan/kern-k3 (source/k3_router_argmax.cu:87-152) behind
// the same entry name and parameter list.  Semantics kept: sig = sigmoid(S); selection key =
// sig + bias; K sequential picks of the largest key, ties to the smallest expert id; output in
// pick order; w = sig / (sum of the K picked sig + 1e-20) * f32(rs[0]), the sum taken as an
// xor-butterfly over the K lanes.
//
// Layout for B200: one WARP per token row (eight rows per 256-thread block, grid-stride), not
// one block per row.  The row's 224 logits are loaded coalesced (7 x 128 B), each lane
// evaluates the sigmoid of the expert it loaded and parks (sig, key) in shared memory, then
// re-reads the 7 experts it owns for selection (expert = 7 * lane + j, a stride-7 pattern that
// is bank-conflict free), so "smallest lane, then smallest slot" is "smallest expert id".
// Each pick is one REDUX.MAX on the monotone u32 key and one REDUX.MIN on the expert id.
//
// The sigmoid is evaluated with IEEE-only operations (k3g::det_sigmoid): the indices depend on
// it, and this makes them reproducible bit for bit by any IEEE host.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {

constexpr int kExperts = 224;
constexpr int kPerLane = kExperts / 32;   // 7
constexpr int kRowsPerBlock = 8;

__device__ __forceinline__ unsigned ord_f32(float f) {
  const unsigned b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <int K>
__device__ __forceinline__ void router_rows(const float* __restrict__ S, const float* __restrict__ bias,
                                            const __nv_bfloat16* __restrict__ rs, int* __restrict__ idx,
                                            float* __restrict__ wts, int B) {
  __shared__ float s_sig[kRowsPerBlock][kExperts];
  __shared__ unsigned s_key[kRowsPerBlock][kExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float rsf = __bfloat162float(rs[0]);
  float bia[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) bia[i] = __ldg(bias + 32 * i + lane);

  for (int row = blockIdx.x * kRowsPerBlock + warp; row < B; row += gridDim.x * kRowsPerBlock) {
    const float* Sr = S + (size_t)row * kExperts;
    float lg[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) lg[i] = __ldcs(Sr + 32 * i + lane);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const float sg = det_sigmoid(lg[i]);
      s_sig[warp][32 * i + lane] = sg;
      s_key[warp][32 * i + lane] = ord_f32(__fadd_rn(sg, bia[i]));
    }
    __syncwarp();
    unsigned o[kPerLane];
    float g[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      o[j] = s_key[warp][lane * kPerLane + j];
      g[j] = s_sig[warp][lane * kPerLane + j];
    }
    __syncwarp();

    int my_e = 0;       // lane r keeps pick r
    float my_w = 0.f;
#pragma unroll
    for (int r = 0; r < K; ++r) {
      unsigned m = o[0];
#pragma unroll
      for (int j = 1; j < kPerLane; ++j) m = max(m, o[j]);
      m = __reduce_max_sync(0xffffffffu, m);
      unsigned mine = 0xffffffffu;
#pragma unroll
      for (int j = kPerLane - 1; j >= 0; --j)
        if (o[j] == m) mine = (unsigned)(lane * kPerLane + j);
      const unsigned ew = __reduce_min_sync(0xffffffffu, mine);
      float gw = 0.f;
      if (mine == ew) {
        const int jw = (int)ew - lane * kPerLane;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
          if (j == jw) { gw = g[j]; o[j] = 0u; }     // 0 is below the key of every real float
      }
      gw = __shfl_sync(0xffffffffu, gw, (int)(ew / kPerLane));
      if (lane == r) { my_e = (int)ew; my_w = gw; }
    }
    float den = (lane < K) ? my_w : 0.f;
#pragma unroll
    for (int off = K / 2; off > 0; off >>= 1) den = __fadd_rn(den, __shfl_xor_sync(0xffffffffu, den, off));
    if (lane < K) {
      wts[(size_t)row * K + lane] = __fmul_rn(__fdiv_rn(my_w, __fadd_rn(den, 1e-20f)), rsf);
      idx[(size_t)row * K + lane] = my_e;
    }
  }
}

template <int K>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* S, const float* bias, const __nv_bfloat16* rs, int* idx,
                                                          float* wts, int B) {
  router_rows<K>(S, bias, rs, idx, wts, B);
}

}  // namespace

// Manifest entry (op router_topk): TOPK = 16, 224 experts (source/k3_router_argmax.cu:59-62).
extern "C" __global__ void __launch_bounds__(256) kern_k3_router_topk(const float* __restrict__ S, const float* __restrict__ bias,
                                                                     const __nv_bfloat16* __restrict__ rs, int* __restrict__ idx,
                                                                     float* __restrict__ wts, int B) {
  router_rows<16>(S, bias, rs, idx, wts, B);
}

#ifndef K3G_CUBIN_ONLY
K3G_API int k3g_router_topk(const void* S, const void* bias, const void* rs, void* idx, void* wts, int B, int experts,
                            int topk, void* stream) {
  K3G_REQUIRE_PTR(S); K3G_REQUIRE_PTR(bias); K3G_REQUIRE_PTR(rs); K3G_REQUIRE_PTR(idx); K3G_REQUIRE_PTR(wts);
  K3G_REQUIRE(experts == kExperts && (topk == 8 || topk == 16) && B >= 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  const int grid = (B + kRowsPerBlock - 1) / kRowsPerBlock;
  if (topk == 8)
    router_topk_kernel<8><<<grid, 256, 0, k3g_stream(stream)>>>((const float*)S, (const float*)bias, (const __nv_bfloat16*)rs,
                                                               (int*)idx, (float*)wts, B);
  else
    router_topk_kernel<16><<<grid, 256, 0, k3g_stream(stream)>>>((const float*)S, (const float*)bias, (const __nv_bfloat16*)rs,
                                                                (int*)idx, (float*)wts, B);
  return k3g_launch_status();
}
#endif
