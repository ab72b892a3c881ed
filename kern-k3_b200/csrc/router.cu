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
// re-reads the keys of the 7 consecutive experts it owns (expert = 7 * lane + j, a stride-7
// pattern that is bank-conflict free).
//
// Selection = a K-way merge of 32 sorted runs.  A candidate is one 64-bit word: the monotone
// image of its biased score in the high half, 255 - expert id in the low half, so unsigned order
// is "larger score first, then smaller expert id" and no two candidates compare equal.  Each
// lane sorts its seven candidates once with a 16-exchange network; after that its best
// remaining candidate always sits in run[0].  A pick is then: one REDUX.MAX over the lanes'
// run[0] scores, one ballot of the lanes that hold that score -- the lowest such lane owns the
// smallest expert id, because lanes own ascending id ranges and a run is already ordered by id
// among equal scores -- one shuffle of the winner's id, and the winner shifts its run up by one.
// The picked experts' sigmoids are fetched from shared memory after the last pick.
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

// Order-preserving map from float to u32: negative values have all bits flipped, the others only the sign bit.
__device__ __forceinline__ unsigned ord_f32(float f) {
  const int b = __float_as_int(f);
  return (unsigned)b ^ ((unsigned)(b >> 31) | 0x80000000u);
}

__device__ __forceinline__ void sort2_desc(unsigned long long& hi, unsigned long long& lo) {
  const unsigned long long a = hi, b = lo;
  hi = a > b ? a : b;
  lo = a > b ? b : a;
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
    __syncwarp();                                    // the previous row's sigmoids have been read by every lane
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const float sg = det_sigmoid(lg[i]);
      s_sig[warp][32 * i + lane] = sg;
      s_key[warp][32 * i + lane] = ord_f32(__fadd_rn(sg, bia[i]));
    }
    __syncwarp();
    unsigned long long run[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane * kPerLane + j;
      run[j] = ((unsigned long long)s_key[warp][e] << 32) | (unsigned)(255 - e);
    }
    // seven candidates, descending: optimal 16-exchange network
    sort2_desc(run[0], run[6]); sort2_desc(run[2], run[3]); sort2_desc(run[4], run[5]);
    sort2_desc(run[0], run[2]); sort2_desc(run[1], run[4]); sort2_desc(run[3], run[6]);
    sort2_desc(run[0], run[1]); sort2_desc(run[2], run[5]); sort2_desc(run[3], run[4]);
    sort2_desc(run[1], run[2]); sort2_desc(run[4], run[6]);
    sort2_desc(run[2], run[3]); sort2_desc(run[4], run[5]);
    sort2_desc(run[1], run[2]); sort2_desc(run[3], run[4]); sort2_desc(run[5], run[6]);

    int my_e = 0;                                    // lane r keeps pick r
#pragma unroll
    for (int r = 0; r < K; ++r) {
      const unsigned head = (unsigned)(run[0] >> 32);            // 0 once a run is used up: below the image of every float
      const unsigned best = __reduce_max_sync(0xffffffffu, head);
      const int winner = __ffs(__ballot_sync(0xffffffffu, head == best)) - 1;
      const int e = 255 - (int)__shfl_sync(0xffffffffu, (unsigned)run[0], winner);
      if (lane == r) my_e = e;
      if (lane == winner) {
#pragma unroll
        for (int j = 0; j + 1 < kPerLane; ++j) run[j] = run[j + 1];
        run[kPerLane - 1] = 0ull;
      }
    }
    const float my_w = lane < K ? s_sig[warp][my_e] : 0.f;
    float den = my_w;
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

// ---- f32 argmax over a logits row, two stages (ops argmax_f32_one / argmax_f32) --------------------
// Replaces kern_k3_argmax_f32_partial / kern_k3_argmax_f32_final (source/k3_router_argmax.cu:186-241):
// largest value under the monotone bit order of ord_f32, ties to the smallest index; stage 1 reduces
// gridDim.y contiguous chunks of the row to (pmax, pidx), an empty chunk giving (-inf, 0x7fffffff);
// stage 2 applies the same rule to the partials (0 when there is none).  A candidate is the pair
// (ord, index); within a thread indices only grow, so a strict compare keeps the smallest; across lanes
// and warps one REDUX.MAX on the order and one REDUX.MIN on the index of whoever matched.
namespace {
constexpr int kNoIndex = 0x7fffffff;

// Block-wide (ord, idx) reduction; every thread returns the winner.  ord == 0 means "no candidate"
// (ord_f32 never returns 0 for a non-NaN float other than -NaN patterns, which order lowest anyway).
__device__ __forceinline__ void block_argmax(unsigned& o, int& i, unsigned* s_ord, int* s_idx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  unsigned m = __reduce_max_sync(0xffffffffu, o);
  int w = __reduce_min_sync(0xffffffffu, o == m ? i : kNoIndex);
  if (lane == 0) { s_ord[warp] = m; s_idx[warp] = w; }
  __syncthreads();
  o = lane < nwarps ? s_ord[lane] : 0u;
  i = lane < nwarps ? s_idx[lane] : kNoIndex;
  m = __reduce_max_sync(0xffffffffu, o);
  w = __reduce_min_sync(0xffffffffu, o == m ? i : kNoIndex);
  o = m; i = w;
}
__device__ __forceinline__ float unord_f32(unsigned o) { return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o); }
__device__ __forceinline__ void take(unsigned& bo, int& bi, float v, int i) {
  const unsigned o = ord_f32(v);
  if (o > bo) { bo = o; bi = i; }
}
}  // namespace

extern "C" __global__ void __launch_bounds__(1024) kern_k3_argmax_f32_partial(const float* __restrict__ logits, float* __restrict__ pmax,
                                                                             int* __restrict__ pidx, int n) {
  __shared__ unsigned s_ord[32];
  __shared__ int s_idx[32];
  const int parts = gridDim.y;
  const int chunk = (n + parts - 1) / parts;
  const int lo = blockIdx.y * chunk, hi = min(lo + chunk, n);
  const float* row = logits + (long long)blockIdx.x * n;
  unsigned bo = 0u;
  int bi = kNoIndex;
  if (((n | chunk) & 3) == 0 && (reinterpret_cast<unsigned long long>(logits) & 15ull) == 0) {
    const float4* v4 = reinterpret_cast<const float4*>(row + lo);
    const int nv = (hi - lo) >> 2;
    for (int u = threadIdx.x; u < nv; u += 2 * blockDim.x) {     // two 16-byte loads in flight per thread
      const int u1 = u + blockDim.x;
      const float4 a = __ldcs(v4 + u);
      float4 b = a;
      if (u1 < nv) b = __ldcs(v4 + u1);
      const int ia = lo + 4 * u, ib = lo + 4 * u1;
      take(bo, bi, a.x, ia); take(bo, bi, a.y, ia + 1); take(bo, bi, a.z, ia + 2); take(bo, bi, a.w, ia + 3);
      if (u1 < nv) { take(bo, bi, b.x, ib); take(bo, bi, b.y, ib + 1); take(bo, bi, b.z, ib + 2); take(bo, bi, b.w, ib + 3); }
    }
  } else {
    for (int j = lo + threadIdx.x; j < hi; j += blockDim.x) take(bo, bi, row[j], j);
  }
  block_argmax(bo, bi, s_ord, s_idx);
  if (threadIdx.x == 0) {
    const int o = blockIdx.x * parts + blockIdx.y;
    const bool none = bo == 0u || bi == kNoIndex;
    pmax[o] = none ? __int_as_float(0xff800000) : unord_f32(bo);
    pidx[o] = none ? kNoIndex : bi;
  }
}

extern "C" __global__ void __launch_bounds__(1024) kern_k3_argmax_f32_final(const float* __restrict__ pmax, const int* __restrict__ pidx,
                                                                           long long* __restrict__ out, int parts) {
  __shared__ unsigned s_ord[32];
  __shared__ int s_idx[32];
  const long long base = (long long)blockIdx.x * parts;
  unsigned bo = 0u;
  int bi = kNoIndex;
  for (int t = threadIdx.x; t < parts; t += blockDim.x) {
    const int i = pidx[base + t];
    if (i == kNoIndex) continue;
    const unsigned o = ord_f32(pmax[base + t]);
    if (o > bo || (o == bo && i < bi)) { bo = o; bi = i; }
  }
  block_argmax(bo, bi, s_ord, s_idx);
  if (threadIdx.x == 0) out[blockIdx.x] = (bo == 0u || bi == kNoIndex) ? 0ll : (long long)bi;
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
K3G_API int k3g_argmax_f32(const void* logits, void* pmax, void* pidx, void* out, int B, int n, int parts, void* stream) {
  K3G_REQUIRE_PTR(logits); K3G_REQUIRE_PTR(pmax); K3G_REQUIRE_PTR(pidx); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE(B >= 0 && n > 0 && parts > 0 && parts <= 65535, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  kern_k3_argmax_f32_partial<<<dim3((unsigned)B, (unsigned)parts, 1), 512, 0, k3g_stream(stream)>>>((const float*)logits, (float*)pmax, (int*)pidx, n);
  kern_k3_argmax_f32_final<<<(unsigned)B, 64, 0, k3g_stream(stream)>>>((const float*)pmax, (const int*)pidx, (long long*)out, parts);
  return k3g_launch_status();
}
#endif
