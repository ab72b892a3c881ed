// Residual stream of K3 prefill: landing add, attention-residual mix, RMSNorm, and the
// fused MXFP8 epilogue.
//
// Replaces, behind the same entry names and parameter lists, the kernels of
// xiaguan/kern-k3 source/k3_residual_v2.cu:
//   kern_k3_attnres_rms           (:260-284)   K1a
//   kern_k3_land_add_attnres_rms  (:295-345)   K1b (bf16 or f32 landing)
//   kern_k3_land_add2             (:349-392)   K1c
// and adds the fusion the reference runs as separate launches:
//   k3g_resnorm_mxfp8_kernel: residual + delta -> residual_out (bf16), RMSNorm * gamma,
//   then the MXFP8 quantisation of source/k3_moe_prefill_v4.cu:111-140 on the normed row
//   while it is still in registers, so every activation byte crosses HBM once.
//
// Geometry.  A row of H = 1024 * VPT bf16 is owned by a team of 128 threads; thread t owns
// the 16-byte vectors t + 128 v, v < VPT.  That is the assignment the reference's fixed-order
// reduction is defined on (serial fma chain per thread, xor-butterfly per warp, the four
// warp partials summed in order), so sums -- and through them the bf16 normed row and the
// UE8M0 scales -- do not depend on how rows are scheduled.  A 32-element MXFP8 group is
// four consecutive vectors, i.e. four adjacent lanes: its amax is two xor-shuffles.
// All row traffic is 16-byte, coalesced, streaming (evict-first); the 14 KB gamma row stays
// cached.  One block = one team; the grid walks rows with stride gridDim.x, so both the
// reference launch (grid = rows) and a persistent launch are valid.
#include "k3g_device.cuh"
#include "k3g_host.h"

namespace k3g {

constexpr int kTeam = 128;
constexpr int kNbMax = 8;

template <int VPT>
__device__ __forceinline__ float team_sumsq(const V8 (&x)[VPT], float* s_red, int lane, int warp) {
  float sq = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = bf_lo(x[v].w[j]), hi = bf_hi(x[v].w[j]);
      sq = __fmaf_rn(lo, lo, sq);
      sq = __fmaf_rn(hi, hi, sq);
    }
  }
  sq = butterfly_sum<32>(sq);
  if (lane == 0) s_red[warp] = sq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kTeam / 32; ++w) tot = __fadd_rn(tot, s_red[w]);
  return tot;
}

// max |bf16| over the team's row from per-thread packed maxima m2 (two 15-bit maxima, packed like the data):
// the maximum of bit patterns, exact and order-free, as kern_quant_fp8_amax_v2 takes it.  One barrier.
__device__ __forceinline__ unsigned team_absmax_bits(unsigned m2, unsigned* s_buf, int lane, int warp) {
  unsigned m = max(m2 & 0xffffu, m2 >> 16);
  m = __reduce_max_sync(0xffffffffu, m);
  if (lane == 0) s_buf[warp] = m;
  __syncthreads();
  return max(max(s_buf[0], s_buf[1]), max(s_buf[2], s_buf[3]));
}

// RMSNorm of the team's row x (bf16 in registers) with optional MXFP8 epilogue.
// amax_dst != nullptr: thread 0 also stores max |normed| of the row there (s_amax: 4 words of shared memory),
// the per-row partial a following per-tensor FP8 quantisation needs instead of its own pass over the tensor.
//   normed = bf16(bf16(x * r) * gamma),  r = rsqrt_rn(fma(sum x^2, 1/H, eps))
template <int VPT, bool STORE_NORMED, bool QUANT>
__device__ __forceinline__ void team_rms_store(const V8 (&x)[VPT], const __nv_bfloat16* __restrict__ gamma,
                                               __nv_bfloat16* __restrict__ normed_row, uint8_t* __restrict__ q_row,
                                               uint8_t* __restrict__ sf_row, float eps, float* s_red, int t,
                                               float* __restrict__ amax_dst = nullptr, unsigned* s_amax = nullptr) {
  constexpr int H = VPT * 1024;
  const int lane = t & 31, warp = t >> 5;
  const float tot = team_sumsq<VPT>(x, s_red, lane, warp);
  const float r = __frsqrt_rn(__fmaf_rn(tot, 1.0f / (float)H, eps));
  unsigned m2 = 0u;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int u = (t + v * kTeam) * 8;
    const V8 g = ld_keep(gamma + u);
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(x[v].w[j]), r), __fmul_rn(bf_hi(x[v].w[j]), r)), g.w[j]);
      m2 = __vmaxu2(m2, o.w[j] & 0x7fff7fffu);
    }
    if (STORE_NORMED) st_stream(normed_row + u, o);
    if (QUANT) {
      unsigned am = absmax8(o);
      am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 1));
      am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 2));
      const int e = ue8m0_exp_from_bf16(am);
      unsigned q0, q1;
      quant8(o, pow2_neg(e), q0, q1);
      st_stream8(q_row + u, q0, q1);
      // the warp's eight scale bytes: lanes 0 and 16 each store four
      unsigned sfb = (unsigned)(e + 127);
      sfb |= __shfl_down_sync(0xffffffffu, sfb, 4) << 8;
      sfb |= __shfl_down_sync(0xffffffffu, sfb, 8) << 16;
      if ((lane & 15) == 0) *reinterpret_cast<unsigned*>(sf_row + (u >> 5)) = sfb;
    }
  }
  if (amax_dst != nullptr) {
    const unsigned m = team_absmax_bits(m2, s_amax, lane, warp);
    if (t == 0) *amax_dst = __uint_as_float(m << 16);
  }
}

// Attention-residual mix of source/k3_residual_v2.cu:122-223: candidates 0..nb-1 are the
// snapshot rows, candidate nb is the prefix row held in x (overwritten with the mix).
//
// Statistics hand-off (source/k3_residual_push_add2.cu:273-279, source/k3_residual_nb_stats.cu:254-258):
//   producer  (sw_other != nullptr): also accumulates dp'_c = sum x_c * sw_other for the snapshot
//             candidates and stores (sq_c, dp'_c) to stats_out[c] -- the numbers the NEXT residual
//             kernel of the layer would compute for the same rows with its own scoring vector;
//   consumer  (nb_stats > 0): takes (sq_c, dp_c) of candidates c < nb_stats from stats_in instead of
//             reading those rows in pass 1.  Same summation order on both sides, so the value read
//             is bit-identical to the value recomputed.
// PAIR: pass 1 takes the snapshot rows two at a time (both rows' loads in flight before the first fma chain) -- worth
// its registers where pass 1 really reads the rows (the producer, the kernels without a hand-off), not in the consumer
// that takes the statistics from the hand-off and skips those reads.
template <int VPT, bool PAIR = false>
__device__ __forceinline__ void team_attnres_mix(V8 (&x)[VPT], const __nv_bfloat16* __restrict__ blk_row,
                                                 const float* __restrict__ sw, int nb, float eps, float* s_mix, int t,
                                                 const float* __restrict__ sw_other = nullptr, float* __restrict__ stats_out = nullptr,
                                                 const float* __restrict__ stats_in = nullptr, int nb_stats = 0) {
  constexpr int H = VPT * 1024;
  constexpr int NW = kTeam / 32;
  const int lane = t & 31, warp = t >> 5;
  const int ncand = nb + 1;
  float* s_oth = s_mix + (kNbMax + 1) * 2 * NW;       // dp' warp partials (producer only)
  // pass 1: (sum x^2, sum x*sw) per candidate (same per-thread order).  Candidates go two at a time so that the loads
  // of both rows are in flight before the first dependent fma chain starts: half as many memory round trips.
  auto reduce_candidate = [&](const V8 (&cvs)[VPT], int c) {
    float sq = 0.f, dp = 0.f, dq = 0.f;
    const bool other = sw_other != nullptr && c < nb;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int u = (t + v * kTeam) * 8;
      const V8 cv = cvs[v];
      const float4 a = __ldg((const float4*)(sw + u)), b = __ldg((const float4*)(sw + u + 4));
      const float s8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = bf_lo(cv.w[j]), hi = bf_hi(cv.w[j]);
        sq = __fmaf_rn(lo, lo, sq);  sq = __fmaf_rn(hi, hi, sq);
        dp = __fmaf_rn(lo, s8[2 * j], dp);  dp = __fmaf_rn(hi, s8[2 * j + 1], dp);
      }
      if (other) {
        const float4 c0 = __ldg((const float4*)(sw_other + u)), c1 = __ldg((const float4*)(sw_other + u + 4));
        const float o8[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          dq = __fmaf_rn(bf_lo(cv.w[j]), o8[2 * j], dq);  dq = __fmaf_rn(bf_hi(cv.w[j]), o8[2 * j + 1], dq);
        }
      }
    }
    sq = butterfly_sum<32>(sq);
    dp = butterfly_sum<32>(dp);
    if (lane == 0) { s_mix[(2 * c) * NW + warp] = sq; s_mix[(2 * c + 1) * NW + warp] = dp; }
    if (other) {
      dq = butterfly_sum<32>(dq);
      if (lane == 0) s_oth[c * NW + warp] = dq;
    }
  };
  int c = nb_stats < nb ? nb_stats : nb;
  for (; PAIR && c + 1 < nb; c += 2) {                // two snapshot rows per round
    V8 ca[VPT], cb[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) ca[v] = ld_plain(blk_row + (size_t)c * H + (t + v * kTeam) * 8);
#pragma unroll
    for (int v = 0; v < VPT; ++v) cb[v] = ld_plain(blk_row + (size_t)(c + 1) * H + (t + v * kTeam) * 8);
    reduce_candidate(ca, c);
    reduce_candidate(cb, c + 1);
  }
  for (; c < nb; ++c) {                               // one row per round (all of them without PAIR, else the odd one left)
    V8 ca[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) ca[v] = ld_plain(blk_row + (size_t)c * H + (t + v * kTeam) * 8);
    reduce_candidate(ca, c);
  }
  reduce_candidate(x, nb);                            // the prefix candidate is the row held in registers
  __syncthreads();
  float sc = -3.0e38f;
  if (lane < ncand) {
    float sqv = 0.f, dpv = 0.f;
    if (lane < nb_stats && lane < nb) {
      sqv = __ldg(stats_in + 2 * lane);
      dpv = __ldg(stats_in + 2 * lane + 1);
    } else {
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        sqv = __fadd_rn(sqv, s_mix[(2 * lane) * NW + w]);
        dpv = __fadd_rn(dpv, s_mix[(2 * lane + 1) * NW + w]);
      }
    }
    sc = __fmul_rn(dpv, __frsqrt_rn(__fmaf_rn(sqv, 1.0f / (float)H, eps)));
    if (stats_out != nullptr && lane < nb && warp == 0) {
      float dqv = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) dqv = __fadd_rn(dqv, s_oth[lane * NW + w]);
      stats_out[2 * lane] = sqv;
      stats_out[2 * lane + 1] = dqv;
    }
  }
  float mx = sc;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float ex = (lane < ncand) ? det_exp(__fadd_rn(sc, -mx)) : 0.f;
  const float den = butterfly_sum<32>(ex);
  const float pmine = __fdiv_rn(ex, den);
  const float pp = __shfl_sync(0xffffffffu, pmine, nb);
  __syncthreads();   // s_mix is reused by the next row of a persistent launch
  // pass 2: mixed = bf16(p_prefix * x + sum_c p_c * cand_c), candidates ascending.  The accumulators of the whole
  // row stay in registers and the candidate loop is the outer one, so all VPT loads of a candidate row are in flight
  // together (they hit L2: pass 1 has just read the row); per element the order of operations is unchanged.
  float acc[VPT][8];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[v][2 * j] = __fmul_rn(pp, bf_lo(x[v].w[j]));
      acc[v][2 * j + 1] = __fmul_rn(pp, bf_hi(x[v].w[j]));
    }
  }
  for (int c = 0; c < nb; ++c) {
    const float pc = __shfl_sync(0xffffffffu, pmine, c);
    V8 cv[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) cv[v] = ld_plain(blk_row + (size_t)c * H + (t + v * kTeam) * 8);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[v][2 * j] = __fmaf_rn(pc, bf_lo(cv[v].w[j]), acc[v][2 * j]);
        acc[v][2 * j + 1] = __fmaf_rn(pc, bf_hi(cv[v].w[j]), acc[v][2 * j + 1]);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
#pragma unroll
    for (int j = 0; j < 4; ++j) x[v].w[j] = pack_bf2(acc[v][2 * j], acc[v][2 * j + 1]);
  }
}

constexpr int kMixSmem = (kNbMax + 1) * 3 * (kTeam / 32);   // sq, dp and dp' warp partials

// ---- fused residual add + RMSNorm + MXFP8 ------------------------------------------------
template <int VPT, bool STORE_NORMED>
__global__ void __launch_bounds__(kTeam, 4) resnorm_mxfp8_kernel(
    const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
    const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ residual_out,
    uint8_t* __restrict__ q, uint8_t* __restrict__ sf, __nv_bfloat16* __restrict__ normed, int rows, float eps) {
  constexpr int H = VPT * 1024;
  __shared__ float s_red[2][kTeam / 32];
  const int t = threadIdx.x;
  int it = 0;
  for (int b = blockIdx.x; b < rows; b += gridDim.x, ++it) {
    const size_t base = (size_t)b * H;
    V8 a[VPT], d[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) a[v] = ld_stream(residual + base + (t + v * kTeam) * 8);
#pragma unroll
    for (int v = 0; v < VPT; ++v) d[v] = ld_stream(delta + base + (t + v * kTeam) * 8);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
#pragma unroll
      for (int j = 0; j < 4; ++j) a[v].w[j] = add_bf2(a[v].w[j], d[v].w[j]);
      st_stream(residual_out + base + (t + v * kTeam) * 8, a[v]);
    }
    team_rms_store<VPT, STORE_NORMED, true>(a, gamma, STORE_NORMED ? normed + base : nullptr, q + base,
                                             sf + (size_t)b * (H / 32), eps, s_red[it & 1], t);
  }
}

// ---- K1a ----------------------------------------------------------------------------------
template <int VPT>
__device__ __forceinline__ void attnres_rms_body(const __nv_bfloat16* __restrict__ prefix, __nv_bfloat16* __restrict__ blocks,
                                                 const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma,
                                                 __nv_bfloat16* __restrict__ normed, int nb, int snapshot, int B, float eps) {
  constexpr int H = VPT * 1024;
  __shared__ float s_red[2][kTeam / 32];
  __shared__ float s_mix[kMixSmem];
  const int t = threadIdx.x;
  int it = 0;
  for (int b = blockIdx.x; b < B; b += gridDim.x, ++it) {
    const size_t base = (size_t)b * H;
    V8 x[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) x[v] = ld_stream(prefix + base + (t + v * kTeam) * 8);
    __nv_bfloat16* blk_row = blocks + (size_t)b * kNbMax * H;
    if (snapshot && nb < kNbMax) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) st_plain(blk_row + (size_t)nb * H + (t + v * kTeam) * 8, x[v]);
    }
    if (nb > 0) team_attnres_mix<VPT, true>(x, blk_row, sw, nb, eps, s_mix, t);
    team_rms_store<VPT, true, false>(x, gamma, normed + base, nullptr, nullptr, eps, s_red[it & 1], t);
  }
}

// ---- K1b ----------------------------------------------------------------------------------
// NR > 0: `partial` is this rank's [NR * B, H] bf16 buffer of partial sums and partial_peer the u64 table of every
// rank's buffer; the landed row is then the ring-order reduce-scatter chain over the NR ranks (peers ascending
// from rank + 1, own last, one bf16 rounding per hop: k3g::rs_chain) of row rank * B + b -- the pull
// reduce-scatter folded into the kernel that consumes it, bit-identical to running the two one after the other.
template <int VPT, bool LB16, int NR = 0>
__device__ __forceinline__ void land_add_attnres_rms_body(const void* __restrict__ partial, const __nv_bfloat16* __restrict__ prefix,
                                                          const __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw,
                                                          const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ prefix2,
                                                          __nv_bfloat16* __restrict__ normed, int nb, int snapshot, int B, float eps,
                                                          const float* __restrict__ stats = nullptr, int nb_stats = 0,
                                                          float* __restrict__ rowmax = nullptr,
                                                          const unsigned long long* __restrict__ partial_peer = nullptr, int rank = 0) {
  constexpr int H = VPT * 1024;
  __shared__ float s_red[2][kTeam / 32];
  __shared__ float s_mix[kMixSmem];
  __shared__ unsigned s_amax[2][kTeam / 32];
  const int t = threadIdx.x;
  if (stats == nullptr) nb_stats = 0;
  constexpr int NRC = NR > 0 ? NR : 1;
  const uint4* ring[NRC];
  if constexpr (NR > 0) rs_bases<NR, NR - 1, 0>((const __nv_bfloat16*)partial, partial_peer, (long long)rank * B * H, rank, ring);
  int it = 0;
  for (int b = blockIdx.x; b < B; b += gridDim.x, ++it) {
    const size_t base = (size_t)b * H;
    V8 x[VPT];
    if constexpr (NR > 1) {
      // pull the NR partial rows with 32-byte loads and land the ring-order chain (k3g::rs_chain_team_row), then add
      rs_chain_team_row<VPT, NR, (NR == 2 ? 2 : 1)>(ring, (long long)(base >> 3), t, x);
      if (!snapshot) {
        V8 pr[VPT];
#pragma unroll
        for (int v = 0; v < VPT; ++v) pr[v] = ld_stream(prefix + base + (t + v * kTeam) * 8);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
#pragma unroll
          for (int j = 0; j < 4; ++j) x[v].w[j] = add_bf2(pr[v].w[j], x[v].w[j]);
        }
      }
#pragma unroll
      for (int v = 0; v < VPT; ++v) st_stream(prefix2 + base + (t + v * kTeam) * 8, x[v]);
    } else if constexpr (NR == 1) {
      // a single rank: the chain is the rank's own partial row; every load of the row issued before the first add
      V8 pr[VPT];
#pragma unroll
      for (int v = 0; v < VPT; ++v) x[v] = rs_chain<1>(ring, (long long)((base >> 3) + t + v * kTeam));
      if (!snapshot) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) pr[v] = ld_stream(prefix + base + (t + v * kTeam) * 8);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
#pragma unroll
          for (int j = 0; j < 4; ++j) x[v].w[j] = add_bf2(pr[v].w[j], x[v].w[j]);
        }
      }
#pragma unroll
      for (int v = 0; v < VPT; ++v) st_stream(prefix2 + base + (t + v * kTeam) * 8, x[v]);
    }
#pragma unroll
    for (int v = 0; v < (NR > 0 ? 0 : VPT); ++v) {
      const size_t off = base + (t + v * kTeam) * 8;
      V8 p;
      if (LB16) {
        p = ld_stream((const __nv_bfloat16*)partial + off);
      } else {
        const V8 f0 = ld_stream((const float*)partial + off), f1 = ld_stream((const float*)partial + off + 4);
        p.w[0] = pack_bf2(__uint_as_float(f0.w[0]), __uint_as_float(f0.w[1]));
        p.w[1] = pack_bf2(__uint_as_float(f0.w[2]), __uint_as_float(f0.w[3]));
        p.w[2] = pack_bf2(__uint_as_float(f1.w[0]), __uint_as_float(f1.w[1]));
        p.w[3] = pack_bf2(__uint_as_float(f1.w[2]), __uint_as_float(f1.w[3]));
      }
      if (snapshot) {
        x[v] = p;
      } else {
        const V8 pr = ld_stream(prefix + off);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[v].w[j] = add_bf2(pr.w[j], p.w[j]);
      }
      st_stream(prefix2 + off, x[v]);
    }
    if (nb > 0)
      team_attnres_mix<VPT>(x, blocks + (size_t)b * kNbMax * H, sw, nb, eps, s_mix, t, nullptr, nullptr,
                            nb_stats > 0 ? stats + (size_t)b * kNbMax * 2 : nullptr, nb_stats);
    team_rms_store<VPT, true, false>(x, gamma, normed + base, nullptr, nullptr, eps, s_red[it & 1], t, rowmax ? rowmax + b : nullptr,
                                     s_amax[it & 1]);
  }
}

// ---- K1a fused with the preceding landing add and the following all-gather ---------------------
// kern_k3_attnres_rms_push of source/k3_residual_push_add2.cu:369-444: hidden = bf16(prefix2 + p1 (+ p2))
// (the K1c expression, f32 adds in that order, one rounding), optional snapshot, attention-residual
// mix with the statistics hand-off, RMSNorm, and the normed row stored to this rank's slice of every
// rank's normed_all (own copy write-back, peer copies streaming).  The barrier is a separate launch.
// ADD = false is the first layer's form (source/k3_residual_push_v3.cu:328-400): the row comes from `prefix2`
// as it is, nothing is added and no hidden row is stored.
template <int VPT, bool ADD = true>
__device__ __forceinline__ void attnres_rms_push_body(__nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw,
                                                      const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ normed_all,
                                                      const unsigned long long* __restrict__ dst_peer, int nb, int snapshot, int B, int rank,
                                                      int nranks, const float* __restrict__ sw_mlp, float* __restrict__ stats,
                                                      const __nv_bfloat16* __restrict__ p1, const __nv_bfloat16* __restrict__ p2,
                                                      const __nv_bfloat16* __restrict__ prefix2, __nv_bfloat16* __restrict__ hidden, int two,
                                                      float eps, float* __restrict__ rowmax_all = nullptr,
                                                      const unsigned long long* __restrict__ rowmax_peer = nullptr) {
  constexpr int H = VPT * 1024;
  __shared__ float s_red[2][kTeam / 32];
  __shared__ float s_mix[kMixSmem];
  __shared__ unsigned s_amax[2][kTeam / 32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nr = nranks < 8 ? nranks : 8;
  __nv_bfloat16* peer[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) peer[q] = (q < nr && q != rank) ? reinterpret_cast<__nv_bfloat16*>(dst_peer[q]) : nullptr;
  int it = 0;
  for (int b = blockIdx.x; b < B; b += gridDim.x, ++it) {
    const size_t base = (size_t)b * H;
    V8 x[VPT];
    if constexpr (!ADD) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) x[v] = ld_stream(prefix2 + base + (t + v * kTeam) * 8);
    } else {
      V8 a[VPT], c[VPT];
#pragma unroll
      for (int v = 0; v < VPT; ++v) a[v] = ld_stream(prefix2 + base + (t + v * kTeam) * 8);
#pragma unroll
      for (int v = 0; v < VPT; ++v) c[v] = ld_stream(p1 + base + (t + v * kTeam) * 8);
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[2 * j] = __fadd_rn(bf_lo(a[v].w[j]), bf_lo(c[v].w[j]));
          f[2 * j + 1] = __fadd_rn(bf_hi(a[v].w[j]), bf_hi(c[v].w[j]));
        }
        if (two) {
          const V8 e = ld_stream(p2 + base + (t + v * kTeam) * 8);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            f[2 * j] = __fadd_rn(f[2 * j], bf_lo(e.w[j]));
            f[2 * j + 1] = __fadd_rn(f[2 * j + 1], bf_hi(e.w[j]));
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) x[v].w[j] = pack_bf2(f[2 * j], f[2 * j + 1]);
        st_plain(hidden + base + (t + v * kTeam) * 8, x[v]);
      }
    }
    __nv_bfloat16* blk_row = blocks + (size_t)b * kNbMax * H;
    if (snapshot && nb < kNbMax) {
#pragma unroll
      for (int v = 0; v < VPT; ++v) st_plain(blk_row + (size_t)nb * H + (t + v * kTeam) * 8, x[v]);
    }
    if (nb > 0)
      team_attnres_mix<VPT, true>(x, blk_row, sw, nb, eps, s_mix, t, stats ? sw_mlp : nullptr, stats ? stats + (size_t)b * kNbMax * 2 : nullptr);
    const float tot = team_sumsq<VPT>(x, s_red[it & 1], lane, warp);
    const float r = __frsqrt_rn(__fmaf_rn(tot, 1.0f / (float)H, eps));
    const size_t dst_off = ((size_t)rank * B + b) * H;
    unsigned m2 = 0u;
    V8 held = V8{{0u, 0u, 0u, 0u}};
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int u = (t + v * kTeam) * 8;
      const V8 g = ld_keep(gamma + u);
      V8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(x[v].w[j]), r), __fmul_rn(bf_hi(x[v].w[j]), r)), g.w[j]);
        m2 = __vmaxu2(m2, o.w[j] & 0x7fff7fffu);
      }
      st_plain(normed_all + dst_off + u, o);            // own slice: the next GEMM reads it, keep it in L2
      // Peer copies leave as 32-byte stores (over NVLink the wider store moves measurably more): vectors go in pairs
      // (v - 1, v); the even lane of a lane pair stores its own and its neighbour's vector v - 1, the odd lane the
      // two vectors v, after the lanes have handed each other the missing halves.
      if ((v & 1) == 0 && v + 1 < VPT) {
        held = o;
      } else if ((v & 1) == 1) {
        const bool odd = (lane & 1) != 0;
        V8 got;
#pragma unroll
        for (int j = 0; j < 4; ++j) got.w[j] = __shfl_xor_sync(0xffffffffu, odd ? held.w[j] : o.w[j], 1);
        V16 w;
#pragma unroll
        for (int j = 0; j < 4; ++j) { w.w[j] = odd ? got.w[j] : held.w[j]; w.w[4 + j] = odd ? o.w[j] : got.w[j]; }
        const int uu = odd ? u - 8 : u - kTeam * 8;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (peer[q] != nullptr) st_stream32(peer[q] + dst_off + uu, w);
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (peer[q] != nullptr) st_stream(peer[q] + dst_off + u, o);
      }
    }
    if (rowmax_all != nullptr) {                        // max |normed| of the row, gathered like the row itself
      const unsigned m = team_absmax_bits(m2, s_amax[it & 1], lane, warp);
      if (t == 0) {
        const float f = __uint_as_float(m << 16);
        const size_t at = (size_t)rank * B + b;
        rowmax_all[at] = f;
        for (int q = 0; q < nr; ++q)
          if (q != rank) reinterpret_cast<float*>(rowmax_peer[q])[at] = f;
      }
    }
  }
}

// ---- K1c ----------------------------------------------------------------------------------
template <int VPT, bool LB16>
__device__ __forceinline__ void land_add2_body(const void* __restrict__ p1, const void* __restrict__ p2,
                                               const __nv_bfloat16* __restrict__ prefix2, __nv_bfloat16* __restrict__ hidden,
                                               int two, int B) {
  constexpr int H = VPT * 1024;
  const int t = threadIdx.x;
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const size_t off = (size_t)b * H + (t + v * kTeam) * 8;
      const V8 pr = ld_stream(prefix2 + off);
      float l1[8], l2[8];
      if (LB16) {
        const V8 a = ld_stream((const __nv_bfloat16*)p1 + off);
#pragma unroll
        for (int j = 0; j < 4; ++j) { l1[2 * j] = bf_lo(a.w[j]); l1[2 * j + 1] = bf_hi(a.w[j]); }
        if (two) {
          const V8 c = ld_stream((const __nv_bfloat16*)p2 + off);
#pragma unroll
          for (int j = 0; j < 4; ++j) { l2[2 * j] = bf_lo(c.w[j]); l2[2 * j + 1] = bf_hi(c.w[j]); }
        }
      } else {
        const V8 a0 = ld_stream((const float*)p1 + off), a1 = ld_stream((const float*)p1 + off + 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) { l1[j] = land_bf(__uint_as_float(a0.w[j])); l1[4 + j] = land_bf(__uint_as_float(a1.w[j])); }
        if (two) {
          const V8 c0 = ld_stream((const float*)p2 + off), c1 = ld_stream((const float*)p2 + off + 4);
#pragma unroll
          for (int j = 0; j < 4; ++j) { l2[j] = land_bf(__uint_as_float(c0.w[j])); l2[4 + j] = land_bf(__uint_as_float(c1.w[j])); }
        }
      }
      V8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float x = __fadd_rn(bf_lo(pr.w[j]), l1[2 * j]), y = __fadd_rn(bf_hi(pr.w[j]), l1[2 * j + 1]);
        if (two) { x = __fadd_rn(x, l2[2 * j]); y = __fadd_rn(y, l2[2 * j + 1]); }
        o.w[j] = pack_bf2(x, y);
      }
      st_stream(hidden + off, o);
    }
  }
}

}  // namespace k3g

using namespace k3g;

// ---- manifest entry points (reference ABI; H = 7168 and eps = 1e-5 are build constants
//      there: source/k3_residual_v2.cu:51-54) ------------------------------------------------
#ifndef K3G_RES_VPT
#define K3G_RES_VPT 7
#endif
#ifndef K3G_RES_EPS
#define K3G_RES_EPS 1e-5f
#endif

extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_attnres_rms(
    const __nv_bfloat16* __restrict__ prefix, __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw,
    const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ normed, int nb, int snapshot, int B) {
  attnres_rms_body<K3G_RES_VPT>(prefix, blocks, sw, gamma, normed, nb, snapshot, B, K3G_RES_EPS);
}

#ifdef K3G_PUSH_V3
// op attnres_rms_push_first_v3 (module k3_residual_push_v3): 11 kernel parameters, reference order.
extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_attnres_rms_push(
    const __nv_bfloat16* __restrict__ prefix, __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw,
    const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ normed_all, const unsigned long long* __restrict__ dst_peer, int nb,
    int snapshot, int B, int rank, int nranks) {
  attnres_rms_push_body<K3G_RES_VPT, false>(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, nullptr, nullptr, nullptr,
                                            nullptr, prefix, nullptr, 0, K3G_RES_EPS);
}
#else
// op attnres_rms_push_add2 (module k3_residual_push_add2): 17 kernel parameters, reference order.
extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_attnres_rms_push(
    __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma,
    __nv_bfloat16* __restrict__ normed_all, const unsigned long long* __restrict__ dst_peer, int nb, int snapshot, int B, int rank,
    int nranks, const float* __restrict__ sw_mlp, float* __restrict__ stats, const __nv_bfloat16* __restrict__ p1,
    const __nv_bfloat16* __restrict__ p2, const __nv_bfloat16* __restrict__ prefix2, __nv_bfloat16* __restrict__ hidden, int two) {
  attnres_rms_push_body<K3G_RES_VPT>(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, sw_mlp, stats, p1, p2, prefix2,
                                     hidden, two, K3G_RES_EPS);
}
#endif

#if defined(K3G_CUBIN_ONLY) && defined(K3G_FUSED_ENTRIES)
// Module k3g_fused_residual: the fusions beyond the reference's call list as cubin entries with fixed parameter lists,
// for a manifest rewritten by `patch_manifest.py --fuse`.  The tensor-parallel width is a build constant (K3G_NR), as in
// the reference's own collectives (source/k3_reducescatter_pull_nr4.cu:135).
#ifndef K3G_NR
#define K3G_NR 4
#endif
// op attnres_rms_push_add2_amax: kern_k3_attnres_rms_push's 17 parameters, then the gathered row maxima and their peer table
extern "C" __global__ void __launch_bounds__(128, 4) kern_k3g_attnres_rms_push_amax(
    __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma,
    __nv_bfloat16* __restrict__ normed_all, const unsigned long long* __restrict__ dst_peer, int nb, int snapshot, int B, int rank,
    int nranks, const float* __restrict__ sw_mlp, float* __restrict__ stats, const __nv_bfloat16* __restrict__ p1,
    const __nv_bfloat16* __restrict__ p2, const __nv_bfloat16* __restrict__ prefix2, __nv_bfloat16* __restrict__ hidden, int two,
    float* __restrict__ rowmax_all, const unsigned long long* __restrict__ rowmax_peer) {
  attnres_rms_push_body<K3G_RES_VPT>(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, sw_mlp, stats, p1, p2, prefix2,
                                     hidden, two, K3G_RES_EPS, rowmax_all, rowmax_peer);
}
// op rs_land_add_attnres_rms (second launch; the first is the arrive barrier): the pull reduce-scatter inside the landing
extern "C" __global__ void __launch_bounds__(128, 4) kern_k3g_rs_land_add_attnres_rms(
    const __nv_bfloat16* __restrict__ partial, const unsigned long long* __restrict__ partial_peer, int rank, int nranks,
    const __nv_bfloat16* __restrict__ prefix, const __nv_bfloat16* __restrict__ blocks, const float* __restrict__ sw,
    const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ prefix2, __nv_bfloat16* __restrict__ normed, int nb, int snapshot,
    int B, const float* __restrict__ stats, int nb_stats, float* __restrict__ rowmax) {
  if (nranks != K3G_NR) return;                        // one module per world size, as the reference's pull kernel
  land_add_attnres_rms_body<K3G_RES_VPT, true, K3G_NR>(partial, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, K3G_RES_EPS, stats,
                                                       nb_stats, rowmax, partial_peer, rank);
}
#endif

#if defined(K3G_CUBIN_ONLY)
// one landing dtype per module, as in the reference (-DLAND_BF16 selects bf16)
#ifdef LAND_BF16
typedef __nv_bfloat16 k3g_land_t;
#define K3G_LAND_IS_BF16 true
#else
typedef float k3g_land_t;
#define K3G_LAND_IS_BF16 false
#endif
extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_land_add_attnres_rms(
    const k3g_land_t* __restrict__ partial, const __nv_bfloat16* __restrict__ prefix, const __nv_bfloat16* __restrict__ blocks,
    const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ prefix2,
    __nv_bfloat16* __restrict__ normed, int nb, int snapshot, int B) {
  land_add_attnres_rms_body<K3G_RES_VPT, K3G_LAND_IS_BF16>(partial, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, K3G_RES_EPS);
}
// ops land_add_attnres_rms_bf16_v2_nb{1..8} (modules k3_residual_nb, k3_residual_nb_stats): one entry per
// candidate count in the reference; the count is a run-time argument here, the entries share one body.
#ifdef K3G_NB_NO_STATS   /* module k3_residual_nb: ten parameters, no statistics hand-off */
#define K3G_NB_ENTRY(K)                                                                                                          \
  extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_land_add_attnres_rms_nb##K(                                       \
      const k3g_land_t* __restrict__ partial, const __nv_bfloat16* __restrict__ prefix, const __nv_bfloat16* __restrict__ blocks, \
      const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ prefix2,                \
      __nv_bfloat16* __restrict__ normed, int nb_in, int snapshot, int B) {                                                       \
    if (nb_in != K) return;                                                                                                      \
    land_add_attnres_rms_body<K3G_RES_VPT, K3G_LAND_IS_BF16>(partial, prefix, blocks, sw, gamma, prefix2, normed, K, snapshot, B, \
                                                             K3G_RES_EPS);                                                       \
  }
#else                    /* module k3_residual_nb_stats: twelve parameters */
#define K3G_NB_ENTRY(K)                                                                                                          \
  extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_land_add_attnres_rms_nb##K(                                       \
      const k3g_land_t* __restrict__ partial, const __nv_bfloat16* __restrict__ prefix, const __nv_bfloat16* __restrict__ blocks, \
      const float* __restrict__ sw, const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ prefix2,                \
      __nv_bfloat16* __restrict__ normed, int nb_in, int snapshot, int B, const float* __restrict__ stats, int nb_stats) {        \
    if (nb_in != K) return;                                                                                                      \
    land_add_attnres_rms_body<K3G_RES_VPT, K3G_LAND_IS_BF16>(partial, prefix, blocks, sw, gamma, prefix2, normed, K, snapshot, B, \
                                                             K3G_RES_EPS, stats, nb_stats);                                      \
  }
#endif
K3G_NB_ENTRY(1) K3G_NB_ENTRY(2) K3G_NB_ENTRY(3) K3G_NB_ENTRY(4) K3G_NB_ENTRY(5) K3G_NB_ENTRY(6) K3G_NB_ENTRY(7) K3G_NB_ENTRY(8)

extern "C" __global__ void __launch_bounds__(128, 4) kern_k3_land_add2(
    const k3g_land_t* __restrict__ p1, const k3g_land_t* __restrict__ p2, const __nv_bfloat16* __restrict__ prefix2,
    __nv_bfloat16* __restrict__ hidden, int two, int B) {
  land_add2_body<K3G_RES_VPT, K3G_LAND_IS_BF16>(p1, p2, prefix2, hidden, two, B);
}
#else

// ---- library build: width- and dtype-generic kernels behind the C ABI ----------------------
template <int VPT>
__global__ void __launch_bounds__(128, 4) attnres_rms_kernel(const __nv_bfloat16* prefix, __nv_bfloat16* blocks, const float* sw,
                                                            const __nv_bfloat16* gamma, __nv_bfloat16* normed, int nb, int snapshot, int B, float eps) {
  attnres_rms_body<VPT>(prefix, blocks, sw, gamma, normed, nb, snapshot, B, eps);
}
template <int VPT, bool LB>
__global__ void __launch_bounds__(128, 4) land_add_attnres_rms_kernel(const void* partial, const __nv_bfloat16* prefix, const __nv_bfloat16* blocks,
                                                                     const float* sw, const __nv_bfloat16* gamma, __nv_bfloat16* prefix2,
                                                                     __nv_bfloat16* normed, int nb, int snapshot, int B, float eps,
                                                                     const float* stats, int nb_stats, float* rowmax) {
  land_add_attnres_rms_body<VPT, LB>(partial, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, eps, stats, nb_stats, rowmax);
}
template <int VPT, int NR>
__global__ void __launch_bounds__(128, 4) rs_land_add_attnres_rms_kernel(const __nv_bfloat16* partial, const unsigned long long* partial_peer, int rank,
                                                                        const __nv_bfloat16* prefix, const __nv_bfloat16* blocks, const float* sw,
                                                                        const __nv_bfloat16* gamma, __nv_bfloat16* prefix2, __nv_bfloat16* normed,
                                                                        int nb, int snapshot, int B, float eps, const float* stats, int nb_stats,
                                                                        float* rowmax) {
  land_add_attnres_rms_body<VPT, true, NR>(partial, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, eps, stats, nb_stats, rowmax,
                                           partial_peer, rank);
}
template <int VPT, bool ADD>
__global__ void __launch_bounds__(128, 4) attnres_rms_push_kernel(__nv_bfloat16* blocks, const float* sw, const __nv_bfloat16* gamma,
                                                                 __nv_bfloat16* normed_all, const unsigned long long* dst_peer, int nb,
                                                                 int snapshot, int B, int rank, int nranks, const float* sw_mlp, float* stats,
                                                                 const __nv_bfloat16* p1, const __nv_bfloat16* p2, const __nv_bfloat16* prefix2,
                                                                 __nv_bfloat16* hidden, int two, float eps, float* rowmax_all,
                                                                 const unsigned long long* rowmax_peer) {
  attnres_rms_push_body<VPT, ADD>(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, sw_mlp, stats, p1, p2, prefix2, hidden, two, eps,
                                  rowmax_all, rowmax_peer);
}
template <int VPT, bool LB>
__global__ void __launch_bounds__(128, 4) land_add2_kernel(const void* p1, const void* p2, const __nv_bfloat16* prefix2,
                                                          __nv_bfloat16* hidden, int two, int B) {
  land_add2_body<VPT, LB>(p1, p2, prefix2, hidden, two, B);
}

#define K3G_DISPATCH_VPT(H, ...)                           \
  switch ((H) / 1024) {                                    \
    case 1: { constexpr int VPT = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int VPT = 2; __VA_ARGS__; } break; \
    case 4: { constexpr int VPT = 4; __VA_ARGS__; } break; \
    case 7: { constexpr int VPT = 7; __VA_ARGS__; } break; \
    case 8: { constexpr int VPT = 8; __VA_ARGS__; } break; \
    default: return K3G_ESHAPE;                            \
  }

static inline int res_grid(int rows, int grid_hint) { return grid_hint > 0 ? (grid_hint < rows ? grid_hint : rows) : rows; }

K3G_API int k3g_resnorm_mxfp8(const void* residual, const void* delta, const void* gamma, void* residual_out, void* q,
                              void* sf, void* normed_opt, int rows, int H, float eps, int grid_hint, void* stream) {
  K3G_REQUIRE_PTR(residual); K3G_REQUIRE_PTR(delta); K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(residual_out);
  K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(sf);
  K3G_REQUIRE_ALIGNED(residual); K3G_REQUIRE_ALIGNED(delta); K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(residual_out);
  K3G_REQUIRE_ALIGNED(q); K3G_REQUIRE_ALIGNED(sf); K3G_REQUIRE_ALIGNED(normed_opt);
  K3G_REQUIRE(rows >= 0 && H > 0 && H % 1024 == 0, K3G_ESHAPE);
  if (rows == 0) return K3G_OK;
  const int grid = res_grid(rows, grid_hint);
  K3G_DISPATCH_VPT(H, {
    if (normed_opt)
      resnorm_mxfp8_kernel<VPT, true><<<grid, kTeam, 0, k3g_stream(stream)>>>(
          (const __nv_bfloat16*)residual, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)residual_out,
          (uint8_t*)q, (uint8_t*)sf, (__nv_bfloat16*)normed_opt, rows, eps);
    else
      resnorm_mxfp8_kernel<VPT, false><<<grid, kTeam, 0, k3g_stream(stream)>>>(
          (const __nv_bfloat16*)residual, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)residual_out,
          (uint8_t*)q, (uint8_t*)sf, nullptr, rows, eps);
  });
  return k3g_launch_status();
}

K3G_API int k3g_attnres_rms(const void* prefix, void* blocks, const void* sw, const void* gamma, void* normed, int nb,
                            int snapshot, int B, int H, float eps, void* stream) {
  K3G_REQUIRE_PTR(prefix); K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(normed);
  K3G_REQUIRE(nb >= 0 && nb <= kNbMax, K3G_ERANGE);
  if (nb > 0 || snapshot) K3G_REQUIRE_PTR(blocks);
  if (nb > 0) K3G_REQUIRE_PTR(sw);
  K3G_REQUIRE_ALIGNED(prefix); K3G_REQUIRE_ALIGNED(blocks); K3G_REQUIRE_ALIGNED(sw); K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(normed);
  K3G_REQUIRE(B >= 0 && H > 0 && H % 1024 == 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  K3G_DISPATCH_VPT(H, (attnres_rms_kernel<VPT><<<B, kTeam, 0, k3g_stream(stream)>>>(
      (const __nv_bfloat16*)prefix, (__nv_bfloat16*)blocks, (const float*)sw, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)normed,
      nb, snapshot, B, eps)));
  return k3g_launch_status();
}

static int land_add_attnres_rms_impl(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                     const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                     int B, int H, float eps, const void* stats, int nb_stats, void* rowmax, void* stream) {
  K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(prefix2); K3G_REQUIRE_PTR(normed);
  if (!snapshot) K3G_REQUIRE_PTR(prefix);
  K3G_REQUIRE(nb >= 0 && nb <= kNbMax, K3G_ERANGE);
  if (nb > 0) { K3G_REQUIRE_PTR(blocks); K3G_REQUIRE_PTR(sw); }
  K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(prefix); K3G_REQUIRE_ALIGNED(blocks); K3G_REQUIRE_ALIGNED(sw);
  K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(prefix2); K3G_REQUIRE_ALIGNED(normed);
  K3G_REQUIRE(B >= 0 && H > 0 && H % 1024 == 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  if (partial_is_bf16) {
    K3G_DISPATCH_VPT(H, (land_add_attnres_rms_kernel<VPT, true><<<B, kTeam, 0, k3g_stream(stream)>>>(
        partial, (const __nv_bfloat16*)prefix, (const __nv_bfloat16*)blocks, (const float*)sw, (const __nv_bfloat16*)gamma,
        (__nv_bfloat16*)prefix2, (__nv_bfloat16*)normed, nb, snapshot, B, eps, (const float*)stats, nb_stats, (float*)rowmax)));
  } else {
    K3G_DISPATCH_VPT(H, (land_add_attnres_rms_kernel<VPT, false><<<B, kTeam, 0, k3g_stream(stream)>>>(
        partial, (const __nv_bfloat16*)prefix, (const __nv_bfloat16*)blocks, (const float*)sw, (const __nv_bfloat16*)gamma,
        (__nv_bfloat16*)prefix2, (__nv_bfloat16*)normed, nb, snapshot, B, eps, (const float*)stats, nb_stats, (float*)rowmax)));
  }
  return k3g_launch_status();
}

K3G_API int k3g_land_add_attnres_rms(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                     const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                     int B, int H, float eps, void* stream) {
  return land_add_attnres_rms_impl(partial, partial_is_bf16, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, H, eps, nullptr, 0,
                                   nullptr, stream);
}

// The per-candidate-count entries of the reference (kern_k3_land_add_attnres_rms_nb1..8) with the
// statistics hand-off: stats [B, 8, 2] = (sum x^2, sum x * sw) of snapshot candidates c < nb_stats, as
// written by k3g_attnres_rms_push; those candidates are not re-read in the scoring pass.
K3G_API int k3g_land_add_attnres_rms_stats(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                           const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                           int B, int H, float eps, const void* stats, int nb_stats, void* stream) {
  K3G_REQUIRE(nb_stats >= 0 && nb_stats <= nb, K3G_ERANGE);
  if (nb_stats > 0) K3G_REQUIRE_PTR(stats);
  return land_add_attnres_rms_impl(partial, partial_is_bf16, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, H, eps, stats,
                                   nb_stats, nullptr, stream);
}

// The same call with the row maxima a following per-tensor FP8 quantisation of `normed` needs:
// rowmax [B] f32 = max |normed[b, :]|, so that quantisation can skip its own pass over the tensor (k3g_quant_fp8_apply).
K3G_API int k3g_land_add_attnres_rms_stats_amax(const void* partial, int partial_is_bf16, const void* prefix, const void* blocks,
                                                const void* sw, const void* gamma, void* prefix2, void* normed, int nb, int snapshot,
                                                int B, int H, float eps, const void* stats, int nb_stats, void* rowmax, void* stream) {
  K3G_REQUIRE(nb_stats >= 0 && nb_stats <= nb, K3G_ERANGE);
  if (nb_stats > 0) K3G_REQUIRE_PTR(stats);
  K3G_REQUIRE_PTR(rowmax);
  return land_add_attnres_rms_impl(partial, partial_is_bf16, prefix, blocks, sw, gamma, prefix2, normed, nb, snapshot, B, H, eps, stats,
                                   nb_stats, rowmax, stream);
}

// kern_k3_attnres_rms_push (op attnres_rms_push_add2): landing add + snapshot + mix + RMSNorm + push of the
// normed row into every rank's normed_all [nranks * B, H]; stats (may be null) receives the hand-off.
// Pull reduce-scatter folded into the residual kernel that consumes it (no counterpart in the reference, which
// runs kern_k3_rs_pull and then kern_k3_land_add_attnres_rms_nbK): `partial` is this rank's [nranks * B, H] bf16
// buffer of partial sums, partial_peer the u64 table of every rank's buffer; row b lands the ring-order chain of
// row rank * B + b over the ranks (as k3g_rs_pull with order 2 (nranks - 1)) and continues as
// k3g_land_add_attnres_rms_stats_amax on it.  Outputs are bit-identical to the two calls in sequence; the
// reduce-scattered tensor itself is never written.  Bracket with k3g_rs_arrive as for k3g_rs_pull.  H = 7168,
// nranks in {1, 2, 4, 8}; stats and rowmax may be null.
K3G_API int k3g_rs_land_add_attnres_rms(const void* partial, const void* partial_peer, int rank, int nranks, const void* prefix,
                                        const void* blocks, const void* sw, const void* gamma, void* prefix2, void* normed, int nb,
                                        int snapshot, int B, int H, float eps, const void* stats, int nb_stats, void* rowmax, void* stream) {
  K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(partial_peer); K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(prefix2); K3G_REQUIRE_PTR(normed);
  if (!snapshot) K3G_REQUIRE_PTR(prefix);
  K3G_REQUIRE(nb >= 0 && nb <= kNbMax && nb_stats >= 0 && nb_stats <= nb, K3G_ERANGE);
  if (nb > 0) { K3G_REQUIRE_PTR(blocks); K3G_REQUIRE_PTR(sw); }
  if (nb_stats > 0) K3G_REQUIRE_PTR(stats);
  K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(prefix); K3G_REQUIRE_ALIGNED(blocks); K3G_REQUIRE_ALIGNED(sw);
  K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(prefix2); K3G_REQUIRE_ALIGNED(normed);
  K3G_REQUIRE(B >= 0 && H == 7168 && (nranks == 1 || nranks == 2 || nranks == 4 || nranks == 8), K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks, K3G_ERANGE);
  if (nranks > 1) K3G_REQUIRE((reinterpret_cast<uintptr_t>(partial) & 31u) == 0, K3G_EALIGN);   // peers are read 32 bytes at a time
  if (B == 0) return K3G_OK;
#define K3G_RS_K1B(NR)                                                                                                                         \
  rs_land_add_attnres_rms_kernel<7, NR><<<B, kTeam, 0, k3g_stream(stream)>>>(                                                                   \
      (const __nv_bfloat16*)partial, (const unsigned long long*)partial_peer, rank, (const __nv_bfloat16*)prefix, (const __nv_bfloat16*)blocks, \
      (const float*)sw, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)prefix2, (__nv_bfloat16*)normed, nb, snapshot, B, eps, (const float*)stats,  \
      nb_stats, (float*)rowmax)
  switch (nranks) {
    case 1: K3G_RS_K1B(1); break;
    case 2: K3G_RS_K1B(2); break;
    case 4: K3G_RS_K1B(4); break;
    default: K3G_RS_K1B(8); break;
  }
#undef K3G_RS_K1B
  return k3g_launch_status();
}

static int attnres_rms_push_impl(void* blocks, const void* sw, const void* gamma, void* normed_all, const void* dst_peer, int nb,
                                 int snapshot, int B, int rank, int nranks, const void* sw_mlp, void* stats, const void* p1,
                                 const void* p2, const void* prefix2, void* hidden, int two, int H, float eps, void* rowmax_all,
                                 const void* rowmax_peer, void* stream) {
  K3G_REQUIRE_PTR(gamma); K3G_REQUIRE_PTR(normed_all); K3G_REQUIRE_PTR(dst_peer); K3G_REQUIRE_PTR(prefix2);
  if (p1) K3G_REQUIRE_PTR(hidden);
  if (two) { K3G_REQUIRE_PTR(p1); K3G_REQUIRE_PTR(p2); }
  K3G_REQUIRE(nb >= 0 && nb <= kNbMax, K3G_ERANGE);
  if (nb > 0 || snapshot) K3G_REQUIRE_PTR(blocks);
  if (nb > 0) K3G_REQUIRE_PTR(sw);
  if (stats) K3G_REQUIRE_PTR(sw_mlp);
  K3G_REQUIRE(nranks >= 1 && nranks <= 8 && B >= 0 && H > 0 && H % 1024 == 0, K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks, K3G_ERANGE);
  K3G_REQUIRE_ALIGNED(blocks); K3G_REQUIRE_ALIGNED(sw); K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(normed_all); K3G_REQUIRE_ALIGNED(sw_mlp);
  K3G_REQUIRE_ALIGNED(p1); K3G_REQUIRE_ALIGNED(p2); K3G_REQUIRE_ALIGNED(prefix2); K3G_REQUIRE_ALIGNED(hidden);
  if (B == 0) return K3G_OK;
  if (p1) {
    K3G_DISPATCH_VPT(H, (attnres_rms_push_kernel<VPT, true><<<B, kTeam, 0, k3g_stream(stream)>>>(
        (__nv_bfloat16*)blocks, (const float*)sw, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)normed_all, (const unsigned long long*)dst_peer, nb,
        snapshot, B, rank, nranks, (const float*)sw_mlp, (float*)stats, (const __nv_bfloat16*)p1, (const __nv_bfloat16*)p2,
        (const __nv_bfloat16*)prefix2, (__nv_bfloat16*)hidden, two, eps, (float*)rowmax_all, (const unsigned long long*)rowmax_peer)));
  } else {                                               // first layer: the row is prefix2 itself
    K3G_DISPATCH_VPT(H, (attnres_rms_push_kernel<VPT, false><<<B, kTeam, 0, k3g_stream(stream)>>>(
        (__nv_bfloat16*)blocks, (const float*)sw, (const __nv_bfloat16*)gamma, (__nv_bfloat16*)normed_all, (const unsigned long long*)dst_peer, nb,
        snapshot, B, rank, nranks, (const float*)sw_mlp, (float*)stats, nullptr, nullptr, (const __nv_bfloat16*)prefix2, nullptr, 0, eps,
        (float*)rowmax_all, (const unsigned long long*)rowmax_peer)));
  }
  return k3g_launch_status();
}

K3G_API int k3g_attnres_rms_push(void* blocks, const void* sw, const void* gamma, void* normed_all, const void* dst_peer, int nb,
                                 int snapshot, int B, int rank, int nranks, const void* sw_mlp, void* stats, const void* p1,
                                 const void* p2, const void* prefix2, void* hidden, int two, int H, float eps, void* stream) {
  return attnres_rms_push_impl(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, sw_mlp, stats, p1, p2, prefix2, hidden, two,
                               H, eps, nullptr, nullptr, stream);
}

// The same call with the row maxima a following per-tensor FP8 quantisation of the gathered normed_all needs:
// rowmax_all [nranks * B] f32 on every rank (rowmax_peer = its peer table) receives max |normed row| at index
// rank * B + b, pushed like the row itself, so that quantisation can skip its own pass (k3g_quant_fp8_apply).
K3G_API int k3g_attnres_rms_push_amax(void* blocks, const void* sw, const void* gamma, void* normed_all, const void* dst_peer, int nb,
                                      int snapshot, int B, int rank, int nranks, const void* sw_mlp, void* stats, const void* p1,
                                      const void* p2, const void* prefix2, void* hidden, int two, int H, float eps, void* rowmax_all,
                                      const void* rowmax_peer, void* stream) {
  K3G_REQUIRE_PTR(rowmax_all); K3G_REQUIRE_PTR(rowmax_peer);
  return attnres_rms_push_impl(blocks, sw, gamma, normed_all, dst_peer, nb, snapshot, B, rank, nranks, sw_mlp, stats, p1, p2, prefix2, hidden, two,
                               H, eps, rowmax_all, rowmax_peer, stream);
}

K3G_API int k3g_land_add2(const void* p1, const void* p2, int partial_is_bf16, const void* prefix2, void* hidden, int two,
                          int B, int H, void* stream) {
  K3G_REQUIRE_PTR(p1); K3G_REQUIRE_PTR(prefix2); K3G_REQUIRE_PTR(hidden);
  if (two) K3G_REQUIRE_PTR(p2);
  K3G_REQUIRE_ALIGNED(p1); K3G_REQUIRE_ALIGNED(p2); K3G_REQUIRE_ALIGNED(prefix2); K3G_REQUIRE_ALIGNED(hidden);
  K3G_REQUIRE(B >= 0 && H > 0 && H % 1024 == 0, K3G_ESHAPE);
  if (B == 0) return K3G_OK;
  if (partial_is_bf16) {
    K3G_DISPATCH_VPT(H, (land_add2_kernel<VPT, true><<<B, kTeam, 0, k3g_stream(stream)>>>(p1, p2, (const __nv_bfloat16*)prefix2,
                                                                                         (__nv_bfloat16*)hidden, two, B)));
  } else {
    K3G_DISPATCH_VPT(H, (land_add2_kernel<VPT, false><<<B, kTeam, 0, k3g_stream(stream)>>>(p1, p2, (const __nv_bfloat16*)prefix2,
                                                                                          (__nv_bfloat16*)hidden, two, B)));
  }
  return k3g_launch_status();
}
#endif  // K3G_CUBIN_ONLY
