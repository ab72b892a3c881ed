// TEST INFRASTRUCTURE — CPU oracle of the K3 MoE-prefill glue ops.
//
// A plain C++/OpenMP restatement of the device kernels of xiaguan/kern-k3 that the
// library re-implements for B200.  Only the test-suite, the smoke check and the
// benchmark's CPU-baseline / reference arm may build, link or call this file; the
// shipped library never does.  Every function cites the reference lines it follows and
// reproduces their accumulation order (thread-serial chain -> warp xor-butterfly ->
// fixed-order sum of warp partials), with the fused multiply-adds the reference build
// (nvcc default -fmad=true) produces written out as std::fmaf.  Compile with
// -ffp-contract=off so the host compiler adds none of its own.
//
// PARITY PIN: the reference ships no unit tests, golden vectors or CPU path for these
// kernels; this oracle is pinned (a) against hand-computable known answers and the
// committed fixtures under tests/golden/, and (b) on a GPU box against the reference's
// own .cu sources compiled for sm_100a (oracle/build_ref.py -> oracle/_ref/*.cubin).
//
// Deviations from the reference arithmetic, chosen so CPU and GPU can agree bit for bit:
//   rsqrtf -> round-to-nearest rsqrt;  expf in the router sigmoid and __expf in the softmax
//   of the attention-residual mix -> k3o::det_exp (a handful of values per row).
// The per-element ex2.approx / rcp.approx / __expf sites (SiLU, output-gate sigmoid) use
// libm here and are compared at bf16 tolerance.
#include "k3o_numerics.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

using namespace k3o;
typedef uint16_t u16;
typedef uint8_t u8;

#define K3O_API extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------ numerics exports
K3O_API uint16_t k3o_f32_to_bf16(float f) { return f2bf(f); }
K3O_API float k3o_bf16_to_f32(uint16_t h) { return bf2f(h); }
K3O_API uint8_t k3o_e4m3_encode(float f) { return e4m3_encode(f); }
K3O_API float k3o_e4m3_decode(uint8_t c) { return e4m3_decode(c); }
K3O_API int k3o_ue8m0_exp(float amax) { return ue8m0_exp(amax); }
K3O_API float k3o_rsqrt_rn(float x) { return rsqrt_rn(x); }
K3O_API float k3o_det_exp(float x) { return det_exp(x); }
K3O_API float k3o_det_sigmoid(float x) { return det_sigmoid(x); }
// The literal formula of the reference, for the equivalence test of ue8m0_exp.
K3O_API int k3o_ue8m0_exp_float_formula(float amax) {
  int e = amax > 0.f ? (int)std::ceil(std::log2(amax / 448.f)) : 0;
  return std::min(std::max(e, -127), 127);
}

// xor-butterfly over n lanes (n a power of two): the value every lane holds after
// `for (o = n/2; o > 0; o >>= 1) v += shfl_xor(v, o)`  (source/k3_residual_v2.cu:94-98).
static inline float butterfly(float* v, int n) {
  for (int o = n / 2; o > 0; o >>= 1)
    for (int i = 0; i < o; ++i) v[i] = v[i] + v[i + o];
  return v[0];
}

// ------------------------------------------------------------------ residual family
// Row reduction of source/k3_residual_v2.cu: 128 threads per row, thread t owns the
// 16-byte vectors t + 128 v (v = 0 .. H/1024 - 1), eight elements each (:128-129, :229-235).
struct RowLayout {
  int H, threads, vpt;
  explicit RowLayout(int h) : H(h), threads(128), vpt(h / 8 / 128) {}
};

// sum over the row of fn(element index), in the reference's order.  fn returns the pair
// (a, b) whose product is accumulated by one fma per element.
template <class F>
static float row_reduce(const RowLayout& L, F fn) {
  float warp_part[4];
  for (int w = 0; w < 4; ++w) {
    float lanes[32];
    for (int l = 0; l < 32; ++l) {
      const int t = w * 32 + l;
      float acc = 0.f;
      for (int v = 0; v < L.vpt; ++v) {
        const int u = (t + v * L.threads) * 8;
        for (int j = 0; j < 8; ++j) {
          float a, b;
          fn(u + j, a, b);
          acc = std::fmaf(a, b, acc);
        }
      }
      lanes[l] = acc;
    }
    warp_part[w] = butterfly(lanes, 32);
  }
  float tot = 0.f;
  for (int w = 0; w < 4; ++w) tot += warp_part[w];       // :239-241
  return tot;
}

// attnres_rms_row (source/k3_residual_v2.cu:107-257).  pv: the prefix candidate (bf16 row,
// overwritten with the mixed row); blk_row: the nb snapshot rows.
// Statistics hand-off: sw_other/stats_out (producer, source/k3_residual_push_add2.cu:273-279) and
// stats_in/nb_stats (consumer, source/k3_residual_nb_stats.cu:254-258); [8][2] floats for this row.
static void attnres_rms_row(const RowLayout& L, const u16* blk_row, u16* pv, const float* sw,
                            const u16* gamma, u16* normed_row, int nb, float eps, const float* sw_other = nullptr,
                            float* stats_out = nullptr, const float* stats_in = nullptr, int nb_stats = 0) {
  const int H = L.H;
  const float invH = 1.0f / (float)H;
  if (nb > 0) {
    const int ncand = nb + 1;
    float sc[32];
    for (int l = 0; l < 32; ++l) sc[l] = -3.0e38f;
    for (int c = 0; c < ncand; ++c) {                    // lane c's candidate (:171-179)
      const u16* x = (c < nb) ? blk_row + (size_t)c * H : pv;
      float sq, dp;
      if (stats_in && c < nb_stats && c < nb) {
        sq = stats_in[2 * c]; dp = stats_in[2 * c + 1];
      } else {
        sq = row_reduce(L, [&](int e, float& a, float& b) { a = bf2f(x[e]); b = a; });
        dp = row_reduce(L, [&](int e, float& a, float& b) { a = bf2f(x[e]); b = sw[e]; });
      }
      if (stats_out && c < nb) {
        stats_out[2 * c] = sq;
        stats_out[2 * c + 1] = row_reduce(L, [&](int e, float& a, float& b) { a = bf2f(x[e]); b = sw_other[e]; });
      }
      sc[c] = dp * rsqrt_rn(std::fmaf(sq, invH, eps));
    }
    float mxv[32];
    for (int l = 0; l < 32; ++l) mxv[l] = sc[l];
    for (int o = 16; o > 0; o >>= 1)
      for (int i = 0; i < o; ++i) mxv[i] = std::fmax(mxv[i], mxv[i + o]);
    const float mx = mxv[0];
    float ex[32], den[32];
    for (int l = 0; l < 32; ++l) { ex[l] = (l < ncand) ? det_exp(sc[l] - mx) : 0.f; den[l] = ex[l]; }
    const float dsum = butterfly(den, 32);
    float p[9];
    for (int c = 0; c < ncand; ++c) p[c] = ex[c] / dsum;
    const float pp = p[nb];
    for (int e = 0; e < H; ++e) {                        // pass 2 (:195-222)
      float acc = pp * bf2f(pv[e]);
      for (int c = 0; c < nb; ++c) acc = std::fmaf(p[c], bf2f(blk_row[(size_t)c * H + e]), acc);
      pv[e] = f2bf(acc);
    }
  }
  const float tot = row_reduce(L, [&](int e, float& a, float& b) { a = bf2f(pv[e]); b = a; });
  const float r = rsqrt_rn(std::fmaf(tot, invH, eps));   // :242
  for (int e = 0; e < H; ++e)                            // :250-254
    normed_row[e] = bfmul(f2bf(bf2f(pv[e]) * r), gamma[e]);
}

// kern_k3_attnres_rms (source/k3_residual_v2.cu:260-284).
K3O_API void k3o_attnres_rms(const u16* prefix, u16* blocks, const float* sw, const u16* gamma,
                             u16* normed, int nb, int snapshot, int B, int H, float eps) {
  const RowLayout L(H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<u16> pv(prefix + (size_t)b * H, prefix + (size_t)(b + 1) * H);
    if (snapshot && nb < 8) std::memcpy(blocks + ((size_t)b * 8 + nb) * H, pv.data(), (size_t)H * 2);
    attnres_rms_row(L, blocks ? blocks + (size_t)b * 8 * H : nullptr, pv.data(), sw, gamma,
                    normed + (size_t)b * H, nb, eps);
  }
}

// kern_k3_land_add_attnres_rms (source/k3_residual_v2.cu:295-345).  partial is bf16
// (LAND_BF16) or f32; p = bf16(partial) first, prefix2 = snapshot ? p : bf16(prefix + p).
K3O_API void k3o_land_add_attnres_rms(const void* partial, int partial_is_bf16, const u16* prefix,
                                      const u16* blocks, const float* sw, const u16* gamma, u16* prefix2,
                                      u16* normed, int nb, int snapshot, int B, int H, float eps) {
  const RowLayout L(H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<u16> pv(H);
    for (int e = 0; e < H; ++e) {
      const size_t off = (size_t)b * H + e;
      const u16 p = partial_is_bf16 ? ((const u16*)partial)[off] : f2bf(((const float*)partial)[off]);
      pv[e] = snapshot ? p : f2bf(bf2f(prefix[off]) + bf2f(p));
      prefix2[off] = pv[e];
    }
    attnres_rms_row(L, blocks ? blocks + (size_t)b * 8 * H : nullptr, pv.data(), sw, gamma,
                    normed + (size_t)b * H, nb, eps);
  }
}

// kern_k3_land_add_attnres_rms_nbK with the statistics of candidates c < nb_stats taken from `stats`
// [B, 8, 2] (source/k3_residual_nb_stats.cu:366-842).
K3O_API void k3o_land_add_attnres_rms_stats(const void* partial, int partial_is_bf16, const u16* prefix, const u16* blocks,
                                            const float* sw, const u16* gamma, u16* prefix2, u16* normed, int nb,
                                            int snapshot, int B, int H, float eps, const float* stats, int nb_stats) {
  const RowLayout L(H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<u16> pv(H);
    for (int e = 0; e < H; ++e) {
      const size_t off = (size_t)b * H + e;
      const u16 p = partial_is_bf16 ? ((const u16*)partial)[off] : f2bf(((const float*)partial)[off]);
      pv[e] = snapshot ? p : f2bf(bf2f(prefix[off]) + bf2f(p));
      prefix2[off] = pv[e];
    }
    attnres_rms_row(L, blocks + (size_t)b * 8 * H, pv.data(), sw, gamma, normed + (size_t)b * H, nb, eps, nullptr, nullptr,
                    stats + (size_t)b * 16, nb_stats);
  }
}

// kern_k3_attnres_rms_push (source/k3_residual_push_add2.cu:369-444): hidden = bf16((prefix2 + p1) + p2),
// snapshot, mix (+ statistics for the next residual kernel), RMSNorm.  `normed` is the row block every
// rank receives at rows [rank * B, (rank + 1) * B) of its normed_all.
K3O_API void k3o_attnres_rms_push(u16* blocks, const float* sw, const u16* gamma, u16* normed, int nb, int snapshot, int B,
                                  const float* sw_mlp, float* stats, const u16* p1, const u16* p2, const u16* prefix2,
                                  u16* hidden, int two, int H, float eps) {
  const RowLayout L(H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<u16> pv(H);
    for (int e = 0; e < H; ++e) {
      const size_t off = (size_t)b * H + e;
      float x = bf2f(prefix2[off]) + bf2f(p1[off]);
      if (two) x += bf2f(p2[off]);
      pv[e] = f2bf(x);
      hidden[off] = pv[e];
    }
    if (snapshot && nb < 8) std::memcpy(blocks + ((size_t)b * 8 + nb) * H, pv.data(), (size_t)H * 2);
    attnres_rms_row(L, blocks ? blocks + (size_t)b * 8 * H : nullptr, pv.data(), sw, gamma, normed + (size_t)b * H, nb, eps,
                    stats ? sw_mlp : nullptr, stats ? stats + (size_t)b * 16 : nullptr);
  }
}

// kern_k3_land_add2 (source/k3_residual_v2.cu:349-392; bf16-partial form
// source/k3_land_bf16.cu:96).
K3O_API void k3o_land_add2(const void* p1, const void* p2, int partial_is_bf16, const u16* prefix2,
                           u16* hidden, int two, int B, int H) {
  const size_t n = (size_t)B * H;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) {
    const float l1 = partial_is_bf16 ? bf2f(((const u16*)p1)[i]) : land(((const float*)p1)[i]);
    float x = bf2f(prefix2[i]) + l1;
    if (two) x += partial_is_bf16 ? bf2f(((const u16*)p2)[i]) : land(((const float*)p2)[i]);
    hidden[i] = f2bf(x);
  }
}

// ------------------------------------------------------------------ quantisation
// kern_quant_fp8_amax_v2 + kern_quant_fp8_apply_v2 (source/k3_quant_fp8_pair_v2.cu:42-95).
K3O_API void k3o_quant_fp8_tensor(const u16* x, u8* y, float* scale_out, long long n) {
  unsigned m = 0;
#pragma omp parallel for reduction(max : m) schedule(static)
  for (long long i = 0; i < n; ++i) m = std::max(m, (unsigned)(x[i] & 0x7fffu));
  const float amax = bf2f((u16)m);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  if (scale_out) scale_out[0] = scale;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < n; ++i) y[i] = e4m3_encode(bf2f(x[i]) * inv);
}

// kern_k3_moe_quant (source/k3_moe_prefill_v4.cu:111-140): MXFP8, one UE8M0 scale per 32.
static inline void mxfp8_group(const u16* x, u8* q, u8* sf) {
  float amax = 0.f;
  for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(bf2f(x[j])));
  const int e = ue8m0_exp(amax);
  const float s = pow2_neg(e);
  *sf = (u8)(e + 127);
  for (int j = 0; j < 32; ++j) q[j] = e4m3_encode(bf2f(x[j]) * s);
}

K3O_API void k3o_moe_quant(const u16* x, u8* q, u8* sf, long long rows, int cols) {
  const long long groups = rows * cols / 32;
#pragma omp parallel for schedule(static)
  for (long long g = 0; g < groups; ++g) mxfp8_group(x + g * 32, q + g * 32, sf + g);
}

// Config-level fusion: residual add + RMSNorm + MXFP8.  It is exactly
// kern_k3_land_add_attnres_rms with nb = 0, snapshot = 0 and a bf16 landing
// (source/k3_residual_v2.cu:295-345, :224-256) followed by kern_k3_moe_quant's formula on
// the bf16 normed row (source/k3_moe_prefill_v4.cu:111-140).  normed_opt may be null.
K3O_API void k3o_resnorm_mxfp8(const u16* residual, const u16* delta, const u16* gamma, u16* residual_out,
                               u8* q, u8* sf, u16* normed_opt, int B, int H, float eps) {
  const RowLayout L(H);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<u16> pv(H), nr(H);
    for (int e = 0; e < H; ++e) {
      const size_t off = (size_t)b * H + e;
      pv[e] = f2bf(bf2f(residual[off]) + bf2f(delta[off]));
      residual_out[off] = pv[e];
    }
    attnres_rms_row(L, nullptr, pv.data(), nullptr, gamma, nr.data(), 0, eps);
    if (normed_opt) std::memcpy(normed_opt + (size_t)b * H, nr.data(), (size_t)H * 2);
    for (int g = 0; g < H / 32; ++g)
      mxfp8_group(nr.data() + g * 32, q + (size_t)b * H + g * 32, sf + (size_t)b * (H / 32) + g);
  }
}

// ------------------------------------------------------------------ router
// kern_k3_router_topk (source/k3_router_argmax.cu:87-152).  K sequential picks of the
// largest biased score, ties to the smallest expert id; weights renormalised over the K
// unbiased scores with the xor-butterfly order of :143-147.  topk must be a power of two.
static inline uint32_t ord_f32(float f) {
  const uint32_t b = f32_bits(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

K3O_API void k3o_router_topk(const float* S, const float* bias, const u16* rs, int* idx, float* wts,
                             int B, int experts, int topk) {
  const float rsf = bf2f(rs[0]);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<float> sig(experts);
    std::vector<uint32_t> key(experts);
    for (int e = 0; e < experts; ++e) {
      sig[e] = det_sigmoid(S[(size_t)b * experts + e]);
      key[e] = ord_f32(sig[e] + bias[e]);
    }
    float w[32];
    int pick[32];
    for (int r = 0; r < topk; ++r) {
      uint32_t m = 0; int best = 0;
      for (int e = 0; e < experts; ++e)
        if (key[e] > m) { m = key[e]; best = e; }        // strict >: ties keep the smaller id
      pick[r] = best; w[r] = sig[best]; key[best] = 0u;
    }
    float den[32];
    for (int r = 0; r < topk; ++r) den[r] = w[r];
    const float d = butterfly(den, topk);
    for (int r = 0; r < topk; ++r) {
      wts[(size_t)b * topk + r] = (w[r] / (d + 1e-20f)) * rsf;
      idx[(size_t)b * topk + r] = pick[r];
    }
  }
}

// ------------------------------------------------------------------ MoE routing tables
// local_expert (source/k3_moe_prefill_v4.cu:100-109).
static inline int local_expert(int id, int rank, int E, int ep_ranks, int strided) {
  if (strided) {
    if (id % ep_ranks != rank) return -1;
    const int e = id / ep_ranks;
    return e < E ? e : -1;
  }
  const int e = id - rank * E;
  return (e >= 0 && e < E) ? e : -1;
}

// kern_k3_moe_route_count (source/k3_moe_prefill_v4.cu:142-157): per 256-token block.
K3O_API void k3o_moe_route_count(const int* ids, int T, int rank, int E, int topk, int ep_ranks,
                                 int strided, int* blockcount) {
  const int blocks = (T + 255) / 256;
  for (int b = 0; b < blocks; ++b) {
    int* cnt = blockcount + (size_t)b * E;
    std::fill(cnt, cnt + E, 0);
    for (int t = b * 256; t < std::min(T, b * 256 + 256); ++t)
      for (int k = 0; k < topk; ++k) {
        const int e = local_expert(ids[(size_t)t * topk + k], rank, E, ep_ranks, strided);
        if (e >= 0) ++cnt[e];
      }
  }
}

// kern_k3_moe_route_tables (source/k3_moe_prefill_v4.cu:159-203).
K3O_API void k3o_moe_route_tables(const int* blockcount, int blocks, int E, int tile, int* blockoff,
                                  int* cta_batch, int* cta_limit, int* num_non_exiting,
                                  int* total_padded, int* route_map) {
  std::vector<int> count(E, 0), off(E + 1, 0);
  for (int e = 0; e < E; ++e)
    for (int b = 0; b < blocks; ++b) count[e] += blockcount[(size_t)b * E + e];
  int run = 0;
  for (int e = 0; e < E; ++e) { off[e] = run; run += (count[e] + tile - 1) / tile; }
  off[E] = run;
  num_non_exiting[0] = run;
  total_padded[0] = run * tile;
  for (int e = 0; e < E; ++e) {
    int r = off[e] * tile;
    for (int b = 0; b < blocks; ++b) { blockoff[(size_t)b * E + e] = r; r += blockcount[(size_t)b * E + e]; }
    for (int p = off[e] * tile + count[e]; p < off[e + 1] * tile; ++p) route_map[p] = 0;
  }
  for (int i = 0; i < off[E]; ++i) {
    int j = 0;
    while (off[j + 1] <= i) ++j;
    cta_batch[i] = j;
    cta_limit[i] = std::min((i + 1) * tile, off[j] * tile + count[j]);
  }
}

// kern_k3_moe_route_scatter (source/k3_moe_prefill_v4.cu:205-252): within a 256-token
// block the rank of an expanded id among the block's ids of the same expert is its
// position in ascending expanded order -- a stable counting sort.
K3O_API void k3o_moe_route_scatter(const int* ids, const int* blockoff, int T, int rank, int E, int topk,
                                   int ep_ranks, int strided, int* route_map, int* exp2perm) {
  const int blocks = (T + 255) / 256;
  for (int b = 0; b < blocks; ++b) {
    std::vector<int> seen(E, 0);
    const long long lo = (long long)b * 256 * topk, hi = std::min((long long)T, (long long)b * 256 + 256) * topk;
    for (long long i = lo; i < hi; ++i) {
      const int e = local_expert(ids[i], rank, E, ep_ranks, strided);
      if (e < 0) { exp2perm[i] = -1; continue; }
      const int row = blockoff[(size_t)b * E + e] + seen[e]++;
      route_map[row] = (int)(i / topk);
      exp2perm[i] = row;
    }
  }
}

// kern_k3_moe_finalize (source/k3_moe_prefill_v4.cu:254-302): live slots in ascending k,
// acc = fma(w, x, acc) from 0, one bf16 rounding.
K3O_API void k3o_moe_finalize(const u16* fc2, const int* exp2perm, const float* wts, u16* out, int T,
                              int cols, int topk) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    for (int c = 0; c < cols; ++c) {
      float acc = 0.f;
      for (int k = 0; k < topk; ++k) {
        const int p = exp2perm[(size_t)t * topk + k];
        if (p >= 0) acc = std::fmaf(wts[(size_t)t * topk + k], bf2f(fc2[(size_t)p * cols + c]), acc);
      }
      out[(size_t)t * cols + c] = f2bf(acc);
    }
  }
}

// Config-level fusion: finalize (above) landed to bf16, then the one-partial residual
// add of kern_k3_land_add2 (source/k3_residual_v2.cu:349-392, two = 0).  Both roundings of
// the unfused pair are kept, so the fused result equals the composition bit for bit.
K3O_API void k3o_finalize_residual(const u16* fc2, const int* exp2perm, const float* wts,
                                   const u16* residual, u16* out, int T, int cols, int topk) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    for (int c = 0; c < cols; ++c) {
      float acc = 0.f;
      for (int k = 0; k < topk; ++k) {
        const int p = exp2perm[(size_t)t * topk + k];
        if (p >= 0) acc = std::fmaf(wts[(size_t)t * topk + k], bf2f(fc2[(size_t)p * cols + c]), acc);
      }
      const size_t o = (size_t)t * cols + c;
      out[o] = f2bf(bf2f(residual[o]) + land(acc));
    }
  }
}

// Config-level dispatch: gather of MXFP8 token rows into expert-sorted order,
// dst row r = src row route_map[r] for r < rows (the row gather the reference leaves to the
// grouped GEMM's TMA, which reads route_map: source/k3_moe_prefill_v4.cu:36-46).
K3O_API void k3o_permute_gather(const u8* q, const u8* sf, const int* route_map, long long rows, int cols,
                                u8* out_q, u8* out_sf) {
  const int sfc = cols / 32;
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    const long long t = route_map[r];
    std::memcpy(out_q + r * cols, q + t * cols, (size_t)cols);
    std::memcpy(out_sf + r * sfc, sf + t * sfc, (size_t)sfc);
  }
}

// ------------------------------------------------------------------ collectives
// Chain order of the reduce-scatter (source/k3_collectives.cu:222-236,
// source/k3_reducescatter_pull_nr4.cu:150-160): ownpos = order >> 1, descend = order & 1.
K3O_API void k3o_rs_sequence(int rank, int W, int order, int* seq) {
  const int ownpos = order >> 1, descend = order & 1;
  int pi = 0;
  for (int j = 0; j < W; ++j) {
    if (j == ownpos) { seq[j] = rank; continue; }
    const int off = descend ? (W - 1 - pi) : (1 + pi);
    seq[j] = (rank + off) % W;
    ++pi;
  }
}

// kern_k3_rs_pull (source/k3_reducescatter_pull_nr4.cu:124-186): partials[q] is rank q's
// full [W * count] buffer; the chunk this rank keeps starts at rank * count; one bf16
// rounding per hop after the first.
K3O_API void k3o_rs_pull(const u16* const* partials, u16* dst, long long count, int rank, int W, int order) {
  int seq[64];
  k3o_rs_sequence(rank, W, order, seq);
  const long long off = (long long)rank * count;
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < count; ++i) {
    float a = bf2f(partials[seq[0]][off + i]);
    for (int k = 1; k < W; ++k) a = land(a + bf2f(partials[seq[k]][off + i]));
    dst[i] = f2bf(a);
  }
}

// kern_k3_allgather4_push payload semantics (source/k3_allgather4_v3.cu:44-59): rank r's
// nbytes land at byte r * nbytes of every rank's destination.
K3O_API void k3o_allgather(const u8* const* srcs, u8* const* dsts, long long nbytes, int W) {
  for (int r = 0; r < W; ++r)
    for (int q = 0; q < W; ++q) std::memcpy(dsts[q] + (long long)r * nbytes, srcs[r], (size_t)nbytes);
}

// The epoch / arrival-counter barrier (source/k3_collectives.cu:23-35, :74-79;
// source/k3_rs_arrive_v2.cu:52-75) simulated with W host threads and atomic counters.
// Each rank: flags[0] += units once per replay (epoch), then per collective call
// flags[slot] += units and poll every peer's flags[slot] >= own flags[0].  absent_rank >= 0
// makes that rank never arrive; the waiters then give up after timeout_us and report.
// status[r] = 0 ok, else 1 + the first peer that never arrived.  Returns the number of
// ranks that timed out.
K3O_API int k3o_sim_barrier(int W, int slots, int replays, int units, int absent_rank, int timeout_us,
                            int* status) {
  std::vector<std::vector<std::atomic<unsigned long long>>> flags(W);
  for (auto& f : flags) { f = std::vector<std::atomic<unsigned long long>>(slots + 1); for (auto& x : f) x.store(0); }
  std::vector<std::thread> th;
  for (int r = 0; r < W; ++r) status[r] = 0;
  for (int r = 0; r < W; ++r) {
    if (r == absent_rank) continue;
    th.emplace_back([&, r] {
      for (int it = 0; it < replays && status[r] == 0; ++it) {
        flags[r][0].fetch_add((unsigned long long)units, std::memory_order_relaxed);
        const unsigned target = (unsigned)flags[r][0].load(std::memory_order_relaxed);
        for (int s = 1; s <= slots && status[r] == 0; ++s) {
          flags[r][s].fetch_add((unsigned long long)units, std::memory_order_release);
          const auto t0 = std::chrono::steady_clock::now();
          for (int q = 0; q < W; ++q) {
            while ((unsigned)flags[q][s].load(std::memory_order_acquire) < target) {
              if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(timeout_us)) {
                status[r] = 1 + q;
                break;
              }
              std::this_thread::yield();
            }
            if (status[r]) break;
          }
        }
      }
    });
  }
  for (auto& t : th) t.join();
  int bad = 0;
  for (int r = 0; r < W; ++r) bad += status[r] != 0;
  return bad;
}

// ------------------------------------------------------------------ MLA prep
// kern_k3_mla_prep_head (source/k3_mla_prep_v2.cu:130-211; bf16-partial form
// source/k3_mla_prep_bf16.cu).  Row of `fused` columns: q_a [0,1536) | kv_a [1536,2048) |
// rope [2048,2112) | gate band.  Sums of squares: unit = 4 consecutive columns, group = 32
// units, lane partial fma chain from 0, 32-lane butterfly, groups summed ascending.
static float mla_group_sum(const float* x /* 128 landed values */) {
  float lanes[32];
  for (int l = 0; l < 32; ++l) {
    float p = 0.f;
    for (int j = 0; j < 4; ++j) p = std::fmaf(x[4 * l + j], x[4 * l + j], p);
    lanes[l] = p;
  }
  return butterfly(lanes, 32);
}

K3O_API void k3o_mla_prep_head(const void* partial, int partial_is_bf16, int fused, const u16* gamma_q,
                               const u16* gamma_kv, const long long* slot_mapping, u16* slab,
                               long long layer_off, long long page_stride, u16* q_norm, int B, float eps) {
  const int QL = 1536, KVL = 512, ROPE = 64, KVA = KVL + ROPE;
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<float> x(QL + KVL + ROPE);
    for (int c = 0; c < QL + KVL + ROPE; ++c) {
      const size_t o = (size_t)b * fused + c;
      x[c] = partial_is_bf16 ? bf2f(((const u16*)partial)[o]) : land(((const float*)partial)[o]);
    }
    float tq = 0.f, tk = 0.f;
    for (int g = 0; g < 12; ++g) tq += mla_group_sum(&x[128 * g]);
    for (int g = 0; g < 4; ++g) tk += mla_group_sum(&x[QL + 128 * g]);
    const float scq = rsqrt_rn(std::fmaf(tq, 1.f / 1536.f, eps));
    const float sck = rsqrt_rn(std::fmaf(tk, 1.f / 512.f, eps));
    for (int c = 0; c < QL; ++c) q_norm[(size_t)b * QL + c] = bfmul(f2bf(x[c] * scq), gamma_q[c]);
    const long long slot = slot_mapping[b];
    if (slot < 0) continue;
    u16* rowp = slab + (slot / 64) * page_stride + layer_off + (slot % 64) * KVA;
    for (int c = 0; c < KVL; ++c) rowp[c] = bfmul(f2bf(x[QL + c] * sck), gamma_kv[c]);
    for (int c = 0; c < ROPE; ++c) rowp[KVL + c] = f2bf(x[QL + KVL + c]);
  }
}

// kern_k3_mla_prep_gate (source/k3_mla_prep_v2.cu:91-118).
K3O_API void k3o_mla_prep_gate(const void* partial, int partial_is_bf16, int fused, int inner, u16* mla_gate,
                               int B) {
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < inner; ++c) {
      const size_t o = (size_t)b * fused + 2112 + c;
      mla_gate[(size_t)b * inner + c] = partial_is_bf16 ? ((const u16*)partial)[o] : f2bf(((const float*)partial)[o]);
    }
}

// Config-level MLA prep with RoPE and packing.  The reference applies no rotation in its
// prep kernel (source/k3_mla_prep_v2.cu lands the rope slice unrotated) and only ships a
// table builder (source/weight_prep.cu:34-45: inv_j = 1 / base^(2j / (2 half)),
// angle = pos * inv_j, cos/sin stored as bf16).  This op fixes the convention: the caller
// supplies that bf16 table [T, 64] = cos(32) | sin(32); pairing is half-split
// (x1 = slice[0:32], x2 = slice[32:64]): o1 = bf16(fma(-x2, sin, x1 * cos)),
// o2 = bf16(fma(x1, sin, x2 * cos)).  kv [T, 576] = latent(512) | k_rope(64);
// q [T, heads, 192] = nope(128) | rope(64).  Outputs: q_out (nope copied, rope rotated),
// k_out [T, heads, 192] rope slots = rotated k_rope broadcast to every head (nope slots are
// the up-projection GEMM's and are not touched), latent_out [T, 512] = RMSNorm(latent) with
// the reduction order of the kv groups of kern_k3_mla_prep_head.
K3O_API void k3o_mla_prep_rope_pack(const u16* kv, const u16* q, const u16* gamma_kv, const u16* rope_tab,
                                    u16* q_out, u16* k_out, u16* latent_out, int T, int heads, float eps) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float x[512];
    for (int c = 0; c < 512; ++c) x[c] = bf2f(kv[(size_t)t * 576 + c]);
    float tk = 0.f;
    for (int g = 0; g < 4; ++g) tk += mla_group_sum(&x[128 * g]);
    const float sck = rsqrt_rn(std::fmaf(tk, 1.f / 512.f, eps));
    for (int c = 0; c < 512; ++c) latent_out[(size_t)t * 512 + c] = bfmul(f2bf(x[c] * sck), gamma_kv[c]);
    const u16* tab = rope_tab + (size_t)t * 64;
    auto rot = [&](const u16* in, u16* out) {
      for (int j = 0; j < 32; ++j) {
        const float c = bf2f(tab[j]), s = bf2f(tab[32 + j]);
        const float x1 = bf2f(in[j]), x2 = bf2f(in[32 + j]);
        out[j] = f2bf(std::fmaf(-x2, s, x1 * c));
        out[32 + j] = f2bf(std::fmaf(x1, s, x2 * c));
      }
    };
    u16 kr[64];
    rot(kv + (size_t)t * 576 + 512, kr);
    for (int h = 0; h < heads; ++h) {
      const size_t o = ((size_t)t * heads + h) * 192;
      std::memcpy(q_out + o, q + o, 128 * 2);
      rot(q + o + 128, q_out + o + 128);
      std::memcpy(k_out + o + 128, kr, 64 * 2);
    }
  }
}

// ------------------------------------------------------------------ KDA span conv + SiLU
// kern_k3_span_gather (source/k3_span_gather_v3.cu:251-293; row math :131-142; window
// :236-248).  Streams s in {q, k, v}; input row i column c of stream s = partial[(at + i) *
// row_stride + s * inner + c]; x_{i<0} comes from the 3-row window; taps cw[s][t][c] (f32, or
// bf16 when taps_bf16).  y = fma(x_i, w3, fma(x_{i-1}, w2, fma(x_{i-3}, w0, x_{i-2} * w1))) -- the
// contraction the reference build produces for `t0*w0 + t1*w1 + t2*w2 + x*w3` (:134), established
// against the reference kernel's own outputs (tests/golden);
// sb = bf16(y); out = bf16(sb * sigmoid(sb)); new window = the last three inputs.
K3O_API void k3o_span_conv_silu(const u16* partial, long long row_stride, const void* cw, int taps_bf16,
                                u16* win /* [3][3][inner] */, u16* out_q, u16* out_k, u16* out_v, int inner,
                                int at, int span) {
  u16* outs[3] = {out_q, out_k, out_v};
  for (int s = 0; s < 3; ++s) {
    u16* w = win + (size_t)s * 3 * inner;
    std::vector<u16> old(w, w + (size_t)3 * inner);
    auto xin = [&](int i, int c) -> float {
      return i < 0 ? bf2f(old[(size_t)(i + 3) * inner + c])
                   : bf2f(partial[(size_t)(at + i) * row_stride + (size_t)s * inner + c]);
    };
    auto tap = [&](int t, int c) -> float {
      const size_t o = ((size_t)s * 4 + t) * inner + c;
      return taps_bf16 ? bf2f(((const u16*)cw)[o]) : ((const float*)cw)[o];
    };
#pragma omp parallel for schedule(static)
    for (int i = 0; i < span; ++i)
      for (int c = 0; c < inner; ++c) {
        float y = xin(i - 2, c) * tap(1, c);             // nvcc contracts t0*w0 + t1*w1 as fma(t0, w0, t1*w1)
        y = std::fmaf(xin(i - 3, c), tap(0, c), y);
        y = std::fmaf(xin(i - 1, c), tap(2, c), y);
        y = std::fmaf(xin(i, c), tap(3, c), y);
        const float sb = land(y);
        const double sg = 1.0 / (1.0 + std::exp(-(double)sb));
        outs[s][(size_t)i * inner + c] = f2bf((float)((double)sb * sg));
      }
    for (int t = 0; t < 3; ++t)
      for (int c = 0; c < inner; ++c) w[(size_t)t * inner + c] = f2bf(xin(span - 3 + t, c));
  }
}

// beta transpose and flow landing of the y == 3 blocks (source/k3_span_gather_v3.cu:267-282).
K3O_API void k3o_span_beta_flow(const float* wsm_partial, int heads, u16* span_beta, u16* span_flow, int at,
                                int span) {
  for (int i = 0; i < span; ++i) {
    const float* row = wsm_partial + (size_t)(at + i) * 256;
    for (int h = 0; h < heads; ++h) span_beta[(size_t)h * span + i] = f2bf(row[h]);
    for (int c = 0; c < 128; ++c) span_flow[(size_t)i * 128 + c] = f2bf(row[96 + c]);
  }
}

// ------------------------------------------------------------------ KDA output gate
// kern_k3_kda_out_gate (source/k3_kda_out_gate_v3.cu:36-118).  Per (row, head): lane owns 8
// consecutive d, ss = fma chain from 0, butterfly over the head's 16 lanes,
// r = rsqrt(fma(ss, 1/128, eps)); o = bf16((a * r) * gamma_o[d]); gt = bf16(sigmoid(g));
// gated = bf16(f32(o) * f32(gt)).  gate element = gate[(at + i) * gate_stride + gate_off + col].
// When q/sf are non-null the gated row is also MXFP8-quantised (config-level epilogue,
// formula of source/k3_moe_prefill_v4.cu:111-140; a 32-group never straddles a head).
K3O_API void k3o_kda_out_gate(const u16* attn, const u16* gate, long long gate_stride, long long gate_off,
                              const float* gamma_o, u16* gated, u8* q, u8* sf, int heads, int at, int span,
                              float eps) {
  const int inner = heads * 128;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < span; ++i) {
    const size_t b = (size_t)(at + i);
    std::vector<u16> row(inner);
    for (int h = 0; h < heads; ++h) {
      const u16* a = attn + (size_t)i * inner + (size_t)h * 128;
      float lanes[16];
      for (int l = 0; l < 16; ++l) {
        float ss = 0.f;
        for (int k = 0; k < 8; ++k) { const float v = bf2f(a[8 * l + k]); ss = std::fmaf(v, v, ss); }
        lanes[l] = ss;
      }
      const float r = rsqrt_rn(std::fmaf(butterfly(lanes, 16), 1.0f / 128.0f, eps));
      for (int d = 0; d < 128; ++d) {
        const u16 o = f2bf((bf2f(a[d]) * r) * gamma_o[d]);
        const float g = bf2f(gate[b * gate_stride + gate_off + (size_t)h * 128 + d]);
        const u16 gt = f2bf((float)(1.0 / (1.0 + std::exp(-(double)g))));
        row[(size_t)h * 128 + d] = bfmul(o, gt);
      }
    }
    if (gated) std::memcpy(gated + b * inner, row.data(), (size_t)inner * 2);
    if (q && sf)
      for (int g = 0; g < inner / 32; ++g)
        mxfp8_group(row.data() + g * 32, q + b * inner + g * 32, sf + b * (inner / 32) + g);
  }
}

// ------------------------------------------------------------------ remaining glue
// kern_k3_situ_rms_bf16 (source/k3_land_fused.cu:123-202).  situ: (4 tanh(g/4) * sigmoid(g)) * 25 tanh(u/25)
// with one bf16 landing (the device uses tanh.approx / ex2.approx: bf16 tolerance).  rms: per 16-byte vector
// an fma chain over its 8 elements, butterfly over each group of 32 consecutive vectors, butterfly over the
// 32 group slots (:76-92, :146-160), rs = rsqrt(sum / h + 1e-5), ln = bf16(x * rs) (x) gamma.
K3O_API void k3o_situ_rms(const u16* sp, u16* act, const u16* lat, const u16* gam, u16* ln, int n, int B, int h, int L) {
#pragma omp parallel for schedule(static)
  for (int row = 0; row < B; ++row)
    for (int i = 0; i < n; ++i) {
      const double g = bf2f(sp[(size_t)row * 2 * n + i]), u = bf2f(sp[(size_t)row * 2 * n + n + i]);
      const double a = 4.0 * std::tanh(g * 0.25), s = 1.0 / (1.0 + std::exp(-g)), c = 25.0 * std::tanh(u * 0.04);
      act[(size_t)row * n + i] = f2bf((float)((a * s) * c));
    }
  const int nvec = h / 8;
#pragma omp parallel for schedule(static)
  for (int row = 0; row < L; ++row) {
    const u16* x = lat + (size_t)row * h;
    float slots[32];
    for (int g = 0; g < 32; ++g) {
      float lanes[32];
      for (int l = 0; l < 32; ++l) {
        const int v = 32 * g + l;
        float p = 0.f;
        if (v < nvec)
          for (int k = 0; k < 8; ++k) { const float f = bf2f(x[8 * v + k]); p = std::fmaf(f, f, p); }
        lanes[l] = p;
      }
      slots[g] = butterfly(lanes, 32);
    }
    const float rs = rsqrt_rn(butterfly(slots, 32) / (float)h + 1e-5f);
    for (int i = 0; i < h; ++i) ln[(size_t)row * h + i] = bfmul(f2bf(bf2f(x[i]) * rs), gam[i]);
  }
}

// kern_sigmoid_mul_bf16 (source/sigmoid_mul.cu:15-44): g = bf16(sigmoid(gate)), out = bf16(attn * g).
K3O_API void k3o_sigmoid_mul(u16* out, const u16* attn, const u16* gate, int tokens, int heads, int head_dim, int gate_tstride,
                             int gate_hstride) {
  const int n = heads * head_dim;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < tokens; ++t)
    for (int j = 0; j < n; ++j) {
      const int hh = j / head_dim, d = j % head_dim;
      const double x = bf2f(gate[(size_t)t * gate_tstride + (size_t)hh * gate_hstride + d]);
      const u16 g = f2bf((float)(1.0 / (1.0 + std::exp(-x))));
      out[(size_t)t * n + j] = bfmul(attn[(size_t)t * n + j], g);
    }
}

K3O_API int k3o_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
