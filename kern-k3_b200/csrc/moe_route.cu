// MoE routing tables, dispatch gather and top-k combine around the grouped expert GEMMs.
//
// Replaces, behind the same entry names and parameter lists, the routing kernels of
// xiaguan/kern-k3 source/k3_moe_prefill_v4.cu:
//   kern_k3_moe_route_count    (:142-157)  per-256-token-block histogram of the local experts
//   kern_k3_moe_route_tables   (:159-203)  tile-padded expert offsets, per-block offsets, CTA work list
//   kern_k3_moe_route_scatter  (:205-252)  stable expert-sorted permutation (route_map, exp2perm)
//   kern_k3_moe_finalize       (:254-302)  out[t] = bf16(sum_k w[t,k] * fc2[exp2perm[t,k]])
// and adds two config-level kernels the reference leaves to other launches:
//   permute_gather     rows of MXFP8 codes + scales copied into expert-sorted order (the reference's
//                      grouped GEMM gathers rows itself through route_map)
//   finalize_residual  finalize fused with the one-partial residual add of kern_k3_land_add2
//                      (source/k3_residual_v2.cu:349-392), keeping both bf16 landings.
//
// All tables are integer-only and deterministic: the rank of an expanded id (t, k) among the ids
// of the same expert inside its 256-token block is its position in ascending (t, k) order (a
// stable counting sort), computed from warp match masks plus a scan over the block's 32-id groups.
#include "k3g_device.cuh"
#include "k3g_host.h"

#include <atomic>

using namespace k3g;

namespace {

constexpr int kMaxE = 64;          // local experts per rank of the drop-in kernels (224 / 4 = 56 in the reference deployment)
constexpr int kMaxEWide = 256;     // C-ABI kernels for expert-parallel groups of 1 or 2 (224 / 112 local experts)
constexpr int kRouteBlock = 256;   // tokens per routing block
constexpr int kMaxTopk = 16;
constexpr int kMaxGroups = kRouteBlock * kMaxTopk / 32;   // 128 groups of 32 expanded ids

// rank >= 0: the slot of expert `id` among rank's E local experts, or -1 (source/k3_moe_prefill_v4.cu:100-109).
// rank < 0 (C ABI only): every owner's experts at once, in owner-major order -- E is then the total expert count,
// owner o holds E / ep_ranks of them and its slots are o * (E / ep_ranks) + its local slot, so the tables of the
// ep_ranks owners come out of one pass, stacked, each equal to that owner's own table shifted by a constant row.
__device__ __forceinline__ int local_expert(int id, int rank, int E, int ep_ranks, int strided) {
  if (rank < 0) {
    if (id < 0 || id >= E) return -1;
    return strided ? (id % ep_ranks) * (E / ep_ranks) + id / ep_ranks : id;
  }
  if (strided) {
    if (id % ep_ranks != rank) return -1;
    const int e = id / ep_ranks;
    return e < E ? e : -1;
  }
  const int e = id - rank * E;
  return (e >= 0 && e < E) ? e : -1;
}

template <int MAXE = kMaxE>
__device__ __forceinline__ void route_count_body(const int* __restrict__ ids, int T, int rank, int E, int topk, int ep_ranks,
                                                 int strided, int* __restrict__ blockcount) {
  __shared__ int cnt[MAXE];
  for (int b = blockIdx.x; b * kRouteBlock < T; b += gridDim.x) {
    if (threadIdx.x < E) cnt[threadIdx.x] = 0;
    __syncthreads();
    const long long lo = (long long)b * kRouteBlock * topk;
    const long long hi = min((long long)T, (long long)(b + 1) * kRouteBlock) * topk;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const int e = local_expert(ids[i], rank, E, ep_ranks, strided);
      if (e >= 0) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x < E) blockcount[(size_t)b * E + threadIdx.x] = cnt[threadIdx.x];
    __syncthreads();
  }
}

template <int MAXE = kMaxE>
__device__ __forceinline__ void route_tables_body(const int* __restrict__ blockcount, int blocks, int E, int tile,
                                                  int* __restrict__ blockoff, int* __restrict__ cta_batch, int* __restrict__ cta_limit,
                                                  int* __restrict__ num_non_exiting, int* __restrict__ total_padded,
                                                  int* __restrict__ route_map) {
  __shared__ int count[MAXE], off[MAXE + 1];
  // count[e]: one warp per expert, lanes over blocks (integer sums: order-free)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int run = 0;
    for (int b = lane; b < blocks; b += 32) run += blockcount[(size_t)b * E + e];
    run = __reduce_add_sync(0xffffffffu, run);
    if (lane == 0) count[e] = run;
  }
  __syncthreads();
  if (warp == 0) {   // exclusive scan of ceil(count / tile) over up to MAXE experts: MAXE / 32 consecutive experts per lane
    constexpr int PER = MAXE / 32;
    int c[PER], mine = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = PER * lane + j;
      c[j] = e < E ? (count[e] + tile - 1) / tile : 0;
      mine += c[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - mine;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = PER * lane + j;
      if (e < E) off[e] = run;
      run += c[j];
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) {
      off[E] = total;
      num_non_exiting[0] = total;
      total_padded[0] = total * tile;
    }
  }
  __syncthreads();
  // blockoff[b][e] = tile * off[e] + (count of e in blocks before b): warp per expert, chunked scan
  for (int e = warp; e < E; e += nwarps) {
    int run = off[e] * tile;
    for (int b0 = 0; b0 < blocks; b0 += 32) {
      const int b = b0 + lane;
      const int c = b < blocks ? blockcount[(size_t)b * E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (b < blocks) blockoff[(size_t)b * E + e] = run + incl - c;
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
    // padding rows of the expert's last tile route token 0
    for (int r = off[e] * tile + count[e] + lane; r < off[e + 1] * tile; r += 32) route_map[r] = 0;
  }
  for (int i = threadIdx.x; i < off[E]; i += blockDim.x) {
    int lo = 0, hi = E;     // largest j with off[j] <= i and off[j + 1] > i
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (off[mid] <= i) lo = mid; else hi = mid; }
    while (off[lo + 1] <= i) ++lo;   // skip experts with no tiles
    cta_batch[i] = lo;
    cta_limit[i] = min((i + 1) * tile, off[lo] * tile + count[lo]);
  }
}

// Shared-memory tables of one scatter block when the tables launch is folded into it.
template <int MAXE>
struct TablesInBlock {
  int count[MAXE];       // tokens per expert over all blocks
  int pre[MAXE];         // ... over the blocks before this one
  int off[MAXE + 1];     // exclusive scan of ceil(count / tile)
  int boff[MAXE];        // this block's row of blockoff
};

// What kern_k3_moe_route_tables computes, restricted to what block `blk` of the scatter needs (its row of
// blockoff), with block 0 also producing the outputs that do not depend on the block: the CTA work list, the
// two scalars and the padding rows of route_map.  Every value equals the stand-alone tables kernel's.
template <int MAXE>
__device__ __forceinline__ void block_tables(TablesInBlock<MAXE>& tb, const int* __restrict__ blockcount, int blocks, int blk, int E,
                                             int tile, int* __restrict__ blockoff, int* __restrict__ cta_batch, int* __restrict__ cta_limit,
                                             int* __restrict__ num_non_exiting, int* __restrict__ total_padded,
                                             int* __restrict__ route_map) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Column sums of blockcount over all blocks (count) and over the blocks before this one (pre).  The block's
  // threads are dealt out as `parts` threads per expert, part p taking the rows p, p + parts, ...: adjacent threads
  // read adjacent experts of one row (coalesced), a thread's loads are independent and issued eight at a time, and the
  // parts meet in shared-memory integer adds (order-free, so the sums are the stand-alone kernel's).
  for (int e = threadIdx.x; e < E; e += blockDim.x) { tb.count[e] = 0; tb.pre[e] = 0; }
  __syncthreads();
  {
    const int parts = max(1, min((int)blockDim.x / E, 16));
    const int e = threadIdx.x % E, part = threadIdx.x / E;
    if (part < parts) {
      int tot = 0, pre = 0;
#pragma unroll 8
      for (int b = part; b < blocks; b += parts) {
        const int c = blockcount[(size_t)b * E + e];
        pre += b < blk ? c : 0;
        tot += c;
      }
      atomicAdd(&tb.count[e], tot);
      atomicAdd(&tb.pre[e], pre);
    }
    if (E > (int)blockDim.x) {                            // more experts than threads: the rest, one thread each
      for (int e2 = threadIdx.x + blockDim.x; e2 < E; e2 += blockDim.x) {
        int tot = 0, pre = 0;
        for (int b = 0; b < blocks; ++b) {
          const int c = blockcount[(size_t)b * E + e2];
          pre += b < blk ? c : 0;
          tot += c;
        }
        tb.count[e2] = tot; tb.pre[e2] = pre;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    constexpr int PER = MAXE / 32;
    int c[PER], mine = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = PER * lane + j;
      c[j] = e < E ? (tb.count[e] + tile - 1) / tile : 0;
      mine += c[j];
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - mine;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = PER * lane + j;
      if (e < E) tb.off[e] = run;
      run += c[j];
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (lane == 0) {
      tb.off[E] = total;
      if (blk == 0) { num_non_exiting[0] = total; total_padded[0] = total * tile; }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int v = tb.off[e] * tile + tb.pre[e];
    tb.boff[e] = v;
    blockoff[(size_t)blk * E + e] = v;
  }
  if (blk == 0) {
    const int nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps)              // padding rows of the expert's last tile route token 0
      for (int r = tb.off[e] * tile + tb.count[e] + lane; r < tb.off[e + 1] * tile; r += 32) route_map[r] = 0;
    for (int i = threadIdx.x; i < tb.off[E]; i += blockDim.x) {
      int lo = 0, hi = E;
      while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (tb.off[mid] <= i) lo = mid; else hi = mid; }
      while (tb.off[lo + 1] <= i) ++lo;
      cta_batch[i] = lo;
      cta_limit[i] = min((i + 1) * tile, tb.off[lo] * tile + tb.count[lo]);
    }
  }
  __syncthreads();
}

// hist: kMaxGroups x MAXE counters in shared memory (a count is at most 32 and a running offset at most 4096, so 16 bits do).
template <int MAXE, typename HistT>
__device__ __forceinline__ void route_scatter_body(const int* __restrict__ ids, const int* __restrict__ blockoff, int T, int rank,
                                                   int E, int topk, int ep_ranks, int strided, int* __restrict__ route_map,
                                                   int* __restrict__ exp2perm, HistT (*hist)[MAXE], TablesInBlock<MAXE>* tb = nullptr,
                                                   const int* __restrict__ blockcount = nullptr, int tile = 0, int* blockoff_out = nullptr,
                                                   int* cta_batch = nullptr, int* cta_limit = nullptr, int* num_non_exiting = nullptr,
                                                   int* total_padded = nullptr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const unsigned below = (1u << lane) - 1u;
  const int groups = kRouteBlock * topk / 32;
  const int nblocks = (T + kRouteBlock - 1) / kRouteBlock;
  for (int blk = blockIdx.x; blk * kRouteBlock < T; blk += gridDim.x) {
    if (tb != nullptr) {
      // the tables launch folded in: this block derives its own row of block offsets from the per-block counts
      // (and block 0 also writes the work list and the padding rows), so nothing waits on a one-block kernel
      block_tables<MAXE>(*tb, blockcount, nblocks, blk, E, tile, blockoff_out, cta_batch, cta_limit, num_non_exiting, total_padded, route_map);
    }
    const int* boff_row = tb != nullptr ? tb->boff : blockoff + (size_t)blk * E;
    const long long base = (long long)blk * kRouteBlock * topk;
    const long long end = (long long)T * topk;
    for (int i = threadIdx.x; i < groups * MAXE; i += blockDim.x) (&hist[0][0])[i] = 0;
    __syncthreads();
    for (int g = warp; g < groups; g += nwarps) {
      const long long i = base + g * 32 + lane;
      int e = -1;
      if (i < end) e = local_expert(ids[i], rank, E, ep_ranks, strided);
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && (peers & below) == 0) hist[g][e] = (HistT)__popc(peers);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int run = 0;
      for (int g = 0; g < groups; ++g) { const int c = hist[g][e]; hist[g][e] = (HistT)run; run += c; }
    }
    __syncthreads();
    for (int g = warp; g < groups; g += nwarps) {
      const long long i = base + g * 32 + lane;
      int e = -1;
      if (i < end) e = local_expert(ids[i], rank, E, ep_ranks, strided);
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (i >= end) continue;
      if (e < 0) { exp2perm[i] = -1; continue; }
      const int row = boff_row[e] + hist[g][e] + __popc(peers & below);
      route_map[row] = (int)(i / topk);
      exp2perm[i] = row;
    }
    __syncthreads();
  }
}

// Combine: one token per 128-thread team pass; live (row, weight) pairs compacted in ascending k.
template <bool RESIDUAL>
__device__ __forceinline__ void finalize_body(const __nv_bfloat16* __restrict__ fc2, const int* __restrict__ exp2perm,
                                              const float* __restrict__ wts, const __nv_bfloat16* __restrict__ residual,
                                              __nv_bfloat16* __restrict__ out, int T, int cols, int topk) {
  __shared__ int s_row[2][kMaxTopk];
  __shared__ float s_w[2][kMaxTopk];
  __shared__ int s_n[2];
  const int nvec = cols >> 3;
  int it = 0;
  for (int t = blockIdx.x; t < T; t += gridDim.x, ++it) {
    const int buf = it & 1;
    if (threadIdx.x < 32) {
      const int k = threadIdx.x;
      const int p = k < topk ? exp2perm[(size_t)t * topk + k] : -1;
      const unsigned live = __ballot_sync(0xffffffffu, p >= 0);
      if (p >= 0) {
        const int pos = __popc(live & ((1u << k) - 1u));
        s_row[buf][pos] = p;
        s_w[buf][pos] = wts[(size_t)t * topk + k];
      }
      if (k == 0) s_n[buf] = __popc(live);
    }
    __syncthreads();
    const int n = s_n[buf];
    // two 16-byte column vectors per thread at a time, rows in chunks of four: eight loads in flight
    for (int v0 = threadIdx.x; v0 < nvec; v0 += 2 * blockDim.x) {
      const int v1 = v0 + blockDim.x;
      const bool two = v1 < nvec;
      float acc0[8], acc1[8];
#pragma unroll
      for (int l = 0; l < 8; ++l) { acc0[l] = 0.f; acc1[l] = 0.f; }
      for (int i = 0; i < n; i += 4) {
        V8 x0[4], x1[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (i + u < n) {
            const __nv_bfloat16* rowp = fc2 + (size_t)s_row[buf][i + u] * cols;
            x0[u] = ld_stream(rowp + v0 * 8);
            if (two) x1[u] = ld_stream(rowp + v1 * 8);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (i + u < n) {
            const float w = s_w[buf][i + u];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc0[2 * j] = __fmaf_rn(w, bf_lo(x0[u].w[j]), acc0[2 * j]);
              acc0[2 * j + 1] = __fmaf_rn(w, bf_hi(x0[u].w[j]), acc0[2 * j + 1]);
              if (two) {
                acc1[2 * j] = __fmaf_rn(w, bf_lo(x1[u].w[j]), acc1[2 * j]);
                acc1[2 * j + 1] = __fmaf_rn(w, bf_hi(x1[u].w[j]), acc1[2 * j + 1]);
              }
            }
          }
        }
      }
      V8 o0, o1;
#pragma unroll
      for (int j = 0; j < 4; ++j) { o0.w[j] = pack_bf2(acc0[2 * j], acc0[2 * j + 1]); o1.w[j] = pack_bf2(acc1[2 * j], acc1[2 * j + 1]); }
      if (RESIDUAL) {
        const V8 r0 = ld_stream(residual + (size_t)t * cols + v0 * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) o0.w[j] = add_bf2(r0.w[j], o0.w[j]);
        if (two) {
          const V8 r1 = ld_stream(residual + (size_t)t * cols + v1 * 8);
#pragma unroll
          for (int j = 0; j < 4; ++j) o1.w[j] = add_bf2(r1.w[j], o1.w[j]);
        }
      }
      st_stream(out + (size_t)t * cols + v0 * 8, o0);
      if (two) st_stream(out + (size_t)t * cols + v1 * 8, o1);
    }
  }
}

// dst row r = src row route_map[r]: `cols` code bytes and cols / 32 scale bytes per row.
// One WARP per destination row, rows walked with a warp stride, the token id of the next row fetched one row ahead.
// A lane moves VB = 32 bytes per access where rows allow it (sm_100's 256-bit ld / st: measured on this part, a
// store-only stream reaches 7.1 TB/s with 32-byte stores against 6.8 TB/s with 16-byte ones, and this kernel writes
// eight bytes for every byte it reads from HBM) and issues up to eight loads -- a whole 7168-byte row -- before its
// first store.  The scale bytes ride as 16-byte vectors.
template <int VB>
__global__ void __launch_bounds__(256) permute_gather_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                                             const int* __restrict__ route_map, long long rows, int cols,
                                                             uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf) {
  using Vec = typename VecOf<VB>::type;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int qv = cols / VB, sfb = cols >> 5;
  const bool sf_vec = (sfb & 15) == 0;
  long long r = warp;
  long long t = r < rows ? route_map[r] : 0;
  while (r < rows) {
    const long long rn = r + nwarps;
    const long long tn = rn < rows ? route_map[rn] : 0;
    const uint8_t* src = q + t * cols;
    uint8_t* dst = out_q + r * cols;
    for (int v0 = lane; v0 < qv; v0 += 8 * 32) {
      Vec x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (v0 + 32 * u < qv) x[u] = ld_keep_vec<VB>(src + (size_t)(v0 + 32 * u) * VB);      // a token row is read once per expert it routes to: keep it cached
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (v0 + 32 * u < qv) st_stream_vec<VB>(dst + (size_t)(v0 + 32 * u) * VB, x[u]);
    }
    if (sf_vec) {
      if (lane < (sfb >> 4)) __stcs(reinterpret_cast<uint4*>(out_sf + r * sfb) + lane, __ldg(reinterpret_cast<const uint4*>(sf + t * sfb) + lane));
    } else {
      for (int b = lane; b < sfb; b += 32) out_sf[r * sfb + b] = sf[t * sfb + b];
    }
    r = rn; t = tn;
  }
}

template <int MAXE>
__global__ void __launch_bounds__(256) route_count_kernel(const int* ids, int T, int rank, int E, int topk, int ep_ranks,
                                                          int strided, int* blockcount) {
  route_count_body<MAXE>(ids, T, rank, E, topk, ep_ranks, strided, blockcount);
}
template <int MAXE>
__global__ void __launch_bounds__(1024) route_tables_kernel(const int* blockcount, int blocks, int E, int tile, int* blockoff,
                                                            int* cta_batch, int* cta_limit, int* nne, int* total, int* route_map) {
  route_tables_body<MAXE>(blockcount, blocks, E, tile, blockoff, cta_batch, cta_limit, nne, total, route_map);
}
__global__ void __launch_bounds__(512) route_scatter_kernel(const int* ids, const int* blockoff, int T, int rank, int E, int topk,
                                                            int ep_ranks, int strided, int* route_map, int* exp2perm) {
  __shared__ int hist[kMaxGroups][kMaxE];
  route_scatter_body<kMaxE, int>(ids, blockoff, T, rank, E, topk, ep_ranks, strided, route_map, exp2perm, hist);
}
// up to 256 local experts: 16-bit counters in 64 KB of dynamic shared memory (opt-in above 48 KB)
__global__ void __launch_bounds__(512) route_scatter_wide_kernel(const int* ids, const int* blockoff, int T, int rank, int E, int topk,
                                                                 int ep_ranks, int strided, int* route_map, int* exp2perm) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  route_scatter_body<kMaxEWide, unsigned short>(ids, blockoff, T, rank, E, topk, ep_ranks, strided, route_map, exp2perm,
                                                reinterpret_cast<unsigned short(*)[kMaxEWide]>(dyn_smem));
}
// tables + scatter in one launch (the per-block counts come from route_count_kernel)
__global__ void __launch_bounds__(512) route_tables_scatter_kernel(const int* ids, const int* blockcount, int T, int rank, int E, int topk,
                                                                   int ep_ranks, int strided, int tile, int* blockoff, int* cta_batch,
                                                                   int* cta_limit, int* nne, int* total, int* route_map, int* exp2perm) {
  __shared__ int hist[kMaxGroups][kMaxE];
  __shared__ TablesInBlock<kMaxE> tb;
  route_scatter_body<kMaxE, int>(ids, nullptr, T, rank, E, topk, ep_ranks, strided, route_map, exp2perm, hist, &tb, blockcount, tile, blockoff,
                                 cta_batch, cta_limit, nne, total);
}
__global__ void __launch_bounds__(512) route_tables_scatter_wide_kernel(const int* ids, const int* blockcount, int T, int rank, int E, int topk,
                                                                        int ep_ranks, int strided, int tile, int* blockoff, int* cta_batch,
                                                                        int* cta_limit, int* nne, int* total, int* route_map, int* exp2perm) {
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  __shared__ TablesInBlock<kMaxEWide> tb;
  route_scatter_body<kMaxEWide, unsigned short>(ids, nullptr, T, rank, E, topk, ep_ranks, strided, route_map, exp2perm,
                                                reinterpret_cast<unsigned short(*)[kMaxEWide]>(dyn_smem), &tb, blockcount, tile, blockoff,
                                                cta_batch, cta_limit, nne, total);
}

// Dispatch to the owning ranks (benchmark configuration 2): the MXFP8 row of every token of this rank's shard is
// stored, once per expert it routes to, straight into the expert-sorted buffer of the rank that owns the expert
// -- a peer address over NVLink, or this rank's own buffer.  One warp per token: the row (cols code bytes and
// cols / 32 scale bytes) is read from HBM once, eight vectors of VB = 32 (or 16) bytes per lane at a time, and each
// chunk is stored to the token's topk destination rows, 1 KB (512 B) contiguous per warp instruction; the scale
// bytes leave as 16-byte stores.  Destination of slot k: owner = rank that holds expert ids[t, k]; row = exp2perm[t, k] of
// the all-owner tables minus the owner's first row (blockoff[owner * per], block 0 of the offsets table).
// Plain stores only: no TMA, no multicast, nothing waits.  The caller follows with a barrier (k3g_rs_arrive).
#ifndef K3G_DISPATCH_MINB
#define K3G_DISPATCH_MINB 2
#endif
#ifndef K3G_DISPATCH_VPL
#define K3G_DISPATCH_VPL 8      /* vectors in flight per lane */
#endif
template <int VB>
__device__ __forceinline__ void permute_dispatch_body(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                                      const int* __restrict__ ids, const int* __restrict__ exp2perm, int B,
                                                      long long token_begin, int topk, int cols, int per, int ep_ranks, int strided,
                                                      unsigned long long my_q, unsigned long long my_sf, int my_base) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  using Vec = typename VecOf<VB>::type;
  const int qv = cols / VB, sfb = cols >> 5;
  const bool sf_vec = (sfb & 15) == 0;
  for (long long b = warp; b < B; b += nwarps) {
    const long long t = token_begin + b;
    int owner = -1, row = -1;
    if (lane < topk) {
      const int id = ids[t * topk + lane];
      row = exp2perm[t * topk + lane];
      if (row >= 0) owner = strided ? id % ep_ranks : id / per;
    }
    const int base = __shfl_sync(0xffffffffu, my_base, owner < 0 ? 0 : owner);
    const unsigned long long dq = __shfl_sync(0xffffffffu, my_q, owner < 0 ? 0 : owner);
    const unsigned long long dsf = __shfl_sync(0xffffffffu, my_sf, owner < 0 ? 0 : owner);
    const long long local_row = row >= 0 ? (long long)(row - base) : -1;
    const uint8_t* src = q + b * cols;
    for (int c0 = 0; c0 < qv; c0 += K3G_DISPATCH_VPL * 32) {             // warp-uniform trip count: the shuffles below need every lane
      const int v0 = c0 + lane;
      Vec x[K3G_DISPATCH_VPL];
#pragma unroll
      for (int u = 0; u < K3G_DISPATCH_VPL; ++u)
        if (v0 + 32 * u < qv) x[u] = ld_stream_vec<VB>(src + (size_t)(v0 + 32 * u) * VB);
      for (int k = 0; k < topk; ++k) {
        const long long r = __shfl_sync(0xffffffffu, local_row, k);
        const unsigned long long d = __shfl_sync(0xffffffffu, dq, k);
        if (r < 0) continue;
        uint8_t* dst = reinterpret_cast<uint8_t*>(d + (unsigned long long)r * cols);
#pragma unroll
        for (int u = 0; u < K3G_DISPATCH_VPL; ++u)
          if (v0 + 32 * u < qv) st_stream_vec<VB>(dst + (size_t)(v0 + 32 * u) * VB, x[u]);
      }
    }
    if (sf_vec) {
      uint4 s4 = make_uint4(0u, 0u, 0u, 0u);
      if (lane < (sfb >> 4)) s4 = __ldcs(reinterpret_cast<const uint4*>(sf + b * sfb) + lane);
      for (int k = 0; k < topk; ++k) {
        const long long r = __shfl_sync(0xffffffffu, local_row, k);
        const unsigned long long d = __shfl_sync(0xffffffffu, dsf, k);
        if (r >= 0 && lane < (sfb >> 4)) __stcs(reinterpret_cast<uint4*>(d + (unsigned long long)r * sfb) + lane, s4);
      }
    } else {
      for (int k = 0; k < topk; ++k) {
        const long long r = __shfl_sync(0xffffffffu, local_row, k);
        const unsigned long long d = __shfl_sync(0xffffffffu, dsf, k);
        if (r < 0) continue;
        for (int i = lane; i < sfb; i += 32) reinterpret_cast<uint8_t*>(d)[r * sfb + i] = sf[b * sfb + i];
      }
    }
  }
}

__global__ void __launch_bounds__(256, K3G_DISPATCH_MINB) permute_dispatch_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                                               const int* __restrict__ ids, const int* __restrict__ exp2perm,
                                                               const int* __restrict__ blockoff, int B, long long token_begin, int topk,
                                                               int cols, int per, int ep_ranks, int strided,
                                                               const unsigned long long* __restrict__ q_peer,
                                                               const unsigned long long* __restrict__ sf_peer) {
  // lane o keeps owner o's buffer addresses and first row
  const int lane = threadIdx.x & 31;
  unsigned long long my_q = 0ull, my_sf = 0ull;
  int my_base = 0;
  if (lane < ep_ranks) { my_q = q_peer[lane]; my_sf = sf_peer[lane]; my_base = blockoff[lane * per]; }
  // 32-byte accesses when every source and destination row starts on a 32-byte boundary (uniform over the grid)
  const bool wide = (cols & 31) == 0 && (reinterpret_cast<unsigned long long>(q) & 31ull) == 0 &&
                    __all_sync(0xffffffffu, (my_q & 31ull) == 0);
  if (wide) permute_dispatch_body<32>(q, sf, ids, exp2perm, B, token_begin, topk, cols, per, ep_ranks, strided, my_q, my_sf, my_base);
  else permute_dispatch_body<16>(q, sf, ids, exp2perm, B, token_begin, topk, cols, per, ep_ranks, strided, my_q, my_sf, my_base);
}

template <bool RESIDUAL>
__global__ void __launch_bounds__(128) finalize_kernel(const __nv_bfloat16* fc2, const int* exp2perm, const float* wts,
                                                       const __nv_bfloat16* residual, __nv_bfloat16* out, int T, int cols, int topk) {
  finalize_body<RESIDUAL>(fc2, exp2perm, wts, residual, out, T, cols, topk);
}

}  // namespace

// ---- manifest entry points: TOPK = 16 and the expert placement are build constants there
//      (source/k3_moe_prefill_v4.cu:87, :100-109) ---------------------------------------------
#ifndef EP_RANKS
#define EP_RANKS 4
#endif
#ifdef EP_STRIDED
#define K3G_EP_STRIDED 1
#else
#define K3G_EP_STRIDED 0
#endif

extern "C" __global__ void __launch_bounds__(256) kern_k3_moe_route_count(const int* __restrict__ ids, int T, int rank, int E,
                                                                         int* __restrict__ blockcount) {
  route_count_body<kMaxE>(ids, T, rank, E, 16, EP_RANKS, K3G_EP_STRIDED, blockcount);
}
extern "C" __global__ void __launch_bounds__(1024) kern_k3_moe_route_tables(const int* __restrict__ blockcount, int blocks, int E, int tile,
                                                                           int* __restrict__ blockoff, int* __restrict__ cta_batch,
                                                                           int* __restrict__ cta_limit, int* __restrict__ num_non_exiting,
                                                                           int* __restrict__ total_padded, int* __restrict__ route_map) {
  route_tables_body<kMaxE>(blockcount, blocks, E, tile, blockoff, cta_batch, cta_limit, num_non_exiting, total_padded, route_map);
}
extern "C" __global__ void __launch_bounds__(512) kern_k3_moe_route_scatter(const int* __restrict__ ids, const int* __restrict__ blockoff,
                                                                           int T, int rank, int E, int* __restrict__ route_map,
                                                                           int* __restrict__ exp2perm) {
  __shared__ int hist[kMaxGroups][kMaxE];
  route_scatter_body<kMaxE, int>(ids, blockoff, T, rank, E, 16, EP_RANKS, K3G_EP_STRIDED, route_map, exp2perm, hist);
}
extern "C" __global__ void __launch_bounds__(128) kern_k3_moe_finalize(const __nv_bfloat16* __restrict__ fc2, const int* __restrict__ exp2perm,
                                                                      const float* __restrict__ wts, __nv_bfloat16* __restrict__ out,
                                                                      int T, int cols) {
  finalize_body<false>(fc2, exp2perm, wts, nullptr, out, T, cols, 16);
}

// ---- load-time expert weight / scale layouts (the formats the grouped GEMM reads) ---------------------
// Replaces kern_k3_moe_w_shuffle / kern_k3_moe_sf_shuffle (source/k3_moe_prefill_v4.cu:304-327).  Row r of the
// GEMM layout takes source row src_row(r): inside every group of 32 rows, row (r % 8) * 4 + (r % 32) / 8; for a
// gated (gate | up) matrix the two halves are then interleaved row by row.
__device__ __forceinline__ int shuffled_src_row(int r, int n, int gated) {
  const int u = (r & ~31) + ((r & 7) << 2) + ((r & 31) >> 3);
  return gated ? ((u & 1) ? n / 2 : 0) + (u >> 1) : u;
}

// dst[e][r][:] = src[e][src_row(r)][:], rows of row_bytes bytes (a multiple of 16), moved as 16-byte vectors.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_moe_w_shuffle(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                                        int experts, int n, int row_bytes, int gated) {
  const int per_row = row_bytes >> 4;
  const long long total = (long long)experts * n * per_row;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nthreads) {
    const long long row = i / per_row;                       // e * n + r
    const int c = (int)(i - row * per_row);
    const long long e = row / n;
    const int r = (int)(row - e * n);
    reinterpret_cast<uint4*>(dst)[i] = __ldg(reinterpret_cast<const uint4*>(src + (e * n + shuffled_src_row(r, n, gated)) * row_bytes) + c);
  }
}

// Scale bytes [e][n][kg] -> 128 x 4 tiles of 512 bytes: byte (r, c) lands at
//   ((r / 128) * (kg / 4) + c / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4
// of expert e's block, read from source row src_row(r).  One thread assembles one 16-byte destination vector
// (four rows 32 apart x four consecutive k groups) from four 4-byte source words, so stores are coalesced.
// n % 128 == 0 and kg % 4 == 0 take that path; other shapes go byte by byte.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_moe_sf_shuffle(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                                         int experts, int n, int kg, int gated) {
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if ((n & 127) == 0 && (kg & 3) == 0 && ((reinterpret_cast<unsigned long long>(src) & 3ull) == 0) &&
      ((reinterpret_cast<unsigned long long>(dst) & 15ull) == 0)) {
    const long long per_expert = (long long)n * kg >> 4;     // 16-byte vectors per expert
    const int kq = kg >> 2;
    for (long long v = tid; v < experts * per_expert; v += nthreads) {
      const long long e = v / per_expert;
      const long long w = v - e * per_expert;                // vector inside the expert: (tile, q) with 32 vectors per tile
      const long long tile = w >> 5;
      const int q = (int)(w & 31);
      const int R = (int)(tile / kq), C = (int)(tile - (long long)R * kq);
      unsigned word[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = R * 128 + j * 32 + q;
        word[j] = __ldg(reinterpret_cast<const unsigned*>(src + (e * n + shuffled_src_row(r, n, gated)) * kg + 4 * C));
      }
      reinterpret_cast<uint4*>(dst)[v] = make_uint4(word[0], word[1], word[2], word[3]);
    }
  } else {
    const long long total = (long long)experts * n * kg;
    for (long long i = tid; i < total; i += nthreads) {
      const int c = (int)(i % kg), r = (int)(i / kg % n);
      const long long e = i / kg / n;
      const long long at = ((long long)(r / 128) * (kg / 4) + c / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4;
      dst[e * n * kg + at] = src[(e * n + shuffled_src_row(r, n, gated)) * kg + c];
    }
  }
}

#ifndef K3G_CUBIN_ONLY
static int check_route(int T, int E, int topk, int ep_ranks) {
  K3G_REQUIRE(T >= 0 && E > 0 && E <= kMaxEWide, K3G_ESHAPE);
  K3G_REQUIRE(topk > 0 && topk <= kMaxTopk && (kRouteBlock * topk) % 32 == 0, K3G_ESHAPE);
  K3G_REQUIRE(ep_ranks > 0, K3G_ESHAPE);
  return K3G_OK;
}

// rank in [0, ep_ranks), or -1 = every owner's experts in owner-major order (E is then the total and must divide evenly)
static int check_route_rank(int rank, int E, int ep_ranks) {
  K3G_REQUIRE(rank >= -1 && rank < ep_ranks, K3G_ERANGE);
  if (rank < 0) K3G_REQUIRE(E % ep_ranks == 0, K3G_ESHAPE);
  return K3G_OK;
}

// Raise the dynamic shared-memory limit of a wide (64 KB histogram) kernel once per device.
template <typename Kernel>
static int opt_in_wide_smem(Kernel kernel, std::atomic<bool>* opted, int bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !opted[dev].load(std::memory_order_acquire)) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    opted[dev].store(true, std::memory_order_release);      // setting the attribute twice is harmless; the flag only saves the call
  }
  return K3G_OK;
}
constexpr int kWideSmem = kMaxGroups * kMaxEWide * (int)sizeof(unsigned short);      // 64 KB

K3G_API int k3g_moe_route_count(const void* ids, int T, int rank, int E, int topk, int ep_ranks, int strided, void* blockcount,
                                void* stream) {
  K3G_REQUIRE_PTR(ids); K3G_REQUIRE_PTR(blockcount);
  if (int rc = check_route(T, E, topk, ep_ranks)) return rc;
  if (int rc = check_route_rank(rank, E, ep_ranks)) return rc;
  if (T == 0) return K3G_OK;
  if (E <= kMaxE)
    route_count_kernel<kMaxE><<<(T + kRouteBlock - 1) / kRouteBlock, 256, 0, k3g_stream(stream)>>>((const int*)ids, T, rank, E, topk, ep_ranks,
                                                                                                 strided, (int*)blockcount);
  else
    route_count_kernel<kMaxEWide><<<(T + kRouteBlock - 1) / kRouteBlock, 256, 0, k3g_stream(stream)>>>((const int*)ids, T, rank, E, topk,
                                                                                                     ep_ranks, strided, (int*)blockcount);
  return k3g_launch_status();
}

K3G_API int k3g_moe_route_tables(const void* blockcount, int blocks, int E, int tile, void* blockoff, void* cta_batch,
                                 void* cta_limit, void* num_non_exiting, void* total_padded, void* route_map, void* stream) {
  K3G_REQUIRE_PTR(blockcount); K3G_REQUIRE_PTR(blockoff); K3G_REQUIRE_PTR(cta_batch); K3G_REQUIRE_PTR(cta_limit);
  K3G_REQUIRE_PTR(num_non_exiting); K3G_REQUIRE_PTR(total_padded); K3G_REQUIRE_PTR(route_map);
  K3G_REQUIRE(blocks >= 0 && E > 0 && E <= kMaxEWide && tile > 0, K3G_ESHAPE);
  if (E <= kMaxE)
    route_tables_kernel<kMaxE><<<1, 1024, 0, k3g_stream(stream)>>>((const int*)blockcount, blocks, E, tile, (int*)blockoff, (int*)cta_batch,
                                                                  (int*)cta_limit, (int*)num_non_exiting, (int*)total_padded, (int*)route_map);
  else
    route_tables_kernel<kMaxEWide><<<1, 1024, 0, k3g_stream(stream)>>>((const int*)blockcount, blocks, E, tile, (int*)blockoff, (int*)cta_batch,
                                                                      (int*)cta_limit, (int*)num_non_exiting, (int*)total_padded, (int*)route_map);
  return k3g_launch_status();
}

K3G_API int k3g_moe_route_scatter(const void* ids, const void* blockoff, int T, int rank, int E, int topk, int ep_ranks,
                                  int strided, void* route_map, void* exp2perm, void* stream) {
  K3G_REQUIRE_PTR(ids); K3G_REQUIRE_PTR(blockoff); K3G_REQUIRE_PTR(route_map); K3G_REQUIRE_PTR(exp2perm);
  if (int rc = check_route(T, E, topk, ep_ranks)) return rc;
  if (int rc = check_route_rank(rank, E, ep_ranks)) return rc;
  if (T == 0) return K3G_OK;
  if (E <= kMaxE) {
    route_scatter_kernel<<<(T + kRouteBlock - 1) / kRouteBlock, 512, 0, k3g_stream(stream)>>>(
        (const int*)ids, (const int*)blockoff, T, rank, E, topk, ep_ranks, strided, (int*)route_map, (int*)exp2perm);
  } else {
    static std::atomic<bool> opted[64];
    if (int rc = opt_in_wide_smem(route_scatter_wide_kernel, opted, kWideSmem)) return rc;
    route_scatter_wide_kernel<<<(T + kRouteBlock - 1) / kRouteBlock, 512, kWideSmem, k3g_stream(stream)>>>(
        (const int*)ids, (const int*)blockoff, T, rank, E, topk, ep_ranks, strided, (int*)route_map, (int*)exp2perm);
  }
  return k3g_launch_status();
}

// route_tables + route_scatter in one launch: every scatter block derives its own row of block offsets from the
// per-block counts, block 0 also writes the work list, the scalars and the padding rows.  All outputs bit-identical
// to k3g_moe_route_tables followed by k3g_moe_route_scatter.
K3G_API int k3g_moe_route_tables_scatter(const void* ids, const void* blockcount, int T, int rank, int E, int topk, int ep_ranks, int strided,
                                         int tile, void* blockoff, void* cta_batch, void* cta_limit, void* num_non_exiting,
                                         void* total_padded, void* route_map, void* exp2perm, void* stream) {
  K3G_REQUIRE_PTR(ids); K3G_REQUIRE_PTR(blockcount); K3G_REQUIRE_PTR(blockoff); K3G_REQUIRE_PTR(cta_batch); K3G_REQUIRE_PTR(cta_limit);
  K3G_REQUIRE_PTR(num_non_exiting); K3G_REQUIRE_PTR(total_padded); K3G_REQUIRE_PTR(route_map); K3G_REQUIRE_PTR(exp2perm);
  if (int rc = check_route(T, E, topk, ep_ranks)) return rc;
  if (int rc = check_route_rank(rank, E, ep_ranks)) return rc;
  K3G_REQUIRE(tile > 0 && T > 0, K3G_ESHAPE);               // T = 0 has no block to write the scalars: use k3g_moe_route_tables
  const int grid = (T + kRouteBlock - 1) / kRouteBlock;
  if (E <= kMaxE) {
    route_tables_scatter_kernel<<<grid, 512, 0, k3g_stream(stream)>>>((const int*)ids, (const int*)blockcount, T, rank, E, topk, ep_ranks,
                                                                     strided, tile, (int*)blockoff, (int*)cta_batch, (int*)cta_limit,
                                                                     (int*)num_non_exiting, (int*)total_padded, (int*)route_map, (int*)exp2perm);
  } else {
    static std::atomic<bool> opted[64];
    if (int rc = opt_in_wide_smem(route_tables_scatter_wide_kernel, opted, kWideSmem)) return rc;
    route_tables_scatter_wide_kernel<<<grid, 512, kWideSmem, k3g_stream(stream)>>>(
        (const int*)ids, (const int*)blockcount, T, rank, E, topk, ep_ranks, strided, tile, (int*)blockoff, (int*)cta_batch, (int*)cta_limit,
        (int*)num_non_exiting, (int*)total_padded, (int*)route_map, (int*)exp2perm);
  }
  return k3g_launch_status();
}

K3G_API int k3g_moe_finalize(const void* fc2, const void* exp2perm, const void* wts, void* out, int T, int cols, int topk,
                             void* stream) {
  K3G_REQUIRE_PTR(fc2); K3G_REQUIRE_PTR(exp2perm); K3G_REQUIRE_PTR(wts); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE_ALIGNED(fc2); K3G_REQUIRE_ALIGNED(out);
  K3G_REQUIRE(T >= 0 && cols > 0 && cols % 8 == 0 && topk > 0 && topk <= kMaxTopk, K3G_ESHAPE);
  if (T == 0) return K3G_OK;
  finalize_kernel<false><<<T, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)fc2, (const int*)exp2perm, (const float*)wts, nullptr,
                                                           (__nv_bfloat16*)out, T, cols, topk);
  return k3g_launch_status();
}

K3G_API int k3g_finalize_residual(const void* fc2, const void* exp2perm, const void* wts, const void* residual, void* out, int T,
                                  int cols, int topk, void* stream) {
  K3G_REQUIRE_PTR(fc2); K3G_REQUIRE_PTR(exp2perm); K3G_REQUIRE_PTR(wts); K3G_REQUIRE_PTR(residual); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE_ALIGNED(fc2); K3G_REQUIRE_ALIGNED(out); K3G_REQUIRE_ALIGNED(residual);
  K3G_REQUIRE(T >= 0 && cols > 0 && cols % 8 == 0 && topk > 0 && topk <= kMaxTopk, K3G_ESHAPE);
  if (T == 0) return K3G_OK;
  finalize_kernel<true><<<T, 128, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)fc2, (const int*)exp2perm, (const float*)wts,
                                                          (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, T, cols, topk);
  return k3g_launch_status();
}

K3G_API int k3g_permute_gather(const void* q, const void* sf, const void* route_map, long long rows, int cols, void* out_q,
                               void* out_sf, void* stream) {
  K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(sf); K3G_REQUIRE_PTR(route_map); K3G_REQUIRE_PTR(out_q); K3G_REQUIRE_PTR(out_sf);
  K3G_REQUIRE_ALIGNED(q); K3G_REQUIRE_ALIGNED(out_q);
  K3G_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0, K3G_ESHAPE);
  if ((cols >> 5) % 16 == 0) { K3G_REQUIRE_ALIGNED(sf); K3G_REQUIRE_ALIGNED(out_sf); }
  if (rows == 0) return K3G_OK;
  long long grid = (rows + 7) / 8;                 // eight warps per block, one row per warp pass
  if (grid > 148 * 64) grid = 148 * 64;            // then rows are walked with a warp stride
  const bool wide = cols % 32 == 0 && ((uintptr_t)q & 31) == 0 && ((uintptr_t)out_q & 31) == 0;    // every row starts on a 32-byte boundary
  if (wide)
    permute_gather_kernel<32><<<(unsigned)grid, 256, 0, k3g_stream(stream)>>>((const uint8_t*)q, (const uint8_t*)sf, (const int*)route_map, rows,
                                                                             cols, (uint8_t*)out_q, (uint8_t*)out_sf);
  else
    permute_gather_kernel<16><<<(unsigned)grid, 256, 0, k3g_stream(stream)>>>((const uint8_t*)q, (const uint8_t*)sf, (const int*)route_map, rows,
                                                                             cols, (uint8_t*)out_q, (uint8_t*)out_sf);
  return k3g_launch_status();
}
K3G_API int k3g_permute_dispatch(const void* q, const void* sf, const void* ids, const void* exp2perm, const void* blockoff, int B,
                                 long long token_begin, int topk, int cols, int experts, int ep_ranks, int strided, const void* out_q_peer,
                                 const void* out_sf_peer, void* stream) {
  K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(sf); K3G_REQUIRE_PTR(ids); K3G_REQUIRE_PTR(exp2perm); K3G_REQUIRE_PTR(blockoff);
  K3G_REQUIRE_PTR(out_q_peer); K3G_REQUIRE_PTR(out_sf_peer);
  K3G_REQUIRE_ALIGNED(q);
  K3G_REQUIRE(B >= 0 && token_begin >= 0 && cols > 0 && cols % 32 == 0 && topk > 0 && topk <= kMaxTopk, K3G_ESHAPE);
  K3G_REQUIRE(ep_ranks >= 1 && ep_ranks <= 8 && experts > 0 && experts <= kMaxEWide && experts % ep_ranks == 0, K3G_ESHAPE);
  if ((cols >> 5) % 16 == 0) K3G_REQUIRE_ALIGNED(sf);
  if (B == 0) return K3G_OK;
  long long grid = (B + 7) / 8;                    // eight warps per block, one token per warp pass
  if (grid > 148 * 8) grid = 148 * 8;
  permute_dispatch_kernel<<<(unsigned)grid, 256, 0, k3g_stream(stream)>>>(
      (const uint8_t*)q, (const uint8_t*)sf, (const int*)ids, (const int*)exp2perm, (const int*)blockoff, B, token_begin, topk, cols,
      experts / ep_ranks, ep_ranks, strided, (const unsigned long long*)out_q_peer, (const unsigned long long*)out_sf_peer);
  return k3g_launch_status();
}
K3G_API int k3g_moe_w_shuffle(const void* src, void* dst, int experts, int n, int row_bytes, int gated, void* stream) {
  K3G_REQUIRE_PTR(src); K3G_REQUIRE_PTR(dst);
  K3G_REQUIRE_ALIGNED(src); K3G_REQUIRE_ALIGNED(dst);
  K3G_REQUIRE(experts >= 0 && n > 0 && n % 32 == 0 && row_bytes > 0 && row_bytes % 16 == 0 && (!gated || n % 64 == 0), K3G_ESHAPE);
  const long long total = (long long)experts * n * (row_bytes / 16);
  if (total == 0) return K3G_OK;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  kern_k3_moe_w_shuffle<<<(unsigned)blocks, 256, 0, k3g_stream(stream)>>>((const unsigned char*)src, (unsigned char*)dst, experts, n, row_bytes, gated);
  return k3g_launch_status();
}

K3G_API int k3g_moe_sf_shuffle(const void* src, void* dst, int experts, int n, int kg, int gated, void* stream) {
  K3G_REQUIRE_PTR(src); K3G_REQUIRE_PTR(dst);
  K3G_REQUIRE(experts >= 0 && n > 0 && n % 128 == 0 && kg > 0 && kg % 4 == 0 && (!gated || n % 64 == 0), K3G_ESHAPE);
  const long long total = (long long)experts * n * kg / 16;
  if (total == 0) return K3G_OK;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  kern_k3_moe_sf_shuffle<<<(unsigned)blocks, 256, 0, k3g_stream(stream)>>>((const unsigned char*)src, (unsigned char*)dst, experts, n, kg, gated);
  return k3g_launch_status();
}
#endif
