// Tensor-parallel collectives as CUDA kernels over NVLink peer pointers, and the fused
// reduce-scatter -> residual/RMSNorm/MXFP8 -> all-gather kernel.
//
// Replaces, behind the same entry names and parameter lists, the collective kernels of
// xiaguan/kern-k3:
//   kern_k3_flags_init, kern_k3_epoch_bump   source/k3_collectives.cu:64-79
//   kern_k3_rs_arrive1                       source/k3_rs_arrive_v2.cu:41-76   (payload-less barrier)
//   kern_k3_rs_pull                          source/k3_reducescatter_pull_nr4.cu:124-186
//   kern_k3_allgather4_push                  source/k3_allgather4_v3.cu:61-116
//
// Protocol (unchanged): every rank owns a table of u64 arrival counters.  flags[0] is the
// epoch: it grows by `units` once per program replay.  A collective call owns a slot; each
// rank adds `units` arrivals to its own flags[slot] and waits until every peer's flags[slot]
// has reached its own flags[0].  Counters are never reset.  A wait is its own launch (or the
// tail of a push kernel whose other blocks never wait), so a spinning block cannot starve
// blocks that have not been scheduled.
//
// Differences from the reference, all on the failure path: a wait is bounded in wall-clock
// time (globaltimer) AND in iterations, and a wait that gives up records
// {1, slot, peer, observed counter} in a caller-visible status word and returns -- the
// reference breaks out silently (source/k3_collectives.cu:121-123).
//
// Remote traffic is plain 16-byte (reduce-scatter loads) and 8/16-byte (all-gather stores)
// vector accesses on peer addresses issued by every CTA; there is no TMA and no multicast
// anywhere in this file.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

#ifndef K3G_SPIN_NS
#define K3G_SPIN_NS 2000000000LL   /* default bound of a wait: 2 s */
#endif
#define K3G_SPIN_ITERS_PER_US 64   /* iteration cap = this * timeout in us (each iteration sleeps >= 64 ns) */
#define K3G_MAX_RANKS 8

// Status of the most recent failed wait of a launch that was given no status pointer:
// {code (1 = timed out), slot, peer, observed counter}.  External linkage, so a runtime that
// loads the cubin can read it with cuModuleGetGlobal("k3g_wait_status_word").
extern "C" { __device__ unsigned k3g_wait_status_word[4]; }
#define g_wait_status k3g_wait_status_word

namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void red_release_sys_add(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Spin until *counter (the full 64-bit arrival count: counters are never reset, and a 32-bit compare would
// pass without waiting for one replay after 2^32 arrivals) reaches target; false and a status record on
// expiry.  The record keeps the low 32 bits of the observed count.
__device__ __forceinline__ bool bounded_wait(const void* counter, unsigned long long target, long long timeout_ns, unsigned* status,
                                             int slot, int peer) {
  const unsigned long long t0 = globaltimer_ns();
  const long long max_iters = (timeout_ns / 1000 + 1) * K3G_SPIN_ITERS_PER_US;
  long long it = 0;
  unsigned long long v;
  while ((v = ld_relaxed_sys_u64(counter)) < target) {
    if (++it > max_iters || (long long)(globaltimer_ns() - t0) > timeout_ns) {
      if (atomicCAS(&status[0], 0u, 1u) == 0u) { status[1] = (unsigned)slot; status[2] = (unsigned)peer; status[3] = (unsigned)v; }
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// One warp: publish `units` arrivals on this rank's slot, then lane q waits for peer q.
__device__ __forceinline__ void arrive_and_wait(unsigned long long* flags, const unsigned long long* flags_peer, int units, int slot,
                                                int nranks, long long timeout_ns, unsigned* status) {
  const int nr = nranks < K3G_MAX_RANKS ? nranks : K3G_MAX_RANKS;
  if (threadIdx.x == 0) red_release_sys_add(flags + slot, (unsigned long long)units);
  const int q = threadIdx.x;
  if (q < nr) {
    const unsigned long long target = flags[0];
    bounded_wait((const void*)(flags_peer[q] + (unsigned long long)slot * 8ull), target, timeout_ns, status, slot, q);
  }
  __syncwarp();
  if (threadIdx.x == 0) fence_acq_rel_sys();
}

// Tail of a push kernel.  The reference publishes one system-scope release-add per block
// (source/k3_allgather4_v3.cu:95-98); a system-scope release is expensive and a grid of a few thousand
// blocks serialises on it.  Here each block fences at device scope and takes a ticket on a device-scope
// counter; the block that draws the last ticket has, by causality, every block's stores ordered before
// it and publishes the whole grid's arrivals (gridDim.x, so the counter protocol is unchanged) with ONE
// system-scope release-add, then re-arms the ticket counter.  Block 0 waits for every peer (lane q polls
// peer q); it is resident from the start, and no other block ever waits, so the grid always drains.
__device__ unsigned g_tail_ticket[64];   // one ticket counter per slot (mod 64): launches on different slots may overlap

// `arrivals` is what the launch publishes on its slot (the epoch counts units, which the reference ties to gridDim.x;
// the C-ABI launches run a smaller, resident grid and publish the caller's `units`).
__device__ __forceinline__ void block_arrive_tail(unsigned long long* flags, const unsigned long long* flags_peer, int slot, int nranks,
                                                  long long timeout_ns, unsigned* status, unsigned arrivals) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned* tk = &g_tail_ticket[slot & 63];
    const unsigned ticket = atomicAdd(tk, 1u);
    if (ticket == gridDim.x - 1) {
      *tk = 0u;                                   // stream order keeps the next launch behind this store
      __threadfence();
      red_release_sys_add(flags + slot, (unsigned long long)arrivals);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < 32) {
    const int nr = nranks < K3G_MAX_RANKS ? nranks : K3G_MAX_RANKS;
    const int q = threadIdx.x;
    if (q < nr) {
      const unsigned long long target = flags[0];
      bounded_wait((const void*)(flags_peer[q] + (unsigned long long)slot * 8ull), target, timeout_ns, status, slot, q);
    }
    __syncwarp();
    if (threadIdx.x == 0) fence_acq_rel_sys();
  }
}

// ---- reduce-scatter, pull form (rs_bases / rs_chain: k3g_device.cuh) ---------------------------
// 32 bytes per access when the chunk allows it: the chain is element-wise, so the wider access needs no exchange.
template <int NR>
__device__ __forceinline__ V16 rs_chain32(const uint4* const (&base)[NR], long long i) {
  V16 x[NR];
#pragma unroll
  for (int k = 0; k < NR; ++k) x[k] = ld_plain32(base[k] + 2 * i);   // all hops' loads issued back to back
  V16 a = x[0];
#pragma unroll
  for (int k = 1; k < NR; ++k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) a.w[j] = add_bf2(a.w[j], x[k].w[j]);
  }
  return a;
}

template <int NR, int OWNPOS, int DESCEND>
__device__ __forceinline__ void rs_pull_body(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                             const unsigned long long* __restrict__ src_peer, long long count, int rank) {
  const long long nvec = count >> 3;
  const uint4* base[NR];
  rs_bases<NR, OWNPOS, DESCEND>(src, src_peer, (long long)rank * count, rank, base);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool wide = (count & 15) == 0 && (reinterpret_cast<unsigned long long>(dst) & 31ull) == 0;
#pragma unroll
  for (int k = 0; k < NR; ++k) wide = wide && (reinterpret_cast<unsigned long long>(base[k]) & 31ull) == 0;
  if (wide) {                                          // uniform over the grid
    const long long n32 = count >> 4;
    long long i = tid;
    for (; i + stride < n32; i += 2 * stride) {        // two 32-byte vectors per hop in flight per thread
      const V16 a = rs_chain32<NR>(base, i), b = rs_chain32<NR>(base, i + stride);
      st_stream32(reinterpret_cast<unsigned char*>(dst) + 32 * i, a);
      st_stream32(reinterpret_cast<unsigned char*>(dst) + 32 * (i + stride), b);
    }
    if (i < n32) st_stream32(reinterpret_cast<unsigned char*>(dst) + 32 * i, rs_chain32<NR>(base, i));
    return;
  }
  long long i = tid;
  for (; i + stride < nvec; i += 2 * stride) {      // two vectors per thread in flight
    const V8 a = rs_chain<NR>(base, i), b = rs_chain<NR>(base, i + stride);
    st_stream(reinterpret_cast<uint4*>(dst) + i, a);
    st_stream(reinterpret_cast<uint4*>(dst) + i + stride, b);
  }
  if (i < nvec) st_stream(reinterpret_cast<uint4*>(dst) + i, rs_chain<NR>(base, i));
}

// Any world size <= 8 and any order, with the chain sequence computed at run time.
__global__ void __launch_bounds__(1024) rs_pull_generic_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                               const unsigned long long* __restrict__ src_peer, long long count,
                                                               int order, int rank, int nranks) {
  const int ownpos = order >> 1, descend = order & 1;
  const long long off = (long long)rank * count, nvec = count >> 3;
  const uint4* base[K3G_MAX_RANKS];
  int pi = 0;
  for (int k = 0; k < nranks; ++k) {
    if (k == ownpos) { base[k] = reinterpret_cast<const uint4*>(src + off); continue; }
    const int o = descend ? (nranks - 1 - pi) : (1 + pi);
    base[k] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src_peer[(rank + o) % nranks]) + off);
    ++pi;
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    V8 a = ld_plain(base[0] + i);
    for (int k = 1; k < nranks; ++k) {
      const V8 x = ld_plain(base[k] + i);
#pragma unroll
      for (int j = 0; j < 4; ++j) a.w[j] = add_bf2(a.w[j], x.w[j]);
    }
    st_stream(reinterpret_cast<uint4*>(dst) + i, a);
  }
}

template <int NR>
__global__ void __launch_bounds__(1024) rs_pull_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, const unsigned long long* src_peer,
                                                       long long count, int rank) {
  rs_pull_body<NR, NR - 1, 0>(src, dst, src_peer, count, rank);    // peers ascending, own partial last
}

// ---- all-gather, push form ---------------------------------------------------------------------
template <int INFLIGHT>
__device__ __forceinline__ void push_span(const unsigned char* __restrict__ s, unsigned char* __restrict__ d,
                                          const unsigned long long* __restrict__ p, long long nb, int rank, int nr, long long tid,
                                          long long stride) {
  // 32 bytes per access when the span and every rank's copy allow it (the same answer in every thread of the grid)
  unsigned long long low = reinterpret_cast<unsigned long long>(s) | reinterpret_cast<unsigned long long>(d) | (unsigned long long)nb;
#pragma unroll
  for (int q = 0; q < K3G_MAX_RANKS; ++q)
    if (q < nr && q != rank) low |= p[q];
  if ((low & 31ull) == 0) {
    const long long n32 = nb >> 5;
    for (long long i0 = tid; i0 < n32; i0 += INFLIGHT * stride) {   // INFLIGHT vectors loaded before the first store: INFLIGHT x (nr - 1) peer stores in flight
      V16 val[INFLIGHT];
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u)
        if (i0 + u * stride < n32) val[u] = ld_stream32(s + ((i0 + u * stride) << 5));
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u) {
        if (i0 + u * stride >= n32) continue;
        const long long eb = (long long)rank * nb + ((i0 + u * stride) << 5);
        *reinterpret_cast<uint4*>(d + eb) = make_uint4(val[u].w[0], val[u].w[1], val[u].w[2], val[u].w[3]);          // own copy: keep in L2 for the consumer
        *reinterpret_cast<uint4*>(d + eb + 16) = make_uint4(val[u].w[4], val[u].w[5], val[u].w[6], val[u].w[7]);
#pragma unroll
        for (int q = 0; q < K3G_MAX_RANKS; ++q)
          if (q < nr && q != rank) st_stream32(reinterpret_cast<unsigned char*>(p[q]) + eb, val[u]);
      }
    }
    return;
  }
  const long long nv = nb >> 4;
  for (long long i = tid; i < nv; i += stride) {
    const V8 val = ld_stream(s + (i << 4));
    const long long eb = (long long)rank * nb + (i << 4);
    st_plain(d + eb, val);                                       // own copy: keep in L2 for the consumer
#pragma unroll
    for (int q = 0; q < K3G_MAX_RANKS; ++q)
      if (q < nr && q != rank) st_stream(reinterpret_cast<unsigned char*>(p[q]) + eb, val);
  }
}

template <int INFLIGHT>
__device__ __forceinline__ void allgather4_body(const unsigned char* s0, unsigned char* d0, const unsigned long long* p0, long long n0,
                                                const unsigned char* s1, unsigned char* d1, const unsigned long long* p1, long long n1,
                                                const unsigned char* s2, unsigned char* d2, const unsigned long long* p2, long long n2,
                                                const unsigned char* s3, unsigned char* d3, const unsigned long long* p3, long long n3,
                                                unsigned long long* flags, const unsigned long long* flags_peer, int slot, int rank,
                                                int nranks, long long timeout_ns, unsigned* status, unsigned arrivals) {
  const int nr = nranks < K3G_MAX_RANKS ? nranks : K3G_MAX_RANKS;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (n0 > 0) push_span<INFLIGHT>(s0, d0, p0, n0, rank, nr, tid, stride);
  if (n1 > 0) push_span<INFLIGHT>(s1, d1, p1, n1, rank, nr, tid, stride);
  if (n2 > 0) push_span<INFLIGHT>(s2, d2, p2, n2, rank, nr, tid, stride);
  if (n3 > 0) push_span<INFLIGHT>(s3, d3, p3, n3, rank, nr, tid, stride);
  block_arrive_tail(flags, flags_peer, slot, nranks, timeout_ns, status, arrivals);
}

// ---- fused: pull reduce-scatter -> residual add -> RMSNorm -> MXFP8 -> push all-gather ----------
// Row b of this rank's shard is global row rank * rows + b.  delta = the ring-order bf16 chain
// over the W partials (peers ascending from rank + 1, own last); the rest is the single-GPU
// fusion (same team layout and reduction order as resnorm.cu); codes and scales are stored to
// every rank's gathered buffers.  The caller brackets this kernel with two arrive launches.
constexpr int kTeam = 128;
#ifndef K3G_FUSED_WIDE_PULL
#define K3G_FUSED_WIDE_PULL 1      /* 32-byte peer loads in the fused kernel; 0 keeps the 16-byte form for comparison builds */
#endif

template <int VPT, int NR>
__global__ void __launch_bounds__(kTeam, 4) rs_resnorm_mxfp8_ag_kernel(
    const __nv_bfloat16* __restrict__ partial, const unsigned long long* __restrict__ partial_peer,
    const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ residual_out,
    uint8_t* __restrict__ q_all, const unsigned long long* __restrict__ q_all_peer, uint8_t* __restrict__ sf_all,
    const unsigned long long* __restrict__ sf_all_peer, int rows, int rank, float eps, int row_begin, int shard_rows) {
  constexpr int H = VPT * 1024;
  // Over NVLink a store of a few bytes costs a whole packet.  With peers (NR > 1) the row's H / 32 scale bytes
  // are therefore collected in shared memory and leave as 16-byte stores, H / 512 per rank, issued by the
  // first threads of the team; a single rank keeps the direct 4-byte stores (free in local HBM, and no extra
  // block barrier per row).
  constexpr bool kStageScales = NR > 1 && (H / 32) % 16 == 0;
  constexpr int kSfVecs = H / 512;                      // 16-byte vectors of scale bytes per row
  __shared__ float s_red[2][kTeam / 32];
  __shared__ __align__(16) unsigned s_sf[2][kStageScales ? H / 128 : 1];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const uint4* base[NR];
  rs_bases<NR, NR - 1, 0>(partial, partial_peer, (long long)rank * shard_rows * H, rank, base);
  uint8_t* qdst[NR];
  uint8_t* sfdst[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    qdst[r] = (r == rank ? q_all : reinterpret_cast<uint8_t*>(q_all_peer[r])) + (size_t)rank * shard_rows * H;
    sfdst[r] = (r == rank ? sf_all : reinterpret_cast<uint8_t*>(sf_all_peer[r])) + (size_t)rank * shard_rows * (H / 32);
  }
  // Phase A pulls the W partial rows chunk by chunk -- every load of a chunk is issued before the
  // first dependent instruction, W x CH 16-byte loads in flight per thread (the NVLink round trip is
  // what has to be covered) -- and lands the ring-order chain; phase B adds the residual.
  constexpr int CH = NR == 1 ? VPT : NR == 2 ? VPT : NR == 4 ? 4 : 2;
  int it = 0;
  for (int b = row_begin + blockIdx.x; b < row_begin + rows; b += gridDim.x, ++it) {
    const size_t rowoff = (size_t)b * H;
    V8 x[VPT];
    if (K3G_FUSED_WIDE_PULL && NR > 1) {
      rs_chain_team_row<VPT, NR, (NR == 2 ? 4 : NR == 4 ? 2 : 1)>(base, (long long)(rowoff >> 3), t, x);
    } else {
#pragma unroll
      for (int v0 = 0; v0 < VPT; v0 += CH) {
        V8 p[CH][NR];
#pragma unroll
        for (int k = 0; k < NR; ++k) {
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            if (v0 + c < VPT) {
              const long long vi = (long long)((rowoff + (t + (v0 + c) * kTeam) * 8) >> 3);
              p[c][k] = NR == 1 ? ld_stream(base[k] + vi) : ld_plain(base[k] + vi);
            }
          }
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          if (v0 + c < VPT) {
            x[v0 + c] = p[c][0];
#pragma unroll
            for (int k = 1; k < NR; ++k) {
#pragma unroll
              for (int j = 0; j < 4; ++j) x[v0 + c].w[j] = add_bf2(x[v0 + c].w[j], p[c][k].w[j]);
            }
          }
        }
      }
    }
    {
      V8 r[VPT];
#pragma unroll
      for (int v = 0; v < VPT; ++v) r[v] = ld_stream(residual + rowoff + (t + v * kTeam) * 8);
#pragma unroll
      for (int v = 0; v < VPT; ++v) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[v].w[j] = add_bf2(r[v].w[j], x[v].w[j]);
      }
#pragma unroll
      for (int v = 0; v < VPT; ++v) st_stream(residual_out + rowoff + (t + v * kTeam) * 8, x[v]);
    }
    // sum of squares in the fixed order, then the normed row + quant epilogue
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
    float* red = s_red[it & 1];
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kTeam / 32; ++w) tot = __fadd_rn(tot, red[w]);
    const float rr = __frsqrt_rn(__fmaf_rn(tot, 1.0f / (float)H, eps));
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
      const int u = (t + v * kTeam) * 8;
      const V8 g = ld_keep(gamma + u);
      V8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o.w[j] = mul_bf2(pack_bf2(__fmul_rn(bf_lo(x[v].w[j]), rr), __fmul_rn(bf_hi(x[v].w[j]), rr)), g.w[j]);
      unsigned am = absmax8(o);
      am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 1));
      am = max_bf16_bits(am, __shfl_xor_sync(0xffffffffu, am, 2));
      const int e = ue8m0_exp_from_bf16(am);
      unsigned q0, q1;
      quant8(o, pow2_neg(e), q0, q1);
      unsigned sfb = (unsigned)(e + 127);
      sfb |= __shfl_down_sync(0xffffffffu, sfb, 4) << 8;
      sfb |= __shfl_down_sync(0xffffffffu, sfb, 8) << 16;
      if (kStageScales && (lane & 15) == 0) s_sf[it & 1][u >> 7] = sfb;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        st_stream8(qdst[r] + rowoff + u, q0, q1);
        if (!kStageScales && (lane & 15) == 0) *reinterpret_cast<unsigned*>(sfdst[r] + (size_t)b * (H / 32) + (u >> 5)) = sfb;
      }
    }
    if (kStageScales) {
      __syncthreads();                                  // the row's scale words are all in s_sf[it & 1]; its next writer is two rows away
      if (t < kSfVecs * NR) {
        const int r = t / kSfVecs, v = t - r * kSfVecs;
        const uint4 w = reinterpret_cast<const uint4*>(s_sf[it & 1])[v];
        uint8_t* row = sfdst[0];
#pragma unroll
        for (int k = 1; k < NR; ++k) row = r == k ? sfdst[k] : row;      // select, so the pointer array stays in registers
        uint4* d = reinterpret_cast<uint4*>(row + (size_t)b * (H / 32)) + v;
        if (r == rank) *d = w; else __stcs(d, w);
      }
    }
  }
}

__global__ void epoch_add_kernel(unsigned long long* flags, int units) {
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&flags[0], (unsigned long long)units);
}
__global__ void __launch_bounds__(32) arrive_kernel(unsigned long long* flags, const unsigned long long* flags_peer, int units, int slot,
                                                    int nranks, long long timeout_ns, unsigned* status) {
  arrive_and_wait(flags, flags_peer, units, slot, nranks, timeout_ns, status ? status : g_wait_status);
}
// Epoch bump and barrier in one launch, for a replay whose first waiting call is a plain barrier: thread 0 advances
// the epoch before anything of this launch reads it.
__global__ void __launch_bounds__(32) epoch_arrive_kernel(unsigned long long* flags, const unsigned long long* flags_peer, int units, int slot,
                                                          int nranks, long long timeout_ns, unsigned* status) {
  if (threadIdx.x == 0) atomicAdd(&flags[0], (unsigned long long)units);
  __syncwarp();
  arrive_and_wait(flags, flags_peer, units, slot, nranks, timeout_ns, status ? status : g_wait_status);
}
// C-ABI launch: 256-thread blocks (room for four 32-byte vectors in flight per thread), several resident per SM
__global__ void __launch_bounds__(256) allgather4_kernel(const unsigned char* s0, unsigned char* d0, const unsigned long long* p0, long long n0,
                                                          const unsigned char* s1, unsigned char* d1, const unsigned long long* p1, long long n1,
                                                          const unsigned char* s2, unsigned char* d2, const unsigned long long* p2, long long n2,
                                                          const unsigned char* s3, unsigned char* d3, const unsigned long long* p3, long long n3,
                                                          unsigned long long* flags, const unsigned long long* flags_peer, int slot, int rank,
                                                          int nranks, long long timeout_ns, unsigned* status, unsigned arrivals) {
  allgather4_body<4>(s0, d0, p0, n0, s1, d1, p1, n1, s2, d2, p2, n2, s3, d3, p3, n3, flags, flags_peer, slot, rank, nranks, timeout_ns,
                     status ? status : g_wait_status, arrivals);
}

// MXFP8 quantisation of this rank's latent rows written straight into every rank's gathered buffers, then two plain
// payloads (the router's indices and weights) and the barrier tail: kern_k3_moe_quant + kern_k3_allgather4_push in one
// launch (the codes are never written locally and read back).  One 32-element group per thread-step, as kern_k3_moe_quant.
template <int NR>
__global__ void __launch_bounds__(256, NR == 1 ? 6 : 4) moe_quant_allgather_kernel(const __nv_bfloat16* __restrict__ x, long long ngroups, unsigned char* q_all,
                                                                  const unsigned long long* __restrict__ q_peer, unsigned char* sf_all,
                                                                  const unsigned long long* __restrict__ sf_peer, const unsigned char* s2,
                                                                  unsigned char* d2, const unsigned long long* p2, long long n2,
                                                                  const unsigned char* s3, unsigned char* d3, const unsigned long long* p3,
                                                                  long long n3, unsigned long long* flags, const unsigned long long* flags_peer,
                                                                  int slot, int rank, long long timeout_ns, unsigned* status, unsigned arrivals) {
  // The world size is a template argument so that the peers' base pointers are a fixed, small set of registers: the
  // kernel then fits several 256-thread blocks per SM, which is what hides the HBM round trip of the one group a
  // thread has in flight (a single rank has no peer code at all).
  unsigned char* qp[NR > 1 ? NR - 1 : 1];
  unsigned char* sp[NR > 1 ? NR - 1 : 1];
#pragma unroll
  for (int k = 0; k + 1 < NR; ++k) {
    const int q = k < rank ? k : k + 1;                            // the peers in ascending order, own rank left out
    qp[k] = reinterpret_cast<unsigned char*>(q_peer[q]);
    sp[k] = reinterpret_cast<unsigned char*>(sf_peer[q]);
  }
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
  for (long long g = tid; g < ngroups; g += stride) {
    const __nv_bfloat16* src = x + g * 32;
    V8 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = ld_plain(src + 8 * j);
    unsigned am = absmax8(v[0]);
#pragma unroll
    for (int j = 1; j < 4; ++j) am = max_bf16_bits(am, absmax8(v[j]));
    const int e = ue8m0_exp_from_bf16(am);
    const float sc = pow2_neg(e);
    V16 o;                                                       // the group's 32 codes: one 32-byte store per rank (a full sector)
    quant8(v[0], sc, o.w[0], o.w[1]);
    quant8(v[1], sc, o.w[2], o.w[3]);
    quant8(v[2], sc, o.w[4], o.w[5]);
    quant8(v[3], sc, o.w[6], o.w[7]);
    const long long at = (long long)rank * ngroups + g;          // group index in the gathered buffers
    *reinterpret_cast<uint4*>(q_all + at * 32) = make_uint4(o.w[0], o.w[1], o.w[2], o.w[3]);
    *reinterpret_cast<uint4*>(q_all + at * 32 + 16) = make_uint4(o.w[4], o.w[5], o.w[6], o.w[7]);
    sf_all[at] = (unsigned char)(e + 127);
#pragma unroll
    for (int k = 0; k + 1 < NR; ++k) {
      st_stream32(qp[k] + at * 32, o);
      sp[k][at] = (unsigned char)(e + 127);
    }
  }
  if (n2 > 0) push_span<1>(s2, d2, p2, n2, rank, NR, tid, stride);
  if (n3 > 0) push_span<1>(s3, d3, p3, n3, rank, NR, tid, stride);
  block_arrive_tail(flags, flags_peer, slot, NR, timeout_ns, status ? status : g_wait_status, arrivals);
}

}  // namespace

// ---- manifest entry points -------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(1024) kern_k3_flags_init(unsigned long long* __restrict__ flags, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) flags[i] = 0ull;
  if (blockIdx.x == 0 && threadIdx.x < 4) g_wait_status[threadIdx.x] = 0u;
}

extern "C" __global__ void __launch_bounds__(1024) kern_k3_epoch_bump(unsigned long long* __restrict__ flags) {
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&flags[0], (unsigned long long)gridDim.x);
}

extern "C" __global__ void __launch_bounds__(32) kern_k3_rs_arrive1(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                                   const unsigned long long* __restrict__ src_peer,
                                                                   unsigned long long* __restrict__ flags,
                                                                   const unsigned long long* __restrict__ flags_peer, long long count,
                                                                   int units, int slot, int order, int rank, int nranks) {
  (void)src; (void)dst; (void)src_peer; (void)count; (void)order; (void)rank;
  arrive_and_wait(flags, flags_peer, units, slot, nranks, K3G_SPIN_NS, g_wait_status);
}

#ifndef K3G_NR
#define K3G_NR 4
#endif
#ifndef K3G_ORDER
#define K3G_ORDER (2 * (K3G_NR - 1))
#endif
extern "C" __global__ void __launch_bounds__(1024) kern_k3_rs_pull(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                                  const unsigned long long* __restrict__ src_peer,
                                                                  unsigned long long* __restrict__ flags,
                                                                  const unsigned long long* __restrict__ flags_peer, long long count,
                                                                  int slot, int order, int rank, int nranks) {
  (void)flags; (void)flags_peer; (void)slot;
  if (nranks != K3G_NR || order != K3G_ORDER) return;   // one module per shape, as in the reference (:135)
  rs_pull_body<K3G_NR, (K3G_ORDER >> 1), (K3G_ORDER & 1)>(src, dst, src_peer, count, rank);
}

extern "C" __global__ void __launch_bounds__(1024) kern_k3_allgather4_push(
    const unsigned char* __restrict__ s0, unsigned char* __restrict__ d0, const unsigned long long* __restrict__ p0, long long n0,
    const unsigned char* __restrict__ s1, unsigned char* __restrict__ d1, const unsigned long long* __restrict__ p1, long long n1,
    const unsigned char* __restrict__ s2, unsigned char* __restrict__ d2, const unsigned long long* __restrict__ p2, long long n2,
    const unsigned char* __restrict__ s3, unsigned char* __restrict__ d3, const unsigned long long* __restrict__ p3, long long n3,
    unsigned long long* __restrict__ flags, const unsigned long long* __restrict__ flags_peer, int slot, int rank, int nranks) {
  allgather4_body<1>(s0, d0, p0, n0, s1, d1, p1, n1, s2, d2, p2, n2, s3, d3, p3, n3, flags, flags_peer, slot, rank, nranks, K3G_SPIN_NS,
                     g_wait_status, gridDim.x);
}

#ifndef K3G_CUBIN_ONLY
// Grid of a push kernel launched through the C ABI: a few resident blocks per SM of a 148-SM part that stride over
// the payload (two 1024-thread blocks, or four 256-thread ones for the four-payload all-gather), instead of `units`
// short-lived blocks; the launch still publishes `units` arrivals, so the counter protocol is the reference's.
static inline unsigned push_grid(int units) { return (unsigned)(units < 296 ? units : 296); }

static int check_world(int rank, int nranks) {
  K3G_REQUIRE(nranks == 1 || nranks == 2 || nranks == 4 || nranks == 8, K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks, K3G_ERANGE);
  return K3G_OK;
}

K3G_API int k3g_flags_init(void* flags, int n, void* stream) {
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE(n > 0, K3G_ESHAPE);
  kern_k3_flags_init<<<1, 256, 0, k3g_stream(stream)>>>((unsigned long long*)flags, n);
  return k3g_launch_status();
}

K3G_API int k3g_epoch_bump(void* flags, int units, void* stream) {
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE(units > 0, K3G_ESHAPE);
  epoch_add_kernel<<<1, 32, 0, k3g_stream(stream)>>>((unsigned long long*)flags, units);
  return k3g_launch_status();
}

K3G_API int k3g_rs_arrive(void* flags, const void* flags_peer, int units, int slot, int nranks, long long timeout_us, void* status,
                          void* stream) {
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE_PTR(flags_peer);
  K3G_REQUIRE(nranks >= 1 && nranks <= K3G_MAX_RANKS && units > 0, K3G_ESHAPE);
  K3G_REQUIRE(slot >= 1 && timeout_us > 0, K3G_ERANGE);
  arrive_kernel<<<1, 32, 0, k3g_stream(stream)>>>((unsigned long long*)flags, (const unsigned long long*)flags_peer, units, slot, nranks,
                                                 timeout_us * 1000LL, (unsigned*)status);
  return k3g_launch_status();
}

K3G_API int k3g_epoch_arrive(void* flags, const void* flags_peer, int units, int slot, int nranks, long long timeout_us, void* status,
                             void* stream) {
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE_PTR(flags_peer);
  K3G_REQUIRE(nranks >= 1 && nranks <= K3G_MAX_RANKS && units > 0, K3G_ESHAPE);
  K3G_REQUIRE(slot >= 1 && timeout_us > 0, K3G_ERANGE);
  epoch_arrive_kernel<<<1, 32, 0, k3g_stream(stream)>>>((unsigned long long*)flags, (const unsigned long long*)flags_peer, units, slot, nranks,
                                                       timeout_us * 1000LL, (unsigned*)status);
  return k3g_launch_status();
}

K3G_API int k3g_rs_pull(const void* src, void* dst, const void* src_peer, long long count, int order, int rank, int nranks, int grid,
                        void* stream) {
  K3G_REQUIRE_PTR(src); K3G_REQUIRE_PTR(dst); K3G_REQUIRE_PTR(src_peer);
  K3G_REQUIRE_ALIGNED(src); K3G_REQUIRE_ALIGNED(dst);
  K3G_REQUIRE(nranks >= 1 && nranks <= K3G_MAX_RANKS && count >= 0 && count % 8 == 0 && grid > 0, K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks && order >= 0 && order < 2 * nranks, K3G_ERANGE);
  if (count == 0) return K3G_OK;
  const __nv_bfloat16* s = (const __nv_bfloat16*)src; __nv_bfloat16* d = (__nv_bfloat16*)dst;
  const unsigned long long* sp = (const unsigned long long*)src_peer;
  cudaStream_t st = k3g_stream(stream);
  const bool pow2 = (nranks & (nranks - 1)) == 0;
  if (pow2 && order == 2 * (nranks - 1)) {
    switch (nranks) {
      case 1: rs_pull_kernel<1><<<grid, 1024, 0, st>>>(s, d, sp, count, rank); break;
      case 2: rs_pull_kernel<2><<<grid, 1024, 0, st>>>(s, d, sp, count, rank); break;
      case 4: rs_pull_kernel<4><<<grid, 1024, 0, st>>>(s, d, sp, count, rank); break;
      default: rs_pull_kernel<8><<<grid, 1024, 0, st>>>(s, d, sp, count, rank); break;
    }
  } else {
    rs_pull_generic_kernel<<<grid, 1024, 0, st>>>(s, d, sp, count, order, rank, nranks);
  }
  return k3g_launch_status();
}

K3G_API int k3g_allgather4_push(const void* s0, void* d0, const void* p0, long long n0, const void* s1, void* d1, const void* p1,
                                long long n1, const void* s2, void* d2, const void* p2, long long n2, const void* s3, void* d3,
                                const void* p3, long long n3, void* flags, const void* flags_peer, int slot, int rank, int nranks,
                                int units, long long timeout_us, void* status, void* stream) {
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE_PTR(flags_peer);
  K3G_REQUIRE(nranks >= 1 && nranks <= K3G_MAX_RANKS && units > 0, K3G_ESHAPE);
  K3G_REQUIRE(rank >= 0 && rank < nranks && slot >= 1 && timeout_us > 0, K3G_ERANGE);
  const void* ss[4] = {s0, s1, s2, s3}; void* dd[4] = {d0, d1, d2, d3}; const void* pp[4] = {p0, p1, p2, p3};
  const long long nn[4] = {n0, n1, n2, n3};
  for (int i = 0; i < 4; ++i) {
    K3G_REQUIRE(nn[i] >= 0 && nn[i] % 16 == 0, K3G_ESHAPE);
    if (nn[i] > 0) { K3G_REQUIRE_PTR(ss[i]); K3G_REQUIRE_PTR(dd[i]); K3G_REQUIRE_PTR(pp[i]); K3G_REQUIRE_ALIGNED(ss[i]); K3G_REQUIRE_ALIGNED(dd[i]); }
  }
  allgather4_kernel<<<push_grid(units) * 2, 256, 0, k3g_stream(stream)>>>(
      (const unsigned char*)s0, (unsigned char*)d0, (const unsigned long long*)p0, n0, (const unsigned char*)s1, (unsigned char*)d1,
      (const unsigned long long*)p1, n1, (const unsigned char*)s2, (unsigned char*)d2, (const unsigned long long*)p2, n2,
      (const unsigned char*)s3, (unsigned char*)d3, (const unsigned long long*)p3, n3, (unsigned long long*)flags,
      (const unsigned long long*)flags_peer, slot, rank, nranks, timeout_us * 1000LL, (unsigned*)status, (unsigned)units);
  return k3g_launch_status();
}

// kern_k3_moe_quant followed by kern_k3_allgather4_push in one launch (no counterpart in the reference): the MXFP8 codes
// and scale bytes of x [rows, cols] bf16 go straight to rows rank * rows .. of every rank's q_all [nranks * rows, cols] /
// sf_all [nranks * rows, cols / 32]; two more byte payloads (s2 -> d2, s3 -> d3: the router's indices and weights) are
// gathered as by k3g_allgather4_push, and the same barrier tail follows.  Gathered bytes identical to the two calls.
K3G_API int k3g_moe_quant_allgather_push(const void* x, int rows, int cols, void* q_all, const void* q_peer, void* sf_all, const void* sf_peer,
                                         const void* s2, void* d2, const void* p2, long long n2, const void* s3, void* d3, const void* p3,
                                         long long n3, void* flags, const void* flags_peer, int slot, int rank, int nranks, int units,
                                         long long timeout_us, void* status, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(q_all); K3G_REQUIRE_PTR(q_peer); K3G_REQUIRE_PTR(sf_all); K3G_REQUIRE_PTR(sf_peer);
  K3G_REQUIRE_PTR(flags); K3G_REQUIRE_PTR(flags_peer);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE((reinterpret_cast<uintptr_t>(q_all) & 31u) == 0, K3G_EALIGN);   // 32-byte code stores, every rank's buffer alike
  K3G_REQUIRE(rows >= 0 && cols > 0 && cols % 32 == 0 && units > 0, K3G_ESHAPE);
  if (const int rc = check_world(rank, nranks)) return rc;       // 1, 2, 4 or 8 ranks
  K3G_REQUIRE(slot >= 1 && timeout_us > 0, K3G_ERANGE);
  const void* ss[2] = {s2, s3}; void* dd[2] = {d2, d3}; const void* pp[2] = {p2, p3};
  const long long nn[2] = {n2, n3};
  for (int i = 0; i < 2; ++i) {
    K3G_REQUIRE(nn[i] >= 0 && nn[i] % 16 == 0, K3G_ESHAPE);
    if (nn[i] > 0) { K3G_REQUIRE_PTR(ss[i]); K3G_REQUIRE_PTR(dd[i]); K3G_REQUIRE_PTR(pp[i]); K3G_REQUIRE_ALIGNED(ss[i]); K3G_REQUIRE_ALIGNED(dd[i]); }
  }
  // 256-thread blocks, one resident wave (six per SM alone, four with peers: the kernel's launch bounds); the launch
  // still publishes `units` arrivals
  const unsigned grid = (unsigned)(units < 148 ? units : 148) * (nranks == 1 ? 6u : 4u);
#define K3G_MQAG(NR_)                                                                                                                        \
  moe_quant_allgather_kernel<NR_><<<grid, 256, 0, k3g_stream(stream)>>>(                                                                    \
      (const __nv_bfloat16*)x, (long long)rows * cols / 32, (unsigned char*)q_all, (const unsigned long long*)q_peer, (unsigned char*)sf_all, \
      (const unsigned long long*)sf_peer, (const unsigned char*)s2, (unsigned char*)d2, (const unsigned long long*)p2, n2,                   \
      (const unsigned char*)s3, (unsigned char*)d3, (const unsigned long long*)p3, n3, (unsigned long long*)flags,                           \
      (const unsigned long long*)flags_peer, slot, rank, timeout_us * 1000LL, (unsigned*)status, (unsigned)units)
  switch (nranks) {
    case 1: K3G_MQAG(1); break;
    case 2: K3G_MQAG(2); break;
    case 4: K3G_MQAG(4); break;
    default: K3G_MQAG(8); break;
  }
#undef K3G_MQAG
  return k3g_launch_status();
}

template <int NR>
static int launch_fused(int H, int grid, cudaStream_t st, const __nv_bfloat16* partial, const unsigned long long* partial_peer,
                        const __nv_bfloat16* residual, const __nv_bfloat16* gamma, __nv_bfloat16* residual_out, uint8_t* q_all,
                        const unsigned long long* q_all_peer, uint8_t* sf_all, const unsigned long long* sf_all_peer, int rows, int rank,
                        float eps, int row_begin, int shard_rows) {
  switch (H / 1024) {
    case 1: rs_resnorm_mxfp8_ag_kernel<1, NR><<<grid, kTeam, 0, st>>>(partial, partial_peer, residual, gamma, residual_out, q_all, q_all_peer, sf_all, sf_all_peer, rows, rank, eps, row_begin, shard_rows); break;
    case 2: rs_resnorm_mxfp8_ag_kernel<2, NR><<<grid, kTeam, 0, st>>>(partial, partial_peer, residual, gamma, residual_out, q_all, q_all_peer, sf_all, sf_all_peer, rows, rank, eps, row_begin, shard_rows); break;
    case 7: rs_resnorm_mxfp8_ag_kernel<7, NR><<<grid, kTeam, 0, st>>>(partial, partial_peer, residual, gamma, residual_out, q_all, q_all_peer, sf_all, sf_all_peer, rows, rank, eps, row_begin, shard_rows); break;
    default: return K3G_ESHAPE;
  }
  return k3g_launch_status();
}

// Fused reduce-scatter -> residual add -> RMSNorm -> MXFP8 -> all-gather (benchmark configuration 1).
// partial: this rank's [nranks * rows, H] bf16 partial sums; partial_peer[r]: rank r's partial.
// residual / residual_out: this rank's [rows, H] shard.  q_all [nranks * rows, H] u8 and
// sf_all [nranks * rows, H / 32] u8 are every rank's gathered outputs (q_all_peer / sf_all_peer
// the peer tables).  Bracket with k3g_rs_arrive before (partials ready) and after (pushes landed).
// The call processes rows [row_begin, row_begin + rows) of the rank's shard of shard_rows rows
// (shard_rows <= 0: the shard has exactly `rows` rows and row_begin must be 0), so a host can
// pipeline a shard in row chunks; residual / residual_out are indexed by shard row.
K3G_API int k3g_rs_resnorm_mxfp8_ag(const void* partial, const void* partial_peer, const void* residual, const void* gamma,
                                    void* residual_out, void* q_all, const void* q_all_peer, void* sf_all, const void* sf_all_peer,
                                    int rows, int H, float eps, int rank, int nranks, int grid_hint, int row_begin, int shard_rows,
                                    void* stream) {
  K3G_REQUIRE_PTR(partial); K3G_REQUIRE_PTR(partial_peer); K3G_REQUIRE_PTR(residual); K3G_REQUIRE_PTR(gamma);
  K3G_REQUIRE_PTR(residual_out); K3G_REQUIRE_PTR(q_all); K3G_REQUIRE_PTR(q_all_peer); K3G_REQUIRE_PTR(sf_all); K3G_REQUIRE_PTR(sf_all_peer);
  K3G_REQUIRE_ALIGNED(partial); K3G_REQUIRE_ALIGNED(residual); K3G_REQUIRE_ALIGNED(gamma); K3G_REQUIRE_ALIGNED(residual_out);
  K3G_REQUIRE_ALIGNED(q_all); K3G_REQUIRE_ALIGNED(sf_all);
  if (int rc = check_world(rank, nranks)) return rc;
  K3G_REQUIRE(rows >= 0 && (H == 1024 || H == 2048 || H == 7168), K3G_ESHAPE);
  if (shard_rows <= 0) shard_rows = rows;                       // whole shard in one call
  K3G_REQUIRE(row_begin >= 0 && row_begin + rows <= shard_rows, K3G_ERANGE);
  if (nranks > 1) K3G_REQUIRE((reinterpret_cast<uintptr_t>(partial) & 31u) == 0, K3G_EALIGN);   // peers are read 32 bytes at a time
  if (rows == 0) return K3G_OK;
  const int grid = grid_hint > 0 && grid_hint < rows ? grid_hint : rows;
  cudaStream_t st = k3g_stream(stream);
#define K3G_FUSED_ARGS H, grid, st, (const __nv_bfloat16*)partial, (const unsigned long long*)partial_peer, (const __nv_bfloat16*)residual, \
    (const __nv_bfloat16*)gamma, (__nv_bfloat16*)residual_out, (uint8_t*)q_all, (const unsigned long long*)q_all_peer, (uint8_t*)sf_all, \
    (const unsigned long long*)sf_all_peer, rows, rank, eps, row_begin, shard_rows
  switch (nranks) {
    case 1: return launch_fused<1>(K3G_FUSED_ARGS);
    case 2: return launch_fused<2>(K3G_FUSED_ARGS);
    case 4: return launch_fused<4>(K3G_FUSED_ARGS);
    default: return launch_fused<8>(K3G_FUSED_ARGS);
  }
#undef K3G_FUSED_ARGS
}

// Read back (and clear) the status record of the most recent failed wait of a launch that was
// given no status pointer.  host_status receives 4 x u32: {code, slot, peer, observed}.
K3G_API int k3g_wait_status(void* host_status, int clear, void* stream) {
  K3G_REQUIRE_PTR(host_status);
  cudaError_t e = cudaMemcpyFromSymbolAsync(host_status, g_wait_status, 16, 0, cudaMemcpyDeviceToHost, k3g_stream(stream));
  if (e != cudaSuccess) return (int)e;
  e = cudaStreamSynchronize(k3g_stream(stream));
  if (e != cudaSuccess) return (int)e;
  if (clear) {
    const unsigned z[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(g_wait_status, z, 16);
  }
  return e == cudaSuccess ? K3G_OK : (int)e;
}
#endif
