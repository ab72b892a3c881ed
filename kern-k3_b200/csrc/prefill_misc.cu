// Once-per-prefill helpers of the prefill program: row copies, the embedding gather, zero fill and the
// attention-length record.  None of them is arithmetic; all are plain byte movement.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   kern_k3_rank_rows         source/k3_prefill.cu:28-40     (op rank_rows)
//   kern_k3_zero_rows         source/k3_prefill.cu:42-47     (op zero_rows)
//   kern_k3_fmha_lens         source/k3_prefill.cu:49-60     (op fmha_lens)
//   kern_embedding_i64_bf16   source/embedding.cu:6-16       (op embedding)
//   kern_copy_rows_bf16       source/copy_rows.cu:23-30
//   kern_last_row_bf16        source/copy_rows.cu:32-37      (op last_row)
//   kern_own_rows             source/copy_rows.cu:39-47
//
// Layout for B200: a row is moved as 16-byte vectors by the whole block when both addresses and the
// row size allow it (two vectors in flight per thread), byte by byte otherwise; blocks stride over rows, so
// any grid is valid and the reference's one-block-per-row dims keep working.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {

__device__ __forceinline__ bool vec_ok(const void* a, const void* b, long long nbytes) {
  return ((reinterpret_cast<unsigned long long>(a) | reinterpret_cast<unsigned long long>(b) | (unsigned long long)nbytes) & 15ull) == 0;
}

// One row of nbytes bytes, moved by the calling block.
__device__ __forceinline__ void copy_row(void* __restrict__ dst, const void* __restrict__ src, long long nbytes) {
  if (vec_ok(dst, src, nbytes)) {
    const uint4* s = static_cast<const uint4*>(src);
    uint4* d = static_cast<uint4*>(dst);
    const long long nv = nbytes >> 4;
    for (long long i = threadIdx.x; i < nv; i += 2 * blockDim.x) {
      const long long j = i + blockDim.x;
      const uint4 a = __ldg(s + i);
      uint4 b = a;
      if (j < nv) b = __ldg(s + j);
      d[i] = a;
      if (j < nv) d[j] = b;
    }
  } else {
    const unsigned char* s = static_cast<const unsigned char*>(src);
    unsigned char* d = static_cast<unsigned char*>(dst);
    for (long long i = threadIdx.x; i < nbytes; i += blockDim.x) d[i] = s[i];
  }
}

}  // namespace

// dst[j] = src[min(rank * own + j, rows - 1)], j < own, rows of row_bytes bytes: a rank's slice of a chunk, the
// last row repeated past the chunk's end.
extern "C" __global__ void __launch_bounds__(1024) kern_k3_rank_rows(void* __restrict__ dst, const void* __restrict__ src, int rank, int own,
                                                                    int row_bytes, int rows) {
  for (int j = blockIdx.x; j < own; j += gridDim.x) {
    const long long r = min((long long)rank * own + j, (long long)rows - 1);
    copy_row(static_cast<char*>(dst) + (long long)j * row_bytes, static_cast<const char*>(src) + r * row_bytes, row_bytes);
  }
}

// Rows [from, to) of buf zeroed, every byte of them (16-byte stores when the span allows).
extern "C" __global__ void __launch_bounds__(1024) kern_k3_zero_rows(void* __restrict__ buf, int row_bytes, int from, int to) {
  if (to <= from) return;
  char* base = static_cast<char*>(buf) + (long long)from * row_bytes;
  const long long nbytes = (long long)(to - from) * row_bytes;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
  if (((reinterpret_cast<unsigned long long>(base) | (unsigned long long)nbytes) & 15ull) == 0) {
    for (long long i = tid; i < (nbytes >> 4); i += nthreads) reinterpret_cast<uint4*>(base)[i] = make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (long long i = tid; i < nbytes; i += nthreads) base[i] = 0;
  }
}

// lens = {kv_len, 0, 0, T, 0, kv_len, 0, 0}: seq_lens_kv at word 0, cum_seq_lens_q at words 2..3, cum_seq_lens_kv at
// words 4..5 of the attention kernel's length record, for a chunk of T rows ending at token seq_lens[0].
extern "C" __global__ void kern_k3_fmha_lens(const int* __restrict__ seq_lens, int* __restrict__ lens, int T) {
  if (blockIdx.x != 0 || threadIdx.x >= 8) return;
  const int kv = seq_lens[0];
  const int t = threadIdx.x;
  lens[t] = (t == 0 || t == 5) ? kv : (t == 3 ? T : 0);
}

// out[r] = table[ids[r]]: one row per block (the grid is the row count, as the reference launches it).
extern "C" __global__ void __launch_bounds__(1024) kern_embedding_i64_bf16(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                                                          __nv_bfloat16* __restrict__ out, int tokens, int hidden) {
  const long long r = blockIdx.x;
  copy_row(out + r * hidden, table + ids[r] * hidden, 2ll * hidden);
}

// dst[r, :width] = src[r, :width] with separate row strides (in elements): one row per block.
extern "C" __global__ void __launch_bounds__(1024) kern_copy_rows_bf16(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ src,
                                                                      int dst_stride, int src_stride, int width) {
  const long long r = blockIdx.x;
  copy_row(dst + r * dst_stride, src + r * src_stride, 2ll * width);
}

// dst[0, :width] = src[rows - 1, :width].
extern "C" __global__ void __launch_bounds__(1024) kern_last_row_bf16(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ src,
                                                                     int src_stride, int width, int rows) {
  if (blockIdx.x != 0) return;
  copy_row(dst, src + (long long)(rows - 1) * src_stride, 2ll * width);
}

// dst[j] = src[min(blocks[rank] + j, rows - 1)]: a rank's slice whose first row is a run-time plan entry; one row
// per block.
extern "C" __global__ void __launch_bounds__(1024) kern_own_rows(void* __restrict__ dst, const void* __restrict__ src, const int* __restrict__ blocks,
                                                                int rank, int row_bytes, int rows) {
  const long long j = blockIdx.x;
  const long long r = min((long long)blocks[rank] + j, (long long)rows - 1);
  copy_row(static_cast<char*>(dst) + j * row_bytes, static_cast<const char*>(src) + r * row_bytes, row_bytes);
}

#ifndef K3G_CUBIN_ONLY
K3G_API int k3g_rank_rows(void* dst, const void* src, int rank, int own, int row_bytes, int rows, void* stream) {
  K3G_REQUIRE_PTR(dst); K3G_REQUIRE_PTR(src);
  K3G_REQUIRE(rank >= 0 && own >= 0 && row_bytes > 0 && rows > 0, K3G_ESHAPE);
  if (own == 0) return K3G_OK;
  kern_k3_rank_rows<<<own, 256, 0, k3g_stream(stream)>>>(dst, src, rank, own, row_bytes, rows);
  return k3g_launch_status();
}

K3G_API int k3g_zero_rows(void* buf, int row_bytes, int from, int to, void* stream) {
  K3G_REQUIRE_PTR(buf);
  K3G_REQUIRE(row_bytes > 0 && from >= 0, K3G_ESHAPE);
  if (to <= from) return K3G_OK;
  const long long nbytes = (long long)(to - from) * row_bytes;
  long long blocks = (nbytes / 16 + 255) / 256;
  blocks = blocks < 1 ? 1 : (blocks > 1184 ? 1184 : blocks);
  kern_k3_zero_rows<<<(unsigned)blocks, 256, 0, k3g_stream(stream)>>>(buf, row_bytes, from, to);
  return k3g_launch_status();
}

K3G_API int k3g_fmha_lens(const void* seq_lens, void* lens, int T, void* stream) {
  K3G_REQUIRE_PTR(seq_lens); K3G_REQUIRE_PTR(lens);
  kern_k3_fmha_lens<<<1, 32, 0, k3g_stream(stream)>>>((const int*)seq_lens, (int*)lens, T);
  return k3g_launch_status();
}

K3G_API int k3g_embedding(const void* ids, const void* table, void* out, int tokens, int hidden, void* stream) {
  K3G_REQUIRE_PTR(ids); K3G_REQUIRE_PTR(table); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE(tokens >= 0 && hidden > 0, K3G_ESHAPE);
  if (tokens == 0) return K3G_OK;
  kern_embedding_i64_bf16<<<tokens, 256, 0, k3g_stream(stream)>>>((const long long*)ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, tokens, hidden);
  return k3g_launch_status();
}

K3G_API int k3g_copy_rows(void* dst, const void* src, int dst_stride, int src_stride, int width, int rows, void* stream) {
  K3G_REQUIRE_PTR(dst); K3G_REQUIRE_PTR(src);
  K3G_REQUIRE(rows >= 0 && width > 0 && dst_stride >= width && src_stride >= width, K3G_ESHAPE);
  if (rows == 0) return K3G_OK;
  kern_copy_rows_bf16<<<rows, 256, 0, k3g_stream(stream)>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, dst_stride, src_stride, width);
  return k3g_launch_status();
}

K3G_API int k3g_last_row(void* dst, const void* src, int src_stride, int width, int rows, void* stream) {
  K3G_REQUIRE_PTR(dst); K3G_REQUIRE_PTR(src);
  K3G_REQUIRE(rows > 0 && width > 0 && src_stride >= width, K3G_ESHAPE);
  kern_last_row_bf16<<<1, 256, 0, k3g_stream(stream)>>>((__nv_bfloat16*)dst, (const __nv_bfloat16*)src, src_stride, width, rows);
  return k3g_launch_status();
}

K3G_API int k3g_own_rows(void* dst, const void* src, const void* blocks, int rank, int own, int row_bytes, int rows, void* stream) {
  K3G_REQUIRE_PTR(dst); K3G_REQUIRE_PTR(src); K3G_REQUIRE_PTR(blocks);
  K3G_REQUIRE(rank >= 0 && own >= 0 && row_bytes > 0 && rows > 0, K3G_ESHAPE);
  if (own == 0) return K3G_OK;
  kern_own_rows<<<own, 256, 0, k3g_stream(stream)>>>(dst, src, (const int*)blocks, rank, row_bytes, rows);
  return k3g_launch_status();
}
#endif  // K3G_CUBIN_ONLY
