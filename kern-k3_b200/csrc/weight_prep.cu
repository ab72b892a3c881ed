// Load-time derived tables: what the checkpoint does not hold and the prefill kernels read as pointers.  Run
// once after load; element-wise, so the only design rule is a grid-stride loop that is correct for any launch.
//
// Replaces, behind the same entry names and parameter lists, xiaguan/kern-k3
//   source/k3_weight_prep.cu   kern_fill_bf16 (:32)  kern_k3_conv_taps (:37)  kern_k3_scoring (:48)  kern_k3_wsm (:54)
//                              kern_k3_mega_sf_pack (:71)  kern_k3_kvb_aug (:81)
//   source/weight_prep.cu      kern_weight_p1_bf16_f32 (:24)  kern_cast_bf16_f32 (:29)  kern_rope_table_bf16 (:34)
//                              kern_fill_f32 / _i32 / _i64 / _u8 (:47-65)  kern_iota_i32 (:67)
//
// The tables feed kernels of this library: the conv taps block [3][4][inner] is what kern_k3_span_gather reads,
// the scoring vector sw = norm * proj what the attention-residual mix reads, the [256, h] small-projection block
// what produces the beta / flow inputs, the cos | sin table what RoPE reads.
#include "k3g_device.cuh"
#include "k3g_host.h"

using namespace k3g;

namespace {
__device__ __forceinline__ long long gtid() { return (long long)blockIdx.x * blockDim.x + threadIdx.x; }
__device__ __forceinline__ long long gsize() { return (long long)gridDim.x * blockDim.x; }
}  // namespace

#define K3G_FILL_KERNEL(NAME, T, VT, EXPR)                                                       \
  extern "C" __global__ void NAME(T* __restrict__ p, int n, VT v) {                              \
    for (long long i = gtid(); i < n; i += gsize()) p[i] = EXPR;                                 \
  }
K3G_FILL_KERNEL(kern_fill_bf16, __nv_bfloat16, float, __float2bfloat16_rn(v))
K3G_FILL_KERNEL(kern_fill_f32, float, float, v)
K3G_FILL_KERNEL(kern_fill_i32, int, int, v)
K3G_FILL_KERNEL(kern_fill_i64, long long, long long, v)
K3G_FILL_KERNEL(kern_fill_u8, unsigned char, int, (unsigned char)v)

// p[i * stride] = start + i * step.
extern "C" __global__ void kern_iota_i32(int* __restrict__ p, int n, int start, int step, int stride) {
  for (long long i = gtid(); i < n; i += gsize()) p[i * stride] = start + (int)i * step;
}

// out[i] = f32(w[i]) + 1 (the "1 + weight" norm convention, exact in f32) and the plain widening cast.
extern "C" __global__ void kern_weight_p1_bf16_f32(const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int n) {
  for (long long i = gtid(); i < n; i += gsize()) out[i] = __fadd_rn(__bfloat162float(w[i]), 1.0f);
}
extern "C" __global__ void kern_cast_bf16_f32(const __nv_bfloat16* __restrict__ w, float* __restrict__ out, int n) {
  for (long long i = gtid(); i < n; i += gsize()) out[i] = __bfloat162float(w[i]);
}

// cos / sin [rows][stride] (first `half` columns of each row): inv = 1 / base^(2 j / (2 half)), angle = r * inv, all in
// f32, landed to bf16.  The reference launches one block per row; any grid / block covers all (r, j) here.
extern "C" __global__ void kern_rope_table_bf16(__nv_bfloat16* __restrict__ cos_t, __nv_bfloat16* __restrict__ sin_t, int rows, int half,
                                                int stride, float base) {
  const long long total = (long long)rows * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gsize()) {
    const int r = (int)(i / half), j = (int)(i - (long long)r * half);
    const float inv = 1.0f / powf(base, (float)(2 * j) / (float)(2 * half));
    const float angle = (float)r * inv;
    cos_t[(long long)r * stride + j] = __float2bfloat16_rn(cosf(angle));
    sin_t[(long long)r * stride + j] = __float2bfloat16_rn(sinf(angle));
  }
}

// cw[s][t][j] = w_s[j][t]: the three conv1d weights [inner][4] f32 transposed into the taps block.  A thread owns one
// channel j: one 16-byte load per stream, four coalesced 4-byte stores.
extern "C" __global__ void kern_k3_conv_taps(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                             float* __restrict__ cw, int inner) {
  const float* w[3] = {q, k, v};
  for (long long j = gtid(); j < inner; j += gsize()) {
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(w[s]) + j);
      cw[(s * 4 + 0) * (long long)inner + j] = t.x;
      cw[(s * 4 + 1) * (long long)inner + j] = t.y;
      cw[(s * 4 + 2) * (long long)inner + j] = t.z;
      cw[(s * 4 + 3) * (long long)inner + j] = t.w;
    }
  }
}

// sw[j] = f32(norm[j]) * f32(proj[j]): the folded attention-residual scoring vector.
extern "C" __global__ void kern_k3_scoring(const __nv_bfloat16* __restrict__ norm, const __nv_bfloat16* __restrict__ proj, float* __restrict__ sw,
                                           int n) {
  for (long long j = gtid(); j < n; j += gsize()) sw[j] = __fmul_rn(__bfloat162float(norm[j]), __bfloat162float(proj[j]));
}

// The KDA small-projection block [256, h]: rows 0..heads = b_proj, rows 96..224 = f_a_proj, the rest zero.
extern "C" __global__ void kern_k3_wsm(const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ f_a, __nv_bfloat16* __restrict__ wsm,
                                       int heads, int h) {
  const long long total = 256ll * h;
  for (long long i = gtid(); i < total; i += gsize()) {
    const int r = (int)(i / h), c = (int)(i - (long long)r * h);
    wsm[i] = r < heads ? b[(long long)r * h + c] : (r >= 96 && r < 224) ? f_a[(long long)(r - 96) * h + c] : __float2bfloat16_rn(0.f);
  }
}

// Scale bytes [experts][n][kg] -> one i32 per (expert, 4 k-groups, row), laid out [experts][kg / 4][n]: row r reads source
// row (r / 128) * 128 + (r % 4) * 32 + (r % 128) / 4, and for a gate | up matrix the halves interleaved by 8 on top.
extern "C" __global__ void kern_k3_mega_sf_pack(const unsigned char* __restrict__ raw, int* __restrict__ out, int experts, int n, int kg,
                                                int interleave) {
  const int words = kg / 4;
  const long long total = (long long)experts * words * n;
  for (long long i = gtid(); i < total; i += gsize()) {
    const int r = (int)(i % n), w = (int)(i / n % words);
    const long long e = i / n / words;
    const int u = (r / 128) * 128 + (r % 4) * 32 + (r % 128) / 4;
    const int sr = interleave ? (((u >> 3) & 1) ? n / 2 : 0) + (u >> 4) * 8 + (u & 7) : u;
    const unsigned char* s = raw + (e * n + sr) * kg + w * 4;
    out[i] = (int)((unsigned)s[0] | ((unsigned)s[1] << 8) | ((unsigned)s[2] << 16) | ((unsigned)s[3] << 24));
  }
}

// The MLA expansion weight [heads * 320, 576] from kv_b_proj [heads * 256, 512]: per head 128 rows of W_UK, 64 rows that
// select the latent row's rope part (identity onto columns 512..575), 128 rows of W_UV; every row padded to 576 with zeros.
extern "C" __global__ void kern_k3_kvb_aug(const __nv_bfloat16* __restrict__ w_kv_b, __nv_bfloat16* __restrict__ out, int n) {
  for (long long i = gtid(); i < n; i += gsize()) {
    const int r = (int)(i / 576), c = (int)(i - (long long)r * 576), h = r / 320, d = r - h * 320;
    __nv_bfloat16 v = __float2bfloat16_rn(0.f);
    if (d < 128 || d >= 192) {
      if (c < 512) v = w_kv_b[((long long)h * 256 + (d < 128 ? d : d - 64)) * 512 + c];
    } else if (c == 512 + (d - 128)) {
      v = __float2bfloat16_rn(1.f);
    }
    out[i] = v;
  }
}

#ifndef K3G_CUBIN_ONLY
static inline unsigned prep_grid(long long n) {
  long long b = (n + 255) / 256;
  return (unsigned)(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

// kind: 0 bf16 (value v), 1 f32 (v), 2 i32 ((int)iv), 3 i64 (iv), 4 u8 ((unsigned char)iv).
K3G_API int k3g_fill(void* p, long long n, int kind, float v, long long iv, void* stream) {
  K3G_REQUIRE_PTR(p);
  K3G_REQUIRE(n >= 0 && n < (1ll << 31) && kind >= 0 && kind <= 4, K3G_ESHAPE);
  if (n == 0) return K3G_OK;
  cudaStream_t st = k3g_stream(stream);
  switch (kind) {
    case 0: kern_fill_bf16<<<prep_grid(n), 256, 0, st>>>((__nv_bfloat16*)p, (int)n, v); break;
    case 1: kern_fill_f32<<<prep_grid(n), 256, 0, st>>>((float*)p, (int)n, v); break;
    case 2: kern_fill_i32<<<prep_grid(n), 256, 0, st>>>((int*)p, (int)n, (int)iv); break;
    case 3: kern_fill_i64<<<prep_grid(n), 256, 0, st>>>((long long*)p, (int)n, iv); break;
    default: kern_fill_u8<<<prep_grid(n), 256, 0, st>>>((unsigned char*)p, (int)n, (int)iv); break;
  }
  return k3g_launch_status();
}

K3G_API int k3g_iota_i32(void* p, int n, int start, int step, int stride, void* stream) {
  K3G_REQUIRE_PTR(p);
  K3G_REQUIRE(n >= 0 && stride > 0, K3G_ESHAPE);
  if (n == 0) return K3G_OK;
  kern_iota_i32<<<prep_grid(n), 256, 0, k3g_stream(stream)>>>((int*)p, n, start, step, stride);
  return k3g_launch_status();
}

K3G_API int k3g_cast_bf16_f32(const void* w, void* out, int n, int plus_one, void* stream) {
  K3G_REQUIRE_PTR(w); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE(n >= 0, K3G_ESHAPE);
  if (n == 0) return K3G_OK;
  if (plus_one) kern_weight_p1_bf16_f32<<<prep_grid(n), 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)w, (float*)out, n);
  else kern_cast_bf16_f32<<<prep_grid(n), 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)w, (float*)out, n);
  return k3g_launch_status();
}

K3G_API int k3g_rope_table(void* cos_t, void* sin_t, int rows, int half, int stride, float base, void* stream) {
  K3G_REQUIRE_PTR(cos_t); K3G_REQUIRE_PTR(sin_t);
  K3G_REQUIRE(rows >= 0 && half > 0 && stride >= half && base > 0.f, K3G_ESHAPE);
  if (rows == 0) return K3G_OK;
  kern_rope_table_bf16<<<prep_grid((long long)rows * half), 256, 0, k3g_stream(stream)>>>((__nv_bfloat16*)cos_t, (__nv_bfloat16*)sin_t, rows, half,
                                                                                        stride, base);
  return k3g_launch_status();
}

K3G_API int k3g_conv_taps(const void* q, const void* k, const void* v, void* cw, int inner, void* stream) {
  K3G_REQUIRE_PTR(q); K3G_REQUIRE_PTR(k); K3G_REQUIRE_PTR(v); K3G_REQUIRE_PTR(cw);
  K3G_REQUIRE_ALIGNED(q); K3G_REQUIRE_ALIGNED(k); K3G_REQUIRE_ALIGNED(v);
  K3G_REQUIRE(inner > 0, K3G_ESHAPE);
  kern_k3_conv_taps<<<prep_grid(inner), 256, 0, k3g_stream(stream)>>>((const float*)q, (const float*)k, (const float*)v, (float*)cw, inner);
  return k3g_launch_status();
}

K3G_API int k3g_scoring(const void* norm, const void* proj, void* sw, int n, void* stream) {
  K3G_REQUIRE_PTR(norm); K3G_REQUIRE_PTR(proj); K3G_REQUIRE_PTR(sw);
  K3G_REQUIRE(n >= 0, K3G_ESHAPE);
  if (n == 0) return K3G_OK;
  kern_k3_scoring<<<prep_grid(n), 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)norm, (const __nv_bfloat16*)proj, (float*)sw, n);
  return k3g_launch_status();
}

K3G_API int k3g_wsm(const void* b, const void* f_a, void* wsm, int heads, int h, void* stream) {
  K3G_REQUIRE_PTR(b); K3G_REQUIRE_PTR(f_a); K3G_REQUIRE_PTR(wsm);
  K3G_REQUIRE(heads >= 0 && heads <= 96 && h > 0, K3G_ESHAPE);
  kern_k3_wsm<<<prep_grid(256ll * h), 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)b, (const __nv_bfloat16*)f_a, (__nv_bfloat16*)wsm, heads, h);
  return k3g_launch_status();
}

K3G_API int k3g_mega_sf_pack(const void* raw, void* out, int experts, int n, int kg, int interleave, void* stream) {
  K3G_REQUIRE_PTR(raw); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE(experts >= 0 && n > 0 && n % 128 == 0 && kg > 0 && kg % 4 == 0 && (!interleave || n % 16 == 0), K3G_ESHAPE);
  const long long total = (long long)experts * (kg / 4) * n;
  if (total == 0) return K3G_OK;
  kern_k3_mega_sf_pack<<<prep_grid(total), 256, 0, k3g_stream(stream)>>>((const unsigned char*)raw, (int*)out, experts, n, kg, interleave);
  return k3g_launch_status();
}

K3G_API int k3g_kvb_aug(const void* w_kv_b, void* out, int heads, void* stream) {
  K3G_REQUIRE_PTR(w_kv_b); K3G_REQUIRE_PTR(out);
  K3G_REQUIRE(heads > 0 && (long long)heads * 320 * 576 < (1ll << 31), K3G_ESHAPE);
  const int n = heads * 320 * 576;
  kern_k3_kvb_aug<<<prep_grid(n), 256, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)w_kv_b, (__nv_bfloat16*)out, n);
  return k3g_launch_status();
}
#endif  // K3G_CUBIN_ONLY
