// Per-tensor bf16 -> E4M3 quantisation for callers that cannot hand over a workspace.
//
// k3g_quant_fp8_tensor (quant.cu) needs a caller-allocated `partials` buffer between its two
// launches.  Some hosts of this library have no way to provide one: a manifest-driven runtime
// that carved up all of its device memory when the program was loaded and has no workspace entry
// for this op, or a serving process that forbids cudaMalloc after start-up because the call
// synchronises the whole device.  For them this file offers the same operation with the
// workspace inside the library: a fixed, file-scope device array.
//
// Consequences of that choice, all documented at the entry point:
//   * the array exists once per GPU that loads the library and lives until the process exits;
//   * its size is a compile-time maximum (2048 block maxima = 8 KB), larger grids are refused;
//   * every call on a device shares it, so two calls whose kernels overlap on that GPU race;
//   * the first call on each device looks the array's address up (a host-side set-up step) and keeps it
//     for the life of the process, so the device's primary context must live that long too.
#include "k3g_device.cuh"
#include "k3g_host.h"

#include <mutex>

using namespace k3g;

#define K3G_STATIC_PARTIALS 2048
#define K3G_NA_THREADS 256
#define K3G_NA_MAX_DEVICES 64

// The workspace.  In host code this name is only a stand-in for the symbol, not a device address:
// the address every launch uses comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float k3g_static_partials[K3G_STATIC_PARTIALS];

namespace {

__device__ __forceinline__ unsigned na_block_max(unsigned m) {
  __shared__ unsigned s[K3G_NA_THREADS / 32];
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
  __syncthreads();
  unsigned r = 0;
#pragma unroll
  for (int w = 0; w < K3G_NA_THREADS / 32; ++w) r = max(r, s[w]);
  __syncthreads();
  return r;
}

// Same arithmetic as kern_quant_fp8_amax_v2 / kern_quant_fp8_apply_v2: exact maximum of the bf16
// magnitudes, scale = amax / 448 (1 when amax is 0), y = e4m3(x * (1 / scale)).
__global__ void __launch_bounds__(K3G_NA_THREADS) na_amax_kernel(const __nv_bfloat16* __restrict__ x, int n, float* __restrict__ partials) {
  const uint4* p = reinterpret_cast<const uint4*>(x);
  const int nv = n >> 3;
  unsigned m = 0;
  for (int i = blockIdx.x * K3G_NA_THREADS + threadIdx.x; i < nv; i += gridDim.x * K3G_NA_THREADS) {
    const uint4 v = p[i];
    const unsigned a[4] = {v.x & 0x7fff7fffu, v.y & 0x7fff7fffu, v.z & 0x7fff7fffu, v.w & 0x7fff7fffu};
#pragma unroll
    for (int j = 0; j < 4; ++j) m = max(m, max(a[j] & 0xffffu, a[j] >> 16));
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) m = max(m, (unsigned)__bfloat16_as_ushort(x[nv * 8 + threadIdx.x]) & 0x7fffu);
  m = na_block_max(m);
  if (threadIdx.x == 0) partials[blockIdx.x] = __uint_as_float(m << 16);   // every launched block writes its own slot
}

__global__ void __launch_bounds__(K3G_NA_THREADS) na_apply_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, int n,
                                                                  const float* __restrict__ partials, int nb, float* __restrict__ scale_out) {
  unsigned m = 0;
  for (int b = threadIdx.x; b < nb; b += K3G_NA_THREADS) m = max(m, __float_as_uint(partials[b]));
  const float amax = __uint_as_float(na_block_max(m));
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = scale;
  const float inv = __fdiv_rn(1.f, scale);
  const int nv = n >> 3;
  for (int i = nv - 1 - (blockIdx.x * K3G_NA_THREADS + threadIdx.x); i >= 0; i -= gridDim.x * K3G_NA_THREADS) {
    const V8 v = ld_stream(x + (size_t)i * 8);
    unsigned q0, q1;
    quant8(v, inv, q0, q1);
    st_stream8(y + (size_t)i * 8, q0, q1);
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
    const int i = nv * 8 + threadIdx.x;
    y[i] = (uint8_t)(e4m3x2(__fmul_rn(__bfloat162float(x[i]), inv), 0.f) & 0xffu);
  }
}

std::mutex g_setup_lock;
float* g_partials_addr[K3G_NA_MAX_DEVICES];   // device address of the workspace, per device ordinal

// Once per device, with that device current: resolve the symbol to its device address.
int workspace_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= K3G_NA_MAX_DEVICES) return K3G_ELIMIT;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (g_partials_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, k3g_static_partials);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
    g_partials_addr[dev] = ptr;
  }
  *out = g_partials_addr[dev];
  return K3G_OK;
}

}  // namespace

// Per-tensor E4M3 quantisation without a caller workspace and without any allocation.
//
//   x [n] bf16 -> y [n] E4M3 codes, scale_out[0] = amax / 448 (1 when the tensor is all zero);
//   results are identical to k3g_quant_fp8_tensor with the same `grid`.
//
// Who this is for: hosts that cannot allocate at call time (see the top of this file).  What it
// costs:
//   * `grid` (blocks per launch = block maxima kept between the two launches) is limited to 2048;
//     a larger value is refused with K3G_ELIMIT before anything is launched;
//   * the 8 KB workspace is a static device array: each GPU the library is loaded on keeps it until
//     the process exits;
//   * all calls on one GPU use the same array.  A call overwrites every slot it later reads, so
//     back-to-back calls on one stream are fine and nothing needs clearing; two calls whose kernels
//     can run at the same time on one GPU (different streams, different host threads) race and
//     must be serialised by the caller;
//   * the first call on each device does a one-time host-side set-up (it looks up the device
//     address of the workspace, with that device current).  Make that first call before starting
//     any stream capture.  The address is cached per device ordinal until the process exits: a
//     process that destroys the device's primary context and creates a new one (cudaDeviceReset, a
//     test harness that tears contexts down) must not call this entry point again on that device,
//     because the cached address belongs to the context that is gone.
// The function itself calls no cudaMalloc / cudaFree and no allocating library routine.
K3G_API int k3g_quant_fp8_tensor_noalloc(const void* x, void* y, void* scale_out, int n, int grid, void* stream) {
  K3G_REQUIRE_PTR(x); K3G_REQUIRE_PTR(y);
  K3G_REQUIRE_ALIGNED(x); K3G_REQUIRE(((uintptr_t)y & 7) == 0, K3G_EALIGN);
  K3G_REQUIRE(n >= 0 && grid > 0, K3G_ESHAPE);
  K3G_REQUIRE(grid <= K3G_STATIC_PARTIALS, K3G_ELIMIT);
  float* partials = nullptr;
  if (int rc = workspace_for_current_device(&partials)) return rc;
  na_amax_kernel<<<grid, K3G_NA_THREADS, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, n, partials);
  na_apply_kernel<<<grid, K3G_NA_THREADS, 0, k3g_stream(stream)>>>((const __nv_bfloat16*)x, (uint8_t*)y, n, partials, grid, (float*)scale_out);
  return k3g_launch_status();
}
