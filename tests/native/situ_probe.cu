// TEST INFRASTRUCTURE -- not part of the shipped library.
//
// Evaluates the SiTU activation element-wise with the kernels' formula (literal = 0) or with the reference's
// formula written out operation for operation (literal = 1, xiaguan/kern-k3 source/k3_land_fused.cu:88-92),
// both taken from the library's own header, so that a test can prove on a GPU that the two agree bit for bit
// on all 2^32 pairs of bf16 inputs.  Built into tests/native/libk3g_probe.so by tests/native/build_probe.py.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "situ_math.cuh"

__global__ void __launch_bounds__(256) situ_probe_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                                         __nv_bfloat16* __restrict__ out, long long n, int literal) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gf = __bfloat162float(g[i]), uf = __bfloat162float(u[i]);
    out[i] = __float2bfloat16_rn(literal ? k3g::situ_reference_form(gf, uf) : k3g::situ_value(gf, uf));
  }
}

// out[i] = bf16(SiTU(g[i], u[i])), i < n.  Returns 0, -1 (null pointer), -2 (n < 0) or a cudaError_t.
extern "C" __attribute__((visibility("default"))) int k3g_test_situ_probe(const void* g, const void* u, void* out, long long n, int literal,
                                                                           void* stream) {
  if (!g || !u || !out) return -1;
  if (n < 0) return -2;
  if (n == 0) return 0;
  const long long blocks = (n + 255) / 256;
  situ_probe_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u,
                                                                                                (__nv_bfloat16*)out, n, literal);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}
