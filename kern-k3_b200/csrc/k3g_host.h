// Host-side conventions of the C ABI: error codes, argument checks, launch check.
//
// Every exported launcher returns 0 on success, a negative K3G_E* code when an argument is
// rejected before anything is launched, or a positive cudaError_t when the launch itself
// failed.  Launchers never allocate, never synchronise and are safe to call while the
// stream is being captured into a CUDA graph (the calling runtime of the reference replays
// its whole program as one graph per rank).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#define K3G_OK 0
#define K3G_ENULL (-1)    /* a required pointer is null */
#define K3G_ESHAPE (-2)   /* a size is not supported (row width, world size, count alignment) */
#define K3G_EALIGN (-3)   /* a pointer is not 16-byte aligned */
#define K3G_ERANGE (-4)   /* an index argument is out of range (rank, slot, nb, order) */
#define K3G_ELIMIT (-5)   /* a size exceeds a built-in maximum */

#define K3G_API extern "C" __attribute__((visibility("default")))

#define K3G_REQUIRE_PTR(p) do { if ((p) == nullptr) return K3G_ENULL; } while (0)
#define K3G_REQUIRE_ALIGNED(p) do { if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return K3G_EALIGN; } while (0)
#define K3G_REQUIRE(cond, code) do { if (!(cond)) return (code); } while (0)

static inline int k3g_launch_status() {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? K3G_OK : (int)e;
}

static inline cudaStream_t k3g_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
