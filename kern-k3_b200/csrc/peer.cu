// Host-side peer-memory plumbing: the part of the reference's external runtime that this
// library has to provide itself to be usable stand-alone.
//
// The reference's runtime allocates every buffer, maps each rank's copy of an `export`ed buffer
// into the other ranks and hands kernels a device array of u64 addresses, one per rank,
// including the caller's own (xiaguan/kern-k3 scripts/gen_collectives_p2p.py:77-86).  With one
// process per GPU the same is done here with CUDA IPC: allocate with cudaMalloc, export a
// 64-byte handle, exchange handles through any host channel (the tests and the benchmark use
// torch.distributed), open the peers' handles, and upload the address table.
//
// These are set-up calls: they allocate and synchronise, unlike the op launchers.
#include "k3g_host.h"
#include <cstring>

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");

K3G_API int k3g_peer_alloc(long long bytes, void** host_out_dptr) {
  K3G_REQUIRE_PTR(host_out_dptr); K3G_REQUIRE(bytes > 0, K3G_ESHAPE);
  const cudaError_t e = cudaMalloc(host_out_dptr, (size_t)bytes);
  return e == cudaSuccess ? K3G_OK : (int)e;
}

K3G_API int k3g_peer_free(void* dptr) {
  const cudaError_t e = cudaFree(dptr);
  return e == cudaSuccess ? K3G_OK : (int)e;
}

K3G_API int k3g_peer_export(void* dptr, void* host_handle64) {
  K3G_REQUIRE_PTR(dptr); K3G_REQUIRE_PTR(host_handle64);
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, dptr);
  if (e != cudaSuccess) return (int)e;
  std::memcpy(host_handle64, &h, 64);
  return K3G_OK;
}

K3G_API int k3g_peer_open(const void* host_handle64, void** host_out_dptr) {
  K3G_REQUIRE_PTR(host_handle64); K3G_REQUIRE_PTR(host_out_dptr);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, host_handle64, 64);
  const cudaError_t e = cudaIpcOpenMemHandle(host_out_dptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? K3G_OK : (int)e;
}

K3G_API int k3g_peer_close(void* dptr) {
  const cudaError_t e = cudaIpcCloseMemHandle(dptr);
  return e == cudaSuccess ? K3G_OK : (int)e;
}

// Library and device identification: returns the SM count of the current device (148 on B200),
// or a negative K3G_E* / positive cudaError_t on failure.  host_cc receives major * 10 + minor.
K3G_API int k3g_device_sms(int* host_cc) {
  int dev = 0, sms = 0, major = 0, minor = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (e != cudaSuccess) return -(int)e - 1000;
  if (host_cc) *host_cc = major * 10 + minor;
  return sms;
}
