// Status strings and ABI version of libhelios_b200.
#include <cstring>

#include "hk_common.cuh"

HK_API const char* hk_status_string(int status) {
  switch (status) {
    case HK_OK: return "ok";
    case HK_ERR_INVALID: return "invalid argument";
    case HK_ERR_UNSUPPORTED: return "unsupported shape";
    case HK_ERR_CUDA: return "CUDA launch error";
    case HK_ERR_WORKSPACE: return "workspace too small";
    case HK_ERR_TIMEOUT: return "bounded device wait expired";
    default: return "unknown status";
  }
}

HK_API int hk_abi_version(void) { return 1; }

// Lets kernels on the current device dereference memory of `peer_device` (buffers of another GPU that
// were mapped into this process, e.g. through CUDA IPC).  Idempotent.
HK_API int hk_enable_peer_access(int peer_device) {
  int cur = 0, n = 0;
  if (cudaGetDevice(&cur) != cudaSuccess || cudaGetDeviceCount(&n) != cudaSuccess) return HK_ERR_CUDA;
  if (peer_device < 0 || peer_device >= n) return HK_ERR_INVALID;
  if (peer_device == cur) return HK_OK;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, cur, peer_device) != cudaSuccess) return HK_ERR_CUDA;
  if (!can) return HK_ERR_UNSUPPORTED;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();   // clear the sticky "already enabled"
    return HK_OK;
  }
  return e == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

// ---- exchange regions for the multi-GPU split-KV decode (one process per GPU) -----------------------
// A region is plain device memory of the calling process's current device with an inter-process handle.
// A peer process opens the handle WITH ITS OWN DEVICE CURRENT: the mapping it gets is valid for kernels of
// that device (peer access over NVLink is enabled on demand by the open call).
HK_API int hk_peer_region_alloc(size_t bytes, void** dev_ptr, void* handle_out_64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!dev_ptr || !handle_out_64 || bytes == 0) return HK_ERR_INVALID;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return HK_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return HK_ERR_CUDA;
  }
  memcpy(handle_out_64, &h, sizeof(h));
  *dev_ptr = p;
  return HK_OK;
}

HK_API int hk_peer_region_open(const void* handle_64, void** dev_ptr) {
  if (!handle_64 || !dev_ptr) return HK_ERR_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return HK_ERR_CUDA;
  }
  *dev_ptr = p;
  return HK_OK;
}

HK_API int hk_peer_region_close(void* dev_ptr) {
  if (!dev_ptr) return HK_OK;
  return cudaIpcCloseMemHandle(dev_ptr) == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}

HK_API int hk_peer_region_free(void* dev_ptr) {
  if (!dev_ptr) return HK_OK;
  return cudaFree(dev_ptr) == cudaSuccess ? HK_OK : HK_ERR_CUDA;
}
