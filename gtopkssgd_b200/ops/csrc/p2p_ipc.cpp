// Peer-to-peer substrate: device allocations that other processes on the same
// NVSwitch box can map (CUDA IPC), so that the exchange kernels can store
// straight into a partner GPU's receive slots.  The reference stages every
// sparse message through host numpy buffers and MPI (allreducer.py:432-456);
// nothing here touches the host after set-up.
//
// Set-up only: these calls allocate, export, import and release.  They are
// never on the per-iteration path.
#include <cuda_runtime.h>
#include <cstring>
#include "host_api.h"

extern "C" {

// Allocates `bytes` of zeroed device memory on the current device with
// cudaMalloc (IPC handles need a whole cudaMalloc allocation).
int gtk_p2p_alloc(unsigned long long bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return GTK_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    return GTK_ERR_CUDA;
  }
  *out = p;
  return GTK_OK;
}

int gtk_p2p_free(void* p) { return cudaFree(p) == cudaSuccess ? GTK_OK : GTK_ERR_CUDA; }

unsigned int gtk_p2p_handle_bytes(void) { return (unsigned int)sizeof(cudaIpcMemHandle_t); }

// Exports the allocation as an opaque handle (64 bytes) for other processes.
int gtk_p2p_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return GTK_ERR_CUDA;
  std::memcpy(handle_out, &h, sizeof(h));
  return GTK_OK;
}

// Maps a peer's allocation into this process; peer access is enabled lazily.
int gtk_p2p_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return GTK_ERR_CUDA;
  *out = p;
  return GTK_OK;
}

int gtk_p2p_unmap(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? GTK_OK : GTK_ERR_CUDA; }

// Same-process peers (several GPUs driven by one process, used by tests):
// enable direct access from the current device to `peer_device`.
int gtk_p2p_enable_peer(int peer_device) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return GTK_ERR_CUDA;
  if (dev == peer_device) return GTK_OK;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess) return GTK_ERR_CUDA;
  if (!can) return GTK_ERR_UNSUPPORTED;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return GTK_OK;
  }
  return e == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

}  // extern "C"
