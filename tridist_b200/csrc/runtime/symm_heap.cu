// Symmetric heap over CUDA IPC and the mapped status block.
//
// Counterpart of the reference's symmetric memory (heap malloc/free and ptr(addr, pe) address
// translation, pydushmem/host.py:239-264) and of its raw IPC pointer list (hipMalloc + IPC handle
// exchange + open, pydushmem/ipc.py:79-116): one cudaMalloc per rank and buffer, handles exchanged
// by the host layer, every peer's copy mapped into this process. The handle exchange itself
// (the reference's MPI allgather, ipc.py:44) is done in Python over torch.distributed.
#include "symm_heap.h"

#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>

#include "../common/status.h"

namespace tdb {

static void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("tridist_b200: ") + what + ": " + cudaGetErrorString(e));
  }
}

void* symm_alloc_local(size_t bytes) {
  void* p = nullptr;
  if (bytes == 0) bytes = 256;
  check(cudaMalloc(&p, bytes), "cudaMalloc(symmetric buffer)");
  check(cudaMemset(p, 0, bytes), "cudaMemset(symmetric buffer)");
  check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  return p;
}

void symm_free_local(void* p) {
  if (p) cudaFree(p);
}

std::string symm_export_handle(void* p) {
  cudaIpcMemHandle_t h;
  check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
  return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void* symm_open_handle(const std::string& handle) {
  if (handle.size() != sizeof(cudaIpcMemHandle_t))
    throw std::runtime_error("tridist_b200: IPC handle has the wrong size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return p;
}

void symm_close_handle(void* p) {
  if (p) cudaIpcCloseMemHandle(p);
}

bool symm_enable_peer_access(int peer_device) {
  int dev = 0;
  check(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev == peer_device) return true;
  int can = 0;
  check(cudaDeviceCanAccessPeer(&can, dev, peer_device), "cudaDeviceCanAccessPeer");
  if (!can) return false;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return true;
  }
  check(e, "cudaDeviceEnablePeerAccess");
  return true;
}

MappedStatus status_alloc() {
  MappedStatus s{nullptr, nullptr};
  void* h = nullptr;
  check(cudaHostAlloc(&h, sizeof(StatusBlock), cudaHostAllocMapped | cudaHostAllocPortable),
        "cudaHostAlloc(status)");
  std::memset(h, 0, sizeof(StatusBlock));
  void* d = nullptr;
  check(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer(status)");
  s.host_ptr = reinterpret_cast<StatusBlock*>(h);
  s.dev_ptr = reinterpret_cast<StatusBlock*>(d);
  return s;
}

void status_free(MappedStatus s) {
  if (s.host_ptr) cudaFreeHost(s.host_ptr);
}

}  // namespace tdb
