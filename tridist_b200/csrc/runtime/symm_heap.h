// Symmetric heap: every rank allocates a buffer of the same size, exports it as
// a CUDA IPC handle, and maps every peer's buffer into its own address space.
// Kernels then address any rank's copy with plain loads/stores over NVLink.
//
// This replaces the reference's DUSHMEM heap (`malloc` / `ptr(addr, pe)` address
// translation, pydushmem/host.py:239-264) and its raw IPC pointer list
// (pydushmem/ipc.py:79-116). The handle exchange itself is done by the Python
// layer over torch.distributed; this file only owns the CUDA calls.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace tdb {

struct StatusBlock;

// Raw device allocation (cudaMalloc, 256-byte aligned, zero-filled).
void* symm_alloc_local(size_t bytes);
void symm_free_local(void* p);

// 64-byte opaque IPC handle of a pointer returned by symm_alloc_local.
std::string symm_export_handle(void* p);
// Maps a peer's allocation; the returned pointer is valid in this process only.
void* symm_open_handle(const std::string& handle);
void symm_close_handle(void* p);

// Enables peer access from the current device to `peer_device` (no-op if the
// two indices are equal or access is already on). Returns false if the pair
// cannot reach each other.
bool symm_enable_peer_access(int peer_device);

// Pinned, device-mapped host block for error records. host_ptr/dev_ptr alias.
struct MappedStatus {
  StatusBlock* host_ptr;
  StatusBlock* dev_ptr;
};
MappedStatus status_alloc();
void status_free(MappedStatus s);

}  // namespace tdb
