// Virtual-memory symmetric allocations and NVSwitch multicast objects, straight on the CUDA
// driver's VMM calls: cuMemCreate / cuMemExportToShareableHandle (POSIX file descriptors) /
// cuMemImportFromShareableHandle / cuMemAddressReserve / cuMemMap / cuMemSetAccess for the
// per-rank buffers that every peer maps, and cuMulticastCreate / cuMulticastAddDevice /
// cuMulticastBindMem for the multicast object whose mapping the kernels address with
// multimem.ld_reduce / multimem.st.
//
// Role in the stack: the reference's symmetric heap hands out buffers that exist at a
// translatable address on every PE (heap malloc / ptr(addr, pe), pydushmem/host.py:239-264); here
// a buffer is one physical allocation per rank, mapped by all ranks, plus one multicast mapping
// that names all ranks' copies at once. The exchange of the file descriptors between the
// processes (Unix-domain sockets) is done by the Python layer (tridist_b200/parallel/vmm.py);
// this file owns the driver calls only.
//
// Every driver call goes through a table of function pointers. The table is either the real
// driver (looked up at run time, so the library needs no link-time dependency on libcuda) or an
// in-process stand-in built on memfd + mmap, which lets the handle exchange, the call order and
// the teardown rules be tested by CPU processes without any GPU.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace tdb {

// Selects the stand-in driver (true) or the real one (false) for all calls below.
void vmm_use_fake_driver(bool on);
// The stand-in's call log, oldest first ("create", "export", "import", "map", "mc_create",
// "mc_add_device", "mc_bind", "mc_unbind", "unmap", "release", ...); cleared by the call.
std::vector<std::string> vmm_fake_call_log();

// True if the current device (real driver) can take part in multicast objects and export POSIX
// file-descriptor handles. `why` names what is missing otherwise.
bool vmm_multicast_supported(std::string* why);

// Allocation size granularity on the current device: a size passed to vmm_create /
// vmm_mc_create must be a multiple of it (covers both the allocation and, if `multicast`, the
// multicast object's recommended granularity for `num_devices` devices).
size_t vmm_granularity(bool multicast, int num_devices);

// A physical allocation on the current device (zero-filled once mapped by vmm_map_local).
// Returns an opaque handle id.
int64_t vmm_create(size_t bytes);
// A file descriptor that another process can turn into a handle with vmm_import; the caller owns
// (and closes) the descriptor.
int vmm_export_fd(int64_t handle);
int64_t vmm_import_fd(int fd);
// Maps the allocation behind `handle` (own or imported) into this process with read / write
// access for the current device; returns the address.
void* vmm_map(int64_t handle, size_t bytes);
void vmm_unmap(void* ptr, size_t bytes);
void vmm_release(int64_t handle);

// Multicast object for `num_devices` devices and `bytes` bytes; created by ONE process, exported
// as a file descriptor to the others (vmm_export_fd / vmm_import_fd work on it too).
int64_t vmm_mc_create(size_t bytes, int num_devices);
// Every process: adds its current device. All processes must have done so before any of them binds.
void vmm_mc_add_device(int64_t mc_handle);
// Binds this process's physical allocation `mem_handle` at offset 0 of the multicast object.
void vmm_mc_bind(int64_t mc_handle, int64_t mem_handle, size_t bytes);
// Unbinds this device's memory again; every process does this, after all of them stopped using
// the multicast mapping and before any of them releases its memory or exits.
void vmm_mc_unbind(int64_t mc_handle, size_t bytes);

}  // namespace tdb
