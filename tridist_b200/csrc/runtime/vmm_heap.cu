// See vmm_heap.h. Two driver tables behind one set of entry points: the CUDA driver's
// virtual-memory and multicast calls, and a memfd + mmap stand-in for CPU-only tests.
#include "vmm_heap.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <mutex>
#include <stdexcept>
#include <unordered_map>

namespace tdb {
namespace {

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error("tridist_b200: " + what); }

// ---------------------------------------------------------------------------------------------
// The real driver, looked up by name at run time
// ---------------------------------------------------------------------------------------------
struct Driver {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                               unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char**);
};

template <typename Fn>
void lookup(Fn& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      p == nullptr)
    fail(std::string("the CUDA driver has no ") + name);
  fn = reinterpret_cast<Fn>(p);
}

const Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    lookup(d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    lookup(d.MemCreate, "cuMemCreate");
    lookup(d.MemRelease, "cuMemRelease");
    lookup(d.MemExportToShareableHandle, "cuMemExportToShareableHandle");
    lookup(d.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    lookup(d.MemAddressReserve, "cuMemAddressReserve");
    lookup(d.MemAddressFree, "cuMemAddressFree");
    lookup(d.MemMap, "cuMemMap");
    lookup(d.MemUnmap, "cuMemUnmap");
    lookup(d.MemSetAccess, "cuMemSetAccess");
    lookup(d.MulticastCreate, "cuMulticastCreate");
    lookup(d.MulticastAddDevice, "cuMulticastAddDevice");
    lookup(d.MulticastBindMem, "cuMulticastBindMem");
    lookup(d.MulticastUnbind, "cuMulticastUnbind");
    lookup(d.MulticastGetGranularity, "cuMulticastGetGranularity");
    lookup(d.DeviceGetAttribute, "cuDeviceGetAttribute");
    lookup(d.GetErrorString, "cuGetErrorString");
  });
  return d;
}

void ok(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* msg = nullptr;
  drv().GetErrorString(r, &msg);
  fail(std::string(what) + " failed: " + (msg ? msg : "unknown driver error") + " (" + std::to_string(int(r)) + ")");
}

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) fail("cudaGetDevice failed");
  // make sure the primary context exists: the VMM calls need a current context
  cudaFree(nullptr);
  return dev;
}

CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// ---------------------------------------------------------------------------------------------
// Handle table shared by both drivers
// ---------------------------------------------------------------------------------------------
struct Entry {
  CUmemGenericAllocationHandle h = 0;   // real driver
  int fd = -1;                          // stand-in: the memfd behind the allocation
  size_t bytes = 0;
  bool multicast = false;
  int devices_added = 0, bound = 0;     // stand-in bookkeeping
};

std::mutex g_mu;
std::unordered_map<int64_t, Entry> g_handles;
int64_t g_next = 1;
bool g_fake = false;
std::vector<std::string> g_log;

int64_t put(const Entry& e) {
  std::lock_guard<std::mutex> lk(g_mu);
  const int64_t id = g_next++;
  g_handles[id] = e;
  return id;
}
Entry& get(int64_t id) {
  auto it = g_handles.find(id);
  if (it == g_handles.end()) fail("unknown VMM handle " + std::to_string(id));
  return it->second;
}
void note(const std::string& s) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_log.push_back(s);
}

}  // namespace

void vmm_use_fake_driver(bool on) { g_fake = on; }

std::vector<std::string> vmm_fake_call_log() {
  std::lock_guard<std::mutex> lk(g_mu);
  std::vector<std::string> out;
  out.swap(g_log);
  return out;
}

bool vmm_multicast_supported(std::string* why) {
  if (g_fake) return true;
  try {
    const int dev = current_device();
    int mc = 0, fd = 0, vmm = 0;
    ok(drv().DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev), "cuDeviceGetAttribute");
    ok(drv().DeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev),
       "cuDeviceGetAttribute");
    ok(drv().DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev), "cuDeviceGetAttribute");
    if (!vmm) { if (why) *why = "no virtual memory management on this device"; return false; }
    if (!fd) { if (why) *why = "allocations cannot be exported as POSIX file descriptors"; return false; }
    if (!mc) { if (why) *why = "the device / fabric does not support multicast objects"; return false; }
    return true;
  } catch (const std::exception& e) {
    if (why) *why = e.what();
    return false;
  }
}

size_t vmm_granularity(bool multicast, int num_devices) {
  if (g_fake) return 4096;
  const int dev = current_device();
  const CUmemAllocationProp prop = alloc_prop(dev);
  size_t g = 0;
  ok(drv().MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (multicast) {
    CUmulticastObjectProp mp;
    std::memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned int>(num_devices);
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    ok(drv().MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
    if (mg > g) g = mg;
  }
  return g;
}

int64_t vmm_create(size_t bytes) {
  Entry e;
  e.bytes = bytes;
  if (g_fake) {
    e.fd = memfd_create("tridist_vmm", 0);
    if (e.fd < 0 || ftruncate(e.fd, static_cast<off_t>(bytes)) != 0) fail("stand-in allocation failed");
    note("create");
    return put(e);
  }
  const int dev = current_device();
  const CUmemAllocationProp prop = alloc_prop(dev);
  ok(drv().MemCreate(&e.h, bytes, &prop, 0), "cuMemCreate");
  return put(e);
}

int vmm_export_fd(int64_t handle) {
  Entry& e = get(handle);
  if (g_fake) {
    note(e.multicast ? "mc_export" : "export");
    const int fd = dup(e.fd);
    if (fd < 0) fail("dup failed");
    return fd;
  }
  int fd = -1;
  ok(drv().MemExportToShareableHandle(&fd, e.h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
     "cuMemExportToShareableHandle");
  return fd;
}

int64_t vmm_import_fd(int fd) {
  Entry e;
  if (g_fake) {
    struct stat st;
    if (fstat(fd, &st) != 0) fail("stand-in import: bad descriptor");
    e.fd = dup(fd);
    e.bytes = static_cast<size_t>(st.st_size);
    note("import");
    return put(e);
  }
  ok(drv().MemImportFromShareableHandle(&e.h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
     "cuMemImportFromShareableHandle");
  return put(e);
}

void* vmm_map(int64_t handle, size_t bytes) {
  Entry& e = get(handle);
  if (g_fake) {
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, e.fd, 0);
    if (p == MAP_FAILED) fail("stand-in map failed");
    note(e.multicast ? "mc_map" : "map");
    return p;
  }
  const int dev = current_device();
  CUdeviceptr ptr = 0;
  ok(drv().MemAddressReserve(&ptr, bytes, 0, 0, 0), "cuMemAddressReserve");
  CUresult r = drv().MemMap(ptr, bytes, 0, e.h, 0);
  if (r != CUDA_SUCCESS) {
    drv().MemAddressFree(ptr, bytes);
    ok(r, "cuMemMap");
  }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = drv().MemSetAccess(ptr, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    drv().MemUnmap(ptr, bytes);
    drv().MemAddressFree(ptr, bytes);
    ok(r, "cuMemSetAccess");
  }
  return reinterpret_cast<void*>(ptr);
}

void vmm_unmap(void* ptr, size_t bytes) {
  if (ptr == nullptr) return;
  if (g_fake) {
    munmap(ptr, bytes);
    note("unmap");
    return;
  }
  ok(drv().MemUnmap(reinterpret_cast<CUdeviceptr>(ptr), bytes), "cuMemUnmap");
  ok(drv().MemAddressFree(reinterpret_cast<CUdeviceptr>(ptr), bytes), "cuMemAddressFree");
}

void vmm_release(int64_t handle) {
  Entry e;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_handles.find(handle);
    if (it == g_handles.end()) return;
    e = it->second;
    g_handles.erase(it);
  }
  if (g_fake) {
    if (e.multicast && e.bound > 0) fail("stand-in: a multicast object was released while memory was still bound to it");
    if (e.fd >= 0) close(e.fd);
    note(e.multicast ? "mc_release" : "release");
    return;
  }
  ok(drv().MemRelease(e.h), "cuMemRelease");
}

int64_t vmm_mc_create(size_t bytes, int num_devices) {
  Entry e;
  e.bytes = bytes;
  e.multicast = true;
  if (g_fake) {
    e.fd = memfd_create("tridist_mc", 0);
    if (e.fd < 0 || ftruncate(e.fd, static_cast<off_t>(bytes)) != 0) fail("stand-in multicast object failed");
    note("mc_create:" + std::to_string(num_devices));
    return put(e);
  }
  current_device();
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned int>(num_devices);
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  ok(drv().MulticastCreate(&e.h, &mp), "cuMulticastCreate");
  return put(e);
}

void vmm_mc_add_device(int64_t mc_handle) {
  Entry& e = get(mc_handle);
  if (g_fake) {
    e.multicast = true;              // an imported object is one too
    ++e.devices_added;
    note("mc_add_device");
    return;
  }
  const int dev = current_device();
  ok(drv().MulticastAddDevice(e.h, dev), "cuMulticastAddDevice");
}

void vmm_mc_bind(int64_t mc_handle, int64_t mem_handle, size_t bytes) {
  Entry& mc = get(mc_handle);
  Entry& mem = get(mem_handle);
  if (g_fake) {
    if (mc.devices_added < 1) fail("stand-in: bind before this device was added to the multicast object");
    ++mc.bound;
    note("mc_bind");
    return;
  }
  ok(drv().MulticastBindMem(mc.h, 0, mem.h, 0, bytes, 0), "cuMulticastBindMem");
}

void vmm_mc_unbind(int64_t mc_handle, size_t bytes) {
  Entry& mc = get(mc_handle);
  if (g_fake) {
    if (mc.bound < 1) fail("stand-in: unbind without a bind");
    --mc.bound;
    note("mc_unbind");
    return;
  }
  const int dev = current_device();
  ok(drv().MulticastUnbind(mc.h, dev, 0, bytes), "cuMulticastUnbind");
}

}  // namespace tdb
