// Native symmetric heap: one physical allocation per rank, mapped into every peer of the node and
// (optionally) bound to an NVSwitch multicast object, built on the driver's virtual-memory API.
//
// Role in the reference: nvls/symmetric_memory.py:41-60, 133-184 gets a symmetric buffer, its peer
// pointers and the multicast pointer from torch.distributed._symmetric_memory.  The kernels of this
// library consume nothing but raw addresses (McbCtx), so the allocator can be replaced: this file is
// the allocator without PyTorch.  Host code only; the driver library is opened at run time, so the
// shared object still loads on a machine without a GPU driver.
//
// Protocol (driven from Python, parallel/symm_heap.py):
//   every rank   mcb_nheap_create      physical memory (shareable as a POSIX file descriptor), local mapping
//   rank 0       mcb_nheap_mc_create   multicast object for `world` devices, exported as a file descriptor
//   ... the file descriptors travel over unix sockets (SCM_RIGHTS) ...
//   every rank   mcb_nheap_map_peer    import a peer's allocation and map it
//   every rank   mcb_nheap_mc_import   (not rank 0) import the multicast object
//   every rank   mcb_nheap_mc_add_device, host barrier, mcb_nheap_mc_bind (bind + map), host barrier
//   every rank   mcb_nheap_destroy     unbind, unmap, release (after a host barrier: nobody still uses the peers)
// Every call returns 0 or a driver error code and writes the failing call's name into `err`.
#include <cuda.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

namespace {

struct Driver {
  void* lib = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  bool ok = false;
};

template <typename F>
bool sym(void* lib, const char* name, F& f) {
  f = reinterpret_cast<F>(dlsym(lib, name));
  return f != nullptr;
}

Driver& driver() {
  static Driver d;
  static bool tried = false;
  if (tried) return d;
  tried = true;
  d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!d.lib) return d;
  bool ok = true;
  ok &= sym(d.lib, "cuGetErrorString", d.GetErrorString);
  ok &= sym(d.lib, "cuDeviceGet", d.DeviceGet);
  ok &= sym(d.lib, "cuDeviceGetAttribute", d.DeviceGetAttribute);
  ok &= sym(d.lib, "cuMemGetAllocationGranularity", d.MemGetAllocationGranularity);
  ok &= sym(d.lib, "cuMemCreate", d.MemCreate);
  ok &= sym(d.lib, "cuMemRelease", d.MemRelease);
  ok &= sym(d.lib, "cuMemAddressReserve", d.MemAddressReserve);
  ok &= sym(d.lib, "cuMemAddressFree", d.MemAddressFree);
  ok &= sym(d.lib, "cuMemMap", d.MemMap);
  ok &= sym(d.lib, "cuMemUnmap", d.MemUnmap);
  ok &= sym(d.lib, "cuMemSetAccess", d.MemSetAccess);
  ok &= sym(d.lib, "cuMemExportToShareableHandle", d.MemExportToShareableHandle);
  ok &= sym(d.lib, "cuMemImportFromShareableHandle", d.MemImportFromShareableHandle);
  ok &= sym(d.lib, "cuMulticastCreate", d.MulticastCreate);
  ok &= sym(d.lib, "cuMulticastAddDevice", d.MulticastAddDevice);
  ok &= sym(d.lib, "cuMulticastBindMem", d.MulticastBindMem);
  ok &= sym(d.lib, "cuMulticastUnbind", d.MulticastUnbind);
  ok &= sym(d.lib, "cuMulticastGetGranularity", d.MulticastGetGranularity);
  d.ok = ok;
  return d;
}

struct Mapping {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr va = 0;
  bool mapped = false;
};

struct NativeHeap {
  int device = 0;
  CUdevice cu_device = 0;
  size_t size = 0;                       // rounded up to the allocation (and multicast) granularity
  Mapping local;
  std::vector<Mapping> peers;
  CUmemGenericAllocationHandle mc = 0;   // multicast object
  bool mc_added = false, mc_bound = false;
  Mapping mc_map;                        // mapping of the multicast object (handle field unused)
};

int fail(CUresult r, const char* what, char* err, int errlen) {
  if (err && errlen > 0) {
    const char* s = nullptr;
    Driver& d = driver();
    if (d.GetErrorString) d.GetErrorString(r, &s);
    snprintf(err, (size_t)errlen, "%s: %s (%d)", what, s ? s : "unknown error", (int)r);
  }
  return r == CUDA_SUCCESS ? -1 : (int)r;
}

#define DRV(call, name)                                         \
  do {                                                          \
    CUresult r_ = (call);                                       \
    if (r_ != CUDA_SUCCESS) return fail(r_, name, err, errlen); \
  } while (0)

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

CUmulticastObjectProp mc_prop(int world, size_t size) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = (unsigned int)world;
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int map_handle(NativeHeap* h, Mapping& m, char* err, int errlen) {
  Driver& d = driver();
  DRV(d.MemAddressReserve(&m.va, h->size, 0, 0, 0), "cuMemAddressReserve");
  CUresult r = d.MemMap(m.va, h->size, 0, m.handle, 0);
  if (r != CUDA_SUCCESS) {
    d.MemAddressFree(m.va, h->size);
    m.va = 0;
    return fail(r, "cuMemMap", err, errlen);
  }
  m.mapped = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV(d.MemSetAccess(m.va, h->size, &acc, 1), "cuMemSetAccess");
  return 0;
}

void unmap(NativeHeap* h, Mapping& m, bool release) {
  Driver& d = driver();
  if (m.mapped) d.MemUnmap(m.va, h->size);
  if (m.va) d.MemAddressFree(m.va, h->size);
  if (release && m.handle) d.MemRelease(m.handle);
  m = Mapping();
}

}  // namespace

extern "C" {

// 1 when the driver library and every entry point used here were found.
int mcb_nheap_available() { return driver().ok ? 1 : 0; }

// 1 when `device` supports multicast objects (NVSwitch), 0 when not, negative on error.
int mcb_nheap_multicast_supported(int device) {
  Driver& d = driver();
  if (!d.ok) return -1;
  CUdevice dev;
  if (d.DeviceGet(&dev, device) != CUDA_SUCCESS) return -1;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return -1;
  return v;
}

// Physical memory on `device` (the calling thread's current context must be that device's), mapped locally.
// `world` > 1 with `multicast` != 0 rounds the size to the multicast granularity as well.  Outputs: the
// heap object, the rounded size, the local address and a file descriptor other processes can import.
int mcb_nheap_create(int device, unsigned long long nbytes, int world, int multicast, void** out_heap,
                     unsigned long long* out_size, unsigned long long* out_ptr, int* out_fd, char* err, int errlen) {
  Driver& d = driver();
  if (!d.ok) return fail(CUDA_ERROR_NOT_INITIALIZED, "libcuda.so.1 (driver library or an entry point missing)", err, errlen);
  if (!out_heap || !out_size || !out_ptr || !out_fd || nbytes == 0 || world < 1) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  NativeHeap* h = new NativeHeap();
  h->device = device;
  CUresult r = d.DeviceGet(&h->cu_device, device);
  if (r != CUDA_SUCCESS) { delete h; return fail(r, "cuDeviceGet", err, errlen); }
  CUmemAllocationProp prop = alloc_prop(device);
  size_t gran = 0;
  r = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS || gran == 0) { delete h; return fail(r, "cuMemGetAllocationGranularity", err, errlen); }
  if (multicast && world > 1) {
    CUmulticastObjectProp mp = mc_prop(world, (size_t)nbytes);
    size_t mg = 0;
    r = d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS || mg == 0) { delete h; return fail(r, "cuMulticastGetGranularity", err, errlen); }
    if (mg > gran) gran = mg;
  }
  h->size = ((size_t)nbytes + gran - 1) / gran * gran;
  r = d.MemCreate(&h->local.handle, h->size, &prop, 0);
  if (r != CUDA_SUCCESS) { delete h; return fail(r, "cuMemCreate", err, errlen); }
  int rc = map_handle(h, h->local, err, errlen);
  if (rc) { unmap(h, h->local, true); delete h; return rc; }
  int fd = -1;
  r = d.MemExportToShareableHandle(&fd, h->local.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { unmap(h, h->local, true); delete h; return fail(r, "cuMemExportToShareableHandle", err, errlen); }
  *out_heap = h;
  *out_size = h->size;
  *out_ptr = (unsigned long long)h->local.va;
  *out_fd = fd;
  return 0;
}

// Import a peer's allocation from a file descriptor received from that process and map it here.
// The descriptor stays the caller's to close.
int mcb_nheap_map_peer(void* heap, int fd, unsigned long long* out_ptr, char* err, int errlen) {
  Driver& d = driver();
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || !out_ptr || fd < 0) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  Mapping m;
  DRV(d.MemImportFromShareableHandle(&m.handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
      "cuMemImportFromShareableHandle");
  int rc = map_handle(h, m, err, errlen);
  if (rc) { unmap(h, m, true); return rc; }
  h->peers.push_back(m);
  *out_ptr = (unsigned long long)m.va;
  return 0;
}

// Rank 0: create the multicast object for `world` devices and export it.
int mcb_nheap_mc_create(void* heap, int world, int* out_fd, char* err, int errlen) {
  Driver& d = driver();
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || !out_fd || world < 2 || h->mc) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  CUmulticastObjectProp mp = mc_prop(world, h->size);
  DRV(d.MulticastCreate(&h->mc, &mp), "cuMulticastCreate");
  int fd = -1;
  DRV(d.MemExportToShareableHandle(&fd, h->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle(multicast)");
  *out_fd = fd;
  return 0;
}

// Other ranks: import the multicast object from rank 0's file descriptor.
int mcb_nheap_mc_import(void* heap, int fd, char* err, int errlen) {
  Driver& d = driver();
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || fd < 0 || h->mc) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  DRV(d.MemImportFromShareableHandle(&h->mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
      "cuMemImportFromShareableHandle(multicast)");
  return 0;
}

// Every rank, before anyone binds: add this rank's device to the object.
int mcb_nheap_mc_add_device(void* heap, char* err, int errlen) {
  Driver& d = driver();
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || !h->mc || h->mc_added) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  DRV(d.MulticastAddDevice(h->mc, h->cu_device), "cuMulticastAddDevice");
  h->mc_added = true;
  return 0;
}

// Every rank, after ALL ranks have added their device (host barrier): bind the local memory at offset 0
// and map the object; returns the multicast address.
int mcb_nheap_mc_bind(void* heap, unsigned long long* out_mc_ptr, char* err, int errlen) {
  Driver& d = driver();
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || !out_mc_ptr || !h->mc_added || h->mc_bound) return fail(CUDA_ERROR_INVALID_VALUE, "arguments", err, errlen);
  DRV(d.MulticastBindMem(h->mc, 0, h->local.handle, 0, h->size, 0), "cuMulticastBindMem");
  h->mc_bound = true;
  h->mc_map.handle = h->mc;
  int rc = map_handle(h, h->mc_map, err, errlen);
  if (rc) return rc;
  *out_mc_ptr = (unsigned long long)h->mc_map.va;
  return 0;
}

// Unbind, unmap and release everything.  Call after a host barrier (no rank may still touch a peer's
// memory or the multicast address) and with no kernel in flight.
void mcb_nheap_destroy(void* heap) {
  NativeHeap* h = static_cast<NativeHeap*>(heap);
  if (!h || !driver().ok) return;
  Driver& d = driver();
  if (h->mc_map.va) { unmap(h, h->mc_map, false); }
  if (h->mc_bound) d.MulticastUnbind(h->mc, h->cu_device, 0, h->size);
  if (h->mc) d.MemRelease(h->mc);
  for (Mapping& m : h->peers) unmap(h, m, true);
  unmap(h, h->local, true);
  delete h;
}

}  // extern "C"
