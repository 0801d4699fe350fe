// Virtual-memory-management allocations that several processes of one node can map, and NVLink
// multicast objects (NVLS) bound to them.
//
// A symmetric region for the gradient reducer is one cuMemCreate allocation per rank, exported as
// a POSIX file descriptor; every rank maps every other rank's allocation (plain peer loads and
// stores) and, where the device supports multicast, all allocations are bound to one multicast
// object whose mapping gives `multimem` instructions the in-switch reduce and broadcast.
//
// The driver entry points are resolved at run time (no link against libcuda).  File descriptors
// travel between the processes in Python (SCM_RIGHTS); this file only creates, imports, maps and
// releases.  Tear-down unmaps and unbinds before releasing so that no peer is left with a
// binding to freed memory.
//
// The reference has no counterpart: its collectives are NCCL calls
// (src/distributed/system_nccl_transport.cpp:39-46).
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/pybind11.h>
#include <unistd.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "ob/runtime.h"

namespace py = pybind11;

namespace ob {
namespace {

template <class Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  const cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    cudaGetLastError();
    throw std::runtime_error(std::string("driver entry point ") + name + " is unavailable");
  }
  return reinterpret_cast<Fn>(p);
}

struct Driver {
  CUresult (*DeviceGet)(CUdevice*, int);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char**);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);

  static Driver& get() {
    static Driver d = [] {
      Driver x;
#define OB_DRV(field, name) x.field = driver_fn<decltype(x.field)>(name)
      OB_DRV(DeviceGet, "cuDeviceGet");
      OB_DRV(DeviceGetAttribute, "cuDeviceGetAttribute");
      OB_DRV(GetErrorString, "cuGetErrorString");
      OB_DRV(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
      OB_DRV(MemCreate, "cuMemCreate");
      OB_DRV(MemRelease, "cuMemRelease");
      OB_DRV(MemExportToShareableHandle, "cuMemExportToShareableHandle");
      OB_DRV(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
      OB_DRV(MemAddressReserve, "cuMemAddressReserve");
      OB_DRV(MemAddressFree, "cuMemAddressFree");
      OB_DRV(MemMap, "cuMemMap");
      OB_DRV(MemUnmap, "cuMemUnmap");
      OB_DRV(MemSetAccess, "cuMemSetAccess");
      OB_DRV(MulticastCreate, "cuMulticastCreate");
      OB_DRV(MulticastAddDevice, "cuMulticastAddDevice");
      OB_DRV(MulticastBindMem, "cuMulticastBindMem");
      OB_DRV(MulticastUnbind, "cuMulticastUnbind");
      OB_DRV(MulticastGetGranularity, "cuMulticastGetGranularity");
#undef OB_DRV
      return x;
    }();
    return d;
  }
};

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* msg = nullptr;
  Driver::get().GetErrorString(r, &msg);
  throw std::runtime_error(std::string(what) + " failed: " + (msg ? msg : "unknown driver error") + " (" +
                           std::to_string(static_cast<int>(r)) + ")");
}

CUdevice device_of(int ordinal) {
  Runtime::instance().cuda(ordinal);  // make sure the primary context exists
  CUdevice d;
  check(Driver::get().DeviceGet(&d, ordinal), "cuDeviceGet");
  return d;
}

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

CUmulticastObjectProp multicast_prop(int world, size_t bytes) {
  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned>(world);
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  prop.flags = 0;
  return prop;
}

// One record per handle this process holds: an allocation (own or imported) with its mapping, or
// a multicast object with its mapping and the binding made by this process.
struct Record {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr va = 0;
  size_t bytes = 0;
  int device = 0;
  bool multicast = false;
  bool bound = false;  // multicast: this process bound memory of `device` at offset 0
  bool live = false;
};
std::mutex g_mu;
std::vector<Record> g_records;

int add_record(const Record& r) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_records.push_back(r);
  return static_cast<int>(g_records.size()) - 1;
}
Record& record(int id) {
  if (id < 0 || id >= static_cast<int>(g_records.size()) || !g_records[id].live) throw std::invalid_argument("unknown memory handle id");
  return g_records[id];
}

CUdeviceptr map_handle(CUmemGenericAllocationHandle h, size_t bytes, size_t align, int device) {
  Driver& d = Driver::get();
  CUdeviceptr va = 0;
  check(d.MemAddressReserve(&va, bytes, align, 0, 0), "cuMemAddressReserve");
  CUresult r = d.MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    d.MemAddressFree(va, bytes);
    check(r, "cuMemMap");
  }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d.MemSetAccess(va, bytes, &access, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap(va, bytes);
    d.MemAddressFree(va, bytes);
    check(r, "cuMemSetAccess");
  }
  return va;
}

}  // namespace

void bind_vmm(py::module_& m) {
  // {"fd_handles": bool, "multicast": bool}; never throws for a missing feature.
  m.def("_vmm_supported", [](int device) {
    py::dict out;
    out["fd_handles"] = false;
    out["multicast"] = false;
    try {
      Driver& d = Driver::get();
      const CUdevice dev = device_of(device);
      int v = 0;
      if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS)
        out["fd_handles"] = v != 0;
      v = 0;
      if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) out["multicast"] = v != 0;
    } catch (const std::exception&) {
    }
    return out;
  });
  // Size granularity that satisfies both the allocator and (if `world` > 1) multicast binding.
  m.def("_vmm_granularity", [](int device, int world, bool multicast) {
    Driver& d = Driver::get();
    device_of(device);
    const CUmemAllocationProp prop = alloc_prop(device);
    size_t g = 0;
    check(d.MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    if (multicast && world > 1) {
      const CUmulticastObjectProp mp = multicast_prop(world, g);
      size_t mg = 0;
      check(d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
      if (mg > g) g = mg;
    }
    return g;
  });
  // Zero-filled device memory shareable through a file descriptor: (id, pointer, fd).  The
  // caller closes the fd once every peer has imported it.
  m.def("_vmm_alloc", [](size_t bytes, size_t align, int device) {
    Driver& d = Driver::get();
    device_of(device);
    DeviceGuard g(device);
    const CUmemAllocationProp prop = alloc_prop(device);
    Record r;
    r.bytes = bytes;
    r.device = device;
    check(d.MemCreate(&r.handle, bytes, &prop, 0), "cuMemCreate");
    try {
      r.va = map_handle(r.handle, bytes, align, device);
    } catch (...) {
      d.MemRelease(r.handle);
      throw;
    }
    OB_CUDA(cudaMemset(reinterpret_cast<void*>(r.va), 0, bytes));
    OB_CUDA(cudaDeviceSynchronize());
    int fd = -1;
    check(d.MemExportToShareableHandle(&fd, r.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    r.live = true;
    const int id = add_record(r);
    return py::make_tuple(id, static_cast<uintptr_t>(r.va), fd);
  });
  // Maps a peer's allocation (received as an fd) for `device`: (id, pointer).
  m.def("_vmm_import", [](int fd, size_t bytes, size_t align, int device) {
    Driver& d = Driver::get();
    device_of(device);
    DeviceGuard g(device);
    Record r;
    r.bytes = bytes;
    r.device = device;
    check(d.MemImportFromShareableHandle(&r.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                         CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle");
    try {
      r.va = map_handle(r.handle, bytes, align, device);
    } catch (...) {
      d.MemRelease(r.handle);
      throw;
    }
    r.live = true;
    const int id = add_record(r);
    return py::make_tuple(id, static_cast<uintptr_t>(r.va));
  });
  // Multicast object over `world` devices: (id, fd).  One rank creates, the others import.
  m.def("_mc_create", [](int world, size_t bytes, int device) {
    Driver& d = Driver::get();
    device_of(device);
    const CUmulticastObjectProp prop = multicast_prop(world, bytes);
    Record r;
    r.bytes = bytes;
    r.device = device;
    r.multicast = true;
    check(d.MulticastCreate(&r.handle, &prop), "cuMulticastCreate");
    int fd = -1;
    const CUresult e = d.MemExportToShareableHandle(&fd, r.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (e != CUDA_SUCCESS) {
      d.MemRelease(r.handle);
      check(e, "cuMemExportToShareableHandle (multicast)");
    }
    r.live = true;
    return py::make_tuple(add_record(r), fd);
  });
  m.def("_mc_import", [](int fd, size_t bytes, int device) {
    Driver& d = Driver::get();
    device_of(device);
    Record r;
    r.bytes = bytes;
    r.device = device;
    r.multicast = true;
    check(d.MemImportFromShareableHandle(&r.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                         CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle (multicast)");
    r.live = true;
    return add_record(r);
  });
  // Every rank adds its device before any rank binds memory.
  m.def("_mc_add_device", [](int mc_id, int device) {
    std::lock_guard<std::mutex> lock(g_mu);
    Record& mc = record(mc_id);
    check(Driver::get().MulticastAddDevice(mc.handle, device_of(device)), "cuMulticastAddDevice");
  });
  // Binds this rank's allocation at offset 0 of the multicast object and maps the object:
  // returns the multicast pointer (same layout as the allocation).
  m.def("_mc_bind_map", [](int mc_id, int alloc_id, size_t align, int device) {
    std::lock_guard<std::mutex> lock(g_mu);
    Record& mc = record(mc_id);
    Record& mem = record(alloc_id);
    if (!mc.multicast || mem.multicast || mem.bytes != mc.bytes) throw std::invalid_argument("multicast bind: mismatched handles");
    DeviceGuard g(device);
    check(Driver::get().MulticastBindMem(mc.handle, 0, mem.handle, 0, mc.bytes, 0), "cuMulticastBindMem");
    mc.bound = true;
    mc.device = device;
    try {
      mc.va = map_handle(mc.handle, mc.bytes, align, device);
    } catch (...) {
      Driver::get().MulticastUnbind(mc.handle, device_of(device), 0, mc.bytes);
      mc.bound = false;
      throw;
    }
    return static_cast<uintptr_t>(mc.va);
  });
  // Unmaps everything, removes this process's multicast bindings, then releases the handles.
  m.def("_vmm_release_all", [] {
    std::lock_guard<std::mutex> lock(g_mu);
    Driver* d = nullptr;
    try {
      d = &Driver::get();
    } catch (const std::exception&) {
      g_records.clear();
      return;
    }
    for (auto& r : g_records) {
      if (!r.live) continue;
      cudaSetDevice(r.device);
      cudaDeviceSynchronize();
    }
    for (auto it = g_records.rbegin(); it != g_records.rend(); ++it) {  // multicast mappings first (created last)
      if (!it->live || !it->multicast) continue;
      if (it->va) { d->MemUnmap(it->va, it->bytes); d->MemAddressFree(it->va, it->bytes); }
      if (it->bound) {
        CUdevice dev;
        if (d->DeviceGet(&dev, it->device) == CUDA_SUCCESS) d->MulticastUnbind(it->handle, dev, 0, it->bytes);
      }
      d->MemRelease(it->handle);
      it->live = false;
    }
    for (auto it = g_records.rbegin(); it != g_records.rend(); ++it) {
      if (!it->live) continue;
      if (it->va) { d->MemUnmap(it->va, it->bytes); d->MemAddressFree(it->va, it->bytes); }
      d->MemRelease(it->handle);
      it->live = false;
    }
    g_records.clear();
  });
  m.def("_close_fd", [](int fd) { if (fd >= 0) ::close(fd); });
}

}  // namespace ob
