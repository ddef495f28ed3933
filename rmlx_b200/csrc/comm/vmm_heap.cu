// Symmetric memory on the virtual-memory-management API: one physical allocation per rank and
// segment, exported as a POSIX file descriptor, imported by every peer and mapped into address
// ranges the process reserved up front, so a segment added later lands right behind the earlier
// ones on every rank and an offset into the heap means the same bytes everywhere. A segment can
// also be bound to an NVLink multicast object: stores to the multicast mapping reach every rank's
// copy, loads with `multimem.ld_reduce` return the sum over the ranks, both done by the switch.
//
// This is the transport layer underneath the heap the collectives sub-allocate from: what the
// reference does with registered RDMA memory regions and a tiered pool
// (crates/rmlx-rdma/src/mr.rs, shared_buffer.rs; crates/rmlx-alloc/src/zero_copy.rs:22-171).
//
// The driver API is reached through cudaGetDriverEntryPoint, so the library has no link-time
// dependency on libcuda (it must load on a box without a GPU).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../common/launch.cuh"
#include "../common/ptx.cuh"

namespace rb {

template <class Fn>
static Fn drv(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return reinterpret_cast<Fn>(p);
}

#define RB_DRV(var, name, type)                \
  static type var = drv<type>(name);           \
  if (!var) return -1000;

#define RB_CU(expr)                                         \
  do {                                                      \
    CUresult _r = (expr);                                   \
    if (_r != CUDA_SUCCESS) return -2000 - static_cast<int>(_r); \
  } while (0)

using PFN_create = CUresult (*)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
using PFN_release = CUresult (*)(CUmemGenericAllocationHandle);
using PFN_export = CUresult (*)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
using PFN_import = CUresult (*)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
using PFN_reserve = CUresult (*)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
using PFN_addrfree = CUresult (*)(CUdeviceptr, size_t);
using PFN_map = CUresult (*)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
using PFN_unmap = CUresult (*)(CUdeviceptr, size_t);
using PFN_setaccess = CUresult (*)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
using PFN_gran = CUresult (*)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
using PFN_mccreate = CUresult (*)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
using PFN_mcadd = CUresult (*)(CUmemGenericAllocationHandle, CUdevice);
using PFN_mcbind = CUresult (*)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
using PFN_mcunbind = CUresult (*)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
using PFN_mcgran = CUresult (*)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
using PFN_devattr = CUresult (*)(int*, CUdevice_attribute, CUdevice);

static CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace rb

using namespace rb;

// bit 0: VMM allocations exportable as file descriptors; bit 1: NVLink multicast objects.
extern "C" int rmlx_vmm_support(int dev) {
  RB_DRV(attr, "cuDeviceGetAttribute", PFN_devattr)
  int fd_ok = 0, mc_ok = 0;
  if (attr(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) != CUDA_SUCCESS) fd_ok = 0;
  if (attr(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) mc_ok = 0;
  return (fd_ok ? 1 : 0) | (mc_ok ? 2 : 0);
}

// Allocation granularity (bytes) of device `dev`; with `world` > 0 the larger of it and the
// multicast granularity for `world` devices, so that a segment can be bound later.
extern "C" long long rmlx_vmm_granularity(int dev, int world) {
  RB_DRV(gran, "cuMemGetAllocationGranularity", PFN_gran)
  const CUmemAllocationProp prop = alloc_prop(dev);
  size_t g = 0;
  RB_CU(gran(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  if (world > 0) {
    RB_DRV(mcgran, "cuMulticastGetGranularity", PFN_mcgran)
    CUmulticastObjectProp mp = {};
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    RB_CU(mcgran(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
    if (mg > g) g = mg;
  }
  return static_cast<long long>(g);
}

// Physical memory on `dev` (bytes: a multiple of the granularity) and its shareable descriptor.
extern "C" int rmlx_vmm_create(int dev, unsigned long long bytes, unsigned long long* handle, int* fd) {
  RB_DRV(create, "cuMemCreate", PFN_create)
  RB_DRV(exp, "cuMemExportToShareableHandle", PFN_export)
  const CUmemAllocationProp prop = alloc_prop(dev);
  CUmemGenericAllocationHandle h;
  RB_CU(create(&h, bytes, &prop, 0));
  int f = -1;
  RB_CU(exp(&f, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *handle = h;
  *fd = f;
  return 0;
}

extern "C" int rmlx_vmm_import(int fd, unsigned long long* handle) {
  RB_DRV(imp, "cuMemImportFromShareableHandle", PFN_import)
  CUmemGenericAllocationHandle h;
  RB_CU(imp(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  *handle = h;
  return 0;
}

extern "C" int rmlx_vmm_release(unsigned long long handle) {
  RB_DRV(rel, "cuMemRelease", PFN_release)
  RB_CU(rel(handle));
  return 0;
}

extern "C" int rmlx_vmm_reserve(unsigned long long bytes, unsigned long long align, unsigned long long* va) {
  RB_DRV(res, "cuMemAddressReserve", PFN_reserve)
  CUdeviceptr p = 0;
  RB_CU(res(&p, bytes, align, 0, 0));
  *va = p;
  return 0;
}

extern "C" int rmlx_vmm_address_free(unsigned long long va, unsigned long long bytes) {
  RB_DRV(fr, "cuMemAddressFree", PFN_addrfree)
  RB_CU(fr(va, bytes));
  return 0;
}

// Map `handle` (a memory or a multicast handle) at `va` and give device `dev` read-write access.
extern "C" int rmlx_vmm_map(unsigned long long va, unsigned long long bytes, unsigned long long handle, int dev) {
  RB_DRV(map, "cuMemMap", PFN_map)
  RB_DRV(acc, "cuMemSetAccess", PFN_setaccess)
  RB_CU(map(va, bytes, 0, handle, 0));
  CUmemAccessDesc d = {};
  d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  d.location.id = dev;
  d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  RB_CU(acc(va, bytes, &d, 1));
  return 0;
}

extern "C" int rmlx_vmm_unmap(unsigned long long va, unsigned long long bytes) {
  RB_DRV(un, "cuMemUnmap", PFN_unmap)
  RB_CU(un(va, bytes));
  return 0;
}

// Zero `bytes` at `va` on the current device and wait for it.
extern "C" int rmlx_vmm_memset(unsigned long long va, unsigned long long bytes) {
  RB_CHECK(cudaMemset(reinterpret_cast<void*>(static_cast<uintptr_t>(va)), 0, bytes));
  RB_CHECK(cudaDeviceSynchronize());
  return 0;
}

// ---- NVLink multicast ----------------------------------------------------------------------------
// One rank creates the object and shares its descriptor; every rank imports it (rmlx_vmm_import),
// adds its device, and only after ALL ranks have added theirs binds its own memory at offset 0.
extern "C" int rmlx_mc_create(int world, unsigned long long bytes, unsigned long long* handle, int* fd) {
  RB_DRV(mc, "cuMulticastCreate", PFN_mccreate)
  RB_DRV(exp, "cuMemExportToShareableHandle", PFN_export)
  CUmulticastObjectProp mp = {};
  mp.numDevices = static_cast<unsigned>(world);
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  RB_CU(mc(&h, &mp));
  int f = -1;
  RB_CU(exp(&f, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *handle = h;
  *fd = f;
  return 0;
}

extern "C" int rmlx_mc_add_device(unsigned long long mc_handle, int dev) {
  RB_DRV(add, "cuMulticastAddDevice", PFN_mcadd)
  RB_CU(add(mc_handle, dev));
  return 0;
}

extern "C" int rmlx_mc_bind(unsigned long long mc_handle, unsigned long long mem_handle, unsigned long long bytes) {
  RB_DRV(bind, "cuMulticastBindMem", PFN_mcbind)
  RB_CU(bind(mc_handle, 0, mem_handle, 0, bytes, 0));
  return 0;
}

extern "C" int rmlx_mc_unbind(unsigned long long mc_handle, int dev, unsigned long long bytes) {
  RB_DRV(unbind, "cuMulticastUnbind", PFN_mcunbind)
  RB_CU(unbind(mc_handle, dev, 0, bytes));
  return 0;
}
