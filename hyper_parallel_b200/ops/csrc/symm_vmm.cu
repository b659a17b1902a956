// Symmetric memory on the CUDA virtual-memory-management API, with NVLink multicast (NVLS).
//
// One rank = one process = one GPU.  Every rank creates a physical allocation that can be shared
// through a POSIX file descriptor, maps it, and maps every peer's allocation next to it (the
// descriptors travel over Unix-domain sockets on the Python side).  On machines whose GPUs sit
// behind an NVSwitch that supports multicast, the ranks additionally bind their allocations to
// ONE multicast object and map it: a `multimem.ld_reduce` on an address of that mapping returns the
// sum over all ranks of the data at the same offset (reduced inside the switch), a `multimem.st`
// writes all ranks' copies at once.
//
// All functions return 0 on success, a CUresult / cudaError code otherwise, or
//   -10 : the driver entry point is missing (driver too old),
//   -11 : the device does not support what was asked for.
// Handles are CUmemGenericAllocationHandle values passed as 64-bit integers.  Nothing here
// launches a kernel.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(fn);
}

#define HPB_DRV(var, name, ...)                                       \
  using var##_t = CUresult (*)(__VA_ARGS__);                          \
  static var##_t var = driver_fn<var##_t>(name);                      \
  if (var == nullptr) return -10

int current_device(CUdevice* dev) {
  int ordinal = 0;
  cudaError_t e = cudaGetDevice(&ordinal);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaFree(nullptr);   // make sure the primary context exists on this thread
  HPB_DRV(p_cuDeviceGet, "cuDeviceGet", CUdevice*, int);
  return static_cast<int>(p_cuDeviceGet(dev, ordinal));
}

CUmemAllocationProp alloc_prop(CUdevice dev) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, size_t bytes, size_t align, CUdevice dev, void** out) {
  HPB_DRV(p_reserve, "cuMemAddressReserve", CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  HPB_DRV(p_map, "cuMemMap", CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  HPB_DRV(p_access, "cuMemSetAccess", CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  HPB_DRV(p_free, "cuMemAddressFree", CUdeviceptr, size_t);
  HPB_DRV(p_unmap, "cuMemUnmap", CUdeviceptr, size_t);
  CUdeviceptr va = 0;
  CUresult r = p_reserve(&va, bytes, align, 0, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  r = p_map(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    p_free(va, bytes);
    return static_cast<int>(r);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = p_access(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    p_unmap(va, bytes);
    p_free(va, bytes);
    return static_cast<int>(r);
  }
  *out = reinterpret_cast<void*>(va);
  return 0;
}

}  // namespace

// *vmm = 1 when shareable VMM allocations can be made on the current device, *multicast = 1 when
// the device also supports NVLink multicast objects.
extern "C" int hpb_vmm_supported(int* vmm, int* multicast) {
  *vmm = 0;
  *multicast = 0;
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_attr, "cuDeviceGetAttribute", int*, CUdevice_attribute, CUdevice);
  int v = 0;
  if (p_attr(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS) *vmm = v;
  v = 0;
  if (p_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) *multicast = v;
  return 0;
}

// Allocation granularity that satisfies both the memory allocator and (when n_devices > 1 and
// multicast != 0) a multicast object over n_devices GPUs.
extern "C" int hpb_vmm_granularity(int n_devices, int multicast, size_t* out) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_gran, "cuMemGetAllocationGranularity", size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUmemAllocationProp prop = alloc_prop(dev);
  size_t g = 0;
  CUresult r = p_gran(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  if (multicast && n_devices > 1) {
    HPB_DRV(p_mcgran, "cuMulticastGetGranularity", size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = n_devices;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    r = p_mcgran(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) return static_cast<int>(r);
    if (mg > g) g = mg;
  }
  *out = g;
  return 0;
}

// Create `bytes` (a multiple of the granularity) of zeroed device memory on the current device,
// map it, and export it as a file descriptor.
extern "C" int hpb_vmm_alloc(size_t bytes, size_t granularity, void** ptr, unsigned long long* handle, int* fd) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_create, "cuMemCreate", CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  HPB_DRV(p_release, "cuMemRelease", CUmemGenericAllocationHandle);
  HPB_DRV(p_export, "cuMemExportToShareableHandle", void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
          unsigned long long);
  CUmemAllocationProp prop = alloc_prop(dev);
  CUmemGenericAllocationHandle h;
  CUresult r = p_create(&h, bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  rc = map_rw(h, bytes, granularity, dev, ptr);
  if (rc) {
    p_release(h);
    return rc;
  }
  cudaError_t e = cudaMemset(*ptr, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  int out_fd = -1;
  r = p_export(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *handle = static_cast<unsigned long long>(h);
  *fd = out_fd;
  return 0;
}

// Map a peer's allocation (received as a file descriptor) into this process for the current device.
extern "C" int hpb_vmm_import(int fd, size_t bytes, size_t granularity, void** ptr, unsigned long long* handle) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_import, "cuMemImportFromShareableHandle", CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  HPB_DRV(p_release, "cuMemRelease", CUmemGenericAllocationHandle);
  CUmemGenericAllocationHandle h;
  CUresult r = p_import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  rc = map_rw(h, bytes, granularity, dev, ptr);
  if (rc) {
    p_release(h);
    return rc;
  }
  *handle = static_cast<unsigned long long>(h);
  return 0;
}

// Unmap a mapping made by hpb_vmm_alloc / hpb_vmm_import / hpb_mc_map and drop its handle.
extern "C" int hpb_vmm_unmap(void* ptr, size_t bytes, unsigned long long handle) {
  HPB_DRV(p_unmap, "cuMemUnmap", CUdeviceptr, size_t);
  HPB_DRV(p_free, "cuMemAddressFree", CUdeviceptr, size_t);
  HPB_DRV(p_release, "cuMemRelease", CUmemGenericAllocationHandle);
  CUresult r = CUDA_SUCCESS;
  if (ptr != nullptr) {
    r = p_unmap(reinterpret_cast<CUdeviceptr>(ptr), bytes);
    CUresult r2 = p_free(reinterpret_cast<CUdeviceptr>(ptr), bytes);
    if (r == CUDA_SUCCESS) r = r2;
  }
  if (handle != 0) {
    CUresult r3 = p_release(static_cast<CUmemGenericAllocationHandle>(handle));
    if (r == CUDA_SUCCESS) r = r3;
  }
  return static_cast<int>(r);
}

// Create a multicast object for n_devices GPUs and `bytes` per GPU; export it as a file descriptor.
extern "C" int hpb_mc_create(int n_devices, size_t bytes, unsigned long long* mc, int* fd) {
  HPB_DRV(p_create, "cuMulticastCreate", CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  HPB_DRV(p_export, "cuMemExportToShareableHandle", void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
          unsigned long long);
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = n_devices;
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  CUresult r = p_create(&h, &mp);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  int out_fd = -1;
  r = p_export(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *mc = static_cast<unsigned long long>(h);
  *fd = out_fd;
  return 0;
}

extern "C" int hpb_mc_import(int fd, unsigned long long* mc) {
  HPB_DRV(p_import, "cuMemImportFromShareableHandle", CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUmemGenericAllocationHandle h;
  CUresult r = p_import(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *mc = static_cast<unsigned long long>(h);
  return 0;
}

// Every rank adds its device; all devices must have been added before any rank binds memory.
extern "C" int hpb_mc_add_device(unsigned long long mc) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_add, "cuMulticastAddDevice", CUmemGenericAllocationHandle, CUdevice);
  return static_cast<int>(p_add(static_cast<CUmemGenericAllocationHandle>(mc), dev));
}

// Bind this rank's allocation [0, bytes) to the multicast object at offset 0 and map the object.
extern "C" int hpb_mc_bind_map(unsigned long long mc, unsigned long long mem_handle, size_t bytes, size_t granularity,
                               void** mc_ptr) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_bind, "cuMulticastBindMem", CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t,
          size_t, unsigned long long);
  CUresult r = p_bind(static_cast<CUmemGenericAllocationHandle>(mc), 0,
                      static_cast<CUmemGenericAllocationHandle>(mem_handle), 0, bytes, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  return map_rw(static_cast<CUmemGenericAllocationHandle>(mc), bytes, granularity, dev, mc_ptr);
}

// Undo hpb_mc_bind_map on this rank: unmap the multicast mapping, unbind this device's memory.
extern "C" int hpb_mc_unbind(unsigned long long mc, void* mc_ptr, size_t bytes) {
  CUdevice dev;
  int rc = current_device(&dev);
  if (rc) return rc;
  HPB_DRV(p_unmap, "cuMemUnmap", CUdeviceptr, size_t);
  HPB_DRV(p_free, "cuMemAddressFree", CUdeviceptr, size_t);
  HPB_DRV(p_unbind, "cuMulticastUnbind", CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  HPB_DRV(p_release, "cuMemRelease", CUmemGenericAllocationHandle);
  CUresult r = CUDA_SUCCESS;
  if (mc_ptr != nullptr) {
    r = p_unmap(reinterpret_cast<CUdeviceptr>(mc_ptr), bytes);
    p_free(reinterpret_cast<CUdeviceptr>(mc_ptr), bytes);
  }
  CUresult r2 = p_unbind(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0, bytes);
  if (r == CUDA_SUCCESS) r = r2;
  p_release(static_cast<CUmemGenericAllocationHandle>(mc));
  return static_cast<int>(r);
}
