#include "symm_heap.h"
#include "host_common.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstring>
#include <unistd.h>

namespace mesh {
namespace {

// Driver entry points are looked up through the runtime so the library has no link-time
// dependency on libcuda (it must load on machines without a driver).
template <typename Fn>
Fn driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

#define DRV(name) \
  static auto fn_##name = driver_fn<decltype(&name)>(#name); \
  if (!fn_##name) return set_error(-100, "driver entry point " #name " not available")

#define DRV_OK(call, what)                                                   \
  do {                                                                       \
    CUresult _r = (call);                                                    \
    if (_r != CUDA_SUCCESS) return set_error(-200 - (int)_r, "%s failed: CUresult %d", what, (int)_r); \
  } while (0)

int ensure_context(int device) {
  MESH_CUDA_OK(cudaSetDevice(device));
  MESH_CUDA_OK(cudaFree(0));
  return 0;
}

CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_rw(CUmemGenericAllocationHandle h, uint64_t size, int device, uint64_t* ptr_out) {
  DRV(cuMemAddressReserve);
  DRV(cuMemMap);
  DRV(cuMemSetAccess);
  DRV(cuMemAddressFree);
  CUdeviceptr va = 0;
  DRV_OK(fn_cuMemAddressReserve(&va, size, 0, 0, 0), "cuMemAddressReserve");
  CUresult r = fn_cuMemMap(va, size, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    fn_cuMemAddressFree(va, size);
    return set_error(-200 - (int)r, "cuMemMap failed: CUresult %d", (int)r);
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV_OK(fn_cuMemSetAccess(va, size, &acc, 1), "cuMemSetAccess");
  *ptr_out = (uint64_t)va;
  return 0;
}

}  // namespace
}  // namespace mesh

using namespace mesh;

extern "C" int mesh_vmm_granularity(int device, int multicast, int world, uint64_t* out) {
  if (int rc = ensure_context(device)) return rc;
  size_t g = 0;
  if (multicast) {
    DRV(cuMulticastGetGranularity);
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = 1 << 21;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    DRV_OK(fn_cuMulticastGetGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
  } else {
    DRV(cuMemGetAllocationGranularity);
    CUmemAllocationProp prop = alloc_prop(device);
    DRV_OK(fn_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
           "cuMemGetAllocationGranularity");
  }
  *out = g;
  return 0;
}

extern "C" int mesh_vmm_alloc(uint64_t size, int device, MeshVmmBlock* out) {
  if (int rc = ensure_context(device)) return rc;
  DRV(cuMemCreate);
  DRV(cuMemExportToShareableHandle);
  DRV(cuMemRelease);
  CUmemAllocationProp prop = alloc_prop(device);
  CUmemGenericAllocationHandle h;
  DRV_OK(fn_cuMemCreate(&h, size, &prop, 0), "cuMemCreate");
  int fd = -1;
  CUresult r = fn_cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    fn_cuMemRelease(h);
    return set_error(-200 - (int)r, "cuMemExportToShareableHandle failed: CUresult %d", (int)r);
  }
  uint64_t ptr = 0;
  if (int rc = map_rw(h, size, device, &ptr)) {
    close(fd);
    fn_cuMemRelease(h);
    return rc;
  }
  out->handle = (uint64_t)h;
  out->ptr = ptr;
  out->size = size;
  out->fd = fd;
  out->device = device;
  return 0;
}

extern "C" int mesh_vmm_import(int fd, uint64_t size, int device, MeshVmmBlock* out) {
  if (int rc = ensure_context(device)) return rc;
  DRV(cuMemImportFromShareableHandle);
  DRV(cuMemRelease);
  CUmemGenericAllocationHandle h;
  DRV_OK(fn_cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
         "cuMemImportFromShareableHandle");
  uint64_t ptr = 0;
  if (int rc = map_rw(h, size, device, &ptr)) {
    fn_cuMemRelease(h);
    return rc;
  }
  out->handle = (uint64_t)h;
  out->ptr = ptr;
  out->size = size;
  out->fd = -1;
  out->device = device;
  return 0;
}

extern "C" int mesh_vmm_free(MeshVmmBlock* blk) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMemRelease);
  if (blk->ptr) {
    fn_cuMemUnmap((CUdeviceptr)blk->ptr, blk->size);
    fn_cuMemAddressFree((CUdeviceptr)blk->ptr, blk->size);
  }
  if (blk->handle) fn_cuMemRelease((CUmemGenericAllocationHandle)blk->handle);
  if (blk->fd >= 0) close(blk->fd);
  memset(blk, 0, sizeof(*blk));
  blk->fd = -1;
  return 0;
}

extern "C" int mesh_mc_supported(int device) {
  int v = 0;
  DRV(cuDeviceGetAttribute);
  if (fn_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v;
}

extern "C" int mesh_mc_create(uint64_t size, int world, uint64_t* mc_handle, int* fd) {
  DRV(cuMulticastCreate);
  DRV(cuMemExportToShareableHandle);
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = world;
  mp.size = size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  DRV_OK(fn_cuMulticastCreate(&h, &mp), "cuMulticastCreate");
  DRV_OK(fn_cuMemExportToShareableHandle(fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
         "cuMemExportToShareableHandle(multicast)");
  *mc_handle = (uint64_t)h;
  return 0;
}

extern "C" int mesh_mc_import(int fd, uint64_t* mc_handle) {
  DRV(cuMemImportFromShareableHandle);
  CUmemGenericAllocationHandle h;
  DRV_OK(fn_cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
         "cuMemImportFromShareableHandle(multicast)");
  *mc_handle = (uint64_t)h;
  return 0;
}

extern "C" int mesh_mc_add_device(uint64_t mc_handle, int device) {
  DRV(cuMulticastAddDevice);
  DRV_OK(fn_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc_handle, device), "cuMulticastAddDevice");
  return 0;
}

extern "C" int mesh_mc_bind_map(uint64_t mc_handle, uint64_t local_handle, uint64_t size, int device,
                                uint64_t* mc_ptr) {
  DRV(cuMulticastBindMem);
  DRV_OK(fn_cuMulticastBindMem((CUmemGenericAllocationHandle)mc_handle, 0,
                               (CUmemGenericAllocationHandle)local_handle, 0, size, 0),
         "cuMulticastBindMem");
  return map_rw((CUmemGenericAllocationHandle)mc_handle, size, device, mc_ptr);
}

extern "C" int mesh_mc_unmap(uint64_t mc_handle, uint64_t mc_ptr, uint64_t size, int device) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMulticastUnbind);
  DRV(cuMemRelease);
  if (mc_ptr) {
    fn_cuMemUnmap((CUdeviceptr)mc_ptr, size);
    fn_cuMemAddressFree((CUdeviceptr)mc_ptr, size);
  }
  fn_cuMulticastUnbind((CUmemGenericAllocationHandle)mc_handle, device, 0, size);
  fn_cuMemRelease((CUmemGenericAllocationHandle)mc_handle);
  return 0;
}

extern "C" int mesh_ipc_alloc(uint64_t size, int device, uint64_t* ptr, unsigned char handle_out[64]) {
  MESH_CUDA_OK(cudaSetDevice(device));
  void* p = nullptr;
  MESH_CUDA_OK(cudaMalloc(&p, size));
  MESH_CUDA_OK(cudaMemset(p, 0, size));
  cudaIpcMemHandle_t h;
  MESH_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle_out, &h, 64);
  *ptr = (uint64_t)p;
  return 0;
}

extern "C" int mesh_ipc_open(const unsigned char handle[64], int device, uint64_t* ptr) {
  MESH_CUDA_OK(cudaSetDevice(device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  MESH_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = (uint64_t)p;
  return 0;
}

extern "C" int mesh_ipc_close(uint64_t ptr) {
  MESH_CUDA_OK(cudaIpcCloseMemHandle((void*)ptr));
  return 0;
}
extern "C" int mesh_ipc_free(uint64_t ptr) {
  MESH_CUDA_OK(cudaFree((void*)ptr));
  return 0;
}

extern "C" int mesh_can_access_peer(int device, int peer) {
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, device, peer) != cudaSuccess) return 0;
  return can;
}

extern "C" int mesh_enable_peer_access(int device, int peer) {
  MESH_CUDA_OK(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  MESH_CUDA_OK(e);
  return 0;
}
