// Symmetric heap: one equally sized device allocation per GPU, mapped into every peer of the
// node, plus (optionally) an NVLS multicast mapping of the same physical memory.
//
// This is the NVLink counterpart of the reference's shared region and registered wire window
// (rdma/mesh.h:173-228, rdma/mesh-verbs.h:94-109): buffers at compiler-fixed offsets that a peer
// can store into directly, and signal words next to them.  Allocation uses the CUDA virtual
// memory management API so that the handle can be exported as a POSIX file descriptor and bound
// to a multicast object; the Python side passes the descriptors between ranks over Unix sockets.
// A plain cudaMalloc + cudaIpc fallback exists for drivers where VMM export is not permitted.
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct MeshVmmBlock {
  uint64_t handle;     // CUmemGenericAllocationHandle
  uint64_t ptr;        // mapped device virtual address
  uint64_t size;       // rounded-up size
  int fd;              // exported POSIX fd (-1 when imported or not exportable)
  int device;
} MeshVmmBlock;

// Granularity (bytes) that sizes are rounded to; multicast=1 asks for the multicast granularity.
int mesh_vmm_granularity(int device, int multicast, int world, uint64_t* out);
// Allocate `size` bytes of device memory on `device`, map it read/write and export an fd.
int mesh_vmm_alloc(uint64_t size, int device, MeshVmmBlock* out);
// Map a peer's allocation (received as an fd) into this process for `device`.
int mesh_vmm_import(int fd, uint64_t size, int device, MeshVmmBlock* out);
int mesh_vmm_free(MeshVmmBlock* blk);

// NVLS: rank 0 creates the multicast object and exports it; everyone imports (rank 0 passes fd=-1 and
// its own handle), adds its device, and after a barrier binds its local block and maps the object.
int mesh_mc_supported(int device);
int mesh_mc_create(uint64_t size, int world, uint64_t* mc_handle, int* fd);
int mesh_mc_import(int fd, uint64_t* mc_handle);
int mesh_mc_add_device(uint64_t mc_handle, int device);
int mesh_mc_bind_map(uint64_t mc_handle, uint64_t local_handle, uint64_t size, int device, uint64_t* mc_ptr);
int mesh_mc_unmap(uint64_t mc_handle, uint64_t mc_ptr, uint64_t size, int device);

// Legacy IPC fallback (64-byte opaque handles that travel through the rendezvous store).
int mesh_ipc_alloc(uint64_t size, int device, uint64_t* ptr, unsigned char handle_out[64]);
int mesh_ipc_open(const unsigned char handle[64], int device, uint64_t* ptr);
int mesh_ipc_close(uint64_t ptr);
int mesh_ipc_free(uint64_t ptr);

int mesh_can_access_peer(int device, int peer);
int mesh_enable_peer_access(int device, int peer);

#ifdef __cplusplus
}
#endif
