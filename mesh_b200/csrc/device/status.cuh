// Device-side status reporting shared by every kernel in this library.
//
// No kernel here traps, asserts or spins without a limit.  A wait that runs out,
// or a bounds/alignment check that fails in a checked build, writes one record
// into a small status block in global memory and the kernel returns normally, so
// the CUDA context stays usable and the host can read what happened.  This plays
// the role of the reference's GPU status word {behind, ahead, first}
// (rdma/mesh-metal.h:76-80) and of its ETIMEDOUT/ECANCELED host codes
// (rdma/mesh.h:15-17).
#pragma once
#include <cstdint>

namespace mesh {

enum StatusCode : int {
  MESH_OK = 0,
  MESH_TIMEOUT = 1,        // a bounded wait ran out
  MESH_CANCELED = 2,       // the abort flag was raised by the host or a peer
  MESH_STALE = 3,          // epoch (membership view) mismatch
  MESH_BOUNDS = 4,         // checked build: index outside its buffer
  MESH_ALIGN = 5,          // checked build: misaligned address or TMA coordinate
  MESH_BAD_ARGUMENT = 6,
};

// Where a wait gave up.  Kept small and stable: the host prints these names.
enum WaitSite : int {
  SITE_NONE = 0,
  SITE_SMEM_FULL = 1,      // MMA warp waiting for TMA data
  SITE_SMEM_EMPTY = 2,     // TMA warp waiting for a free stage
  SITE_TMEM_FULL = 3,      // epilogue waiting for an accumulator
  SITE_TMEM_EMPTY = 4,     // MMA warp waiting for the epilogue to drain TMEM
  SITE_PEER_FLAG = 5,      // waiting for a flag written by another GPU
  SITE_LOCAL_FLAG = 6,     // waiting for a flag written by another CTA of this GPU
  SITE_BARRIER = 7,        // cross-GPU barrier
  SITE_STORE_DRAIN = 8,    // waiting for own bulk stores
  SITE_HOST_FLAG = 9,      // waiting for a word the host writes
};

// 64 bytes; one per communicator / op stream.  `code` is written with atomicCAS so
// the first failure wins and later ones only bump `count`.
struct Status {
  int code;
  int site;
  int block;
  int thread;
  unsigned long long expected;
  unsigned long long seen;
  unsigned long long aux;
  int count;
  int abort;               // host- or peer-raised: bounded waits observe it and give up
  int epoch;               // membership view id the plan was built for
  int pad[3];
};

static_assert(sizeof(Status) == 64, "Status layout is read by the host through ctypes");

#ifdef __CUDACC__
__device__ __forceinline__ void status_record(Status* st, int code, int site,
                                              unsigned long long expected = 0,
                                              unsigned long long seen = 0,
                                              unsigned long long aux = 0) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site;
    st->block = (int)blockIdx.x;
    st->thread = (int)threadIdx.x;
    st->expected = expected;
    st->seen = seen;
    st->aux = aux;
    __threadfence_system();
  }
  atomicAdd(&st->count, 1);
}

__device__ __forceinline__ bool status_aborted(const Status* st) {
  if (st == nullptr) return false;
  return *reinterpret_cast<const volatile int*>(&st->abort) != 0;
}
#endif

}  // namespace mesh
