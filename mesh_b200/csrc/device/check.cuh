// Checked build: index and alignment checks inside the kernels.
//
// Compiled with -DMESH_CHECK=1 (the library `libmesh_b200_check.so`, chosen at load time by MESH_CHECK=1), every
// MESH_CHECK_INDEX / MESH_CHECK_ALIGNED below tests its condition; a failed check writes one MESH_BOUNDS or MESH_ALIGN
// record {expected = limit, seen = value, aux = source line} into the status block and evaluates to false, and the
// kernel skips the access it guards.  Nothing traps and nothing asserts: the context stays usable and the host reads
// the record after the step.  In the regular build both macros are the constant `true` and cost nothing.  This is the
// stand-in for a memory checker on machines where none may run.  The checks sit where an index comes from data (a
// routing table, a peer's header, a tile descriptor built on the device) rather than from the launch geometry.
#pragma once
#include "status.cuh"

namespace mesh {

constexpr int SITE_CHECK = 10;

#if defined(MESH_CHECK) && MESH_CHECK
__device__ __forceinline__ bool check_index(long long i, long long n, Status* st, int line) {
  if (i >= 0 && i < n) return true;
  status_record(st, MESH_BOUNDS, SITE_CHECK, (unsigned long long)n, (unsigned long long)i, (unsigned long long)line);
  return false;
}
__device__ __forceinline__ bool check_aligned(unsigned long long v, unsigned long long align, Status* st, int line) {
  if ((v % align) == 0) return true;
  status_record(st, MESH_ALIGN, SITE_CHECK, align, v, (unsigned long long)line);
  return false;
}
#define MESH_CHECK_INDEX(i, n, st) (::mesh::check_index((long long)(i), (long long)(n), (st), __LINE__))
#define MESH_CHECK_ALIGNED(v, a, st) (::mesh::check_aligned((unsigned long long)(v), (unsigned long long)(a), (st), __LINE__))
#define MESH_CHECKED_BUILD 1
#else
#define MESH_CHECK_INDEX(i, n, st) (true)
#define MESH_CHECK_ALIGNED(v, a, st) (true)
#define MESH_CHECKED_BUILD 0
#endif

}  // namespace mesh
