// Words shared by the host and a CUDA stream: the stream itself can wait for a word to reach a value and can write a
// value when it gets there, with no kernel involved (cuStreamWaitValue32 / cuStreamWriteValue32).  This is the
// host <-> device half of the reference's host publish / arrived / wait on plan words
// (rdma/mesh-collective.c:17-90): the host publishes by storing to pinned memory, work queued behind a stream wait
// starts when the store lands, and the host learns that the stream got past a point from a stream write.
// Values only grow (the comparison is >=), like every other counter in this library.
#include <cuda.h>
#include <cuda_runtime.h>
#include <mutex>

#include "host_common.h"

namespace mesh {
namespace {

typedef CUresult (*WaitFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
typedef CUresult (*WriteFn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
WaitFn g_wait = nullptr;
WriteFn g_write = nullptr;

bool lookup() {
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_wait = (WaitFn)p;
    p = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_write = (WriteFn)p;
  });
  return g_wait != nullptr && g_write != nullptr;
}

// device-side address of a pinned host word (or of device memory, unchanged)
int device_address(const void* word, CUdeviceptr* out) {
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, word);
  if (e != cudaSuccess) return set_error((int)e, "host word: %s", cudaGetErrorString(e));
  if (at.type == cudaMemoryTypeHost || at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) {
    *out = (CUdeviceptr)(at.devicePointer ? at.devicePointer : word);
    return 0;
  }
  return set_error(-2, "host word: the word must live in pinned host memory or device memory");
}

}  // namespace
}  // namespace mesh

using namespace mesh;

// Everything queued on `stream` after this call waits until *word >= value (32-bit, wrap-aware signed difference).
extern "C" int mesh_stream_wait_value(void* stream, const void* word, unsigned int value) {
  if (((uintptr_t)word & 3) != 0) return set_error(-2, "host word: the word must be 4-byte aligned");
  if (!lookup()) return set_error(-100, "stream memory operations are not available from this driver");
  cudaFree(nullptr);                         // a context is current on this thread
  CUdeviceptr p;
  if (int rc = device_address(word, &p)) return rc;
  CUresult r = g_wait((CUstream)stream, p, value, CU_STREAM_WAIT_VALUE_GEQ);
  return r == CUDA_SUCCESS ? 0 : set_error(-101, "cuStreamWaitValue32 failed: CUresult %d", (int)r);
}

// The stream stores `value` into *word once everything queued before this call has finished.
extern "C" int mesh_stream_write_value(void* stream, void* word, unsigned int value) {
  if (((uintptr_t)word & 3) != 0) return set_error(-2, "host word: the word must be 4-byte aligned");
  if (!lookup()) return set_error(-100, "stream memory operations are not available from this driver");
  cudaFree(nullptr);
  CUdeviceptr p;
  if (int rc = device_address(word, &p)) return rc;
  CUresult r = g_write((CUstream)stream, p, value, CU_STREAM_WRITE_VALUE_DEFAULT);
  return r == CUDA_SUCCESS ? 0 : set_error(-101, "cuStreamWriteValue32 failed: CUresult %d", (int)r);
}
