// Host helpers shared by every launcher in the library: last-error text (thread local),
// the cuTensorMapEncodeTiled entry point (looked up through the CUDA runtime so the library
// never links against libcuda), and cached device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mesh {

int set_error(int code, const char* fmt, ...);
int last_error_code();
const char* last_error_text();

bool encode_tiled(CUtensorMap* tm, CUtensorMapDataType dtype, int rank, const void* base,
                  const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box,
                  const cuuint32_t* elem_strides, CUtensorMapSwizzle swizzle);

int sm_count();
// Programmatic dependent launch between consecutive kernels of a stream (MESH_PDL=0 switches it off).
bool pdl_enabled();

#define MESH_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess) return ::mesh::set_error((int)_e, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

}  // namespace mesh
