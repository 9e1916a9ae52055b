#include "host_common.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace mesh {

static thread_local char g_err[512] = "";
static thread_local int g_code = 0;

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  g_code = code;
  return code;
}
int last_error_code() { return g_code; }
const char* last_error_text() { return g_err; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
  });
  return fn;
}

bool encode_tiled(CUtensorMap* tm, CUtensorMapDataType dtype, int rank, const void* base,
                  const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box,
                  const cuuint32_t* elem_strides, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error(-100, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  // The encoder is a driver call and wants a context current on the calling thread.  A thread that has only ever
  // had its device selected (an autograd worker whose device is the default one, for instance) has none bound until
  // its first runtime call that needs one: make that call here, once per thread.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  CUresult r = fn(tm, dtype, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {          // the context changed under this thread: bind again and retry once
    cudaFree(nullptr);
    r = fn(tm, dtype, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box, elem_strides,
           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    set_error(-101, "cuTensorMapEncodeTiled failed: CUresult %d (rank %d, dims %llu x %llu, box %u x %u)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return false;
  }
  return true;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MESH_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace mesh

extern "C" const char* mesh_last_error(void) { return mesh::last_error_text(); }
extern "C" int mesh_sm_count(void) { return mesh::sm_count(); }
// 1 when this library was compiled with -DMESH_CHECK=1 (index / alignment checks inside the kernels).
extern "C" int mesh_checked_build(void) {
#if defined(MESH_CHECK) && MESH_CHECK
  return 1;
#else
  return 0;
#endif
}
