// RMSNorm backward whose scratch lives in the library image (see noalloc_api.h for who needs
// this and for the rules of use).  Self-contained on purpose: it shares no code path with
// rmsnorm.cu, only the arithmetic.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>
#include "noalloc_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

constexpr int NA_THREADS = 256;
constexpr int NA_VEC = 4;   // 4 vectors * 8 elements * 256 threads = 8192 columns

// Per-block partial sums of dy * x * rstd, [MESH_NOALLOC_MAX_BLOCKS][MESH_NOALLOC_MAX_COLS].
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_partials[MESH_NOALLOC_MAX_BLOCKS * MESH_NOALLOC_MAX_COLS];

__device__ __forceinline__ float na_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float na_block_sum(float v, float* sh) {
  v = na_warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    t = na_warp_sum(t);
    if (l == 0) sh[0] = t;
  }
  __syncthreads();
  t = sh[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ void na_unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 na_pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// Block b walks rows b, b + gridDim.x, ...; writes dx for each and leaves its column sums in
// partials[b][0..cols).  Every block owns at least one row, so every partial row that the
// reduction reads was written by this launch.
__global__ void __launch_bounds__(NA_THREADS)
na_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows, int cols,
                      float w_offset) {
  __shared__ float sh[32];
  const int nvec = cols >> 3;
  float dwacc[NA_VEC][8];
#pragma unroll
  for (int i = 0; i < NA_VEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * cols);
    const float r = rstd[row];
    float xv[NA_VEC][8], gv[NA_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NA_VEC; ++i) {
      const int c = threadIdx.x + i * NA_THREADS;
      if (c < nvec) {
        float w8[8];
        na_unpack8(xr[c], xv[i]);
        na_unpack8(gr[c], gv[i]);
        na_unpack8(reinterpret_cast<const uint4*>(w)[c], w8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gv[i][j] * xv[i][j] * r;
          gv[i][j] *= (w8[j] + w_offset);
          dot += gv[i][j] * xv[i][j];
        }
      }
    }
    dot = na_block_sum(dot, sh);
    const float coef = dot * r * r * r / (float)cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < NA_VEC; ++i) {
      const int c = threadIdx.x + i * NA_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gv[i][j] * r - xv[i][j] * coef;
        dr[c] = na_pack8(o);
      }
    }
  }
  float* out = partials + (size_t)blockIdx.x * MESH_NOALLOC_MAX_COLS;
#pragma unroll
  for (int i = 0; i < NA_VEC; ++i) {
    const int c = threadIdx.x + i * NA_THREADS;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[c * 8 + j] = dwacc[i][j];
    }
  }
}

__global__ void na_dw_reduce_kernel(const float* __restrict__ partials, float* __restrict__ dw, int blocks, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partials[(size_t)b * MESH_NOALLOC_MAX_COLS + c];
  dw[c] = s;
}

// Device address of the partials array, looked up once per device with that device current.
constexpr int NA_MAX_DEVICES = 64;
float* g_partials_addr[NA_MAX_DEVICES] = {nullptr};
std::mutex g_partials_lock;

int partials_for_current_device(float** out) {
  std::lock_guard<std::mutex> hold(g_partials_lock);
  int dev = -1;
  MESH_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NA_MAX_DEVICES) return set_error(-8, "rmsnorm_bwd_noalloc: device index %d out of range", dev);
  if (g_partials_addr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_partials);
    if (e != cudaSuccess)
      return set_error((int)e, "rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                       cudaGetErrorString(e));
    g_partials_addr[dev] = static_cast<float*>(p);
  }
  *out = g_partials_addr[dev];
  return 0;
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                        float* dw, int rows, int cols, float w_offset, void* stream) {
  using namespace mesh;
  if (rows <= 0) return 0;
  if (cols <= 0 || cols % 8)
    return set_error(-2, "rmsnorm_bwd_noalloc: cols (%d) must be a positive multiple of 8", cols);
  if (cols > MESH_NOALLOC_MAX_COLS)
    return set_error(-3, "rmsnorm_bwd_noalloc: cols (%d) exceeds the built-in scratch (%d columns); use "
                         "mesh_rmsnorm_bwd with your own scratch instead", cols, MESH_NOALLOC_MAX_COLS);
  // A caller with raw pointers gets an error code for a bad one, not a device fault: the kernels read dy, x, w and
  // write dx as 16-byte vectors and always write dw.
  if (!dy || !x || !w || !rstd || !dx || !dw)
    return set_error(-2, "rmsnorm_bwd_noalloc: a null pointer was passed (dy, x, w, rstd, dx and dw are all required)");
  if ((((uintptr_t)dy | (uintptr_t)x | (uintptr_t)w | (uintptr_t)dx) & 15) || ((uintptr_t)rstd & 3) || ((uintptr_t)dw & 3))
    return set_error(-2, "rmsnorm_bwd_noalloc: dy, x, w and dx must be 16-byte aligned, rstd and dw 4-byte aligned");
  float* partials = nullptr;
  if (int rc = partials_for_current_device(&partials)) return rc;
  const int blocks = rows < MESH_NOALLOC_MAX_BLOCKS ? rows : MESH_NOALLOC_MAX_BLOCKS;
  na_rmsnorm_bwd_kernel<<<blocks, NA_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, partials,
      rows, cols, w_offset);
  MESH_CUDA_OK(cudaGetLastError());
  na_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, (cudaStream_t)stream>>>(partials, dw, blocks, cols);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
