// RMSNorm forward (+ fused residual add) and backward for bf16 activations, fp32 math.
// One CTA per row, 16-byte vector accesses, the row kept in registers between the reduction
// and the scaling pass so that x is read from HBM once.
// Reference semantics: the `rms` entry of NORMS, compiler/mesh_compiler/operations.py:6671-6682.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "ops_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

constexpr int NORM_THREADS = 256;
constexpr int MAX_VEC_PER_THREAD = 8;   // 8 vectors * 8 elements * 256 threads = 16384 columns

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) sh[0] = t;
  }
  __syncthreads();
  t = sh[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return q;
}

// VPT = 16-byte vectors per thread (a row has up to VPT * 256 of them): sized to the row so that the registers
// holding the row stay few and several CTAs per SM keep enough loads in flight to fill HBM.  RPP rows are processed
// per pass (their loads are all issued before the first reduction), which doubles the bytes in flight for narrow rows.
template <int VPT, int RPP>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int rows, int cols,
                   float eps, float w_offset) {
  __shared__ float sh[RPP][32];
  const int nvec = cols >> 3;
  for (int row0 = blockIdx.x * RPP; row0 < rows; row0 += gridDim.x * RPP) {
    float v[RPP][VPT][8];
    float ss[RPP];
#pragma unroll
    for (int q = 0; q < RPP; ++q) {
      const int row = row0 + q;
      ss[q] = 0.f;
      if (row < rows) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
        const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * cols) : nullptr;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int c = threadIdx.x + i * NORM_THREADS;
          if (c < nvec) {
            unpack8(xr[c], v[q][i]);
            if (rr) {
              float r8[8];
              unpack8(rr[c], r8);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q][i][j] += r8[j];
              if (res_out) {
                // the sum is rounded to bf16 once and that rounded value is what gets normalised
                uint4 qv = pack8(v[q][i]);
                reinterpret_cast<uint4*>(res_out + (size_t)row * cols)[c] = qv;
                unpack8(qv, v[q][i]);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss[q] += v[q][i][j] * v[q][i][j];
          }
        }
      }
    }
    // RPP block reductions share the barriers
    const int wi = threadIdx.x >> 5, l = threadIdx.x & 31;
#pragma unroll
    for (int q = 0; q < RPP; ++q) {
      ss[q] = warp_sum(ss[q]);
      if (l == 0) sh[q][wi] = ss[q];
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < RPP; ++q) {
      float t = (l < (NORM_THREADS >> 5)) ? sh[q][l] : 0.f;
      ss[q] = warp_sum(t);
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < RPP; ++q) {
      const int row = row0 + q;
      if (row >= rows) continue;
      const float rstd = rsqrtf(ss[q] / (float)cols + eps);
      if (rstd_out && threadIdx.x == 0) rstd_out[row] = rstd;
      uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * cols);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < nvec) {
          float w8[8], o[8];
          unpack8(reinterpret_cast<const uint4*>(w)[c], w8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[q][i][j] * rstd * (w8[j] + w_offset);
          yr[c] = pack8(o);
        }
      }
    }
  }
}

// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; writes dx per row and keeps a
// per-thread running sum of dy*x*rstd for its columns, stored to dw_partial[blockIdx.x][cols].
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int cols,
                   float w_offset) {
  __shared__ float sh[32];
  const int nvec = cols >> 3;
  float dwacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * cols);
    const float r = rstd[row];
    float xv[VPT][8], gv[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float w8[8];
        unpack8(xr[c], xv[i]);
        unpack8(gr[c], gv[i]);
        unpack8(reinterpret_cast<const uint4*>(w)[c], w8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += gv[i][j] * xv[i][j] * r;
          gv[i][j] *= (w8[j] + w_offset);          // gv now holds w*dy
          dot += gv[i][j] * xv[i][j];
        }
      }
    }
    dot = block_sum(dot, sh);
    const float coef = dot * r * r * r / (float)cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + (size_t)row * cols);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = gv[i][j] * r - xv[i][j] * coef;
        dr[c] = pack8(o);
      }
    }
  }
  if (dw_partial) {
    float* out = dw_partial + (size_t)blockIdx.x * cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) out[c * 8 + j] = dwacc[i][j];
      }
    }
  }
}

__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw, int blocks,
                                         int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[(size_t)b * cols + c];
  dw[c] = s;
}

}  // namespace
}  // namespace mesh

using namespace mesh;

extern "C" int mesh_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                                float* rstd, int rows, int cols, float eps, float w_offset, void* stream) {
  if (rows <= 0) return 0;
  if (cols % 8 || cols > NORM_THREADS * MAX_VEC_PER_THREAD * 8)
    return set_error(-2, "rmsnorm: cols must be a multiple of 8 and <= %d", NORM_THREADS * MAX_VEC_PER_THREAD * 8);
  const int nvec = cols / 8;
#define FWD(V, R)                                                                                                  \
  do {                                                                                                             \
    const int passes = (rows + (R) - 1) / (R);                                                                     \
    const int grid = passes < 148 * 16 ? passes : 148 * 16;                                                        \
    rmsnorm_fwd_kernel<V, R><<<grid, NORM_THREADS, 0, (cudaStream_t)stream>>>(                                      \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,        \
        (__nv_bfloat16*)residual_out, rstd, rows, cols, eps, w_offset);                                            \
  } while (0)
  const bool many = rows >= 148 * 8;        // enough rows that pairing them does not idle SMs
  if (nvec <= NORM_THREADS) { if (many) FWD(1, 2); else FWD(1, 1); }
  else if (nvec <= 2 * NORM_THREADS) { if (many) FWD(2, 2); else FWD(2, 1); }
  else if (nvec <= 4 * NORM_THREADS) FWD(4, 1);
  else FWD(8, 1);
#undef FWD
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_rmsnorm_bwd_blocks(int rows) { return rows < 592 ? rows : 592; }

extern "C" int mesh_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                                float* dw_partial, int blocks, int rows, int cols, float w_offset, void* stream) {
  if (rows <= 0) return 0;
  if (cols % 8 || cols > NORM_THREADS * MAX_VEC_PER_THREAD * 8)
    return set_error(-2, "rmsnorm: cols must be a multiple of 8 and <= %d", NORM_THREADS * MAX_VEC_PER_THREAD * 8);
  if (blocks <= 0 || blocks > 1024) return set_error(-2, "rmsnorm_bwd: blocks out of range");
  const int nvec = cols / 8;
#define BWD(V)                                                                                                     \
  rmsnorm_bwd_kernel<V><<<blocks, NORM_THREADS, 0, (cudaStream_t)stream>>>(                                         \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx,         \
      dw_partial, rows, cols, w_offset)
  if (nvec <= NORM_THREADS) BWD(1);
  else if (nvec <= 2 * NORM_THREADS) BWD(2);
  else if (nvec <= 4 * NORM_THREADS) BWD(4);
  else BWD(8);
#undef BWD
  MESH_CUDA_OK(cudaGetLastError());
  if (dw && dw_partial) {
    rmsnorm_dw_reduce_kernel<<<(cols + 255) / 256, 256, 0, (cudaStream_t)stream>>>(dw_partial, dw, blocks, cols);
    MESH_CUDA_OK(cudaGetLastError());
  }
  return 0;
}
