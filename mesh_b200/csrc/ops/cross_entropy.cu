// Cross-entropy over a vocabulary shard: the per-row statistics in one pass over the logits, and the gradient in one.
//
// With the output projection column-parallel a rank holds logits[:, v0:v1].  The loss of a row needs the row's
// maximum, its sum of exponentials and the target's logit over the WHOLE vocabulary; each rank computes them over its
// columns here (online max / sum, the reference's statistics of compiler/mesh_compiler/operations.py:6281-6330), two
// tiny all-reduces combine them, and the gradient (softmax - onehot) * g is formed from the logits again, so no fp32
// copy of the logits or of their exponentials is ever stored.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "ops_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ void online(float& m, float& s, float x) {
  if (x > m) { s = s * __expf(m - x) + 1.f; m = x; }
  else s += __expf(x - m);
}
__device__ __forceinline__ void merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -CUDART_INF_F) { m = mm; s = 0.f; return; }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

// row_max[r], row_sum[r] (relative to row_max[r]) and target_logit[r] (0 when the target is not in this shard or ignored)
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int rows, int cols, const long long* __restrict__ targets,
                long long vocab_start, long long ignore_index, float* __restrict__ row_max, float* __restrict__ row_sum,
                float* __restrict__ target_logit) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  const bool vec = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* x = logits + (long long)r * ld;
    float m = -CUDART_INF_F, s = 0.f;
    int done = 0;
    if (vec) {
      const int nv = cols >> 3;
      for (int v = threadIdx.x; v < nv; v += CE_THREADS) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          online(m, s, f.x);
          online(m, s, f.y);
        }
      }
      done = nv << 3;
    }
    for (int c = done + threadIdx.x; c < cols; c += CE_THREADS) online(m, s, __bfloat162float(x[c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      merge(m, s, m2, s2);
    }
    if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float M = sm[0], S = ss[0];
      for (int w = 1; w < CE_THREADS / 32; ++w) merge(M, S, sm[w], ss[w]);
      row_max[r] = M;
      row_sum[r] = S;
      const long long t = targets[r], local = t - vocab_start;
      target_logit[r] = (t != ignore_index && local >= 0 && local < cols) ? __bfloat162float(x[local]) : 0.f;
    }
    __syncthreads();
  }
}

// d[r, c] = (exp(x - gmax[r]) / gsum[r] - [c == target]) * gscale[r]; gscale = upstream gradient, 0 for ignored rows
__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, __nv_bfloat16* __restrict__ d, long long ldd, int rows, int cols,
               const long long* __restrict__ targets, long long vocab_start, const float* __restrict__ gmax,
               const float* __restrict__ gsum, const float* __restrict__ gscale) {
  const bool vec = (ld % 8 == 0) && (ldd % 8 == 0) && (((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(d)) & 15) == 0);
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* x = logits + (long long)r * ld;
    __nv_bfloat16* o = d + (long long)r * ldd;
    const float mx = gmax[r], g = gscale[r];
    const float inv = g / gsum[r];
    const long long local = targets[r] - vocab_start;
    int done = 0;
    if (vec) {
      const int nv = cols >> 3;
      for (int v = threadIdx.x; v < nv; v += CE_THREADS) {
        uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + v);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          float a = __expf(f.x - mx) * inv, b = __expf(f.y - mx) * inv;
          const int c = v * 8 + 2 * i;
          if (c == local) a -= g;
          if (c + 1 == local) b -= g;
          h[i] = __floats2bfloat162_rn(a, b);
        }
        reinterpret_cast<uint4*>(o)[v] = q;
      }
      done = nv << 3;
    }
    for (int c = done + threadIdx.x; c < cols; c += CE_THREADS) {
      float a = __expf(__bfloat162float(x[c]) - mx) * inv;
      if (c == local) a -= g;
      o[c] = __float2bfloat16_rn(a);
    }
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_ce_stats_bf16(const void* logits, long long ld, int rows, int cols, const long long* targets,
                                  long long vocab_start, long long ignore_index, float* row_max, float* row_sum,
                                  float* target_logit, void* stream) {
  using namespace mesh;
  if (rows <= 0 || cols <= 0) return 0;
  if (!logits || !targets || !row_max || !row_sum || !target_logit) return set_error(-2, "ce_stats: null argument");
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  ce_stats_kernel<<<grid, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, rows, cols, targets, vocab_start,
                                                                ignore_index, row_max, row_sum, target_logit);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_ce_grad_bf16(const void* logits, long long ld, void* dlogits, long long ldd, int rows, int cols,
                                 const long long* targets, long long vocab_start, const float* gmax, const float* gsum,
                                 const float* gscale, void* stream) {
  using namespace mesh;
  if (rows <= 0 || cols <= 0) return 0;
  if (!logits || !dlogits || !targets || !gmax || !gsum || !gscale) return set_error(-2, "ce_grad: null argument");
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  ce_grad_kernel<<<grid, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, (__nv_bfloat16*)dlogits, ldd, rows, cols,
                                                               targets, vocab_start, gmax, gsum, gscale);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
