// sum(a * b) over two bf16 vectors, fp32 result in one launch: a training loop's scalar (a loss against fixed
// targets, a gradient-norm probe) without the four or five elementwise launches of the tensor-op formulation.
// Blocks leave their partial sums in `partials`; the block that takes the last ticket adds them in block order, so
// the result does not depend on which block finishes last.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "ops_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

constexpr int DS_THREADS = 256;

__global__ void __launch_bounds__(DS_THREADS)
dot_sum_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, long long n,
               float* __restrict__ out, float* __restrict__ partials, unsigned int* __restrict__ ticket) {
  __shared__ float sh[DS_THREADS / 32];
  __shared__ unsigned int last;
  const long long nv = n >> 3;
  const uint4* av = reinterpret_cast<const uint4*>(a);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)DS_THREADS + threadIdx.x; i < nv; i += (long long)gridDim.x * DS_THREADS) {
    const uint4 x = __ldg(av + i), y = __ldg(bv + i);
    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&x);
    const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = __bfloat1622float2(xh[j]), yf = __bfloat1622float2(yh[j]);
      acc += xf.x * yf.x + xf.y * yf.y;
    }
  }
  if (blockIdx.x == 0)
    for (long long i = (nv << 3) + threadIdx.x; i < n; i += DS_THREADS) acc += __bfloat162float(a[i]) * __bfloat162float(b[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < DS_THREADS / 32; ++w) s += sh[w];
    partials[blockIdx.x] = s;
    __threadfence();
    last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {
    __threadfence();
    float s = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += 32) s += __ldcg(partials + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) {
      *out = s;
      *ticket = 0u;            // ready for the next launch on this scratch
    }
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_dot_sum_blocks(void) { return 296; }

extern "C" int mesh_dot_sum_bf16(const void* a, const void* b, long long n, float* out, float* partials,
                                 unsigned int* ticket, void* stream) {
  using namespace mesh;
  if (n < 0 || !out || !partials || !ticket) return set_error(-2, "dot_sum: bad arguments");
  if (((uintptr_t)a | (uintptr_t)b) & 15) return set_error(-2, "dot_sum: operands must be 16-byte aligned");
  long long want = (n / 8 + DS_THREADS - 1) / DS_THREADS;
  int grid = (int)(want < 1 ? 1 : (want > 296 ? 296 : want));
  dot_sum_kernel<<<grid, DS_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, n, out,
                                                             partials, ticket);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
