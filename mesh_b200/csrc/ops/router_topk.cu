// MoE router: softmax over experts followed by top-k selection, one warp per token.
// Reference semantics: `softmax(x W_r).topk(k)` of examples/ep.py:15-22 and the ranked
// selection of compiler/mesh_compiler/operations.py:6519-6608; ties resolve to the lower index.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "ops_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

constexpr int MAX_PER_LANE = 8;   // experts <= 256

template <bool FP32>
__global__ void router_topk_kernel(const void* __restrict__ logits_v, const float* __restrict__ bias,
                                   float* __restrict__ weights, int* __restrict__ indices, int tokens, int experts,
                                   int k, int renorm) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
    float v[MAX_PER_LANE];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      float x = -CUDART_INF_F;
      if (e < experts) {
        if (FP32) x = reinterpret_cast<const float*>(logits_v)[(size_t)t * experts + e];
        else x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits_v)[(size_t)t * experts + e]);
        if (bias) x += bias[e];
      }
      v[i] = x;
      mx = fmaxf(mx, x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      v[i] = (lane + 32 * i < experts) ? __expf(v[i] - mx) : -1.f;   // -1 marks "not a candidate"
      if (v[i] > 0.f) sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    float ksum = 0.f;
    float my_w = 0.f;
    int my_i = 0;
    for (int j = 0; j < k; ++j) {
      // lane-local best (lowest index wins ties), then warp arg-max on (value, -index)
      float bv = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (v[i] > bv) { bv = v[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if ((bi & 31) == lane) v[bi >> 5] = -1.f;     // remove the winner
      if (lane == j) { my_w = bv * inv; my_i = bi; }
      ksum += bv * inv;
    }
    if (lane < k) {
      weights[(size_t)t * k + lane] = renorm ? my_w / ksum : my_w;
      indices[(size_t)t * k + lane] = my_i;
    }
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_router_topk(const void* logits, int logits_is_fp32, const float* bias, float* weights,
                                int* indices, int tokens, int experts, int k, int renorm, void* stream) {
  using namespace mesh;
  if (tokens <= 0) return 0;
  if (experts > 32 * MAX_PER_LANE || experts < 1) return set_error(-2, "router_topk: experts must be in [1, 256]");
  if (k < 1 || k > 32 || k > experts) return set_error(-2, "router_topk: k out of range");
  const int wpb = 8;
  int grid = (tokens + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  if (logits_is_fp32)
    router_topk_kernel<true><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(logits, bias, weights, indices, tokens,
                                                                          experts, k, renorm);
  else
    router_topk_kernel<false><<<grid, wpb * 32, 0, (cudaStream_t)stream>>>(logits, bias, weights, indices, tokens,
                                                                           experts, k, renorm);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
