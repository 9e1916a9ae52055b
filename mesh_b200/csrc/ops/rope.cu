// Rotate-half rotary position embedding, in place, bf16 activations with fp32 cos/sin tables.
// Reference model: examples/pl.py:17-28 (cached cos/sin, rotate-half); theta is folded into the
// tables by the caller (1e6 for the E2B-class config).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "ops_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace {

// One thread rotates 8 consecutive pairs (i, i + hd/2): two 16-byte loads, two 16-byte stores.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens,
                            int heads, int hd, long long ld, int inverse) {
  const int half = hd >> 1;
  const int vec_per_head = half >> 3;
  const long long total = (long long)tokens * heads * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const int h = (int)((idx / vec_per_head) % heads);
    const int t = (int)(idx / ((long long)vec_per_head * heads));
    const int p = pos[t];
    __nv_bfloat16* base = x + (long long)t * ld + (long long)h * hd + v * 8;
    uint4 lo = *reinterpret_cast<uint4*>(base);
    uint4 hi = *reinterpret_cast<uint4*>(base + half);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
    float c[8], s[8];
    *reinterpret_cast<float4*>(c) = c4[0];
    *reinterpret_cast<float4*>(c + 4) = c4[1];
    *reinterpret_cast<float4*>(s) = s4[0];
    *reinterpret_cast<float4*>(s + 4) = s4[1];
    __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 a = __bfloat1622float2(l2[i]);
      float2 b = __bfloat1622float2(h2[i]);
      const float s0 = inverse ? -s[2 * i] : s[2 * i], s1 = inverse ? -s[2 * i + 1] : s[2 * i + 1];
      float2 oa, ob;
      oa.x = a.x * c[2 * i] - b.x * s0;
      ob.x = b.x * c[2 * i] + a.x * s0;
      oa.y = a.y * c[2 * i + 1] - b.y * s1;
      ob.y = b.y * c[2 * i + 1] + a.y * s1;
      l2[i] = __floats2bfloat162_rn(oa.x, oa.y);
      h2[i] = __floats2bfloat162_rn(ob.x, ob.y);
    }
    *reinterpret_cast<uint4*>(base) = lo;
    *reinterpret_cast<uint4*>(base + half) = hi;
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_rope(void* x, const int* positions, const float* cos_t, const float* sin_t, int tokens, int heads,
                         int head_dim, long long ld, int inverse, void* stream) {
  using namespace mesh;
  if (tokens <= 0 || heads <= 0) return 0;
  if (head_dim % 16 || ld % 8) return set_error(-2, "rope: head_dim must be a multiple of 16 and ld of 8");
  const long long total = (long long)tokens * heads * (head_dim / 16);
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  rope_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, positions, cos_t, sin_t, tokens, heads,
                                                      head_dim, ld, inverse);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
