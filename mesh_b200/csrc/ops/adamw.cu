// Fused AdamW step over a flat shard: bf16 parameters with fp32 master weights and fp32 moments.
// One pass over memory: reads grad (bf16 or fp32), master, m, v; writes master, m, v and the bf16 copy.
// (The reference has no optimizer — training returns gradients and the caller applies updates,
// compiler/mesh_compiler/ir.py:79-84; the sharded optimizer is this build's addition for the hybrid training config.)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "../runtime/host_common.h"

namespace mesh {
namespace {

template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g;
    if constexpr (sizeof(G) == 2) g = __bfloat162float(grad[i]) * grad_scale;
    else g = grad[i] * grad_scale;
    float w = master[i];
    float mi = beta1 * m[i] + (1.f - beta1) * g;
    float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    const float mhat = mi / bc1, vhat = vi / bc2;
    w = w * (1.f - lr * wd) - lr * mhat / (sqrtf(vhat) + eps);
    master[i] = w; m[i] = mi; v[i] = vi;
    if (param) param[i] = __float2bfloat16_rn(w);
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_adamw_step(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* param_bf16,
                               long long n, float lr, float beta1, float beta2, float eps, float wd, int step,
                               float grad_scale, void* stream) {
  using namespace mesh;
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  int grid = (int)((n + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(master, m, v, (const __nv_bfloat16*)grad,
        (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  else
    adamw_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(master, m, v, (const float*)grad, (__nv_bfloat16*)param_bf16,
        n, lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
