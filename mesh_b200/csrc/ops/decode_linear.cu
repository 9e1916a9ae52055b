// Stand-alone launches of the decode-time linear layer (the layer itself: decode_linear.cuh).
#include "decode_linear.cuh"

namespace mesh {
namespace decode {

template <int W4, int U>
__global__ void __launch_bounds__(THREADS) decode_linear_kernel(const LinArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  // Let the next kernel of the stream start its own weight requests now.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  linear_body<W4, U>(a, smem, [] { asm volatile("griddepcontrol.wait;" ::: "memory"); });
}

}  // namespace decode
}  // namespace mesh

using namespace mesh;
using namespace mesh::decode;

extern "C" int mesh_decode_linear(const MeshDecodeLinear* d, void* stream) {
  LinArgs a;
  int variant = 0;
  const int rc = lin_prepare(d, a, variant);
  if (rc) return rc;
  const size_t smem = lin_smem_bytes(d->K, d->B);
  void (*kern)(const LinArgs) = nullptr;
  switch (variant) {
    case LIN_W4N_U2: kern = decode_linear_kernel<1, 2>; break;
    case LIN_W4N_U1: kern = decode_linear_kernel<1, 1>; break;
    case LIN_BF16_U4: kern = decode_linear_kernel<0, 4>; break;
    case LIN_BF16_U1: kern = decode_linear_kernel<0, 1>; break;
    case LIN_W8_U4: kern = decode_linear_kernel<3, 4>; break;
    case LIN_W8_U2: kern = decode_linear_kernel<3, 2>; break;
    case LIN_W8_U1: kern = decode_linear_kernel<3, 1>; break;
    case LIN_W4W_U2: kern = decode_linear_kernel<2, 2>; break;
    default: kern = decode_linear_kernel<2, 1>; break;
  }
  static bool configured[LIN_VARIANTS] = {false, false, false, false, false, false, false, false, false};
  if (!configured[variant]) {
    MESH_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured[variant] = true;
  }
  int grid = a.n_groups;
  // CTAs per SM: two fill the machine with loads in flight (measured: one CTA per SM, which would leave room for a
  // CTA of the next kernel to start early, loses a fifth of the decode rate).  MESH_DECODE_CTAS_PER_SM=1 and
  // MESH_DECODE_L2_PREFETCH=1 (each CTA asks for its own rows before waiting for the previous kernel) remain as
  // switches for experiments.
  static int per_sm = -1, prefetch = -1;
  if (per_sm < 0) {
    const char* e = getenv("MESH_DECODE_CTAS_PER_SM");
    per_sm = (e && e[0] == '1') ? 1 : 2;
    const char* f = getenv("MESH_DECODE_L2_PREFETCH");
    prefetch = (f && f[0] == '1') ? 1 : 0;
  }
  a.l2_prefetch = prefetch;       // rows are multiples of 16 bytes in every format (K % 256 == 0)
  const int cap = sm_count() * (smem > 100 * 1024 ? 1 : per_sm);
  if (grid > cap) grid = cap;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MESH_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, a));
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
