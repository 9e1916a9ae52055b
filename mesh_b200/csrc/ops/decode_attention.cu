// Stand-alone launch of the decode-time attention (the work itself: decode_attention.cuh).
#include "decode_attention.cuh"

namespace mesh {
namespace decode_att {

// Grid = (splits, kv_heads, batch * tokens): one work item per CTA.
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) decode_attention_kernel(const AttArgs A) {
  extern __shared__ float sm_acc_raw[];                  // [ATT_WARPS][group][HD]
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // q and the newest cache row come from the previous kernel
  if (A.q_heads / A.kv_heads <= 4) attention_item<HD, 4>(A, blockIdx.x, blockIdx.y, blockIdx.z, sm_acc_raw);
  else attention_item<HD, MAX_GROUPS>(A, blockIdx.x, blockIdx.y, blockIdx.z, sm_acc_raw);
}

}  // namespace decode_att
}  // namespace mesh


extern "C" int mesh_decode_attention_scratch_floats(int B, int q_heads, int head_dim, int splits) {
  return B * q_heads * splits * (head_dim + 2);
}

extern "C" int mesh_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* pos, void* out,
                                     float* scratch, int* counters, int B, int tokens_per_seq, int q_heads, int kv_heads,
                                     int head_dim, int max_seq, int window, float scale, int splits, void* stream) {
  using namespace mesh;
  using namespace mesh::decode_att;
  if (B <= 0) return 0;
  if (q_heads % kv_heads || q_heads / kv_heads > MAX_GROUPS) return set_error(-2, "decode_attention: group size must be 1..8");
  if (splits < 1 || splits > 64) return set_error(-2, "decode_attention: splits must be 1..64");
  if (tokens_per_seq < 1) tokens_per_seq = 1;
  dim3 grid(splits, kv_heads, B * tokens_per_seq);
  const size_t smem = (size_t)ATT_WARPS * (q_heads / kv_heads) * head_dim * sizeof(float);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(ATT_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  AttArgs A;
  memset(&A, 0, sizeof(A));
  A.q = (const __nv_bfloat16*)q; A.kc = (const __nv_bfloat16*)k_cache; A.vc = (const __nv_bfloat16*)v_cache; A.pos = pos;
  A.out = (__nv_bfloat16*)out; A.scratch = scratch; A.counters = counters;
  A.q_heads = q_heads; A.kv_heads = kv_heads; A.max_seq = max_seq; A.window = window; A.scale = scale; A.splits = splits;
  A.T = tokens_per_seq; A.B = B; A.head_dim = head_dim;
#define LAUNCH(HD)                                                                                          \
  if (smem > 48 * 1024) {                                                                                   \
    static bool cfg = false;                                                                                \
    if (!cfg) { MESH_CUDA_OK(cudaFuncSetAttribute(decode_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)); cfg = true; } \
  }                                                                                                         \
  cfg.gridDim = grid;                                                                                       \
  MESH_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_attention_kernel<HD>, A))
  if (head_dim == 256) { LAUNCH(256); }
  else if (head_dim == 128) { LAUNCH(128); }
  else if (head_dim == 64) { LAUNCH(64); }
  else return set_error(-2, "decode_attention: head_dim must be 64, 128 or 256");
#undef LAUNCH
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
