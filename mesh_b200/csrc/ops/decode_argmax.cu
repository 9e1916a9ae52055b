// Vocabulary-parallel greedy selection: one CTA per sequence finds (max logit, lowest index) over
// this rank's vocabulary shard, exchanges that 8-byte pair with every rank, and all ranks pick the
// same winner (highest value, lowest global index on ties) without ever gathering logits.
#include <cuda_runtime.h>
#include <math_constants.h>
#include "decode_api.h"
#include "../device/ptx.cuh"
#include "../runtime/host_common.h"
#include <cstring>

namespace mesh {
namespace {

constexpr int AM_THREADS = 1024;

__global__ void __launch_bounds__(AM_THREADS)
decode_argmax_kernel(const float* __restrict__ logits, long long ldl, int vocab_local, int vocab_offset,
                     int* __restrict__ tokens_out, int* __restrict__ pos, int rank, int world,
                     uint2* const* __restrict__ xchg_unused, uint2* x0, uint2* x1, uint2* x2, uint2* x3, uint2* x4,
                     uint2* x5, uint2* x6, uint2* x7, uint32_t* step, Status* st) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int b = blockIdx.x;
  const uint32_t seq = (step ? *step : 0u) + 1u;
  const float* row = logits + (long long)b * ldl;
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab_local; i += AM_THREADS) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }          // ascending i per thread: first maximum kept
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp != 0) return;
  best = sv[lane];
  bi = si[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  int gidx = bi + vocab_offset;
  if (world > 1) {
    uint2* peers[8] = {x0, x1, x2, x3, x4, x5, x6, x7};
    // slot layout on every rank: [parity(seq & 1)][src rank][sequence][2 words]: {value bits, seq}, {index, seq}
    const long long base = ((long long)(seq & 1u) * world * 8 + (long long)rank * 8 + b) * 2;
    if (lane < world) {
      uint2* p = peers[lane] + base;
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(best)), "r"(seq) : "memory");
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p + 1), "r"((uint32_t)gidx), "r"(seq) : "memory");
    }
    float v = -CUDART_INF_F;
    int id = 0x7fffffff;
    if (lane < world) {
      const uint2* p = peers[rank] + ((long long)(seq & 1u) * world * 8 + (long long)lane * 8 + b) * 2;
      uint2 w0, w1;
      unsigned long long t0 = 0;
      uint32_t it = 0;
      while (true) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w0.x), "=r"(w0.y) : "l"(p) : "memory");
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w1.x), "=r"(w1.y) : "l"(p + 1) : "memory");
        if (w0.y == seq && w1.y == seq) break;
        if (((++it) & 0x3ffu) == 0) {
          if (t0 == 0) t0 = globaltimer_ns();
          else if (globaltimer_ns() - t0 > MESH_WAIT_LIMIT_NS || status_aborted(st)) {
            status_record(st, MESH_TIMEOUT, SITE_PEER_FLAG, seq, w0.y, (unsigned long long)p);
            break;
          }
        }
      }
      v = __uint_as_float(w0.x);
      id = (int)w1.x;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
    }
    gidx = id;
  }
  if (lane == 0) {
    tokens_out[b] = gidx;
    if (pos) pos[b] += 1;
    // the last sequence's CTA to finish advances the step word (every CTA has read it by then:
    // the counter below is only bumped after this CTA's own read at the top)
    if (step) {
      __threadfence();
      const unsigned done = atomicAdd(step + 1, 1u);
      if (done == gridDim.x - 1) { step[1] = 0; __threadfence(); atomicAdd(step, 1u); }
    }
  }
}

}  // namespace
}  // namespace mesh

extern "C" int mesh_decode_argmax(const float* logits, long long ldl, int B, int vocab_local, int vocab_offset,
                                  int* tokens_out, int* pos, int rank, int world, void* const* xchg, uint32_t* step,
                                  void* status, void* stream) {
  using namespace mesh;
  if (B < 1 || B > 8) return set_error(-2, "decode_argmax: batch must be 1..8");
  if (world < 1 || world > 8) return set_error(-4, "decode_argmax: world out of range");
  uint2* x[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int r = 0; r < world && xchg; ++r) x[r] = (uint2*)xchg[r];
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)B);
  cfg.blockDim = dim3(AM_THREADS);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  uint2* const* none = nullptr;
  MESH_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_argmax_kernel, logits, ldl, vocab_local, vocab_offset, tokens_out, pos, rank,
                                  world, none, x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], step, (Status*)status));
  return 0;
}
