// Split-KV attention for decoding: one query token per sequence, grouped-query heads, optional
// sliding window.  Grid = (splits, kv_heads, batch): a CTA scores its slice of the keys for all the
// query heads that share one KV head (so K and V are read once per group), keeps the online-softmax
// triple (m, l, acc) per head, and the last CTA of a (sequence, kv head) to finish merges the
// partials.  Semantics: blockwise attention with (m, s, acc) merging and GQA by viewing query heads
// as [kv_heads, group] (compiler/mesh_compiler/operations.py:7081-7166, :7072-7078); the window is
// the E2B-class local layer (design/e2b-crossover-2026-09-16.md:42-52).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "decode_api.h"
#include "../runtime/host_common.h"
#include <cstring>

namespace mesh {
namespace decode_att {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = 8;
constexpr int MAX_GROUPS = 8;    // query heads per KV head, at most
constexpr int MAX_HD = 256;

// Each warp takes keys j = warp, warp+8, ... of the CTA's slice.  A lane owns head_dim/32 = up to 8
// consecutive dims (16 bytes of K and of V per key).
struct AttArgs {
  const __nv_bfloat16* q; const __nv_bfloat16* kc; const __nv_bfloat16* vc; const int* pos;
  __nv_bfloat16* out; float* scratch; int* counters;
  int q_heads, kv_heads, max_seq, window; float scale; int splits, T;
  int B, head_dim;                                   // used by callers that loop over the work items themselves
};

// One work item (split, kv head, sequence-token b) of the attention; `sm_acc_raw`: ATT_WARPS * group * HD floats of
// shared memory.  The ATT_THREADS computing threads call it together (`sync` is their barrier).
struct AttBlockSync { __device__ __forceinline__ void operator()() const { __syncthreads(); } };

template <int HD, int MAXG, class Sync = AttBlockSync>
__device__ __forceinline__ void attention_item(const AttArgs& A, int split, int kvh, int b, float* sm_acc_raw,
                                               Sync sync = Sync{}) {
  constexpr int PER = HD / 32;                       // dims per lane
  constexpr int MAX_GROUP = MAXG;
  // no __restrict__ here: inside a step kernel q and the newest cache row were written by an earlier phase of the
  // same kernel, and a read-only (non-coherent) load could return what the line held before
  const __nv_bfloat16* q = A.q;
  const __nv_bfloat16* kc = A.kc;
  const __nv_bfloat16* vc = A.vc;
  const int* pos = A.pos;
  __nv_bfloat16* out = A.out;
  float* scratch = A.scratch;
  int* counters = A.counters;
  const int q_heads = A.q_heads, kv_heads = A.kv_heads, max_seq = A.max_seq, window = A.window, splits = A.splits, T = A.T;
  const float scale = A.scale;
  // b indexes (sequence, query token); the cache belongs to the sequence
  const int seq_idx = b / T;
  const int group = q_heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = pos[seq_idx] + (b - seq_idx * T);
  const int lo_all = (window > 0) ? max(0, p - window + 1) : 0;
  const int n_keys = p + 1 - lo_all;
  const int per_split = (n_keys + splits - 1) / splits;
  const int lo = lo_all + split * per_split;
  const int hi = min(p + 1, lo + per_split);

  // query vectors of the group, scaled, in registers
  float qv[MAX_GROUP][PER];
#pragma unroll
  for (int g = 0; g < MAX_GROUP; ++g) {
    if (g < group) {
      const __nv_bfloat16* qp = q + ((long long)b * q_heads + kvh * group + g) * HD + lane * PER;
#pragma unroll
      for (int i = 0; i < PER; ++i) qv[g][i] = __bfloat162float(qp[i]) * scale;
    }
  }
  float m[MAX_GROUP], l[MAX_GROUP], acc[MAX_GROUP][PER];
#pragma unroll
  for (int g = 0; g < MAX_GROUP; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[g][i] = 0.f;
  }
  const __nv_bfloat16* kbase = kc + ((long long)seq_idx * kv_heads + kvh) * max_seq * HD + lane * PER;
  const __nv_bfloat16* vbase = vc + ((long long)seq_idx * kv_heads + kvh) * max_seq * HD + lane * PER;
  for (int j = lo + warp; j < hi; j += ATT_WARPS) {
    float kf[PER], vf[PER];
    if constexpr (PER == 8) {
      const uint4 kq = *reinterpret_cast<const uint4*>(kbase + (long long)j * HD);
      const uint4 vq = *reinterpret_cast<const uint4*>(vbase + (long long)j * HD);
      const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kq);
      const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vq);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(kh[i]), c = __bfloat1622float2(vh[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y; vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        kf[i] = __bfloat162float(kbase[(long long)j * HD + i]);
        vf[i] = __bfloat162float(vbase[(long long)j * HD + i]);
      }
    }
#pragma unroll
    for (int g = 0; g < MAX_GROUP; ++g) {
      if (g < group) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) s += qv[g][i] * kf[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m[g], s);
        const float corr = __expf(m[g] - mn), w = __expf(s - mn);
        l[g] = l[g] * corr + w;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[g][i] = acc[g][i] * corr + w * vf[i];
        m[g] = mn;
      }
    }
  }
  // ---- merge the 8 warps of the CTA through shared memory
  __shared__ float sm_m[ATT_WARPS][MAX_GROUP], sm_l[ATT_WARPS][MAX_GROUP];
  auto sm_acc = [&](int w, int g, int d) -> float& { return sm_acc_raw[((long long)w * group + g) * HD + d]; };
#pragma unroll
  for (int g = 0; g < MAX_GROUP; ++g) {
    if (g < group) {
      if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
      for (int i = 0; i < PER; ++i) sm_acc(warp, g, lane * PER + i) = acc[g][i];
    }
  }
  sync();
  // thread -> (head g, dims d, d + 256/..): 256 threads cover HD dims for one head at a time
  float* part = scratch + (((long long)b * q_heads + kvh * group) * splits + split) * (HD + 2);
  for (int g = 0; g < group; ++g) {
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) ll += (sm_m[w][g] == -CUDART_INF_F) ? 0.f : sm_l[w][g] * __expf(sm_m[w][g] - mm);
    float* pg = part + (long long)g * splits * (HD + 2);
    for (int d = threadIdx.x; d < HD; d += ATT_THREADS) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w)
        a += (sm_m[w][g] == -CUDART_INF_F) ? 0.f : sm_acc(w, g, d) * __expf(sm_m[w][g] - mm);
      pg[d] = a;
    }
    if (threadIdx.x == 0) { pg[HD] = mm; pg[HD + 1] = ll; }
  }
  // ---- the last CTA of this (sequence, kv head) merges the splits
  __shared__ int is_last;
  __threadfence();
  sync();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&counters[b * kv_heads + kvh], 1);
    is_last = (done == splits - 1);
    if (is_last) counters[b * kv_heads + kvh] = 0;      // ready for the next launch
  }
  sync();
  if (!is_last) return;
  __threadfence();
  // weights of every (head, split) first — 64 independent loads at most — then the value sums
  // run over independent loads too (no load -> branch -> load chains through L2)
  __shared__ float w_s[MAX_GROUP][64];
  __shared__ float inv_s[MAX_GROUP];
  const float* pbase = scratch + (((long long)b * q_heads + kvh * group) * splits) * (HD + 2);
  for (int idx = threadIdx.x; idx < group * splits; idx += ATT_THREADS) {
    const int g = idx / splits, s = idx % splits;
    w_s[g][s] = __ldcg(pbase + ((long long)g * splits + s) * (HD + 2) + HD);          // m of the split
  }
  sync();
  if ((int)threadIdx.x < group) {
    const int g = threadIdx.x;
    float mm = -CUDART_INF_F;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, w_s[g][s]);
    float ll = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = w_s[g][s];
      const float wgt = (ms == -CUDART_INF_F) ? 0.f : __expf(ms - mm);
      ll += wgt * __ldcg(pbase + ((long long)g * splits + s) * (HD + 2) + HD + 1);
      w_s[g][s] = wgt;
    }
    inv_s[g] = ll > 0.f ? 1.f / ll : 0.f;
  }
  sync();
  for (int idx = threadIdx.x; idx < group * HD; idx += ATT_THREADS) {
    const int g = idx / HD, d = idx % HD;
    const float* pg = pbase + (long long)g * splits * (HD + 2) + d;
    float a = 0.f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) a += __ldcg(pg + (long long)s * (HD + 2)) * w_s[g][s];
    out[((long long)b * q_heads + kvh * group + g) * HD + d] = __float2bfloat16_rn(a * inv_s[g]);
  }
}

}  // namespace decode_att
}  // namespace mesh
