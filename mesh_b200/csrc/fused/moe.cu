// Expert-parallel routed MoE: dispatch and combine fused with their all-to-all over NVLink peer memory,
// and the device-side planning that lets the expert GEMMs run as descriptor-driven tcgen05 launches
// with no host round trip.
//
//   moe_count     per-expert slot of every (token, choice) and this rank's expert histogram, pushed to
//                 every rank as 8-byte {count, sequence} words
//   moe_plan      from the P x E histogram matrix: where each sender's rows start inside each receiver's
//                 compact per-expert regions (padded to 256 rows), this rank's row layout, and the tile
//                 descriptor tables of its six grouped GEMMs (forward GLU / down, backward dgrad x2, wgrad x2)
//   moe_zero_pad  zero the padding rows of this rank's receive buffer (they feed the ragged-K wgrads)
//   moe_dispatch  every (token, choice) row is stored straight into the destination rank's expert region
//                 (optionally scaled: the backward pass sends w * dOut), then arrival counters are raised
//   moe_combine   after a ready exchange, every token pulls its k expert rows from the peers and sums them
//                 with its routing weights (optionally also the dot products <y, dOut> = gradients of the weights)
//
// Semantics follow the reference's GShard-style example (examples/ep.py:15-70): softmax router, top-k, slots
// assigned in token order, capacity-limited (rows past the receive capacity are dropped and their weight is
// zero), expert SwiGLU, weighted combine; its all-to-all is MPI_Alltoallv with per-pair counts
// (rdma/mesh_compile.py:1571-1579): counts are exchanged, blocks travel at their own sizes, never padded to the largest.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "moe_api.h"
#include "../device/check.cuh"
#include "../device/ptx.cuh"
#include "../gemm/gemm_api.h"
#include "../runtime/host_common.h"

namespace mesh {
namespace moe {

constexpr int R = MESH_MOE_MAX_RANKS;
constexpr int MAX_E = MESH_MOE_MAX_EXPERTS;

__device__ __forceinline__ void ll_store(uint2* p, uint32_t v, uint32_t seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v), "r"(seq) : "memory");
}
__device__ __forceinline__ bool ll_load(const uint2* p, uint32_t seq, uint32_t& v, Status* st) {
  uint2 w;
  unsigned long long t0 = 0;
  uint32_t it = 0;
  while (true) {
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
    if (w.y == seq) { v = w.x; return true; }
    if (((++it) & 0x3ffu) == 0) {
      if (t0 == 0) t0 = globaltimer_ns();
      else if (globaltimer_ns() - t0 > MESH_WAIT_LIMIT_NS || status_aborted(st)) {
        status_record(st, MESH_TIMEOUT, SITE_PEER_FLAG, seq, w.y, (unsigned long long)p);
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- count
// slot[i] = number of earlier entries (token order) routed to the same expert.  A block ranks a chunk of 1024 entries
// (lanes that chose the same expert find each other with a match, warps are ordered through a small table in shared
// memory) and leaves the chunk's histogram in `work`; the block that finishes last turns the histograms into each
// chunk's starting slot per expert, adds them to the slots, and pushes the totals to every rank.
constexpr int COUNT_CHUNK = 1024;

__global__ void __launch_bounds__(COUNT_CHUNK)
moe_count_kernel(const int* __restrict__ idx, int n_entries, int* __restrict__ slot, int experts, int rank, int world,
                 int* __restrict__ work, uint2* c0, uint2* c1, uint2* c2, uint2* c3, uint2* c4, uint2* c5, uint2* c6,
                 uint2* c7, uint32_t seq) {
  __shared__ int cnt[32][MAX_E];            // [warp][expert]: entries of the warp, then entries of the warps before it
  __shared__ int last_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunks = gridDim.x;
  int* hist = work;                         // [chunks][experts]
  int* done = work + (long long)chunks * experts;
  for (int j = threadIdx.x; j < 32 * MAX_E; j += blockDim.x) (&cnt[0][0])[j] = 0;
  __syncthreads();
  const int i = blockIdx.x * COUNT_CHUNK + threadIdx.x;
  const bool valid = i < n_entries;
  const int e = valid ? idx[i] : -1 - lane;                                  // invalid lanes match nobody
  const bool good = valid && e >= 0 && e < experts;
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int in_warp = __popc(same & ((1u << lane) - 1u));
  if (good && in_warp == 0) cnt[warp][e] = __popc(same);
  __syncthreads();
  if ((int)threadIdx.x < experts) {                                          // exclusive scan over the warps
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = cnt[w][threadIdx.x];
      cnt[w][threadIdx.x] = run;
      run += c;
    }
    hist[(long long)blockIdx.x * experts + threadIdx.x] = run;
  }
  __syncthreads();
  if (good) slot[i] = cnt[warp][e] + in_warp;
  else if (valid) slot[i] = 0;
  // ---- the last block to finish completes the slots
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int d = atomicAdd(done, 1);
    last_s = (d == chunks - 1);
    if (last_s) *done = 0;                                                   // ready for the next launch
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  if ((int)threadIdx.x < experts) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      int* h = hist + (long long)c * experts + threadIdx.x;
      const int n = __ldcg(h);
      *h = run;
      run += n;
    }
    if (world > 0) {
      uint2* peers[8] = {c0, c1, c2, c3, c4, c5, c6, c7};
      // count matrix on every rank: [parity][src rank][expert]
      for (int r = 0; r < world; ++r)
        ll_store(peers[r] + ((long long)(seq & 1u) * world + rank) * experts + threadIdx.x, (uint32_t)run, seq);
    }
  }
  __syncthreads();
  for (int j = COUNT_CHUNK + (int)threadIdx.x; j < n_entries; j += COUNT_CHUNK) {   // chunk 0 starts at slot 0
    const int ej = idx[j];
    if (ej >= 0 && ej < experts) slot[j] = __ldcg(slot + j) + hist[(long long)(j / COUNT_CHUNK) * experts + ej];
  }
}

// ------------------------------------------------------------------------------------------- plan
struct PlanArgs {
  const uint2* counts;         // this rank's count matrix [2][world][experts]
  uint32_t seq;
  int rank, world, experts, cap_rows;
  int d_model, d_ff;           // expert shapes: W1 [2*d_ff, d_model], W2 [d_model, d_ff]
  int* send_base;              // [experts]: first row for this sender in the destination's region of expert e
  int* layout;                 // [3 * local experts + 2]: n_e..., base_e..., padded_e..., total_rows, dropped flag
  MeshTileDesc* t_glu; MeshTileDesc* t_down; MeshTileDesc* t_dh; MeshTileDesc* t_dx; MeshTileDesc* t_dw2; MeshTileDesc* t_dw1;
  int* n_tiles;                // [6]
  int max_tiles;
  Status* status;
};

__global__ void __launch_bounds__(512) moe_plan_kernel(const PlanArgs a) {
  __shared__ int C[R][MAX_E];
  __shared__ int n_loc[MAX_E], base_loc[MAX_E], pad_loc[MAX_E];
  __shared__ int ok_s;
  const int E = a.experts, P = a.world, El = E / P;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  for (int i = threadIdx.x; i < P * E; i += blockDim.x) {
    uint32_t v = 0;
    if (!ll_load(a.counts + (long long)(a.seq & 1u) * P * E + i, a.seq, v, a.status)) ok_s = 0;
    C[i / E][i % E] = (int)v;
  }
  __syncthreads();
  if (!ok_s) {
    if (threadIdx.x < 6) a.n_tiles[threadIdx.x] = 0;
    return;
  }
  // every destination's layout is the same function of the matrix; this rank needs all of them as a sender
  if (threadIdx.x < E) {
    const int e = threadIdx.x, d = e / El, el = e % El;
    int base = 0;
    for (int k = 0; k < el; ++k) {
      int n = 0;
      for (int s = 0; s < P; ++s) n += C[s][d * El + k];
      base += (n + 255) / 256 * 256;
    }
    int before = 0;
    for (int s = 0; s < a.rank; ++s) before += C[s][e];
    a.send_base[e] = base + before;
    if (d == a.rank) {
      int n = 0;
      for (int s = 0; s < P; ++s) n += C[s][e];
      n_loc[el] = n;
      base_loc[el] = base;
      pad_loc[el] = (n + 255) / 256 * 256;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0, dropped = 0;
    for (int el = 0; el < El; ++el) {
      // rows past the capacity are dropped by the senders; the receiver clips its regions the same way
      if (base_loc[el] + pad_loc[el] > a.cap_rows) {
        dropped = 1;
        const int room = max(0, a.cap_rows - base_loc[el]) / 256 * 256;
        pad_loc[el] = min(pad_loc[el], room);
        n_loc[el] = min(n_loc[el], pad_loc[el]);
      }
      a.layout[el] = n_loc[el];
      a.layout[El + el] = base_loc[el];
      a.layout[2 * El + el] = pad_loc[el];
      total = max(total, base_loc[el] + pad_loc[el]);
    }
    a.layout[3 * El] = total;
    a.layout[3 * El + 1] = dropped;
  }
  __syncthreads();
  // ---- tile tables (pair tiles: 256 output rows each).  Table t of expert el holds cnt[t][el] descriptors starting at
  // off[t][el]; thread 0 lays the offsets out (6 x local experts additions), then every warp writes the descriptors of
  // its experts, a lane per tile: the tables are thousands of 32-byte records, far too many for one thread.
  __shared__ int off[6][MAX_E + 1];
  const int D = a.d_model, F = a.d_ff;
  const int ntn[6] = {(F + 127) / 128, (D + 255) / 256, (F + 255) / 256, (D + 255) / 256, (F + 255) / 256, (D + 255) / 256};
  const int dw_mt[2] = {(D + 255) / 256, (2 * F + 255) / 256};
  if (threadIdx.x < 6) {
    const int t = threadIdx.x;
    int n = 0;
    for (int el = 0; el < El; ++el) {
      off[t][el] = n;
      const int rows = pad_loc[el];
      n += t < 4 ? (rows / 256) * ntn[t] : (rows >= 64 ? dw_mt[t - 4] * ntn[t] : 0);
    }
    off[t][El] = n;
    a.n_tiles[t] = min(n, a.max_tiles);
  }
  __syncthreads();
  MeshTileDesc* const tab[6] = {a.t_glu, a.t_down, a.t_dh, a.t_dx, a.t_dw2, a.t_dw1};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int el = warp; el < El; el += nwarps) {
    const int base = base_loc[el], kb = pad_loc[el] / 64;
#pragma unroll
    for (int t = 0; t < 6; ++t) {
      const int cnt = off[t][el + 1] - off[t][el];
      for (int j = lane; j < cnt; j += 32) {
        const int at = off[t][el] + j;
        if (at >= a.max_tiles) break;
        const int mt = j / ntn[t], nt = j - mt * ntn[t];
        const int row = base + mt * 256;
        MeshTileDesc d;
        if (t == 0) d = MeshTileDesc{row, 0, D / 64, el * 2 * F + nt * 128, 0, row, nt * 128, 0};            // h = act(x W1g^T) * (x W1u^T)
        else if (t == 1) d = MeshTileDesc{row, 0, F / 64, el * D + nt * 256, 0, row, nt * 256, 0};           // y = h W2^T
        else if (t == 2) d = MeshTileDesc{row, 0, D / 64, nt * 256, el * D, row, nt * 256, 0};               // dH = dY W2   (W2 stacked [El*D, F], MN-major)
        else if (t == 3) d = MeshTileDesc{row, 0, (2 * F) / 64, nt * 256, el * 2 * F, row, nt * 256, 0};     // dX = dGU W1  (W1 stacked [El*2F, D], MN-major)
        else if (t == 4) d = MeshTileDesc{mt * 256, base, kb, nt * 256, 0, el * D + mt * 256, nt * 256, 0};  // dW2[el] = dY^T h   [D, F]
        else d = MeshTileDesc{mt * 256, base, kb, nt * 256, 0, el * 2 * F + mt * 256, nt * 256, 0};          // dW1[el] = dGU^T x  [2F, D]
        tab[t][at] = d;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------- zero padding rows
__global__ void moe_zero_pad_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ layout, int local_experts,
                                    int d_model) {
  const int el = blockIdx.y;
  const int n = layout[el], base = layout[local_experts + el], pad = layout[2 * local_experts + el];
  const long long vec_per_row = d_model / 8;
  const long long total = (long long)(pad - n) * vec_per_row;
  uint4* p = reinterpret_cast<uint4*>(buf + (long long)(base + n) * d_model);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    p[i] = make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------- dispatch
struct DispatchArgs {
  const __nv_bfloat16* x; int tokens, k, d_model;
  const int* idx; const int* slot; const int* send_base; const float* scale;     // scale [tokens, k] or nullptr
  int* meta;                                   // [tokens, k]: row in the destination buffer, or -1 when dropped
  int local_experts, cap_rows, rank, world;
  __nv_bfloat16* recv[R];                      // every rank's receive buffer [cap_rows, d_model]
  uint32_t* arrived[R];                        // every rank's arrival counter for this buffer
  Status* status;
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const DispatchArgs a) {
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_entries = a.tokens * a.k;
  const int vec = a.d_model / 8;
  for (int i = blockIdx.x * warps + warp; i < n_entries; i += gridDim.x * warps) {
    const int e = a.idx[i];
    if (!MESH_CHECK_INDEX(e, a.local_experts * a.world, a.status)) continue;      // an expert id from the router
    const int dest = e / a.local_experts;
    const int row = a.send_base[e] + a.slot[i];
    if (!MESH_CHECK_INDEX(row, 1ll << 30, a.status)) continue;                    // negative: a broken plan
    if (row >= a.cap_rows) {
      if (lane == 0) a.meta[i] = -1;
      continue;
    }
    if (lane == 0) a.meta[i] = row;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + (long long)(i / a.k) * a.d_model);
    uint4* dst = reinterpret_cast<uint4*>(a.recv[dest] + (long long)row * a.d_model);
    if (a.scale == nullptr) {
      for (int v = lane; v < vec; v += 32) dst[v] = __ldg(src + v);
    } else {
      const float s = a.scale[i];
      for (int v = lane; v < vec; v += 32) {
        uint4 q = __ldg(src + v);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float2 f = __bfloat1622float2(h[c]);
          h[c] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        dst[v] = q;
      }
    }
  }
  __syncthreads();                      // the signalling threads' system-scope release covers the block's stores
  if ((int)threadIdx.x < a.world) red_release_sys_add(a.arrived[threadIdx.x], 1u);
}

// ------------------------------------------------------------------------------------------- ready exchange
__global__ void moe_signal_kernel(int world, uint32_t* r0, uint32_t* r1, uint32_t* r2, uint32_t* r3, uint32_t* r4,
                                  uint32_t* r5, uint32_t* r6, uint32_t* r7) {
  uint32_t* peers[8] = {r0, r1, r2, r3, r4, r5, r6, r7};
  __threadfence_system();
  if ((int)threadIdx.x < world) red_release_sys_add(peers[threadIdx.x], 1u);
}

// ------------------------------------------------------------------------------------------- combine
struct CombineArgs {
  int tokens, k, d_model, local_experts, world;
  const int* idx; const int* meta; const float* weight;        // weight nullptr: plain sum (backward of dispatch)
  const __nv_bfloat16* src[R];                 // every rank's expert-output buffer [cap_rows, d_model]
  int cap_rows;                                // rows of every expert-output buffer (checked build)
  const uint32_t* ready; uint32_t ready_expect;               // this rank's counter: all peers finished their experts
  __nv_bfloat16* out;                          // [tokens, d_model]
  const __nv_bfloat16* dot_with; float* dots;  // optional: dots[t, j] = <row, dot_with[t]>
  Status* status;
};

__global__ void __launch_bounds__(256) moe_combine_kernel(const CombineArgs a) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flag_ge(a.ready, a.ready_expect, a.status, SITE_PEER_FLAG) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vec = a.d_model / 8;       // 16-byte vectors per row; a lane owns vectors lane, lane+32, ...
  for (int t = blockIdx.x * warps + warp; t < a.tokens; t += gridDim.x * warps) {
    for (int v = lane; v < vec; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < a.k; ++j) {
        const int row = a.meta[t * a.k + j];
        if (row < 0) continue;
        const int dest = a.idx[t * a.k + j] / a.local_experts;
        if (!MESH_CHECK_INDEX(dest, a.world, a.status) || !MESH_CHECK_INDEX(row, a.cap_rows, a.status)) continue;
        const float w = a.weight ? a.weight[t * a.k + j] : 1.f;
        const uint4 q = __ldcg(reinterpret_cast<const uint4*>(a.src[dest] + (long long)row * a.d_model) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float2 f = __bfloat1622float2(h[c]);
          acc[2 * c] += w * f.x;
          acc[2 * c + 1] += w * f.y;
        }
      }
      if (a.out) {
        uint4 o;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int c = 0; c < 4; ++c) h[c] = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
        reinterpret_cast<uint4*>(a.out + (long long)t * a.d_model)[v] = o;
      }
    }
    if (a.dots) {
      for (int j = 0; j < a.k; ++j) {
        const int row = a.meta[t * a.k + j];
        float d = 0.f;
        if (row >= 0) {
          const int dest = a.idx[t * a.k + j] / a.local_experts;
          for (int v = lane; v < vec; v += 32) {
            const uint4 q = __ldcg(reinterpret_cast<const uint4*>(a.src[dest] + (long long)row * a.d_model) + v);
            const uint4 g = __ldg(reinterpret_cast<const uint4*>(a.dot_with + (long long)t * a.d_model) + v);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
            const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              float2 f = __bfloat1622float2(h[c]), gg = __bfloat1622float2(gh[c]);
              d += f.x * gg.x + f.y * gg.y;
            }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) a.dots[t * a.k + j] = d;
      }
    }
  }
}

}  // namespace moe
}  // namespace mesh

using namespace mesh;
using namespace mesh::moe;

extern "C" int mesh_moe_count_work_ints(int n_entries, int experts) {
  return (n_entries + COUNT_CHUNK - 1) / COUNT_CHUNK * experts + 1;
}

extern "C" int mesh_moe_count(const int* idx, int n_entries, int* slot, int experts, int rank, int world,
                              void* const* count_ptrs, uint32_t seq, int* work, void* stream) {
  if (experts > MAX_E || world > R || experts % world) return set_error(-2, "moe_count: experts <= %d, divisible by world <= %d", MAX_E, R);
  if (n_entries < 1 || work == nullptr) return set_error(-2, "moe_count: no entries or no work buffer");
  uint2* c[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int r = 0; r < world; ++r) c[r] = (uint2*)count_ptrs[r];
  const int chunks = (n_entries + COUNT_CHUNK - 1) / COUNT_CHUNK;
  moe_count_kernel<<<chunks, COUNT_CHUNK, 0, (cudaStream_t)stream>>>(idx, n_entries, slot, experts, rank, world, work, c[0],
                                                                     c[1], c[2], c[3], c[4], c[5], c[6], c[7], seq);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_moe_plan(const MeshMoePlan* m, void* stream) {
  if (m->d_model % 256 || m->d_ff % 64) return set_error(-2, "moe_plan: d_model %% 256 and d_ff %% 64 must be 0");
  PlanArgs a;
  a.counts = (const uint2*)m->counts; a.seq = m->seq; a.rank = m->rank; a.world = m->world; a.experts = m->experts;
  a.cap_rows = m->cap_rows; a.d_model = m->d_model; a.d_ff = m->d_ff;
  a.send_base = m->send_base; a.layout = m->layout;
  a.t_glu = (MeshTileDesc*)m->tables[0]; a.t_down = (MeshTileDesc*)m->tables[1]; a.t_dh = (MeshTileDesc*)m->tables[2];
  a.t_dx = (MeshTileDesc*)m->tables[3]; a.t_dw2 = (MeshTileDesc*)m->tables[4]; a.t_dw1 = (MeshTileDesc*)m->tables[5];
  a.n_tiles = m->n_tiles; a.max_tiles = m->max_tiles; a.status = (Status*)m->status;
  moe_plan_kernel<<<1, 512, 0, (cudaStream_t)stream>>>(a);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_moe_zero_pad(void* buf, const int* layout, int local_experts, int d_model, void* stream) {
  dim3 grid(32, local_experts);
  moe_zero_pad_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, layout, local_experts, d_model);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_moe_dispatch(const MeshMoeDispatch* m, void* stream) {
  if (m->d_model % 8) return set_error(-2, "moe_dispatch: d_model must be a multiple of 8");
  DispatchArgs a;
  a.x = (const __nv_bfloat16*)m->x; a.tokens = m->tokens; a.k = m->k; a.d_model = m->d_model;
  a.idx = m->idx; a.slot = m->slot; a.send_base = m->send_base; a.scale = m->scale; a.meta = m->meta;
  a.local_experts = m->local_experts; a.cap_rows = m->cap_rows; a.rank = m->rank; a.world = m->world;
  for (int r = 0; r < m->world; ++r) { a.recv[r] = (__nv_bfloat16*)m->recv[r]; a.arrived[r] = (uint32_t*)m->arrived[r]; }
  a.status = (Status*)m->status;
  moe_dispatch_kernel<<<MESH_MOE_DISPATCH_BLOCKS, 256, 0, (cudaStream_t)stream>>>(a);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_moe_signal(int world, void* const* ready_ptrs, void* stream) {
  uint32_t* r[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int i = 0; i < world; ++i) r[i] = (uint32_t*)ready_ptrs[i];
  moe_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(world, r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7]);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_moe_combine(const MeshMoeCombine* m, void* stream) {
  CombineArgs a;
  a.tokens = m->tokens; a.k = m->k; a.d_model = m->d_model; a.local_experts = m->local_experts; a.world = m->world;
  a.idx = m->idx; a.meta = m->meta; a.weight = m->weight;
  for (int r = 0; r < m->world; ++r) a.src[r] = (const __nv_bfloat16*)m->src[r];
  a.ready = (const uint32_t*)m->ready; a.ready_expect = m->ready_expect;
  a.out = (__nv_bfloat16*)m->out; a.dot_with = (const __nv_bfloat16*)m->dot_with; a.dots = m->dots;
  a.status = (Status*)m->status;
  a.cap_rows = m->cap_rows > 0 ? m->cap_rows : (1 << 30);
  int grid = (m->tokens + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  moe_combine_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
