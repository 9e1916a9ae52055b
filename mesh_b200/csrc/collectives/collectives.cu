// Collective kernels over the symmetric heap: publish -> bounded wait -> pull (see coll_api.h).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "coll_api.h"
#include "../device/check.cuh"
#include "../device/ptx.cuh"
#include "../runtime/host_common.h"

namespace mesh {
namespace coll {

constexpr int THREADS = 512;
// One block per SM at most: every block waits for every block of every rank, so all of a launch's blocks must be
// resident at once.
constexpr int MAX_BLOCKS = 148;
constexpr int R = MESH_COLL_MAX_RANKS;

struct Comm {
  int rank, world;
  uint8_t* staging[R];
  uint32_t* arrived[R];
  uint32_t expect_a, expect_b;
  uint64_t staging_bytes;
  Status* status;
};

struct VTable {          // per-rank sizes/offsets of the v-collectives, passed by value
  uint64_t a[R + 1];
  uint64_t b[R + 1];
};

__device__ __forceinline__ uint64_t gtid() { return (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; }
__device__ __forceinline__ uint64_t gsize() { return (uint64_t)gridDim.x * blockDim.x; }

// Grid-cooperative byte copy.  16-byte vectors when both ends allow it, bytes otherwise.
__device__ void copy_bytes(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, uint64_t n) {
  if (n == 0) return;
  const bool vec = (((uintptr_t)dst | (uintptr_t)src) & 15) == 0;
  if (vec) {
    const uint64_t nv = n >> 4;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const uint64_t step = gsize();
    uint64_t i = gtid();
    for (; i < nv; i += 4 * step) {        // all of a round's loads are issued before its first store
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * step < nv) v[u] = s[i + u * step];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * step < nv) d[i + u * step] = v[u];
    }
    for (uint64_t j = (nv << 4) + gtid(); j < n; j += step) dst[j] = src[j];
  } else {
    for (uint64_t j = gtid(); j < n; j += gsize()) dst[j] = src[j];
  }
}

// All of this block's earlier stores are made visible system-wide, then one arrival on every
// rank's counter for (step, this rank).  The barrier orders every thread's stores before the signalling threads,
// whose system-scope release is cumulative over them: one fence per signalling thread instead of one per thread
// of the block (a system-scope fence costs microseconds).
__device__ __forceinline__ void signal_all(const Comm& c, int step) {
  __syncthreads();
  if ((int)threadIdx.x < c.world)
    red_release_sys_add(c.arrived[threadIdx.x] + step * c.world + c.rank, 1u);
}

// Bounded wait until the ranks in `mask` have published this call.  False: give up (status written).
__device__ __forceinline__ bool wait_ranks(const Comm& c, int step, uint32_t expect, uint32_t mask) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < c.world && ((mask >> threadIdx.x) & 1u)) {
    if (!wait_flag_ge(c.arrived[c.rank] + step * c.world + threadIdx.x, expect, c.status, SITE_PEER_FLAG)) ok_s = 0;
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  __syncthreads();
  return ok;
}

// ------------------------------------------------------------------------------ element access
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <> struct Acc<__half> { using type = float; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return (typename Acc<T>::type)v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }

template <typename A> __device__ __forceinline__ A combine(A x, A y, int op) {
  switch (op) {
    case MESH_MAX: return x > y ? x : y;
    case MESH_MIN: return x < y ? x : y;
    case MESH_PROD: return x * y;
    default: return x + y;
  }
}

// One 16-byte vector of the result from the `nw` vectors w[0..nw) (fixed order 0..nw-1).
template <typename T, int NW>
__device__ __forceinline__ uint4 reduce_vec(const uint4 (&w)[NW], int nw, int op, float avg) {
  using A = typename Acc<T>::type;
  constexpr int V = 16 / sizeof(T);
  A acc[V];
  const T* e0 = reinterpret_cast<const T*>(&w[0]);
#pragma unroll
  for (int k = 0; k < V; ++k) acc[k] = to_acc<T>(e0[k]);
#pragma unroll
  for (int r = 1; r < NW; ++r) {
    if (r < nw) {
      const T* e = reinterpret_cast<const T*>(&w[r]);
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] = combine<A>(acc[k], to_acc<T>(e[k]), op);
    }
  }
  uint4 o;
  T* eo = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int k = 0; k < V; ++k) {
    if (op == MESH_AVG) acc[k] = (A)((float)acc[k] * avg);
    eo[k] = from_acc<T>(acc[k]);
  }
  return o;
}

// Vector part of the pull reduction with the number of ranks W known at compile time and U vectors per thread in
// flight from every rank (the loads cross NVLink: bytes in flight set the rate).
template <typename T, int W, int U>
__device__ void reduce_pull_vec(const Comm& c, uint64_t src_byte_off, T* __restrict__ out, uint64_t nv, int op) {
  const float avg = 1.0f / (float)c.world;
  const uint4* src[W];
#pragma unroll
  for (int r = 0; r < W; ++r) src[r] = reinterpret_cast<const uint4*>(c.staging[r < c.world ? r : 0] + src_byte_off);
  const uint64_t step = gsize();
  uint64_t i = gtid();
  for (; i + (U - 1) * step < nv; i += U * step) {
    uint4 w[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < c.world) w[u][r] = __ldcg(src[r] + i + u * step);
#pragma unroll
    for (int u = 0; u < U; ++u) reinterpret_cast<uint4*>(out)[i + u * step] = reduce_vec<T, W>(w[u], c.world, op, avg);
  }
  for (; i < nv; i += step) {
    uint4 w[W];
#pragma unroll
    for (int r = 0; r < W; ++r)
      if (r < c.world) w[r] = __ldcg(src[r] + i);
    reinterpret_cast<uint4*>(out)[i] = reduce_vec<T, W>(w, c.world, op, avg);
  }
}

template <typename T> __device__ __forceinline__ T ld_elem(const uint8_t* base, uint64_t i) {
  return __ldcg(reinterpret_cast<const T*>(base) + i);
}
template <> __device__ __forceinline__ __nv_bfloat16 ld_elem<__nv_bfloat16>(const uint8_t* base, uint64_t i) {
  unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(base) + i);
  return *reinterpret_cast<__nv_bfloat16*>(&raw);
}
template <> __device__ __forceinline__ __half ld_elem<__half>(const uint8_t* base, uint64_t i) {
  unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(base) + i);
  return *reinterpret_cast<__half*>(&raw);
}

// out[i] = reduce over ranks (fixed order 0..world-1) of src_r[i], for i in [0, n): the sources
// are `world` buffers at the same offset of each rank's staging.
template <typename T>
__device__ void reduce_pull(const Comm& c, uint64_t src_byte_off, T* __restrict__ out, uint64_t n, int op) {
  using A = typename Acc<T>::type;
  constexpr int V = 16 / sizeof(T);
  const bool vec = (((uintptr_t)out) & 15) == 0 && (src_byte_off & 15) == 0;
  uint64_t done = 0;
  if (vec) {
    const uint64_t nv = n / V;
    if (c.world <= 2) reduce_pull_vec<T, 2, 4>(c, src_byte_off, out, nv, op);
    else if (c.world <= 4) reduce_pull_vec<T, 4, 2>(c, src_byte_off, out, nv, op);
    else reduce_pull_vec<T, R, 1>(c, src_byte_off, out, nv, op);
    done = nv * V;
  }
  const float avg = 1.0f / (float)c.world;
  for (uint64_t i = done + gtid(); i < n; i += gsize()) {
    A acc = to_acc<T>(ld_elem<T>(c.staging[0] + src_byte_off, i));
    for (int r = 1; r < c.world; ++r) acc = combine<A>(acc, to_acc<T>(ld_elem<T>(c.staging[r] + src_byte_off, i)), op);
    if (op == MESH_AVG) acc = (A)((float)acc * avg);
    out[i] = from_acc<T>(acc);
  }
}

constexpr uint64_t HDR = MESH_COLL_HEADER_BYTES;

// ------------------------------------------------------------------------------ kernels
template <typename T>
__global__ void __launch_bounds__(THREADS) allreduce_kernel(Comm c, const T* in, T* out, uint64_t count, int op, int two_shot) {
  const uint32_t all = (1u << c.world) - 1u;
  copy_bytes(c.staging[c.rank] + HDR, reinterpret_cast<const uint8_t*>(in), count * sizeof(T));
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, all)) return;
  if (!two_shot) {
    reduce_pull<T>(c, HDR, out, count, op);
    return;
  }
  // two-shot: this rank reduces its slice into the second half of its own staging, then every rank
  // gathers the reduced slices.
  constexpr uint64_t V = 16 / sizeof(T);
  const uint64_t per = ((count + c.world - 1) / c.world + V - 1) / V * V;
  const uint64_t half = (c.staging_bytes / 2) & ~(uint64_t)15;
  const uint64_t lo = min(count, (uint64_t)c.rank * per), hi = min(count, lo + per);
  T* mine = reinterpret_cast<T*>(c.staging[c.rank] + HDR + half) + lo;
  reduce_pull<T>(c, HDR + lo * sizeof(T), mine, hi - lo, op);
  signal_all(c, 1);
  if (!wait_ranks(c, 1, c.expect_b, all)) return;
  for (int s = 0; s < c.world; ++s) {
    const int r = (c.rank + s) % c.world;                // start with the own slice, then spread over peers
    const uint64_t l = min(count, (uint64_t)r * per), h = min(count, l + per);
    copy_bytes(reinterpret_cast<uint8_t*>(out + l), c.staging[r] + HDR + half + l * sizeof(T), (h - l) * sizeof(T));
  }
}

__global__ void __launch_bounds__(THREADS) allgatherv_kernel(Comm c, const uint8_t* in, uint8_t* out, VTable t) {
  // t.a = counts (bytes), t.b = displacements (bytes) in the output
  copy_bytes(c.staging[c.rank] + HDR, in, t.a[c.rank]);
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  for (int s = 0; s < c.world; ++s) {
    const int r = (c.rank + s) % c.world;
    copy_bytes(out + t.b[r], c.staging[r] + HDR, t.a[r]);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) reduce_scatter_kernel(Comm c, const T* in, T* out, VTable t, int op) {
  // t.a = element counts per rank, t.b = element offsets (prefix sums) in the input
  copy_bytes(c.staging[c.rank] + HDR, reinterpret_cast<const uint8_t*>(in), t.b[c.world] * sizeof(T));
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  reduce_pull<T>(c, HDR + t.b[c.rank] * sizeof(T), out, t.a[c.rank], op);
}

__global__ void __launch_bounds__(THREADS) alltoallv_kernel(Comm c, const uint8_t* in, uint8_t* out, VTable t) {
  // t.a = this rank's send offsets (world+1), t.b = its receive offsets (world+1), in bytes.  The
  // send offsets are published in the staging header so that readers find their block.
  if (blockIdx.x == 0 && (int)threadIdx.x <= c.world)
    reinterpret_cast<uint64_t*>(c.staging[c.rank])[threadIdx.x] = t.a[threadIdx.x];
  copy_bytes(c.staging[c.rank] + HDR + t.a[0], in + t.a[0], t.a[c.world] - t.a[0]);
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  for (int s = 0; s < c.world; ++s) {
    const int r = (c.rank + s) % c.world;
    const volatile uint64_t* hdr = reinterpret_cast<const volatile uint64_t*>(c.staging[r]);
    const uint64_t lo = hdr[c.rank], hi = hdr[c.rank + 1];
    // the block's bounds come from the sender's header: in a checked build they must lie inside its staging buffer
    if (!MESH_CHECK_INDEX(hi, c.staging_bytes + 1, c.status) || !MESH_CHECK_INDEX(lo, hi + 1, c.status)) continue;
    const uint64_t room = t.b[r + 1] - t.b[r];
    copy_bytes(out + t.b[r], c.staging[r] + HDR + lo, min(hi - lo, room));
  }
}

// Staging buffers alternate call by call, so call k+2 overwrites what call k published.  That is safe only if every
// rank's call k+1 saw every peer's arrival for call k+1 (a peer arrives after its call k has finished, by stream
// order).  Hence every rank of a broadcast or a reduce waits for all arrivals, also the ranks that read nothing.
__global__ void __launch_bounds__(THREADS) broadcast_kernel(Comm c, uint8_t* buf, uint64_t bytes, int root) {
  if (c.rank == root) copy_bytes(c.staging[c.rank] + HDR, buf, bytes);
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  if (c.rank == root) return;
  copy_bytes(buf, c.staging[root] + HDR, bytes);
}

template <typename T>
__global__ void __launch_bounds__(THREADS) reduce_kernel(Comm c, const T* in, T* out, uint64_t count, int op, int root) {
  copy_bytes(c.staging[c.rank] + HDR, reinterpret_cast<const uint8_t*>(in), count * sizeof(T));
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  if (c.rank != root) return;
  reduce_pull<T>(c, HDR, out, count, op);
}

__global__ void __launch_bounds__(THREADS) barrier_kernel(Comm c) {
  signal_all(c, 0);
  wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u);
}

// Block-scope byte copy (the calling block copies all n bytes), eight 16-byte loads in flight per thread: the
// source may be a peer's memory, where the latency is a few microseconds.
__device__ void copy_bytes_block(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, uint64_t n) {
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const uint64_t nv = n >> 4, step = blockDim.x;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    uint64_t i = threadIdx.x;
    for (; i < nv; i += 8 * step) {        // all of a round's loads are issued before its first store
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * step < nv) v[u] = __ldcg(s + i + u * step);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * step < nv) d[i + u * step] = v[u];
    }
    for (uint64_t j = (nv << 4) + threadIdx.x; j < n; j += step) dst[j] = src[j];
  } else {
    for (uint64_t j = threadIdx.x; j < n; j += blockDim.x) dst[j] = src[j];
  }
}

// Pipelined point-to-point exchange: one launch plays this rank's sending and receiving roles of a message (or of a
// collective permute) at once.  A message travels in pieces through a ring of `depth` slots in the SENDER's memory:
// the sender stages a piece locally and raises `ready` at the receiver; the receiver pulls the piece over NVLink
// straight into its destination and raises `ack` at the sender, which frees the slot.  Pulling keeps the expensive
// step (a system-scope fence behind stores that crossed the link) off the path: the only stores that cross are the
// counters.  `nb` blocks per role each move 1/nb of every piece.  Counters are monotonic: `ready` counts
// sender-block arrivals, `ack` receiver-block arrivals; the `*_base` values are the totals of all earlier messages
// on the channel, known to both ends from the call sequence.
struct XferChan {
  uint8_t* slot; uint32_t* ready; uint32_t* ack; uint32_t ready_base, ack_base;
};
struct Xfer {
  int n_send, has_recv, nb, depth;
  XferChan send[R];
  XferChan recv;
  const uint8_t* in; uint8_t* out;
  uint64_t send_bytes, recv_bytes, piece;
  Status* st;
};

__global__ void __launch_bounds__(THREADS) exchange_kernel(const __grid_constant__ Xfer x) {
  __shared__ int ok_s;
  const int role = blockIdx.x / x.nb, b = blockIdx.x % x.nb;
  const bool sender = role < x.n_send;
  const XferChan& ch = sender ? x.send[role] : x.recv;
  const uint64_t bytes = sender ? x.send_bytes : x.recv_bytes;
  const uint64_t pieces = (bytes + x.piece - 1) / x.piece;
  if (sender) {
    // every earlier message on this channel has been pulled, so the whole ring is free
    if (threadIdx.x == 0) ok_s = wait_flag_ge(ch.ack, ch.ack_base, x.st, SITE_PEER_FLAG) ? 1 : 0;
    __syncthreads();
    if (!ok_s) return;
  }
  for (uint64_t i = 0; i < pieces; ++i) {
    const uint64_t lo = i * x.piece, len = min(x.piece, bytes - lo);
    const uint64_t part = ((len + x.nb - 1) / x.nb + 15) & ~(uint64_t)15;
    const uint64_t p0 = min(len, (uint64_t)b * part), p1 = min(len, p0 + part);
    uint8_t* slot = ch.slot + (i % x.depth) * x.piece;
    if (sender) {
      if (i >= (uint64_t)x.depth) {
        if (threadIdx.x == 0)
          ok_s = wait_flag_ge(ch.ack, ch.ack_base + (uint32_t)(i - x.depth + 1) * x.nb, x.st, SITE_PEER_FLAG) ? 1 : 0;
        __syncthreads();
        if (!ok_s) return;
      }
      copy_bytes_block(slot + p0, x.in + lo + p0, p1 - p0);
      __syncthreads();                    // then thread 0's release covers the whole block's stores
      if (threadIdx.x == 0) red_release_sys_add(ch.ready, 1u);
    } else {
      if (threadIdx.x == 0)
        ok_s = wait_flag_ge(ch.ready, ch.ready_base + (uint32_t)(i + 1) * x.nb, x.st, SITE_PEER_FLAG) ? 1 : 0;
      __syncthreads();
      if (!ok_s) return;
      copy_bytes_block(x.out + lo + p0, slot + p0, p1 - p0);
      __syncthreads();                    // every thread's loads have returned (their values were stored)
      if (threadIdx.x == 0) red_release_sys_add(ch.ack, 1u);
    }
  }
}

__global__ void wait_flag_test_kernel(const uint32_t* flag, uint32_t expect, unsigned long long limit_ns, Status* st) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_flag_ge(flag, expect, st, SITE_HOST_FLAG, limit_ns);
}

// ------------------------------------------------------------------------------ in-switch all-reduce (NVLS)
// With a multicast mapping of the heap, one `multimem.ld_reduce` returns the sum over every rank's copy of an address
// (the switch adds) and one `multimem.st` writes a value into every rank's copy.  Two-shot form: this rank reduces its
// slice through the multicast address of the staging buffers' first half and broadcasts the result into their
// second half; after the second round of signals every rank copies the complete result out of its own memory.
// Sum only; bf16 / f16 accumulate in fp32 inside the switch.
template <typename T> struct McOps;
template <> struct McOps<float> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct McOps<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct McOps<__half> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

template <typename T>
__global__ void __launch_bounds__(THREADS) allreduce_mc_kernel(Comm c, uint8_t* mc_staging, const T* in, T* out, uint64_t count) {
  const uint32_t all = (1u << c.world) - 1u;
  constexpr uint64_t V = 16 / sizeof(T);
  const uint64_t padded = (count + V - 1) / V * V;
  copy_bytes(c.staging[c.rank] + HDR, reinterpret_cast<const uint8_t*>(in), count * sizeof(T));
  // the tail of the last vector must not hold stale data: it is summed by the switch like everything else
  for (uint64_t i = count + gtid(); i < padded; i += gsize()) reinterpret_cast<T*>(c.staging[c.rank] + HDR)[i] = T(0);
  signal_all(c, 0);
  if (!wait_ranks(c, 0, c.expect_a, all)) return;
  const uint64_t nv = padded / V;
  const uint64_t per = (nv + c.world - 1) / c.world;
  const uint64_t lo = min(nv, (uint64_t)c.rank * per), hi = min(nv, lo + per);
  const uint64_t half = (c.staging_bytes / 2) & ~(uint64_t)15;
  uint4* src = reinterpret_cast<uint4*>(mc_staging + HDR);
  uint4* dst = reinterpret_cast<uint4*>(mc_staging + HDR + half);
  for (uint64_t i = lo + gtid(); i < hi; i += gsize()) McOps<T>::st(dst + i, McOps<T>::ld(src + i));
  signal_all(c, 1);
  if (!wait_ranks(c, 1, c.expect_b, all)) return;
  copy_bytes(reinterpret_cast<uint8_t*>(out), c.staging[c.rank] + HDR + half, count * sizeof(T));
}

// ------------------------------------------------------------------------------ host side
static int make_comm(const MeshCommArgs* a, Comm* c) {
  if (a->world < 1 || a->world > R) return set_error(-4, "collective: world %d out of range", a->world);
  c->rank = a->rank;
  c->world = a->world;
  for (int r = 0; r < a->world; ++r) {
    c->staging[r] = (uint8_t*)a->staging[r];
    c->arrived[r] = a->arrived[r];
  }
  c->expect_a = a->expect_a;
  c->expect_b = a->expect_b;
  c->staging_bytes = a->staging_bytes;
  c->status = (Status*)a->status;
  return 0;
}

static int grid_of(const MeshCommArgs* a) {
  int n = a->nblocks;
  if (n < 1) n = 1;
  if (n > MAX_BLOCKS) n = MAX_BLOCKS;
  return n;
}

template <typename T>
static int launch_allreduce(const Comm& c, int grid, const void* in, void* out, uint64_t count, int op, int two, cudaStream_t s) {
  allreduce_kernel<T><<<grid, THREADS, 0, s>>>(c, (const T*)in, (T*)out, count, op, two);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
template <typename T>
static int launch_rs(const Comm& c, int grid, const void* in, void* out, const VTable& t, int op, cudaStream_t s) {
  reduce_scatter_kernel<T><<<grid, THREADS, 0, s>>>(c, (const T*)in, (T*)out, t, op);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
template <typename T>
static int launch_reduce(const Comm& c, int grid, const void* in, void* out, uint64_t count, int op, int root, cudaStream_t s) {
  reduce_kernel<T><<<grid, THREADS, 0, s>>>(c, (const T*)in, (T*)out, count, op, root);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

static uint64_t esize(int dtype) {
  switch (dtype) {
    case MESH_F32: case MESH_I32: return 4;
    case MESH_BF16: case MESH_F16: return 2;
    case MESH_I64: case MESH_F64: return 8;
    default: return 1;
  }
}

#define MESH_DISPATCH_DTYPE(dtype, CALL)                                  \
  switch (dtype) {                                                        \
    case MESH_F32: return CALL(float);                                    \
    case MESH_BF16: return CALL(__nv_bfloat16);                           \
    case MESH_F16: return CALL(__half);                                   \
    case MESH_I32: return CALL(int);                                      \
    case MESH_I64: return CALL(long long);                                \
    case MESH_F64: return CALL(double);                                   \
    case MESH_U8: return CALL(unsigned char);                             \
    default: return set_error(-9, "collective: unsupported dtype %d", dtype); \
  }

}  // namespace coll
}  // namespace mesh

using namespace mesh;
using namespace mesh::coll;

extern "C" int mesh_coll_max_blocks(void) { return MAX_BLOCKS; }

extern "C" int mesh_coll_allreduce(const MeshCommArgs* a, const void* in, void* out, uint64_t count, int dtype, int op,
                                   int two_shot, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  const uint64_t bytes = count * esize(dtype);
  const uint64_t cap = two_shot ? (a->staging_bytes / 2 & ~15ull) : a->staging_bytes;
  if (bytes > cap) return set_error(-10, "allreduce: %llu bytes exceed the staging capacity %llu", (unsigned long long)bytes, (unsigned long long)cap);
  const int grid = grid_of(a);
#define CALL(T) launch_allreduce<T>(c, grid, in, out, count, op, two_shot, (cudaStream_t)stream)
  MESH_DISPATCH_DTYPE(dtype, CALL)
#undef CALL
}

// In-switch variant: `mc_staging` is the multicast address of this call's staging buffer.  Sum of f32 / bf16 / f16 only.
extern "C" int mesh_coll_allreduce_mc(const MeshCommArgs* a, void* mc_staging, const void* in, void* out, uint64_t count,
                                      int dtype, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  if (mc_staging == nullptr) return set_error(-11, "allreduce_mc: the heap has no multicast mapping");
  const uint64_t bytes = (count * esize(dtype) + 15) & ~15ull;
  if (bytes > (a->staging_bytes / 2 & ~15ull)) return set_error(-10, "allreduce_mc: message exceeds half the staging buffer");
  const int grid = grid_of(a);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case MESH_F32: allreduce_mc_kernel<float><<<grid, THREADS, 0, s>>>(c, (uint8_t*)mc_staging, (const float*)in, (float*)out, count); break;
    case MESH_BF16: allreduce_mc_kernel<__nv_bfloat16><<<grid, THREADS, 0, s>>>(c, (uint8_t*)mc_staging, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, count); break;
    case MESH_F16: allreduce_mc_kernel<__half><<<grid, THREADS, 0, s>>>(c, (uint8_t*)mc_staging, (const __half*)in, (__half*)out, count); break;
    default: return set_error(-9, "allreduce_mc: sums of f32, bf16 and f16 only");
  }
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_coll_allgatherv(const MeshCommArgs* a, const void* in, void* out, const uint64_t* counts,
                                    const uint64_t* displs, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  VTable t;
  for (int r = 0; r < a->world; ++r) {
    t.a[r] = counts[r];
    t.b[r] = displs[r];
    if (counts[r] > a->staging_bytes) return set_error(-10, "allgather: block exceeds the staging capacity");
  }
  allgatherv_kernel<<<grid_of(a), THREADS, 0, (cudaStream_t)stream>>>(c, (const uint8_t*)in, (uint8_t*)out, t);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_coll_allgather(const MeshCommArgs* a, const void* in, void* out, uint64_t bytes_per_rank, void* stream) {
  uint64_t counts[R], displs[R];
  for (int r = 0; r < a->world && r < R; ++r) {
    counts[r] = bytes_per_rank;
    displs[r] = bytes_per_rank * r;
  }
  return mesh_coll_allgatherv(a, in, out, counts, displs, stream);
}

extern "C" int mesh_coll_reduce_scatter(const MeshCommArgs* a, const void* in, void* out, const uint64_t* counts_elems,
                                        int dtype, int op, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  VTable t;
  uint64_t off = 0;
  for (int r = 0; r < a->world; ++r) {
    t.a[r] = counts_elems[r];
    t.b[r] = off;
    off += counts_elems[r];
  }
  t.b[a->world] = off;
  if (off * esize(dtype) > a->staging_bytes) return set_error(-10, "reduce_scatter: input exceeds the staging capacity");
  const int grid = grid_of(a);
#define CALL(T) launch_rs<T>(c, grid, in, out, t, op, (cudaStream_t)stream)
  MESH_DISPATCH_DTYPE(dtype, CALL)
#undef CALL
}

extern "C" int mesh_coll_alltoallv(const MeshCommArgs* a, const void* in, void* out, const uint64_t* send_off,
                                   const uint64_t* recv_off, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  VTable t;
  for (int r = 0; r <= a->world; ++r) {
    t.a[r] = send_off[r];
    t.b[r] = recv_off[r];
  }
  if (send_off[a->world] > a->staging_bytes) return set_error(-10, "alltoall: input exceeds the staging capacity");
  alltoallv_kernel<<<grid_of(a), THREADS, 0, (cudaStream_t)stream>>>(c, (const uint8_t*)in, (uint8_t*)out, t);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_coll_broadcast(const MeshCommArgs* a, void* buf, uint64_t bytes, int root, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  if (bytes > a->staging_bytes) return set_error(-10, "broadcast: message exceeds the staging capacity");
  broadcast_kernel<<<grid_of(a), THREADS, 0, (cudaStream_t)stream>>>(c, (uint8_t*)buf, bytes, root);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_coll_reduce(const MeshCommArgs* a, const void* in, void* out, uint64_t count, int dtype, int op,
                                int root, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  if (count * esize(dtype) > a->staging_bytes) return set_error(-10, "reduce: message exceeds the staging capacity");
  const int grid = grid_of(a);
#define CALL(T) launch_reduce<T>(c, grid, in, out, count, op, root, (cudaStream_t)stream)
  MESH_DISPATCH_DTYPE(dtype, CALL)
#undef CALL
}

extern "C" int mesh_coll_barrier(const MeshCommArgs* a, void* stream) {
  Comm c;
  if (int rc = make_comm(a, &c)) return rc;
  barrier_kernel<<<1, THREADS, 0, (cudaStream_t)stream>>>(c);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_p2p_exchange(const MeshXferArgs* a, void* stream) {
  if (a->n_send < 0 || a->n_send > R || a->nb < 1 || a->nb > 64 || a->depth < 1 || a->piece == 0 || (a->piece & 15))
    return set_error(-4, "p2p_exchange: bad arguments");
  Xfer x;
  x.n_send = a->n_send; x.has_recv = a->has_recv; x.nb = a->nb; x.depth = a->depth;
  for (int i = 0; i < a->n_send; ++i)
    x.send[i] = XferChan{(uint8_t*)a->send[i].slot, a->send[i].ready, a->send[i].ack, a->send[i].ready_base, a->send[i].ack_base};
  x.recv = XferChan{(uint8_t*)a->recv.slot, a->recv.ready, a->recv.ack, a->recv.ready_base, a->recv.ack_base};
  x.in = (const uint8_t*)a->in; x.out = (uint8_t*)a->out;
  x.send_bytes = a->send_bytes; x.recv_bytes = a->recv_bytes; x.piece = a->piece;
  x.st = (Status*)a->status;
  const int roles = a->n_send + (a->has_recv ? 1 : 0);
  if (roles == 0) return 0;
  exchange_kernel<<<roles * a->nb, THREADS, 0, (cudaStream_t)stream>>>(x);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_wait_flag_test(const uint32_t* flag, uint32_t expect, uint64_t limit_ns, void* status, void* stream) {
  wait_flag_test_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag, expect, limit_ns, (Status*)status);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
