// Collective kernels over the symmetric heap: publish -> bounded wait -> pull (see coll_api.h).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "coll_api.h"
#include "../device/ptx.cuh"
#include "../runtime/host_common.h"

namespace mesh {
namespace coll {

constexpr int THREADS = 512;
constexpr int MAX_BLOCKS = 64;
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
    for (; i + 3 * step < nv; i += 4 * step) {
      uint4 v0 = s[i], v1 = s[i + step], v2 = s[i + 2 * step], v3 = s[i + 3 * step];
      d[i] = v0; d[i + step] = v1; d[i + 2 * step] = v2; d[i + 3 * step] = v3;
    }
    for (; i < nv; i += step) d[i] = s[i];
    for (uint64_t j = (nv << 4) + gtid(); j < n; j += step) dst[j] = src[j];
  } else {
    for (uint64_t j = gtid(); j < n; j += gsize()) dst[j] = src[j];
  }
}

// All of this block's earlier stores are made visible system-wide, then one arrival on every
// rank's counter for (step, this rank).
__device__ __forceinline__ void signal_all(const Comm& c, int step) {
  __threadfence_system();
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

// out[i] = reduce over ranks (fixed order 0..world-1) of src_r[i], for i in [0, n): the sources
// are `world` buffers at the same offset of each rank's staging.
template <typename T>
__device__ void reduce_pull(const Comm& c, uint64_t src_byte_off, T* __restrict__ out, uint64_t n, int op) {
  using A = typename Acc<T>::type;
  constexpr int V = 16 / sizeof(T);
  const bool vec = (((uintptr_t)out) & 15) == 0 && (src_byte_off & 15) == 0;
  const float avg = 1.0f / (float)c.world;
  uint64_t done = 0;
  if (vec) {
    const uint64_t nv = n / V;
    for (uint64_t i = gtid(); i < nv; i += gsize()) {
      uint4 w[R];
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r < c.world) w[r] = __ldcg(reinterpret_cast<const uint4*>(c.staging[r] + src_byte_off) + i);
      A acc[V];
      const T* e0 = reinterpret_cast<const T*>(&w[0]);
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] = to_acc<T>(e0[k]);
#pragma unroll
      for (int r = 1; r < R; ++r) {
        if (r < c.world) {
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
      reinterpret_cast<uint4*>(out)[i] = o;
    }
    done = nv * V;
  }
  for (uint64_t i = done + gtid(); i < n; i += gsize()) {
    A acc = to_acc<T>(reinterpret_cast<const volatile T*>(c.staging[0] + src_byte_off)[i]);
    for (int r = 1; r < c.world; ++r)
      acc = combine<A>(acc, to_acc<T>(reinterpret_cast<const volatile T*>(c.staging[r] + src_byte_off)[i]), op);
    if (op == MESH_AVG) acc = (A)((float)acc * avg);
    out[i] = from_acc<T>(acc);
  }
}
// volatile reads of bf16/half need plain types
template <> __device__ void reduce_pull<__nv_bfloat16>(const Comm& c, uint64_t off, __nv_bfloat16* __restrict__ out,
                                                      uint64_t n, int op);
template <> __device__ void reduce_pull<__half>(const Comm& c, uint64_t off, __half* __restrict__ out, uint64_t n, int op);

template <typename T16, typename Cvt>
__device__ void reduce_pull16(const Comm& c, uint64_t src_byte_off, T16* __restrict__ out, uint64_t n, int op, Cvt) {
  const bool vec = (((uintptr_t)out) & 15) == 0 && (src_byte_off & 15) == 0;
  const float avg = 1.0f / (float)c.world;
  uint64_t done = 0;
  if (vec) {
    const uint64_t nv = n / 8;
    for (uint64_t i = gtid(); i < nv; i += gsize()) {
      uint4 w[R];
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r < c.world) w[r] = __ldcg(reinterpret_cast<const uint4*>(c.staging[r] + src_byte_off) + i);
      float acc[8];
      const T16* e0 = reinterpret_cast<const T16*>(&w[0]);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = to_acc<T16>(e0[k]);
#pragma unroll
      for (int r = 1; r < R; ++r) {
        if (r < c.world) {
          const T16* e = reinterpret_cast<const T16*>(&w[r]);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] = combine<float>(acc[k], to_acc<T16>(e[k]), op);
        }
      }
      uint4 o;
      T16* eo = reinterpret_cast<T16*>(&o);
#pragma unroll
      for (int k = 0; k < 8; ++k) eo[k] = from_acc<T16>(op == MESH_AVG ? acc[k] * avg : acc[k]);
      reinterpret_cast<uint4*>(out)[i] = o;
    }
    done = nv * 8;
  }
  for (uint64_t i = done + gtid(); i < n; i += gsize()) {
    const unsigned short* p0 = reinterpret_cast<const unsigned short*>(c.staging[0] + src_byte_off);
    unsigned short raw = __ldcg(p0 + i);
    float acc = to_acc<T16>(*reinterpret_cast<T16*>(&raw));
    for (int r = 1; r < c.world; ++r) {
      raw = __ldcg(reinterpret_cast<const unsigned short*>(c.staging[r] + src_byte_off) + i);
      acc = combine<float>(acc, to_acc<T16>(*reinterpret_cast<T16*>(&raw)), op);
    }
    out[i] = from_acc<T16>(op == MESH_AVG ? acc * avg : acc);
  }
}
template <> __device__ void reduce_pull<__nv_bfloat16>(const Comm& c, uint64_t off, __nv_bfloat16* __restrict__ out,
                                                      uint64_t n, int op) {
  reduce_pull16<__nv_bfloat16>(c, off, out, n, op, 0);
}
template <> __device__ void reduce_pull<__half>(const Comm& c, uint64_t off, __half* __restrict__ out, uint64_t n, int op) {
  reduce_pull16<__half>(c, off, out, n, op, 0);
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
    const uint64_t room = t.b[r + 1] - t.b[r];
    copy_bytes(out + t.b[r], c.staging[r] + HDR + lo, min(hi - lo, room));
  }
}

__global__ void __launch_bounds__(THREADS) broadcast_kernel(Comm c, uint8_t* buf, uint64_t bytes, int root) {
  if (c.rank == root) copy_bytes(c.staging[c.rank] + HDR, buf, bytes);
  signal_all(c, 0);
  if (c.rank == root) return;
  if (!wait_ranks(c, 0, c.expect_a, 1u << root)) return;
  copy_bytes(buf, c.staging[root] + HDR, bytes);
}

template <typename T>
__global__ void __launch_bounds__(THREADS) reduce_kernel(Comm c, const T* in, T* out, uint64_t count, int op, int root) {
  copy_bytes(c.staging[c.rank] + HDR, reinterpret_cast<const uint8_t*>(in), count * sizeof(T));
  signal_all(c, 0);
  if (c.rank != root) return;
  if (!wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u)) return;
  reduce_pull<T>(c, HDR, out, count, op);
}

__global__ void __launch_bounds__(THREADS) barrier_kernel(Comm c) {
  signal_all(c, 0);
  wait_ranks(c, 0, c.expect_a, (1u << c.world) - 1u);
}

__global__ void __launch_bounds__(THREADS) p2p_send_kernel(uint8_t* slot, uint32_t* ready, const uint32_t* ack, uint32_t seq,
                                                         const uint8_t* in, uint64_t bytes, Status* st) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flag_ge(ack, seq - 1, st, SITE_PEER_FLAG) ? 1 : 0;   // slot is free again
  __syncthreads();
  if (!ok_s) return;
  copy_bytes(slot, in, bytes);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) red_release_sys_add(ready, 1u);     // one arrival per block; receiver expects seq*blocks
}

__global__ void __launch_bounds__(THREADS) p2p_recv_kernel(const uint8_t* slot, const uint32_t* ready, uint32_t* ack,
                                                         uint32_t expect_ready, uint8_t* out, uint64_t bytes, Status* st) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = wait_flag_ge(ready, expect_ready, st, SITE_PEER_FLAG) ? 1 : 0;
  __syncthreads();
  if (!ok_s) return;
  copy_bytes(out, slot, bytes);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) red_release_sys_add(ack, 1u);
}

__global__ void wait_flag_test_kernel(const uint32_t* flag, uint32_t expect, unsigned long long limit_ns, Status* st) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_flag_ge(flag, expect, st, SITE_HOST_FLAG, limit_ns);
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

// p2p messages use a fixed grid so that `ready` advances by the same amount per message on both ends
static const int P2P_BLOCKS = 16;
extern "C" int mesh_p2p_send(const MeshP2PArgs* a, const void* in, uint64_t bytes, void* stream) {
  p2p_send_kernel<<<P2P_BLOCKS, THREADS, 0, (cudaStream_t)stream>>>((uint8_t*)a->slot, a->ready, a->ack,
                                                                   (a->seq - 1) * P2P_BLOCKS + 1, (const uint8_t*)in, bytes,
                                                                   (Status*)a->status);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
extern "C" int mesh_p2p_recv(const MeshP2PArgs* a, void* out, uint64_t bytes, void* stream) {
  p2p_recv_kernel<<<P2P_BLOCKS, THREADS, 0, (cudaStream_t)stream>>>((const uint8_t*)a->slot, a->ready, a->ack,
                                                                   a->seq * P2P_BLOCKS, (uint8_t*)out, bytes,
                                                                   (Status*)a->status);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int mesh_wait_flag_test(const uint32_t* flag, uint32_t expect, uint64_t limit_ns, void* status, void* stream) {
  wait_flag_test_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag, expect, limit_ns, (Status*)status);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}
