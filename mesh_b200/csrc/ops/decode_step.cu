// One decoded token per sequence as ONE cooperative kernel.
//
// A decoder step is ~150 small dependent operations (per layer: QKV projection, attention, output projection, GLU,
// down projection; then the vocabulary projection and the selection).  Launched one by one, every boundary costs a
// launch, a ramp of CTAs, the staging of x and a drained memory pipeline: at batch 1 that, not HBM, bounds the step.
// Here a persistent grid (as many CTAs as are resident at once) walks a list of operations; every CTA takes its share
// of each, and a grid barrier with split arrive / wait separates them: a CTA arrives when its share is written,
// requests the first weights of the next layer (they depend on nothing computed here) and only then waits, so HBM
// keeps streaming across the boundaries.  The layers are the bodies the stand-alone kernels run (decode_linear.cuh,
// decode_attention.cuh), so the results are theirs bit for bit.
//
// Reference counterpart: the prepared machine that runs a whole decoder step without returning to the host between
// layers (design/prepared-machine.md; rdma/mesh-dataflow.c:287-317 starts it once and lets signals order the parts).
#include "decode_linear.cuh"
#include "decode_attention.cuh"
#include <math_constants.h>
#include <vector>

namespace mesh {
namespace decode {

enum DevOpKind { DOP_EMBED = 0, DOP_LINEAR = 1, DOP_ATTENTION = 2, DOP_ARGMAX_PART = 3, DOP_ARGMAX_FINAL = 4 };

struct EmbArgs { const __nv_bfloat16* table; const int* tok; __nv_bfloat16* x; int B, d; };

struct ArgmaxArgs {
  const float* logits; long long ldl; int B, vocab_local, vocab_offset;
  int* tokens_out; int* pos; int rank, world;
  uint2* xchg[MESH_DEC_MAX_RANKS];
  uint32_t* step; float* part_v; int* part_i; Status* status;
};

struct __align__(16) StepOp {
  int kind, variant;
  LinArgs lin;
  decode_att::AttArgs att;
  EmbArgs emb;
  ArgmaxArgs am;
};
static_assert(sizeof(StepOp) % 16 == 0, "operations are copied to shared memory 16 bytes at a time");

// Grid barrier with split phases.  bar[0]: arrivals of the current barrier, bar[1]: barriers completed so far
// (only grows).  Every CTA arrives at every barrier of the step, whatever happened to it, so the two words stay
// consistent from launch to launch; a wait is bounded and records where it gave up.
struct GridBarrier {
  uint32_t* bar;
  uint32_t target;          // value of bar[1] that ends the next wait
  Status* st;
  bool ok;
  unsigned long long* waited;   // shared-memory word (thread 0 adds the nanoseconds it spent waiting) or nullptr

  __device__ __forceinline__ void arrive() {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(bar, 1u);
      if (old == gridDim.x - 1) {
        *reinterpret_cast<volatile uint32_t*>(bar) = 0u;
        __threadfence();
        red_release_gpu_add(bar + 1, 1u);
      }
    }
    ++target;
  }
  // Polls with relaxed loads (an acquire on every poll would also invalidate this SM's L1 under the CTA that shares
  // it) and a short sleep between them; one acquire fence orders what follows after the word has been seen.
  __device__ __forceinline__ void wait() {
    if (threadIdx.x == 0 && ok) {
      const volatile uint32_t* gen = reinterpret_cast<const volatile uint32_t*>(bar + 1);
      uint32_t v = *gen;
      if ((int32_t)(v - target) < 0) {
        const unsigned long long t0 = globaltimer_ns();
        uint32_t it = 0;
        while (true) {
          __nanosleep(20);
          v = *gen;
          if ((int32_t)(v - target) >= 0) break;
          if (((++it) & 0xffu) == 0) {
            if (globaltimer_ns() - t0 > MESH_WAIT_LIMIT_NS || status_aborted(st)) {
              status_record(st, MESH_TIMEOUT, SITE_LOCAL_FLAG, target, v, (unsigned long long)bar);
              break;
            }
          }
        }
        if (waited) *waited += globaltimer_ns() - t0;
      }
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
    }
    __syncthreads();
  }
};

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// (max, lowest index) over the CTA; the result is valid in warp 0.
__device__ __forceinline__ void block_maxloc(float& best, int& bi) {
  __shared__ float sv[THREADS / 32];
  __shared__ int si[THREADS / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    better(best, bi, ov, oi);
  }
  __syncthreads();                       // the arrays may still be read from the previous call
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < THREADS / 32 ? sv[lane] : -CUDART_INF_F;
    bi = lane < THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      better(best, bi, ov, oi);
    }
  }
}

// Every CTA scans a contiguous slice of the vocabulary shard for every sequence.
__device__ __forceinline__ void argmax_part(const ArgmaxArgs& a) {
  const int per = ((a.vocab_local + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;
  const int lo = (int)blockIdx.x * per, hi = min(a.vocab_local, lo + per);
  for (int b = 0; b < a.B; ++b) {
    const float* row = a.logits + (long long)b * a.ldl;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = lo + (int)threadIdx.x; i < hi; i += THREADS) {
      const float v = __ldcg(row + i);
      if (v > best) { best = v; bi = i; }
    }
    block_maxloc(best, bi);
    if (threadIdx.x == 0) {
      a.part_v[(long long)b * gridDim.x + blockIdx.x] = best;
      a.part_i[(long long)b * gridDim.x + blockIdx.x] = bi;
    }
  }
}

// CTA b < B merges the slices of sequence b, exchanges the pair with the other ranks, writes the token.
__device__ __forceinline__ void argmax_final(const ArgmaxArgs& a) {
  const int b = blockIdx.x;
  if (b >= a.B) return;
  const uint32_t seq = (a.step ? *reinterpret_cast<volatile uint32_t*>(a.step) : 0u) + 1u;
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += THREADS)
    better(best, bi, __ldcg(a.part_v + (long long)b * gridDim.x + i), __ldcg(a.part_i + (long long)b * gridDim.x + i));
  block_maxloc(best, bi);
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  int gidx = bi + a.vocab_offset;
  if (a.world > 1) {
    // slot layout on every rank: [parity(seq & 1)][src rank][sequence][2 words]: {value bits, seq}, {index, seq}
    const long long base = ((long long)(seq & 1u) * a.world * 8 + (long long)a.rank * 8 + b) * 2;
    if (lane < a.world) {
      uint2* p = a.xchg[lane] + base;
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(best)), "r"(seq) : "memory");
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p + 1), "r"((uint32_t)gidx), "r"(seq) : "memory");
    }
    float v = -CUDART_INF_F;
    int id = 0x7fffffff;
    if (lane < a.world) {
      const uint2* p = a.xchg[a.rank] + ((long long)(seq & 1u) * a.world * 8 + (long long)lane * 8 + b) * 2;
      uint2 w0, w1;
      unsigned long long t0 = 0;
      uint32_t it = 0;
      while (true) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w0.x), "=r"(w0.y) : "l"(p) : "memory");
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w1.x), "=r"(w1.y) : "l"(p + 1) : "memory");
        if (w0.y == seq && w1.y == seq) break;
        if (((++it) & 0x3ffu) == 0) {
          if (t0 == 0) t0 = globaltimer_ns();
          else if (globaltimer_ns() - t0 > MESH_WAIT_LIMIT_NS || status_aborted(a.status)) {
            status_record(a.status, MESH_TIMEOUT, SITE_PEER_FLAG, seq, w0.y, (unsigned long long)p);
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
      better(v, id, ov, oi);
    }
    gidx = id;
  }
  if (lane == 0) {
    a.tokens_out[b] = gidx;
    if (a.pos) a.pos[b] += 1;
    if (a.step) {                          // the last sequence's CTA advances the step word
      __threadfence();
      const unsigned done = atomicAdd(a.step + 1, 1u);
      if (done == (unsigned)a.B - 1u) { a.step[1] = 0; __threadfence(); atomicAdd(a.step, 1u); }
    }
  }
}

// Every kind of operation is a function of its own, not inlined into the step kernel: the compiler then allocates
// registers for each body as it does for the stand-alone kernel, instead of for the union of all of them.
struct WaitInputs {
  GridBarrier gb;
  bool needed;
  __device__ __forceinline__ void operator()() { if (needed) gb.wait(); }
};

template <int W4, int U>
__device__ __noinline__ void linear_phase(const LinArgs* a, uint8_t* smem, GridBarrier gb, bool wait) {
  linear_body<W4, U>(*a, smem, WaitInputs{gb, wait});
}

template <int HD>
__device__ __noinline__ void attention_phase(const decode_att::AttArgs* Ap, uint8_t* smem) {
  const decode_att::AttArgs& A = *Ap;
  const int items = A.splits * A.kv_heads * A.B;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int split = it % A.splits, kvh = (it / A.splits) % A.kv_heads, b = it / (A.splits * A.kv_heads);
    decode_att::attention_item<HD, 4>(A, split, kvh, b, reinterpret_cast<float*>(smem));
    __syncthreads();
  }
}

__device__ __noinline__ void embed_phase(const EmbArgs* ep) {
  const EmbArgs& e = *ep;
  const int nvec = e.d >> 3;
  for (int idx = blockIdx.x * THREADS + threadIdx.x; idx < e.B * nvec; idx += gridDim.x * THREADS) {
    const int b = idx / nvec, v = idx - b * nvec;
    const long long row = *reinterpret_cast<const volatile int*>(e.tok + b);
    reinterpret_cast<uint4*>(e.x + (long long)b * e.d)[v] = reinterpret_cast<const uint4*>(e.table + row * e.d)[v];
  }
}

__device__ __noinline__ void argmax_part_phase(const ArgmaxArgs* a) { argmax_part(*a); }
__device__ __noinline__ void argmax_final_phase(const ArgmaxArgs* a) { argmax_final(*a); }

__device__ __forceinline__ void linear_phase_dispatch(int variant, const LinArgs* a, uint8_t* smem, GridBarrier gb, bool wait) {
  switch (variant) {
    case LIN_W4N_U2: linear_phase<1, 2>(a, smem, gb, wait); break;
    case LIN_W4N_U1: linear_phase<1, 1>(a, smem, gb, wait); break;
    case LIN_BF16_U4: linear_phase<0, 4>(a, smem, gb, wait); break;
    case LIN_BF16_U1: linear_phase<0, 1>(a, smem, gb, wait); break;
    case LIN_W8_U4: linear_phase<3, 4>(a, smem, gb, wait); break;
    case LIN_W8_U2: linear_phase<3, 2>(a, smem, gb, wait); break;
    case LIN_W8_U1: linear_phase<3, 1>(a, smem, gb, wait); break;
    case LIN_W4W_U2: linear_phase<2, 2>(a, smem, gb, wait); break;
    default: linear_phase<2, 1>(a, smem, gb, wait); break;
  }
}

__global__ void __launch_bounds__(THREADS, 2)
decode_step_kernel(const StepOp* __restrict__ ops, int n_ops, uint32_t* bar, Status* st, unsigned long long* trace) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ StepOp op;
  __shared__ uint32_t gen0;
  __shared__ unsigned long long waited_s;
  if (threadIdx.x == 0) { gen0 = ld_acquire_gpu(bar + 1); waited_s = 0; }
  __syncthreads();
  // trace (optional): CTA 0 and the last CTA write, per operation, {start, end of its share, nanoseconds waited}
  const bool tracing = trace != nullptr && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && threadIdx.x == 0;
  unsigned long long* my_trace = trace ? trace + (blockIdx.x == 0 ? 0 : 3ll * n_ops) : nullptr;
  GridBarrier gb{bar, gen0, st, true, trace ? &waited_s : nullptr};
  for (int i = 0; i < n_ops; ++i) {
    if (tracing) { my_trace[3 * i] = globaltimer_ns(); waited_s = 0; }
    {
      const uint4* src = reinterpret_cast<const uint4*>(ops + i);
      uint4* dst = reinterpret_cast<uint4*>(&op);
      for (int w = threadIdx.x; w < (int)(sizeof(StepOp) / 16); w += THREADS) dst[w] = src[w];
    }
    __syncthreads();
    const bool live = !status_aborted(st);           // a cancelled step still meets its barriers, and does nothing else
    gb.ok = live;
    const bool wait = i > 0;
    if (!live || op.kind != DOP_LINEAR) {
      if (wait) gb.wait();
    }
    if (live) {
      if (op.kind == DOP_LINEAR) {
        linear_phase_dispatch(op.variant, &op.lin, smem, gb, wait);
      } else if (op.kind == DOP_ATTENTION) {
        if (op.att.head_dim == 256) attention_phase<256>(&op.att, smem);
        else if (op.att.head_dim == 128) attention_phase<128>(&op.att, smem);
        else attention_phase<64>(&op.att, smem);
      } else if (op.kind == DOP_EMBED) {
        embed_phase(&op.emb);
      } else if (op.kind == DOP_ARGMAX_PART) {
        argmax_part_phase(&op.am);
      } else {
        argmax_final_phase(&op.am);
      }
    }
    if (tracing) { my_trace[3 * i + 1] = globaltimer_ns(); my_trace[3 * i + 2] = waited_s; }
    if (i + 1 < n_ops) gb.arrive();
    else __syncthreads();
  }
}

}  // namespace decode
}  // namespace mesh

using namespace mesh;
using namespace mesh::decode;

namespace {
constexpr int MAX_ARGMAX_OPS = 8;
int step_ctas_per_sm(int smem) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_step_kernel, THREADS, (size_t)smem) != cudaSuccess) return 0;
  return n > 2 ? 2 : n;
}
}  // namespace

extern "C" size_t mesh_decode_step_bytes(int n_ops) { return (size_t)(n_ops + MAX_ARGMAX_OPS) * sizeof(StepOp); }

extern "C" int mesh_decode_step_max_grid(void) { return sm_count() * 2; }

extern "C" int mesh_decode_step_prepare(const MeshDecodeOp* ops, int n_ops, void* dev_ops, size_t dev_bytes, int* n_dev,
                                        int* grid, int* smem_out) {
  if (n_ops < 1) return set_error(-2, "decode_step: no operations");
  std::vector<StepOp> out;
  out.reserve(n_ops + MAX_ARGMAX_OPS);
  size_t smem = 0;
  int argmaxes = 0;
  for (int i = 0; i < n_ops; ++i) {
    const MeshDecodeOp& o = ops[i];
    StepOp s;
    memset(&s, 0, sizeof(s));
    if (o.kind == MESH_DEC_OP_LINEAR) {
      s.kind = DOP_LINEAR;
      const int rc = lin_prepare(&o.lin, s.lin, s.variant);
      if (rc) return rc;
      s.lin.l2_prefetch = 0;
      s.lin.next_w = nullptr;
      s.lin.next_bytes = 0;
      smem = std::max(smem, lin_smem_bytes(o.lin.K, o.lin.B));
    } else if (o.kind == MESH_DEC_OP_ATTENTION) {
      if (o.B < 1 || o.q_heads % o.kv_heads || o.q_heads / o.kv_heads > 4)
        return set_error(-2, "decode_step: attention groups of 1..4 query heads per KV head");
      if (o.splits < 1 || o.splits > 64) return set_error(-2, "decode_step: attention splits must be 1..64");
      if (o.head_dim != 64 && o.head_dim != 128 && o.head_dim != 256)
        return set_error(-2, "decode_step: head_dim must be 64, 128 or 256");
      s.kind = DOP_ATTENTION;
      decode_att::AttArgs& A = s.att;
      A.q = (const __nv_bfloat16*)o.q; A.kc = (const __nv_bfloat16*)o.k_cache; A.vc = (const __nv_bfloat16*)o.v_cache;
      A.pos = o.pos; A.out = (__nv_bfloat16*)o.att_out; A.scratch = o.scratch; A.counters = o.counters;
      A.q_heads = o.q_heads; A.kv_heads = o.kv_heads; A.max_seq = o.max_seq; A.window = o.window; A.scale = o.scale;
      A.splits = o.splits; A.T = 1; A.B = o.B; A.head_dim = o.head_dim;
      smem = std::max(smem, (size_t)decode_att::ATT_WARPS * (o.q_heads / o.kv_heads) * o.head_dim * sizeof(float));
    } else if (o.kind == MESH_DEC_OP_EMBED) {
      if (o.d_model % 8 || o.B < 1) return set_error(-2, "decode_step: embedding rows must be a multiple of 8 wide");
      s.kind = DOP_EMBED;
      s.emb.table = (const __nv_bfloat16*)o.table; s.emb.tok = o.tok; s.emb.x = (__nv_bfloat16*)o.x;
      s.emb.B = o.B; s.emb.d = o.d_model;
    } else if (o.kind == MESH_DEC_OP_ARGMAX) {
      if (o.B < 1 || o.B > 8) return set_error(-2, "decode_step: batch must be 1..8");
      if (o.world < 1 || o.world > MESH_DEC_MAX_RANKS) return set_error(-4, "decode_step: world out of range");
      if (++argmaxes > MAX_ARGMAX_OPS / 2) return set_error(-2, "decode_step: too many selections in one step");
      s.kind = DOP_ARGMAX_PART;
      ArgmaxArgs& a = s.am;
      a.logits = o.logits; a.ldl = o.ldl; a.B = o.B; a.vocab_local = o.vocab_local; a.vocab_offset = o.vocab_offset;
      a.tokens_out = o.tokens_out; a.pos = o.pos_inc; a.rank = o.rank; a.world = o.world;
      for (int r = 0; r < o.world; ++r) a.xchg[r] = (uint2*)o.xchg[r];
      a.step = o.step; a.part_v = o.part_v; a.part_i = o.part_i; a.status = (Status*)o.status;
      out.push_back(s);
      s.kind = DOP_ARGMAX_FINAL;
    } else {
      return set_error(-2, "decode_step: unknown operation");
    }
    out.push_back(s);
  }
  if (out.size() * sizeof(StepOp) > dev_bytes) return set_error(-2, "decode_step: operation buffer too small");
  if (smem > 220 * 1024) return set_error(-2, "decode_step: a layer needs more shared memory than a CTA has");
  static bool configured = false;
  if (!configured) {
    MESH_CUDA_OK(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured = true;
  }
  const int per_sm = step_ctas_per_sm((int)smem);
  if (per_sm < 1) return set_error(-3, "decode_step: the kernel does not fit on an SM");
  MESH_CUDA_OK(cudaMemcpy(dev_ops, out.data(), out.size() * sizeof(StepOp), cudaMemcpyHostToDevice));
  *n_dev = (int)out.size();
  *grid = sm_count() * per_sm;
  *smem_out = (int)smem;
  return 0;
}

extern "C" int mesh_decode_step_run(const void* dev_ops, int n_dev, uint32_t* barrier, void* status, int grid, int smem,
                                    unsigned long long* trace, void* stream) {
  const StepOp* ops = (const StepOp*)dev_ops;
  Status* st = (Status*)status;
  void* args[] = {(void*)&ops, (void*)&n_dev, (void*)&barrier, (void*)&st, (void*)&trace};
  // cooperative: the launch fails unless every CTA of the grid is resident at once, which the barrier needs
  MESH_CUDA_OK(cudaLaunchCooperativeKernel((const void*)decode_step_kernel, dim3((unsigned)grid), dim3(THREADS), args,
                                           (size_t)smem, (cudaStream_t)stream));
  return 0;
}
