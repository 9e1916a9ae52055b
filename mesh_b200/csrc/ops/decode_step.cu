// One decoded token per sequence as ONE cooperative kernel.
//
// A decoder step is ~150 small dependent operations (per layer: QKV projection, attention, output projection, GLU,
// down projection; then the vocabulary projection and the selection).  Launched one by one, every boundary costs a
// launch, a ramp of CTAs, the staging of x and a drained memory pipeline: at batch 1 that, not HBM, bounds the step.
// Here a persistent grid (one CTA per SM, launched cooperatively) walks a list of operations; every CTA takes its share
// of each, and a grid barrier with split arrive / wait separates them.  Eight warps of a CTA compute; a ninth streams
// the weights of ALL layers, in order, through a ring of stages in shared memory (cp.async.bulk, one copy per weight
// row and stage, completion counted on an mbarrier) and is held back only by the ring's capacity, never by a barrier,
// so HBM keeps streaming while the computing warps wait for the layer before, stage x and reduce.  The layers are the
// arithmetic of the stand-alone kernels (decode_linear.cuh, decode_attention.cuh) with the sums over k taken stage by
// stage, so the results agree with theirs to rounding.
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

// Warps 0..7 compute (THREADS threads, their barrier is named barrier 1); warp 8 streams weights.
constexpr int S_THREADS = THREADS + 32;
constexpr int MAX_STAGES = 16;
constexpr int ROW_PAD = 64;            // bytes between the rows of a stage: a quarter warp's 16-byte reads miss each other's banks

struct ComputeSync {
  __device__ __forceinline__ void operator()() const { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }
};

// Grid barrier with split phases.  bar[0]: arrivals of the current barrier, bar[1]: barriers completed so far
// (only grows).  Every CTA arrives at every barrier of the step, whatever happened to it, so the two words stay
// consistent from launch to launch; a wait is bounded and records where it gave up.  Called by the computing threads.
struct GridBarrier {
  uint32_t* bar;
  uint32_t target;          // value of bar[1] that ends the next wait
  Status* st;
  bool ok;
  unsigned long long* waited;   // shared-memory word (thread 0 adds the nanoseconds it spent waiting) or nullptr

  __device__ __forceinline__ void arrive() {
    ComputeSync{}();
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
  // Polls with relaxed loads (an acquire on every poll would also invalidate the SM's L1 each time) and a short sleep
  // between them; one acquire fence orders what follows after the word has been seen.
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
    ComputeSync{}();
  }
};

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// (max, lowest index) over the computing threads; the result is valid in warp 0.
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
  ComputeSync{}();                       // the arrays may still be read from the previous call
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  ComputeSync{}();
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
__device__ __noinline__ void argmax_part_phase(const ArgmaxArgs* ap) {
  const ArgmaxArgs& a = *ap;
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
__device__ __noinline__ void argmax_final_phase(const ArgmaxArgs* ap) {
  const ArgmaxArgs& a = *ap;
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

template <int HD>
__device__ __noinline__ void attention_phase(const decode_att::AttArgs* Ap, uint8_t* smem) {
  const decode_att::AttArgs& A = *Ap;
  const int items = A.splits * A.kv_heads * A.B;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    const int split = it % A.splits, kvh = (it / A.splits) % A.kv_heads, b = it / (A.splits * A.kv_heads);
    decode_att::attention_item<HD, 4>(A, split, kvh, b, reinterpret_cast<float*>(smem), ComputeSync{});
    ComputeSync{}();
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

// ---------------------------------------------------------------------------------------------- streamed weights
// The ring of weight stages in shared memory.  A stage holds, for one 16-row group, KT consecutive k of every row
// (KT = 8 warps x the chunk a warp multiplies at a time), rows ROW_PAD bytes apart, then the rows' scales.  The
// producer warp walks the same (operation, group, k block) sequence as the computing warps, one stage each, and is
// held back only by the ring's capacity: it does not wait at grid barriers, so weights keep arriving while the
// computing warps wait for the layer before, stage x and reduce.
struct Ring {
  uint32_t base;            // shared address of slot 0
  uint32_t slot_bytes;
  int n_stages;
  uint32_t full0, empty0;   // shared addresses of the barrier arrays (8 bytes apart)
  int stage;
  uint32_t phase;
  __device__ __forceinline__ uint32_t slot() const { return base + (uint32_t)stage * slot_bytes; }
  __device__ __forceinline__ uint32_t full() const { return full0 + 8u * stage; }
  __device__ __forceinline__ uint32_t empty() const { return empty0 + 8u * stage; }
  __device__ __forceinline__ void advance() { if (++stage == n_stages) { stage = 0; phase ^= 1u; } }
};

template <int W4, int U> struct StageGeom {
  static constexpr int CH = ChunkK<W4, U>::value;                 // k per warp and stage
  static constexpr int KT = CH * WARPS;                           // k per stage
  static constexpr int ROWB = W4 == 0 ? KT * 2 : (W4 == 3 ? KT : KT / 2);   // bytes of one row's codes
  static constexpr int RS = ROWB + ROW_PAD;
  static constexpr int SROWB = W4 == 0 ? 0 : KT / 64 * 2;         // bytes of one row's scales
  static constexpr int BYTES = 16 * RS + 16 * SROWB;
};

__host__ __device__ inline void variant_geom(int variant, int& kt, int& rowb, int& srowb) {
  switch (variant) {
    case LIN_BF16_U4: kt = StageGeom<0, 4>::KT; rowb = StageGeom<0, 4>::ROWB; srowb = 0; break;
    case LIN_BF16_U1: kt = StageGeom<0, 1>::KT; rowb = StageGeom<0, 1>::ROWB; srowb = 0; break;
    case LIN_W8_U4: kt = StageGeom<3, 4>::KT; rowb = StageGeom<3, 4>::ROWB; srowb = StageGeom<3, 4>::SROWB; break;
    case LIN_W8_U2: kt = StageGeom<3, 2>::KT; rowb = StageGeom<3, 2>::ROWB; srowb = StageGeom<3, 2>::SROWB; break;
    case LIN_W8_U1: kt = StageGeom<3, 1>::KT; rowb = StageGeom<3, 1>::ROWB; srowb = StageGeom<3, 1>::SROWB; break;
    case LIN_W4W_U2: kt = StageGeom<2, 2>::KT; rowb = StageGeom<2, 2>::ROWB; srowb = StageGeom<2, 2>::SROWB; break;
    case LIN_W4W_U1: kt = StageGeom<2, 1>::KT; rowb = StageGeom<2, 1>::ROWB; srowb = StageGeom<2, 1>::SROWB; break;
    default: kt = 0; rowb = 0; srowb = 0; break;               // the narrow 4-bit readers are not streamed
  }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_half(uint32_t addr) {
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
  return __half2float(__ushort_as_half(h));
}

// This warp's chunk of a stage -> registers, in the layout `mma_chunk` multiplies.
template <int W4, int U>
__device__ __forceinline__ void load_chunk_stage(uint32_t slot, int warp, int g8, int t4, Chunk<W4, U>& c) {
  using G = StageGeom<W4, U>;
  constexpr int WB = W4 == 0 ? G::CH * 2 : (W4 == 3 ? G::CH : G::CH / 2);     // bytes of a warp's k range in a row
  const uint32_t ra = slot + (uint32_t)g8 * G::RS + (uint32_t)warp * WB + (uint32_t)t4 * 16;
  const uint32_t rb = ra + 8u * G::RS;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    c.a[u] = lds128(ra + 64u * u);
    c.b[u] = lds128(rb + 64u * u);
  }
  if constexpr (W4 != 0) {
    constexpr int BLK = W4 == 2 ? 128 : 64;
    const uint32_t sc = slot + 16u * G::RS;
    const int k_lane = warp * G::CH + lane_k<W4>(t4);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t idx = (uint32_t)((k_lane + u * BLK) >> 6) * 2u;
      c.sa[u] = lds_half(sc + (uint32_t)g8 * G::SROWB + idx);
      c.sb[u] = lds_half(sc + (uint32_t)(g8 + 8) * G::SROWB + idx);
    }
  }
}

// One linear layer on the computing warps, weights taken from the ring.  `dead`: CTA-wide word set by whoever gave up
// a wait; from then on nobody waits (the results are garbage and the status block says why), but every thread still
// meets every barrier, so nothing hangs.
template <int W4, int U>
__device__ __forceinline__ void linear_stream(const LinArgs& a, uint8_t* work, Ring& ring, GridBarrier gb, bool wait,
                                              volatile int* dead) {
  using G = StageGeom<W4, U>;
  const int K = a.K;
  const int xstride = K * 2 + a.xpad;
  uint8_t* xs = work;
  float* red = reinterpret_cast<float*>(work + (size_t)a.B * (K * 2 + XPAD));
  float* fin = red + WARPS * 16 * NB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  const int kstages = K / G::KT;
  if (wait) gb.wait();
  if ((int)blockIdx.x < a.n_groups) stage_x(a, xs, xstride, ComputeSync{});      // a CTA with no group of this layer stages nothing
  const uint8_t* xrow = xs + (g8 < a.B ? g8 : a.B - 1) * xstride + (warp * G::CH + lane_k<W4>(t4)) * 2;
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  for (int grp = blockIdx.x; grp < a.n_groups; grp += gridDim.x) {
    for (int ks = 0; ks < kstages; ++ks) {
      if (!*dead) mbar_wait(ring.full(), ring.phase, dead, a.status, SITE_SMEM_FULL);
      Chunk<W4, U> ch;
      load_chunk_stage<W4, U>(ring.slot(), warp, g8, t4, ch);
      mma_chunk<W4, U>(ch, xrow + (size_t)ks * G::KT * 2, c);
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty());
      ring.advance();
    }
    finish_group(a, grp, c, red, fin, ComputeSync{});
    c[0] = c[1] = c[2] = c[3] = 0.f;
  }
}

__device__ __forceinline__ void linear_stream_dispatch(int variant, const LinArgs& a, uint8_t* work, Ring& ring,
                                                       GridBarrier gb, bool wait, volatile int* dead) {
  switch (variant) {
    case LIN_BF16_U4: linear_stream<0, 4>(a, work, ring, gb, wait, dead); break;
    case LIN_BF16_U1: linear_stream<0, 1>(a, work, ring, gb, wait, dead); break;
    case LIN_W8_U4: linear_stream<3, 4>(a, work, ring, gb, wait, dead); break;
    case LIN_W8_U2: linear_stream<3, 2>(a, work, ring, gb, wait, dead); break;
    case LIN_W8_U1: linear_stream<3, 1>(a, work, ring, gb, wait, dead); break;
    case LIN_W4W_U2: linear_stream<2, 2>(a, work, ring, gb, wait, dead); break;
    default: linear_stream<2, 1>(a, work, ring, gb, wait, dead); break;
  }
}

// The producer warp: every linear layer of the step, in order, one stage per (group, k block).
__device__ __forceinline__ void stream_weights(const StepOp* ops, int n_ops, Ring ring, Status* st, volatile int* dead) {
  const int lane = threadIdx.x & 31;
  int in_flight = 0;                       // stages issued since the ring was last known drained (capped at n_stages)
  bool ok = !status_aborted(st);
  for (int i = 0; ok && i < n_ops; ++i) {
    const StepOp* o = ops + i;
    if (o->kind != DOP_LINEAR) continue;
    const LinHot hot{o->lin.w, o->lin.scales, o->lin.K, o->lin.mode, o->lin.up_off, o->lin.head_dim};
    const int n_groups = o->lin.n_groups;
    int kt, rowb, srowb;
    variant_geom(o->variant, kt, rowb, srowb);
    const int kstages = hot.K / kt;
    const long long row_bytes = (long long)rowb * kstages;                  // a whole row of codes
    const long long srow_bytes = (long long)srowb * kstages;
    const uint32_t rs = (uint32_t)rowb + ROW_PAD;
    for (int grp = blockIdx.x; ok && grp < n_groups; grp += gridDim.x) {
      int rA, rB;
      group_rows(hot, grp, rA, rB);
      const int r16 = lane & 15;
      const long long row = r16 < 8 ? rA + r16 : rB + (r16 - 8);
      for (int ks = 0; ks < kstages; ++ks) {
        int good = 1;
        if (lane == 0) good = mbar_wait(ring.empty(), ring.phase ^ 1u, dead, st, SITE_SMEM_EMPTY) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good || *dead) { ok = false; break; }
        if (lane == 0) mbar_expect_tx(ring.full(), 16u * (uint32_t)(rowb + srowb));
        __syncwarp();
        if (lane < 16) {
          bulk_load_1d(ring.slot() + (uint32_t)r16 * rs, reinterpret_cast<const uint8_t*>(hot.w) + row * row_bytes + (long long)ks * rowb,
                       (uint32_t)rowb, ring.full());
        } else if (srowb) {
          bulk_load_1d(ring.slot() + 16u * rs + (uint32_t)r16 * srowb,
                       reinterpret_cast<const uint8_t*>(hot.scales) + row * srow_bytes + (long long)ks * srowb, (uint32_t)srowb,
                       ring.full());
        }
        if (in_flight < ring.n_stages) ++in_flight;
        ring.advance();
      }
    }
  }
  if (!ok) {
    // Something gave up.  The copies already issued still land in this CTA's shared memory: wait for them (bounded)
    // before the CTA may exit.  A stage's full barrier completes when its bytes have arrived, read or not.
    for (int n = 0; n < in_flight; ++n) {
      ring.stage = ring.stage == 0 ? ring.n_stages - 1 : ring.stage - 1;
      if (ring.stage == ring.n_stages - 1) ring.phase ^= 1u;
      if (lane == 0) {
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(ring.full(), ring.phase) && globaltimer_ns() - t0 < MESH_WAIT_LIMIT_NS) { __nanosleep(100); }
      }
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(S_THREADS, 1)
decode_step_kernel(const StepOp* __restrict__ ops, int n_ops, uint32_t* bar, Status* st, unsigned long long* trace,
                   int ring_off, int slot_bytes, int n_stages) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ StepOp op;
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
  __shared__ uint32_t gen0;
  __shared__ unsigned long long waited_s;
  __shared__ int dead_s;
  if (threadIdx.x == 0) {
    gen0 = ld_acquire_gpu(bar + 1);
    waited_s = 0;
    dead_s = 0;
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), WARPS);
    }
    fence_mbar_init();
  }
  __syncthreads();
  Ring ring{smem_u32(smem + ring_off), (uint32_t)slot_bytes, n_stages, smem_u32(&full_bar[0]), smem_u32(&empty_bar[0]), 0, 0u};
  if (threadIdx.x >= THREADS) {
    stream_weights(ops, n_ops, ring, st, &dead_s);
    return;
  }
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
    ComputeSync{}();
    // a cancelled step still meets its barriers (and a layer still walks its stages), and stores garbage
    const bool live = !status_aborted(st);
    gb.ok = live && !dead_s;
    const bool wait = i > 0;
    if (op.kind == DOP_LINEAR) {
      linear_stream_dispatch(op.variant, op.lin, smem, ring, gb, wait, &dead_s);
    } else {
      if (wait) gb.wait();
      if (live) {
        if (op.kind == DOP_ATTENTION) {
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
    }
    if (tracing) { my_trace[3 * i + 1] = globaltimer_ns(); my_trace[3 * i + 2] = waited_s; }
    if (i + 1 < n_ops) gb.arrive();
    else ComputeSync{}();
  }
}

}  // namespace decode
}  // namespace mesh

using namespace mesh;
using namespace mesh::decode;

namespace {
constexpr int MAX_ARGMAX_OPS = 8;
constexpr int STEP_SMEM = 220 * 1024;
}  // namespace

extern "C" size_t mesh_decode_step_bytes(int n_ops) { return (size_t)(n_ops + MAX_ARGMAX_OPS) * sizeof(StepOp); }

extern "C" int mesh_decode_step_max_grid(void) { return sm_count(); }

extern "C" int mesh_decode_step_prepare(const MeshDecodeOp* ops, int n_ops, void* dev_ops, size_t dev_bytes,
                                        MeshDecodeStepPlan* plan) {
  if (n_ops < 1) return set_error(-2, "decode_step: no operations");
  std::vector<StepOp> out;
  out.reserve(n_ops + MAX_ARGMAX_OPS);
  size_t work = 0, slot = 0;
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
      int kt, rowb, srowb;
      variant_geom(s.variant, kt, rowb, srowb);
      if (kt == 0) return set_error(-2, "decode_step: a layer of this width has no streamed form (K must be a multiple of 1024 for 4-bit weights)");
      if (((uintptr_t)o.lin.w & 15) || ((uintptr_t)o.lin.scales & 15))
        return set_error(-2, "decode_step: weights and scales must be 16-byte aligned");
      work = std::max(work, lin_smem_bytes(o.lin.K, o.lin.B));
      slot = std::max(slot, (size_t)16 * (rowb + ROW_PAD) + (size_t)16 * srowb);
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
      work = std::max(work, (size_t)decode_att::ATT_WARPS * (o.q_heads / o.kv_heads) * o.head_dim * sizeof(float));
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
  work = (work + 1023) & ~(size_t)1023;
  slot = (slot + 127) & ~(size_t)127;
  if (slot == 0) slot = 128;
  if (work + 2 * slot > (size_t)STEP_SMEM) return set_error(-2, "decode_step: a layer needs more shared memory than a CTA has");
  int n_stages = (int)(((size_t)STEP_SMEM - work) / slot);
  if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
  static bool configured = false;
  if (!configured) {
    MESH_CUDA_OK(cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STEP_SMEM));
    configured = true;
  }
  const int smem = (int)(work + (size_t)n_stages * slot);
  int per_sm = 0;
  MESH_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, S_THREADS, (size_t)smem));
  if (per_sm < 1) return set_error(-3, "decode_step: the kernel does not fit on an SM");
  MESH_CUDA_OK(cudaMemcpy(dev_ops, out.data(), out.size() * sizeof(StepOp), cudaMemcpyHostToDevice));
  plan->n_dev = (int)out.size();
  plan->grid = sm_count();
  plan->smem = smem;
  plan->ring_off = (int)work;
  plan->slot_bytes = (int)slot;
  plan->n_stages = n_stages;
  return 0;
}

extern "C" int mesh_decode_step_run(const void* dev_ops, const MeshDecodeStepPlan* plan, uint32_t* barrier, void* status,
                                    unsigned long long* trace, void* stream) {
  const StepOp* ops = (const StepOp*)dev_ops;
  Status* st = (Status*)status;
  int n_dev = plan->n_dev, ring_off = plan->ring_off, slot_bytes = plan->slot_bytes, n_stages = plan->n_stages;
  if (n_stages < 2 || n_stages > MAX_STAGES) return set_error(-2, "decode_step: plan not prepared");
  void* args[] = {(void*)&ops, (void*)&n_dev, (void*)&barrier, (void*)&st, (void*)&trace,
                  (void*)&ring_off, (void*)&slot_bytes, (void*)&n_stages};
  // cooperative: the launch fails unless every CTA of the grid is resident at once, which the barrier needs
  MESH_CUDA_OK(cudaLaunchCooperativeKernel((const void*)decode_step_kernel, dim3((unsigned)plan->grid), dim3(S_THREADS), args,
                                           (size_t)plan->smem, (cudaStream_t)stream));
  return 0;
}
