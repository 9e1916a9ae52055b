// Persistent warp-specialised bf16 GEMM for sm_100a:  D[M,N] = A[M,K] * B[N,K]^T.
//
//   warp 0      TMA producer   (cp.async.bulk.tensor into a 4-stage shared-memory ring)
//   warp 1      MMA issuer     (tcgen05.mma, 128x256x16, accumulators in TMEM, 2 buffers)
//   warps 2..5  epilogue       (tcgen05.ld -> registers -> fused math -> swizzled smem -> TMA store,
//                               or direct stores to a peer GPU + arrival flags)
//
// Either operand may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]),
// which covers forward, dgrad and wgrad of a linear layer without any transposed copy.
// Fusions that live in this kernel:
//   * SwiGLU / GeGLU forward  (gate and up weights are two row ranges of one B matrix and
//     land in the two halves of one accumulator; the epilogue writes act(g)*u and,
//     optionally, g and u for the backward pass),
//   * SwiGLU / GeGLU backward (the epilogue of dA = dY*Wd reads g,u and writes dg,du),
//   * all-gather -> GEMM      (the producer waits on per-row-block arrival flags; tiles
//     are visited starting from this rank's own rows; spare warps push this rank's rows
//     into every peer's gathered buffer),
//   * GEMM -> reduce-scatter  (the epilogue stores each tile to the rank that owns its
//     rows and raises that rank's arrival counter; a tail phase sums the arrived
//     partials).
// This covers the computations K1-K3 of the reference's operation table
// (compiler/mesh_compiler/operations.py:1191-1272 contraction, :544-588 pointwise) and
// its partial-sum reduction (compiler/mesh_compiler/placement.py:812-834).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "../device/check.cuh"
#include "../device/ptx.cuh"

namespace mesh {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_WARPS = 4;
constexpr int EPI_BOX_COLS = 32;             // bf16 columns per TMA store box (64 B rows)
constexpr int EPI_BOX_BYTES = 32 * EPI_BOX_COLS * 2;   // 2 KiB
constexpr int EPI_BUFS = 4;                  // staging boxes per epilogue warp
constexpr int STAGING_BYTES = EPI_WARPS * EPI_BUFS * EPI_BOX_BYTES;   // 32 KiB
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int COMM_WARPS = 4;                // extra warps of the all-gather variant
constexpr int AG_SPLIT = 8;                  // parts per 128-row block pushed by the comm warps
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

enum Epilogue : int {
  EPI_STORE = 0,        // D = acc
  EPI_GLU_FWD = 1,      // D = act(g) * u  (+ optional D2 = [g | u])
  EPI_GLU_BWD = 2,      // D = [dg | du] from acc = dAct and aux = [g | u]
  EPI_SCATTER = 3,      // partial tile -> owner rank's receive slot (+ arrival counter)
};
enum Activation : int { ACT_SILU = 0, ACT_GELU_TANH = 1 };

constexpr int MAX_RANKS = 8;

// Descriptor-driven (grouped / ragged) mode: the persistent kernel walks a device-resident list of tiles
// instead of a dense grid, so problems whose sizes are only known on the GPU (tokens per expert after a
// dispatch) run without a host round trip.  Coordinates are in elements of the stored matrices.
struct TileDesc {
  int a_mn0;      // first row (K-major A) or column (MN-major A) of this tile in A
  int k0;         // first K coordinate (both operands)
  int k_blocks;   // number of 64-wide K blocks
  int b_mn0;      // first row (K-major B) or column (MN-major B) in B, expert offset included
  int b_k0;       // extra K offset of B (MN-major stacked weights: expert * rows)
  int d_row0;     // first output row
  int d_col0;     // first output column
  int pad;
};

struct Params {
  CUtensorMap tmA, tmB, tmD, tmD2;
  const TileDesc* tiles;    // nullptr: dense grid
  const int* n_tiles_dev;   // number of valid descriptors (device word)
  CUtensorMap tmA2;                    // all-gather: this rank's own rows, read straight from the source
  CUtensorMap tmRS[MAX_RANKS];         // reduce-scatter: rank o's receive buffer as a [.., 64]-column matrix
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int m_units;              // m-tiles (single CTA) or pairs of m-tiles (cta_group::2) the scheduler walks
  int act;
  int b_up_rows;            // GLU_FWD: row offset of the "up" weights inside B
  int d_up_cols;            // GLU_FWD (D2) / GLU_BWD (D and aux): column offset of the "up" half
  int has_d2;
  const __nv_bfloat16* aux; // GLU_BWD: [g | u], row-major
  long long ld_aux;
  Status* status;
  // ---- all-gather -> GEMM -------------------------------------------------------------
  const uint32_t* a_ready;  // one counter per `a_ready_rows` rows of A; tile waits for >= a_ready_value
  uint32_t a_ready_value;
  int a_ready_rows;
  int m_rotate;             // first m-tile visited (own shard first)
  int ag_split;             // parts per 128-row block pushed by the comm warps
  // push side (run by the comm warps): this rank's rows `ag_src` [ag_rows_per_rank, ag_ld] are
  // stored into every rank's gathered buffer `ag_dst[d]` at row rank*ag_rows_per_rank, and the
  // destination's arrival counter `ag_flags[d][block]` is raised once per part.
  const __nv_bfloat16* ag_src;
  __nv_bfloat16* ag_dst[MAX_RANKS];
  uint32_t* ag_flags[MAX_RANKS];
  int ag_rows_per_rank;
  long long ag_ld;          // elements per row
  int rank, world;
  // ---- GEMM -> reduce-scatter -----------------------------------------------------------
  // rs_recv: this rank's receive buffer, tile-contiguous: [src rank][m-tile][n-tile][4 column
  // chunks][128 rows][64 columns]; a (chunk, 32-row quarter) is one contiguous 4 KiB TMA store box.
  const __nv_bfloat16* rs_recv;
  uint32_t* rs_count[MAX_RANKS];       // rs_count[o]: rank o's arrival counters, one per (m-tile of o, n-tile)
  uint32_t rs_expect;                  // counter value that means "all world partials of this tile arrived"
  __nv_bfloat16* rs_out;               // this rank's reduced output [rows_per_rank][N]
  int rs_rows_per_rank;
  // ---- kernel-to-kernel dataflow (consecutive launches of one stream that overlap) -----------
  // A consumer launched as a programmatic dependent starts while its producer's last wave of tiles still runs and
  // reads the producer's output row block by row block: the producer's epilogue warps raise `d_done[row / 128]`
  // once per (tile, warp) after their stores have completed, the consumer's TMA warp waits on `a_ready` (rows of a
  // K-major A, as in the all-gather) or on `k_ready` (K rows of an MN-major operand) before it loads.
  uint32_t* d_done;
  const uint32_t* k_ready;  // one counter per `k_ready_rows` K rows; a K block waits for >= k_ready_value
  uint32_t k_ready_value;
  int k_ready_rows;
  int pdl_trigger;          // let the next launch of the stream start during this kernel's last wave
  int a_extent, b_extent;   // rows (MN extent) of the stored A and B matrices: bounds for descriptor tiles (checked build)
  // ---- GEMM -> all-reduce: the reduce tail also broadcasts every summed tile -------------------
  __nv_bfloat16* ar_out[MAX_RANKS];    // every rank's full output [M, N]; nullptr: reduce-scatter only
  uint32_t* ar_flag[MAX_RANKS];        // ar_flag[r]: rank r's arrival counter, one arrival per (tile, source rank)
  uint32_t ar_expect;
  // ---- group-quantised B (weights): codes + one fp16 scale per 64 k of a row ------------------
  // The B stages of the shared-memory ring are then not filled by TMA: four extra warps read the codes with plain
  // loads, dequantise them in registers ((code - 8) * scale for 4-bit, (code - 128) * scale for 8-bit) and store bf16
  // into the stage in the layout a 128-byte-swizzled TMA load would have produced, so the MMA side is unchanged.
  const uint8_t* bq_codes;  // [rows, K/2] (4-bit, eight codes per 32-bit word in nibble order 0,4,1,5,2,6,3,7) or [rows, K]
  const __half* bq_scales;  // [rows, K/64]
  long long bq_row_bytes, bq_scale_ld;
  int bq_rows;
};

// ------------------------------------------------------------------------------------------
// Hardware approximations (ex2/rcp/tanh .approx, ~2^-11 relative error) are ample for values
// that are rounded to bf16 right after, and keep the epilogue well under the MMA time per tile.
__device__ __forceinline__ float fast_sigmoid(float g) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return r;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ float act_fwd(float g, int act) {
  if (act == ACT_SILU) {
    return g * fast_sigmoid(g);
  } else {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float t = fast_tanh(k0 * (g + k1 * g * g * g));
    return 0.5f * g * (1.f + t);
  }
}
// returns act(g) and writes d act / d g
__device__ __forceinline__ float act_fwd_bwd(float g, int act, float& dact) {
  if (act == ACT_SILU) {
    float s = fast_sigmoid(g);
    dact = s * (1.f + g * (1.f - s));
    return g * s;
  } else {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float t = fast_tanh(k0 * (g + k1 * g * g * g));
    dact = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
    return 0.5f * g * (1.f + t);
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t w) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&w);
  return __bfloat1622float2(v);
}

// Write 32 fp32 values (one row, 32 columns) as bf16 into a [32 rows][64 B] staging box laid
// out with the 64-byte TMA swizzle: 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage_row(uint32_t box_smem, int row, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w0 = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
    uint32_t w1 = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
    uint32_t w2 = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
    uint32_t w3 = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
    uint32_t addr = box_smem + row * 64 + ((j ^ ((row >> 1) & 3)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                 : "memory");
  }
}

// Same for one half (32 columns) of a [32 rows][128 B] box with the 128-byte swizzle:
// 16-byte chunk j of row r sits at chunk j ^ (r & 7).  `half` selects columns [0,32) or [32,64).
__device__ __forceinline__ void stage_row128(uint32_t box_smem, int row, int half, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t w0 = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
    uint32_t w1 = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
    uint32_t w2 = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
    uint32_t w3 = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
    uint32_t addr = box_smem + row * 128 + (((half * 4 + j) ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                 : "memory");
  }
}

struct TileCoord {
  int m_idx, n_idx;
};

// Tiles are walked in groups of 8 m-tiles so that the CTAs running at the same time share
// A and B tiles in L2.  `m_rotate` shifts the m order (all-gather: own rows first).
__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles, int m_rotate) {
  constexpr int GROUP_M = 8;
  int per_group = GROUP_M * n_tiles;
  int group = tile / per_group;
  int first_m = group * GROUP_M;
  int group_m = min(GROUP_M, m_tiles - first_m);
  int in_group = tile - group * per_group;
  TileCoord c;
  c.m_idx = first_m + in_group % group_m;
  c.n_idx = in_group / group_m;
  c.m_idx += m_rotate;
  if (c.m_idx >= m_tiles) c.m_idx -= m_tiles;
  return c;
}

// PAIR: two CTAs of a cluster work on one 256-row tile with tcgen05 cta_group::2.  Each CTA loads
// its own 128 rows of A and its own half of the B tile (plain TMA loads, no multicast); the
// leader CTA issues the MMAs for both, so every SM pulls a third less from L2 per FLOP.
struct Work {
  int m0, ka0, kb0, k_blocks, bn0, d_row0, d_col0;
};
// Resolve tile number `tile` for the CTA with rank `cta_rank` in its pair.
__device__ __forceinline__ Work get_work(const Params& p, int tile, int cta_rank, int ctas, int tile_n) {
  Work w;
  if (p.tiles != nullptr) {
    const TileDesc d = p.tiles[tile];
    w.m0 = d.a_mn0 + cta_rank * BM;
    w.ka0 = d.k0;
    w.kb0 = d.k0 + d.b_k0;
    w.k_blocks = d.k_blocks;
    w.bn0 = d.b_mn0;
    w.d_row0 = d.d_row0 + cta_rank * BM;
    w.d_col0 = d.d_col0;
  } else {
    TileCoord tc = tile_coord(tile, p.m_units, p.n_tiles, p.m_rotate);
    w.m0 = (tc.m_idx * ctas + cta_rank) * BM;
    w.ka0 = w.kb0 = 0;
    w.k_blocks = p.k_blocks;
    w.bn0 = tc.n_idx * tile_n;
    w.d_row0 = w.m0;
    w.d_col0 = w.bn0;
  }
  return w;
}

// four 8-bit codes -> two bf16x2 words (c - 128) * s, exact until the final rounding to bf16
__device__ __forceinline__ void dequant_bytes(uint32_t w, float s, uint32_t& lo, uint32_t& hi) {
  const float k = 8388736.f;                                      // 2^23 + 128
  const float f0 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)) - k) * s;
  const float f1 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)) - k) * s;
  const float f2 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)) - k) * s;
  const float f3 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)) - k) * s;
  lo = pack_bf16(f0, f1);
  hi = pack_bf16(f2, f3);
}
// eight 4-bit codes of one word (nibble order 0,4,1,5,2,6,3,7 = k 0..7) -> eight bf16 (c - 8) * s, in k order
__device__ __forceinline__ uint4 dequant_nibbles(uint32_t p, __nv_bfloat162 s2) {
  const __nv_bfloat162 bias2 = __floats2bfloat162_rn(136.f, 136.f);
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t t = ((p >> (4 * i)) & 0x000F000Fu) | 0x43004300u;          // bf16(128 + code) in both halves
    __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), bias2), s2);
    o[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// BQ: 0 = B comes by TMA (bf16); 4 / 8 = B is group-quantised and is dequantised into the stages by extra warps.
template <int A_MN, int B_MN, int EPI, bool AG, int BN_T, bool PAIR, int BQ = 0>
__global__ void __launch_bounds__(NUM_THREADS + ((AG || BQ != 0) ? 32 * COMM_WARPS : 0), 1)
gemm_kernel(const __grid_constant__ Params p) {
  static_assert(!(AG && BQ != 0), "the extra warps push the all-gather or dequantise weights, not both");
  static_assert(BQ == 0 || (!B_MN && (EPI == EPI_STORE)), "quantised weights: K-major B, plain store epilogue");
  // tile width is a template parameter: 256 or 128; a CTA stages BN (single) or BN/2 (pair) rows of B
  constexpr int BN = BN_T;
  constexpr int CTAS = PAIR ? 2 : 1;
  constexpr int BN_CTA = BN / CTAS;
  constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr int STAGES = (STAGE_BYTES == 48 * 1024) ? 4 : (STAGE_BYTES == 32 * 1024 ? 6 : 8);
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  static_assert(STAGES * STAGE_BYTES == gemm::STAGES * gemm::STAGE_BYTES, "every variant uses the same shared memory");
  static_assert(EPI != EPI_GLU_FWD || BN == 256, "GLU forward keeps gate and up halves in one 256-wide accumulator");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA0 = smem_base;
  const uint32_t sB0 = smem_base + STAGES * A_STAGE_BYTES;
  const uint32_t sStage0 = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bars = sStage0 + STAGING_BYTES;
  // barrier map (8 B each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then words
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + STAGES * STAGE_BYTES + STAGING_BYTES + 8 * (2 * STAGES + 4));
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a unit is one m-tile, or a pair of them; in descriptor mode the count lives on the device
  const int total_tiles = p.tiles != nullptr ? *p.n_tiles_dev : p.m_units * p.n_tiles;
  constexpr int TILE_N = (EPI == EPI_GLU_FWD) ? BN / 2 : BN;
  const int tile_first = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1 + (BQ != 0 ? COMM_WARPS * CTAS : 0));   // + one arrival per dequantising warp
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EPI_WARPS * CTAS);
    }
    *abort_smem = 0;
    fence_mbar_init();
    prefetch_tmap(&p.tmA);
    if (BQ == 0) prefetch_tmap(&p.tmB);
    if (EPI != EPI_SCATTER) prefetch_tmap(&p.tmD);
  }
  if (warp == 0) {
    tmem_alloc<CTAS>(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ===================================================================== TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int k_checked = 0;       // K row blocks already seen complete (counters only grow)
      if (p.pdl_trigger && tile_first + tile_step >= total_tiles) griddep_launch_dependents();
      for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
        const Work wk = get_work(p, tile, (int)cta_rank, CTAS, TILE_N);
        const int m0 = wk.m0, n0 = wk.bn0;
        // checked build: a tile descriptor built on the device names coordinates inside its matrices, on the 16-byte
        // grid that a TMA copy needs (an unaligned innermost coordinate is an illegal instruction); a bad tile is
        // recorded and the kernel unwinds
        if (p.tiles != nullptr &&
            !(MESH_CHECK_INDEX(m0 - (int)cta_rank * BM, p.a_extent, p.status) && MESH_CHECK_INDEX(n0, p.b_extent, p.status) &&
              MESH_CHECK_ALIGNED(wk.ka0, 8, p.status) && MESH_CHECK_ALIGNED(wk.kb0, 8, p.status) &&
              MESH_CHECK_ALIGNED(A_MN ? m0 : 0, 64, p.status) && MESH_CHECK_ALIGNED(B_MN ? n0 : 0, 64, p.status))) {
          ok = false; *abort_smem = 1; break;
        }
        // this CTA's last tile: the next launch may take the SMs that other CTAs are about to leave
        if (p.pdl_trigger && tile + tile_step >= total_tiles && tile != tile_first) griddep_launch_dependents();
        // all-gather: this rank's own rows are read straight from the source shard (no wait);
        // rows that arrive from other GPUs wait for their arrival counter.
        const int own_lo = AG ? p.rank * p.ag_rows_per_rank : 0;
        const bool own = AG && m0 >= own_lo && m0 < own_lo + p.ag_rows_per_rank;
        if (p.a_ready != nullptr && !own && (p.tiles != nullptr || m0 < p.M)) {
          ok = wait_flag_ge(p.a_ready + m0 / p.a_ready_rows, p.a_ready_value, p.status, SITE_LOCAL_FLAG);
          if (!ok) { *abort_smem = 1; break; }
          fence_proxy_async_all();   // data was written through the generic proxy, TMA reads it
        }
        for (int kb = 0; kb < wk.k_blocks; ++kb) {
          const int ka = wk.ka0 + kb * BK, kbb = wk.kb0 + kb * BK;      // K coordinates in A and in B
          if (p.k_ready != nullptr) {
            const int need = (ka + BK - 1) / p.k_ready_rows + 1;
            while (ok && k_checked < need) {
              ok = wait_flag_ge(p.k_ready + k_checked, p.k_ready_value, p.status, SITE_LOCAL_FLAG);
              ++k_checked;
              if (ok && k_checked == need) fence_proxy_async_all();
            }
            if (!ok) { *abort_smem = 1; break; }
          }
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, p.status, SITE_SMEM_EMPTY);
          if (!ok) break;
          const uint32_t sA = sA0 + stage * A_STAGE_BYTES;
          const uint32_t sB = sB0 + stage * B_STAGE_BYTES;
          if constexpr (!PAIR) {
            const uint32_t fb = full_bar(stage);
            mbar_expect_tx(fb, BQ != 0 ? A_STAGE_BYTES : STAGE_BYTES);
            if (A_MN) tma_load_3d(sA, &p.tmA, fb, 0, ka, m0 / 64);
            else if (own) tma_load_2d(sA, &p.tmA2, fb, ka, m0 - own_lo);
            else      tma_load_2d(sA, &p.tmA, fb, ka, m0);
            if (BQ != 0) {
              // B is written by the dequantising warps
            } else if (EPI == EPI_GLU_FWD) {
              tma_load_2d(sB, &p.tmB, fb, kbb, n0);
              tma_load_2d(sB + B_STAGE_BYTES / 2, &p.tmB, fb, kbb, p.b_up_rows + n0);
            } else if (B_MN) {
              tma_load_3d(sB, &p.tmB, fb, 0, kbb, n0 / 64);
            } else {
              tma_load_2d(sB, &p.tmB, fb, kbb, n0);
            }
          } else {
            // Both CTAs' bytes are counted on the leader's barrier; only the leader arms it.
            if (cta_rank == 0) mbar_expect_tx(full_bar(stage), 2 * (BQ != 0 ? A_STAGE_BYTES : STAGE_BYTES));
            const uint32_t fb = mapa_u32(full_bar(stage), 0);
            if (A_MN) tma_load_3d_pair(sA, &p.tmA, fb, 0, ka, m0 / 64);
            else if (own) tma_load_2d_pair(sA, &p.tmA2, fb, ka, m0 - own_lo);
            else      tma_load_2d_pair(sA, &p.tmA, fb, ka, m0);
            if (BQ != 0) {
              // B is written by the dequantising warps
            } else if (EPI == EPI_GLU_FWD) {
              // leader stages the gate rows, its peer the up rows: accumulator columns [0,128) | [128,256)
              tma_load_2d_pair(sB, &p.tmB, fb, kbb, (cta_rank ? p.b_up_rows : 0) + n0);
            } else if (B_MN) {
              tma_load_3d_pair(sB, &p.tmB, fb, 0, kbb, (n0 + (int)cta_rank * BN_CTA) / 64);
            } else {
              tma_load_2d_pair(sB, &p.tmB, fb, kbb, n0 + (int)cta_rank * BN_CTA);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ===================================================================== MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM * CTAS, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step, ++t) {
        const int acc = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_smem, p.status, SITE_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int tile_k_blocks = p.tiles != nullptr ? p.tiles[tile].k_blocks : p.k_blocks;
        for (int kb = 0; kb < tile_k_blocks; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_smem, p.status, SITE_SMEM_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sA = sA0 + stage * A_STAGE_BYTES;
          const uint32_t sB = sB0 + stage * B_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 k-elements = 32 B inside the 128 B swizzle row; 8-row groups 1 KiB apart.
            // MN-major: 16 k-rows = 2 KiB; 64-element MN groups one TMA box (64 rows * 128 B) apart.
            const uint64_t da = A_MN ? umma_smem_desc(sA + k * 2048, 8192, 1024)
                                     : umma_smem_desc(sA + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sB + k * 2048, 8192, 1024)
                                     : umma_smem_desc(sB + k * 32, 16, 1024);
            umma_f16<CTAS>(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // stage is free (in both CTAs of a pair) once these MMAs have read it
          if constexpr (PAIR) umma_commit_pair(empty_bar(stage), 3);
          else umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if constexpr (PAIR) umma_commit_pair(tfull_bar(acc), 3);
          else umma_commit(tfull_bar(acc));
        }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ===================================================================== epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const uint32_t my_staging = sStage0 + (warp - 2) * EPI_BUFS * EPI_BOX_BYTES;
    int buf = 0;
    bool ok = true;
    int t = 0;
    // Claim a staging box: at most EPI_BUFS-1 earlier stores may still be reading smem.
    auto claim_box = [&]() -> uint32_t {
      if (lane == 0) tma_store_wait_read<EPI_BUFS - 1>();
      __syncwarp();
      uint32_t b = my_staging + buf * EPI_BOX_BYTES;
      buf = (buf + 1) & (EPI_BUFS - 1);
      return b;
    };
    auto emit_box = [&](const CUtensorMap* tm, uint32_t box, int col, int row) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(tm, box, col, row);
        tma_store_commit();
      }
    };
    for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step, ++t) {
      const Work wk = get_work(p, tile, (int)cta_rank, CTAS, TILE_N);
      const int m0 = wk.d_row0;
      const int acc = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      ok = mbar_wait(tfull_bar(acc), acc_phase, abort_smem, p.status, SITE_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);      // tcgen05.ld below is warp-collective
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      const int grow = m0 + row_in_tile;

      if constexpr (EPI == EPI_STORE) {
        const int n0 = wk.d_col0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          uint32_t box = claim_box();
          stage_row(box, lane, v);
          emit_box(&p.tmD, box, n0 + c * 32, m0 + q * 32);
        }
      } else if constexpr (EPI == EPI_GLU_FWD) {
        const int n0 = wk.d_col0;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          if (n0 + c * 32 >= p.N) break;
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c * 32, rg);
          tmem_ld_32x32(taddr + BN / 2 + c * 32, ru);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i)
            v[i] = act_fwd(__uint_as_float(rg[i]), p.act) * __uint_as_float(ru[i]);
          uint32_t box = claim_box();
          stage_row(box, lane, v);
          emit_box(&p.tmD, box, n0 + c * 32, m0 + q * 32);
          if (p.has_d2) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rg[i]);
            box = claim_box();
            stage_row(box, lane, v);
            emit_box(&p.tmD2, box, n0 + c * 32, m0 + q * 32);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ru[i]);
            box = claim_box();
            stage_row(box, lane, v);
            emit_box(&p.tmD2, box, p.d_up_cols + n0 + c * 32, m0 + q * 32);
          }
        }
      } else if constexpr (EPI == EPI_GLU_BWD) {
        // g,u are fetched with coalesced loads (4 lanes per 64-byte row segment), one chunk
        // ahead, transposed through the staging boxes, and the same boxes then carry dg,du out.
        const int n0 = wk.d_col0;
        const int lrow = lane >> 2, lchunk = lane & 3;        // loader role: row (of 8), 16-byte chunk
        const int n_chunks = min(BN / 32, (p.N - n0 + 31) / 32);
        uint4 gq[4], uq[4];
        auto fetch = [&](int c) {
          const int col = n0 + c * 32 + lchunk * 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = m0 + q * 32 + lrow + 8 * i;
            const bool in = (r < p.M) && (col < p.N);
            const __nv_bfloat16* ptr = p.aux + (long long)r * p.ld_aux + col;
            gq[i] = in ? __ldg(reinterpret_cast<const uint4*>(ptr)) : make_uint4(0, 0, 0, 0);
            uq[i] = in ? __ldg(reinterpret_cast<const uint4*>(ptr + p.d_up_cols)) : make_uint4(0, 0, 0, 0);
          }
        };
        fetch(0);
#pragma unroll 1
        for (int c = 0; c < n_chunks; ++c) {
          const int col = n0 + c * 32;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          // boxes of this chunk: set (c & 1); the stores issued two chunks ago must have left them
          if (lane == 0) tma_store_wait_read<2>();
          __syncwarp();
          const uint32_t gbox = my_staging + ((c & 1) * 2) * EPI_BOX_BYTES;
          const uint32_t ubox = gbox + EPI_BOX_BYTES;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = lrow + 8 * i;
            const uint32_t off = rr * 64 + ((lchunk ^ ((rr >> 1) & 3)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(gbox + off), "r"(gq[i].x), "r"(gq[i].y),
                         "r"(gq[i].z), "r"(gq[i].w) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ubox + off), "r"(uq[i].x), "r"(uq[i].y),
                         "r"(uq[i].z), "r"(uq[i].w) : "memory");
          }
          if (c + 1 < n_chunks) fetch(c + 1);
          __syncwarp();
          float dg[32], du[32];
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t off = lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4);
            uint32_t gw[4], uw[4];
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(gw[0]), "=r"(gw[1]), "=r"(gw[2]), "=r"(gw[3])
                         : "r"(gbox + off) : "memory");
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(uw[0]), "=r"(uw[1]), "=r"(uw[2]), "=r"(uw[3])
                         : "r"(ubox + off) : "memory");
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              float2 g2 = unpack_bf16(gw[h]);
              float2 u2 = unpack_bf16(uw[h]);
              const int i = 8 * j + 2 * h;
              float da0 = __uint_as_float(r[i]), da1 = __uint_as_float(r[i + 1]);
              float d0, d1;
              float a0 = act_fwd_bwd(g2.x, p.act, d0);
              float a1 = act_fwd_bwd(g2.y, p.act, d1);
              dg[i] = da0 * u2.x * d0;
              dg[i + 1] = da1 * u2.y * d1;
              du[i] = da0 * a0;
              du[i + 1] = da1 * a1;
            }
          }
          __syncwarp();                       // every lane has read its g,u row before it is overwritten
          stage_row(gbox, lane, dg);
          stage_row(ubox, lane, du);
          emit_box(&p.tmD, gbox, col, m0 + q * 32);
          if (lane == 0) {
            tma_store_2d(&p.tmD, ubox, p.d_up_cols + col, m0 + q * 32);
            tma_store_commit();
          }
        }
      } else {  // EPI_SCATTER: partial tile goes to the rank that owns these rows
        const int owner = m0 / p.rs_rows_per_rank;
        const int owner_m_tile = (m0 - owner * p.rs_rows_per_rank) / BM;
        const int m_tiles_local = p.rs_rows_per_rank / BM;
        // row of the [.., 64]-column view where this warp's first box of the tile starts
        const int n_idx = wk.d_col0 / BN;
        const int row_base = (((p.rank * m_tiles_local + owner_m_tile) * p.n_tiles + n_idx) * (BN / 64)) * BM + q * 32;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          if (n_idx * BN + c * 64 >= p.N) break;
          if (lane == 0) tma_store_wait_read<1>();     // two 4 KiB boxes per warp, used alternately
          __syncwarp();
          const uint32_t box = my_staging + (c & 1) * 2 * EPI_BOX_BYTES;
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 64 + hlf * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            stage_row128(box, lane, hlf, v);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&p.tmRS[owner], box, 0, row_base + c * BM);
            tma_store_commit();
          }
        }
        // publish: wait until this warp's bulk stores are complete, order them before the flag at
        // system scope, then one arrival per warp on the owner's counter for this tile
        if (lane == 0) {
          tma_store_wait_all<0>();
          fence_proxy_async_all();
          red_release_sys_add(p.rs_count[owner] + owner_m_tile * p.n_tiles + n_idx, 1u);
        }
        __syncwarp();
      }
      // accumulator fully read: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && cta_rank != 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
        else mbar_arrive(tempty_bar(acc));
      }
      if (EPI != EPI_SCATTER && p.d_done != nullptr && m0 < p.M) {
        // this warp's 32 rows of the tile are in global memory: one arrival on the row block's counter
        if (lane == 0) {
          tma_store_wait_all<0>();
          fence_proxy_async_all();
          red_release_gpu_add(p.d_done + m0 / BM, 1u);
        }
        __syncwarp();
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  } else if (BQ != 0) {
    // ===================================================================== weight dequantisation
    // 128 threads fill this CTA's B stage for every k block: a thread takes half rows (32 k = 64 bytes of bf16 = four
    // 16-byte chunks), reads their codes one k block ahead, and stores chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)
    // inside 1 KiB groups of 8 rows: the image of a 128-byte-swizzled TMA load.
    const int tid = (warp - (2 + EPI_WARPS)) * 32 + lane;
    constexpr int NT = COMM_WARPS * 32;
    constexpr int UNITS = BN_CTA * 2 / NT;                 // half rows per thread and k block (1, 2 or 4)
    static_assert(BN_CTA * 2 % NT == 0, "half rows must divide among the dequantising threads");
    constexpr int WORDS = BQ == 4 ? 4 : 8;                 // 32-bit code words per half row
    const int my_tiles = tile_first < total_tiles ? (total_tiles - tile_first + tile_step - 1) / tile_step : 0;
    const int steps = my_tiles * p.k_blocks;
    uint32_t cur[UNITS][WORDS], nxt[UNITS][WORDS];
    float cur_s[UNITS], nxt_s[UNITS];
    auto fetch = [&](int step, uint32_t (&w)[UNITS][WORDS], float (&sc)[UNITS]) {
      const int ti = step / p.k_blocks, kb = step - ti * p.k_blocks;
      const Work wk = get_work(p, tile_first + ti * tile_step, (int)cta_rank, CTAS, TILE_N);
      const int n_base = wk.bn0 + (int)cta_rank * BN_CTA;
      const int k0 = wk.kb0 + kb * BK;
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        const int unit = tid + u * NT, row = unit >> 1, half = unit & 1;
        const int n = n_base + row;
        if (n < p.bq_rows) {
          const uint8_t* src = p.bq_codes + (long long)n * p.bq_row_bytes + (BQ == 4 ? (k0 >> 1) + half * 16 : k0 + half * 32);
          const uint4 q0 = __ldg(reinterpret_cast<const uint4*>(src));
          w[u][0] = q0.x; w[u][1] = q0.y; w[u][2] = q0.z; w[u][3] = q0.w;
          if constexpr (BQ == 8) {
            const uint4 q1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
            w[u][4] = q1.x; w[u][5] = q1.y; w[u][6] = q1.z; w[u][7] = q1.w;
          }
          sc[u] = __half2float(p.bq_scales[(long long)n * p.bq_scale_ld + (k0 >> 6)]);
        } else {
#pragma unroll
          for (int j = 0; j < WORDS; ++j) w[u][j] = BQ == 4 ? 0x88888888u : 0x80808080u;    // codes of zero
          sc[u] = 0.f;
        }
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    if (steps > 0) fetch(0, cur, cur_s);
    for (int step = 0; ok && step < steps; ++step) {
      if (step + 1 < steps) fetch(step + 1, nxt, nxt_s);
      ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, p.status, SITE_SMEM_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t sB = sB0 + stage * B_STAGE_BYTES;
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        const int unit = tid + u * NT, row = unit >> 1, half = unit & 1;
        const uint32_t row_addr = sB + (row >> 3) * 1024 + (row & 7) * 128;
        const __nv_bfloat162 s2 = __floats2bfloat162_rn(cur_s[u], cur_s[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          if constexpr (BQ == 4) {
            v = dequant_nibbles(cur[u][j], s2);
          } else {
            dequant_bytes(cur[u][2 * j], cur_s[u], v.x, v.y);
            dequant_bytes(cur[u][2 * j + 1], cur_s[u], v.z, v.w);
          }
          const uint32_t addr = row_addr + ((((uint32_t)(half * 4 + j)) ^ ((uint32_t)row & 7u)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
      }
      fence_proxy_async_smem();               // the tensor core reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) {
        if (PAIR && cta_rank != 0) mbar_arrive_cluster(mapa_u32(full_bar(stage), 0));
        else mbar_arrive(full_bar(stage));
      }
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        cur_s[u] = nxt_s[u];
#pragma unroll
        for (int j = 0; j < WORDS; ++j) cur[u][j] = nxt[u][j];
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
  } else if (AG) {
    // ===================================================================== all-gather push
    // The comm warps of all CTAs together store this rank's rows into every rank's gathered buffer: first to the rank
    // before this one, then the one before that, and so on, the own copy last, because each consumer walks its tiles
    // starting from its own rows (read from the source, no wait) and continuing with the next rank's.  128-row blocks
    // go in `ag_split` parts, each raising the destination's counter once; with enough parts that one destination
    // occupies every CTA, the ranks send along one permutation at a time and each block arrives at the full rate of a
    // port, in the order it is needed, instead of all blocks arriving together at the end.
    const int cw = warp - (2 + EPI_WARPS);
    const int tid = cw * 32 + lane;
    constexpr int NT = COMM_WARPS * 32;
    const int split = p.ag_split;
    const int blocks_per_rank = p.ag_rows_per_rank / p.a_ready_rows;
    const long long vec_per_block = (p.ag_ld / 8) * p.a_ready_rows;   // 16-byte vectors
    const long long per_part = (vec_per_block + split - 1) / split;
    const int units = blocks_per_rank * p.world * split;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
      const int part = unit % split;
      const int blk = (unit / split) % blocks_per_rank;
      const int step = (unit / (split * blocks_per_rank) + 1) % p.world;   // 1 .. world-1, then 0 (the own copy)
      const int dest = (p.rank - step + p.world) % p.world;
      const long long row0 = (long long)blk * p.a_ready_rows;
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_src + row0 * p.ag_ld);
      uint4* dst = reinterpret_cast<uint4*>(
          p.ag_dst[dest] + ((long long)p.rank * p.ag_rows_per_rank + row0) * p.ag_ld);
      const long long beg = part * per_part;
      const long long end = min(vec_per_block, beg + per_part);
      long long i = beg + tid;
      for (; i + 7 * NT < end; i += 8 * NT) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(src + i + u * NT);
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[i + u * NT] = v[u];
      }
      for (; i < end; i += NT) dst[i] = __ldg(src + i);
      // named barrier among the comm warps only (id 1), then one arrival for this part: the release below is
      // cumulative over the stores the barrier ordered before it, so one system-scope fence serves the group
      asm volatile("bar.sync 1, %0;" ::"n"(COMM_WARPS * 32) : "memory");
      if (tid == 0)
        red_release_sys_add(p.ag_flags[dest] + p.rank * blocks_per_rank + blk, 1u);
    }
  }

  // ------------------------------------------------------------------------- teardown
  if (p.pdl_trigger) griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA frees TMEM or exits while its peer still uses the pair
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
  }

  if constexpr (EPI == EPI_SCATTER) {
    // =================================================================== reduce tail
    // Sum the `world` partial copies of every (m-tile, n-tile) of this rank's rows once
    // its arrival counter shows that all of them landed.
    // A tile is cut into `split` row slices when there are fewer tiles than CTAs (few rows per rank at large world
    // sizes), so that every SM takes part in the sum.
    const int my_m_tiles = (p.rs_rows_per_rank + BM - 1) / BM;
    const int tiles_mine = my_m_tiles * p.n_tiles;
    int split = 1;                       // all-reduce counts one arrival per tile on the other ranks: tiles stay whole
    while (p.ar_out[0] == nullptr && split < 8 && tiles_mine * split * 2 <= (int)gridDim.x) split *= 2;
    const int items = tiles_mine * split;
    const int slice_rows = BM / split;
    __shared__ int item_ok;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int tile_i = item / split, slice = item - tile_i * split;
      const int mt = tile_i / p.n_tiles, nt = tile_i % p.n_tiles;
      if (threadIdx.x == 0) {
        item_ok = wait_flag_ge(p.rs_count[p.rank] + tile_i, p.rs_expect, p.status, SITE_PEER_FLAG) ? 1 : 0;
      }
      __syncthreads();
      const bool good = item_ok != 0;
      __syncthreads();
      if (!good) break;
      const int cols = min(BN, p.N - nt * BN);
      const int m_tiles_local = p.rs_rows_per_rank / BM;
      constexpr int TILE_ELEMS = BM * BN;
      // one 16-byte vector per thread and step: (chunk c, row r, vector v) with v fastest
      const int per_chunk = slice_rows * 8;
      for (int idx = threadIdx.x; idx < (BN / 64) * per_chunk; idx += blockDim.x) {
        const int c = idx / per_chunk, in_chunk = idx - c * per_chunk;
        const int v = in_chunk & 7, r = slice * slice_rows + (in_chunk >> 3);
        if (c * 64 + v * 8 >= cols) continue;
        const long long in_tile = (long long)c * (BM * 64) + r * 64 + v * 8;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint4 w[MAX_RANKS];
#pragma unroll
        for (int s = 0; s < MAX_RANKS; ++s) {       // all sources in flight, then a fixed-order sum
          if (s < p.world) {
            const long long tile = ((long long)s * m_tiles_local + mt) * p.n_tiles + nt;
            w[s] = __ldcg(reinterpret_cast<const uint4*>(p.rs_recv + tile * TILE_ELEMS + in_tile));
          }
        }
#pragma unroll
        for (int s = 0; s < MAX_RANKS; ++s) {
          if (s < p.world) {
            const uint32_t ww[4] = {w[s].x, w[s].y, w[s].z, w[s].w};
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              float2 f = unpack_bf16(ww[h]);
              acc[2 * h] += f.x;
              acc[2 * h + 1] += f.y;
            }
          }
        }
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]);
        o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]);
        o.w = pack_bf16(acc[6], acc[7]);
        const long long at = (long long)(mt * BM + r) * p.N + nt * BN + c * 64 + v * 8;
        if (p.rs_out != nullptr) *reinterpret_cast<uint4*>(p.rs_out + at) = o;
        if (p.ar_out[0] != nullptr) {
          // all-reduce: the summed tile goes into every rank's full output, at this rank's rows
          const long long full = (long long)p.rank * p.rs_rows_per_rank * p.N + at;
#pragma unroll
          for (int d = 0; d < MAX_RANKS; ++d)
            if (d < p.world) *reinterpret_cast<uint4*>(p.ar_out[d] + full) = o;
        }
      }
      if (p.ar_out[0] != nullptr) {
        // one arrival per tile on every other rank's counter; the barrier orders the block's stores before the
        // signalling threads, whose system-scope release is cumulative over them
        __syncthreads();
        if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) red_release_sys_add(p.ar_flag[threadIdx.x], 1u);
      }
    }
    if (p.ar_out[0] != nullptr) {
      // the full output is complete here once every other rank's tiles have arrived
      if (threadIdx.x == 0) item_ok = wait_flag_ge(p.ar_flag[p.rank], p.ar_expect, p.status, SITE_PEER_FLAG) ? 1 : 0;
      __syncthreads();
    }
  }
  // A kernel that started before its predecessor had finished does not finish before it: whoever is ordered after
  // this kernel in the stream is then ordered after the whole chain.
  griddep_wait();
}

}  // namespace gemm
}  // namespace mesh
