// Host side of the tcgen05 GEMM: argument checks, TMA descriptor encoding, launch.
#include "gemm_sm100.cuh"
#include "gemm_api.h"
#include "../runtime/host_common.h"

#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>

namespace mesh {
namespace gemm {

// 2-D map over a row-major bf16 matrix [rows, cols] with leading dimension ld (elements).
static bool make_map_2d(CUtensorMap* tm, const void* base, uint64_t cols, uint64_t rows, uint64_t ld,
                        uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swz) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, swz);
}

// 3-D map that makes a row-major [k_rows, mn_cols] matrix look like [mn_cols/64][k_rows][64], so
// that one box {64, 64, groups} lands in shared memory as `groups` consecutive 8 KiB
// [64 k-rows][128 B] slabs — the MN-major canonical layout tcgen05 expects.
static bool make_map_mn(CUtensorMap* tm, const void* base, uint64_t mn_cols, uint64_t k_rows, uint64_t ld,
                        uint32_t groups) {
  cuuint64_t dims[3] = {64, k_rows, mn_cols / 64};
  cuuint64_t strides[2] = {ld * 2, 128};
  cuuint32_t box[3] = {64, 64, groups};
  cuuint32_t estr[3] = {1, 1, 1};
  return encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int A_MN, int B_MN, int EPI, bool AG, int BNV, bool PAIR, int BQ = 0>
static int launch(const Params& p, int ctas, cudaStream_t stream, bool dependent) {
  auto kern = gemm_kernel<A_MN, B_MN, EPI, AG, BNV, PAIR, BQ>;
  static bool configured = false;   // per instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return set_error((int)e, "cudaFuncSetAttribute(gemm smem): %s", cudaGetErrorString(e));
    configured = true;
  }
  const int threads = NUM_THREADS + ((AG || BQ != 0) ? 32 * COMM_WARPS : 0);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_error((int)e, "gemm launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace gemm
}  // namespace mesh

using namespace mesh;
using namespace mesh::gemm;

extern "C" int mesh_gemm_choose_tile_n(int M, int N, int ctas) {
  if (ctas <= 0) ctas = sm_count();
  const long m_tiles = (M + BM - 1) / BM;
  auto eff = [&](int bn) {
    const long tiles = m_tiles * ((N + bn - 1) / bn);
    const long waves = (tiles + ctas - 1) / ctas;
    return (double)tiles / (double)(waves * ctas) * ((double)N / (double)(((N + bn - 1) / bn) * bn));
  };
  // a 128-wide tile re-reads A twice as often and runs nearer the shared-memory limit: it has to
  // win by a clear margin before it is chosen
  return eff(128) * 0.80 > eff(256) ? 128 : 256;
}

extern "C" int mesh_gemm_bf16(const MeshGemmArgs* a, void* stream_v) {
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return set_error(-1, "gemm: empty problem");
  if (a->K % 8 || a->N % 8 || a->lda % 8 || a->ldb % 8)
    return set_error(-2, "gemm: K, N and leading dimensions must be multiples of 8 (16-byte TMA rule)");
  if ((uintptr_t)a->A % 16 || (uintptr_t)a->B % 16) return set_error(-2, "gemm: operands must be 16-byte aligned");
  if (a->a_mn && (a->M % 64)) return set_error(-3, "gemm: MN-major A needs M %% 64 == 0");
  if (a->b_mn && (a->N % 64)) return set_error(-3, "gemm: MN-major B needs N %% 64 == 0");
  if ((a->epi == EPI_GLU_FWD || a->epi == EPI_GLU_BWD) && (a->N % 32))
    return set_error(-3, "gemm: GLU epilogues need N %% 32 == 0");
  if (a->epi == EPI_GLU_FWD && a->b_mn) return set_error(-3, "gemm: GLU forward needs K-major weights");
  if (a->world > MESH_MAX_RANKS) return set_error(-4, "gemm: world > %d", MESH_MAX_RANKS);

  Params p;
  memset(&p, 0, sizeof(p));
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.m_tiles = (a->M + BM - 1) / BM;
  int ctas = a->num_ctas > 0 ? a->num_ctas : sm_count();
  // Tile width: 256 by default; 128 when that fills the last wave of CTAs much better.
  int bn = a->tile_n;
  if (a->epi == EPI_GLU_FWD) bn = 256;
  if (bn != 128 && bn != 256) bn = mesh_gemm_choose_tile_n(a->M, a->N, ctas);
  const int tile_n = (a->epi == EPI_GLU_FWD) ? BN / 2 : bn;
  p.n_tiles = (a->N + tile_n - 1) / tile_n;
  // cta_group::2 pairs (256-row tiles) unless switched off or the problem has a single m-tile
  const bool pair = a->pair >= 0 && p.m_tiles >= 2 && ctas >= 2 && (a->tiles == nullptr || a->pair > 0);
  const int cta_per_unit = pair ? 2 : 1;
  if (pair) ctas &= ~1;
  p.m_units = (p.m_tiles + cta_per_unit - 1) / cta_per_unit;
  const int bn_cta = bn / cta_per_unit;
  p.k_blocks = (a->K + BK - 1) / BK;
  p.act = a->act;
  p.b_up_rows = a->b_up_rows;
  p.d_up_cols = a->d_up_cols;
  p.has_d2 = a->D2 != nullptr;
  p.aux = (const __nv_bfloat16*)a->aux;
  p.ld_aux = a->ld_aux;
  p.status = (Status*)a->status;
  p.d_done = (uint32_t*)a->d_done;
  p.k_ready = (const uint32_t*)a->k_ready;
  p.k_ready_value = a->k_ready_value;
  p.k_ready_rows = a->k_ready_rows > 0 ? a->k_ready_rows : BM;
  if (a->k_ready != nullptr && (p.k_ready_rows % BK)) return set_error(-5, "gemm: k_ready_rows must be a multiple of 64");
  p.pdl_trigger = (a->pdl & 2) ? 1 : 0;
  const bool dependent = (a->pdl & 1) != 0 && pdl_enabled();
  const int bq = a->b_bits;
  if (bq != 0) {
    if (bq != 4 && bq != 8) return set_error(-3, "gemm: quantised weights are 4-bit or 8-bit (b_bits %d)", bq);
    if (a->b_mn || a->a_mn || a->epi != EPI_STORE || a->tiles != nullptr || a->ag_src != nullptr)
      return set_error(-3, "gemm: quantised weights need K-major operands, a plain store epilogue and a dense grid");
    if (a->K % 64) return set_error(-3, "gemm: quantised weights need K %% 64 == 0 (one scale per 64 k)");
    if (a->b_scales == nullptr || (uintptr_t)a->B % 16 || ((bq == 4 ? a->K / 2 : a->K) % 16))
      return set_error(-2, "gemm: quantised weights need scales and 16-byte aligned code rows");
    p.bq_codes = (const uint8_t*)a->B;
    p.bq_scales = (const __half*)a->b_scales;
    p.bq_row_bytes = bq == 4 ? a->K / 2 : a->K;
    p.bq_scale_ld = a->K / 64;
    p.bq_rows = a->b_rows ? a->b_rows : a->N;
  }
  p.a_extent = a->a_mn ? a->M : (a->a_rows ? a->a_rows : a->M);
  p.b_extent = a->b_mn ? a->N : (a->b_rows ? a->b_rows : a->N);
  p.tiles = (const TileDesc*)a->tiles;
  p.n_tiles_dev = (const int*)a->n_tiles_dev;
  p.a_ready = (const uint32_t*)a->a_ready;
  p.a_ready_value = a->a_ready_value;
  p.a_ready_rows = a->a_ready_rows > 0 ? a->a_ready_rows : BM;
  p.m_rotate = a->m_rotate;   // converted to scheduling units below
  p.ag_split = a->ag_split > 0 ? a->ag_split : 8;
  p.rank = a->rank; p.world = a->world > 0 ? a->world : 1;
  const bool ag = a->ag_src != nullptr;
  if (ag) {
    if (a->ag_rows_per_rank % p.a_ready_rows || a->ag_ld % 8)
      return set_error(-5, "gemm: all-gather rows per rank must be a multiple of the flag granularity");
    p.ag_src = (const __nv_bfloat16*)a->ag_src;
    for (int r = 0; r < p.world; ++r) {
      p.ag_dst[r] = (__nv_bfloat16*)a->ag_dst[r];
      p.ag_flags[r] = (uint32_t*)a->ag_flags[r];
    }
    p.ag_rows_per_rank = a->ag_rows_per_rank;
    p.ag_ld = a->ag_ld;
    if ((uintptr_t)a->ag_src % 16) return set_error(-2, "gemm: all-gather source must be 16-byte aligned");
    if (!make_map_2d(&p.tmA2, a->ag_src, (uint64_t)a->K, (uint64_t)a->ag_rows_per_rank, (uint64_t)a->ag_ld, BK, BM,
                     CU_TENSOR_MAP_SWIZZLE_128B))
      return last_error_code();
  }
  if (a->epi == EPI_SCATTER) {
    if (a->rs_rows_per_rank % BM) return set_error(-5, "gemm: reduce-scatter rows per rank must be a multiple of 128");
    // every rank's receive buffer viewed as a [rows, 64] matrix: one box = one contiguous 4 KiB run
    const uint64_t n_tiles_rs = (uint64_t)p.n_tiles;
    const uint64_t view_rows = (uint64_t)p.world * (a->rs_rows_per_rank / BM) * n_tiles_rs * (bn / 64) * BM;
    for (int r = 0; r < p.world; ++r) {
      p.rs_count[r] = (uint32_t*)a->rs_count[r];
      if (!make_map_2d(&p.tmRS[r], a->rs_recv[r], 64, view_rows, 64, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B))
        return last_error_code();
    }
    for (int r = 0; r < p.world; ++r) {
      p.ar_out[r] = (__nv_bfloat16*)a->ar_out[r];
      p.ar_flag[r] = (uint32_t*)a->ar_flag[r];
    }
    p.ar_expect = a->ar_expect;
    if (p.ar_out[0] != nullptr && (a->N % 8)) return set_error(-5, "gemm: all-reduce output needs N %% 8 == 0");
    p.rs_recv = (const __nv_bfloat16*)a->rs_recv[p.rank];
    p.rs_expect = a->rs_expect;
    p.rs_out = (__nv_bfloat16*)a->rs_out;
    p.rs_rows_per_rank = a->rs_rows_per_rank;
  }

  // ---- tensor maps
  bool ok = true;
  if (a->a_mn) ok = ok && make_map_mn(&p.tmA, a->A, (uint64_t)a->M, (uint64_t)(a->a_rows ? a->a_rows : a->K), (uint64_t)a->lda, BM / 64);
  else         ok = ok && make_map_2d(&p.tmA, a->A, (uint64_t)a->K, (uint64_t)(a->a_rows ? a->a_rows : a->M),
                                      (uint64_t)a->lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t b_rows = (uint64_t)(a->b_rows ? a->b_rows : a->N);
  // MN-major B: b_rows (when given) is the number of stored K rows (stacked per-expert weights are taller than K)
  if (bq != 0) { /* no tensor map: the dequantising warps read B */ }
  else if (a->b_mn) ok = ok && make_map_mn(&p.tmB, a->B, (uint64_t)a->N, (uint64_t)(a->b_rows ? a->b_rows : a->K), (uint64_t)a->ldb, bn_cta / 64);
  else         ok = ok && make_map_2d(&p.tmB, a->B, (uint64_t)a->K, b_rows, (uint64_t)a->ldb, BK,
                                      a->epi == EPI_GLU_FWD ? BN / 2 : bn_cta, CU_TENSOR_MAP_SWIZZLE_128B);
  if (a->epi != EPI_SCATTER) {
    if (a->ldd % 8 || (uintptr_t)a->D % 16) return set_error(-2, "gemm: D must be 16-byte aligned with ld %% 8 == 0");
    const uint64_t d_cols = (uint64_t)(a->d_cols ? a->d_cols : a->N);
    const uint64_t d_rows = (uint64_t)(a->d_rows ? a->d_rows : a->M);
    ok = ok && make_map_2d(&p.tmD, a->D, d_cols, d_rows, (uint64_t)a->ldd, EPI_BOX_COLS, 32,
                           CU_TENSOR_MAP_SWIZZLE_64B);
    if (a->D2) {
      const uint64_t d2_cols = (uint64_t)(a->d2_cols ? a->d2_cols : 2 * a->N);
      ok = ok && make_map_2d(&p.tmD2, a->D2, d2_cols, d_rows, (uint64_t)a->ldd2, EPI_BOX_COLS, 32,
                             CU_TENSOR_MAP_SWIZZLE_64B);
    }
  }
  if (!ok) return last_error_code();

  const int tiles = p.m_units * p.n_tiles * cta_per_unit;
  if (!ag && a->epi != EPI_SCATTER && a->tiles == nullptr && ctas > tiles) ctas = tiles;
  if (a->tiles != nullptr && a->max_tiles > 0 && ctas > a->max_tiles * cta_per_unit) ctas = a->max_tiles * cta_per_unit;
  if (pair) {
    if (p.m_rotate % 2) p.m_rotate = 0; else p.m_rotate /= 2;   // rotation is only an ordering hint
  }

#define MESH_LAUNCH(AM, BMJ, E, G)                                          \
  do {                                                                      \
    constexpr int E128 = ((E) == EPI_GLU_FWD ? EPI_STORE : (E));            \
    if (bn == 128 && (E) != EPI_GLU_FWD) {                                  \
      if (pair) return launch<AM, BMJ, E128, G, 128, true>(p, ctas, stream, dependent); \
      return launch<AM, BMJ, E128, G, 128, false>(p, ctas, stream, dependent);         \
    }                                                                       \
    if (pair) return launch<AM, BMJ, E, G, 256, true>(p, ctas, stream, dependent);     \
    return launch<AM, BMJ, E, G, 256, false>(p, ctas, stream, dependent);              \
  } while (0)
  if (bq != 0) {
#define MESH_LAUNCH_Q(Q)                                                               \
    do {                                                                               \
      if (bn == 128) {                                                                 \
        if (pair) return launch<0, 0, EPI_STORE, false, 128, true, Q>(p, ctas, stream, dependent);  \
        return launch<0, 0, EPI_STORE, false, 128, false, Q>(p, ctas, stream, dependent);           \
      }                                                                                \
      if (pair) return launch<0, 0, EPI_STORE, false, 256, true, Q>(p, ctas, stream, dependent);    \
      return launch<0, 0, EPI_STORE, false, 256, false, Q>(p, ctas, stream, dependent);             \
    } while (0)
    if (bq == 4) MESH_LAUNCH_Q(4);
    MESH_LAUNCH_Q(8);
#undef MESH_LAUNCH_Q
  }
  switch (a->epi) {
    case EPI_STORE:
      if (ag) {
        if (!a->a_mn && !a->b_mn) MESH_LAUNCH(0, 0, EPI_STORE, true);
        if (!a->a_mn && a->b_mn) MESH_LAUNCH(0, 1, EPI_STORE, true);
        return set_error(-6, "gemm: all-gather fusion needs K-major activations");
      }
      if (!a->a_mn && !a->b_mn) MESH_LAUNCH(0, 0, EPI_STORE, false);
      if (!a->a_mn && a->b_mn) MESH_LAUNCH(0, 1, EPI_STORE, false);
      if (a->a_mn && !a->b_mn) MESH_LAUNCH(1, 0, EPI_STORE, false);
      MESH_LAUNCH(1, 1, EPI_STORE, false);
    case EPI_GLU_FWD:
      if (a->a_mn) return set_error(-6, "gemm: GLU forward needs K-major activations");
      if (ag) MESH_LAUNCH(0, 0, EPI_GLU_FWD, true);
      MESH_LAUNCH(0, 0, EPI_GLU_FWD, false);
    case EPI_GLU_BWD:
      if (a->a_mn) return set_error(-6, "gemm: GLU backward needs K-major dY");
      if (ag) {
        if (a->b_mn) MESH_LAUNCH(0, 1, EPI_GLU_BWD, true);
        MESH_LAUNCH(0, 0, EPI_GLU_BWD, true);
      }
      if (a->b_mn) MESH_LAUNCH(0, 1, EPI_GLU_BWD, false);
      MESH_LAUNCH(0, 0, EPI_GLU_BWD, false);
    case EPI_SCATTER:
      if (a->a_mn) return set_error(-6, "gemm: reduce-scatter fusion needs K-major A");
      if (a->b_mn) MESH_LAUNCH(0, 1, EPI_SCATTER, false);
      MESH_LAUNCH(0, 0, EPI_SCATTER, false);
    default:
      return set_error(-7, "gemm: unknown epilogue %d", a->epi);
  }
#undef MESH_LAUNCH
}
