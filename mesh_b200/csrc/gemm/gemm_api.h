// C ABI of the GEMM library (loaded through ctypes; no torch headers involved).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MESH_MAX_RANKS 8

// All leading dimensions are in elements (bf16).  Pointers are device pointers; peer
// pointers (ag_dst, ag_flags, rs_recv, rs_count) come from the symmetric heap.
// One tile of a descriptor-driven GEMM (same layout as mesh::gemm::TileDesc).  In pair mode a descriptor
// covers 256 output rows: the second CTA of the pair adds 128 to a_mn0 and d_row0.
typedef struct MeshTileDesc { int a_mn0, k0, k_blocks, b_mn0, b_k0, d_row0, d_col0, pad; } MeshTileDesc;

typedef struct MeshGemmArgs {
  const void* A;
  const void* B;
  void* D;
  void* D2;
  const void* aux;
  int M, N, K;
  long long lda, ldb, ldd, ldd2, ld_aux;
  int a_rows, b_rows;          // rows of the stored A / B matrices (TMA bounds)
  int d_cols, d2_cols;         // columns of the stored D / D2 matrices (TMA bounds)
  int d_rows;                  // rows of the stored D (0: M); grouped launches write a taller stacked matrix
  int a_mn, b_mn;              // 1: operand is stored [K, rows] (MN-major)
  int epi, act;
  int b_up_rows, d_up_cols;
  void* status;
  // all-gather -> GEMM
  const void* a_ready;
  uint32_t a_ready_value;
  int a_ready_rows;
  int m_rotate;
  const void* ag_src;
  void* ag_dst[MESH_MAX_RANKS];
  void* ag_flags[MESH_MAX_RANKS];
  int ag_rows_per_rank;
  long long ag_ld;
  int rank, world;
  // GEMM -> reduce-scatter
  void* rs_recv[MESH_MAX_RANKS];
  void* rs_count[MESH_MAX_RANKS];
  uint32_t rs_expect;
  void* rs_out;
  int rs_rows_per_rank;
  int num_ctas;                // 0: one per SM
  int tile_n;                  // 0: choose; 128 or 256: width of the output tile
  int pair;                    // 0: cta_group::2 pairs when possible; -1: single-CTA tiles
  // descriptor-driven mode (grouped / ragged GEMMs): device list of MeshTileDesc and its device length
  const void* tiles;
  const void* n_tiles_dev;
  int max_tiles;               // upper bound of *n_tiles_dev (grid sizing only)
  // kernel-to-kernel dataflow between consecutive launches of one stream (see Params in gemm_sm100.cuh)
  void* d_done;                // counters per 128 output rows, raised by the epilogue (4 per tile); NULL: none
  const void* k_ready;         // counters per `k_ready_rows` K rows that a K block waits for; NULL: none
  uint32_t k_ready_value;
  int k_ready_rows;
  // group-quantised weights: B = codes ([N, K/2] 4-bit in nibble order 0,4,1,5,2,6,3,7 per 32-bit word, or [N, K] 8-bit),
  // b_scales = fp16 [N, K/64]; value = (code - 8 or 128) * scale.  Dequantised in registers on the way to the tensor cores.
  const void* b_scales;
  int b_bits;                  // 0: bf16 B; 4 or 8
  int pdl;                     // bit 0: may start before the previous launch of the stream has finished (every input
                               // that launch writes is guarded by a_ready / k_ready); bit 1: let the next launch
                               // start during this kernel's last wave
  // GEMM -> all-reduce (with epi = scatter): after a rank has summed a tile of its rows it stores the tile into every
  // rank's full output `ar_out[r]` ([M, N] bf16 in the symmetric heap) and raises `ar_flag[r]`; the kernel ends once
  // this rank's counter shows every other rank's tiles (`ar_expect`, cumulative over uses).  NULL ar_out[0]: reduce-scatter only.
  void* ar_out[MESH_MAX_RANKS];
  void* ar_flag[MESH_MAX_RANKS];
  uint32_t ar_expect;
  // all-gather: parts a 128-row block is pushed in (each part raises the block's counter once, so a block is there
  // when its counter has grown by ag_split); 0: 8.  With blocks_per_rank * ag_split >= CTAs, all CTAs push to one
  // destination at a time, in the order the destinations need the rows.
  int ag_split;
} MeshGemmArgs;

// Returns 0 or a negative error (bad shape/alignment) or a positive cudaError_t.
int mesh_gemm_bf16(const MeshGemmArgs* args, void* stream);
// Tile width the launcher picks for an M x N problem on `ctas` CTAs (0: one per SM).
int mesh_gemm_choose_tile_n(int M, int N, int ctas);
const char* mesh_last_error(void);

#ifdef __cplusplus
}
#endif
