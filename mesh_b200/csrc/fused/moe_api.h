// C ABI of the expert-parallel MoE kernels (see moe.cu).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define MESH_MOE_MAX_RANKS 8
#define MESH_MOE_MAX_EXPERTS 256
#define MESH_MOE_DISPATCH_BLOCKS 296

// idx int32 [n_entries] (token-major, k choices per token) -> slot[n_entries]; this rank's histogram is pushed to
// every rank's count matrix (count_ptrs[d]: uint2 [2][world][experts]).
// work: int32 [mesh_moe_count_work_ints(n_entries, experts)], zero before the first call (the kernel leaves its
// counter zero).
int mesh_moe_count_work_ints(int n_entries, int experts);
int mesh_moe_count(const int* idx, int n_entries, int* slot, int experts, int rank, int world, void* const* count_ptrs,
                   uint32_t seq, int* work, void* stream);

typedef struct MeshMoePlan {
  const void* counts; uint32_t seq;
  int rank, world, experts, cap_rows, d_model, d_ff;
  int* send_base;            // int32 [experts]
  int* layout;               // int32 [3 * experts/world + 2]
  void* tables[6];           // MeshTileDesc [max_tiles] each: glu, down, dh, dx, dw2, dw1
  int* n_tiles;              // int32 [6]
  int max_tiles;
  void* status;
} MeshMoePlan;
int mesh_moe_plan(const MeshMoePlan* m, void* stream);
int mesh_moe_zero_pad(void* buf, const int* layout, int local_experts, int d_model, void* stream);

typedef struct MeshMoeDispatch {
  const void* x; int tokens, k, d_model;
  const int* idx; const int* slot; const int* send_base; const float* scale; int* meta;
  int local_experts, cap_rows, rank, world;
  void* recv[MESH_MOE_MAX_RANKS];
  void* arrived[MESH_MOE_MAX_RANKS];
  void* status;
} MeshMoeDispatch;
int mesh_moe_dispatch(const MeshMoeDispatch* m, void* stream);
int mesh_moe_signal(int world, void* const* ready_ptrs, void* stream);

typedef struct MeshMoeCombine {
  int tokens, k, d_model, local_experts, world;
  const int* idx; const int* meta; const float* weight;
  const void* src[MESH_MOE_MAX_RANKS];
  const void* ready; uint32_t ready_expect;
  void* out; const void* dot_with; float* dots;
  void* status;
  int cap_rows;                 // rows of every source buffer (bounds of the rows named by `meta`)
} MeshMoeCombine;
int mesh_moe_combine(const MeshMoeCombine* m, void* stream);

#ifdef __cplusplus
}
#endif
