// C ABI of the decode-time kernels: skinny fused linear layers, split-KV attention for one query
// token per sequence, and vocabulary-parallel greedy selection.
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define MESH_DEC_MAX_RANKS 8
enum MeshDecodeMode { MESH_DEC_STORE = 0, MESH_DEC_GLU = 1, MESH_DEC_QKV = 2, MESH_DEC_ALLREDUCE = 3 };

typedef struct MeshDecodeLinear {
  const void* x; long long ldx; int B, K, N;      // x [B, K] bf16; N = output rows handled (GLU: gate rows)
  const void* norm_w; float eps, norm_off;         // optional RMSNorm prologue
  const void* w; const void* scales; int w4;       // bf16 [rows, K] or 4-bit codes [rows, K/2] + fp16 scales [rows, K/64]
  int mode, act, up_off;
  void* out; long long ldo; int out_f32;
  int q_heads, kv_heads, head_dim;
  const int* pos; const float* cos_t; const float* sin_t;
  void* q_out; void* k_cache; void* v_cache; int max_seq;
  int rank, world;
  void* ar_recv[MESH_DEC_MAX_RANKS];
  const uint32_t* step_ptr; uint32_t calls_per_step, call_index;   // all-reduce sequence = *step_ptr * calls + index + 1
  const void* residual; long long ldr;
  void* status;
  const void* next_w; unsigned long long next_bytes;   // optional: bytes to prefetch into L2 for the layer that follows
} MeshDecodeLinear;

int mesh_decode_linear(const MeshDecodeLinear* d, void* stream);

// One query token per sequence against the KV cache.  q [B, q_heads, hd] bf16; caches
// [B, kv_heads, max_seq, hd]; keys used: (max(0, pos-window+1) .. pos] when window > 0, else [0, pos].
// scratch: fp32 [B * q_heads * splits * (hd + 2)], counters: int32 [B * kv_heads] (zero before first use;
// the kernel leaves them zero).  out [B, q_heads * hd] bf16.
// tokens_per_seq > 1 (prefill): q is [B, T, q_heads, hd], query t of sequence b sits at position pos[b] + t and
// sees keys up to itself; scratch/counters/out are sized for B * T "sequences".
int mesh_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* pos, void* out,
                          float* scratch, int* counters, int B, int tokens_per_seq, int q_heads, int kv_heads,
                          int head_dim, int max_seq, int window, float scale, int splits, void* stream);
int mesh_decode_attention_scratch_floats(int B, int q_heads, int head_dim, int splits);

// Greedy selection over a vocabulary shard: (max logit, lowest index) per sequence, then MAXLOC over
// ranks with 8 bytes per rank (design/prepared-machine.md: "Vocabulary selection follows MAXLOC").
// logits fp32 [B, ldl]; vocab_offset: first id of this shard; tokens_out int32[B]; pos (may be NULL) is
// incremented by one per sequence.  xchg[d]: rank d's exchange slots uint2[world * 8 * 2].
// step (device word, may be NULL): the exchange's sequence number is *step + 1 and the kernel increments *step.
int mesh_decode_argmax(const float* logits, long long ldl, int B, int vocab_local, int vocab_offset, int* tokens_out,
                       int* pos, int rank, int world, void* const* xchg, uint32_t* step, void* status, void* stream);

// A whole decode step as ONE cooperative kernel: the operations run in order, every CTA of the grid (one per SM) takes
// its share of each, and a grid barrier separates them.  In every CTA one warp streams the weights of all the layers,
// in order, through a ring of stages in shared memory; it never waits at a barrier, so HBM keeps streaming while the
// computing warps wait for the layer before, stage x, reduce and store.
enum MeshDecodeOpKind { MESH_DEC_OP_EMBED = 0, MESH_DEC_OP_LINEAR = 1, MESH_DEC_OP_ATTENTION = 2, MESH_DEC_OP_ARGMAX = 3 };

typedef struct MeshDecodeOp {
  int kind;
  MeshDecodeLinear lin;                                  // LINEAR
  // ATTENTION: arguments of mesh_decode_attention with one query token per sequence
  const void* q; const void* k_cache; const void* v_cache; const int* pos; void* att_out; float* scratch; int* counters;
  int B, q_heads, kv_heads, head_dim, max_seq, window; float scale; int splits;
  // EMBED: x[b, :] = table[tok[b], :]  (bf16 rows of d_model, a multiple of 8)
  const void* table; const int* tok; void* x; int d_model;
  // ARGMAX: arguments of mesh_decode_argmax; part_v / part_i: scratch for batch * mesh_decode_step_max_grid() pairs
  const float* logits; long long ldl; int vocab_local, vocab_offset; int* tokens_out; int* pos_inc; int rank, world;
  void* xchg[MESH_DEC_MAX_RANKS]; uint32_t* step; float* part_v; int* part_i;
  void* status;
} MeshDecodeOp;

// How a prepared step is launched: filled by mesh_decode_step_prepare, passed back to mesh_decode_step_run.
typedef struct MeshDecodeStepPlan {
  int n_dev;          // device operations (a selection is two)
  int grid;           // CTAs: one per SM
  int smem;           // dynamic shared memory per CTA
  int ring_off;       // bytes of per-layer work area in front of the weight ring
  int slot_bytes;     // bytes of one weight stage
  int n_stages;       // stages of the ring
} MeshDecodeStepPlan;

// Bytes of device memory that hold the translated operations of a step of n_ops operations.
size_t mesh_decode_step_bytes(int n_ops);
// Largest grid a step kernel is launched with on this device.
int mesh_decode_step_max_grid(void);
// Checks and translates the operations into dev_ops (a synchronous copy) and fills the launch plan.
int mesh_decode_step_prepare(const MeshDecodeOp* ops, int n_ops, void* dev_ops, size_t dev_bytes, MeshDecodeStepPlan* plan);
// One step.  barrier: two zeroed 32-bit words that belong to this step program (left consistent by every run that
// did not time out inside the barrier itself).  trace (may be NULL): 2 * 3 * n_dev 64-bit words; the first and the last
// CTA write {start, end of own share, nanoseconds spent waiting} (globaltimer) for every operation.
int mesh_decode_step_run(const void* dev_ops, const MeshDecodeStepPlan* plan, uint32_t* barrier, void* status,
                         unsigned long long* trace, void* stream);

#ifdef __cplusplus
}
#endif
