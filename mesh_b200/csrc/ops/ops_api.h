// C ABI of the single-GPU ops (norms, rotary embedding, router, quantised matmul, attention).
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

// y = x * rsqrt(mean(x^2) + eps) * (w + w_offset); if `residual` != NULL, first x += residual (written
// back to `residual_out` when given).  rstd[rows] (fp32) is written when non-NULL.
int mesh_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                     float* rstd, int rows, int cols, float eps, float w_offset, void* stream);
// dx from dy, x, w, rstd; dw_partial[blocks][cols] fp32 scratch is reduced into dw (fp32) by a second
// kernel.  `blocks` rows of scratch are used (<= 1024).
int mesh_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                     float* dw_partial, int blocks, int rows, int cols, float w_offset, void* stream);
int mesh_rmsnorm_bwd_blocks(int rows);

// Rotate-half rotary embedding, in place, on x[tokens, heads, head_dim] (row stride `ld` elements
// per token).  cos/sin are fp32 [max_pos, head_dim/2]; positions int32[tokens].  inverse=1 applies
// the transpose rotation (backward pass).
int mesh_rope(void* x, const int* positions, const float* cos_t, const float* sin_t, int tokens, int heads,
              int head_dim, long long ld, int inverse, void* stream);

// out[0] = sum(a[i] * b[i]) for bf16 a, b of n elements (fp32 accumulation, one launch, result independent of block
// timing).  Scratch: `partials` fp32[mesh_dot_sum_blocks()] and a zero-initialised `ticket` word, left at zero; calls
// that share scratch must be ordered on one stream.
int mesh_dot_sum_bf16(const void* a, const void* b, long long n, float* out, float* partials, unsigned int* ticket,
                      void* stream);
int mesh_dot_sum_blocks(void);

// Cross-entropy over a vocabulary shard logits[rows, cols] (bf16, row stride ld): per-row maximum, sum of exponentials
// relative to that maximum, and the target's logit when the target (int64 global class id) lies in
// [vocab_start, vocab_start + cols) and is not ignore_index (else 0).
int mesh_ce_stats_bf16(const void* logits, long long ld, int rows, int cols, const long long* targets, long long vocab_start,
                       long long ignore_index, float* row_max, float* row_sum, float* target_logit, void* stream);
// d = (exp(logits - gmax) / gsum - onehot(target)) * gscale, bf16 (may be the logits buffer itself); gmax, gsum: the
// whole-vocabulary statistics; gscale[rows]: upstream gradient, 0 for ignored rows.
int mesh_ce_grad_bf16(const void* logits, long long ld, void* dlogits, long long ldd, int rows, int cols,
                      const long long* targets, long long vocab_start, const float* gmax, const float* gsum,
                      const float* gscale, void* stream);

// softmax over experts then top-k (k <= 8, experts <= 256).  bias (fp32[experts], may be NULL) is added
// to the logits before the softmax.  weights fp32[tokens,k] (renormalised over the k when renorm),
// indices int32[tokens,k]; ties go to the lower expert index.
int mesh_router_topk(const void* logits, int logits_is_fp32, const float* bias, float* weights, int* indices,
                     int tokens, int experts, int k, int renorm, void* stream);

// Flash attention forward (tcgen05).  q/k/v are 2-D row-major views: row = batch * T + token, head h of q at
// columns [q_col0 + h*head_dim, ...) of a matrix with `q_cols` columns and leading dimension ldq (same for k, v with
// KV heads).  Logical positions for the masks: q_pos = q_off + i*q_stride, k_pos = k_off + j*k_stride.
typedef struct MeshFlashArgs {
  const void* q; const void* k; const void* v; void* out; float* lse;
  long long ldq, ldk, ldv, ldo;
  int q_cols, k_cols, v_cols, q_col0, k_col0, v_col0;
  int B, H, Hkv, Tq, Tk, head_dim;
  int causal, window;
  int q_off, q_stride, k_off, k_stride;
  float scale;
  void* status;
  // dropout of the attention probabilities (0: none), drawn as csrc/device/philox.cuh describes: a function of the
  // logical coordinates, so every shard of a sequence drops what one device would
  float dropout_p;
  unsigned long long seed;
  unsigned int site, execution;
  int head_off, heads_total;     // logical head of local head h is head_off + h of heads_total (0: H); head-sharded layers
} MeshFlashArgs;
int mesh_flash_attention_fwd(const MeshFlashArgs* a, void* stream);

// Backward of the same attention: `fwd` describes q, k, v, the masks and `lse` exactly as in the forward call.
// `dq` is a zero-initialised fp32 accumulator [B*Tq, ld_dq]; dk/dv are bf16 outputs [B*Tk, ld_dkv], unless the
// fp32 accumulators dk_acc/dv_acc are given, which are added to instead (a KV chunk visited by several ranks).
typedef struct MeshFlashBwdArgs {
  MeshFlashArgs fwd;
  const void* dout; const float* delta;
  long long ld_do; int do_cols, do_col0;
  float* dq; void* dk; void* dv; float* dk_acc; float* dv_acc;
  long long ld_dq, ld_dkv;
} MeshFlashBwdArgs;
int mesh_flash_attention_bwd(const MeshFlashBwdArgs* a, void* stream);

#ifdef __cplusplus
}
#endif
