// Flash attention backward on tcgen05 / TMEM.
//
// One CTA owns one block of 128 keys of one KV head and walks the query blocks (of every query head of
// the group) that can see it.  Per query block, five tensor-core products run from the same shared-memory
// tiles, with no transposed copies — a transposed operand is the same bytes read through an MN-major
// descriptor:
//     S  = Q K^T            dP = dO V^T                      (accumulators in TMEM, one row per thread)
//     P  = exp(S*scale - L)  dS = P o (dP - Delta) * scale   (threads, written to shared memory as bf16)
//     dV += P^T dO          dK += dS^T Q                     (accumulate in TMEM across all query blocks)
//     dQ  = dS K            -> added to a float accumulator in global memory (several key blocks add to it)
// L is the log-sum-exp of the forward pass and Delta = rowsum(dO o O).  With the global L of a ring
// attention the same kernel yields each KV chunk's contribution (chunks are visited one at a time by
// the caller), masks are evaluated on logical positions exactly as in the forward kernel.
// Reference semantics: the backward of the blockwise attention of compiler/mesh_compiler/operations.py:7081-7166.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <cstring>
#include "ops_api.h"
#include "../device/philox.cuh"
#include "../device/ptx.cuh"
#include "../runtime/host_common.h"

namespace mesh {
namespace fab {

constexpr int BQ = 128, BKV = 128;
constexpr int SM_THREADS = 256;       // 8 softmax warps: threads r and r + 128 share row r, half of the columns each
constexpr int THREADS = 288;          // + 1 copy/MMA warp

struct Params {
  CUtensorMap tmQ, tmK, tmV, tmdO;           // boxes {64, 128}
  const float* lse; const float* delta;      // [B, H, Tq]
  float* dq;                                 // fp32 [B*Tq, H*hd], zeroed by the caller
  __nv_bfloat16* dk; __nv_bfloat16* dv;      // [B*Tk, Hkv*hd] (bf16, written) ...
  float* dk_acc; float* dv_acc;              // ... or fp32 accumulators that are added to (ring attention)
  long long ld_dq, ld_dkv;
  int B, H, Hkv, Tq, Tk;
  int q_col0, k_col0, v_col0, do_col0;
  int causal, window, q_off, q_stride, k_off, k_stride;
  float scale, scale_log2;
  Status* status;
  DropoutKey drop;
  int head_off, heads_total;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
  tmem_ld_32x32(addr, r);
  tmem_ld_wait();
}

// bf16 row piece (32 columns) into the [kv/64][128 rows][128 B] swizzled tile
__device__ __forceinline__ void store_row32(uint32_t tile, int row, int c, const uint32_t (&w)[16]) {
  const uint32_t row_base = tile + (c / 2) * (128 * 128) + row * 128;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t chunk = ((c & 1) * 4 + j) ^ (row & 7);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + (chunk << 4)), "r"(w[4 * j]), "r"(w[4 * j + 1]),
                 "r"(w[4 * j + 2]), "r"(w[4 * j + 3]) : "memory");
  }
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 1) flash_bwd_kernel(const __grid_constant__ Params p) {
  constexpr int KC = HD / 64;
  constexpr int TILE = 128 * HD * 2;          // Q, dO, K, V tiles
  constexpr int PT = 128 * 128 * 2;           // P, dS tiles
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = sK + TILE, sQ = sV + TILE, sdO = sQ + TILE, sP = sdO + TILE, sdS = sP + PT;
  const uint32_t bars = sdS + PT;
  auto bar = [&](int i) { return bars + 8u * i; };
  constexpr int KV_FULL = 0, Q_FULL = 1, SDP_FULL = 2, PDS_FULL = 3, MMA2_DONE = 4, DQ_READ = 5;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + 4 * TILE + 2 * PT + 8 * 8);
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // TMEM columns: S / dQ at 0, dP at 128, dV at 256, dK at 256 + HD
  constexpr int C_S = 0, C_DP = 128, C_DV = 256, C_DK = 256 + HD;
  static_assert(C_DK + HD <= 512, "head_dim up to 128 fits tensor memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  const int k0 = jb * BKV;

  // query blocks that can see this key block
  const int kpos_lo = p.k_off + k0 * p.k_stride;
  const int kpos_hi = p.k_off + (min(k0 + BKV, p.Tk) - 1) * p.k_stride;
  int i_lo = 0, i_hi = (p.Tq + BQ - 1) / BQ;
  if (p.causal) {
    // queries with q_pos >= kpos_lo
    const int qmin = kpos_lo - p.q_off <= 0 ? 0 : (kpos_lo - p.q_off + p.q_stride - 1) / p.q_stride;
    i_lo = max(i_lo, qmin / BQ);
  }
  if (p.window > 0) {
    // queries with q_pos < kpos_hi + window
    const int qmax_pos = kpos_hi + p.window - 1;
    const int qmax = qmax_pos - p.q_off < 0 ? -1 : (qmax_pos - p.q_off) / p.q_stride;
    i_hi = min(i_hi, qmax / BQ + 1);
    if (qmax < 0) i_hi = 0;
  }
  const int n_q = max(0, i_hi - i_lo);
  const int n_iter = n_q * group;

  if (threadIdx.x == 0) {
    mbar_init(bar(KV_FULL), 1);
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(SDP_FULL), 1);
    mbar_init(bar(PDS_FULL), SM_THREADS);
    mbar_init(bar(MMA2_DONE), 1);
    mbar_init(bar(DQ_READ), SM_THREADS);
    *abort_smem = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc<1>(smem_u32(tmem_slot), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 8) {
    if (lane == 0 && n_iter > 0) {
      const int k_row = b * p.Tk + k0;
      mbar_expect_tx(bar(KV_FULL), 2 * TILE);
      for (int kc = 0; kc < KC; ++kc) {
        tma_load_2d(sK + kc * (128 * 128), &p.tmK, bar(KV_FULL), p.k_col0 + hk * HD + kc * 64, k_row);
        tma_load_2d(sV + kc * (128 * 128), &p.tmV, bar(KV_FULL), p.v_col0 + hk * HD + kc * 64, k_row);
      }
      constexpr uint32_t id_s = umma_idesc_bf16(128, 128, 0, 0);        // Q K^T and dO V^T: both K-major over head_dim
      constexpr uint32_t id_t = umma_idesc_bf16(128, HD, 1, 1);         // P^T dO and dS^T Q: A and B MN-major, K = queries
      constexpr uint32_t id_q = umma_idesc_bf16(128, HD, 0, 1);         // dS K: A K-major over keys, B = K MN-major
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_smem, p.status, SITE_SMEM_FULL);
      for (int it = 0; ok && it < n_iter; ++it) {
        const int g = it / n_q, i = i_lo + it % n_q;
        const int h = hk * group + g;
        // Q and dO of this block may be overwritten once the second group of products of the previous iteration is done
        if (it > 0) {
          ok = mbar_wait(bar(MMA2_DONE), (it - 1) & 1, abort_smem, p.status, SITE_SMEM_EMPTY);
          if (!ok) break;
        }
        const int q_row = b * p.Tq + i * BQ;
        mbar_expect_tx(bar(Q_FULL), 2 * TILE);
        for (int kc = 0; kc < KC; ++kc) {
          tma_load_2d(sQ + kc * (128 * 128), &p.tmQ, bar(Q_FULL), p.q_col0 + h * HD + kc * 64, q_row);
          tma_load_2d(sdO + kc * (128 * 128), &p.tmdO, bar(Q_FULL), p.do_col0 + h * HD + kc * 64, q_row);
        }
        ok = mbar_wait(bar(Q_FULL), it & 1, abort_smem, p.status, SITE_SMEM_FULL);
        if (!ok) break;
        // the S / dQ columns are free once the threads have read dQ of the previous iteration
        if (it > 0) {
          ok = mbar_wait(bar(DQ_READ), (it - 1) & 1, abort_smem, p.status, SITE_TMEM_EMPTY);
          if (!ok) break;
        }
        tc_fence_after();
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t off = kc * (128 * 128) + k * 32;
            umma_f16<1>(tmem + C_S, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), id_s, (kc | k) ? 1u : 0u);
            umma_f16<1>(tmem + C_DP, umma_smem_desc(sdO + off, 16, 1024), umma_smem_desc(sV + off, 16, 1024), id_s, (kc | k) ? 1u : 0u);
          }
        umma_commit(bar(SDP_FULL));
        // second group: needs P and dS from the threads
        ok = mbar_wait(bar(PDS_FULL), it & 1, abort_smem, p.status, SITE_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k) {
          // transposed reads: MN = keys (groups of 64, one [128 rows][128 B] slab apart), K = the 128 query rows
          const uint64_t a_pt = umma_smem_desc(sP + k * 2048, 128 * 128, 1024);
          const uint64_t a_dst = umma_smem_desc(sdS + k * 2048, 128 * 128, 1024);
          const uint64_t b_do = umma_smem_desc(sdO + k * 2048, 128 * 128, 1024);
          const uint64_t b_q = umma_smem_desc(sQ + k * 2048, 128 * 128, 1024);
          umma_f16<1>(tmem + C_DV, a_pt, b_do, id_t, (it | k) ? 1u : 0u);
          umma_f16<1>(tmem + C_DK, a_dst, b_q, id_t, (it | k) ? 1u : 0u);
          // dQ = dS K: A = dS as written (K-major over the keys), B = K tile read MN-major
          const uint64_t a_ds = umma_smem_desc(sdS + (k / 4) * (128 * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t b_k = umma_smem_desc(sK + k * 2048, 128 * 128, 1024);
          umma_f16<1>(tmem + C_S, a_ds, b_k, id_q, k ? 1u : 0u);
        }
        umma_commit(bar(MMA2_DONE));
      }
    }
  } else {
    const int row = threadIdx.x & 127;                // == TMEM lane; query row in the loop, key row at the end
    const int half = threadIdx.x >> 7;                // which 64 key columns of S / dP, which half of the dQ/dK/dV columns
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    for (int it = 0; ok && it < n_iter; ++it) {
      const int g = it / n_q, i = i_lo + it % n_q;
      const int h = hk * group + g;
      const int qi = i * BQ + row;
      const int qpos = p.q_off + qi * p.q_stride;
      const bool qreal = qi < p.Tq;
      const float L = qreal ? p.lse[((long long)b * p.H + h) * p.Tq + qi] : -CUDART_INF_F;
      const float dl = qreal ? p.delta[((long long)b * p.H + h) * p.Tq + qi] : 0.f;
      // rows with no visible key at all (L = -inf) and rows past the end get P = 0 through an infinite offset
      const float negL2 = (L == -CUDART_INF_F) ? -CUDART_INF_F : -L * 1.4426950408889634f;
      // does a mask or the end of the keys / queries cut into this (query block, key block) pair?
      const int qpos_lo = p.q_off + i * BQ * p.q_stride, qpos_hi = p.q_off + (i * BQ + BQ - 1) * p.q_stride;
      const bool masked = (k0 + BKV > p.Tk) || (p.causal && kpos_hi > qpos_lo) ||
                          (p.window > 0 && kpos_lo <= qpos_hi - p.window);
      ok = mbar_wait(bar(SDP_FULL), it & 1, abort_smem, p.status, SITE_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // P and dS may be overwritten: SDP_FULL of this iteration was issued after the MMA warp had waited for the
      // previous iteration's second group of products, which read them
      DropoutRow dr;
      if (p.drop.p > 0.f) dr.begin((uint32_t)(b * p.heads_total + p.head_off + h), (uint32_t)qpos);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(lane_addr + C_S + half * 64 + c * 32, rs);
        tmem_ld_32x32(lane_addr + C_DP + half * 64 + c * 32, rp);
        tmem_ld_wait();
        uint32_t wp[16], wd[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            float pr = ex2_approx(fmaf(__uint_as_float(rs[e + u]), p.scale_log2, negL2));
            if (masked) {
              const int kj = k0 + half * 64 + c * 32 + e + u;
              const int kpos = p.k_off + kj * p.k_stride;
              const bool vis = kj < p.Tk && (!p.causal || kpos <= qpos) && (p.window <= 0 || kpos > qpos - p.window);
              pr = vis ? pr : 0.f;
            }
            // dropout: dV sees the dropped, rescaled probabilities; dP comes back through the same mask
            float m = 1.f;
            if (p.drop.p > 0.f) {
              const uint32_t kpos = (uint32_t)(p.k_off + (k0 + half * 64 + c * 32 + e + u) * p.k_stride);
              m = dr.keep(p.drop, kpos) ? p.drop.inv_keep : 0.f;
            }
            pv[u] = pr * m;
            dv[u] = pr * (__uint_as_float(rp[e + u]) * m - dl) * p.scale;
          }
          __nv_bfloat162 hp = __floats2bfloat162_rn(pv[0], pv[1]);
          __nv_bfloat162 hd2 = __floats2bfloat162_rn(dv[0], dv[1]);
          wp[e / 2] = *reinterpret_cast<uint32_t*>(&hp);
          wd[e / 2] = *reinterpret_cast<uint32_t*>(&hd2);
        }
        store_row32(sP, row, half * 2 + c, wp);
        store_row32(sdS, row, half * 2 + c, wd);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar(PDS_FULL));
      // dQ tile of this (query block, key block): add this thread's half of the row into the float accumulator
      ok = mbar_wait(bar(MMA2_DONE), it & 1, abort_smem, p.status, SITE_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float* dq = p.dq + ((long long)b * p.Tq + qi) * p.ld_dq + h * HD + half * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + C_S + half * (HD / 2) + c * 32, r);
        if (qreal) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + c * 32 + e), "f"(__uint_as_float(r[e])),
                         "f"(__uint_as_float(r[e + 1])), "f"(__uint_as_float(r[e + 2])), "f"(__uint_as_float(r[e + 3])) : "memory");
        }
      }
      tc_fence_before();
      mbar_arrive(bar(DQ_READ));
    }
    // ---- dK, dV of this key block (thread = key row, half of the head dimension)
    ok = __all_sync(0xffffffffu, ok);
    if (ok && n_iter > 0) {
      const int kj = k0 + row;
      const long long off = ((long long)b * p.Tk + kj) * p.ld_dkv + hk * HD + half * (HD / 2);
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const int col0 = (which ? C_DK : C_DV) + half * (HD / 2);
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + col0 + c * 32, r);
          if (kj >= p.Tk) continue;
          if (p.dk_acc) {
            float* dst = (which ? p.dk_acc : p.dv_acc) + off + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              float4 cur = *reinterpret_cast<float4*>(dst + e);
              cur.x += __uint_as_float(r[e]); cur.y += __uint_as_float(r[e + 1]);
              cur.z += __uint_as_float(r[e + 2]); cur.w += __uint_as_float(r[e + 3]);
              *reinterpret_cast<float4*>(dst + e) = cur;
            }
          } else {
            __nv_bfloat16* dst = (which ? p.dk : p.dv) + off + c * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                hb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
              *reinterpret_cast<uint4*>(dst + j * 8) = o;
            }
          }
        }
      }
    } else if (n_iter == 0 && !p.dk_acc && half == 0) {
      // nothing sees this key block: its gradients are zero
      const int kj = k0 + row;
      if (kj < p.Tk) {
        const long long off = ((long long)b * p.Tk + kj) * p.ld_dkv + hk * HD;
        for (int e = 0; e < HD; e += 8) {
          *reinterpret_cast<uint4*>(p.dk + off + e) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(p.dv + off + e) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc<1>(tmem, 512);
  }
}

static bool map2d(CUtensorMap* tm, const void* base, uint64_t cols, uint64_t rows, uint64_t ld) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  return encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int HD>
static int launch(const MeshFlashBwdArgs* a, cudaStream_t stream) {
  constexpr int SMEM = 4 * 128 * HD * 2 + 2 * 128 * 128 * 2 + 1024 + 256;
  Params p;
  memset(&p, 0, sizeof(p));
  const MeshFlashArgs& f = a->fwd;
  if (!map2d(&p.tmQ, f.q, (uint64_t)f.q_cols, (uint64_t)f.B * f.Tq, (uint64_t)f.ldq)) return last_error_code();
  if (!map2d(&p.tmK, f.k, (uint64_t)f.k_cols, (uint64_t)f.B * f.Tk, (uint64_t)f.ldk)) return last_error_code();
  if (!map2d(&p.tmV, f.v, (uint64_t)f.v_cols, (uint64_t)f.B * f.Tk, (uint64_t)f.ldv)) return last_error_code();
  if (!map2d(&p.tmdO, a->dout, (uint64_t)a->do_cols, (uint64_t)f.B * f.Tq, (uint64_t)a->ld_do)) return last_error_code();
  p.lse = f.lse; p.delta = a->delta; p.dq = a->dq; p.dk = (__nv_bfloat16*)a->dk; p.dv = (__nv_bfloat16*)a->dv;
  p.dk_acc = a->dk_acc; p.dv_acc = a->dv_acc;
  p.ld_dq = a->ld_dq; p.ld_dkv = a->ld_dkv;
  p.B = f.B; p.H = f.H; p.Hkv = f.Hkv; p.Tq = f.Tq; p.Tk = f.Tk;
  p.q_col0 = f.q_col0; p.k_col0 = f.k_col0; p.v_col0 = f.v_col0; p.do_col0 = a->do_col0;
  p.causal = f.causal; p.window = f.window;
  p.q_off = f.q_off; p.q_stride = f.q_stride > 0 ? f.q_stride : 1; p.k_off = f.k_off; p.k_stride = f.k_stride > 0 ? f.k_stride : 1;
  p.scale = f.scale; p.scale_log2 = f.scale * 1.4426950408889634f;
  p.status = (Status*)f.status;
  p.drop.p = f.dropout_p > 0.f ? f.dropout_p : 0.f;
  p.drop.inv_keep = p.drop.p > 0.f ? 1.f / (1.f - p.drop.p) : 1.f;
  p.drop.k0 = (uint32_t)(f.seed & 0xffffffffull) ^ (f.execution * 0x9E3779B9u);
  p.drop.k1 = (uint32_t)(f.seed >> 32);
  p.drop.site = f.site;
  p.head_off = f.head_off; p.heads_total = f.heads_total > 0 ? f.heads_total : f.H;
  static bool configured = false;
  if (!configured) {
    MESH_CUDA_OK(cudaFuncSetAttribute(flash_bwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured = true;
  }
  dim3 grid((f.Tk + BKV - 1) / BKV, f.Hkv, f.B);
  flash_bwd_kernel<HD><<<grid, THREADS, SMEM, stream>>>(p);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace fab
}  // namespace mesh

extern "C" int mesh_flash_attention_bwd(const MeshFlashBwdArgs* a, void* stream) {
  using namespace mesh;
  const MeshFlashArgs& f = a->fwd;
  if (f.H % f.Hkv) return set_error(-2, "flash_attention_bwd: query heads must be a multiple of KV heads");
  if (f.lse == nullptr || a->delta == nullptr || a->dq == nullptr) return set_error(-2, "flash_attention_bwd: lse, delta and dq are required");
  if (a->ld_dq % 4 || a->ld_dkv % 8) return set_error(-2, "flash_attention_bwd: gradient leading dimensions are misaligned");
  switch (f.head_dim) {
    case 64: return fab::launch<64>(a, (cudaStream_t)stream);
    case 128: return fab::launch<128>(a, (cudaStream_t)stream);
    default: return set_error(-2, "flash_attention_bwd: head_dim must be 64 or 128 (dK and dV live in tensor memory)");
  }
}
