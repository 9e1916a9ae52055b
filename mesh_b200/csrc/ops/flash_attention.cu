// Flash attention forward on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// One CTA owns 128 query rows of one head.  Warp 8 is the copy/MMA warp: it streams K and V blocks
// through a 2-stage shared-memory ring and issues  S = Q K^T  and  O += P V  as tcgen05.mma with the
// accumulators in tensor memory (S double-buffered, O resident for the whole KV sweep).  Warps 0-7 are
// the softmax warps, two per scheduler so that one hides the other's latencies: threads r and r + 128 share
// query row r, each taking half of the key columns of a block — tcgen05.ld hands a thread its part of the row, so
// the row max costs one exchange through shared memory and the row sum none until the end.  A thread reads its
// scores once and keeps them in registers (the S buffer is handed back to the MMA warp at once), writes P (bf16)
// into shared memory in the swizzled K-major layout the second MMA reads, and rescales its half of the row of O
// in tensor memory only when the running max has moved by more than 2^8 (P stays within bf16/fp32 range; the
// final division by the row sum makes the result independent of the reference point).  Blocks that no mask
// touches take a path without position arithmetic.
// V is consumed MN-major straight from its row-major [kv, head_dim] tile: no transposes anywhere.
//
// Semantics (compiler/mesh_compiler/operations.py:7081-7166): blockwise online softmax with (m, s, acc)
// merging, causal and sliding-window masks on *logical* positions (q_pos = q_off + i*q_stride,
// k_pos = k_off + j*k_stride, which covers striped context-parallel layouts, :7044-7069), GQA by mapping
// query head h to KV head h / group (:7072-7078); the log-sum-exp is returned so partial results over
// KV chunks (ring attention) can be merged.  Fully masked KV blocks are skipped.
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
namespace fa {

constexpr int BQ = 128;
constexpr int SM_THREADS = 256;       // 8 softmax warps
constexpr int THREADS = 288;          // + 1 copy/MMA warp

struct Params {
  CUtensorMap tmQ, tmK, tmV;          // 2-D maps over [rows, cols] views; boxes {64, 128} / {64, BKV}
  __nv_bfloat16* out; long long ldo;  // [B*Tq, H*hd]
  float* lse;                         // [B, H, Tq]
  int B, H, Hkv, Tq, Tk;
  int q_col0, k_col0, v_col0;         // first column of head 0 inside the stored matrices
  int causal, window;
  int q_off, q_stride, k_off, k_stride;
  float scale_log2;                   // softmax scale * log2(e)
  Status* status;
  DropoutKey drop;
  int head_off, heads_total;                    // drop.p == 0: no dropout
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
struct Cfg {
  static constexpr int BKV = HD <= 128 ? 128 : 64;
  static constexpr int KC = HD / 64;                    // 64-wide chunks along head_dim
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int SMEM = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 + 256 + 2 * 2 * 128 * 4;
  static constexpr int S_COLS = BKV;                    // per S buffer
  static constexpr int O_COL0 = 256;                    // S0 at 0, S1 at 128, O from 256
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 1) flash_fwd_kernel(const __grid_constant__ Params p) {
  using C = Cfg<HD>;
  constexpr int BKV = C::BKV, KC = C::KC;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;
  const uint32_t sK0 = sQ + C::Q_BYTES;                 // 2 stages of K then 2 of V
  const uint32_t sV0 = sK0 + 2 * C::KV_BYTES;
  const uint32_t sP = sV0 + 2 * C::KV_BYTES;
  const uint32_t bars = sP + C::P_BYTES;
  // barriers: q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, o_done
  auto bar = [&](int i) { return bars + 8u * i; };
  constexpr int Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 3, S_FULL = 5, S_EMPTY = 7, P_FULL = 9, O_DONE = 10;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + C::Q_BYTES + 4 * C::KV_BYTES + C::P_BYTES + 8 * 12);
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(tmem_slot + 4);      // [2 parities][2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * BQ;

  // KV block range visible to this query block (logical positions)
  const int qpos_lo = p.q_off + q0 * p.q_stride;
  const int qpos_hi = p.q_off + (min(q0 + BQ, p.Tq) - 1) * p.q_stride;
  int j_lo = 0, j_hi = (p.Tk + BKV - 1) / BKV;          // [j_lo, j_hi)
  if (p.causal) {
    // keys with k_pos <= qpos_hi:  j*k_stride + k_off <= qpos_hi
    const int kmax = (qpos_hi - p.k_off) >= 0 ? (qpos_hi - p.k_off) / p.k_stride : -1;
    j_hi = min(j_hi, kmax / BKV + 1);
    if (kmax < 0) j_hi = 0;
  }
  if (p.window > 0) {
    const int kmin_pos = qpos_lo - p.window + 1;          // smallest visible key position
    const int kmin = kmin_pos - p.k_off <= 0 ? 0 : (kmin_pos - p.k_off + p.k_stride - 1) / p.k_stride;
    j_lo = max(j_lo, kmin / BKV);
  }
  const int n_blocks = max(0, j_hi - j_lo);

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(KV_FULL + s), 1);
      mbar_init(bar(KV_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(S_EMPTY + s), SM_THREADS);
    }
    mbar_init(bar(P_FULL), SM_THREADS);
    mbar_init(bar(O_DONE), 1);
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
    if (lane == 0 && n_blocks > 0) {
      // ------------------------------------------------------------------ copy + MMA issue
      const int q_row = b * p.Tq + q0;
      mbar_expect_tx(bar(Q_FULL), C::Q_BYTES);
      for (int kc = 0; kc < KC; ++kc)
        tma_load_2d(sQ + kc * (BQ * 128), &p.tmQ, bar(Q_FULL), p.q_col0 + h * HD + kc * 64, q_row);
      auto load_kv = [&](int it) {
        const int s = it & 1;
        const int k_row = b * p.Tk + (j_lo + it) * BKV;
        mbar_expect_tx(bar(KV_FULL + s), 2 * C::KV_BYTES);
        for (int kc = 0; kc < KC; ++kc) {
          tma_load_2d(sK0 + s * C::KV_BYTES + kc * (BKV * 128), &p.tmK, bar(KV_FULL + s), p.k_col0 + hk * HD + kc * 64, k_row);
          tma_load_2d(sV0 + s * C::KV_BYTES + kc * (BKV * 128), &p.tmV, bar(KV_FULL + s), p.v_col0 + hk * HD + kc * 64, k_row);
        }
      };
      constexpr uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BQ, HD, 0, 1);          // B = V is MN-major
      auto issue_s = [&](int it) {
        const int s = it & 1;
        const uint32_t d = tmem + s * 128;
        const uint32_t k_base = sK0 + s * C::KV_BYTES;
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16<1>(d, umma_smem_desc(sQ + kc * (BQ * 128) + k * 32, 16, 1024),
                        umma_smem_desc(k_base + kc * (BKV * 128) + k * 32, 16, 1024), idesc_s, (kc | k) ? 1u : 0u);
        umma_commit(bar(S_FULL + s));
      };
      bool ok = true;
      load_kv(0);
      if (n_blocks > 1) load_kv(1);
      ok = mbar_wait(bar(Q_FULL), 0, abort_smem, p.status, SITE_SMEM_FULL);
      if (ok) ok = mbar_wait(bar(KV_FULL + 0), 0, abort_smem, p.status, SITE_SMEM_FULL);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int it = 0; ok && it < n_blocks; ++it) {
        const int s = it & 1;
        // next S while the softmax warps work on this one
        if (it + 1 < n_blocks) {
          ok = mbar_wait(bar(KV_FULL + (s ^ 1)), ((it + 1) >> 1) & 1, abort_smem, p.status, SITE_SMEM_FULL);
          if (!ok) break;
          if (it + 1 >= 2) {     // the S buffer must have been read out by the softmax warps (iteration it-1)
            ok = mbar_wait(bar(S_EMPTY + (s ^ 1)), ((it - 1) >> 1) & 1, abort_smem, p.status, SITE_TMEM_EMPTY);
            if (!ok) break;
          }
          tc_fence_after();
          issue_s(it + 1);
        }
        // O += P V once the softmax warps have written P (and rescaled O)
        ok = mbar_wait(bar(P_FULL), it & 1, abort_smem, p.status, SITE_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_base = sV0 + s * C::KV_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // A = P: K-major over kv, 64-wide chunks [kv/64][128 rows][128 B]; B = V: MN-major, groups of 64 head dims
          const uint64_t da = umma_smem_desc(sP + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t db = umma_smem_desc(v_base + k * 2048, BKV * 128, 1024);
          umma_f16<1>(tmem + C::O_COL0, da, db, idesc_o, (it | k) ? 1u : 0u);
        }
        umma_commit(bar(KV_EMPTY + s));            // K/V stage and P are free once these MMAs are done
        umma_commit(bar(O_DONE));
        if (it + 2 < n_blocks) {
          ok = mbar_wait(bar(KV_EMPTY + s), (it >> 1) & 1, abort_smem, p.status, SITE_SMEM_EMPTY);
          if (!ok) break;
          load_kv(it + 2);
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- softmax warps
    constexpr int HALF = BKV / 2;                     // key columns of a block per thread
    constexpr int NCH = HALF / 32;                    // 32-column TMEM loads per thread and block
    const int row = threadIdx.x & 127;                // == TMEM lane
    const int half = threadIdx.x >> 7;                // which half of the key columns (and of the O columns)
    const int qi = q0 + row;
    const int qpos = p.q_off + qi * p.q_stride;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float thr = 8.f / p.scale_log2;             // the reference point moves when the max grew by > 2^8
    float m_ref = -CUDART_INF_F, l = 0.f;             // reference point (identical in both threads of a row), own sum
    bool ok = true;
    // Every softmax warp runs all n_blocks iterations and meets the others at the named barrier in each, also after
    // a wait has run out (ok == false, warp-uniform): it then skips the work, so the barrier counts stay equal.
    for (int it = 0; it < n_blocks; ++it) {
      const int s = it & 1;
      if (ok) {
        ok = mbar_wait(bar(S_FULL + s), (it >> 1) & 1, abort_smem, p.status, SITE_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      const int kbase = (j_lo + it) * BKV;
      // does any mask or the end of the keys cut into this block (for some row of the tile)?
      const int kpos_lo = p.k_off + kbase * p.k_stride, kpos_hi = p.k_off + (kbase + BKV - 1) * p.k_stride;
      const bool masked = (kbase + BKV > p.Tk) || (p.causal && kpos_hi > qpos_lo) ||
                          (p.window > 0 && kpos_lo <= qpos_hi - p.window);
      // this thread's scores, read once
      uint32_t r[NCH][32];
      float mx = -CUDART_INF_F;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld_32x32(lane_addr + s * 128 + half * HALF + c * 32, r[c]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar(S_EMPTY + s));                // the MMA warp may overwrite this S buffer
        if (masked) {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kj = kbase + half * HALF + c * 32 + i;
              const int kpos = p.k_off + kj * p.k_stride;
              const bool vis = kj < p.Tk && (!p.causal || kpos <= qpos) && (p.window <= 0 || kpos > qpos - p.window);
              if (!vis) r[c][i] = 0xff800000u;        // -inf: exp2 gives an exact zero
              mx = fmaxf(mx, __uint_as_float(r[c][i]));
            }
        } else {
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              mx = fmaxf(mx, fmaxf(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1])));
        }
      }
      // row max = max of the two halves
      float* xm = xchg + (it & 1) * 256;
      xm[half * 128 + row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(SM_THREADS) : "memory");
      mx = fmaxf(mx, xm[(half ^ 1) * 128 + row]);
      if (!ok) continue;
      float alpha = 1.f;
      if (mx > m_ref + thr) {                         // also the first block with a visible key (m_ref = -inf)
        alpha = ex2_approx((m_ref - mx) * p.scale_log2);          // ex2(-inf) = 0
        m_ref = mx;
      }
      const float neg_ms = (m_ref == -CUDART_INF_F) ? 0.f : -m_ref * p.scale_log2;
      // The exponentials are computed into registers first: they need nothing from the previous block's P V
      // product, which the tensor core is still running.
      float sum = 0.f;
      uint32_t w[NCH][16];
      DropoutRow dr;
      if (p.drop.p > 0.f) dr.begin((uint32_t)(b * p.heads_total + p.head_off + h), (uint32_t)qpos);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(r[c][i]), p.scale_log2, neg_ms));
          float p1 = ex2_approx(fmaf(__uint_as_float(r[c][i + 1]), p.scale_log2, neg_ms));
          sum += p0 + p1;                         // the row sum is that of the undropped probabilities
          if (p.drop.p > 0.f) {
            const uint32_t kpos = (uint32_t)(p.k_off + (kbase + half * HALF + c * 32 + i) * p.k_stride);
            p0 = dr.keep(p.drop, kpos) ? p0 * p.drop.inv_keep : 0.f;
            p1 = dr.keep(p.drop, kpos + (uint32_t)p.k_stride) ? p1 * p.drop.inv_keep : 0.f;
          }
          __nv_bfloat162 hb = __floats2bfloat162_rn(p0, p1);
          w[c][i / 2] = *reinterpret_cast<uint32_t*>(&hb);
        }
      }
      // P of the previous block must have been consumed before it is overwritten, and O must be final
      if (it > 0) {
        ok = mbar_wait(bar(O_DONE), (it - 1) & 1, abort_smem, p.status, SITE_TMEM_EMPTY);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) continue;
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        // 32 columns = 64 bytes = 4 pieces of 16 B inside the 128-byte swizzled row of their 64-column chunk
        const int col = half * HALF + c * 32;
        const uint32_t row_base = sP + (col / 64) * (BQ * 128) + row * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t chunk = (((col % 64) / 32) * 4 + j) ^ (row & 7);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + (chunk << 4)), "r"(w[c][4 * j]),
                       "r"(w[c][4 * j + 1]), "r"(w[c][4 * j + 2]), "r"(w[c][4 * j + 3]) : "memory");
        }
      }
      l = l * alpha + sum;
      // rescale this thread's half of the row of O (never for the first block: the first PV MMA overwrites O).
      // tcgen05.ld / .st are warp-collective: the decision must be the same for all 32 rows of a warp
      if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < HD / 64; ++c) {
          uint32_t o[32];
          const uint32_t addr = lane_addr + C::O_COL0 + half * (HD / 2) + c * 32;
          tmem_ld_32x32(addr, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
              "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
              ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]),
                "r"(o[6]), "r"(o[7]), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]),
                "r"(o[15]), "r"(o[16]), "r"(o[17]), "r"(o[18]), "r"(o[19]), "r"(o[20]), "r"(o[21]), "r"(o[22]), "r"(o[23]),
                "r"(o[24]), "r"(o[25]), "r"(o[26]), "r"(o[27]), "r"(o[28]), "r"(o[29]), "r"(o[30]), "r"(o[31])
              : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // P (generic-proxy stores) must be visible to the tensor core's async proxy
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar(P_FULL));
    }
    // ---- epilogue: O / l -> bf16 rows, log-sum-exp
    if (ok && n_blocks > 0) {
      ok = mbar_wait(bar(O_DONE), (n_blocks - 1) & 1, abort_smem, p.status, SITE_TMEM_FULL);
      tc_fence_after();
    }
    ok = __all_sync(0xffffffffu, ok);      // the TMEM loads below are warp-collective: every lane takes part,
    // the row sum is the sum of the two halves' sums (both are relative to the same reference point)
    float* xl = xchg + (n_blocks & 1) * 256;
    xl[half * 128 + row] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(SM_THREADS) : "memory");
    l += xl[(half ^ 1) * 128 + row];
    if (ok) {                              // only the global stores are predicated on the row being real
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((long long)b * p.Tq + qi) * p.ldo + h * HD + half * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld_32x32(lane_addr + C::O_COL0 + half * (HD / 2) + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q4;
          __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&q4);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            hb[i] = __floats2bfloat162_rn(__uint_as_float(o[8 * j + 2 * i]) * inv, __uint_as_float(o[8 * j + 2 * i + 1]) * inv);
          if (qi < p.Tq) *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = q4;
        }
      }
      if (p.lse && qi < p.Tq && half == 0)
        p.lse[((long long)b * p.H + h) * p.Tq + qi] =
            l > 0.f ? (m_ref * p.scale_log2 + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc<1>(tmem, 512);
  }
}

static bool map2d(CUtensorMap* tm, const void* base, uint64_t cols, uint64_t rows, uint64_t ld, uint32_t box_rows) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t es[2] = {1, 1};
  return encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int HD>
static int launch(const MeshFlashArgs* a, cudaStream_t stream) {
  using C = Cfg<HD>;
  Params p;
  memset(&p, 0, sizeof(p));
  if (!map2d(&p.tmQ, a->q, (uint64_t)a->q_cols, (uint64_t)a->B * a->Tq, (uint64_t)a->ldq, BQ)) return last_error_code();
  if (!map2d(&p.tmK, a->k, (uint64_t)a->k_cols, (uint64_t)a->B * a->Tk, (uint64_t)a->ldk, C::BKV)) return last_error_code();
  if (!map2d(&p.tmV, a->v, (uint64_t)a->v_cols, (uint64_t)a->B * a->Tk, (uint64_t)a->ldv, C::BKV)) return last_error_code();
  p.out = (__nv_bfloat16*)a->out; p.ldo = a->ldo; p.lse = a->lse;
  p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.Tq = a->Tq; p.Tk = a->Tk;
  p.q_col0 = a->q_col0; p.k_col0 = a->k_col0; p.v_col0 = a->v_col0;
  p.causal = a->causal; p.window = a->window;
  p.q_off = a->q_off; p.q_stride = a->q_stride > 0 ? a->q_stride : 1;
  p.k_off = a->k_off; p.k_stride = a->k_stride > 0 ? a->k_stride : 1;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.status = (Status*)a->status;
  p.drop.p = a->dropout_p > 0.f ? a->dropout_p : 0.f;
  p.drop.inv_keep = p.drop.p > 0.f ? 1.f / (1.f - p.drop.p) : 1.f;
  p.drop.k0 = (uint32_t)(a->seed & 0xffffffffull) ^ (a->execution * 0x9E3779B9u);
  p.drop.k1 = (uint32_t)(a->seed >> 32);
  p.drop.site = a->site;
  p.head_off = a->head_off; p.heads_total = a->heads_total > 0 ? a->heads_total : a->H;
  static bool configured = false;
  if (!configured) {
    MESH_CUDA_OK(cudaFuncSetAttribute(flash_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    configured = true;
  }
  dim3 grid((a->Tq + BQ - 1) / BQ, a->H, a->B);
  flash_fwd_kernel<HD><<<grid, THREADS, C::SMEM, stream>>>(p);
  MESH_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace fa
}  // namespace mesh

extern "C" int mesh_flash_attention_fwd(const MeshFlashArgs* a, void* stream) {
  using namespace mesh;
  if (a->H % a->Hkv) return set_error(-2, "flash_attention: query heads must be a multiple of KV heads");
  if (a->ldq % 8 || a->ldk % 8 || a->ldv % 8 || a->ldo % 8 || a->q_col0 % 8 || a->k_col0 % 8 || a->v_col0 % 8)
    return set_error(-2, "flash_attention: leading dimensions and head offsets must be multiples of 8 elements");
  if (a->Tq % 1 || a->B < 1) return set_error(-2, "flash_attention: empty problem");
  if (!(a->dropout_p >= 0.f && a->dropout_p < 1.f)) return set_error(-2, "flash_attention: dropout_p must be in [0, 1)");
  switch (a->head_dim) {
    case 64: return fa::launch<64>(a, (cudaStream_t)stream);
    case 128: return fa::launch<128>(a, (cudaStream_t)stream);
    case 256: return fa::launch<256>(a, (cudaStream_t)stream);
    default: return set_error(-2, "flash_attention: head_dim must be 64, 128 or 256");
  }
}
