// Skinny (batch <= 8) linear layers for token-by-token decoding: y[b, n] = sum_k x[b, k] W[n, k].
//
// Decoding is bound by the bytes of W, so the kernel is organised around streaming W once at full
// HBM rate: a CTA owns 16 rows of W (two groups of 8), its 8 warps split K, each lane pulls 16-byte
// pieces of two rows straight from global memory into mma.sync A fragments (the k order inside a
// 32-wide block is permuted identically for W and x, which a dot product does not notice), the
// batch is the 8-wide N side of m16n8k16, and partial sums meet in shared memory.  Around that
// core sit the fusions that remove the launches between the layers of a decoder block:
//   prologue   RMSNorm of x (recomputed by every CTA: duplicated cheap compute is free,
//              design/collective-goals.md:27-29)
//   weights    bf16, or 4-bit codes with one fp16 scale per 64 k (dequantised in registers with a
//              mask, subtract and multiply per pair; reference: `mesh::fragment` coded weights,
//              rdma/mesh_code.py:9-16, compiler/mesh_compiler/operations.py:6996-7040)
//   epilogue   store | GLU (gate and up rows in one CTA) | QKV + RoPE + KV-cache append |
//              one-shot all-reduce across GPUs + residual add (row-parallel projections of a
//              tensor-parallel block: 8-byte {value, sequence} words stored into every peer and
//              polled locally, so one NVLink crossing per reduction, K2 of the reference's table).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "decode_api.h"
#include "../device/ptx.cuh"
#include "../runtime/host_common.h"
#include <cstdlib>
#include <cstring>

namespace mesh {
namespace decode {

constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int NB = 8;                 // batch columns of the MMA
constexpr int XPAD = 64;              // bytes of padding per x row in shared memory (bank spread)

struct LinArgs {
  const __nv_bfloat16* x; long long ldx; int B, K;
  const __nv_bfloat16* norm_w; float eps, norm_off;   // prologue RMSNorm (norm_w == nullptr: none)
  const void* w; const __half* scales;                // weights [N, K] bf16, or packed 4-bit [N, K/2] + scales [N, K/64]
  int n_groups;                                       // 16-row groups this launch covers
  int mode, act;
  int up_off;                                         // GLU: row offset of the up weights; QKV: unused
  void* out; long long ldo; int out_f32;              // STORE/GLU output [B, N]
  // QKV + RoPE + cache append
  int q_heads, kv_heads, head_dim;                    // local heads; rows = (q_heads + 2 kv_heads) * head_dim
  const int* pos; const float* cos_t; const float* sin_t;
  __nv_bfloat16* q_out;                               // [B, q_heads * head_dim]
  __nv_bfloat16* k_cache; __nv_bfloat16* v_cache;     // [B, kv_heads, max_seq, head_dim]
  int max_seq;
  // all-reduce + residual
  int rank, world;
  uint2* ar_recv[MESH_DEC_MAX_RANKS];                 // ar_recv[d]: rank d's slots [world][N * 8]
  const uint32_t* step_ptr; uint32_t calls_per_step, call_index;   // sequence number = step * calls + index + 1
  const __nv_bfloat16* residual; long long ldr;       // [B, N]
  Status* status;
  int l2_prefetch;
  const uint8_t* next_w; unsigned long long next_bytes;   // weights of the linear layer that follows in the stream
  int xpad;                                           // bytes of padding per x row in shared memory (bank spread)
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8 packed 4-bit codes (nibble order 0,4,1,5,2,6,3,7 = k 0..7) -> four bf16x2 words (c - 8) * s
__device__ __forceinline__ void dequant8(uint32_t p, __nv_bfloat162 s2, __nv_bfloat162 bias2, uint32_t (&o)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t t = ((p >> (4 * i)) & 0x000F000Fu) | 0x43004300u;          // bf16(128 + code) in both halves
    // (128 + c) - 136 is exact in bf16; folding the 136*s into an fma addend would round it first
    __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&t), bias2), s2);
    o[i] = *reinterpret_cast<uint32_t*>(&v);
  }
}

__device__ __forceinline__ float dec_act(float g, int act) {
  if (act == 0) {
    return g / (1.f + __expf(-g));
  } else {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
  }
}

// What the weight loads of the main loop read of a layer's arguments, held in registers: the arguments themselves may
// sit in shared memory (a step kernel), where every barrier would force them to be read again.
struct LinHot {
  const void* w; const __half* scales; int K, mode, up_off, head_dim;
};

// first row of the two 8-row groups a CTA works on
template <class Args>
__device__ __forceinline__ void group_rows(const Args& a, int g, int& rA, int& rB) {
  if (a.mode == MESH_DEC_GLU) {
    rA = g * 8;
    rB = a.up_off + g * 8;
  } else if (a.mode == MESH_DEC_QKV) {
    const int per_head = a.head_dim / 16;               // groups per head: rows i..i+8 and i+hd/2..
    const int h = g / per_head, j = g % per_head;
    rA = h * a.head_dim + j * 8;
    rB = rA + a.head_dim / 2;
  } else {
    rA = g * 16;
    rB = rA + 8;
  }
}

// One pipeline step = one chunk of CH k-values of one 16-row group for this warp's K slice.
// bf16: CH = 32*U (U 16-byte loads per row); 4-bit: CH = 64*U (U pairs of 32-bit words per row).
// Weight formats (template parameter W4): 0 = bf16; 1 = 4-bit codes read as 4-byte words (any K % 512 == 0);
// 2 = 4-bit codes read 16 bytes at a time (a lane takes 32 consecutive k of a 128-wide block: four times the bytes in
// flight per load instruction, which is what a latency-bound stream of quarter-size weights needs); 3 = 8-bit codes,
// 16 bytes = 16 consecutive k per lane.  A dot product does not notice the order of k as long as W and x agree.
template <int W4, int U>
struct Chunk {
  uint4 a[W4 == 1 ? (U + 1) / 2 : U];  // bf16 / wide formats: U x 16 B of row A;  format 1: U x {word0, word1}
  uint4 b[W4 == 1 ? (U + 1) / 2 : U];
  float sa[W4 ? U : 1], sb[W4 ? U : 1];
};

template <int W4, int U> struct ChunkK { static constexpr int value = (W4 == 0 ? 32 : W4 == 1 ? 64 : W4 == 2 ? 128 : 64) * U; };
// byte offset inside an x row of the first k this lane multiplies in a chunk
template <int W4> __device__ __forceinline__ int lane_k(int t4) { return W4 == 2 ? t4 * 32 : (W4 == 3 ? t4 * 16 : t4 * 8); }

// four 8-bit codes -> two bf16x2 words (c - 128) * s, exact until the final rounding to bf16
__device__ __forceinline__ void dequant_b4(uint32_t w, float s, uint32_t& lo, uint32_t& hi) {
  const float k = 8388736.f;                                      // 2^23 + 128
  const float f0 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)) - k) * s;
  const float f1 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)) - k) * s;
  const float f2 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)) - k) * s;
  const float f3 = (__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)) - k) * s;
  __nv_bfloat162 a = __floats2bfloat162_rn(f0, f1), b = __floats2bfloat162_rn(f2, f3);
  lo = *reinterpret_cast<uint32_t*>(&a);
  hi = *reinterpret_cast<uint32_t*>(&b);
}

template <int W4, int U>
__device__ __forceinline__ void load_chunk(const LinHot& a, int grp, int kb, int k_lo, int g8, int t4, Chunk<W4, U>& c) {
  int rA, rB;
  group_rows(a, grp, rA, rB);
  const int K = a.K;
  if constexpr (!W4) {
    const __nv_bfloat16* wA = reinterpret_cast<const __nv_bfloat16*>(a.w) + (long long)(rA + g8) * K + k_lo + kb + t4 * 8;
    const __nv_bfloat16* wB = reinterpret_cast<const __nv_bfloat16*>(a.w) + (long long)(rB + g8) * K + k_lo + kb + t4 * 8;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      c.a[u] = __ldcs(reinterpret_cast<const uint4*>(wA + 32 * u));
      c.b[u] = __ldcs(reinterpret_cast<const uint4*>(wB + 32 * u));
    }
  } else if constexpr (W4 == 2 || W4 == 3) {
    constexpr int KPB = W4 == 2 ? 2 : 1;                  // k values per byte
    constexpr int BLK = W4 == 2 ? 128 : 64;               // k per 16-byte load of a quad of lanes
    const long long row_bytes = K / KPB;
    const uint8_t* wA = reinterpret_cast<const uint8_t*>(a.w) + (long long)(rA + g8) * row_bytes + (k_lo + kb) / KPB + t4 * 16;
    const uint8_t* wB = reinterpret_cast<const uint8_t*>(a.w) + (long long)(rB + g8) * row_bytes + (k_lo + kb) / KPB + t4 * 16;
    const int k_lane = k_lo + kb + lane_k<W4>(t4);
    const __half* sA = a.scales + (long long)(rA + g8) * (K / 64);
    const __half* sB = a.scales + (long long)(rB + g8) * (K / 64);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      c.a[u] = __ldcs(reinterpret_cast<const uint4*>(wA + u * (BLK / KPB)));
      c.b[u] = __ldcs(reinterpret_cast<const uint4*>(wB + u * (BLK / KPB)));
      c.sa[u] = __half2float(sA[(k_lane + u * BLK) >> 6]);
      c.sb[u] = __half2float(sB[(k_lane + u * BLK) >> 6]);
    }
  } else {
    const uint32_t* wA = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.w) + (long long)(rA + g8) * (K / 2)) + ((k_lo + kb) >> 3) + t4;
    const uint32_t* wB = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(a.w) + (long long)(rB + g8) * (K / 2)) + ((k_lo + kb) >> 3) + t4;
    const __half* sA = a.scales + (long long)(rA + g8) * (K / 64) + ((k_lo + kb) >> 6);
    const __half* sB = a.scales + (long long)(rB + g8) * (K / 64) + ((k_lo + kb) >> 6);
    uint32_t* pa = reinterpret_cast<uint32_t*>(c.a);
    uint32_t* pb = reinterpret_cast<uint32_t*>(c.b);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      pa[2 * u] = __ldcs(wA + 8 * u);
      pa[2 * u + 1] = __ldcs(wA + 8 * u + 4);
      pb[2 * u] = __ldcs(wB + 8 * u);
      pb[2 * u + 1] = __ldcs(wB + 8 * u + 4);
      c.sa[u] = __half2float(sA[u]);
      c.sb[u] = __half2float(sB[u]);
    }
  }
}

template <int W4, int U>
__device__ __forceinline__ void mma_chunk(const Chunk<W4, U>& c, const uint8_t* xp, float (&acc)[4]) {
  if constexpr (!W4) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xp + 64 * u);
      mma_bf16(acc, c.a[u].x, c.b[u].x, c.a[u].y, c.b[u].y, xv.x, xv.y);
      mma_bf16(acc, c.a[u].z, c.b[u].z, c.a[u].w, c.b[u].w, xv.z, xv.w);
    }
  } else if constexpr (W4 == 2) {
    const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __nv_bfloat162 sa2 = __floats2bfloat162_rn(c.sa[u], c.sa[u]), sb2 = __floats2bfloat162_rn(c.sb[u], c.sb[u]);
      const uint32_t pa[4] = {c.a[u].x, c.a[u].y, c.a[u].z, c.a[u].w};
      const uint32_t pb[4] = {c.b[u].x, c.b[u].y, c.b[u].z, c.b[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {                       // word j: 8 consecutive k = two MMAs
        uint32_t wa[4], wb[4];
        dequant8(pa[j], sa2, off, wa);
        dequant8(pb[j], sb2, off, wb);
        const uint4 xv = *reinterpret_cast<const uint4*>(xp + 256 * u + 16 * j);
        mma_bf16(acc, wa[0], wb[0], wa[1], wb[1], xv.x, xv.y);
        mma_bf16(acc, wa[2], wb[2], wa[3], wb[3], xv.z, xv.w);
      }
    }
  } else if constexpr (W4 == 3) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t pa[4] = {c.a[u].x, c.a[u].y, c.a[u].z, c.a[u].w};
      const uint32_t pb[4] = {c.b[u].x, c.b[u].y, c.b[u].z, c.b[u].w};
      const uint4 x0 = *reinterpret_cast<const uint4*>(xp + 128 * u);
      const uint4 x1 = *reinterpret_cast<const uint4*>(xp + 128 * u + 16);
      const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {                       // word j: 4 consecutive k = one MMA
        uint32_t al, ah, bl, bh;
        dequant_b4(pa[j], c.sa[u], al, ah);
        dequant_b4(pb[j], c.sb[u], bl, bh);
        mma_bf16(acc, al, bl, ah, bh, xw[2 * j], xw[2 * j + 1]);
      }
    }
  } else {
    const uint32_t* pa = reinterpret_cast<const uint32_t*>(c.a);
    const uint32_t* pb = reinterpret_cast<const uint32_t*>(c.b);
    const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __nv_bfloat162 sa2 = __floats2bfloat162_rn(c.sa[u], c.sa[u]), sb2 = __floats2bfloat162_rn(c.sb[u], c.sb[u]);
      uint32_t wa[4], wb[4];
      dequant8(pa[2 * u], sa2, off, wa);
      dequant8(pb[2 * u], sb2, off, wb);
      uint4 xv = *reinterpret_cast<const uint4*>(xp + 128 * u);
      mma_bf16(acc, wa[0], wb[0], wa[1], wb[1], xv.x, xv.y);
      mma_bf16(acc, wa[2], wb[2], wa[3], wb[3], xv.z, xv.w);
      dequant8(pa[2 * u + 1], sa2, off, wa);
      dequant8(pb[2 * u + 1], sb2, off, wb);
      xv = *reinterpret_cast<const uint4*>(xp + 128 * u + 64);
      mma_bf16(acc, wa[0], wb[0], wa[1], wb[1], xv.x, xv.y);
      mma_bf16(acc, wa[2], wb[2], wa[3], wb[3], xv.z, xv.w);
    }
  }
}

// Barrier among the threads that compute a layer: the whole CTA of a stand-alone launch.
struct BlockSync { __device__ __forceinline__ void operator()() const { __syncthreads(); } };

// The B rows of x -> shared memory, optionally RMS-normalised.  Called by the THREADS computing threads together.
template <class Sync>
__device__ __forceinline__ void stage_x(const LinArgs& a, uint8_t* xs, int xstride, Sync sync) {
  __shared__ float rstd_s[NB];
  const int K = a.K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const int nvec = K >> 3;
    for (int b = warp; b < a.B; b += WARPS) {
      float ss = 0.f;
      for (int v = lane; v < nvec; v += 32) {
        const uint4 q = *reinterpret_cast<const uint4*>(a.x + (long long)b * a.ldx + v * 8);
        *reinterpret_cast<uint4*>(xs + b * xstride + v * 16) = q;
        if (a.norm_w) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
      if (a.norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) rstd_s[b] = rsqrtf(ss / (float)K + a.eps);
      }
    }
    sync();
    if (a.norm_w) {
      for (int idx = threadIdx.x; idx < a.B * nvec; idx += THREADS) {
        const int b = idx / nvec, v = idx % nvec;
        uint4* p = reinterpret_cast<uint4*>(xs + b * xstride + v * 16);
        uint4 q = *p;
        const uint4 wq = *reinterpret_cast<const uint4*>(a.norm_w + v * 8);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq);
        const float r = rstd_s[b];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          float2 w = __bfloat1622float2(wh[i]);
          h[i] = __floats2bfloat162_rn(f.x * r * (w.x + a.norm_off), f.y * r * (w.y + a.norm_off));
        }
        *p = q;
      }
      sync();
    }
  }

}

// K-split reduction of one 16-row group through shared memory, then the layer's epilogue.  c: this thread's partial
// sums (c0,c1 = row g8, batch 2t,2t+1; c2,c3 = row g8+8).  Ends with the computing threads in step.
template <class Sync>
__device__ __forceinline__ void finish_group(const LinArgs& a, int grp, float (&c)[4], float* red, float* fin, Sync sync) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
    int rA, rB;
    group_rows(a, grp, rA, rB);
    // ---- K-split reduction through shared memory: c0,c1 = (row g8, batch 2t,2t+1); c2,c3 = row g8+8
    float* my = red + warp * 16 * NB;
    my[g8 * NB + 2 * t4] = c[0];
    my[g8 * NB + 2 * t4 + 1] = c[1];
    my[(g8 + 8) * NB + 2 * t4] = c[2];
    my[(g8 + 8) * NB + 2 * t4 + 1] = c[3];
    sync();
    if (threadIdx.x < 16 * NB) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += red[w * 16 * NB + threadIdx.x];
      fin[threadIdx.x] = s;
    }
    sync();
    // ---- epilogue: thread e = (row r of 16, batch n)
    if (threadIdx.x < 16 * NB) {
      const int r = threadIdx.x / NB, n = threadIdx.x % NB;
      const float val = fin[threadIdx.x];
      const int row = (r < 8) ? rA + r : rB + (r - 8);
      if (a.mode == MESH_DEC_STORE) {
        if (n < a.B) {
          float val = fin[threadIdx.x];
          if (a.residual) val += __bfloat162float(a.residual[(long long)n * a.ldr + row]);
          if (a.out_f32) reinterpret_cast<float*>(a.out)[(long long)n * a.ldo + row] = val;
          else reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)n * a.ldo + row] = __float2bfloat16_rn(val);
        }
      } else if (a.mode == MESH_DEC_GLU) {
        if (r < 8 && n < a.B) {
          const float u = fin[(r + 8) * NB + n];
          reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)n * a.ldo + row] = __float2bfloat16_rn(dec_act(val, a.act) * u);
        }
      } else if (a.mode == MESH_DEC_QKV) {
        if (r < 8 && n < a.B) {
          const int hd = a.head_dim, half = hd / 2;
          const int h = row / hd, i = row % hd;            // i < half
          const float lo = val, hi = fin[(r + 8) * NB + n];
          const int p = a.pos[n];
          float o_lo = lo, o_hi = hi;
          if (h < a.q_heads + a.kv_heads) {                  // q and k heads are rotated
            const float cs = a.cos_t[(long long)p * half + i], sn = a.sin_t[(long long)p * half + i];
            o_lo = lo * cs - hi * sn;
            o_hi = hi * cs + lo * sn;
          }
          __nv_bfloat16* dst;
          if (h < a.q_heads) {
            dst = a.q_out + (long long)n * a.q_heads * hd + h * hd;
          } else if (h < a.q_heads + a.kv_heads) {
            dst = a.k_cache + (((long long)n * a.kv_heads + (h - a.q_heads)) * a.max_seq + p) * hd;
          } else {
            dst = a.v_cache + (((long long)n * a.kv_heads + (h - a.q_heads - a.kv_heads)) * a.max_seq + p) * hd;
          }
          dst[i] = __float2bfloat16_rn(o_lo);
          dst[i + half] = __float2bfloat16_rn(o_hi);
        }
      } else {   // MESH_DEC_ALLREDUCE: one-shot sum over ranks of this row group, plus the residual
        if (n < a.B) {
          // the two halves of the slot array alternate call by call, so a fast peer's next
          // reduction never lands on words a slow rank has not read yet
          const uint32_t ar_seq = (a.step_ptr ? *a.step_ptr : 0u) * a.calls_per_step + a.call_index + 1u;
          const long long per_src = (long long)a.n_groups * 16 * NB;
          const long long slot = (long long)(ar_seq & 1u) * a.world * per_src + (long long)row * NB + n;
          const uint2 word = make_uint2(__float_as_uint(val), ar_seq);
          for (int d = 0; d < a.world; ++d) {
            uint2* p = a.ar_recv[d] + (long long)a.rank * per_src + slot;
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word.x), "r"(word.y) : "memory");
          }
          float sum = 0.f;
          bool ok = true;
          for (int s = 0; s < a.world && ok; ++s) {
            const uint2* p = a.ar_recv[a.rank] + (long long)s * per_src + slot;
            uint2 w;
            unsigned long long t0 = 0;
            uint32_t it = 0;
            while (true) {
              asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
              if (w.y == ar_seq) break;
              if (((++it) & 0x3ffu) == 0) {
                if (t0 == 0) t0 = globaltimer_ns();
                else if (globaltimer_ns() - t0 > MESH_WAIT_LIMIT_NS || status_aborted(a.status)) {
                  status_record(a.status, MESH_TIMEOUT, SITE_PEER_FLAG, ar_seq, w.y, (unsigned long long)p);
                  ok = false;
                  break;
                }
              }
            }
            sum += __uint_as_float(w.x);
          }
          if (ok) {
            if (a.residual) sum += __bfloat162float(a.residual[(long long)n * a.ldr + row]);
            reinterpret_cast<__nv_bfloat16*>(a.out)[(long long)n * a.ldo + row] = __float2bfloat16_rn(sum);
          }
        }
      }
    }
  sync();
}

// Shared memory a launch needs for a layer of width K and batch B: the staged rows of x plus the K-split partials.
__host__ __device__ inline size_t lin_smem_bytes(int K, int B) {
  return (size_t)B * ((size_t)K * 2 + XPAD) + (size_t)(WARPS + 1) * 16 * NB * sizeof(float);
}

// The whole layer for one CTA of a grid of `gridDim.x` (groups blockIdx.x, blockIdx.x + gridDim.x, ...).
// `wait_inputs()` is called once, after the first weights have been requested and before x is read: a stand-alone
// launch waits there for the kernel before it in the stream, a step kernel for the grid barrier of the previous layer.
// Only the B rows of x that exist are staged; the MMA's batch columns past B repeat row B - 1 and are never stored.
template <int W4, int U, class Wait>
__device__ __forceinline__ void linear_body(const LinArgs& a, uint8_t* smem, Wait wait_inputs) {
  const int K = a.K;
  const int xstride = K * 2 + a.xpad;                             // bytes per x row
  uint8_t* xs = smem;                                             // [B][xstride]
  float* red = reinterpret_cast<float*>(smem + (size_t)a.B * (K * 2 + XPAD));   // [WARPS][16][NB]
  float* fin = red + WARPS * 16 * NB;                             // [16][NB]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  constexpr int CH = ChunkK<W4, U>::value;
  const int kslice = K / WARPS;
  const int k_lo = warp * kslice;
  const int chunks = kslice / CH;
  const int my_groups = (a.n_groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int steps = my_groups * chunks;

  // The weights of this layer do not depend on the layer before it, so the first chunk is requested before waiting.
  const LinHot hot{a.w, a.scales, a.K, a.mode, a.up_off, a.head_dim};
  Chunk<W4, U> c0, c1;
  if (steps > 0) load_chunk<W4, U>(hot, blockIdx.x, 0, k_lo, g8, t4, c0);
  if (a.l2_prefetch) {
    // Every row this CTA will read is requested into L2 now, while the kernel before this one in the stream is
    // still running (this kernel's CTAs are resident beside it): HBM keeps streaming across the kernel boundary and
    // the loads below find their bytes in L2.  One bulk prefetch per row (16 rows per group).
    const long long row_bytes = W4 == 0 ? (long long)K * 2 : (W4 == 3 ? (long long)K : (long long)K / 2);
    for (int i = threadIdx.x; i < my_groups * 16; i += THREADS) {
      int rA, rB;
      group_rows(a, blockIdx.x + (i >> 4) * gridDim.x, rA, rB);
      const int row = ((i & 15) < 8) ? rA + (i & 15) : rB + (i & 15) - 8;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(a.w) + (long long)row * row_bytes;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)row_bytes) : "memory");
    }
  }
  wait_inputs();

  stage_x(a, xs, xstride, BlockSync{});

  const uint8_t* xbase = xs + (g8 < a.B ? g8 : a.B - 1) * xstride + (k_lo + lane_k<W4>(t4)) * 2;
  float c[4] = {0.f, 0.f, 0.f, 0.f};

  // The layer that follows streams weights that depend on nothing computed here: ask for them to be brought into L2
  // now, behind this kernel's own loads, so that HBM keeps streaming through this kernel's reduction and epilogue,
  // the kernel boundary and the next kernel's prologue.  Every CTA requests its slice in 16 KiB pieces.
  if (a.next_w != nullptr) {
    constexpr unsigned long long PIECE = 16384;
    const unsigned long long pieces = (a.next_bytes + PIECE - 1) / PIECE;
    for (unsigned long long i = (unsigned long long)blockIdx.x * THREADS + threadIdx.x; i < pieces;
         i += (unsigned long long)gridDim.x * THREADS) {
      const unsigned long long off = i * PIECE;
      const uint32_t n = (uint32_t)((a.next_bytes - off < PIECE ? a.next_bytes - off : PIECE) & ~15ull);
      if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.next_w + off), "r"(n) : "memory");
    }
  }

  // Two register sets alternate: while one chunk feeds the tensor cores the next one is in flight,
  // across group boundaries too, so the stream of weight loads never drains.
  for (int step = 0; step < steps; ++step) {
    const int gi = step / chunks, ci = step - gi * chunks;
    const int grp = blockIdx.x + gi * gridDim.x;
    if (step + 1 < steps) {
      const int gn = (step + 1) / chunks, cn = (step + 1) - gn * chunks;
      if (step & 1) load_chunk<W4, U>(hot, blockIdx.x + gn * gridDim.x, cn * CH, k_lo, g8, t4, c0);
      else          load_chunk<W4, U>(hot, blockIdx.x + gn * gridDim.x, cn * CH, k_lo, g8, t4, c1);
    }
    if (step & 1) mma_chunk<W4, U>(c1, xbase + ci * CH * 2, c);
    else          mma_chunk<W4, U>(c0, xbase + ci * CH * 2, c);
    if (ci != chunks - 1) continue;
    finish_group(a, grp, c, red, fin, BlockSync{});
    c[0] = c[1] = c[2] = c[3] = 0.f;
  }
}

// Kernel variants (weight format, chunk width), chosen from the layer's shape by `lin_prepare`.
enum LinVariant { LIN_W4N_U2 = 0, LIN_W4N_U1 = 1, LIN_BF16_U4 = 2, LIN_BF16_U1 = 3, LIN_W8_U4 = 4, LIN_W8_U2 = 5,
                  LIN_W8_U1 = 6, LIN_W4W_U2 = 7, LIN_W4W_U1 = 8, LIN_VARIANTS = 9 };

// Checks a layer description and translates it into kernel arguments and a variant.  0 on success.
inline int lin_prepare(const MeshDecodeLinear* d, LinArgs& a, int& variant) {
  if (d->B < 1 || d->B > NB) return set_error(-2, "decode_linear: batch must be 1..8");
  if (d->K % 256) return set_error(-2, "decode_linear: K must be a multiple of 256");
  if (d->w4 != 0 && d->w4 != 1 && d->w4 != 8) return set_error(-2, "decode_linear: weight format must be 0 (bf16), 1 (4-bit) or 8 (8-bit)");
  if (d->w4 && d->K % 512) return set_error(-2, "decode_linear: quantised weights need K %% 512 == 0");
  if (d->N % 16) return set_error(-2, "decode_linear: N must be a multiple of 16");
  if (d->world > MESH_DEC_MAX_RANKS) return set_error(-4, "decode_linear: world too large");
  memset(&a, 0, sizeof(a));
  a.x = (const __nv_bfloat16*)d->x; a.ldx = d->ldx; a.B = d->B; a.K = d->K;
  a.norm_w = (const __nv_bfloat16*)d->norm_w; a.eps = d->eps; a.norm_off = d->norm_off;
  a.w = d->w; a.scales = (const __half*)d->scales;
  a.n_groups = d->N / 16;
  a.mode = d->mode; a.act = d->act; a.up_off = d->up_off;
  a.out = d->out; a.ldo = d->ldo; a.out_f32 = d->out_f32;
  a.q_heads = d->q_heads; a.kv_heads = d->kv_heads; a.head_dim = d->head_dim;
  a.pos = d->pos; a.cos_t = d->cos_t; a.sin_t = d->sin_t;
  a.q_out = (__nv_bfloat16*)d->q_out; a.k_cache = (__nv_bfloat16*)d->k_cache; a.v_cache = (__nv_bfloat16*)d->v_cache;
  a.max_seq = d->max_seq;
  a.rank = d->rank; a.world = d->world > 0 ? d->world : 1;
  for (int r = 0; r < a.world; ++r) a.ar_recv[r] = (uint2*)d->ar_recv[r];
  a.step_ptr = d->step_ptr; a.calls_per_step = d->calls_per_step; a.call_index = d->call_index;
  a.residual = (const __nv_bfloat16*)d->residual; a.ldr = d->ldr;
  a.status = (Status*)d->status;
  a.next_w = (const uint8_t*)d->next_w; a.next_bytes = d->next_bytes;
  if (((uintptr_t)a.next_w & 15) != 0) { a.next_w = nullptr; a.next_bytes = 0; }
  if (d->mode == MESH_DEC_QKV) {
    if (d->head_dim % 16 || (d->q_heads + 2 * d->kv_heads) * d->head_dim != d->N)
      return set_error(-2, "decode_linear: qkv rows must equal (q_heads + 2 kv_heads) * head_dim");
  }
  if (d->mode == MESH_DEC_GLU) a.n_groups = d->N / 8;   // N = gate rows; every group pairs 8 gate + 8 up rows
  if (lin_smem_bytes(d->K, d->B) > 220 * 1024) return set_error(-2, "decode_linear: K too large for shared memory");
  const int kslice = d->K / WARPS;
  // chunk width: 128 k per step when the slice allows it (4 x 16 B per row in flight, twice), else one block
  const bool wide = kslice % 128 == 0;
  a.xpad = XPAD;
  static int narrow4 = -1;
  if (narrow4 < 0) { const char* e = getenv("MESH_DECODE_W4_NARROW"); narrow4 = (e && e[0] == '1') ? 1 : 0; }
  if (d->w4 == 8) {
    // 8-bit codes, 16 bytes (16 k) per lane and load: chunks of 64 k per quad of lanes
    variant = kslice % 256 == 0 ? LIN_W8_U4 : kslice % 128 == 0 ? LIN_W8_U2 : LIN_W8_U1;
    a.xpad = 16;
  } else if (d->w4 && kslice % 128 == 0 && !narrow4) {
    // 4-bit codes, 16 bytes (32 k) per lane and load: chunks of 128 k per quad of lanes
    variant = kslice % 256 == 0 ? LIN_W4W_U2 : LIN_W4W_U1;
    a.xpad = 16;
  } else if (d->w4) {
    variant = wide ? LIN_W4N_U2 : LIN_W4N_U1;
  } else {
    variant = wide ? LIN_BF16_U4 : LIN_BF16_U1;
  }
  return 0;
}

// Runs the layer with the body that `variant` names.
template <class Wait>
__device__ __forceinline__ void linear_dispatch(int variant, const LinArgs& a, uint8_t* smem, Wait wait_inputs) {
  switch (variant) {
    case LIN_W4N_U2: linear_body<1, 2>(a, smem, wait_inputs); break;
    case LIN_W4N_U1: linear_body<1, 1>(a, smem, wait_inputs); break;
    case LIN_BF16_U4: linear_body<0, 4>(a, smem, wait_inputs); break;
    case LIN_BF16_U1: linear_body<0, 1>(a, smem, wait_inputs); break;
    case LIN_W8_U4: linear_body<3, 4>(a, smem, wait_inputs); break;
    case LIN_W8_U2: linear_body<3, 2>(a, smem, wait_inputs); break;
    case LIN_W8_U1: linear_body<3, 1>(a, smem, wait_inputs); break;
    case LIN_W4W_U2: linear_body<2, 2>(a, smem, wait_inputs); break;
    default: linear_body<2, 1>(a, smem, wait_inputs); break;
  }
}

}  // namespace decode
}  // namespace mesh
