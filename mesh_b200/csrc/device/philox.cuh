// Philox4x32-10 (Salmon et al., SC 2011) on the device, and the keep-mask of attention dropout.
//
// A dropout decision is a pure function of the element's LOGICAL coordinates (batch*heads + head, query position,
// key position in the unsharded sequence), the seed, the draw site and the execution number: a rank that holds any
// shard of the sequence - contiguous, striped, a ring chunk - drops exactly the elements one device would (the
// reference keys its generator by unsharded coordinates for the same reason, compiler/mesh_compiler/operations.py:
// 7143-7158, :7201-7275).  One Philox call serves four consecutive key positions:
//     counter = (key_pos >> 2, query_pos, batch*heads + head, site),  key = (seed_lo ^ execution * 0x9E3779B9, seed_hi),
//     u = (word[key_pos & 3] >> 8) * 2^-24,  keep iff u >= p.
// `mesh_b200/ops/philox.py::attention_keep_mask` states the same function with tensor arithmetic (the tests' oracle).
#pragma once
#include <cstdint>

namespace mesh {

struct Philox4 { uint32_t w[4]; };

__device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += W0; k1 += W1;
  }
  return Philox4{{c0, c1, c2, c3}};
}

struct DropoutKey {
  uint32_t k0, k1, site;
  float p, inv_keep;         // drop probability, 1 / (1 - p)
};

// Keep decisions for one (head, query position) row, with the last group of four key positions cached: a thread
// that walks consecutive key positions pays one Philox call per four of them.
struct DropoutRow {
  uint32_t bh, qpos, group;
  Philox4 words;
  __device__ __forceinline__ void begin(uint32_t bh_, uint32_t qpos_) { bh = bh_; qpos = qpos_; group = 0xffffffffu; }
  __device__ __forceinline__ bool keep(const DropoutKey& k, uint32_t kpos) {
    const uint32_t g = kpos >> 2;
    if (g != group) {
      words = philox4x32_10(g, qpos, bh, k.site, k.k0, k.k1);
      group = g;
    }
    const uint32_t w = words.w[kpos & 3u];
    return (float)(w >> 8) * (1.0f / 16777216.0f) >= k.p;
  }
};

}  // namespace mesh
