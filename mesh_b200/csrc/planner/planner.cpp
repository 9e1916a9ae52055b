// Planner: algorithm choice per collective size, workspace layout with multi-execution copies, and
// plan archives.  On a uniform NVSwitch fabric the reference's route/tree packing and LP transfer
// ordering (rdma/mesh-collective.c:818-1121) collapse: every peer is one hop away at the same
// bandwidth, so what remains of `mesh_plan` is (a) grouping declared transfers into demands with a
// closed-form alpha + n*beta choice of algorithm, (b) placing every buffer (lifetime colouring) once
// per `copies` so that execution t uses copy t mod copies (plan_unroll, :390), (c) save / load of the
// result (mesh_plan_save / mesh_plan_load, :3151, :3272) with 8-byte alignment and a checksum.
// All arithmetic is integer or IEEE in a fixed order: every rank computes the same plan.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" int64_t mesh_graph_colour(int n, const int* start, const int* end, const int64_t* size, int64_t align, int64_t* offset);

extern "C" {

enum MeshAlgo { MESH_ALGO_ONE_SHOT = 0, MESH_ALGO_TWO_SHOT = 1, MESH_ALGO_NVLS = 2, MESH_ALGO_COPY_ENGINE = 3 };

// Time model (microseconds) of an all-reduce of `bytes` over `world` ranks:
//   one-shot : alpha + (world-1) * bytes / bw           every rank reads every peer's whole buffer
//   two-shot : 2*alpha + 2 * (world-1)/world * bytes / bw
//   nvls     : alpha_nvls + bytes / bw_nvls              in-switch reduction, when the heap has a multicast mapping
int mesh_plan_choose_allreduce(uint64_t bytes, int world, double alpha_us, double gbps_per_dir, int nvls_available,
                               double* est_us_out) {
  if (world <= 1) { if (est_us_out) *est_us_out = 0.0; return MESH_ALGO_ONE_SHOT; }
  const double bw = gbps_per_dir * 1e3;                   // bytes per microsecond
  const double one = alpha_us + (double)(world - 1) * (double)bytes / bw;
  const double two = 2.0 * alpha_us + 2.0 * (double)(world - 1) / (double)world * (double)bytes / bw;
  const double nv = nvls_available ? (1.5 * alpha_us + (double)bytes / bw) : 1e300;
  int algo = MESH_ALGO_ONE_SHOT;
  double best = one;
  if (two < best) { best = two; algo = MESH_ALGO_TWO_SHOT; }
  if (nv < best) { best = nv; algo = MESH_ALGO_NVLS; }
  if (est_us_out) *est_us_out = best;
  return algo;
}

// Buffers with lifetimes -> offsets; the whole layout is repeated `copies` times back to back.
// offsets_out[c * n + i] = offset of buffer i in copy c.  Returns the bytes of ONE copy.
int64_t mesh_plan_layout(int n, const int* start, const int* end, const int64_t* size, int64_t align, int copies,
                         int64_t* offsets_out) {
  std::vector<int64_t> off(n > 0 ? n : 1);
  int64_t one = mesh_graph_colour(n, start, end, size, align, off.data());
  one = (one + align - 1) / align * align;
  for (int c = 0; c < copies; ++c)
    for (int i = 0; i < n; ++i) offsets_out[(int64_t)c * n + i] = (int64_t)c * one + off[i];
  return one;
}

// ---- archives: header {magic, version, epoch, words, checksum} + 8-byte words
struct PlanHeader { uint64_t magic, version, epoch, words, checksum; };
static const uint64_t PLAN_MAGIC = 0x4d4553485f504c4eull;   // "MESH_PLN"

static uint64_t fnv(const uint64_t* w, uint64_t n) {
  uint64_t h = 1469598103934665603ull;
  for (uint64_t i = 0; i < n; ++i) { h ^= w[i]; h *= 1099511628211ull; }
  return h;
}

int mesh_plan_save(const char* path, uint64_t epoch, const uint64_t* words, uint64_t n) {
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  PlanHeader h{PLAN_MAGIC, 1, epoch, n, fnv(words, n)};
  int ok = fwrite(&h, sizeof(h), 1, f) == 1 && (n == 0 || fwrite(words, 8, n, f) == n);
  ok = ok && fflush(f) == 0;
  fclose(f);
  return ok ? 0 : -2;
}

// Returns the number of words (<= cap copied), -1 cannot open, -2 bad header, -3 checksum, -4 cap too small.
int64_t mesh_plan_load(const char* path, uint64_t* epoch_out, uint64_t* words, uint64_t cap) {
  FILE* f = fopen(path, "rb");
  if (!f) return -1;
  PlanHeader h;
  if (fread(&h, sizeof(h), 1, f) != 1 || h.magic != PLAN_MAGIC || h.version != 1) { fclose(f); return -2; }
  if (h.words > cap) { fclose(f); return -4; }
  if (h.words && fread(words, 8, h.words, f) != h.words) { fclose(f); return -2; }
  fclose(f);
  if (fnv(words, h.words) != h.checksum) return -3;
  if (epoch_out) *epoch_out = h.epoch;
  return (int64_t)h.words;
}

}  // extern "C"
