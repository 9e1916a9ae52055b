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

// ---- declared transfers -> demands -> an order on the links
//
// A compiled step declares its transfers with the step that produces the value (`at`: where the transfer sits in the
// plan) and the step that first reads the result (`read`).  The planner
//   1. groups transfers into demands: reductions of one axis whose results nobody reads before the group's last
//      member exists (gradient all-reduces) are sent as one flat message up to `bucket_bytes` (the reference groups
//      declared rows into demands, rdma/mesh-collective.c:1791); every other transfer is a demand of its own;
//   2. gives every demand an algorithm (closed form alpha + n*beta), the number of pieces it takes through a staging
//      buffer of `staging_bytes`, and a duration;
//   3. orders the demands of every axis on that axis's links: earliest deadline first among the demands whose value
//      exists (release = the producing step's time, deadline = the first reader's time, both from `step_us` per plan
//      step), one demand at a time per axis (plan_schedule, :928, orders by completion times from an LP; on a uniform
//      fabric with one resource per axis the list schedule is what remains);
//   4. reports for every demand its start, end and how long its reader waits for it (`exposed_us`), and for the step the
//      sum of link time, the exposed part and the makespan: what an overlapping executor can hide and what it cannot.
enum MeshVerb { MESH_VERB_ALL_REDUCE = 0, MESH_VERB_ALL_GATHER = 1, MESH_VERB_REDUCE_SCATTER = 2, MESH_VERB_ALL_TO_ALL = 3,
                MESH_VERB_POINT = 4 };

typedef struct MeshTransferIn {
  int64_t bytes;        // bytes of the whole value on one rank
  int32_t axis, verb;
  int32_t at, read;     // plan step of the transfer, plan step of the first reader (>= at)
  int32_t groupable;    // 1: a reduction whose result is only read at `read` and may travel with others
  int32_t pad;
} MeshTransferIn;

typedef struct MeshTransferOut {
  int32_t demand;       // demand this transfer belongs to
  int32_t algo;         // MeshAlgo of the demand
  int32_t pieces;       // staging-buffer pieces of the demand
  int32_t order;        // position of the demand on its axis
  double start_us, end_us, exposed_us;
} MeshTransferOut;

static double verb_time_us(int verb, uint64_t bytes, int world, double alpha_us, double bw, int nvls, int* algo) {
  *algo = MESH_ALGO_ONE_SHOT;
  if (world <= 1) return 0.0;
  const double frac = (double)(world - 1) / (double)world;
  switch (verb) {
    case MESH_VERB_ALL_REDUCE: {
      double est = 0.0;
      *algo = mesh_plan_choose_allreduce(bytes, world, alpha_us, bw / 1e3, nvls, &est);
      return est;
    }
    case MESH_VERB_ALL_GATHER:
    case MESH_VERB_REDUCE_SCATTER:
    case MESH_VERB_ALL_TO_ALL:
      return alpha_us + frac * (double)bytes / bw;
    default:
      *algo = MESH_ALGO_COPY_ENGINE;
      return alpha_us + (double)bytes / bw;
  }
}

// summary_out[0..3] = {sum of link time, sum of exposed time, makespan, number of demands}.  Returns 0, or -1 on bad input.
int mesh_plan_transfers(int n, const MeshTransferIn* in, int n_axes, const int* world_of_axis, double step_us,
                        double alpha_us, double gbps_per_dir, int nvls_available, int64_t bucket_bytes,
                        int64_t staging_bytes, MeshTransferOut* out, double* summary_out) {
  if (n < 0 || n_axes < 1 || step_us < 0 || gbps_per_dir <= 0) return -1;
  const double bw = gbps_per_dir * 1e3;                   // bytes per microsecond
  struct Demand { int axis, verb, first_at, last_at, first_read; int64_t bytes; std::vector<int> members; int algo, pieces;
                  double dur, start, end; int order; bool done; };
  std::vector<Demand> demands;
  // 1. grouping, in plan order (the order every rank sees)
  std::vector<int> idx(n);
  for (int i = 0; i < n; ++i) idx[i] = i;
  for (int a = 1; a < n; ++a)                              // insertion sort by (at, index): stable and tiny
    for (int b = a; b > 0 && in[idx[b]].at < in[idx[b - 1]].at; --b) { int t = idx[b]; idx[b] = idx[b - 1]; idx[b - 1] = t; }
  std::vector<int> open_of_axis(n_axes, -1);              // the demand of each axis that still takes members
  for (int k = 0; k < n; ++k) {
    const MeshTransferIn& t = in[idx[k]];
    if (t.axis < 0 || t.axis >= n_axes || t.read < t.at || t.bytes < 0) return -1;
    int d = -1;
    if (t.groupable && t.verb == MESH_VERB_ALL_REDUCE && bucket_bytes > 0) {
      d = open_of_axis[t.axis];
      // joining must not hold anybody's result back: every member exists before the earliest reader of the group
      if (d >= 0 && (demands[d].bytes + t.bytes > bucket_bytes || t.at >= demands[d].first_read || t.read <= demands[d].last_at))
        d = -1;
    }
    if (d < 0) {
      demands.push_back(Demand{t.axis, t.verb, t.at, t.at, t.read, 0, {}, 0, 1, 0.0, 0.0, 0.0, 0, false});
      d = (int)demands.size() - 1;
      // a transfer that stands alone leaves the axis's open group as it is
      if (t.groupable && t.verb == MESH_VERB_ALL_REDUCE && bucket_bytes > 0) open_of_axis[t.axis] = d;
    }
    Demand& g = demands[d];
    g.bytes += t.bytes;
    g.last_at = t.at > g.last_at ? t.at : g.last_at;
    g.first_read = t.read < g.first_read ? t.read : g.first_read;
    g.members.push_back(idx[k]);
  }
  // 2. algorithm, pieces, duration
  for (Demand& g : demands) {
    const int world = world_of_axis[g.axis];
    g.dur = verb_time_us(g.verb, (uint64_t)g.bytes, world, alpha_us, bw, nvls_available, &g.algo);
    g.pieces = staging_bytes > 0 ? (int)((g.bytes + staging_bytes - 1) / staging_bytes) : 1;
    if (g.pieces < 1) g.pieces = 1;
    if (g.pieces > 1) g.dur += (g.pieces - 1) * alpha_us;                   // every further piece pays a latency
  }
  // 3. earliest deadline first per axis, non-preemptive, with release times
  double link_sum = 0.0, exposed_sum = 0.0, makespan = 0.0;
  for (int ax = 0; ax < n_axes; ++ax) {
    double now = 0.0;
    int placed = 0, total = 0;
    for (const Demand& g : demands) total += g.axis == ax;
    while (placed < total) {
      int pick = -1;
      double next_release = 1e300;
      for (int d = 0; d < (int)demands.size(); ++d) {
        const Demand& g = demands[d];
        if (g.axis != ax || g.done) continue;
        const double rel = (double)(g.last_at + 1) * step_us;
        if (rel <= now) {
          if (pick < 0 || g.first_read < demands[pick].first_read ||
              (g.first_read == demands[pick].first_read && g.last_at < demands[pick].last_at)) pick = d;
        } else if (rel < next_release) {
          next_release = rel;
        }
      }
      if (pick < 0) { now = next_release; continue; }
      Demand& g = demands[pick];
      g.start = now;
      g.end = now + g.dur;
      g.order = placed++;
      g.done = true;
      now = g.end;
      link_sum += g.dur;
      const double deadline = (double)g.first_read * step_us;
      if (g.end > deadline) exposed_sum += g.end - deadline;
      if (g.end > makespan) makespan = g.end;
    }
  }
  for (int d = 0; d < (int)demands.size(); ++d) {
    const Demand& g = demands[d];
    const double deadline = (double)g.first_read * step_us;
    for (int m : g.members)
      out[m] = MeshTransferOut{d, g.algo, g.pieces, g.order, g.start, g.end, g.end > deadline ? g.end - deadline : 0.0};
  }
  if (summary_out) {
    summary_out[0] = link_sum; summary_out[1] = exposed_sum; summary_out[2] = makespan; summary_out[3] = (double)demands.size();
  }
  return 0;
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
