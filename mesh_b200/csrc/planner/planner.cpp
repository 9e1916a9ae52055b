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
#include <cmath>
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

// ---- executions in flight: the steady state of a plan that is started again and again
//
// One execution of a standing plan is a set of tasks (its steps) with durations, each on one resource (this processor's
// compute stream, the links of one grid axis), and dependences between them; a dependence may also reach into a later
// execution (`lag` executions later: a collective's staging is reused by the same collective of the next execution, an
// accumulator is read by the next step).  Started every `period`, executions overlap, and the questions of the
// reference's template / unroll stage (rdma/mesh-collective.c:244, :390: copies and lags) are: how short can the period
// be, when does every task start within its execution, and how many executions are alive at once - that many sets of
// buffers (`copies`) are needed for the period to hold.  This is modulo scheduling:
//   * the period is bounded below by the busiest resource (the sum of its tasks' durations) and by every dependence
//     cycle (its durations divided by its lags: found by bisection on the period with a longest-path test);
//   * tasks are placed in dependence order at the earliest time that respects their predecessors and finds their
//     resource free modulo the period; when a task finds no room within one period the period grows a little and the
//     placement starts over (bounded);
//   * latency = the span of one execution under those starts; copies = ceil(latency / period).
// Returns 0, -1 on bad input (a dependence cycle without lag, an unknown task or resource), -2 when no period was found
// within the attempts.  summary_out[0..4] = {period, latency, copies, resource bound, recurrence bound}.
static bool has_positive_cycle(int n, int m, const int* eu, const int* ev, const int* lag, const double* dur, double period) {
  std::vector<double> dist(n, 0.0);
  for (int it = 0; it <= n; ++it) {
    bool moved = false;
    for (int e = 0; e < m; ++e) {
      const double w = dur[eu[e]] - period * (double)lag[e];
      if (dist[eu[e]] + w > dist[ev[e]] + 1e-9) { dist[ev[e]] = dist[eu[e]] + w; moved = true; }
    }
    if (!moved) return false;
  }
  return true;
}

int mesh_plan_pipeline(int n, const double* dur, const int* resource, int n_resources, int m, const int* eu, const int* ev,
                       const int* lag, double* start_out, double* summary_out) {
  if (n < 0 || m < 0 || n_resources < 1) return -1;
  for (int i = 0; i < n; ++i)
    if (dur[i] < 0 || resource[i] < 0 || resource[i] >= n_resources) return -1;
  for (int e = 0; e < m; ++e)
    if (eu[e] < 0 || eu[e] >= n || ev[e] < 0 || ev[e] >= n || lag[e] < 0) return -1;
  if (n == 0) {
    if (summary_out) { summary_out[0] = summary_out[1] = summary_out[3] = summary_out[4] = 0.0; summary_out[2] = 1.0; }
    return 0;
  }
  // order within one execution (edges without lag must be acyclic)
  std::vector<int> indeg(n, 0), order;
  for (int e = 0; e < m; ++e) if (lag[e] == 0) indeg[ev[e]]++;
  for (int i = 0; i < n; ++i) if (!indeg[i]) order.push_back(i);
  for (size_t k = 0; k < order.size(); ++k)
    for (int e = 0; e < m; ++e)
      if (lag[e] == 0 && eu[e] == order[k] && --indeg[ev[e]] == 0) order.push_back(ev[e]);
  if ((int)order.size() != n) return -1;
  // bounds on the period
  std::vector<double> busy(n_resources, 0.0);
  double total = 0.0, longest = 0.0;
  for (int i = 0; i < n; ++i) { busy[resource[i]] += dur[i]; total += dur[i]; if (dur[i] > longest) longest = dur[i]; }
  double res_bound = 0.0;
  for (double b : busy) if (b > res_bound) res_bound = b;
  double rec_bound = 0.0;
  bool any_lag = false;
  for (int e = 0; e < m; ++e) any_lag |= lag[e] > 0;
  if (any_lag && total > 0) {
    double lo = 0.0, hi = total;                           // a cycle holds at most every task once per unit of lag
    if (has_positive_cycle(n, m, eu, ev, lag, dur, hi)) return -1;
    for (int it = 0; it < 60; ++it) {
      const double mid = 0.5 * (lo + hi);
      if (has_positive_cycle(n, m, eu, ev, lag, dur, mid)) lo = mid; else hi = mid;
    }
    rec_bound = hi;
  }
  double period = res_bound > rec_bound ? res_bound : rec_bound;
  if (period <= 0) period = longest > 0 ? longest : 1.0;
  struct Busy { double from, to; };                       // within [0, period), from <= to (a wrapped task makes two)
  std::vector<double> start(n, 0.0);
  for (int attempt = 0; attempt < 160; ++attempt) {
    std::vector<std::vector<Busy>> table(n_resources);
    std::vector<char> placed(n, 0);
    bool ok = true;
    for (int k = 0; k < n && ok; ++k) {
      const int v = order[k];
      double est = 0.0;
      for (int e = 0; e < m; ++e)
        if (ev[e] == v && placed[eu[e]]) {
          const double t = start[eu[e]] + dur[eu[e]] - period * (double)lag[e];
          if (t > est) est = t;
        }
      // earliest t in [est, est + period) whose window [t, t + dur) is free modulo the period
      double t = est;
      bool found = dur[v] <= 0;
      for (int guard = 0; guard < 4 * n + 8 && !found; ++guard) {
        const double a = std::fmod(t, period), b = a + dur[v];
        double bump = -1.0;
        for (const Busy& z : table[resource[v]]) {
          const bool hit = (a < z.to - 1e-9 && z.from < b - 1e-9) || (b > period && z.from < b - period - 1e-9);
          if (hit) {
            // move to the end of the interval we ran into (in unwrapped time)
            double to = z.to;
            if (!(a < z.to - 1e-9 && z.from < b - 1e-9)) to += period;      // hit through the wrapped part
            const double cand = t + (to - a);
            if (cand > bump) bump = cand;
          }
        }
        if (bump < 0) found = true;
        else { t = bump; if (t - est >= period - 1e-9) break; }
      }
      if (!found || dur[v] > period + 1e-9) { ok = false; break; }
      start[v] = t;
      placed[v] = 1;
      if (dur[v] > 0) {
        const double a = std::fmod(t, period), b = a + dur[v];
        if (b <= period + 1e-9) table[resource[v]].push_back(Busy{a, b < period ? b : period});
        else { table[resource[v]].push_back(Busy{a, period}); table[resource[v]].push_back(Busy{0.0, b - period}); }
      }
    }
    // dependences that reach back from a later task of the order to an earlier one (lag > 0) were not seen when the
    // earlier one was placed: check them now
    for (int e = 0; e < m && ok; ++e)
      if (start[ev[e]] + period * (double)lag[e] + 1e-9 < start[eu[e]] + dur[eu[e]]) ok = false;
    if (ok) {
      double first = 1e300, last = 0.0;
      for (int i = 0; i < n; ++i) {
        if (start[i] < first) first = start[i];
        if (start[i] + dur[i] > last) last = start[i] + dur[i];
      }
      const double latency = last - first;
      for (int i = 0; i < n; ++i) start_out[i] = start[i] - first;
      if (summary_out) {
        summary_out[0] = period;
        summary_out[1] = latency;
        summary_out[2] = std::ceil(latency / period - 1e-9) < 1.0 ? 1.0 : std::ceil(latency / period - 1e-9);
        summary_out[3] = res_bound;
        summary_out[4] = rec_bound;
      }
      return 0;
    }
    period *= 1.02;
  }
  return -2;
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
