// Graph algorithms used by the compiler, the planner and the share solver (host only).
//
// What the reference keeps in rdma/mesh-graph.c and what survives on a uniform NVSwitch fabric:
//   * topological levels / longest path                      (mesh-graph.c DFS / closure / longest path)
//   * exact overlap of box-strided views and the RAW/WAR/WAW dependence relation over them
//                                                             (mesh_graph_dependences_views, :2751; the
//                                                              reference calls isl, box views need none)
//   * lifetime colouring of buffers, greedy by size           (mesh_graph_greedy_by_size, :4881; chains/fat cover)
//   * coupled share solve: minimise sum over stages of the slowest rank's time, linear in the shares,
//     with per-rank caps                                      (mesh_graph_shares_coupled, :2072; HiGHS there,
//                                                              a dense simplex here)
//   * cycle mean of a weighted graph (throughput bound of a software-pipelined plan, :2370)
//   * signature check: every member of a group issues the same ordered list of synchronising operations
// Critical path, list scheduling, chain cover, minimum arborescence and concurrent flow live in routing.cpp.
// Deterministic by construction (integer or IEEE arithmetic in a fixed order), so every rank
// derives the same result from the same input.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

extern "C" {

// ---------------------------------------------------------------------------------- topological levels
// level[v] = length of the longest path ending in v; returns 0, or -1 when the graph has a cycle.
int mesh_graph_levels(int n, int m, const int* src, const int* dst, int* level) {
  std::vector<int> indeg(n, 0), head(n + 1, 0), adj(m);
  for (int e = 0; e < m; ++e) { ++indeg[dst[e]]; ++head[src[e] + 1]; }
  for (int v = 0; v < n; ++v) head[v + 1] += head[v];
  std::vector<int> fill(head.begin(), head.end() - 1);
  for (int e = 0; e < m; ++e) adj[fill[src[e]]++] = dst[e];
  std::vector<int> q;
  q.reserve(n);
  for (int v = 0; v < n; ++v) { level[v] = 0; if (!indeg[v]) q.push_back(v); }
  for (size_t i = 0; i < q.size(); ++i) {
    int v = q[i];
    for (int k = head[v]; k < head[v + 1]; ++k) {
      int w = adj[k];
      level[w] = std::max(level[w], level[v] + 1);
      if (--indeg[w] == 0) q.push_back(w);
    }
  }
  return (int)q.size() == n ? 0 : -1;
}

// ---------------------------------------------------------------------------------- strided views
// A view is the set { base + sum_i k_i * stride[i] + [0, elem) : 0 <= k_i < size[i] } of byte addresses.
struct View { int64_t base; int ndim; const int64_t* size; const int64_t* stride; int64_t elem; };

static void extent(const View& v, int64_t& lo, int64_t& hi) {
  lo = v.base; hi = v.base + v.elem;
  for (int i = 0; i < v.ndim; ++i) {
    if (v.size[i] <= 0) { hi = lo; return; }
    int64_t d = (v.size[i] - 1) * v.stride[i];
    if (d >= 0) hi += d; else lo += d;
  }
}

// Does some element of `a` (fixing dims [0, d)) overlap view b?  Exact, by enumeration of a's outer
// dimensions with interval pruning; b is handled the same way one level down.
static bool overlap_rec(const View& a, int d, int64_t a_off, const View& b, int e, int64_t b_off, int64_t& budget) {
  // bounding intervals of the remaining sub-boxes
  int64_t alo = a_off, ahi = a_off + a.elem, blo = b_off, bhi = b_off + b.elem;
  for (int i = d; i < a.ndim; ++i) { int64_t s = (a.size[i] - 1) * a.stride[i]; if (s >= 0) ahi += s; else alo += s; }
  for (int i = e; i < b.ndim; ++i) { int64_t s = (b.size[i] - 1) * b.stride[i]; if (s >= 0) bhi += s; else blo += s; }
  if (ahi <= blo || bhi <= alo) return false;
  if (d == a.ndim && e == b.ndim) return true;
  if (--budget < 0) return true;                       // out of budget: answer conservatively (may conflict)
  // a dense remaining sub-box is exactly its bounding interval
  auto dense = [](const View& v, int from) {
    int64_t run = v.elem;
    for (int i = v.ndim - 1; i >= from; --i) {
      if (v.size[i] == 1) continue;
      if (std::llabs(v.stride[i]) != run) return false;
      run *= v.size[i];
    }
    return true;
  };
  bool da = dense(a, d), db = dense(b, e);
  if (da && db) return true;
  // split the non-dense view with the larger outer stride
  bool split_a = !da && (db || e == b.ndim || (d < a.ndim && std::llabs(a.stride[d]) >= std::llabs(b.stride[e])));
  if (split_a) {
    for (int64_t k = 0; k < a.size[d]; ++k)
      if (overlap_rec(a, d + 1, a_off + k * a.stride[d], b, e, b_off, budget)) return true;
    return false;
  }
  for (int64_t k = 0; k < b.size[e]; ++k)
    if (overlap_rec(a, d, a_off, b, e + 1, b_off + k * b.stride[e], budget)) return true;
  return false;
}

int mesh_graph_views_overlap(int64_t base_a, int nd_a, const int64_t* size_a, const int64_t* stride_a, int64_t elem_a,
                             int64_t base_b, int nd_b, const int64_t* size_b, const int64_t* stride_b, int64_t elem_b) {
  View a{base_a, nd_a, size_a, stride_a, elem_a}, b{base_b, nd_b, size_b, stride_b, elem_b};
  int64_t alo, ahi, blo, bhi;
  extent(a, alo, ahi);
  extent(b, blo, bhi);
  if (ahi <= blo || bhi <= alo) return 0;
  int64_t budget = 1 << 20;
  return overlap_rec(a, 0, a.base, b, 0, b.base, budget) ? 1 : 0;
}

// Accesses in program order: access k belongs to operation op[k], is a write when is_write[k], and touches
// buffer buf[k] through a view (views packed 8 int64 each: base, elem, size[3], stride[3]).
// Emits dependence edges (earlier op -> later op) with kind 0 RAW, 1 WAR, 2 WAW; returns the count
// (or -needed when `cap` is too small).  Transitively implied pairs are still listed.
int mesh_graph_dependences(int n_acc, const int* op, const int* is_write, const int* buf, const int64_t* views,
                           int cap, int* e_src, int* e_dst, int* e_kind) {
  int count = 0;
  for (int j = 0; j < n_acc; ++j) {
    for (int i = 0; i < j; ++i) {
      if (buf[i] != buf[j] || op[i] == op[j]) continue;
      if (!is_write[i] && !is_write[j]) continue;
      const int64_t* a = views + 8 * i;
      const int64_t* b = views + 8 * j;
      if (!mesh_graph_views_overlap(a[0], 3, a + 2, a + 5, a[1], b[0], 3, b + 2, b + 5, b[1])) continue;
      int kind = is_write[i] ? (is_write[j] ? 2 : 0) : 1;
      if (count < cap) { e_src[count] = op[i]; e_dst[count] = op[j]; e_kind[count] = kind; }
      ++count;
    }
  }
  return count <= cap ? count : -count;
}

// ---------------------------------------------------------------------------------- lifetime colouring
// Buffers with lifetimes [start, end] (inclusive step indices) and sizes; assigns byte offsets so that
// buffers alive at the same time never overlap.  Greedy by size (largest first, lowest fitting offset).
// Returns the total bytes needed.
int64_t mesh_graph_colour(int n, const int* start, const int* end, const int64_t* size, int64_t align, int64_t* offset) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return size[a] > size[b]; });
  std::vector<int> placed;
  int64_t total = 0;
  if (align <= 0) align = 1;
  for (int idx : order) {
    int64_t sz = (size[idx] + align - 1) / align * align;
    std::vector<std::pair<int64_t, int64_t>> busy;
    for (int p : placed)
      if (!(end[p] < start[idx] || end[idx] < start[p])) {
        int64_t ps = (size[p] + align - 1) / align * align;
        busy.emplace_back(offset[p], offset[p] + ps);
      }
    std::sort(busy.begin(), busy.end());
    int64_t at = 0;
    for (auto& b : busy) {
      if (at + sz <= b.first) break;
      at = std::max(at, b.second);
    }
    offset[idx] = at;
    total = std::max(total, at + sz);
    placed.push_back(idx);
  }
  return total;
}

// ---------------------------------------------------------------------------------- dense simplex
// minimise c.x  subject to  A x <= b, x >= 0  (b may be negative: a big-M style phase one is folded in by
// adding one artificial column).  Small dense problems only.  Returns 0 ok, 1 infeasible, 2 unbounded.
static int simplex(int m, int n, std::vector<std::vector<double>>& T, std::vector<int>& basis) {
  // T is (m+1) x (n+m+1): rows 0..m-1 constraints with slacks, row m objective (to minimise); last col = rhs
  const double EPS = 1e-10;
  const int cols = n + m;
  for (int iter = 0; iter < 200000; ++iter) {
    int piv_c = -1;
    for (int j = 0; j < cols; ++j)
      if (T[m][j] < -EPS) { piv_c = j; break; }           // Bland: lowest index with negative reduced cost
    if (piv_c < 0) return 0;
    int piv_r = -1;
    double best = 0;
    for (int i = 0; i < m; ++i) {
      if (T[i][piv_c] > EPS) {
        double r = T[i][cols] / T[i][piv_c];
        if (piv_r < 0 || r < best - EPS || (std::fabs(r - best) <= EPS && basis[i] < basis[piv_r])) { piv_r = i; best = r; }
      }
    }
    if (piv_r < 0) return 2;
    double p = T[piv_r][piv_c];
    for (int j = 0; j <= cols; ++j) T[piv_r][j] /= p;
    for (int i = 0; i <= m; ++i) {
      if (i == piv_r) continue;
      double f = T[i][piv_c];
      if (std::fabs(f) < EPS) continue;
      for (int j = 0; j <= cols; ++j) T[i][j] -= f * T[piv_r][j];
    }
    basis[piv_r] = piv_c;
  }
  return 2;
}

// Coupled share solve.  `parts` model parts, `ranks` ranks, `stages` stages.  Variables x[p][j] >= 0 with
// sum_j x[p][j] = 1 and x[p][j] <= upper[j].  Stage s on rank j costs fixed[s*ranks+j] + sum_p coef[(s*ranks+j)*parts+p] * x[p][j];
// the stage's time is the slowest rank plus comm[s*parts+p] * max_j x[p][j] for every part it communicates.
// Minimises the sum of stage times.  shares_out[p*ranks+j].  Returns 0 on success.
int mesh_graph_shares_coupled(int parts, int ranks, int stages, const double* fixed, const double* coef, const double* comm,
                              const double* upper, double* shares_out, double* objective_out) {
  // variables: x (parts*ranks), z_s (stages), y_p (parts; y_p >= x[p][j])
  const int nx = parts * ranks, nz = stages, ny = parts;
  const int n = nx + nz + ny;
  // constraints (all as <=):
  //  (a) fixed + sum coef x - z_s + sum_p comm[s][p]*0 <= 0    for every (s, j)   [comm enters the objective through y]
  //  (b) x[p][j] - y_p <= 0
  //  (c) x[p][j] <= upper[j]
  //  (d) sum_j x[p][j] <= 1 and -sum_j x[p][j] <= -1
  const int m = stages * ranks + nx + nx + 2 * parts;
  std::vector<std::vector<double>> A(m, std::vector<double>(n, 0.0));
  std::vector<double> b(m, 0.0), c(n, 0.0);
  int r = 0;
  for (int s = 0; s < stages; ++s)
    for (int j = 0; j < ranks; ++j, ++r) {
      for (int p = 0; p < parts; ++p) A[r][p * ranks + j] = coef[(s * ranks + j) * parts + p];
      A[r][nx + s] = -1.0;
      b[r] = -fixed[s * ranks + j];
    }
  for (int p = 0; p < parts; ++p)
    for (int j = 0; j < ranks; ++j, ++r) { A[r][p * ranks + j] = 1.0; A[r][nx + nz + p] = -1.0; }
  for (int p = 0; p < parts; ++p)
    for (int j = 0; j < ranks; ++j, ++r) { A[r][p * ranks + j] = 1.0; b[r] = upper ? upper[j] : 1.0; }
  for (int p = 0; p < parts; ++p) {
    for (int j = 0; j < ranks; ++j) { A[r][p * ranks + j] = 1.0; A[r + 1][p * ranks + j] = -1.0; }
    b[r] = 1.0; b[r + 1] = -1.0;
    r += 2;
  }
  for (int s = 0; s < stages; ++s) c[nx + s] = 1.0;
  for (int p = 0; p < parts; ++p) {
    double w = 0;
    for (int s = 0; s < stages; ++s) w += comm ? comm[s * parts + p] : 0.0;
    c[nx + nz + p] = w;
  }
  // phase one with a single artificial variable a >= 0 subtracted from every row whose rhs is negative
  std::vector<std::vector<double>> T(m + 1, std::vector<double>(n + 1 + m + 1, 0.0));
  const int N = n + 1;                                 // structural columns incl. the artificial (index n)
  std::vector<int> basis(m);
  for (int i = 0; i < m; ++i) {
    for (int j = 0; j < n; ++j) T[i][j] = A[i][j];
    T[i][n] = -1.0;
    T[i][N + i] = 1.0;
    T[i][N + m] = b[i];
    basis[i] = N + i;
  }
  int worst = -1;
  for (int i = 0; i < m; ++i) if (b[i] < 0 && (worst < 0 || b[i] < b[worst])) worst = i;
  if (worst >= 0) {
    T[m].assign(N + m + 1, 0.0);
    T[m][n] = 1.0;                                     // minimise the artificial
    // pivot the artificial in at the most negative row: makes every rhs non-negative
    double pv = T[worst][n];
    for (int j = 0; j <= N + m; ++j) T[worst][j] /= pv;
    for (int i = 0; i <= m; ++i) {
      if (i == worst) continue;
      double f = T[i][n];
      if (f == 0) continue;
      for (int j = 0; j <= N + m; ++j) T[i][j] -= f * T[worst][j];
    }
    basis[worst] = n;
    if (simplex(m, N, T, basis) != 0) return 1;
    if (std::fabs(T[m][N + m]) > 1e-7) return 1;       // infeasible
    // drive the artificial out of the basis if it is still there (at zero)
    for (int i = 0; i < m; ++i) {
      if (basis[i] != n) continue;
      int pc = -1;
      for (int j = 0; j < N + m; ++j) if (j != n && std::fabs(T[i][j]) > 1e-9) { pc = j; break; }
      if (pc < 0) continue;
      double p = T[i][pc];
      for (int j = 0; j <= N + m; ++j) T[i][j] /= p;
      for (int k = 0; k <= m; ++k) {
        if (k == i) continue;
        double f = T[k][pc];
        if (f == 0) continue;
        for (int j = 0; j <= N + m; ++j) T[k][j] -= f * T[i][j];
      }
      basis[i] = pc;
    }
    for (int i = 0; i <= m; ++i) T[i][n] = 0.0;         // forbid the artificial from re-entering
  }
  // phase two objective, expressed in the current basis
  T[m].assign(N + m + 1, 0.0);
  for (int j = 0; j < n; ++j) T[m][j] = c[j];
  for (int i = 0; i < m; ++i) {
    int bj = basis[i];
    double cb = bj < n ? c[bj] : 0.0;
    if (cb == 0) continue;
    for (int j = 0; j <= N + m; ++j) T[m][j] -= cb * T[i][j];
  }
  T[m][n] = 0.0;
  int rc = simplex(m, N, T, basis);
  if (rc != 0) return rc;
  std::vector<double> x(N + m, 0.0);
  for (int i = 0; i < m; ++i) x[basis[i]] = T[i][N + m];
  for (int k = 0; k < nx; ++k) shares_out[k] = x[k];
  if (objective_out) *objective_out = -T[m][N + m];
  return 0;
}

// ---------------------------------------------------------------------------------- maximum cycle mean
// Karp's algorithm on a graph with edge weights (time) and unit token counts: the throughput bound of a
// software-pipelined plan.  Returns -1 when the graph is acyclic.
double mesh_graph_cycle_mean(int n, int m, const int* src, const int* dst, const double* w) {
  const double NEG = -1e300;
  std::vector<std::vector<double>> D(n + 1, std::vector<double>(n, NEG));
  for (int v = 0; v < n; ++v) D[0][v] = 0.0;
  for (int k = 1; k <= n; ++k)
    for (int e = 0; e < m; ++e)
      if (D[k - 1][src[e]] > NEG / 2) D[k][dst[e]] = std::max(D[k][dst[e]], D[k - 1][src[e]] + w[e]);
  double best = -1.0;
  bool any = false;
  for (int v = 0; v < n; ++v) {
    if (D[n][v] <= NEG / 2) continue;
    double worst = 1e300;
    for (int k = 0; k < n; ++k)
      if (D[k][v] > NEG / 2) worst = std::min(worst, (D[n][v] - D[k][v]) / (n - k));
    if (!any || worst > best) { best = worst; any = true; }
  }
  return any ? best : -1.0;
}

// ---------------------------------------------------------------------------------- signature check
// seqs: for each of `members` processors a list of `len[i]` operation ids (concatenated).  Every member
// must issue the same sequence.  Returns -1 when they agree, else the first position that differs.
int mesh_graph_signature_check(int members, const int* len, const int64_t* seqs) {
  if (members <= 1) return -1;
  std::vector<const int64_t*> at(members);
  const int64_t* p = seqs;
  for (int i = 0; i < members; ++i) { at[i] = p; p += len[i]; }
  int shortest = *std::min_element(len, len + members);
  for (int k = 0; k < shortest; ++k)
    for (int i = 1; i < members; ++i)
      if (at[i][k] != at[0][k]) return k;
  for (int i = 1; i < members; ++i)
    if (len[i] != len[0]) return shortest;
  return -1;
}

}  // extern "C"
