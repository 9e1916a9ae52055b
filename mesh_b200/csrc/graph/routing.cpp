// Scheduling and routing algorithms of the graph library (host only, deterministic).
//
// The transfer planner of the reference works on a cable graph where a transfer may have to be relayed and several
// trees share thin links (rdma/mesh-graph.c: concurrent flow :561, tree packing :645, list scheduling :792, chain
// cover :1651, minimum arborescence in the tree packer).  Inside one NVSwitch node every peer is one hop away, but the
// same questions come back one level up - several nodes joined by a network, or a processor graph given by the
// caller - so the algorithms are kept, over plain edge lists:
//   * weighted longest path (critical path) of a DAG
//   * list scheduling of a DAG on P identical processors by critical-path priority
//   * minimum chain cover of a DAG (Dilworth): the fewest streams / buffers that can hold all its nodes in order
//   * minimum spanning arborescence (Chu-Liu / Edmonds): the cheapest broadcast tree from a root
//   * maximum concurrent flow (Garg-Koenemann) for commodities over capacitated edges: the largest common fraction
//     of every demand that the links can carry at once, and the flow on every edge
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <functional>
#include <limits>
#include <queue>
#include <vector>

namespace {

struct Csr {
  std::vector<int> head, adj, eid;
  Csr(int n, int m, const int* src, const int* dst) : head(n + 1, 0), adj(m), eid(m) {
    for (int e = 0; e < m; ++e) ++head[src[e] + 1];
    for (int v = 0; v < n; ++v) head[v + 1] += head[v];
    std::vector<int> pos(head.begin(), head.end() - 1);
    for (int e = 0; e < m; ++e) { adj[pos[src[e]]] = dst[e]; eid[pos[src[e]]++] = e; }
  }
};

bool topo_order(int n, int m, const int* src, const int* dst, const Csr& g, std::vector<int>& order) {
  std::vector<int> indeg(n, 0);
  for (int e = 0; e < m; ++e) ++indeg[dst[e]];
  std::priority_queue<int, std::vector<int>, std::greater<int>> q;       // smallest id first: deterministic
  for (int v = 0; v < n; ++v) if (!indeg[v]) q.push(v);
  order.clear();
  while (!q.empty()) {
    const int v = q.top(); q.pop();
    order.push_back(v);
    for (int i = g.head[v]; i < g.head[v + 1]; ++i) if (--indeg[g.adj[i]] == 0) q.push(g.adj[i]);
  }
  return (int)order.size() == n;
}

}  // namespace

extern "C" {

// tail[v] = cost[v] + the heaviest path that starts after v (so max over v is the critical path).  -1 on a cycle.
int mesh_graph_longest_path(int n, int m, const int* src, const int* dst, const double* cost, double* tail) {
  Csr g(n, m, src, dst);
  std::vector<int> order;
  if (!topo_order(n, m, src, dst, g, order)) return -1;
  for (int k = n - 1; k >= 0; --k) {
    const int v = order[k];
    double best = 0;
    for (int i = g.head[v]; i < g.head[v + 1]; ++i) best = std::max(best, tail[g.adj[i]]);
    tail[v] = cost[v] + best;
  }
  return 0;
}

// Start time and processor of every node on `procs` identical processors; ready nodes are taken by decreasing
// critical-path length (ties: smaller id).  Returns the makespan through *makespan.  -1 on a cycle.
int mesh_graph_list_schedule(int n, int m, const int* src, const int* dst, const double* cost, int procs, double* start,
                             int* proc, double* makespan) {
  if (procs < 1) return -2;
  std::vector<double> tail(n, 0.0);
  if (mesh_graph_longest_path(n, m, src, dst, cost, tail.data()) != 0) return -1;
  Csr g(n, m, src, dst);
  std::vector<int> indeg(n, 0);
  for (int e = 0; e < m; ++e) ++indeg[dst[e]];
  std::vector<double> ready_at(n, 0.0), free_at(procs, 0.0);
  auto worse = [&](int a, int b) { return tail[a] != tail[b] ? tail[a] < tail[b] : a > b; };
  std::priority_queue<int, std::vector<int>, decltype(worse)> ready(worse);
  for (int v = 0; v < n; ++v) if (!indeg[v]) ready.push(v);
  // event-driven: nodes whose predecessors are done by time t are ready; pick the earliest free processor
  std::vector<std::pair<double, int>> running;     // (finish, node)
  int done = 0;
  double t = 0, span = 0;
  while (done < n) {
    // start as many ready nodes as there are processors free at time t
    bool progressed = true;
    while (progressed && !ready.empty()) {
      progressed = false;
      int best = -1;
      for (int p = 0; p < procs; ++p) if (free_at[p] <= t && (best < 0 || free_at[p] < free_at[best])) best = p;
      if (best < 0) break;
      const int v = ready.top(); ready.pop();
      start[v] = std::max(t, ready_at[v]);
      proc[v] = best;
      free_at[best] = start[v] + cost[v];
      running.push_back({free_at[best], v});
      progressed = true;
    }
    if (running.empty()) return -1;
    // advance to the next finish
    auto it = std::min_element(running.begin(), running.end());
    t = it->first;
    const int v = it->second;
    running.erase(it);
    span = std::max(span, t);
    ++done;
    for (int i = g.head[v]; i < g.head[v + 1]; ++i) {
      const int w = g.adj[i];
      ready_at[w] = std::max(ready_at[w], t);
      if (--indeg[w] == 0) ready.push(w);
    }
  }
  *makespan = span;
  return 0;
}

// Minimum chain cover of a DAG over its reachability order: chain[v] in [0, k); returns k (or -1 on a cycle).
// Dilworth / Fulkerson: n minus a maximum matching of the bipartite graph {(u, v): v reachable from u}.
int mesh_graph_chains(int n, int m, const int* src, const int* dst, int* chain) {
  Csr g(n, m, src, dst);
  std::vector<int> order;
  if (!topo_order(n, m, src, dst, g, order)) return -1;
  // transitive closure by reverse topological order (bitsets)
  const int W = (n + 63) / 64;
  std::vector<uint64_t> reach((size_t)n * W, 0);
  for (int k = n - 1; k >= 0; --k) {
    const int v = order[k];
    for (int i = g.head[v]; i < g.head[v + 1]; ++i) {
      const int w = g.adj[i];
      reach[(size_t)v * W + w / 64] |= 1ull << (w % 64);
      for (int x = 0; x < W; ++x) reach[(size_t)v * W + x] |= reach[(size_t)w * W + x];
    }
  }
  std::vector<int> match_r(n, -1), match_l(n, -1);
  std::vector<char> seen;
  std::function<bool(int)> augment = [&](int u) {
    for (int v = 0; v < n; ++v) {
      if (!((reach[(size_t)u * W + v / 64] >> (v % 64)) & 1) || seen[v]) continue;
      seen[v] = 1;
      if (match_r[v] < 0 || augment(match_r[v])) { match_r[v] = u; match_l[u] = v; return true; }
    }
    return false;
  };
  for (int u : order) { seen.assign(n, 0); augment(u); }
  int k = 0;
  std::vector<int> id(n, -1);
  for (int v : order) {
    if (match_r[v] < 0) {                 // v starts a chain: follow the matching
      for (int x = v; x >= 0; x = match_l[x]) id[x] = k;
      ++k;
    }
  }
  for (int v = 0; v < n; ++v) chain[v] = id[v];
  return k;
}

// Minimum spanning arborescence rooted at `root` (Chu-Liu / Edmonds, O(VE)).  parent_edge[v] = index of the edge
// entering v (-1 for the root).  Returns 0 and the total weight, or -1 when some node cannot be reached.
int mesh_graph_arborescence(int n, int m, const int* src, const int* dst, const double* w, int root, int* parent_edge,
                            double* total) {
  struct E { int u, v; double w; int id; };
  std::vector<E> edges;
  for (int e = 0; e < m; ++e) if (src[e] != dst[e]) edges.push_back({src[e], dst[e], w[e], e});
  // Recursive contraction, keeping for every contracted edge the original edge it stands for and the cycle edge it
  // displaces, so that the tree can be expanded at the end.
  struct Level { std::vector<E> edges; std::vector<int> in_edge, comp; int n, root; };
  std::vector<Level> levels;
  int cur_n = n, cur_root = root;
  std::vector<E> cur = edges;
  std::vector<int> orig_of(cur.size());
  for (size_t i = 0; i < cur.size(); ++i) orig_of[i] = (int)i;
  std::vector<std::vector<int>> chosen_stack;      // per level: chosen incoming edge index (into level's edges) per node
  double sum = 0;
  for (;;) {
    std::vector<int> in(cur_n, -1);
    for (size_t i = 0; i < cur.size(); ++i) {
      const E& e = cur[i];
      if (e.v == cur_root || e.u == e.v) continue;
      if (in[e.v] < 0 || e.w < cur[in[e.v]].w || (e.w == cur[in[e.v]].w && e.id < cur[in[e.v]].id)) in[e.v] = (int)i;
    }
    for (int v = 0; v < cur_n; ++v) if (v != cur_root && in[v] < 0) return -1;
    // find cycles among the chosen edges
    std::vector<int> comp(cur_n, -1), mark(cur_n, -1);
    int comps = 0;
    for (int v = 0; v < cur_n; ++v) {
      int x = v;
      while (x != cur_root && mark[x] < 0 && comp[x] < 0) { mark[x] = v; x = cur[in[x]].u; }
      if (x != cur_root && comp[x] < 0 && mark[x] == v) {        // a new cycle through x
        for (int y = cur[in[x]].u; y != x; y = cur[in[y]].u) comp[y] = comps;
        comp[x] = comps++;
      }
    }
    Level lv{cur, in, comp, cur_n, cur_root};
    if (comps == 0) { levels.push_back(lv); break; }
    for (int v = 0; v < cur_n; ++v) if (comp[v] < 0) comp[v] = comps++;
    lv.comp = comp;
    levels.push_back(lv);
    std::vector<E> next;
    for (size_t i = 0; i < cur.size(); ++i) {
      const E& e = cur[i];
      const int cu = comp[e.u], cv = comp[e.v];
      if (cu == cv) continue;
      double wgt = e.w;
      // entering a contracted cycle costs the edge minus the cycle edge it replaces
      bool in_cycle = false;
      for (int v = 0; v < cur_n; ++v) if (v != e.v && comp[v] == cv) { in_cycle = true; break; }
      if (in_cycle && e.v != cur_root) wgt -= cur[in[e.v]].w;
      next.push_back({cu, cv, wgt, (int)i});            // id = index into this level's edges
    }
    cur_root = comp[cur_root];
    cur_n = comps;
    cur = next;
  }
  // expand from the innermost level outwards
  std::vector<int> pick = levels.back().in_edge;        // per node of the last level: chosen edge index at that level
  for (int L = (int)levels.size() - 1; L > 0; --L) {
    const Level& outer = levels[L - 1];
    std::vector<int> outer_pick = outer.in_edge;         // default: the cycle edges
    for (int c = 0; c < levels[L].n; ++c) {
      if (c == levels[L].root || pick[c] < 0) continue;
      const int oe = levels[L].edges[pick[c]].id;         // edge index at the outer level
      outer_pick[outer.edges[oe].v] = oe;                 // it enters this node, displacing its cycle edge
    }
    pick = outer_pick;
  }
  for (int v = 0; v < n; ++v) parent_edge[v] = -1;
  for (int v = 0; v < n; ++v) {
    if (v == root) continue;
    const E& e = levels[0].edges[pick[v]];
    parent_edge[v] = e.id;
    sum += w[e.id];
  }
  *total = sum;
  return 0;
}

// Maximum concurrent flow (Garg-Koenemann with Fleischer's phases): commodities (s_i, t_i, demand_i) over directed
// edges with capacities.  Returns lambda (every demand can be routed at that fraction at once, within 1 - 3 eps of
// the optimum) and flow[k * m + e] = flow of commodity k on edge e at that lambda.  -1 if a commodity has no path.
double mesh_graph_concurrent_flow(int n, int m, const int* src, const int* dst, const double* cap, int k, const int* s,
                                  const int* t, const double* demand, double eps, double* flow) {
  Csr g(n, m, src, dst);
  const double delta = std::pow((1 + eps) / std::pow((1 + eps) * m, 1.0 / eps), 1.0);
  std::vector<double> len(m);
  for (int e = 0; e < m; ++e) len[e] = delta / cap[e];
  for (long long i = 0; i < (long long)k * m; ++i) flow[i] = 0;
  auto total_len = [&] { double d = 0; for (int e = 0; e < m; ++e) d += len[e] * cap[e]; return d; };
  std::vector<double> dist(n);
  std::vector<int> via(n);
  int phases = 0;
  while (total_len() < 1.0 && phases < 100000) {
    for (int c = 0; c < k; ++c) {
      double left = demand[c];
      while (left > 1e-15 && total_len() < 1.0) {
        // shortest path under the current lengths (Dijkstra)
        std::fill(dist.begin(), dist.end(), std::numeric_limits<double>::infinity());
        std::fill(via.begin(), via.end(), -1);
        using QE = std::pair<double, int>;
        std::priority_queue<QE, std::vector<QE>, std::greater<QE>> q;
        dist[s[c]] = 0; q.push({0, s[c]});
        while (!q.empty()) {
          auto [d, v] = q.top(); q.pop();
          if (d > dist[v]) continue;
          for (int i = g.head[v]; i < g.head[v + 1]; ++i) {
            const int w2 = g.adj[i], e = g.eid[i];
            if (dist[v] + len[e] < dist[w2]) { dist[w2] = dist[v] + len[e]; via[w2] = e; q.push({dist[w2], w2}); }
          }
        }
        if (via[t[c]] < 0 && s[c] != t[c]) return -1;
        double bottleneck = left;
        for (int v = t[c]; v != s[c]; v = src[via[v]]) bottleneck = std::min(bottleneck, cap[via[v]]);
        for (int v = t[c]; v != s[c]; v = src[via[v]]) {
          const int e = via[v];
          flow[(long long)c * m + e] += bottleneck;
          len[e] *= 1 + eps * bottleneck / cap[e];
        }
        left -= bottleneck;
      }
    }
    ++phases;
  }
  // scale so that no capacity is exceeded: the flow routed is `phases` demands, over capacity by log_{1+eps}(1/delta)
  const double scale = std::log((1 + eps) / delta) / std::log(1 + eps);
  double lambda = std::numeric_limits<double>::infinity();
  for (long long i = 0; i < (long long)k * m; ++i) flow[i] /= scale;
  for (int c = 0; c < k; ++c) {
    double out = 0;
    for (int e = 0; e < m; ++e) {
      if (src[e] == s[c]) out += flow[(long long)c * m + e];
      if (dst[e] == s[c]) out -= flow[(long long)c * m + e];
    }
    lambda = std::min(lambda, out / demand[c]);
  }
  // report flows at exactly lambda of every demand
  for (int c = 0; c < k; ++c) {
    double out = 0;
    for (int e = 0; e < m; ++e) {
      if (src[e] == s[c]) out += flow[(long long)c * m + e];
      if (dst[e] == s[c]) out -= flow[(long long)c * m + e];
    }
    const double f = out > 0 ? lambda * demand[c] / out : 0;
    for (int e = 0; e < m; ++e) flow[(long long)c * m + e] *= f;
  }
  return lambda;
}

}  // extern "C"
