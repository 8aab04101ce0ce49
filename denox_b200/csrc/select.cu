// Schedule selection over a hypergraph of candidate dispatches.
//
// Nodes are tensors, a hyperedge is one way to compute its destination tensor(s) from its source tensors (one
// fused or un-fused dispatch of one kernel variant), weighted with the latency the benchmark database holds for
// it.  The schedule is the cheapest set of edges that derives the outputs from the inputs.  This restates, on a
// plain adjacency structure, what the reference does in
//   common/src/denox/algorithm/minimum_const_subgraph.hpp:45-353   (branch and bound over the open frontier,
//       lower bound h(v) = min over incoming edges of w(e) + max over sources of h(u), cheapest edge first,
//       states memoised on (done restricted to the ancestors of the open set, open set)),
//   compiler/src/denox/compiler/dce/prune_topological.cpp:86-152    (before the search: only edges that belong
//       to a sub-graph with the minimal NUMBER of dispatches survive),
//   compiler/src/denox/compiler/selection/selection.cpp:21,116      (1 hour for an edge the database has no
//       timing for).
// One extension: an edge may have two destinations (a conv that writes its full resolution output and the 2x2
// max pooled one); firing it makes both available.
#include "select.h"
#include <algorithm>
#include <functional>
#include <map>
#include <unordered_map>

namespace dnxcu {
namespace {

using Bits = std::vector<uint64_t>;
inline void bset(Bits &b, int i, bool v) {
  if (v) b[i >> 6] |= 1ull << (i & 63);
  else b[i >> 6] &= ~(1ull << (i & 63));
}
inline bool bget(const Bits &b, int i) { return (b[i >> 6] >> (i & 63)) & 1ull; }

struct Solver {
  const HyperGraph &g;
  int N, M;
  std::vector<std::vector<int>> incoming;  // per node: edges that produce it
  std::vector<int> topo;                   // nodes, sources before destinations
  std::vector<double> h, he;
  std::vector<Bits> anc;
  bool ok = true;

  explicit Solver(const HyperGraph &gr) : g(gr), N(gr.n_nodes), M((int)gr.edges.size()) {
    incoming.assign(N, {});
    for (int e = 0; e < M; ++e)
      for (int d : g.edges[e].dst) incoming[d].push_back(e);
    // topological order of the nodes (Kahn over "all sources of some producing edge known")
    std::vector<int> state(N, 0);
    std::function<bool(int)> visit = [&](int v) -> bool {
      if (state[v] == 2) return true;
      if (state[v] == 1) return false;  // cycle
      state[v] = 1;
      for (int e : incoming[v])
        for (int u : g.edges[e].src)
          if (!visit(u)) return false;
      state[v] = 2;
      topo.push_back(v);
      return true;
    };
    for (int v = 0; v < N && ok; ++v) ok = visit(v);
    if (!ok) return;
    const int words = (N + 63) / 64;
    h.assign(N, 0.0);
    anc.assign(N, Bits(words, 0));
    for (int v : topo) {
      bool first = true;
      double best = 0.0;
      for (int e : incoming[v]) {
        double mx = 0.0;
        for (int u : g.edges[e].src) {
          mx = std::max(mx, h[u]);
          bset(anc[v], u, true);
          for (int w = 0; w < words; ++w) anc[v][w] |= anc[u][w];
        }
        const double cand = g.edges[e].weight + mx;
        if (first || cand < best) {
          best = cand;
          first = false;
        }
      }
      h[v] = best;
    }
    he.assign(M, 0.0);
    for (int e = 0; e < M; ++e) {
      double mx = 0.0;
      for (int u : g.edges[e].src) mx = std::max(mx, h[u]);
      he[e] = g.edges[e].weight + mx;
    }
  }

  struct Key {
    Bits done;
    std::vector<int> open;
    bool operator==(const Key &o) const { return open == o.open && done == o.done; }
  };
  struct KeyHash {
    size_t operator()(const Key &k) const {
      uint64_t x = 0xE6C6DAE8F56DA2A9ull;
      auto mix = [&](uint64_t v) { x ^= v + 0x9E3779B97F4A7C15ull + (x << 6) + (x >> 2); };
      for (int v : k.open) mix((uint64_t)v);
      for (uint64_t w : k.done) mix(w);
      return (size_t)x;
    }
  };

  bool solve(const std::vector<int> &inputs, const std::vector<int> &outputs, std::vector<int> &best_edges,
             double &best_cost) {
    if (!ok) return false;
    const int words = (N + 63) / 64;
    Bits done(words, 0);
    for (int v : inputs) bset(done, v, true);
    std::vector<int> open;
    for (int v : outputs)
      if (!bget(done, v)) open.push_back(v);
    std::sort(open.begin(), open.end());
    open.erase(std::unique(open.begin(), open.end()), open.end());
    std::unordered_map<Key, double, KeyHash> memo;
    bool have = false;
    std::vector<int> cur;
    std::function<void(double)> rec = [&](double cost) {
      if (have && cost >= best_cost) return;
      if (open.empty()) {
        have = true;
        best_cost = cost;
        best_edges = cur;
        return;
      }
      Key key;
      key.open = open;
      key.done.assign(words, 0);
      for (int v : open)
        for (int w = 0; w < words; ++w) key.done[w] |= anc[v][w];
      for (int w = 0; w < words; ++w) key.done[w] &= done[w];
      auto it = memo.find(key);
      if (it != memo.end()) {
        if (it->second <= cost) return;
        it->second = cost;
      } else {
        memo.emplace(std::move(key), cost);
      }
      // next node to derive: the one that is cheapest to reach (keeps the frontier small on U-Nets)
      int v = open[0];
      for (int u : open)
        if (h[u] < h[v]) v = u;
      std::vector<int> inc = incoming[v];
      std::stable_sort(inc.begin(), inc.end(), [&](int a, int b) { return he[a] < he[b]; });
      for (int e : inc) {
        // firing e makes all its destinations available and asks for its sources
        std::vector<int> newly_done, added;
        for (int d : g.edges[e].dst)
          if (!bget(done, d)) {
            bset(done, d, true);
            newly_done.push_back(d);
          }
        std::vector<int> saved_open = open;
        open.erase(std::remove_if(open.begin(), open.end(), [&](int x) { return bget(done, x); }), open.end());
        for (int u : g.edges[e].src)
          if (!bget(done, u) && !std::binary_search(open.begin(), open.end(), u))
            open.insert(std::lower_bound(open.begin(), open.end(), u), u);
        cur.push_back(e);
        rec(cost + g.edges[e].weight);
        cur.pop_back();
        open.swap(saved_open);
        for (int d : newly_done) bset(done, d, false);
      }
    };
    rec(0.0);
    return have;
  }
};

// Orders the chosen edges so that every edge's sources are available when it fires.
bool firing_order(const HyperGraph &g, const std::vector<int> &inputs, std::vector<int> &edges) {
  std::vector<char> avail(g.n_nodes, 0);
  for (int v : inputs) avail[v] = 1;
  std::vector<int> order;
  std::vector<char> used(edges.size(), 0);
  for (size_t round = 0; round < edges.size(); ++round) {
    bool progress = false;
    for (size_t i = 0; i < edges.size(); ++i) {
      if (used[i]) continue;
      const HyperEdge &e = g.edges[edges[i]];
      bool ready = true;
      for (int u : e.src) ready = ready && avail[u];
      if (!ready) continue;
      used[i] = 1;
      for (int d : e.dst) avail[d] = 1;
      order.push_back(edges[i]);
      progress = true;
    }
    if (!progress) break;
  }
  if (order.size() != edges.size()) return false;
  edges.swap(order);
  return true;
}

}  // namespace

bool minimum_cost_subgraph(const HyperGraph &g, const std::vector<int> &inputs, const std::vector<int> &outputs,
                           std::vector<int> &chosen, double *cost) {
  for (const HyperEdge &e : g.edges) {
    if (e.dst.empty()) return false;
    for (int v : e.src)
      if (v < 0 || v >= g.n_nodes) return false;
    for (int v : e.dst)
      if (v < 0 || v >= g.n_nodes) return false;
  }
  for (int v : inputs)
    if (v < 0 || v >= g.n_nodes) return false;
  for (int v : outputs)
    if (v < 0 || v >= g.n_nodes) return false;
  Solver s(g);
  double c = 0.0;
  chosen.clear();
  if (!s.solve(inputs, outputs, chosen, c)) return false;
  if (!firing_order(g, inputs, chosen)) return false;
  if (cost) *cost = c;
  return true;
}

// Parallel edges (same sources, same destinations): only the cheapest can ever be chosen.  The reference computes
// this pruned graph too (selection.cpp:129-131) but then searches the un-pruned one (selection.cpp:135-137); the
// result is the same, the search is shorter.
void prune_duplicate_edges(HyperGraph &g) {
  std::map<std::pair<std::vector<int>, std::vector<int>>, int> best;
  for (int e = 0; e < (int)g.edges.size(); ++e) {
    std::vector<int> s = g.edges[e].src, d = g.edges[e].dst;
    std::sort(s.begin(), s.end());
    std::sort(d.begin(), d.end());
    auto key = std::make_pair(s, d);
    auto it = best.find(key);
    if (it == best.end() || g.edges[e].weight < g.edges[it->second].weight) best[key] = e;
  }
  std::vector<HyperEdge> kept;
  std::vector<int> ids;
  for (auto &kv : best) ids.push_back(kv.second);
  std::sort(ids.begin(), ids.end());
  for (int e : ids) kept.push_back(g.edges[e]);
  g.edges.swap(kept);
}

// Keeps the edges that belong to at least one sub-graph with the minimal number of dispatches
// (prune_topological.cpp:86-152).  Parallel edges count as one topological edge with the smallest dispatch count
// among them; parallel edges with more dispatches than that are dropped.  An edge is part of some optimal
// sub-graph exactly when making it half a dispatch cheaper makes the optimum half a dispatch cheaper.
bool prune_topological(HyperGraph &g, const std::vector<int> &inputs, const std::vector<int> &outputs) {
  std::map<std::pair<std::vector<int>, std::vector<int>>, std::vector<int>> groups;
  for (int e = 0; e < (int)g.edges.size(); ++e) {
    std::vector<int> s = g.edges[e].src, d = g.edges[e].dst;
    std::sort(s.begin(), s.end());
    std::sort(d.begin(), d.end());
    groups[std::make_pair(s, d)].push_back(e);
  }
  HyperGraph t;
  t.n_nodes = g.n_nodes;
  std::vector<std::vector<int>> members;
  for (auto &kv : groups) {
    int mn = g.edges[kv.second[0]].dispatches;
    for (int e : kv.second) mn = std::min(mn, g.edges[e].dispatches);
    std::vector<int> keep;
    for (int e : kv.second)
      if (g.edges[e].dispatches == mn) keep.push_back(e);
    HyperEdge te;
    te.src = kv.first.first;
    te.dst = kv.first.second;
    te.weight = (double)mn;
    te.dispatches = mn;
    te.payload = (int)members.size();
    t.edges.push_back(te);
    members.push_back(keep);
  }
  std::vector<int> chosen;
  double best = 0.0;
  if (!minimum_cost_subgraph(t, inputs, outputs, chosen, &best)) return false;
  std::vector<char> keep_edge(g.edges.size(), 0);
  for (int te = 0; te < (int)t.edges.size(); ++te) {
    HyperGraph probe = t;
    probe.edges[te].weight -= 0.5;
    double c = 0.0;
    std::vector<int> ch;
    if (minimum_cost_subgraph(probe, inputs, outputs, ch, &c) && c <= best - 0.25)
      for (int e : members[te]) keep_edge[e] = 1;
  }
  std::vector<HyperEdge> kept;
  for (int e = 0; e < (int)g.edges.size(); ++e)
    if (keep_edge[e]) kept.push_back(g.edges[e]);
  g.edges.swap(kept);
  return true;
}

}  // namespace dnxcu
