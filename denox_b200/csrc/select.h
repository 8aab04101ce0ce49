// Hypergraph of candidate dispatches and the schedule search over it (select.cu).
#pragma once
#include <stdint.h>
#include <vector>

namespace dnxcu {

struct HyperEdge {
  std::vector<int> src;  // tensors the dispatch reads
  std::vector<int> dst;  // tensors it writes (one, or two for a conv with a pooled second output)
  double weight = 0.0;   // latency in ms, or the sentinel for "never benchmarked"
  int dispatches = 1;    // kernels the edge stands for
  int payload = -1;      // caller's index
};

struct HyperGraph {
  int n_nodes = 0;
  std::vector<HyperEdge> edges;
};

// 1 hour in ms: the weight of an edge the database has no timing for (selection.cpp:21).
constexpr double kUnbenchmarkedMs = 3600000.0;

// Cheapest set of edges that derives `outputs` from `inputs`, in an order in which they can fire.
// false: the outputs cannot be derived (or the graph has a cycle).
bool minimum_cost_subgraph(const HyperGraph &g, const std::vector<int> &inputs, const std::vector<int> &outputs,
                           std::vector<int> &chosen, double *cost);
// Of parallel edges only the cheapest stays.
void prune_duplicate_edges(HyperGraph &g);
// Only edges of sub-graphs with the minimal number of dispatches stay.  false: outputs not derivable.
bool prune_topological(HyperGraph &g, const std::vector<int> &inputs, const std::vector<int> &outputs);

}  // namespace dnxcu
