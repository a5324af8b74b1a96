// Index-based graph IR: nodes are uids, edges reference a layer slot plus
// producer / consumer node indices. It provides what the Python executor and
// the pipeline runtime need from a graph without owning any tensor: Kahn
// ordering, uid generation, degree queries, and the ratio partitioner that
// cuts the sorted edge list into pipeline stages.
//
// Behavioural reference: src/nn/graph.cpp:111-189,360-367 (sort, uids) and
// src/partitioner/graph_partitioner.cpp:101-260 (boundaries, largest-remainder
// rounding).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace tnnb {

struct IrEdge {
  uint64_t layer = 0;
  std::vector<uint64_t> producers;
  std::vector<uint64_t> consumers;
};

struct GraphIR {
  std::vector<std::string> nodes;
  std::vector<uint64_t> inputs;
  std::vector<uint64_t> outputs;
  std::vector<IrEdge> edges;
  uint64_t uid_counter = 0;

  uint64_t add_node(const std::string& uid);  // throws on duplicates
  uint64_t add_auto_node();                   // "node_<k>", skipping used names
  void rename_node(uint64_t idx, const std::string& uid);
  uint64_t add_edge(uint64_t layer, std::vector<uint64_t> producers, std::vector<uint64_t> consumers);
  int64_t find(const std::string& uid) const;

  // FIFO Kahn order over edges. Returns the permutation (new position -> old
  // edge index) and reorders `edges`; nodes are reordered as: never-produced
  // nodes in creation order, then consumers in sorted-edge order. `node_perm`
  // (new -> old) is filled when non-null. Throws on a cycle.
  std::vector<uint64_t> sort(std::vector<uint64_t>* node_perm = nullptr);

  int in_degree(uint64_t node) const;
  int out_degree(uint64_t node) const;
};

struct IrPartition {
  GraphIR graph;                       // node/edge indices local to the stage
  std::vector<std::string> input_uids;   // consumed here, produced earlier
  std::vector<std::string> output_uids;  // produced here and needed later (or never consumed)
  uint64_t start_layer = 0;            // offset in the sorted edge list
  uint64_t layer_count = 0;
  std::vector<uint64_t> edge_ids;      // indices into the full graph's sorted edges
};

// Largest-remainder split of `total` edges by positive ratios; throws if a
// stage would be empty.
std::vector<uint64_t> resolve_layer_counts(const std::vector<double>& ratios, uint64_t total);

// The graph must already be sorted. Edge `layer` ids are kept as-is so that
// stages keep referring to the caller's layer objects.
std::vector<IrPartition> partition_graph(const GraphIR& g, const std::vector<double>& ratios);

}  // namespace tnnb
