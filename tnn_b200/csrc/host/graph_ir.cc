#include "graph_ir.h"

#include <algorithm>
#include <cmath>
#include <deque>
#include <numeric>
#include <stdexcept>
#include <unordered_map>
#include <unordered_set>

namespace tnnb {

int64_t GraphIR::find(const std::string& uid) const {
  for (size_t i = 0; i < nodes.size(); ++i)
    if (nodes[i] == uid) return static_cast<int64_t>(i);
  return -1;
}

uint64_t GraphIR::add_node(const std::string& uid) {
  if (find(uid) >= 0) throw std::runtime_error("duplicate node uid: " + uid);
  nodes.push_back(uid);
  return nodes.size() - 1;
}

uint64_t GraphIR::add_auto_node() {
  for (;;) {
    std::string uid = "node_" + std::to_string(uid_counter++);
    if (find(uid) < 0) {
      nodes.push_back(uid);
      return nodes.size() - 1;
    }
  }
}

void GraphIR::rename_node(uint64_t idx, const std::string& uid) {
  if (idx >= nodes.size()) throw std::out_of_range("node index");
  const int64_t other = find(uid);
  if (other >= 0 && static_cast<uint64_t>(other) != idx) throw std::runtime_error("duplicate node uid: " + uid);
  nodes[idx] = uid;
}

uint64_t GraphIR::add_edge(uint64_t layer, std::vector<uint64_t> producers, std::vector<uint64_t> consumers) {
  for (uint64_t n : producers)
    if (n >= nodes.size()) throw std::out_of_range("edge producer is not a node");
  for (uint64_t n : consumers)
    if (n >= nodes.size()) throw std::out_of_range("edge consumer is not a node");
  edges.push_back({layer, std::move(producers), std::move(consumers)});
  return edges.size() - 1;
}

int GraphIR::in_degree(uint64_t node) const {
  int d = 0;
  for (const auto& e : edges) d += static_cast<int>(std::count(e.consumers.begin(), e.consumers.end(), node));
  return d;
}

int GraphIR::out_degree(uint64_t node) const {
  int d = 0;
  for (const auto& e : edges) d += static_cast<int>(std::count(e.producers.begin(), e.producers.end(), node));
  return d;
}

std::vector<uint64_t> GraphIR::sort(std::vector<uint64_t>* node_perm) {
  const size_t ne = edges.size(), nn = nodes.size();
  std::vector<char> produced(nn, 0);
  for (const auto& e : edges)
    for (uint64_t c : e.consumers) produced[c] = 1;
  std::vector<std::vector<uint64_t>> dependents(nn);
  for (size_t i = 0; i < ne; ++i)
    for (uint64_t p : edges[i].producers) dependents[p].push_back(i);
  std::vector<int> pending(ne, 0);
  std::deque<uint64_t> ready;
  for (size_t i = 0; i < ne; ++i) {
    for (uint64_t p : edges[i].producers) pending[i] += produced[p] ? 1 : 0;
    if (pending[i] == 0) ready.push_back(i);
  }
  std::vector<uint64_t> order;
  order.reserve(ne);
  while (!ready.empty()) {
    const uint64_t i = ready.front();
    ready.pop_front();
    order.push_back(i);
    for (uint64_t c : edges[i].consumers)
      for (uint64_t j : dependents[c])
        if (--pending[j] == 0) ready.push_back(j);
  }
  if (order.size() != ne) throw std::runtime_error("Graph contains a cycle; topological sort failed");

  std::vector<IrEdge> sorted;
  sorted.reserve(ne);
  for (uint64_t i : order) sorted.push_back(edges[i]);

  std::vector<uint64_t> nperm;  // new -> old
  std::vector<char> placed(nn, 0);
  for (size_t n = 0; n < nn; ++n)
    if (!produced[n]) {
      nperm.push_back(n);
      placed[n] = 1;
    }
  for (const auto& e : sorted)
    for (uint64_t c : e.consumers)
      if (!placed[c]) {
        placed[c] = 1;
        nperm.push_back(c);
      }
  std::vector<uint64_t> inv(nn, 0);
  for (size_t i = 0; i < nperm.size(); ++i) inv[nperm[i]] = i;
  std::vector<std::string> new_nodes(nn);
  for (size_t i = 0; i < nn; ++i) new_nodes[i] = nodes[nperm[i]];
  for (auto& e : sorted) {
    for (auto& p : e.producers) p = inv[p];
    for (auto& c : e.consumers) c = inv[c];
  }
  for (auto& i : inputs) i = inv[i];
  for (auto& o : outputs) o = inv[o];
  nodes = std::move(new_nodes);
  edges = std::move(sorted);
  if (node_perm) *node_perm = nperm;
  return order;
}

std::vector<uint64_t> resolve_layer_counts(const std::vector<double>& ratios, uint64_t total) {
  if (ratios.empty()) {
    if (total == 0) return {};
    throw std::runtime_error("partitioner requires at least one partition ratio");
  }
  if (total == 0) throw std::runtime_error("partitioner cannot apply partition ratios to an empty graph");
  double sum = 0.0;
  for (double r : ratios) {
    if (!std::isfinite(r) || r <= 0.0) throw std::runtime_error("partition ratios must be finite and greater than zero");
    sum += r;
  }
  const size_t k = ratios.size();
  std::vector<uint64_t> counts(k);
  std::vector<std::pair<double, size_t>> frac(k);
  uint64_t assigned = 0;
  for (size_t i = 0; i < k; ++i) {
    const double exact = ratios[i] / sum * static_cast<double>(total);
    counts[i] = static_cast<uint64_t>(std::floor(exact));
    frac[i] = {exact - static_cast<double>(counts[i]), i};
    assigned += counts[i];
  }
  std::stable_sort(frac.begin(), frac.end(), [](const auto& a, const auto& b) {
    return a.first != b.first ? a.first > b.first : a.second < b.second;
  });
  for (uint64_t i = 0; i < total - assigned; ++i) ++counts[frac[i % k].second];
  for (uint64_t c : counts)
    if (c == 0) throw std::runtime_error("partition ratios resolve to an empty partition for this graph");
  return counts;
}

std::vector<IrPartition> partition_graph(const GraphIR& g, const std::vector<double>& ratios) {
  const std::vector<uint64_t> counts = resolve_layer_counts(ratios, g.edges.size());
  std::vector<IrPartition> parts;
  uint64_t offset = 0;
  for (uint64_t cnt : counts) {
    IrPartition part;
    part.start_layer = offset;
    part.layer_count = cnt;
    std::unordered_map<uint64_t, uint64_t> local;  // full node idx -> local idx
    std::vector<uint64_t> order;                   // local -> full
    auto ensure = [&](uint64_t n) {
      auto it = local.find(n);
      if (it != local.end()) return it->second;
      const uint64_t li = part.graph.add_node(g.nodes[n]);
      local.emplace(n, li);
      order.push_back(n);
      return li;
    };
    std::unordered_set<uint64_t> produced, consumed, later;
    for (uint64_t e = offset; e < offset + cnt; ++e) {
      const IrEdge& ed = g.edges[e];
      std::vector<uint64_t> ps, cs;
      for (uint64_t p : ed.producers) {
        consumed.insert(p);
        ps.push_back(ensure(p));
      }
      for (uint64_t c : ed.consumers) {
        produced.insert(c);
        cs.push_back(ensure(c));
      }
      part.graph.add_edge(ed.layer, ps, cs);
      part.edge_ids.push_back(e);
    }
    for (uint64_t e = offset + cnt; e < g.edges.size(); ++e)
      for (uint64_t p : g.edges[e].producers)
        if (produced.count(p)) later.insert(p);
    for (uint64_t n : order) {
      const bool prod = produced.count(n) > 0, cons = consumed.count(n) > 0;
      if (cons && !prod) {
        part.input_uids.push_back(g.nodes[n]);
        part.graph.inputs.push_back(local[n]);
      }
      if (prod && (!cons || later.count(n))) {
        part.output_uids.push_back(g.nodes[n]);
        part.graph.outputs.push_back(local[n]);
      }
    }
    parts.push_back(std::move(part));
    offset += cnt;
  }
  return parts;
}

}  // namespace tnnb
