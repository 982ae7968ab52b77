#include "planner.h"
#include <algorithm>
#include <unordered_map>
#include <unordered_set>

namespace fluidml {
namespace worker {

flow::Sequence Planner::TopologicalSort(const flow::Flow &flow) {
  const size_t n = flow.nodes.size();
  std::unordered_map<const flow::Region *, size_t> producer;
  for (size_t i = 0; i < n; ++i) producer[flow.nodes[i]->output.get()] = i;
  std::vector<std::vector<size_t>> consumers(n);
  std::vector<size_t> pending(n, 0);
  for (size_t i = 0; i < n; ++i) {
    std::unordered_set<size_t> deps;
    for (const auto &r : flow.nodes[i]->inputs) {
      auto it = producer.find(r.get());
      if (it != producer.end()) deps.insert(it->second);
    }
    for (size_t d : deps) consumers[d].push_back(i);
    pending[i] = deps.size();
  }
  for (auto &c : consumers) std::sort(c.begin(), c.end());
  std::vector<size_t> waiting;
  for (size_t i = 0; i < n; ++i)
    if (pending[i] == 0) waiting.push_back(i);
  flow::Sequence seq;
  while (!waiting.empty()) {
    const size_t i = waiting.back();
    waiting.pop_back();
    seq.nodes.push_back(flow.nodes[i]);
    for (size_t c : consumers[i])
      if (--pending[c] == 0) waiting.push_back(c);
  }
  if (seq.nodes.size() != n) throw Error("the flow has a cycle or a node whose producer is missing");
  seq.regions = flow.regions;
  return seq;
}

std::vector<memory::Info> Planner::Lifetimes(const flow::Sequence &sequence, bool reference_scratch) {
  std::unordered_map<const flow::Region *, std::pair<size_t, size_t>> life;
  auto touch = [&](const flow::RegionPtr &r, size_t i) {
    if (!r->NeedMemoryAllocation()) return;
    auto it = life.find(r.get());
    if (it == life.end()) life[r.get()] = {i, i};
    else { it->second.first = std::min(it->second.first, i); it->second.second = std::max(it->second.second, i); }
  };
  for (size_t i = 0; i < sequence.nodes.size(); ++i) {
    const auto &node = sequence.nodes[i];
    for (const auto &r : node->inputs) touch(r, i);
    touch(node->output, i);
  }
  std::vector<memory::Info> infos;
  for (const auto &r : sequence.regions) {
    auto it = life.find(r.get());
    if (it == life.end()) continue;  // unused or not an arena tenant
    infos.push_back({r->name, it->second.first, it->second.second, r->meta.GetSize()});
  }
  for (size_t i = 0; i < sequence.nodes.size(); ++i) {
    const auto &node = sequence.nodes[i];
    const size_t bytes = reference_scratch ? node->reference_buffer_size : node->buffer_size;
    if (bytes > 0) infos.push_back({node->name, i, i, bytes});
  }
  return infos;
}

memory::Index Planner::Plan(const std::vector<memory::Info> &infos, MemoryPlanKind kind, size_t alignment) {
  if (kind == MemoryPlanKind::kLinear) {
    memory::PlainInfos q;
    for (auto i : infos) q.Push(std::move(i));
    return memory::LinearPlan(alignment).Run(q);
  }
  memory::GreedyInfos q;
  for (auto i : infos) q.Push(std::move(i));
  return memory::GreedyPlan(alignment).Run(q);
}

}  // namespace worker
}  // namespace fluidml
