// worker::Planner -- execution order, tensor lifetimes and the arena plan
// (reference: src/worker/planner.cpp:22-108 TopologicalSort, :236-293 lifetimes + plan).
#pragma once
#include "flow.h"
#include "memory.h"

namespace fluidml {
namespace worker {

enum class MemoryPlanKind { kLinear, kGreedy };

class Planner {
public:
  // Kahn's algorithm with a LIFO worklist, as the reference (planner.cpp:74-95), made
  // deterministic: the worklist is seeded in node order and consumers become ready in node
  // order (the reference's order depends on unordered_map iteration, flow.cpp:78-85).
  // A node also waits for the producer of a graph OUTPUT it reads back.
  static flow::Sequence TopologicalSort(const flow::Flow &flow);

  // One Info per inner region (first producer/consumer index .. last, bytes = meta size) in
  // region order, then one per node with scratch, lifetime [i, i] (planner.cpp:261-291).
  // `reference_scratch` selects the reference kernels' scratch sizes (Softmax / LayerNorm
  // row buffers, padded conv input) instead of this back end's (split-K partial tiles).
  static std::vector<memory::Info> Lifetimes(const flow::Sequence &sequence, bool reference_scratch);

  static memory::Index Plan(const std::vector<memory::Info> &infos, MemoryPlanKind kind,
                            size_t alignment);
};

}  // namespace worker
}  // namespace fluidml
