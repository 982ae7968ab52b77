// worker::Converter -- graph::Graph -> flow::Flow (reference: include/worker/converter.h,
// src/worker/converter.cpp:114-352).
#pragma once
#include "flow.h"
#include "graph.h"

namespace fluidml {
namespace worker {

class Converter {
public:
  static flow::Flow Run(const graph::Graph &graph);
};

}  // namespace worker
}  // namespace fluidml
