// Flow-level fusion passes.  The reference defines three graph fusions
// (src/optimization/graph/{add_div_erf_add_mul_fusion,gather_add_fusion,
// unsqueeze_sub_mul_fusion}.cpp) that its pipeline never runs
// (src/optimization/graph/manager.cpp:30-34 has no caller); here those patterns and the
// GEMM / LayerNorm / Softmax epilogue fusions run before planning.
#pragma once
#include "flow.h"

namespace fluidml {
namespace worker {

class FusionPasses {
public:
  // Rewrites `flow` in place; returns the number of nodes removed.
  static size_t Run(flow::Flow &flow);
};

}  // namespace worker
}  // namespace fluidml
