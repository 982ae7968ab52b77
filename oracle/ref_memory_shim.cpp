// C-ABI shim over the reference's own memory planner, compiled together with the reference
// sources where they lie (src/structure/memory/{greedy,linear,info,index}.cpp of
// sgjzfzzf/FluidML; these four files need nothing but the C++ standard library).
// TEST INFRASTRUCTURE ONLY: used to check this repository's planner port against the
// reference's actual code on the same lifetime tables.
#include "structure/memory/greedy.h"
#include "structure/memory/index.h"
#include "structure/memory/info.h"
#include "structure/memory/linear.h"
#include <cstddef>
#include <memory>
#include <string>

extern "C" int ref_memory_plan(int greedy, int n, const char *const *names, const size_t *start,
                               const size_t *end, const size_t *size, size_t *offset_out,
                               size_t *maximum_out) {
  using namespace fluidml::memory;
  std::unique_ptr<Infos> infos;
  std::unique_ptr<Plan> plan;
  if (greedy) {
    infos = std::make_unique<GreedyInfos>();
    plan = std::make_unique<GreedyPlan>();
  } else {
    infos = std::make_unique<PlainInfos>();
    plan = std::make_unique<LinearPlan>();
  }
  for (int i = 0; i < n; ++i) infos->Push(Info(std::string(names[i]), start[i], end[i], size[i]));
  Index index = plan->Run(*infos);
  for (int i = 0; i < n; ++i) offset_out[i] = index.Get(names[i]);
  *maximum_out = index.GetMaximum();
  return 0;
}
