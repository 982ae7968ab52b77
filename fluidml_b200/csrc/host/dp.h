// Dynamic-programming layout search (reference: src/evaluation/dp.cpp, eval.cpp) with a GPU
// cost model in place of measured CPU kernel times.
#pragma once
#include "flow.h"
#include "json.h"
#include <map>
#include <unordered_map>

namespace fluidml {
namespace evaluation {

class DynamicProgrammingPlan {
public:
  bool HasLayout(const std::string &name) const { return plan_.count(name) != 0; }
  const std::vector<size_t> &GetLayout(const std::string &name) const { return plan_.at(name); }
  // First writer wins, as unordered_map::insert does in the reference (dp.cpp:705-729, :861-875).
  void Insert(const std::string &name, const std::vector<size_t> &layout) { plan_.insert({name, layout}); }
  json::Value ToJson() const;
  const std::map<std::string, std::vector<size_t>> &All() const { return plan_; }

private:
  std::map<std::string, std::vector<size_t>> plan_;
};

// cost(kernel kind + parameters, operand shapes, operand layouts, output layout) in
// nanoseconds on the GPU, memoised per distinct key (reference KernelEval: measured CPU
// nanoseconds memoised per layout tuple, eval.cpp:64-100, :261-302).
class CostModel {
public:
  CostModel(bool constant_cost, int gemm_precision) : constant_(constant_cost), precision_(gemm_precision) {}
  size_t GetTimeCost(const flow::Node &node, const std::vector<std::vector<size_t>> &input_layouts,
                     const std::vector<size_t> &output_layout);
  json::Value ToJson() const;

private:
  bool constant_;
  int precision_;
  struct Record { std::string kernel; std::vector<std::vector<int64_t>> shapes; std::vector<std::vector<size_t>> layouts; size_t cost; };
  std::unordered_map<std::string, size_t> memo_;
  std::vector<Record> records_;
};

class DynamicProgrammingTable {
public:
  DynamicProgrammingTable(bool constant_cost, int gemm_precision) : cost_(constant_cost, gemm_precision) {}
  DynamicProgrammingPlan Run(const flow::Flow &flow);
  json::Value ToJson() const;

private:
  CostModel cost_;
};

}  // namespace evaluation
}  // namespace fluidml
