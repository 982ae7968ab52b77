// Lowering of a planned flow to a device program and its execution:
//   Lowering   which regions alias which (no-op reshapes, transposes that are pure stride
//              permutations), per-node scratch sizes;
//   Builder    replaces GeneralBuilder (src/worker/builder.cpp:149-608): uploads constants
//              physically permuted to their layouts (:273-361), binds every region to the
//              arena / weight blob / interface buffers, and walks the sequence calling
//              kernel->Launch to record the launch plan;
//   Runner     replaces Lower + Runner (src/worker/lower.cpp:37-59, runner.cpp:56-120):
//              captures the launch plan into a CUDA graph once; per Invoke copies inputs in,
//              replays the graph `epoch` times between two events, copies outputs out and
//              returns the average nanoseconds per replay.
#pragma once
#include "kernel.h"
#include "memory.h"
#include <map>
#include <memory>
#include <string>
#include <unordered_map>

namespace fluidml {
namespace worker {

struct Options {
  int device = 0;
  int gemm_precision = FML_GEMM_AUTO;
  bool fusion = true;
  bool cuda_graph = true;
  size_t alignment = 256;
  bool dp_constant_cost = false;
  bool autotune = true;  // tune GEMM tile / split-K choices on the device at Compile
  bool weight_prefetch = true;  // GEMMs ask L2 to fetch the next GEMM's weights while they run
  // Runs of constant-weight GEMM (+ LayerNorm) and attention nodes over 128 rows become one
  // resident program each (one persistent kernel, fml_resident_*) instead of one launch per
  // node.  Off by default: on this part a dependent exchange through L2 inside one kernel costs
  // about what a kernel boundary costs, and the separate kernels are the faster plan.
  bool resident = false;
  // Directory of the plan cache (empty: none).  A compiled model leaves its DP layouts and the
  // tuned GEMM tiles there, keyed by a hash of the model bytes and the options that shape the
  // plan, so that compiling the same model again skips the layout search and the on-device tuning.
  std::string plan_cache;
  // node name -> (tile_n, split_k): read by the Builder as presets, filled with what it tuned
  std::shared_ptr<std::map<std::string, std::pair<int, int>>> gemm_tiles;
};

// region -> the region whose memory it shares (itself when it owns memory).
using AliasMap = std::unordered_map<const flow::Region *, flow::RegionPtr>;

class Lowering {
public:
  // Walks the sequence; a single-input node whose kernel can express its output as a view of
  // its input (GetView), and whose output is an inner region, shares its input's memory: the
  // output region is marked as a view with explicit strides and offset.
  static AliasMap ComputeAliases(const flow::Sequence &sequence, const kernel::KernelOptions &ko);
  // Fills node->buffer_size with what each node's kernel asks for.  Uses aligned placeholder
  // addresses: planned offsets are multiples of the alignment, so the real operands take the
  // same path.
  static void ComputeScratch(const flow::Sequence &sequence, const kernel::KernelOptions &ko);
  // Lifetimes with aliases merged into their owners.
  static std::vector<memory::Info> Lifetimes(const flow::Sequence &sequence, const AliasMap &aliases);
};

struct IoBinding {
  std::string name;
  void *device = nullptr;
  size_t bytes = 0;
};

struct Program {
  std::vector<kernel::Launch> launches;
  std::vector<IoBinding> inputs, outputs;
  void *arena = nullptr, *weights = nullptr, *io = nullptr;
  size_t arena_bytes = 0, weight_bytes = 0, io_bytes = 0;
  size_t aliased_nodes = 0;
  std::map<std::string, int> kernel_histogram;
  std::vector<fml_resident *> resident_programs;  // owned
  size_t resident_stages = 0, resident_scratch_bytes = 0;
  ~Program();
  Program() = default;
  Program(const Program &) = delete;
};

class Builder {
public:
  static std::unique_ptr<Program> Run(const flow::Flow &flow, const flow::Sequence &sequence,
                                      const memory::Index &index, const AliasMap &aliases,
                                      const Options &options);
};

class Runner {
public:
  Runner(std::unique_ptr<Program> program, const Options &options);
  ~Runner();
  // `args`: name -> host pointer for every interface tensor.  Returns ns per epoch.
  size_t Run(const std::unordered_map<std::string, void *> &args, size_t epoch);
  const Program &GetProgram() const { return *program_; }
  // Tracing: replays the launch list eagerly `passes` times with an event pair around every
  // launch (weights are cold in each pass, as in a real forward pass) and returns the summed
  // microseconds and launch count per kernel name, plus the cost of an empty event pair under
  // the key "(empty event pair)".
  struct KernelTime { double us = 0; size_t launches = 0; };
  std::map<std::string, KernelTime> Profile(const std::unordered_map<std::string, void *> &args, size_t passes);
  // In-graph breakdown from kernel-start stamps: per kernel name the microseconds per pass from
  // each of its launches' start to the next launch's start (median over `passes` inner replays
  // of the captured graph) and its launches per pass; `pass_us` receives their sum.  With no
  // arguments the pass runs on whatever the interface buffers hold (zeros after Compile).
  // `per_launch_us`, when given, receives the period of every entry of the launch list in order.
  std::map<std::string, KernelTime> Trace(const std::unordered_map<std::string, void *> &args, size_t passes, double *pass_us,
                                          std::vector<double> *per_launch_us = nullptr);

private:
  void Replay();
  std::unique_ptr<Program> program_;
  Options options_;
  void *stream_ = nullptr;
  void *graph_exec_ = nullptr;
  void *ev_start_ = nullptr, *ev_stop_ = nullptr;
};

}  // namespace worker
}  // namespace fluidml
