// fluidml::worker::Executor -- the drop-in boundary.  Same class, namespace and member
// signatures as the reference's include/worker/executor.h:15-44; an application that
// compiled an ONNX model with FluidML and invoked it on the CPU links against this library
// instead and runs on a B200.
//
//   MakePlainLinear / MakePlainGreedy / MakeDPGreedy(name, epoch)
//       default layouts + bump arena / default layouts + greedy arena / dynamic-programming
//       layout search (GPU cost model) + greedy arena.  `epoch` = forward passes timed per
//       Invoke (reference: src/worker/executor.cpp:76-89).
//   Compile(input, mlir, llvm, json)
//       `input` is an ONNX file (or stream).  The optional dump arguments stay accepted:
//       `mlir` receives the launch plan as text, `llvm` the kernel/tiling table, `json`
//       {dp_table, plan, arena} (reference: src/worker/executor.cpp:91-133).
//   Invoke(args)
//       keys are the ONNX graph input and output names, values raw HOST pointers to dense
//       row-major buffers of the static shape; outputs are written in place.  A missing name
//       throws std::out_of_range (reference: src/worker/runner.cpp:70).  Returns the average
//       device time of one forward pass in nanoseconds (reference: wall time of the JIT'd
//       function, src/worker/runner.cpp:101-119); copies are outside the timed region there
//       and here.
//
// Errors are std::runtime_error (fluidml::Error); the reference asserts or is undefined.
// An Executor owns one device, one stream, its weights and its arena; instances are not
// thread-safe, distinct instances may be driven from distinct threads.
#ifndef FLUIDML_WORKER_EXECUTOR_H_
#define FLUIDML_WORKER_EXECUTOR_H_

#include <fstream>
#include <memory>
#include <optional>
#include <string>
#include <string_view>
#include <unordered_map>

namespace fluidml {
namespace worker {

class Executor {
public:
  virtual ~Executor() = default;
  virtual void Compile(std::istream &input, std::ofstream *mlir = nullptr,
                       std::ofstream *llvm = nullptr, std::ofstream *json = nullptr) = 0;
  virtual void Compile(std::string_view input,
                       std::optional<std::string_view> mlir = std::nullopt,
                       std::optional<std::string_view> llvm = std::nullopt,
                       std::optional<std::string_view> json = std::nullopt) = 0;
  virtual size_t Invoke(const std::unordered_map<std::string, void *> &args) = 0;

  static std::unique_ptr<Executor> MakePlainLinear(std::string &&name, size_t epoch = 1);
  static std::unique_ptr<Executor> MakePlainGreedy(std::string &&name, size_t epoch = 1);
  static std::unique_ptr<Executor> MakeDPGreedy(std::string &&name, size_t epoch = 1);

  // ---- additions of this back end (no counterpart in the reference) -------------------
  // Options, set before Compile: "device" (CUDA ordinal), "gemm_precision" (auto | fp32 |
  // 3xtf32 | tf32), "fusion" (0/1), "cuda_graph" (0/1), "alignment" (arena tenant alignment
  // in bytes), "dp_cost" (model | constant), "autotune" (0/1: time GEMM tile choices on the
  // device during Compile, as the reference's MatMul/Gemm generators time loop orders).  Environment variables FLUIDML_<KEY> give the
  // defaults.
  virtual void SetOption(const std::string &key, const std::string &value) = 0;
  // Compile-time facts as JSON text: arena bytes (aligned, unaligned, reference-equivalent),
  // weight bytes, launches per forward pass, kernel histogram.
  virtual std::string GetStatsJson() const = 0;

protected:
  Executor() = default;
  Executor(const Executor &) = delete;
  Executor(Executor &&) = default;
};

} // namespace worker
} // namespace fluidml

#endif
