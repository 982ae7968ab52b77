// Host-side Kernel objects.  In the reference a Kernel's Run() EMITS MLIR for one operator
// (include/structure/kernel/kernel/kernel.h:9-88); here Run() RECORDS the CUDA launches of
// that operator into a launch plan, calling the C ABI of the kernel library when the plan
// is replayed.  The taxonomy is the reference's: four arity x scratch signatures and one
// concrete class per operator kernel, with the same GetKernelName() strings.
#pragma once
#include "flow.h"
#include "fluidml_cuda.h"
#include <functional>

namespace fluidml {
namespace kernel {

// One recorded launch: a closure over tensor descriptors and scalars.  Returns fml_status.
struct Launch {
  std::string node, kernel;
  std::function<int(void *stream)> fn;
};

class LaunchRecorder {
public:
  void Add(std::string kernel, std::function<int(void *)> fn) {
    launches_.push_back({current_node_, std::move(kernel), std::move(fn)});
  }
  void SetNode(const std::string &name) { current_node_ = name; }
  const std::vector<Launch> &Launches() const { return launches_; }

private:
  std::string current_node_;
  std::vector<Launch> launches_;
};

// Scratch from the arena for kernels that ask for some through GetBufferSize(), with the
// lifetime of the one node (the reference's per-node buffer, src/worker/planner.cpp:283-291).
// None of the CUDA kernels needs any at present: Softmax and LayerNorm reduce in registers,
// Conv pads implicitly and split-K GEMMs reduce inside a cluster.
struct Buffer {
  void *data = nullptr;
  size_t bytes = 0;
};

class Kernel {
public:
  virtual ~Kernel() = default;
  virtual std::string GetKernelName() const = 0;
  // Uniform entry used by the builder; the four signature classes route it to their Run().
  virtual void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &inputs,
                      const fml_tensor &output, const Buffer &buffer) const = 0;
  // Scratch bytes this kernel needs for these operands.
  virtual size_t GetBufferSize(const std::vector<fml_tensor> &inputs, const fml_tensor &output) const {
    (void)inputs;
    (void)output;
    return 0;
  }
  // When the output is just another way of addressing the input's bytes (a reshape that
  // splits or merges contiguous dims, a transpose, a slice), fills `view` with the output's
  // shape and the strides / data pointer that realise it over `input`, and returns true: the
  // node then needs no launch and no memory of its own.
  virtual bool GetView(const fml_tensor &input, const fml_tensor &output, fml_tensor *view) const {
    (void)input; (void)output; (void)view;
    return false;
  }

  // Constant device bytes this kernel streams on every launch (its weights), if any; and the
  // hint that a later kernel's such bytes may be fetched into L2 while this one runs.
  virtual bool StreamedConstant(const void **ptr, size_t *bytes) const {
    (void)ptr; (void)bytes;
    return false;
  }
  virtual void SetPrefetch(const void *ptr, size_t bytes) { (void)ptr; (void)bytes; }
  // Tile choices that can be carried from one Compile to the next (GEMM tile_n / split_k): a
  // preset replaces the on-device tuning; TunedTiles reports what Launch ended up using.
  virtual void PresetTiles(int tile_n, int split_k) { (void)tile_n; (void)split_k; }
  virtual bool TunedTiles(int *tile_n, int *split_k) const { (void)tile_n; (void)split_k; return false; }
  // Stage of a resident program (fml_resident_stage) that computes what this kernel's launch
  // computes on these operands, if the kernel has such a form: a constant-weight GEMM with its
  // epilogue, or the attention core.  `out_external` is left for the builder to decide.
  virtual bool DescribeResident(const std::vector<fml_tensor> &inputs, const fml_tensor &output,
                                fml_resident_stage *stage) const {
    (void)inputs; (void)output; (void)stage;
    return false;
  }
  // A LayerNorm over the last axis without a residual input can ride in the epilogue of the
  // resident GEMM stage that produces its input.
  virtual bool DescribeLayerNorm(const fml_tensor &input, fml_tensor *scale, fml_tensor *bias, float *eps) const {
    (void)input; (void)scale; (void)bias; (void)eps;
    return false;
  }

protected:
  Kernel() = default;
};

class SingleInputWithoutBufferKernel : public Kernel {
public:
  virtual void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const = 0;
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &out,
              const Buffer &) const override { Run(rec, in.at(0), out); }
};

class SingleInputWithBufferKernel : public Kernel {
public:
  virtual void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output,
                   const Buffer &buffer) const = 0;
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &out,
              const Buffer &b) const override { Run(rec, in.at(0), out, b); }
};

class DoubleInputsWithoutBufferKernel : public Kernel {
public:
  virtual void Run(LaunchRecorder &rec, const fml_tensor &lhs, const fml_tensor &rhs,
                   const fml_tensor &output) const = 0;
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &out,
              const Buffer &) const override { Run(rec, in.at(0), in.at(1), out); }
};

class DoubleInputsWithBufferKernel : public Kernel {
public:
  virtual void Run(LaunchRecorder &rec, const fml_tensor &lhs, const fml_tensor &rhs,
                   const fml_tensor &output, const Buffer &buffer) const = 0;
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &out,
              const Buffer &b) const override { Run(rec, in.at(0), in.at(1), out, b); }
};

// Maps a constant region to its device view (uploaded by the builder).
using ConstResolver = std::function<fml_tensor(const flow::RegionPtr &)>;

struct KernelOptions {
  int gemm_precision = FML_GEMM_AUTO;  // fml_gemm_precision for MatMul / Gemm / Conv
  bool autotune = false;               // tune GEMM tiles on the device while recording (needs real buffers)
};

// node -> kernel object (reference: SelectKernel, src/worker/utils.cpp:80-335).
std::unique_ptr<Kernel> SelectKernel(const flow::Node &node, const ConstResolver &resolve,
                                     const KernelOptions &options);

// Describes a region as an fml_tensor over `data` with the strides of its layout.
fml_tensor MakeTensor(const flow::Region &region, void *data);

}  // namespace kernel
}  // namespace fluidml
