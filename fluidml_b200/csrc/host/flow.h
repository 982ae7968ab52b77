// Typed flow IR the kernels are selected from: regions (tensors with a layout), nodes (one
// per kernel launch group) and the flow / sequence containers.
//
// Carries over from the reference's structure/flow/ only what the hot path needs: the
// region facts (name, meta, layout -> strides, who owns the memory:
// include/structure/flow/region.h:12-99), the node taxonomy (one kind per reference kernel,
// include/structure/flow/node.h) and the per-node scratch size
// (src/structure/flow/node.cpp:500-519, :972-985, :1355-1368).
#pragma once
#include "base.h"
#include <unordered_map>

namespace fluidml {
namespace flow {

struct Region {
  enum Kind { kInner, kInput, kOutput, kConstant } kind = kInner;
  std::string name;
  Meta meta;
  std::vector<size_t> layout;        // layout[i] = physical position of logical dim i
  std::shared_ptr<Tensor> constant;  // kConstant only, logical row-major bytes
  // Only inner regions live in the planned arena; interface tensors are caller buffers and
  // constants are baked (reference: src/structure/flow/region.cpp:66,94).
  bool NeedMemoryAllocation() const { return kind == kInner; }
  // A region that is a view of another tensor's bytes (set by the lowering for reshapes,
  // transposes and slices that need no copy) carries explicit element strides and an element
  // offset from its owner's base; otherwise the strides follow from the layout.
  bool is_view = false;
  std::vector<int64_t> view_strides;
  int64_t view_offset = 0;
  std::vector<int64_t> GetStrides() const {
    return is_view ? view_strides : utils::GenStrides(meta.GetShape(), layout);
  }
};
using RegionPtr = std::shared_ptr<Region>;

enum class Kind {
  // one per reference kernel (src/structure/kernel/kernel/*.cpp)
  AddConstant, AddCommon, AddDivErfAddMulMul, AveragePoolWithoutPadding, Cast, Clip, Concat2,
  ConvWithoutPadding, ConvWithPadding, CumSum, DivConstantRhs, DivCommon, Dropout, Equal, Erf,
  Flatten, GatherConstantIndexScalar, GatherConstantIndicesTensor, GatherConstantDataTensor,
  GatherConstantDataTensorAddTensorLhsAddTensorLhs, GemmConstantBias,
  LayerNormalizationConstantScaleBias, MatMul, MaxPoolWithoutPadding, MulConstant, MulCommon,
  Neg, Not, Pad, Pow, ReduceMean, Relu, Reshape, Slice, Softmax, Sqrt, Squeeze, SubConstantLhs,
  SubCommon, Tanh, Transpose, Unsqueeze, UnsqueezeSubLhsScalarMulRhsScalar,
  WhereConstantCondConstantScalarY, WhereConstantCondConstantTensorY,
  // operators the reference has no kernel for
  Sigmoid, Identity,
  // fused nodes produced by the fusion passes of this back end
  FusedGemm,       // MatMul/Gemm + divisor + bias + activation + residual epilogue
  FusedSoftmax,    // softmax(x / divisor + mask)
  FusedLayerNorm,  // LayerNorm(x + residual)
  Silu,            // x * sigmoid(x)
  FusedAttention,  // softmax(Q K^T / divisor + mask) V; inputs: Q, K^T, V, [mask]
  FusedMulAdd,     // a * b + c, broadcast; inputs: a, b, c
  FusedMulAddChain,   // a0*b0 + a1*b1 + ... in the rounding order of the Mul / Add chain it replaces; inputs: a0, b0, a1, b1, ...
  Rotary,             // rotary position embedding over the first `value` features; inputs: x, cos, sin
  SqueezeExciteGate,  // act2(W2 act1(W1 mean_hw(x) + b1) + b2); consts: W1, [b1], W2, [b2]; has_bias / has_bias2 = b1 / b2 present; act, act2
};
const char *KindName(Kind k);

struct Node {
  Kind kind;
  std::string name;
  // Variable-or-constant operands in kernel order: 1 (single-input kinds) or 2 (double-input
  // kinds) as in the reference's arity taxonomy; fused kinds may add a third (residual / mask).
  std::vector<RegionPtr> inputs;
  // Constants captured by the node rather than passed as operands (reference: stored inside
  // the node object): Gemm weights/bias, LayerNorm scale/bias, Gather table or indices, Where
  // condition / y, Conv weights / bias, embedding addends, fused bias.
  std::vector<RegionPtr> consts;
  RegionPtr output;

  // parameters (which ones are meaningful depends on the kind)
  Type scalar_type = Type::kFloat32;
  double value = 0.0, value2 = 0.0;  // scalar constants
  int64_t axis = 0, group = 1;
  float epsilon = 1e-5f, alpha = 1.0f, beta = 1.0f;
  bool trans_a = false, trans_b = false;
  std::vector<int64_t> perm, axes, starts, pads, strides, dilations, kernel_shape;
  // fused GEMM epilogue
  float divisor = 1.0f;
  int act = 0;
  int act2 = 0;            // SqueezeExciteGate: activation of the second layer
  bool has_bias2 = false;  // SqueezeExciteGate: the second layer has a bias
  bool has_in_scale = false;  // Conv: inputs[1] scales x per (image, channel) (a Mul folded into the convolution)
  float act_param[3] = {1.4142135381698608f, 1.0f, 0.5f};
  bool has_bias = false, has_residual = false, has_mask = false;
  bool b_is_const = false;  // FusedGemm: B is a captured constant (consts[0]) rather than inputs[1]
  // Scratch bytes the REFERENCE kernel of this kind needs (one float per row for Softmax and
  // LayerNorm, a padded copy for ConvWithPadding); used to report the reference-equivalent
  // arena.  The CUDA kernels need none of it.
  size_t reference_buffer_size = 0;
  // Scratch bytes this back end needs (split-K partial tiles), filled by the planner.
  size_t buffer_size = 0;
};
using NodePtr = std::shared_ptr<Node>;

struct Flow {
  std::string name;
  std::vector<NodePtr> nodes;      // graph order
  std::vector<RegionPtr> regions;  // creation order: inputs/outputs/inner/constants
  std::vector<std::string> inputs, outputs;
  std::unordered_map<std::string, RegionPtr> by_name;
  RegionPtr Get(const std::string &n) const {
    auto it = by_name.find(n);
    if (it == by_name.end()) throw Error("flow has no region '" + n + "'");
    return it->second;
  }
};

// Nodes in execution order plus the regions (reference: structure/flow/sequence.h).
struct Sequence {
  std::vector<NodePtr> nodes;
  std::vector<RegionPtr> regions;
};

}  // namespace flow
}  // namespace fluidml
