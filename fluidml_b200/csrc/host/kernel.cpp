// Concrete kernels: one class per reference operator kernel
// (src/structure/kernel/kernel/<op>.cpp), each recording calls into the CUDA kernel library,
// and SelectKernel (reference: src/worker/utils.cpp:80-335) as a switch over the node kind.
#include "kernel.h"
#include <algorithm>

namespace fluidml {
namespace kernel {

fml_tensor MakeTensor(const flow::Region &region, void *data) {
  fml_tensor t;
  memset(&t, 0, sizeof(t));
  t.data = data;
  t.dtype = (int32_t)region.meta.GetType();
  t.rank = (int32_t)region.meta.GetRank();
  if (t.rank > FML_MAX_RANK) throw Error("tensor '" + region.name + "' has more than 8 dimensions");
  if (region.is_view) {
    const size_t es = GetSizeFromType(region.meta.GetType());
    t.data = data ? (char *)data + region.view_offset * (int64_t)es : nullptr;
  }
  const std::vector<int64_t> strides = region.GetStrides();
  for (int i = 0; i < t.rank; ++i) {
    t.shape[i] = region.meta.GetShape()[i];
    t.stride[i] = strides[i];
  }
  return t;
}

namespace {

bool SameStrides(const fml_tensor &a, const fml_tensor &b) {
  if (a.rank != b.rank) return false;
  for (int i = 0; i < a.rank; ++i)
    if (a.shape[i] != b.shape[i] || (a.shape[i] != 1 && a.stride[i] != b.stride[i])) return false;
  return true;
}

// Strides that address `in` through the shape of `out` without moving data, if they exist:
// runs of input dims that are contiguous with each other may be split or merged freely.
bool ReshapeView(const fml_tensor &in, const fml_tensor &out, fml_tensor *view) {
  *view = out;
  view->data = in.data;
  int view_d = out.rank - 1;
  if (in.rank == 0) {
    for (int i = 0; i < out.rank; ++i) view->stride[i] = 1;
    return true;
  }
  int64_t chunk_base = in.stride[in.rank - 1], tensor_numel = 1, view_numel = 1;
  for (int d = in.rank - 1; d >= 0; --d) {
    tensor_numel *= in.shape[d];
    if (d == 0 || (in.shape[d - 1] != 1 && in.stride[d - 1] != tensor_numel * chunk_base)) {
      while (view_d >= 0 && (view_numel < tensor_numel || out.shape[view_d] == 1)) {
        view->stride[view_d] = view_numel * chunk_base;
        view_numel *= out.shape[view_d];
        --view_d;
      }
      if (view_numel != tensor_numel) return false;
      if (d > 0) {
        chunk_base = in.stride[d - 1];
        tensor_numel = 1;
        view_numel = 1;
      }
    }
  }
  return view_d == -1;
}

bool RowMajor(const fml_tensor &t) {
  int64_t s = 1;
  for (int i = t.rank - 1; i >= 0; --i) {
    if (t.shape[i] != 1 && t.stride[i] != s) return false;
    s *= t.shape[i];
  }
  return true;
}

// View of `in` with the dims permuted: view.dim[i] = in.dim[perm[i]].
fml_tensor Permuted(const fml_tensor &in, const std::vector<int64_t> &perm) {
  fml_tensor v = in;
  for (int i = 0; i < in.rank; ++i) {
    v.shape[i] = in.shape[perm[i]];
    v.stride[i] = in.stride[perm[i]];
  }
  return v;
}

void *Offset(const fml_tensor &t, int64_t elems) {
  size_t es = t.dtype == FML_I64 ? 8 : t.dtype == FML_BOOL ? 1 : 4;
  return (char *)t.data + elems * (int64_t)es;
}

// ------------------------------------------------------------------ elementwise
class UnaryElementwise : public SingleInputWithoutBufferKernel {
public:
  UnaryElementwise(const char *name, int op, double p0 = 0.0, double p1 = 0.0)
      : name_(name), op_(op), p0_(p0), p1_(p1) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const int op = op_;
    const double p0 = p0_, p1 = p1_;
    rec.Add(name_, [=](void *s) { return fml_elementwise(op, &input, nullptr, &output, p0, p1, s); });
  }

private:
  const char *name_;
  int op_;
  double p0_, p1_;
};

class BinaryElementwise : public DoubleInputsWithoutBufferKernel {
public:
  BinaryElementwise(const char *name, int op) : name_(name), op_(op) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &lhs, const fml_tensor &rhs,
           const fml_tensor &output) const override {
    const int op = op_;
    rec.Add(name_, [=](void *s) { return fml_elementwise(op, &lhs, &rhs, &output, 0.0, 0.0, s); });
  }

private:
  const char *name_;
  int op_;
};

#define UNARY_KERNEL(Class, op, ...)                                                       \
  struct Class : UnaryElementwise { Class(double p0 = 0.0, double p1 = 0.0) : UnaryElementwise(#Class, op, p0, p1) {} };
#define BINARY_KERNEL(Class, op)                                                           \
  struct Class : BinaryElementwise { Class() : BinaryElementwise(#Class, op) {} };

UNARY_KERNEL(AddConstantKernel, FML_ADD_SCALAR)       // add.cpp:22-79
UNARY_KERNEL(MulConstantKernel, FML_MUL_SCALAR)       // mul.cpp:19-54
UNARY_KERNEL(DivConstantRhsKernel, FML_DIV_SCALAR)    // div.cpp:18-66
UNARY_KERNEL(SubConstantLhsKernel, FML_RSUB_SCALAR)   // sub.cpp:16-67
UNARY_KERNEL(PowKernel, FML_POW_SCALAR)               // pow.cpp:15-61
UNARY_KERNEL(ClipKernel, FML_CLIP)                    // clip.cpp:13-48
UNARY_KERNEL(EqualKernel, FML_EQUAL_SCALAR)           // equal.cpp:14-51
UNARY_KERNEL(ErfKernel, FML_ERF)                      // erf.cpp:18-45
UNARY_KERNEL(TanhKernel, FML_TANH)                    // tanh.cpp:12-40
UNARY_KERNEL(SqrtKernel, FML_SQRT)                    // sqrt.cpp:13-36
UNARY_KERNEL(NegKernel, FML_NEG)                      // neg.cpp:17-40
UNARY_KERNEL(NotKernel, FML_NOT)                      // not.cpp:11-41
UNARY_KERNEL(ReluKernel, FML_RELU)                    // relu.cpp:12-46
UNARY_KERNEL(CastKernel, FML_CAST)                    // cast.cpp:12-62
UNARY_KERNEL(SigmoidKernel, FML_SIGMOID)              // no reference kernel
UNARY_KERNEL(SiluKernel, FML_SILU)                    // Sigmoid + Mul fused
BINARY_KERNEL(AddCommonKernel, FML_ADD)               // add.cpp:83-124
BINARY_KERNEL(MulCommonKernel, FML_MUL)               // mul.cpp:56-99
BINARY_KERNEL(DivCommonKernel, FML_DIV)               // div.cpp:70-105
BINARY_KERNEL(SubCommonKernel, FML_SUB)               // sub.cpp:71-99

// dropout.cpp:13-33: identity.  Aliased away when the two layouts agree.
class DropoutKernel : public SingleInputWithoutBufferKernel {
public:
  std::string GetKernelName() const override { return "DropoutKernel"; }
  bool GetView(const fml_tensor &in, const fml_tensor &out, fml_tensor *view) const override {
    *view = in;
    (void)out;
    return true;
  }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    rec.Add("DropoutKernel", [=](void *s) { return fml_copy_strided(&input, &output, s); });
  }
};

// add_div_erf_add_mul_mul.cpp:29-132: (x + bias) * (erf((x + bias) / c0) + c1) * c2
class AddDivErfAddMulMulKernel : public SingleInputWithoutBufferKernel {
public:
  AddDivErfAddMulMulKernel(fml_tensor bias, float c0, float c1, float c2) : bias_(bias), c0_(c0), c1_(c1), c2_(c2) {}
  std::string GetKernelName() const override { return "AddDivErfAddMulMulKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor bias = bias_;
    const float c0 = c0_, c1 = c1_, c2 = c2_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_bias_gelu(&input, &bias, &output, c0, c1, c2, s); });
  }

private:
  fml_tensor bias_;
  float c0_, c1_, c2_;
};

// unsqueeze_sub_mul.cpp:19-70: out = (c - unsqueeze(x)) * m
class UnsqueezeSubLhsScalarMulRhsScalarKernel : public SingleInputWithoutBufferKernel {
public:
  UnsqueezeSubLhsScalarMulRhsScalarKernel(double sub, double mul) : sub_(sub), mul_(mul) {}
  std::string GetKernelName() const override { return "UnsqueezeSubLhsScalarMulRhsScalarKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    // the unsqueezed input is the input seen through the output's shape: the e-th element of
    // one is the e-th of the other, and the inserted dims have extent 1
    fml_tensor view = output;
    view.data = input.data;
    int j = 0;
    for (int i = 0; i < output.rank; ++i) {
      if (j < input.rank && input.shape[j] == output.shape[i]) view.stride[i] = input.stride[j++];
      else view.stride[i] = 0;
    }
    const double a = sub_, m = mul_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_elementwise(FML_RSUB_MUL_SCALAR, &view, nullptr, &output, a, m, s); });
  }

private:
  double sub_, mul_;
};

// where.cpp:30-80 / :90-150
class WhereKernel : public SingleInputWithoutBufferKernel {
public:
  WhereKernel(const char *name, fml_tensor cond, bool has_y, fml_tensor y, float y_scalar)
      : name_(name), cond_(cond), has_y_(has_y), y_(y), y_scalar_(y_scalar) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor cond = cond_, y = y_;
    const bool has_y = has_y_;
    const float ys = y_scalar_;
    rec.Add(name_, [=](void *s) { return fml_where(&cond, &input, has_y ? &y : nullptr, ys, &output, s); });
  }

private:
  const char *name_;
  fml_tensor cond_;
  bool has_y_;
  fml_tensor y_;
  float y_scalar_;
};

// MulCommon -> AddCommon in one launch (mul.cpp + add.cpp of the reference run as two loop nests)
class FusedMulAddKernel : public Kernel {
public:
  std::string GetKernelName() const override { return "FusedMulAddKernel"; }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output, const Buffer &) const override {
    const fml_tensor a = in.at(0), b = in.at(1), c = in.at(2);
    rec.Add(GetKernelName(), [=](void *s) { return fml_mul_add(&a, &b, &c, &output, s); });
  }
};

// Slice, Slice, Neg, Concat, Mul, Mul, Add, Concat of a rotary position embedding in one launch
class RotaryKernel : public Kernel {
public:
  explicit RotaryKernel(int64_t rot) : rot_(rot) {}
  std::string GetKernelName() const override { return "RotaryKernel"; }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output, const Buffer &) const override {
    const fml_tensor x = in.at(0), c = in.at(1), sn = in.at(2);
    const int64_t rot = rot_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_rotary(&x, &c, &sn, rot, &output, s); });
  }

private:
  int64_t rot_;
};

// A chain MulCommon -> FusedMulAdd -> FusedMulAdd ... that sums products, in one launch
class FusedMulAddChainKernel : public Kernel {
public:
  std::string GetKernelName() const override { return "FusedMulAddChainKernel"; }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output, const Buffer &) const override {
    const std::vector<fml_tensor> ops = in;  // a0, b0, a1, b1, ...
    rec.Add(GetKernelName(), [=](void *s) {
      const int n = (int)(ops.size() / 2);
      std::vector<const fml_tensor *> a(n), b(n);
      for (int i = 0; i < n; ++i) { a[i] = &ops[2 * i]; b[i] = &ops[2 * i + 1]; }
      return fml_sum_of_products(n, a.data(), b.data(), &output, s);
    });
  }
};

// ReduceMean over H, W -> 1 x 1 Conv -> 1 x 1 Conv (the gate of a squeeze-and-excite block) in one
// launch (reduce_mean.cpp + conv.cpp twice in the reference)
class SqueezeExciteGateKernel : public SingleInputWithoutBufferKernel {
public:
  SqueezeExciteGateKernel(fml_tensor w1, bool has_b1, fml_tensor b1, fml_tensor w2, bool has_b2, fml_tensor b2, int act1, int act2)
      : w1_(w1), b1_(b1), w2_(w2), b2_(b2), has_b1_(has_b1), has_b2_(has_b2), act1_(act1), act2_(act2) {}
  std::string GetKernelName() const override { return "SqueezeExciteGateKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor w1 = w1_, b1 = b1_, w2 = w2_, b2 = b2_;
    const bool hb1 = has_b1_, hb2 = has_b2_;
    const int a1 = act1_, a2 = act2_;
    rec.Add(GetKernelName(), [=](void *s) {
      return fml_squeeze_excite_gate(&input, &w1, hb1 ? &b1 : nullptr, &w2, hb2 ? &b2 : nullptr, a1, a2, &output, s);
    });
  }

private:
  fml_tensor w1_, b1_, w2_, b2_;
  bool has_b1_, has_b2_;
  int act1_, act2_;
};

// ------------------------------------------------------------------ data movement
// reshape.cpp:18-64, unsqueeze.cpp:20-63, squeeze.cpp:17-54, flatten.cpp:15-63
class ReshapeLikeKernel : public SingleInputWithoutBufferKernel {
public:
  explicit ReshapeLikeKernel(const char *name) : name_(name) {}
  std::string GetKernelName() const override { return name_; }
  bool GetView(const fml_tensor &in, const fml_tensor &out, fml_tensor *view) const override {
    return ReshapeView(in, out, view);
  }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    rec.Add(name_, [=](void *s) { return fml_reshape_copy(&input, &output, s); });
  }

private:
  const char *name_;
};

// transpose.cpp:19-48
class TransposeKernel : public SingleInputWithoutBufferKernel {
public:
  explicit TransposeKernel(std::vector<int64_t> perm) : perm_(std::move(perm)) {}
  std::string GetKernelName() const override { return "TransposeKernel"; }
  bool GetView(const fml_tensor &in, const fml_tensor &out, fml_tensor *view) const override {
    *view = Permuted(in, perm_);
    (void)out;
    return true;
  }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor view = Permuted(input, perm_);
    rec.Add(GetKernelName(), [=](void *s) { return fml_copy_strided(&view, &output, s); });
  }

private:
  std::vector<int64_t> perm_;
};

// slice.cpp:17-55
class SliceKernel : public SingleInputWithoutBufferKernel {
public:
  explicit SliceKernel(std::vector<int64_t> starts) : starts_(std::move(starts)) {}
  std::string GetKernelName() const override { return "SliceKernel"; }
  bool GetView(const fml_tensor &input, const fml_tensor &output, fml_tensor *view) const override {
    *view = input;
    int64_t off = 0;
    for (int i = 0; i < input.rank; ++i) {
      off += starts_[i] * input.stride[i];
      view->shape[i] = output.shape[i];
    }
    view->data = Offset(input, off);
    return true;
  }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    fml_tensor view;
    GetView(input, output, &view);
    rec.Add(GetKernelName(), [=](void *s) { return fml_copy_strided(&view, &output, s); });
  }

private:
  std::vector<int64_t> starts_;
};

// concat.cpp:18-68
class Concat2Kernel : public DoubleInputsWithoutBufferKernel {
public:
  explicit Concat2Kernel(int64_t axis) : axis_(axis) {}
  std::string GetKernelName() const override { return "Concat2Kernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &lhs, const fml_tensor &rhs,
           const fml_tensor &output) const override {
    const int axis = (int)axis_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_concat2(&lhs, &rhs, &output, axis, s); });
  }

private:
  int64_t axis_;
};

// pad.cpp:15-51
class PadKernel : public SingleInputWithoutBufferKernel {
public:
  explicit PadKernel(std::vector<int64_t> pads) : pads_(std::move(pads)) {}
  std::string GetKernelName() const override { return "PadKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const std::vector<int64_t> begin(pads_.begin(), pads_.begin() + input.rank);
    rec.Add(GetKernelName(), [=](void *s) { return fml_pad(&input, &output, begin.data(), s); });
  }

private:
  std::vector<int64_t> pads_;
};

// gather.cpp:100-139: one index along `axis` -> a view of the input, copied
class GatherConstantIndexScalarKernel : public SingleInputWithoutBufferKernel {
public:
  GatherConstantIndexScalarKernel(int64_t axis, int64_t index) : axis_(axis), index_(index) {}
  std::string GetKernelName() const override { return "GatherConstantIndexScalarKernel"; }
  // One index along one axis is a view: the input without that axis, starting `index` steps in.
  bool GetView(const fml_tensor &input, const fml_tensor &output, fml_tensor *view) const override {
    if (index_ < 0 || index_ >= input.shape[axis_]) throw Error("Gather: constant index is outside the gathered axis");
    *view = output;
    view->data = Offset(input, index_ * input.stride[axis_]);
    for (int i = 0, j = 0; i < input.rank; ++i)
      if (i != axis_) view->stride[j++] = input.stride[i];
    return true;
  }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    fml_tensor view;
    GetView(input, output, &view);
    rec.Add(GetKernelName(), [=](void *s) { return fml_copy_strided(&view, &output, s); });
  }

private:
  int64_t axis_, index_;
};

// gather.cpp:149-186 (constant indices, variable data) and :195-272 (constant table)
class GatherKernel : public SingleInputWithoutBufferKernel {
public:
  GatherKernel(const char *name, fml_tensor constant, bool constant_is_table, int64_t axis)
      : name_(name), constant_(constant), constant_is_table_(constant_is_table), axis_(axis) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor c = constant_;
    const int axis = (int)axis_;
    if (constant_is_table_) rec.Add(name_, [=](void *s) { return fml_gather(&c, &input, &output, axis, s); });
    else rec.Add(name_, [=](void *s) { return fml_gather(&input, &c, &output, axis, s); });
  }

private:
  const char *name_;
  fml_tensor constant_;
  bool constant_is_table_;
  int64_t axis_;
};

// gather_add_add.cpp:25-163
class GatherConstantDataTensorAddTensorLhsAddTensorLhsKernel : public SingleInputWithoutBufferKernel {
public:
  GatherConstantDataTensorAddTensorLhsAddTensorLhsKernel(fml_tensor table, fml_tensor add0, fml_tensor add1)
      : table_(table), add0_(add0), add1_(add1) {}
  std::string GetKernelName() const override { return "GatherConstantDataTensorAddTensorLhsAddTensorLhsKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor t = table_, a0 = add0_, a1 = add1_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_embedding(&t, &input, &a0, &a1, &output, s); });
  }

private:
  fml_tensor table_, add0_, add1_;
};

// ------------------------------------------------------------------ reductions
// softmax.cpp:22-139 (+ the fused divisor / mask variant)
class SoftmaxKernel : public Kernel {
public:
  SoftmaxKernel(int64_t axis, float divisor, bool has_mask) : axis_(axis), divisor_(divisor), has_mask_(has_mask) {}
  std::string GetKernelName() const override { return has_mask_ || divisor_ != 1.0f ? "FusedSoftmaxKernel" : "SoftmaxKernel"; }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output,
              const Buffer &) const override {
    const fml_tensor x = in.at(0), mask = has_mask_ ? in.at(1) : fml_tensor{};
    const bool hm = has_mask_;
    const float d = divisor_;
    const int axis = (int)axis_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_softmax(&x, hm ? &mask : nullptr, d, &output, axis, s); });
  }

private:
  int64_t axis_;
  float divisor_;
  bool has_mask_;
};

// matmul.cpp:5-44 -> softmax.cpp:22-139 -> matmul.cpp:5-44 of one attention head group, fused
class AttentionKernel : public Kernel {
public:
  AttentionKernel(float divisor, bool has_mask) : divisor_(divisor), has_mask_(has_mask) {}
  std::string GetKernelName() const override { return "FusedAttentionKernel"; }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output,
              const Buffer &) const override {
    const fml_tensor q = in.at(0), kt = in.at(1), v = in.at(2), mask = has_mask_ ? in.at(3) : fml_tensor{};
    const bool hm = has_mask_;
    const float d = divisor_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_attention(&q, &kt, &v, hm ? &mask : nullptr, d, &output, s); });
  }
  bool DescribeResident(const std::vector<fml_tensor> &in, const fml_tensor &output, fml_resident_stage *st) const override {
    memset(st, 0, sizeof(*st));
    st->kind = FML_RESIDENT_ATTENTION;
    st->out = output;
    st->q = in.at(0); st->kt = in.at(1); st->v = in.at(2);
    if (has_mask_) st->mask = in.at(3);
    st->divisor = divisor_;
    return true;
  }

private:
  float divisor_;
  bool has_mask_;
};

// layer_normalization.cpp:33-220 (+ the fused residual variant)
class LayerNormalizationConstantScaleBiasKernel : public Kernel {
public:
  LayerNormalizationConstantScaleBiasKernel(fml_tensor scale, fml_tensor bias, int64_t axis, float eps, bool residual)
      : scale_(scale), bias_(bias), axis_(axis), eps_(eps), residual_(residual) {}
  std::string GetKernelName() const override {
    return residual_ ? "FusedLayerNormalizationKernel" : "LayerNormalizationConstantScaleBiasKernel";
  }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output,
              const Buffer &) const override {
    const fml_tensor x = in.at(0), r = residual_ ? in.at(1) : fml_tensor{}, g = scale_, b = bias_;
    const bool hr = residual_;
    const int axis = (int)axis_;
    const float eps = eps_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_layernorm(&x, hr ? &r : nullptr, &g, &b, &output, axis, eps, s); });
  }
  bool DescribeLayerNorm(const fml_tensor &input, fml_tensor *scale, fml_tensor *bias, float *eps) const override {
    if (residual_ || (axis_ != input.rank - 1 && axis_ != -1)) return false;
    *scale = scale_; *bias = bias_; *eps = eps_;
    return true;
  }

private:
  fml_tensor scale_, bias_;
  int64_t axis_;
  float eps_;
  bool residual_;
};

class ReduceMeanKernel : public SingleInputWithoutBufferKernel {  // reduce_mean.cpp:16-98
public:
  explicit ReduceMeanKernel(std::vector<int64_t> axes) : axes_(std::move(axes)) {}
  std::string GetKernelName() const override { return "ReduceMeanKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    std::vector<int32_t> flags(input.rank, 0);
    for (int64_t a : axes_) flags.at(a) = 1;
    rec.Add(GetKernelName(), [=](void *s) { return fml_reduce_mean(&input, &output, flags.data(), s); });
  }

private:
  std::vector<int64_t> axes_;
};

class CumSumKernel : public SingleInputWithoutBufferKernel {  // cum_sum.cpp:53-87
public:
  explicit CumSumKernel(int64_t axis) : axis_(axis) {}
  std::string GetKernelName() const override { return "CumSumKernel"; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const int axis = (int)axis_;
    rec.Add(GetKernelName(), [=](void *s) { return fml_cumsum(&input, &output, axis, s); });
  }

private:
  int64_t axis_;
};

// ------------------------------------------------------------------ GEMM family
// matmul.cpp:28-59, gemm.cpp:39-182 and the fused epilogue variant.  inputs: A, B (B may be a
// captured constant), optional residual; bias captured or passed.
class GemmLikeKernel : public Kernel {
public:
  struct Config {
    const char *name;
    fml_gemm_params params;
    bool has_const_b = false, has_bias = false, has_residual = false, bias_is_input = false;
    fml_tensor const_b{}, bias{};
    bool trans_a = false, trans_b = false, autotune = false;
  };
  explicit GemmLikeKernel(Config c) : c_(c) {}
  std::string GetKernelName() const override { return c_.name; }
  bool StreamedConstant(const void **ptr, size_t *bytes) const override {
    if (!c_.has_const_b) return false;
    size_t n = 4;
    for (int i = 0; i < c_.const_b.rank; ++i) n *= (size_t)c_.const_b.shape[i];
    *ptr = c_.const_b.data;
    *bytes = n;
    return true;
  }
  void SetPrefetch(const void *ptr, size_t bytes) override {
    c_.params.l2_prefetch = ptr;
    c_.params.l2_prefetch_bytes = bytes;
  }
  void PresetTiles(int tile_n, int split_k) override {
    c_.params.tile_n = tile_n;
    c_.params.split_k = split_k;
    c_.autotune = false;
  }
  bool TunedTiles(int *tile_n, int *split_k) const override {
    if (tuned_tn_ <= 0) return false;
    *tile_n = tuned_tn_;
    *split_k = tuned_sk_;
    return true;
  }

  void Resolve(const std::vector<fml_tensor> &in, fml_tensor &a, fml_tensor &b, fml_tensor &bias,
               fml_tensor &res) const {
    size_t k = 0;
    a = in.at(k++);
    b = c_.has_const_b ? c_.const_b : in.at(k++);
    if (c_.trans_a) std::swap(a.shape[a.rank - 2], a.shape[a.rank - 1]), std::swap(a.stride[a.rank - 2], a.stride[a.rank - 1]);
    if (c_.trans_b) std::swap(b.shape[b.rank - 2], b.shape[b.rank - 1]), std::swap(b.stride[b.rank - 2], b.stride[b.rank - 1]);
    bias = c_.bias;
    if (c_.has_bias && c_.bias_is_input) bias = in.at(k++);
    if (c_.has_residual) res = in.at(k++);
  }
  bool DescribeResident(const std::vector<fml_tensor> &in, const fml_tensor &output, fml_resident_stage *st) const override {
    const fml_gemm_params &p = c_.params;
    if (!c_.has_const_b || c_.trans_a || c_.bias_is_input) return false;
    if (p.alpha != 1.0f || (c_.has_bias && p.beta != 1.0f) || (p.divisor != 1.0f && p.divisor != 0.0f)) return false;
    if (p.precision == FML_GEMM_FP32 || p.precision == FML_GEMM_TF32) return false;  // the resident GEMM is 3xTF32
    if (p.act < FML_ACT_NONE || p.act > FML_ACT_SIGMOID) return false;
    fml_tensor a, b, bias{}, res{};
    Resolve(in, a, b, bias, res);
    if (b.rank != 2 || (c_.has_bias && bias.rank != 1)) return false;
    memset(st, 0, sizeof(*st));
    st->kind = FML_RESIDENT_GEMM;
    st->out = output; st->a = a; st->w = b;
    if (c_.has_bias) st->bias = bias;
    if (c_.has_residual) st->residual = res;
    st->act = p.act;
    for (int i = 0; i < 3; ++i) st->act_param[i] = p.act_param[i];
    return true;
  }
  void Launch(LaunchRecorder &rec, const std::vector<fml_tensor> &in, const fml_tensor &output,
              const Buffer &buf) const override {
    fml_tensor a, b, bias{}, res{};
    Resolve(in, a, b, bias, res);
    Config c = c_;
    c.params.b_constant = c.has_const_b ? 1 : 0;
    if (c.autotune) {  // device buffers are live while the builder records: try the candidates now
      fml_gemm_params tuned;
      if (fml_gemm_autotune(&a, &b, &output, c.has_bias ? &bias : nullptr, c.has_residual ? &res : nullptr,
                            &c.params, nullptr, &tuned) != FML_OK)
        throw Error(std::string(c.name) + ": " + fml_last_error());
      c.params = tuned;
      tuned_tn_ = tuned.tile_n;
      tuned_sk_ = tuned.split_k;
    }
    rec.Add(c.name, [=](void *s) {
      return fml_gemm(&a, &b, &output, c.has_bias ? &bias : nullptr, c.has_residual ? &res : nullptr, &c.params, s);
    });
  }

private:
  Config c_;
  mutable int tuned_tn_ = 0, tuned_sk_ = 0;
};

// conv.cpp:27-280
class ConvKernel : public SingleInputWithoutBufferKernel {
public:
  ConvKernel(const char *name, fml_tensor w, bool has_bias, fml_tensor bias, fml_conv_params p)
      : name_(name), w_(w), has_bias_(has_bias), bias_(bias), p_(p) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const fml_tensor w = w_, b = bias_;
    const bool hb = has_bias_;
    const fml_conv_params p = p_;
    rec.Add(name_, [=](void *s) { return fml_conv(&input, &w, hb ? &b : nullptr, &output, &p, s); });
  }

private:
  const char *name_;
  fml_tensor w_;
  bool has_bias_;
  fml_tensor bias_;
  fml_conv_params p_;
};

// mul.cpp + conv.cpp: the per-channel gate multiplies x inside the convolution's operand gather
class ScaledConvKernel : public DoubleInputsWithoutBufferKernel {
public:
  ScaledConvKernel(const char *name, fml_tensor w, bool has_bias, fml_tensor bias, fml_conv_params p)
      : name_(name), w_(w), has_bias_(has_bias), bias_(bias), p_(p) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &x, const fml_tensor &scale, const fml_tensor &output) const override {
    const fml_tensor w = w_, b = bias_;
    const bool hb = has_bias_;
    const fml_conv_params p = p_;
    rec.Add(name_, [=](void *s) { return fml_conv_scaled(&x, &scale, &w, hb ? &b : nullptr, &output, &p, s); });
  }

private:
  const char *name_;
  fml_tensor w_;
  bool has_bias_;
  fml_tensor bias_;
  fml_conv_params p_;
};

// maxpool.cpp:17-82, averagepool.cpp:19-87
class PoolKernel : public SingleInputWithoutBufferKernel {
public:
  PoolKernel(const char *name, int mode, std::vector<int64_t> k, std::vector<int64_t> s)
      : name_(name), mode_(mode), k_(std::move(k)), s_(std::move(s)) {}
  std::string GetKernelName() const override { return name_; }
  void Run(LaunchRecorder &rec, const fml_tensor &input, const fml_tensor &output) const override {
    const int mode = mode_;
    const std::vector<int64_t> k = k_, st = s_;
    rec.Add(name_, [=](void *s) { return fml_pool2d(&input, &output, mode, k.data(), st.data(), s); });
  }

private:
  const char *name_;
  int mode_;
  std::vector<int64_t> k_, s_;
};

fml_gemm_params DefaultGemmParams(const KernelOptions &o) {
  fml_gemm_params p;
  fml_gemm_default_params(&p);
  p.precision = o.gemm_precision;
  return p;
}

}  // namespace

std::unique_ptr<Kernel> SelectKernel(const flow::Node &n, const ConstResolver &resolve,
                                     const KernelOptions &options) {
  using flow::Kind;
  auto C = [&](size_t i) { return resolve(n.consts.at(i)); };
  switch (n.kind) {
  case Kind::AddConstant: return std::make_unique<AddConstantKernel>(n.value);
  case Kind::MulConstant: return std::make_unique<MulConstantKernel>(n.value);
  case Kind::DivConstantRhs: return std::make_unique<DivConstantRhsKernel>(n.value);
  case Kind::SubConstantLhs: return std::make_unique<SubConstantLhsKernel>(n.value);
  case Kind::Pow: return std::make_unique<PowKernel>(n.value);
  case Kind::Clip: return std::make_unique<ClipKernel>(n.value, n.value2);
  case Kind::Equal: return std::make_unique<EqualKernel>(n.value);
  case Kind::Erf: return std::make_unique<ErfKernel>();
  case Kind::Tanh: return std::make_unique<TanhKernel>();
  case Kind::Sqrt: return std::make_unique<SqrtKernel>();
  case Kind::Neg: return std::make_unique<NegKernel>();
  case Kind::Not: return std::make_unique<NotKernel>();
  case Kind::Relu: return std::make_unique<ReluKernel>();
  case Kind::Cast: return std::make_unique<CastKernel>();
  case Kind::Sigmoid: return std::make_unique<SigmoidKernel>();
  case Kind::Silu: return std::make_unique<SiluKernel>();
  case Kind::FusedMulAdd: return std::make_unique<FusedMulAddKernel>();
  case Kind::FusedMulAddChain: return std::make_unique<FusedMulAddChainKernel>();
  case Kind::Rotary: return std::make_unique<RotaryKernel>((int64_t)n.value);
  case Kind::SqueezeExciteGate: {
    size_t k = 0;
    const fml_tensor w1 = C(k++);
    const fml_tensor b1 = n.has_bias ? C(k++) : fml_tensor{};
    const fml_tensor w2 = C(k++);
    const fml_tensor b2 = n.has_bias2 ? C(k++) : fml_tensor{};
    return std::make_unique<SqueezeExciteGateKernel>(w1, n.has_bias, b1, w2, n.has_bias2, b2, n.act, n.act2);
  }
  case Kind::AddCommon: return std::make_unique<AddCommonKernel>();
  case Kind::MulCommon: return std::make_unique<MulCommonKernel>();
  case Kind::DivCommon: return std::make_unique<DivCommonKernel>();
  case Kind::SubCommon: return std::make_unique<SubCommonKernel>();
  case Kind::Dropout:
  case Kind::Identity: return std::make_unique<DropoutKernel>();
  case Kind::AddDivErfAddMulMul:
    return std::make_unique<AddDivErfAddMulMulKernel>(C(0), n.act_param[0], n.act_param[1], n.act_param[2]);
  case Kind::UnsqueezeSubLhsScalarMulRhsScalar:
    return std::make_unique<UnsqueezeSubLhsScalarMulRhsScalarKernel>(n.value, n.value2);
  case Kind::WhereConstantCondConstantScalarY:
    return std::make_unique<WhereKernel>("WhereConstantCondConstantScalarYKernel", C(0), false, fml_tensor{}, (float)n.value);
  case Kind::WhereConstantCondConstantTensorY:
    return std::make_unique<WhereKernel>("WhereConstantCondConstantTensorYKernel", C(0), true, C(1), 0.0f);
  case Kind::Reshape: return std::make_unique<ReshapeLikeKernel>("ReshapeKernel");
  case Kind::Unsqueeze: return std::make_unique<ReshapeLikeKernel>("UnsqueezeKernel");
  case Kind::Squeeze: return std::make_unique<ReshapeLikeKernel>("SqueezeKernel");
  case Kind::Flatten: return std::make_unique<ReshapeLikeKernel>("FlattenKernel");
  case Kind::Transpose: return std::make_unique<TransposeKernel>(n.perm);
  case Kind::Slice: return std::make_unique<SliceKernel>(n.starts);
  case Kind::Concat2: return std::make_unique<Concat2Kernel>(n.axis);
  case Kind::Pad: return std::make_unique<PadKernel>(n.pads);
  case Kind::GatherConstantIndexScalar:
    return std::make_unique<GatherConstantIndexScalarKernel>(n.axis, (int64_t)n.value);
  case Kind::GatherConstantIndicesTensor:
    return std::make_unique<GatherKernel>("GatherConstantIndicesTensorKernel", C(0), false, n.axis);
  case Kind::GatherConstantDataTensor:
    return std::make_unique<GatherKernel>("GatherConstantDataTensorKernel", C(0), true, 0);
  case Kind::GatherConstantDataTensorAddTensorLhsAddTensorLhs:
    return std::make_unique<GatherConstantDataTensorAddTensorLhsAddTensorLhsKernel>(C(0), C(1), C(2));
  case Kind::Softmax: return std::make_unique<SoftmaxKernel>(n.axis, 1.0f, false);
  case Kind::FusedSoftmax: return std::make_unique<SoftmaxKernel>(n.axis, n.divisor, n.has_mask);
  case Kind::FusedAttention: return std::make_unique<AttentionKernel>(n.divisor, n.has_mask);
  case Kind::LayerNormalizationConstantScaleBias:
    return std::make_unique<LayerNormalizationConstantScaleBiasKernel>(C(0), C(1), n.axis, n.epsilon, false);
  case Kind::FusedLayerNorm:
    return std::make_unique<LayerNormalizationConstantScaleBiasKernel>(C(0), C(1), n.axis, n.epsilon, true);
  case Kind::ReduceMean: return std::make_unique<ReduceMeanKernel>(n.axes);
  case Kind::CumSum: return std::make_unique<CumSumKernel>(n.axis);
  case Kind::MatMul: {
    GemmLikeKernel::Config c;
    c.name = "MatMulKernel";
    c.params = DefaultGemmParams(options);
    c.autotune = options.autotune;
    return std::make_unique<GemmLikeKernel>(c);
  }
  case Kind::GemmConstantBias: {
    GemmLikeKernel::Config c;
    c.name = "GemmConstantWeightsBiasKernel";
    c.params = DefaultGemmParams(options);
    c.autotune = options.autotune;
    c.params.alpha = n.alpha;
    c.params.beta = n.beta;
    c.has_const_b = true;
    c.const_b = C(0);
    c.has_bias = true;
    c.bias = C(1);
    c.trans_a = n.trans_a;
    c.trans_b = n.trans_b;
    return std::make_unique<GemmLikeKernel>(c);
  }
  case Kind::FusedGemm: {
    GemmLikeKernel::Config c;
    c.name = "FusedGemmKernel";
    c.params = DefaultGemmParams(options);
    c.autotune = options.autotune;
    c.params.alpha = n.alpha;
    c.params.beta = n.beta;
    c.params.divisor = n.divisor;
    c.params.act = n.act;
    for (int i = 0; i < 3; ++i) c.params.act_param[i] = n.act_param[i];
    c.trans_a = n.trans_a;
    c.trans_b = n.trans_b;
    size_t k = 0;
    // inputs: A, [B if variable], [variable addend if has_mask], [residual];
    // consts: [B if captured], [bias if has_bias]
    if (n.b_is_const) { c.has_const_b = true; c.const_b = C(k++); }
    if (n.has_bias) { c.has_bias = true; c.bias = C(k++); }
    if (n.has_mask) { c.has_bias = true; c.bias_is_input = true; }  // a variable addend (attention mask)
    c.has_residual = n.has_residual;
    return std::make_unique<GemmLikeKernel>(c);
  }
  case Kind::ConvWithoutPadding:
  case Kind::ConvWithPadding: {
    fml_conv_params p;
    memset(&p, 0, sizeof(p));
    const size_t nd = n.strides.size();
    for (size_t i = 0; i < 2; ++i) {
      p.pads_begin[i] = i < nd ? n.pads.at(i) : 0;
      p.strides[i] = i < nd ? n.strides.at(i) : 1;
      p.dilations[i] = i < nd ? n.dilations.at(i) : 1;
    }
    p.group = n.group;
    p.act = n.act;
    p.precision = options.gemm_precision;
    const char *name = n.kind == Kind::ConvWithPadding ? "ConvWithPaddingKernel" : "ConvWithoutPaddingKernel";
    if (n.has_in_scale) return std::make_unique<ScaledConvKernel>(name, C(0), n.has_bias, n.has_bias ? C(1) : fml_tensor{}, p);
    return std::make_unique<ConvKernel>(name, C(0), n.has_bias, n.has_bias ? C(1) : fml_tensor{}, p);
  }
  case Kind::MaxPoolWithoutPadding:
    return std::make_unique<PoolKernel>("MaxPoolWithoutPaddingKernel", 0, n.kernel_shape, n.strides);
  case Kind::AveragePoolWithoutPadding:
    return std::make_unique<PoolKernel>("AveragePoolWithoutPaddingKernel", 1, n.kernel_shape, n.strides);
  }
  throw Error(std::string("no kernel for flow node kind ") + flow::KindName(n.kind));
}

}  // namespace kernel

namespace flow {
const char *KindName(Kind k) {
  static const char *names[] = {
      "AddConstant", "AddCommon", "AddDivErfAddMulMul", "AveragePoolWithoutPadding", "Cast", "Clip", "Concat2",
      "ConvWithoutPadding", "ConvWithPadding", "CumSum", "DivConstantRhs", "DivCommon", "Dropout", "Equal", "Erf",
      "Flatten", "GatherConstantIndexScalar", "GatherConstantIndicesTensor", "GatherConstantDataTensor",
      "GatherConstantDataTensorAddTensorLhsAddTensorLhs", "GemmConstantBias",
      "LayerNormalizationConstantScaleBias", "MatMul", "MaxPoolWithoutPadding", "MulConstant", "MulCommon", "Neg",
      "Not", "Pad", "Pow", "ReduceMean", "Relu", "Reshape", "Slice", "Softmax", "Sqrt", "Squeeze", "SubConstantLhs",
      "SubCommon", "Tanh", "Transpose", "Unsqueeze", "UnsqueezeSubLhsScalarMulRhsScalar",
      "WhereConstantCondConstantScalarY", "WhereConstantCondConstantTensorY", "Sigmoid", "Identity", "FusedGemm",
      "FusedSoftmax", "FusedLayerNorm", "Silu", "FusedAttention", "FusedMulAdd", "FusedMulAddChain", "Rotary", "SqueezeExciteGate"};
  return names[(int)k];
}
}  // namespace flow
}  // namespace fluidml
