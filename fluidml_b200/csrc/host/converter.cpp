// Converter: graph::Graph -> flow::Flow.  Picks the node *variant* of every ONNX operator
// from which operands are constant scalars ("constS", rank-0 initialisers), constant tensors
// ("constT") or variables ("var"), as src/worker/converter.cpp does (one convertXNode per
// operator, :354-2632).  Patterns the reference leaves to __builtin_unreachable()
// (:268-274) raise an Error here.
#include "converter.h"
#include <algorithm>
#include <numeric>

namespace fluidml {
namespace worker {
namespace {

using graph::Value;
using flow::Kind;

struct Ctx {
  const graph::Graph &g;
  flow::Flow &f;

  flow::RegionPtr Region(const std::string &name) {
    auto it = f.by_name.find(name);
    if (it != f.by_name.end()) return it->second;
    const Value &v = g.Get(name);
    auto r = std::make_shared<flow::Region>();
    r->name = name;
    r->meta = v.meta;
    r->layout = utils::GenDefaultLayout(v.meta.GetRank());
    switch (v.kind) {
    case Value::kInput: r->kind = flow::Region::kInput; break;
    case Value::kOutput: r->kind = flow::Region::kOutput; break;
    case Value::kConstant: r->kind = flow::Region::kConstant; r->constant = v.constant; break;
    default: r->kind = flow::Region::kInner; break;
    }
    f.regions.push_back(r);
    f.by_name[name] = r;
    return r;
  }
  bool IsVar(const std::string &n) const { return g.Get(n).kind != Value::kConstant; }
  bool IsConstS(const std::string &n) const { return g.Get(n).IsScalarConstant(); }
  bool IsConstT(const std::string &n) const { return g.Get(n).IsTensorConstant(); }
  const Tensor &Const(const std::string &n) const { return *g.Get(n).constant; }
};

[[noreturn]] void Unsupported(const graph::Node &n, const std::string &why) {
  throw Error("operator " + n.op_type + " (node '" + n.name + "'): " + why);
}

flow::NodePtr Make(Ctx &c, const graph::Node &n, Kind kind) {
  auto node = std::make_shared<flow::Node>();
  node->kind = kind;
  node->name = n.name;
  node->output = c.Region(n.outputs.at(0));
  return node;
}

void NeedInputs(const graph::Node &n, size_t lo, size_t hi) {
  if (n.inputs.size() < lo || n.inputs.size() > hi) Unsupported(n, "unexpected number of inputs");
}

size_t RowsBytes(const Meta &m, int64_t axis) {  // one element per row along `axis`
  int64_t n = 1;
  for (size_t i = 0; i < m.GetRank(); ++i)
    if ((int64_t)i != axis) n *= m.GetShape()[i];
  return (size_t)n * GetSizeFromType(m.GetType());
}

// Add / Mul: (var,var), (constT,var), (var,constT) -> Common; (var,constS)/(constS,var) ->
// Constant(type, value)   [converter.cpp:354-452, :1584-1669]
flow::NodePtr ConvertAddMul(Ctx &c, const graph::Node &n, Kind common, Kind constant) {
  NeedInputs(n, 2, 2);
  const std::string &a = n.inputs[0], &b = n.inputs[1];
  if (c.IsConstS(a) != c.IsConstS(b) || (c.IsConstS(a) && c.IsConstS(b))) {
    if (c.IsConstS(a) && c.IsConstS(b)) Unsupported(n, "both operands are scalar constants");
    const std::string &var = c.IsConstS(a) ? b : a, &cs = c.IsConstS(a) ? a : b;
    auto node = Make(c, n, constant);
    node->inputs = {c.Region(var)};
    node->scalar_type = c.Const(cs).GetMeta().GetType();
    node->value = c.Const(cs).AsDouble();
    return node;
  }
  if (!c.IsVar(a) && !c.IsVar(b)) Unsupported(n, "both operands are constant tensors");
  auto node = Make(c, n, common);
  node->inputs = {c.Region(a), c.Region(b)};
  return node;
}

flow::NodePtr ConvertUnary(Ctx &c, const graph::Node &n, Kind kind) {
  NeedInputs(n, 1, 1);
  if (!c.IsVar(n.inputs[0])) Unsupported(n, "input must be a variable tensor");
  auto node = Make(c, n, kind);
  node->inputs = {c.Region(n.inputs[0])};
  return node;
}

std::vector<int64_t> AxesOf(Ctx &c, const graph::Node &n, size_t input_index) {
  if (n.inputs.size() > input_index && !n.inputs[input_index].empty()) {
    if (!c.IsConstT(n.inputs[input_index]) && !c.IsConstS(n.inputs[input_index]))
      Unsupported(n, "axes must be a constant");
    return c.Const(n.inputs[input_index]).AsInts();
  }
  if (n.HasAttr("axes")) return n.Ints("axes");
  Unsupported(n, "axes are missing");
}

flow::NodePtr ConvertNode(Ctx &c, const graph::Node &n) {
  const std::string &op = n.op_type;
  if (op == "Add") return ConvertAddMul(c, n, Kind::AddCommon, Kind::AddConstant);
  if (op == "Mul") return ConvertAddMul(c, n, Kind::MulCommon, Kind::MulConstant);
  if (op == "Div") {  // (var,constS) -> DivConstantRhs; (var,var) -> DivCommon [:922-994]
    NeedInputs(n, 2, 2);
    if (c.IsVar(n.inputs[0]) && c.IsConstS(n.inputs[1])) {
      auto node = Make(c, n, Kind::DivConstantRhs);
      node->inputs = {c.Region(n.inputs[0])};
      node->scalar_type = c.Const(n.inputs[1]).GetMeta().GetType();
      node->value = c.Const(n.inputs[1]).AsDouble();
      return node;
    }
    if (c.IsVar(n.inputs[0]) && c.IsVar(n.inputs[1])) {
      auto node = Make(c, n, Kind::DivCommon);
      node->inputs = {c.Region(n.inputs[0]), c.Region(n.inputs[1])};
      return node;
    }
    Unsupported(n, "accepted operand patterns are (variable, scalar constant) and (variable, variable)");
  }
  if (op == "Sub") {  // (constS,var) -> SubConstantLhs; (var,var) -> SubCommon [:2264-2345]
    NeedInputs(n, 2, 2);
    if (c.IsConstS(n.inputs[0]) && c.IsVar(n.inputs[1])) {
      auto node = Make(c, n, Kind::SubConstantLhs);
      node->inputs = {c.Region(n.inputs[1])};
      node->scalar_type = c.Const(n.inputs[0]).GetMeta().GetType();
      node->value = c.Const(n.inputs[0]).AsDouble();
      return node;
    }
    if (c.IsVar(n.inputs[0]) && c.IsVar(n.inputs[1])) {
      auto node = Make(c, n, Kind::SubCommon);
      node->inputs = {c.Region(n.inputs[0]), c.Region(n.inputs[1])};
      return node;
    }
    Unsupported(n, "accepted operand patterns are (scalar constant, variable) and (variable, variable)");
  }
  if (op == "Pow") {  // (var,constS) only [:1812-1855]
    NeedInputs(n, 2, 2);
    if (!(c.IsVar(n.inputs[0]) && c.IsConstS(n.inputs[1]))) Unsupported(n, "exponent must be a scalar constant");
    auto node = Make(c, n, Kind::Pow);
    node->inputs = {c.Region(n.inputs[0])};
    node->value = c.Const(n.inputs[1]).AsDouble();
    return node;
  }
  if (op == "Erf") return ConvertUnary(c, n, Kind::Erf);
  if (op == "Tanh") return ConvertUnary(c, n, Kind::Tanh);
  if (op == "Sqrt") return ConvertUnary(c, n, Kind::Sqrt);
  if (op == "Neg") return ConvertUnary(c, n, Kind::Neg);
  if (op == "Not") return ConvertUnary(c, n, Kind::Not);
  if (op == "Relu") return ConvertUnary(c, n, Kind::Relu);
  if (op == "Sigmoid") return ConvertUnary(c, n, Kind::Sigmoid);
  if (op == "Identity") return ConvertUnary(c, n, Kind::Identity);
  if (op == "Dropout") {  // identity [:996-1058]
    auto node = Make(c, n, Kind::Dropout);
    node->inputs = {c.Region(n.inputs.at(0))};
    return node;
  }
  if (op == "Cast") {  // `to` attribute [:596-639]
    auto node = ConvertUnary(c, n, Kind::Cast);
    if (!n.HasAttr("to")) Unsupported(n, "missing 'to'");
    return node;
  }
  if (op == "Clip") {  // (X, constS min, constS max) or min/max attributes [:641-710]
    auto node = Make(c, n, Kind::Clip);
    node->inputs = {c.Region(n.inputs.at(0))};
    node->value = -3.402823466e+38;
    node->value2 = 3.402823466e+38;
    if (n.inputs.size() > 1 && !n.inputs[1].empty()) node->value = c.Const(n.inputs[1]).AsDouble();
    else if (n.HasAttr("min")) node->value = n.Float("min", 0);
    if (n.inputs.size() > 2 && !n.inputs[2].empty()) node->value2 = c.Const(n.inputs[2]).AsDouble();
    else if (n.HasAttr("max")) node->value2 = n.Float("max", 0);
    return node;
  }
  if (op == "MatMul") {  // any two operands, at least one variable [:1488-1525]
    NeedInputs(n, 2, 2);
    if (!c.IsVar(n.inputs[0]) && !c.IsVar(n.inputs[1])) Unsupported(n, "both operands are constants");
    auto node = Make(c, n, Kind::MatMul);
    node->inputs = {c.Region(n.inputs[0]), c.Region(n.inputs[1])};
    return node;
  }
  if (op == "Gemm") {  // A var, B constT, C constT; alpha/beta/transA/transB [:1357-1422]
    NeedInputs(n, 3, 3);
    if (!c.IsVar(n.inputs[0]) || !c.IsConstT(n.inputs[1]) || !c.IsConstT(n.inputs[2]))
      Unsupported(n, "needs a variable A and constant-tensor B and C");
    auto node = Make(c, n, Kind::GemmConstantBias);
    node->inputs = {c.Region(n.inputs[0])};
    node->consts = {c.Region(n.inputs[1]), c.Region(n.inputs[2])};
    // ONNX defaults (1, 1).  The reference defaults absent alpha/beta to 0
    // (converter.cpp:1394-1409), which no exporter relies on.
    node->alpha = n.Float("alpha", 1.0f);
    node->beta = n.Float("beta", 1.0f);
    node->trans_a = n.Int("transA", 0) != 0;
    node->trans_b = n.Int("transB", 0) != 0;
    return node;
  }
  if (op == "Softmax") {  // axis default -1 [:2111-2157, node.cpp:1370-1372]
    auto node = ConvertUnary(c, n, Kind::Softmax);
    const int64_t rank = (int64_t)node->inputs[0]->meta.GetRank();
    int64_t axis = n.Int("axis", -1);
    if (axis < 0) axis += rank;
    if (axis < 0 || axis >= rank) Unsupported(n, "axis out of range");
    node->axis = axis;
    node->reference_buffer_size = RowsBytes(node->inputs[0]->meta, axis);
    return node;
  }
  if (op == "LayerNormalization") {  // X var, scale constT, bias constT [:1424-1486]
    NeedInputs(n, 3, 3);
    if (!c.IsVar(n.inputs[0]) || !c.IsConstT(n.inputs[1]) || !c.IsConstT(n.inputs[2]))
      Unsupported(n, "needs a variable X and constant scale and bias");
    auto node = Make(c, n, Kind::LayerNormalizationConstantScaleBias);
    node->inputs = {c.Region(n.inputs[0])};
    node->consts = {c.Region(n.inputs[1]), c.Region(n.inputs[2])};
    const int64_t rank = (int64_t)node->inputs[0]->meta.GetRank();
    int64_t axis = n.Int("axis", -1);  // ONNX default; the reference's node default is 1 (node.h:672)
    if (axis < 0) axis += rank;
    if (axis != rank - 1) Unsupported(n, "only normalisation over the last axis is implemented");
    node->axis = axis;
    node->epsilon = n.Float("epsilon", 1e-5f);
    node->reference_buffer_size = RowsBytes(node->inputs[0]->meta, axis);
    return node;
  }
  if (op == "Gather") {  // [:1192-1292]
    NeedInputs(n, 2, 2);
    int64_t axis = n.Int("axis", 0);
    const std::string &data = n.inputs[0], &ind = n.inputs[1];
    if (axis < 0) axis += (int64_t)c.g.Get(data).meta.GetRank();
    if (c.IsVar(data) && c.IsConstS(ind)) {
      auto node = Make(c, n, Kind::GatherConstantIndexScalar);
      node->inputs = {c.Region(data)};
      node->consts = {c.Region(ind)};
      node->axis = axis;
      node->value = (double)c.Const(ind).AsInt();
      return node;
    }
    if (c.IsVar(data) && c.IsConstT(ind)) {
      auto node = Make(c, n, Kind::GatherConstantIndicesTensor);
      node->inputs = {c.Region(data)};
      node->consts = {c.Region(ind)};
      node->axis = axis;
      return node;
    }
    if (c.IsConstT(data) && c.IsVar(ind)) {
      if (axis != 0) Unsupported(n, "a constant table is gathered along axis 0 only");
      auto node = Make(c, n, Kind::GatherConstantDataTensor);
      node->inputs = {c.Region(ind)};
      node->consts = {c.Region(data)};
      node->axis = 0;
      return node;
    }
    Unsupported(n, "accepted patterns: (variable, constant index) and (constant table, variable indices)");
  }
  if (op == "Where") {  // cond constT (bool), X var, Y constS / constT [:2559-2632]
    NeedInputs(n, 3, 3);
    if (!c.IsConstT(n.inputs[0]) || !c.IsVar(n.inputs[1]))
      Unsupported(n, "needs a constant condition and a variable X");
    if (c.IsConstS(n.inputs[2])) {
      auto node = Make(c, n, Kind::WhereConstantCondConstantScalarY);
      node->inputs = {c.Region(n.inputs[1])};
      node->consts = {c.Region(n.inputs[0])};
      node->value = c.Const(n.inputs[2]).AsDouble();
      return node;
    }
    if (c.IsConstT(n.inputs[2])) {
      auto node = Make(c, n, Kind::WhereConstantCondConstantTensorY);
      node->inputs = {c.Region(n.inputs[1])};
      node->consts = {c.Region(n.inputs[0]), c.Region(n.inputs[2])};
      return node;
    }
    Unsupported(n, "Y must be a constant");
  }
  if (op == "Reshape") {  // shape must be constant; only the static shapes matter [:1966-2023]
    NeedInputs(n, 2, 2);
    if (!c.IsConstT(n.inputs[1])) Unsupported(n, "shape must be a constant tensor");
    auto node = Make(c, n, Kind::Reshape);
    node->inputs = {c.Region(n.inputs[0])};
    if (node->inputs[0]->meta.GetElementsNum() != node->output->meta.GetElementsNum())
      Unsupported(n, "element count changes");
    return node;
  }
  if (op == "Transpose") {  // perm default = reversed [:2390-2443]
    auto node = ConvertUnary(c, n, Kind::Transpose);
    node->perm = n.Ints("perm");
    const size_t rank = node->inputs[0]->meta.GetRank();
    if (node->perm.empty())
      for (size_t i = 0; i < rank; ++i) node->perm.push_back((int64_t)(rank - 1 - i));
    if (node->perm.size() != rank) Unsupported(n, "perm has the wrong length");
    return node;
  }
  if (op == "Unsqueeze" || op == "Squeeze") {  // axes constT or attribute [:2445-2494, :2202-2262]
    auto node = Make(c, n, op == "Unsqueeze" ? Kind::Unsqueeze : Kind::Squeeze);
    node->inputs = {c.Region(n.inputs.at(0))};
    node->axes = AxesOf(c, n, 1);
    return node;
  }
  if (op == "Flatten") {  // axis default 1 [:1147-1190]
    auto node = ConvertUnary(c, n, Kind::Flatten);
    node->axis = n.Int("axis", 1);
    return node;
  }
  if (op == "ReduceMean") {  // keepdims = 1 only [:1857-1924, reduce_mean.cpp:56-63]
    auto node = Make(c, n, Kind::ReduceMean);
    node->inputs = {c.Region(n.inputs.at(0))};
    node->axes = AxesOf(c, n, 1);
    if (n.Int("keepdims", 1) != 1) Unsupported(n, "only keepdims=1 is implemented");
    const int64_t rank = (int64_t)node->inputs[0]->meta.GetRank();
    for (auto &a : node->axes) if (a < 0) a += rank;
    return node;
  }
  if (op == "Slice") {  // starts/ends/axes/steps all constant, steps 1 [:2025-2109]
    if (n.inputs.size() < 3) Unsupported(n, "needs constant starts and ends");
    auto node = Make(c, n, Kind::Slice);
    node->inputs = {c.Region(n.inputs[0])};
    const size_t rank = node->inputs[0]->meta.GetRank();
    std::vector<int64_t> starts = c.Const(n.inputs[1]).AsInts(), axes;
    if (n.inputs.size() > 3 && !n.inputs[3].empty()) axes = c.Const(n.inputs[3]).AsInts();
    else { axes.resize(starts.size()); std::iota(axes.begin(), axes.end(), 0); }
    if (n.inputs.size() > 4 && !n.inputs[4].empty())
      for (int64_t s : c.Const(n.inputs[4]).AsInts()) if (s != 1) Unsupported(n, "steps must be 1");
    node->starts.assign(rank, 0);
    for (size_t i = 0; i < axes.size(); ++i) {
      int64_t ax = axes[i] < 0 ? axes[i] + (int64_t)rank : axes[i];
      int64_t st = starts[i] < 0 ? starts[i] + node->inputs[0]->meta.GetShape()[ax] : starts[i];
      node->starts.at(ax) = st;
    }
    for (size_t i = 0; i < rank; ++i)
      if (node->starts[i] + node->output->meta.GetShape()[i] > node->inputs[0]->meta.GetShape()[i])
        Unsupported(n, "slice leaves the input");
    return node;
  }
  if (op == "Concat") {  // exactly two inputs [:712-756]
    NeedInputs(n, 2, 2);
    auto node = Make(c, n, Kind::Concat2);
    node->inputs = {c.Region(n.inputs[0]), c.Region(n.inputs[1])};
    int64_t axis = n.Int("axis", 0);
    if (axis < 0) axis += (int64_t)node->output->meta.GetRank();
    node->axis = axis;
    return node;
  }
  if (op == "Pad") {  // pads constT [2*rank]; constant mode, value 0 [:1750-1810]
    if (n.inputs.size() < 2) Unsupported(n, "needs constant pads");
    auto node = Make(c, n, Kind::Pad);
    node->inputs = {c.Region(n.inputs[0])};
    node->pads = c.Const(n.inputs[1]).AsInts();
    if (node->pads.size() != 2 * node->inputs[0]->meta.GetRank()) Unsupported(n, "pads has the wrong length");
    return node;
  }
  if (op == "Equal") {  // (var int64, constS) [:1060-1106]
    NeedInputs(n, 2, 2);
    if (!c.IsVar(n.inputs[0]) || !c.IsConstS(n.inputs[1])) Unsupported(n, "needs (variable, scalar constant)");
    auto node = Make(c, n, Kind::Equal);
    node->inputs = {c.Region(n.inputs[0])};
    node->scalar_type = c.Const(n.inputs[1]).GetMeta().GetType();
    node->value = c.Const(n.inputs[1]).AsDouble();
    return node;
  }
  if (op == "CumSum") {  // axis constS; exclusive = reverse = 0 [:863-920]
    NeedInputs(n, 2, 2);
    if (n.Int("exclusive", 0) || n.Int("reverse", 0)) Unsupported(n, "exclusive/reverse are not implemented");
    auto node = Make(c, n, Kind::CumSum);
    node->inputs = {c.Region(n.inputs[0])};
    int64_t axis = c.Const(n.inputs[1]).AsInt();
    if (axis < 0) axis += (int64_t)node->inputs[0]->meta.GetRank();
    node->axis = axis;
    return node;
  }
  if (op == "Conv") {  // X var, W constT, optional B constT [:758-861]
    NeedInputs(n, 2, 3);
    if (!c.IsVar(n.inputs[0]) || !c.IsConstT(n.inputs[1])) Unsupported(n, "needs a variable X and constant W");
    const size_t nd = c.g.Get(n.inputs[0]).meta.GetRank() - 2;
    std::vector<int64_t> pads = n.Ints("pads");
    if (pads.empty()) pads.assign(2 * nd, 0);
    const bool padded = std::any_of(pads.begin(), pads.end(), [](int64_t p) { return p != 0; });
    auto node = Make(c, n, padded ? Kind::ConvWithPadding : Kind::ConvWithoutPadding);
    node->inputs = {c.Region(n.inputs[0])};
    node->consts = {c.Region(n.inputs[1])};
    if (n.inputs.size() > 2 && !n.inputs[2].empty()) { node->consts.push_back(c.Region(n.inputs[2])); node->has_bias = true; }
    node->pads = pads;
    node->strides = n.Ints("strides");
    node->dilations = n.Ints("dilations");
    if (node->strides.empty()) node->strides.assign(nd, 1);
    if (node->dilations.empty()) node->dilations.assign(nd, 1);
    node->kernel_shape = n.Ints("kernel_shape");
    node->group = n.Int("group", 1);
    if (nd < 1 || nd > 2) Unsupported(n, "only 1-D and 2-D convolutions are implemented");
    for (size_t i = 0; i < nd; ++i)
      if (pads[i] != pads[i + nd]) {
        // asymmetric padding is fine for the implicit-padding kernel as long as the output
        // shape in value_info agrees; nothing to do
      }
    if (padded) {  // size of the padded copy the reference materialises (node.cpp:500-519)
      std::vector<int64_t> s = node->inputs[0]->meta.GetShape();
      for (size_t i = 0; i < nd; ++i) s[i + 2] += pads[i] + pads[i + nd];
      node->reference_buffer_size = (size_t)std::accumulate(s.begin(), s.end(), (int64_t)1, std::multiplies<int64_t>()) * 4;
    }
    return node;
  }
  if (op == "MaxPool" || op == "AveragePool") {  // no padding [:1527-1582, :519-594]
    auto node = ConvertUnary(c, n, op == "MaxPool" ? Kind::MaxPoolWithoutPadding : Kind::AveragePoolWithoutPadding);
    for (int64_t p : n.Ints("pads")) if (p != 0) Unsupported(n, "pools take no padding");
    node->kernel_shape = n.Ints("kernel_shape");
    node->strides = n.Ints("strides");
    if (node->kernel_shape.size() != 2) Unsupported(n, "only 2-D pools are implemented");
    if (node->strides.empty()) node->strides.assign(2, 1);
    return node;
  }
  Unsupported(n, "no flow node exists for this operator");
}

}  // namespace

flow::Flow Converter::Run(const graph::Graph &g) {
  flow::Flow f;
  f.name = g.name;
  Ctx c{g, f};
  f.inputs = g.inputs;
  f.outputs = g.outputs;
  for (const auto &name : g.inputs) c.Region(name);
  for (const auto &name : g.outputs) c.Region(name);
  for (const graph::Node &n : g.nodes) {
    if (n.outputs.size() < 1) throw Error("node '" + n.name + "' has no output");
    f.nodes.push_back(ConvertNode(c, n));
  }
  return f;
}

}  // namespace worker
}  // namespace fluidml
