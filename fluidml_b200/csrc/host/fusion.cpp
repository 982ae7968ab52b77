#include "fusion.h"
#include <cstdlib>
#include "fluidml_cuda.h"
#include <algorithm>
#include <unordered_map>
#include <unordered_set>

namespace fluidml {
namespace worker {
namespace {

using flow::Kind;
using flow::NodePtr;
using flow::RegionPtr;

struct Rewriter {
  flow::Flow &f;
  std::unordered_map<const flow::Region *, std::vector<NodePtr>> consumers;
  std::unordered_map<const flow::Region *, NodePtr> producer;
  std::unordered_set<const flow::Node *> dead;

  explicit Rewriter(flow::Flow &flow) : f(flow) { Index(); }

  void Index() {
    consumers.clear();
    producer.clear();
    for (const auto &n : f.nodes) {
      if (dead.count(n.get())) continue;
      producer[n->output.get()] = n;
      for (const auto &r : n->inputs) consumers[r.get()].push_back(n);
    }
  }
  // The only consumer of `r`, provided `r` is an inner tensor nobody else reads.
  NodePtr Sole(const RegionPtr &r) {
    if (r->kind != flow::Region::kInner) return nullptr;
    auto it = consumers.find(r.get());
    if (it == consumers.end() || it->second.size() != 1) return nullptr;
    return it->second[0];
  }
  NodePtr SoleOfKind(const RegionPtr &r, Kind k) {
    NodePtr n = Sole(r);
    return n && n->kind == k ? n : nullptr;
  }
  void Kill(const NodePtr &n) { dead.insert(n.get()); }
  void Commit() {
    f.nodes.erase(std::remove_if(f.nodes.begin(), f.nodes.end(),
                                 [&](const NodePtr &n) { return dead.count(n.get()) != 0; }),
                  f.nodes.end());
    dead.clear();
    Index();
  }
};

bool IsConst(const RegionPtr &r) { return r->kind == flow::Region::kConstant; }

// The operand of a two-input node that is not `x`.
RegionPtr Other(const NodePtr &n, const RegionPtr &x) { return n->inputs[0] == x ? n->inputs[1] : n->inputs[0]; }

bool IsGemmLike(const NodePtr &n) {
  return n->kind == Kind::MatMul || n->kind == Kind::FusedGemm || n->kind == Kind::GemmConstantBias;
}

// MatMul / Gemm -> FusedGemm, keeping operands and attributes.
void PromoteToFusedGemm(const NodePtr &n) {
  if (n->kind == Kind::FusedGemm) return;
  if (n->kind == Kind::MatMul) {
    if (IsConst(n->inputs[1])) {
      n->consts = {n->inputs[1]};
      n->inputs = {n->inputs[0]};
      n->b_is_const = true;
    }
  } else {  // GemmConstantBias: consts = {B, C}
    n->b_is_const = true;
    n->has_bias = true;
  }
  n->kind = Kind::FusedGemm;
}

// ---- gather_add_fusion.cpp: Gather(table, ids) + constT + constT -> one embedding kernel
bool FuseEmbedding(Rewriter &rw, const NodePtr &g) {
  if (g->kind != Kind::GatherConstantDataTensor || g->consts[0]->meta.GetType() != Type::kFloat32) return false;
  NodePtr a0 = rw.SoleOfKind(g->output, Kind::AddCommon);
  if (!a0 || !IsConst(Other(a0, g->output))) return false;
  NodePtr a1 = rw.SoleOfKind(a0->output, Kind::AddCommon);
  if (!a1 || !IsConst(Other(a1, a0->output))) return false;
  g->kind = Kind::GatherConstantDataTensorAddTensorLhsAddTensorLhs;
  g->consts = {g->consts[0], Other(a0, g->output), Other(a1, a0->output)};
  g->output = a1->output;
  rw.Kill(a0);
  rw.Kill(a1);
  return true;
}

// ---- unsqueeze_sub_mul_fusion.cpp: Unsqueeze(+Unsqueeze) -> c - x -> * m
bool FuseMask(Rewriter &rw, const NodePtr &u) {
  if (u->kind != Kind::Unsqueeze || u->inputs[0]->meta.GetType() != Type::kFloat32) return false;
  std::vector<NodePtr> chain = {u};
  NodePtr cur = u;
  while (NodePtr nx = rw.SoleOfKind(cur->output, Kind::Unsqueeze)) { chain.push_back(nx); cur = nx; }
  NodePtr sub = rw.SoleOfKind(cur->output, Kind::SubConstantLhs);
  if (!sub) return false;
  NodePtr mul = rw.SoleOfKind(sub->output, Kind::MulConstant);
  if (!mul) return false;
  u->kind = Kind::UnsqueezeSubLhsScalarMulRhsScalar;
  u->value = sub->value;
  u->value2 = mul->value;
  u->output = mul->output;
  for (size_t i = 1; i < chain.size(); ++i) rw.Kill(chain[i]);
  rw.Kill(sub);
  rw.Kill(mul);
  return true;
}

// ---- MatMul/Gemm + constant bias -> epilogue
bool FuseBias(Rewriter &rw, const NodePtr &mm) {
  if (mm->kind != Kind::MatMul && !(mm->kind == Kind::FusedGemm && !mm->has_bias && !mm->has_mask && mm->act == 0 && !mm->has_residual)) return false;
  NodePtr add = rw.SoleOfKind(mm->output, Kind::AddCommon);
  if (!add) return false;
  RegionPtr bias = Other(add, mm->output);
  if (!IsConst(bias) || bias->meta.GetType() != Type::kFloat32) return false;
  if (add->output->meta != mm->output->meta) return false;  // the bias must not widen the result
  PromoteToFusedGemm(mm);
  mm->consts.push_back(bias);
  mm->has_bias = true;
  mm->output = add->output;
  rw.Kill(add);
  return true;
}

// ---- add_div_erf_add_mul_fusion.cpp: t -> t/c0 -> erf -> +c1 -> t*(.) -> *c2
// `t` is produced by `src`; returns the final Mul node and the constants.
bool MatchGelu(Rewriter &rw, const RegionPtr &t, NodePtr &div, NodePtr &erf, NodePtr &add, NodePtr &mul0, NodePtr &mul1) {
  if (t->kind != flow::Region::kInner) return false;
  auto it = rw.consumers.find(t.get());
  if (it == rw.consumers.end() || it->second.size() != 2) return false;
  div = mul0 = nullptr;
  for (const auto &c : it->second) {
    if (c->kind == Kind::DivConstantRhs) div = c;
    else if (c->kind == Kind::MulCommon) mul0 = c;
  }
  if (!div || !mul0) return false;
  erf = rw.SoleOfKind(div->output, Kind::Erf);
  if (!erf) return false;
  add = rw.SoleOfKind(erf->output, Kind::AddConstant);
  if (!add) return false;
  if (rw.Sole(add->output) != mul0 || Other(mul0, t) != add->output) return false;
  mul1 = rw.SoleOfKind(mul0->output, Kind::MulConstant);
  return mul1 != nullptr;
}

bool FuseGeluIntoGemm(Rewriter &rw, const NodePtr &mm) {
  if (!IsGemmLike(mm) || mm->act != 0 || mm->has_residual) return false;
  NodePtr div, erf, add, mul0, mul1;
  if (!MatchGelu(rw, mm->output, div, erf, add, mul0, mul1)) return false;
  PromoteToFusedGemm(mm);
  mm->act = FML_ACT_GELU_ERF;
  mm->act_param[0] = (float)div->value;
  mm->act_param[1] = (float)add->value;
  mm->act_param[2] = (float)mul1->value;
  mm->output = mul1->output;
  for (const auto &k : {div, erf, add, mul0, mul1}) rw.Kill(k);
  return true;
}

// Add(x, const bias) followed by the GELU chain, when no GEMM produced x: the reference's
// AddDivErfAddMulMul kernel.
bool FuseBiasGelu(Rewriter &rw, const NodePtr &a) {
  if (a->kind != Kind::AddCommon) return false;
  RegionPtr bias, x;
  if (IsConst(a->inputs[0]) && !IsConst(a->inputs[1])) { bias = a->inputs[0]; x = a->inputs[1]; }
  else if (IsConst(a->inputs[1]) && !IsConst(a->inputs[0])) { bias = a->inputs[1]; x = a->inputs[0]; }
  else return false;
  if (a->output->meta != x->meta) return false;
  NodePtr div, erf, add, mul0, mul1;
  if (!MatchGelu(rw, a->output, div, erf, add, mul0, mul1)) return false;
  a->kind = Kind::AddDivErfAddMulMul;
  a->inputs = {x};
  a->consts = {bias};
  a->act_param[0] = (float)div->value;
  a->act_param[1] = (float)add->value;
  a->act_param[2] = (float)mul1->value;
  a->output = mul1->output;
  for (const auto &k : {div, erf, add, mul0, mul1}) rw.Kill(k);
  return true;
}

// ---- GEMM -> Tanh / Relu / Sigmoid
bool FuseActivation(Rewriter &rw, const NodePtr &mm) {
  const bool conv = mm->kind == Kind::ConvWithPadding || mm->kind == Kind::ConvWithoutPadding;
  if (!(IsGemmLike(mm) || conv) || mm->act != 0 || mm->has_residual) return false;
  NodePtr act = rw.Sole(mm->output);
  if (!act) return false;
  int code = act->kind == Kind::Tanh ? FML_ACT_TANH : act->kind == Kind::Relu ? FML_ACT_RELU
             : act->kind == Kind::Sigmoid ? FML_ACT_SIGMOID : 0;
  if (!code) return false;
  if (!conv) PromoteToFusedGemm(mm);
  mm->act = code;
  mm->output = act->output;
  rw.Kill(act);
  return true;
}

// ---- GEMM + residual Add -> epilogue
bool FuseResidual(Rewriter &rw, const NodePtr &mm) {
  if (!IsGemmLike(mm) || mm->has_residual) return false;
  NodePtr add = rw.SoleOfKind(mm->output, Kind::AddCommon);
  if (!add) return false;
  RegionPtr res = Other(add, mm->output);
  if (IsConst(res) || res->meta != mm->output->meta || add->output->meta != mm->output->meta) return false;
  // the residual must not itself depend on this GEMM: it would, only if the GEMM's output had
  // another consumer, which Sole() excluded
  PromoteToFusedGemm(mm);
  mm->inputs.push_back(res);
  mm->has_residual = true;
  mm->output = add->output;
  rw.Kill(add);
  return true;
}

// ---- Add(x, r) -> LayerNorm, when the Add did not fold into a GEMM
bool FuseAddLayerNorm(Rewriter &rw, const NodePtr &add) {
  if (add->kind != Kind::AddCommon || IsConst(add->inputs[0]) || IsConst(add->inputs[1])) return false;
  if (add->inputs[0]->meta != add->output->meta || add->inputs[1]->meta != add->output->meta) return false;
  NodePtr ln = rw.SoleOfKind(add->output, Kind::LayerNormalizationConstantScaleBias);
  if (!ln) return false;
  ln->kind = Kind::FusedLayerNorm;
  ln->inputs = {add->inputs[0], add->inputs[1]};
  ln->has_residual = true;
  rw.Kill(add);
  return true;
}

// ---- x / c -> + mask -> Softmax  (attention scores); the mask may also be a constant-condition
// Where that replaces masked scores by a scalar (a causal mask): Where(cond, s, y) feeds the
// softmax the same values as s + m with m = cond ? 0 : y whenever y is so negative that
// s + y rounds to y (the usual float lowest), so it becomes a baked additive mask.
bool FuseScaledMaskedSoftmax(Rewriter &rw, const NodePtr &div) {
  if (div->kind != Kind::DivConstantRhs) return false;
  NodePtr nx = rw.Sole(div->output);
  if (!nx) return false;
  NodePtr add = nullptr, where = nullptr, sm = nullptr;
  if (nx->kind == Kind::AddCommon) {
    add = nx;
    if (add->output->meta != div->output->meta) return false;
    sm = rw.SoleOfKind(add->output, Kind::Softmax);
  } else if (nx->kind == Kind::WhereConstantCondConstantScalarY) {
    where = nx;
    // s + y == y needs |y| >= 2^25 |s|: accept the float lowest and anything within 2^-40 of it
    if (where->output->meta != div->output->meta || !(where->value <= -3.0e26) ||
        where->consts.empty() || !where->consts[0]->constant)
      return false;
    sm = rw.SoleOfKind(where->output, Kind::Softmax);
  } else if (nx->kind == Kind::Softmax) {
    sm = nx;
  }
  if (!sm || sm->axis != (int64_t)sm->output->meta.GetRank() - 1) return false;
  RegionPtr mask = nullptr;
  if (where) {
    const RegionPtr &cond = where->consts[0];
    const int64_t n = (int64_t)cond->meta.GetElementsNum();
    std::vector<uint8_t> bytes((size_t)n * 4);
    float *m = reinterpret_cast<float *>(bytes.data());
    const float y = (float)where->value;
    for (int64_t i = 0; i < n; ++i) m[i] = cond->constant->AsInt(i) ? 0.0f : y;
    mask = std::make_shared<flow::Region>();
    mask->kind = flow::Region::kConstant;
    mask->name = where->name + "_additive_mask";
    mask->meta = Meta(Type::kFloat32, cond->meta.GetShape());
    mask->layout = utils::GenDefaultLayout(cond->meta.GetRank());
    mask->constant = std::make_shared<Tensor>(mask->meta, std::move(bytes));
    rw.f.regions.push_back(mask);
    rw.f.by_name[mask->name] = mask;
  }
  sm->kind = Kind::FusedSoftmax;
  sm->divisor = (float)div->value;
  sm->inputs = {div->inputs[0]};
  if (add) {
    sm->inputs.push_back(Other(add, div->output));
    sm->has_mask = true;
    rw.Kill(add);
  } else if (where) {
    sm->inputs.push_back(mask);
    sm->has_mask = true;
    rw.Kill(where);
  }
  rw.Kill(div);
  return true;
}

// ---- MatMul(Q, K^T) -> [scaled, masked] Softmax -> MatMul(P, V): one attention kernel when
// K and V of a head fit in shared memory
bool FuseAttention(Rewriter &rw, const NodePtr &qk) {
  if (qk->kind != Kind::MatMul || qk->inputs.size() != 2 || IsConst(qk->inputs[0]) || IsConst(qk->inputs[1])) return false;
  NodePtr sm = rw.Sole(qk->output);
  if (!sm || (sm->kind != Kind::Softmax && sm->kind != Kind::FusedSoftmax) || sm->inputs[0] != qk->output) return false;
  const size_t rank = sm->output->meta.GetRank();
  if (rank < 2 || rank > 4 || sm->axis != (int64_t)rank - 1) return false;
  NodePtr pv = rw.SoleOfKind(sm->output, Kind::MatMul);
  if (!pv || pv->inputs.size() != 2 || pv->inputs[0] != sm->output || IsConst(pv->inputs[1])) return false;
  const RegionPtr &q = qk->inputs[0], &kt = qk->inputs[1], &v = pv->inputs[1];
  const auto &qs = q->meta.GetShape(), &ks = kt->meta.GetShape(), &vs = v->meta.GetShape();
  if (qs.size() != rank || ks.size() != rank || vs.size() != rank) return false;
  if (q->meta.GetType() != Type::kFloat32 || kt->meta.GetType() != Type::kFloat32 || v->meta.GetType() != Type::kFloat32) return false;
  for (size_t i = 0; i + 2 < rank; ++i)
    if (qs[i] != ks[i] || qs[i] != vs[i]) return false;  // no batch broadcasting between the operands
  if (!fml_attention_supported(qs[rank - 2], ks[rank - 1], qs[rank - 1], vs[rank - 1])) return false;
  // The CUDA-core fused kernel computes in fp32 FMA (about 10 TFLOP/s): it wins while the three
  // launches it replaces are latency-bound; larger blocks are fused only when the tensor-core
  // attention kernel takes their head sizes (otherwise the score products are faster as GEMMs).
  double flops = 4.0 * (double)qs[rank - 2] * (double)ks[rank - 1] * (double)qs[rank - 1];
  for (size_t i = 0; i + 2 < rank; ++i) flops *= (double)qs[i];
  {
    // FLUIDML_ATTENTION_FUSION_MFLOP moves the limit (for measurements); blocks the tensor-core
    // kernel takes are fused up to `tc_limit`: beyond a few key blocks its serial phases lose to
    // the two batched tensor-core GEMMs around a softmax.
    static const double limit = [] { const char *e = getenv("FLUIDML_ATTENTION_FUSION_MFLOP"); return e ? atof(e) * 1e6 : 256e6; }();
    static const double tc_limit = [] { const char *e = getenv("FLUIDML_ATTENTION_TC_FUSION_MFLOP"); return e ? atof(e) * 1e6 : 256e6; }();
    const bool tc = fml_attention_on_tensor_cores(qs[rank - 2], ks[rank - 1], qs[rank - 1], vs[rank - 1]) != 0;
    if (flops > (tc ? std::max(limit, tc_limit) : limit)) return false;
  }
  qk->kind = Kind::FusedAttention;
  qk->inputs = {q, kt, v};
  qk->divisor = sm->kind == Kind::FusedSoftmax ? sm->divisor : 1.0f;
  qk->has_mask = sm->kind == Kind::FusedSoftmax && sm->has_mask;
  if (qk->has_mask) qk->inputs.push_back(sm->inputs[1]);
  qk->output = pv->output;
  rw.Kill(sm);
  rw.Kill(pv);
  return true;
}

// ---- Sigmoid(x) * x
bool FuseSilu(Rewriter &rw, const NodePtr &sg) {
  if (sg->kind != Kind::Sigmoid) return false;
  NodePtr mul = rw.SoleOfKind(sg->output, Kind::MulCommon);
  if (!mul || Other(mul, sg->output) != sg->inputs[0]) return false;
  sg->kind = Kind::Silu;
  sg->output = mul->output;
  rw.Kill(mul);
  return true;
}

// ---- Mul -> Add: one pass over the data instead of two (the span convolution of ConvBERT is a
// chain of nine such pairs, rotary embeddings two).  Same two roundings as the separate kernels.
bool FuseMulAdd(Rewriter &rw, const NodePtr &mul) {
  if (mul->kind != Kind::MulCommon || mul->inputs.size() != 2) return false;
  NodePtr add = rw.SoleOfKind(mul->output, Kind::AddCommon);
  if (!add || add->inputs.size() != 2 || add->inputs[0] == add->inputs[1]) return false;
  const RegionPtr other = Other(add, mul->output);
  for (const RegionPtr &r : {mul->inputs[0], mul->inputs[1], other, add->output})
    if (r->meta.GetType() != Type::kFloat32) return false;
  // the addend must not depend on this product (it cannot: the product has one consumer)
  mul->kind = Kind::FusedMulAdd;
  mul->inputs = {mul->inputs[0], mul->inputs[1], other};
  mul->output = add->output;
  rw.Kill(add);
  return true;
}

// ---- ReduceMean over H, W -> 1 x 1 Conv (+act) -> 1 x 1 Conv (+act): the gate of a squeeze-and-
// excite block.  Three launches that move a few kilobytes each become one (FLUIDML_FUSE_SE=0
// keeps them apart, for comparisons).
bool FuseSqueezeExcite(Rewriter &rw, const NodePtr &rm) {
  static const bool enabled = [] { const char *e = getenv("FLUIDML_FUSE_SE"); return !(e && e[0] == '0'); }();
  if (!enabled || rm->kind != Kind::ReduceMean) return false;
  const RegionPtr &x = rm->inputs[0];
  if (x->meta.GetRank() != 4 || x->meta.GetType() != Type::kFloat32) return false;
  std::vector<int64_t> axes = rm->axes;
  std::sort(axes.begin(), axes.end());
  if (axes != std::vector<int64_t>{2, 3}) return false;
  auto gate_conv = [](const NodePtr &cv, int64_t in_channels) {
    if (!cv || cv->group != 1 || cv->consts.empty() || cv->inputs.size() != 1) return false;
    const auto &ws = cv->consts[0]->meta.GetShape();
    if (ws.size() != 4 || ws[1] != in_channels || ws[2] != 1 || ws[3] != 1) return false;
    if (cv->consts[0]->meta.GetType() != Type::kFloat32 || !utils::IsDefaultLayout(cv->consts[0]->layout)) return false;
    if (cv->has_bias && (cv->consts.size() < 2 || cv->consts[1]->meta.GetElementsNum() != ws[0])) return false;
    for (int64_t s : cv->strides) if (s != 1) return false;
    for (int64_t d : cv->dilations) if (d != 1) return false;
    return cv->act == FML_ACT_NONE || cv->act == FML_ACT_RELU || cv->act == FML_ACT_TANH || cv->act == FML_ACT_SIGMOID ||
           cv->act == FML_ACT_SILU;
  };
  const int64_t C = x->meta.GetShape()[1];
  NodePtr c1 = rw.SoleOfKind(rm->output, Kind::ConvWithoutPadding);
  if (!gate_conv(c1, C)) return false;
  const int64_t Cr = c1->consts[0]->meta.GetShape()[0];
  NodePtr c2 = rw.SoleOfKind(c1->output, Kind::ConvWithoutPadding);
  if (!gate_conv(c2, Cr) || c2->consts[0]->meta.GetShape()[0] != C) return false;
  if (C > 4096 || Cr > 512 || x->meta.GetShape()[0] > 65535) return false;  // limits of fml_squeeze_excite_gate
  rm->kind = Kind::SqueezeExciteGate;
  rm->consts.clear();
  rm->consts.push_back(c1->consts[0]);
  if (c1->has_bias) rm->consts.push_back(c1->consts[1]);
  rm->consts.push_back(c2->consts[0]);
  if (c2->has_bias) rm->consts.push_back(c2->consts[1]);
  rm->has_bias = c1->has_bias;
  rm->has_bias2 = c2->has_bias;
  rm->act = c1->act;
  rm->act2 = c2->act;
  rm->output = c2->output;
  rw.Kill(c1);
  rw.Kill(c2);
  return true;
}

// ---- Mul(x [N, C, H, W], gate [N, C, 1, 1]) -> group-1 Conv: the gate multiplies x while the
// convolution gathers its operand (same fp32 rounding of the product), so the gated tensor -- the
// widest of a squeeze-and-excite block -- is neither written nor read back.
bool FuseGateIntoConv(Rewriter &rw, const NodePtr &mul) {
  if (mul->kind != Kind::MulCommon || mul->inputs.size() != 2) return false;
  NodePtr cv = rw.Sole(mul->output);
  if (!cv || (cv->kind != Kind::ConvWithPadding && cv->kind != Kind::ConvWithoutPadding)) return false;
  if (cv->group != 1 || cv->has_in_scale || cv->inputs.size() != 1 || cv->inputs[0] != mul->output) return false;
  const auto &os = mul->output->meta.GetShape();
  if (os.size() != 4 || mul->output->meta.GetType() != Type::kFloat32 || os[1] > 4096) return false;
  auto is_gate = [&](const RegionPtr &r) {
    const auto &gs = r->meta.GetShape();
    return r->meta.GetType() == Type::kFloat32 && gs.size() == 4 && (gs[0] == os[0] || gs[0] == 1) &&
           (gs[1] == os[1] || gs[1] == 1) && gs[2] == 1 && gs[3] == 1;
  };
  RegionPtr x, gate;
  if (mul->inputs[0]->meta.GetShape() == os && is_gate(mul->inputs[1])) { x = mul->inputs[0]; gate = mul->inputs[1]; }
  else if (mul->inputs[1]->meta.GetShape() == os && is_gate(mul->inputs[0])) { x = mul->inputs[1]; gate = mul->inputs[0]; }
  else return false;
  if (os[2] * os[3] == 1) return false;  // a gate times a gate: nothing to save
  cv->inputs = {x, gate};
  cv->has_in_scale = true;
  rw.Kill(mul);
  return true;
}

// ---- MulCommon -> FusedMulAdd -> FusedMulAdd ...: a sum of products (ConvBERT's span convolution
// adds nine windows times nine softmax columns) becomes one pass.  Matched at the last node of the
// chain and walked back to the plain product it starts from; every intermediate sum must have the
// next link as its only reader.  Same rounding order as the chain.
bool FuseMulAddChain(Rewriter &rw, const NodePtr &last) {
  if (last->kind != Kind::FusedMulAdd || last->inputs.size() != 3) return false;
  {  // `last` must end the chain: its result is not the addend of another link
    NodePtr next = rw.Sole(last->output);
    if (next && next->kind == Kind::FusedMulAdd && next->inputs.size() == 3 && next->inputs[2] == last->output) return false;
  }
  std::vector<NodePtr> links = {last};  // from the end backwards
  NodePtr head;                         // the MulCommon the chain starts from
  for (;;) {
    const RegionPtr &addend = links.back()->inputs[2];
    auto it = rw.producer.find(addend.get());
    if (it == rw.producer.end() || rw.Sole(addend) != links.back()) return false;
    const NodePtr &prod = it->second;
    if (prod->kind == Kind::FusedMulAdd && prod->inputs.size() == 3) { links.push_back(prod); continue; }
    if (prod->kind == Kind::MulCommon && prod->inputs.size() == 2) { head = prod; break; }
    return false;
  }
  const size_t pairs = links.size() + 1;
  if (pairs < 3 || pairs > 12) return false;  // fml_sum_of_products takes up to 12
  std::vector<RegionPtr> ops = {head->inputs[0], head->inputs[1]};
  for (size_t i = links.size(); i-- > 0;) { ops.push_back(links[i]->inputs[0]); ops.push_back(links[i]->inputs[1]); }
  for (const RegionPtr &r : ops)
    if (r->meta.GetType() != Type::kFloat32) return false;
  if (last->output->meta.GetType() != Type::kFloat32) return false;
  last->kind = Kind::FusedMulAddChain;
  last->inputs = ops;
  rw.Kill(head);
  for (size_t i = 1; i < links.size(); ++i) rw.Kill(links[i]);
  return true;
}

// ---- Rotary position embedding as exported (GPT-NeoX):
//   xr = x[..., :rot]; xp = x[..., rot:]
//   out = Concat(xr * cos + Concat(-xr[..., rot/2:], xr[..., :rot/2]) * sin, xp)
// Matched at the final Concat (after FuseMulAdd has made `xr * cos + (...)` one node); ten nodes per
// projection (five of them launches) become one.
bool FuseRotary(Rewriter &rw, const NodePtr &cat) {
  if (cat->kind != Kind::Concat2 || cat->inputs.size() != 2) return false;
  const RegionPtr &y = cat->output;
  const size_t rank = y->meta.GetRank();
  if (rank < 1 || y->meta.GetType() != Type::kFloat32) return false;
  const int64_t last = (int64_t)rank - 1;
  if (cat->axis != last && cat->axis != -1) return false;
  auto producer_of = [&](const RegionPtr &r) -> NodePtr {
    auto it = rw.producer.find(r.get());
    return it == rw.producer.end() ? nullptr : it->second;
  };
  // a Slice along the last axis only: returns its start there, -1 otherwise
  auto last_axis_slice = [&](const NodePtr &n) -> int64_t {
    if (!n || n->kind != Kind::Slice || n->inputs.size() != 1 || n->starts.size() != rank) return -1;
    const auto &is = n->inputs[0]->meta.GetShape(), &os = n->output->meta.GetShape();
    if (is.size() != rank || os.size() != rank) return -1;
    for (size_t i = 0; i + 1 < rank; ++i)
      if (n->starts[i] != 0 || is[i] != os[i]) return -1;
    return n->starts[rank - 1];
  };
  NodePtr fma = producer_of(cat->inputs[0]), pass = producer_of(cat->inputs[1]);
  if (!fma || fma->kind != Kind::FusedMulAdd || fma->inputs.size() != 3 || rw.Sole(fma->output) != cat) return false;
  NodePtr xr = producer_of(fma->inputs[0]);
  RegionPtr cosv = fma->inputs[1];
  if (last_axis_slice(xr) != 0) {  // the product may be written cos * xr
    xr = producer_of(fma->inputs[1]);
    cosv = fma->inputs[0];
    if (last_axis_slice(xr) != 0) return false;
  }
  const RegionPtr &src = xr->inputs[0];
  const int64_t rot = xr->output->meta.GetShape()[rank - 1], D = src->meta.GetShape()[rank - 1];
  if (rot < 2 || (rot & 1) || last_axis_slice(pass) != rot || pass->inputs[0] != src ||
      pass->output->meta.GetShape()[rank - 1] != D - rot || rw.Sole(pass->output) != cat)
    return false;
  NodePtr mul = producer_of(fma->inputs[2]);
  if (!mul || mul->kind != Kind::MulCommon || mul->inputs.size() != 2 || rw.Sole(mul->output) != fma) return false;
  NodePtr half_cat = producer_of(mul->inputs[0]);
  RegionPtr sinv = mul->inputs[1];
  if (!half_cat || half_cat->kind != Kind::Concat2) { half_cat = producer_of(mul->inputs[1]); sinv = mul->inputs[0]; }
  if (!half_cat || half_cat->kind != Kind::Concat2 || half_cat->inputs.size() != 2 || rw.Sole(half_cat->output) != mul ||
      (half_cat->axis != last && half_cat->axis != -1))
    return false;
  NodePtr neg = producer_of(half_cat->inputs[0]), lo = producer_of(half_cat->inputs[1]);
  if (!neg || neg->kind != Kind::Neg || rw.Sole(neg->output) != half_cat) return false;
  NodePtr hi = producer_of(neg->inputs[0]);
  if (last_axis_slice(hi) != rot / 2 || last_axis_slice(lo) != 0 || hi->inputs[0] != xr->output || lo->inputs[0] != xr->output ||
      hi->output->meta.GetShape()[rank - 1] != rot / 2 || lo->output->meta.GetShape()[rank - 1] != rot / 2 ||
      rw.Sole(hi->output) != neg || rw.Sole(lo->output) != half_cat)
    return false;
  // xr is read by the two half slices and the product, by nobody else
  {
    auto it = rw.consumers.find(xr->output.get());
    if (it == rw.consumers.end() || it->second.size() != 3 || xr->output->kind != flow::Region::kInner) return false;
  }
  for (const RegionPtr &t : {cosv, sinv}) {
    const auto &ts = t->meta.GetShape();
    if (t->meta.GetType() != Type::kFloat32 || ts.empty() || ts.size() > rank || ts.back() != rot) return false;
  }
  if (src->meta.GetType() != Type::kFloat32) return false;
  cat->kind = Kind::Rotary;
  cat->inputs = {src, cosv, sinv};
  cat->value = (double)rot;
  for (const NodePtr &n : {fma, pass, xr, mul, half_cat, neg, hi, lo}) rw.Kill(n);
  return true;
}

// ---- Conv -> SiLU: the activation rides in the convolution's epilogue
bool FuseSiluIntoConv(Rewriter &rw, const NodePtr &cv) {
  if ((cv->kind != Kind::ConvWithPadding && cv->kind != Kind::ConvWithoutPadding) || cv->act != 0) return false;
  NodePtr silu = rw.SoleOfKind(cv->output, Kind::Silu);
  if (!silu) return false;
  cv->act = FML_ACT_SILU;
  cv->output = silu->output;
  rw.Kill(silu);
  return true;
}

// ---- GEMMs that read the same activations with constant weights (the Q, K, V projections):
// one GEMM over the concatenated weights, the original outputs become column slices of its
// result (views, no copy).  Fewer launches and one pass over the shared A operand.
bool MergeSiblingGemms(flow::Flow &f) {
  auto eligible = [](const NodePtr &n) {
    if (n->kind != Kind::FusedGemm || !n->b_is_const || n->trans_a || n->trans_b || n->act != 0 ||
        n->has_residual || n->has_mask || n->divisor != 1.0f || n->alpha != 1.0f || n->beta != 1.0f)
      return false;
    if (n->inputs.size() != 1 || n->output->kind != flow::Region::kInner) return false;
    const RegionPtr &w = n->consts[0];
    if (w->meta.GetRank() != 2 || w->meta.GetType() != Type::kFloat32 || !utils::IsDefaultLayout(w->layout)) return false;
    // the merge copies K * N weights and N bias values per sibling: both constants must hold exactly that
    const int64_t K = w->meta.GetShape()[0], N = w->meta.GetShape()[1];
    if (!w->constant || w->constant->Bytes().size() != (size_t)K * (size_t)N * 4) return false;
    if (n->has_bias) {
      if (n->consts.size() < 2 || n->consts[1]->meta.GetRank() != 1 || n->consts[1]->meta.GetShape()[0] != N) return false;
      if (n->consts[1]->meta.GetType() != Type::kFloat32 || !n->consts[1]->constant ||
          n->consts[1]->constant->Bytes().size() != (size_t)N * 4)
        return false;
    }
    return true;
  };
  for (size_t i = 0; i < f.nodes.size(); ++i) {
    const NodePtr &first = f.nodes[i];
    if (!eligible(first)) continue;
    std::vector<NodePtr> group = {first};
    for (size_t j = i + 1; j < f.nodes.size(); ++j) {
      const NodePtr &n = f.nodes[j];
      if (!eligible(n) || n->inputs[0] != first->inputs[0] || n->has_bias != first->has_bias) continue;
      if (n->consts[0]->meta.GetShape()[0] != first->consts[0]->meta.GetShape()[0]) continue;
      const auto &sa = n->output->meta.GetShape(), &sb = first->output->meta.GetShape();
      if (sa.size() != sb.size() || !std::equal(sa.begin(), sa.end() - 1, sb.begin())) continue;
      group.push_back(n);
    }
    if (group.size() < 2) continue;
    const int64_t K = first->consts[0]->meta.GetShape()[0];
    int64_t total = 0;
    for (const auto &n : group) total += n->consts[0]->meta.GetShape()[1];
    // concatenated weights [K, total] and bias [total]
    std::vector<uint8_t> wbytes((size_t)K * total * 4), bbytes((size_t)total * 4);
    int64_t col = 0;
    for (const auto &n : group) {
      const int64_t N = n->consts[0]->meta.GetShape()[1];
      const uint8_t *src = n->consts[0]->constant->Bytes().data();
      for (int64_t k = 0; k < K; ++k) memcpy(wbytes.data() + ((size_t)k * total + col) * 4, src + (size_t)k * N * 4, (size_t)N * 4);
      if (n->has_bias) memcpy(bbytes.data() + (size_t)col * 4, n->consts[1]->constant->Bytes().data(), (size_t)N * 4);
      col += N;
    }
    auto make_const = [&](const std::string &name, std::vector<int64_t> shape, std::vector<uint8_t> bytes) {
      auto r = std::make_shared<flow::Region>();
      r->kind = flow::Region::kConstant;
      r->name = name;
      r->meta = Meta(Type::kFloat32, shape);
      r->layout = utils::GenDefaultLayout(shape.size());
      r->constant = std::make_shared<Tensor>(r->meta, std::move(bytes));
      f.regions.push_back(r);
      f.by_name[name] = r;
      return r;
    };
    const std::string base = first->name + "_merged";
    RegionPtr wcat = make_const(base + ".w", {K, total}, std::move(wbytes));
    RegionPtr bcat = first->has_bias ? make_const(base + ".b", {total}, std::move(bbytes)) : nullptr;
    auto merged = std::make_shared<flow::Region>();
    merged->kind = flow::Region::kInner;
    merged->name = base;
    std::vector<int64_t> mshape = first->output->meta.GetShape();
    mshape.back() = total;
    merged->meta = Meta(Type::kFloat32, mshape);
    merged->layout = utils::GenDefaultLayout(mshape.size());
    f.regions.push_back(merged);
    f.by_name[base] = merged;
    // slices that hand the original outputs back
    std::vector<NodePtr> slices;
    col = 0;
    for (const auto &n : group) {
      auto sl = std::make_shared<flow::Node>();
      sl->kind = Kind::Slice;
      sl->name = n->name + "_slice";
      sl->inputs = {merged};
      sl->output = n->output;
      sl->starts.assign(mshape.size(), 0);
      sl->starts.back() = col;
      col += n->consts[0]->meta.GetShape()[1];
      slices.push_back(sl);
    }
    first->consts.clear();
    first->consts.push_back(wcat);
    if (bcat) first->consts.push_back(bcat);
    first->output = merged;
    std::unordered_set<const flow::Node *> gone;
    for (size_t g = 1; g < group.size(); ++g) gone.insert(group[g].get());
    std::vector<NodePtr> next;
    for (const auto &n : f.nodes) {
      if (gone.count(n.get())) continue;
      next.push_back(n);
      if (n == first) next.insert(next.end(), slices.begin(), slices.end());
    }
    f.nodes = std::move(next);
    return true;
  }
  return false;
}

}  // namespace

size_t FusionPasses::Run(flow::Flow &flow) {
  const size_t before = flow.nodes.size();
  Rewriter rw(flow);
  using Pass = bool (*)(Rewriter &, const NodePtr &);
  // order matters: bias before GELU / activation before residual, residual before Add+LN
  const Pass passes[] = {FuseEmbedding, FuseMask, FuseBias, FuseGeluIntoGemm, FuseBiasGelu, FuseActivation,
                         FuseResidual, FuseAddLayerNorm, FuseScaledMaskedSoftmax, FuseAttention, FuseSilu, FuseSiluIntoConv, FuseSqueezeExcite, FuseGateIntoConv, FuseMulAdd, FuseRotary, FuseMulAddChain};
  for (Pass pass : passes) {
    bool again = true;
    while (again) {
      again = false;
      for (size_t i = 0; i < flow.nodes.size(); ++i) {
        const NodePtr n = flow.nodes[i];
        if (rw.dead.count(n.get())) continue;
        if (pass(rw, n)) { rw.Commit(); again = true; break; }
      }
    }
  }
  while (MergeSiblingGemms(flow)) {}
  // drop tensors nothing refers to any more
  std::unordered_set<const flow::Region *> live;
  for (const auto &n : flow.nodes) {
    live.insert(n->output.get());
    for (const auto &r : n->inputs) live.insert(r.get());
    for (const auto &r : n->consts) live.insert(r.get());
  }
  std::vector<RegionPtr> kept;
  for (const auto &r : flow.regions) {
    if (live.count(r.get()) || r->kind == flow::Region::kInput || r->kind == flow::Region::kOutput) kept.push_back(r);
    else flow.by_name.erase(r->name);
  }
  flow.regions = std::move(kept);
  return before - flow.nodes.size();
}

}  // namespace worker
}  // namespace fluidml
