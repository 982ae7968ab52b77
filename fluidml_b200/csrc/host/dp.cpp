// Layout search.
//
// What is kept from the reference (src/evaluation/dp.cpp):
//   - the flow is split into chains: the longest unit-weight path first, then the longest
//     path through what remains, and so on (SubFlowsBuilder, dp.cpp:137-568, :570-669);
//   - on each chain a memoised min-cost recursion over (tensor, layout) picks the cheapest
//     combination, trying every permutation of every tensor's dims
//     (DPOnNoOverlapFlowWoker::runOn, dp.cpp:753-842; utils::GenAllOrders);
//   - interface tensors and constants cost nothing in any layout (dp.cpp:761-765);
//   - per-kernel costs are memoised per (kernel, shapes, layouts) and dumped as
//     {KernelName: [{shapes, layouts, time_cost}]} (eval.cpp:136-152, :352-372).
// What differs, on purpose:
//   - the cost of a kernel is a GPU model (bytes over HBM bandwidth scaled by how coalesced
//     each operand is in that layout; tensor-core or CUDA-core time for contractions; a fixed
//     launch cost that vanishes when the node degenerates into an alias) instead of a CPU
//     measurement that takes hours (README.md:15);
//   - a tensor's layout is decided by the chain that PRODUCES it, with the cost of its
//     consumers outside the chain added in; the reference lets the first chain that touches
//     a tensor decide (first-wins insert, dp.cpp:705-729, :861-875), so a consumer could fix
//     a layout its producer then pays for;
//   - plan extraction takes the arg-min terminal layout, not the first enumerated one, and
//     permutations are tried identity-first so ties keep the default layout;
//   - the chains are re-planned against each other until nothing changes (at most 4 rounds).
#include "dp.h"
#include "fluidml_cuda.h"
#include <algorithm>
#include <functional>
#include <limits>
#include <set>
#include <sstream>
#include <unordered_set>

namespace fluidml {
namespace evaluation {

namespace {

// Constants fitted to this library's kernels on a B200, each timed as a run of identical
// launches inside one CUDA graph (the way they run in a compiled model):
//   GEMM on tensor cores, 3xTF32: 128x768x768 8.1 us, 128x768x2304 11.0, 128x768x3072 11.3,
//     128x3072x768 15.2, 1024x768x3072 28.6, 2048x1024x4096 98.9, 8192x4096x4096 1417;
//   GEMM on CUDA cores (an operand layout the tensor-core kernel does not take):
//     128x768x3072 84 us, 128x3072x768 278, 2048x1024x4096 596, 8192x4096x4096 10167;
//   LayerNormalization over a contiguous axis: 128x768 2.8 us, 1024x768 3.5, 2048x1024 4.3;
//     over a strided axis: 18, 41, 76;  attention 12 heads x 128 x 64: 10 us, 9.3 TFLOP/s at
//     batch 32;  element-wise add of 8.4 M floats 16.5 us (6.1 TB/s), of 98 K floats 1.7 us.
constexpr double kHbmBytesPerNs = 6500.0;        // copy-like kernels at full size
constexpr double kTf32FlopsPerNs = 540000.0;     // TF32 passes of the tensor-core GEMM, large shapes
constexpr double kFp32FlopsPerNs = 28000.0;      // CUDA-core FMA GEMM / convolution, large shapes
constexpr double kLaunchNs = 2500.0;             // one more kernel in the graph
constexpr double kGemmFixedNs = 5000.0;          // tensor-core GEMM: pipeline fill, split-K sum, epilogue
constexpr double kGemmStreamBytesPerNs = 3000.0; // operand streaming of one GEMM launch
constexpr double kFp32NsPerK = 90.0;             // CUDA-core GEMM: serial depth of the k loop
constexpr double kAttentionFixedNs = 3000.0;     // staging K and V, softmax, exit
constexpr double kAttentionFlopsPerNs = 9300.0;  // fp32 FMA attention, achieved
constexpr double kStridedEfficiency = 0.125;     // 4 useful bytes per 32-byte sector
constexpr double kStridedRowEfficiency = 0.035;  // row reductions walking a strided axis
constexpr double kStridedRowNsPerElement = 20.0; // ... and their serial depth along the row
constexpr double kTileEfficiency = 0.7;          // shared-memory tile transpose

using Layout = std::vector<size_t>;

std::vector<int64_t> StridesOf(const flow::Region &r, const Layout &l) {
  return utils::GenStrides(r.meta.GetShape(), l);
}

// stride of the dim that is physically innermost among dims of extent > 1
int InnermostDim(const std::vector<int64_t> &shape, const std::vector<int64_t> &strides) {
  int best = -1;
  for (size_t i = 0; i < shape.size(); ++i)
    if (shape[i] > 1 && (best < 0 || strides[i] < strides[best])) best = (int)i;
  return best;
}

bool IsRowMajor(const std::vector<int64_t> &shape, const std::vector<int64_t> &strides) {
  int64_t s = 1;
  for (size_t i = shape.size(); i-- > 0;) {
    if (shape[i] != 1 && strides[i] != s) return false;
    s *= shape[i];
  }
  return true;
}

std::string Key(const flow::Node &n, const std::vector<Layout> &ins, const Layout &out) {
  std::ostringstream k;
  k << flow::KindName(n.kind) << '|' << n.axis << '|' << n.trans_a << n.trans_b << '|';
  for (int64_t p : n.perm) k << p << ',';
  k << '|';
  auto put = [&](const flow::Region &r, const Layout &l) {
    for (int64_t d : r.meta.GetShape()) k << d << 'x';
    k << ':';
    for (size_t p : l) k << p;
    k << ';';
  };
  for (size_t i = 0; i < n.inputs.size(); ++i) put(*n.inputs[i], ins[i]);
  for (const auto &c : n.consts) put(*c, c->layout);
  put(*n.output, out);
  return k.str();
}

}  // namespace

json::Value DynamicProgrammingPlan::ToJson() const {
  json::Value o = json::Value::Object();
  for (const auto &kv : plan_) {
    json::Value a = json::Value::Array();
    for (size_t p : kv.second) a.Push(json::Value((double)p));
    o.Set(kv.first, a);
  }
  return o;
}

size_t CostModel::GetTimeCost(const flow::Node &n, const std::vector<Layout> &ins, const Layout &out) {
  if (constant_) return 1;  // the reference's -DDP_DEBUG mode (eval.cpp:73-77, :268-272)
  const std::string key = Key(n, ins, out);
  auto it = memo_.find(key);
  if (it != memo_.end()) return it->second;

  using flow::Kind;
  const flow::Region &o = *n.output;
  const std::vector<int64_t> os = StridesOf(o, out);
  std::vector<std::vector<int64_t>> is;
  for (size_t i = 0; i < n.inputs.size(); ++i) is.push_back(StridesOf(*n.inputs[i], ins[i]));
  const double obytes = (double)o.meta.GetSize();
  double cost = kLaunchNs;

  // bytes of an operand read through the output's iteration order: coalesced when the
  // operand's stride along the output's physically innermost dim is 1 (or it is broadcast)
  auto read_cost = [&](const flow::Region &r, const std::vector<int64_t> &rs) {
    const int od = InnermostDim(o.meta.GetShape(), os);
    double eff = 1.0;
    if (od >= 0) {
      const int shift = (int)o.meta.GetRank() - (int)r.meta.GetRank();
      const int rd = od - shift;
      if (rd >= 0 && r.meta.GetShape()[rd] > 1 && rs[rd] != 1) eff = kStridedEfficiency;
    }
    return (double)r.meta.GetSize() / (kHbmBytesPerNs * eff);
  };
  const double write_cost = obytes / kHbmBytesPerNs;  // kernels walk the output in physical order

  switch (n.kind) {
  case Kind::Reshape: case Kind::Unsqueeze: case Kind::Squeeze: case Kind::Flatten: {
    const bool alias = IsRowMajor(n.inputs[0]->meta.GetShape(), is[0]) && IsRowMajor(o.meta.GetShape(), os) &&
                       o.kind == flow::Region::kInner;
    cost = alias ? 0.0 : kLaunchNs + 2.0 * obytes / (kHbmBytesPerNs * 0.5);
    break;
  }
  case Kind::Dropout: case Kind::Identity: {
    cost = (is[0] == os && o.kind == flow::Region::kInner) ? 0.0 : kLaunchNs + 2.0 * obytes / (kHbmBytesPerNs * kTileEfficiency);
    break;
  }
  case Kind::Transpose: {
    std::vector<int64_t> ps(os.size());
    bool alias = o.kind == flow::Region::kInner;
    for (size_t i = 0; i < os.size(); ++i) {
      ps[i] = is[0][n.perm[i]];
      if (o.meta.GetShape()[i] > 1 && ps[i] != os[i]) alias = false;
    }
    if (alias) { cost = 0.0; break; }
    const int od = InnermostDim(o.meta.GetShape(), os);
    const bool both_contig = od >= 0 && ps[od] == 1;
    cost = kLaunchNs + 2.0 * obytes / (kHbmBytesPerNs * (both_contig ? 1.0 : kTileEfficiency));
    break;
  }
  case Kind::MatMul: case Kind::FusedGemm: case Kind::GemmConstantBias: {
    const flow::Region &a = *n.inputs[0];
    const bool b_captured = n.kind == Kind::GemmConstantBias || (n.kind == Kind::FusedGemm && n.b_is_const);
    const flow::Region &b = b_captured ? *n.consts[0] : *n.inputs[1];
    std::vector<int64_t> as = is[0];
    std::vector<int64_t> bs = b_captured ? StridesOf(b, b.layout) : is[1];
    const size_t ra = a.meta.GetRank(), rb = b.meta.GetRank(), ro = o.meta.GetRank();
    int64_t a_sm = as[ra - 2], a_sk = as[ra - 1], b_sk = bs[rb - 2], b_sn = bs[rb - 1];
    if (n.trans_a) std::swap(a_sm, a_sk);
    if (n.trans_b) std::swap(b_sk, b_sn);
    const int64_t M = o.meta.GetShape()[ro - 2], N = o.meta.GetShape()[ro - 1];
    const int64_t K = n.trans_a ? a.meta.GetShape()[ra - 2] : a.meta.GetShape()[ra - 1];
    double batch = 1;
    for (size_t i = 0; i + 2 < ro; ++i) batch *= (double)o.meta.GetShape()[i];
    const double flops = 2.0 * batch * (double)M * (double)N * (double)K;
    const double bytes = (double)a.meta.GetSize() + (double)b.meta.GetSize() + obytes;
    const bool const_b = b.kind == flow::Region::kConstant;  // baked in whatever layout suits
    const bool tc = precision_ != FML_GEMM_FP32 && a_sk == 1 && a_sm % 4 == 0 &&
                    (const_b || ((b_sk == 1 && b_sn % 4 == 0) || (b_sn == 1 && b_sk % 4 == 0))) &&
                    M >= 32 && N >= 16 && K >= 16;
    const double passes = precision_ == FML_GEMM_TF32 ? 1.0 : 3.0;
    const int64_t c_sm = os[ro - 2], c_sn = os[ro - 1];
    const double c_eff = (c_sn == 1 || c_sm == 1) ? 1.0 : kStridedEfficiency;
    if (M <= 32) {  // the skinny kernel: a weight-streaming matrix-vector product, any strides
      cost = kLaunchNs + bytes / kGemmStreamBytesPerNs;
    } else if (tc) {
      const double stream = (bytes - obytes) / kGemmStreamBytesPerNs + obytes / (kGemmStreamBytesPerNs * c_eff);
      cost = kLaunchNs + kGemmFixedNs + std::max(flops * passes / kTf32FlopsPerNs, stream);
    } else {
      const double stream = (bytes - obytes) / kHbmBytesPerNs + obytes / (kHbmBytesPerNs * c_eff);
      cost = kLaunchNs + std::max({flops / kFp32FlopsPerNs, (double)K * kFp32NsPerK, stream});
    }
    break;
  }
  case Kind::FusedAttention: {
    // Q [.., Sq, D], K^T [.., D, Sk], V [.., Sk, Dv].  The kernel takes any strides; it loads
    // rows of Q, V and the output along their last axis and K^T along either of its last two,
    // so those are the axes that must be contiguous for coalesced access.
    const auto &kt = n.inputs[1]->meta.GetShape();
    const double flops = 2.0 * (double)n.inputs[0]->meta.GetElementsNum() * (double)kt.back()   // scores
                         + 2.0 * (double)o.meta.GetElementsNum() * (double)kt.back();            // context
    const size_t r = o.meta.GetRank();
    const bool dflt = os[r - 1] == 1 && is[0][r - 1] == 1 && is[2][r - 1] == 1 && (is[1][r - 1] == 1 || is[1][r - 2] == 1);
    double bytes = obytes;
    for (const auto &r : n.inputs) bytes += (double)r->meta.GetSize();
    cost = kLaunchNs + kAttentionFixedNs + std::max(flops / kAttentionFlopsPerNs, bytes / kHbmBytesPerNs) * (dflt ? 1.0 : 8.0);
    break;
  }
  case Kind::Softmax: case Kind::FusedSoftmax: case Kind::LayerNormalizationConstantScaleBias:
  case Kind::FusedLayerNorm: case Kind::CumSum: {
    // one warp per row: fast only when the reduced axis is contiguous on both sides
    const bool contig = is[0][n.axis] == 1 && os[n.axis] == 1;
    double bytes = obytes + (double)n.inputs[0]->meta.GetSize();
    for (size_t i = 1; i < n.inputs.size(); ++i) bytes += (double)n.inputs[i]->meta.GetSize();
    cost = contig ? kLaunchNs + bytes / kHbmBytesPerNs
                  : kLaunchNs + std::max(bytes / (kHbmBytesPerNs * kStridedRowEfficiency),
                                         (double)o.meta.GetShape()[n.axis] * kStridedRowNsPerElement);
    break;
  }
  case Kind::ConvWithPadding: case Kind::ConvWithoutPadding: case Kind::MaxPoolWithoutPadding:
  case Kind::AveragePoolWithoutPadding: {
    // NCHW kernels: anything but the default layout on either side strides every access
    const bool dflt = IsRowMajor(n.inputs[0]->meta.GetShape(), is[0]) && IsRowMajor(o.meta.GetShape(), os);
    double flops = 0;
    if (!n.consts.empty()) {
      double w = 1;
      for (size_t i = 1; i < n.consts[0]->meta.GetRank(); ++i) w *= (double)n.consts[0]->meta.GetShape()[i];
      flops = 2.0 * (double)o.meta.GetElementsNum() * w;
    }
    const double bytes = obytes + (double)n.inputs[0]->meta.GetSize();
    cost = kLaunchNs + std::max(flops / kFp32FlopsPerNs, bytes / kHbmBytesPerNs) * (dflt ? 1.0 : 8.0);
    break;
  }
  case Kind::SqueezeExciteGate: {
    // one pass over x (planes read along their rows), a few kilobytes of weights, two cluster phases
    const bool dflt = IsRowMajor(n.inputs[0]->meta.GetShape(), is[0]);
    cost = kLaunchNs + 2000.0 + (double)n.inputs[0]->meta.GetSize() / kHbmBytesPerNs * (dflt ? 1.0 : 8.0);
    break;
  }
  default: {  // elementwise, gathers, where, slice, concat, pad, reduce-mean
    cost = kLaunchNs + write_cost;
    for (size_t i = 0; i < n.inputs.size(); ++i) cost += read_cost(*n.inputs[i], is[i]);
    for (const auto &c : n.consts)
      if (c->meta.GetSize() <= o.meta.GetSize()) cost += (double)c->meta.GetSize() / kHbmBytesPerNs;
    break;
  }
  }
  const size_t result = (size_t)(cost + 0.5);
  memo_[key] = result;
  Record rec;
  rec.kernel = std::string(flow::KindName(n.kind)) + "Kernel";
  for (size_t i = 0; i < n.inputs.size(); ++i) { rec.shapes.push_back(n.inputs[i]->meta.GetShape()); rec.layouts.push_back(ins[i]); }
  rec.shapes.push_back(o.meta.GetShape());
  rec.layouts.push_back(out);
  rec.cost = result;
  records_.push_back(std::move(rec));
  return result;
}

json::Value CostModel::ToJson() const {
  json::Value root = json::Value::Object();
  std::map<std::string, json::Value> by_kernel;
  for (const Record &r : records_) {
    json::Value e = json::Value::Object();
    const char *names3[] = {"lhs", "rhs", "output"}, *names2[] = {"input", "output"};
    const size_t n = r.shapes.size();
    for (size_t i = 0; i < n; ++i) {
      std::string nm = n == 2 ? names2[i] : n == 3 ? names3[i] : (i + 1 == n ? "output" : "input" + std::to_string(i));
      json::Value s = json::Value::Array(), l = json::Value::Array();
      for (int64_t d : r.shapes[i]) s.Push(json::Value((double)d));
      for (size_t p : r.layouts[i]) l.Push(json::Value((double)p));
      e.Set(nm + "_shape", s);
      e.Set(nm + "_layout", l);
    }
    e.Set("time_cost", json::Value((double)r.cost));
    auto it = by_kernel.find(r.kernel);
    if (it == by_kernel.end()) it = by_kernel.emplace(r.kernel, json::Value::Array()).first;
    it->second.Push(e);
  }
  for (auto &kv : by_kernel) root.Set(kv.first, kv.second);
  return root;
}

json::Value DynamicProgrammingTable::ToJson() const {
  json::Value o = json::Value::Object();
  o.Set("evaluator", cost_.ToJson());
  return o;
}

DynamicProgrammingPlan DynamicProgrammingTable::Run(const flow::Flow &flow) {
  const size_t n = flow.nodes.size();
  // ---- graph structure
  std::unordered_map<const flow::Region *, size_t> producer;
  for (size_t i = 0; i < n; ++i) producer[flow.nodes[i]->output.get()] = i;
  std::vector<std::vector<size_t>> preds(n), succs(n);
  std::unordered_map<const flow::Region *, std::vector<size_t>> consumers;
  for (size_t i = 0; i < n; ++i)
    for (const auto &r : flow.nodes[i]->inputs) {
      consumers[r.get()].push_back(i);
      auto it = producer.find(r.get());
      if (it != producer.end()) { preds[i].push_back(it->second); succs[it->second].push_back(i); }
    }
  // topological order (nodes are usually already sorted; do not rely on it)
  std::vector<size_t> order;
  {
    std::vector<size_t> indeg(n);
    for (size_t i = 0; i < n; ++i) indeg[i] = preds[i].size();
    std::vector<size_t> ready;
    for (size_t i = n; i-- > 0;) if (!indeg[i]) ready.push_back(i);
    while (!ready.empty()) {
      size_t i = ready.back(); ready.pop_back(); order.push_back(i);
      for (size_t s : succs[i]) if (--indeg[s] == 0) ready.push_back(s);
    }
    if (order.size() != n) throw Error("layout search: the flow has a cycle");
  }
  // ---- chains: longest path through the unassigned nodes, repeatedly
  std::vector<std::vector<size_t>> chains;
  std::vector<bool> taken(n, false);
  size_t left = n;
  while (left) {
    std::vector<int64_t> len(n, 0), from(n, -1);
    int64_t best = -1;
    for (size_t i : order) {
      if (taken[i]) continue;
      len[i] = 1;
      for (size_t p : preds[i])
        if (!taken[p] && len[p] + 1 > len[i]) { len[i] = len[p] + 1; from[i] = (int64_t)p; }
      if (best < 0 || len[i] > len[best]) best = (int64_t)i;
    }
    std::vector<size_t> chain;
    for (int64_t i = best; i >= 0; i = from[i]) chain.push_back((size_t)i);
    std::reverse(chain.begin(), chain.end());
    for (size_t i : chain) taken[i] = true;
    left -= chain.size();
    chains.push_back(std::move(chain));
  }

  // ---- candidate layouts per region: every permutation, identity first, one per distinct
  // stride vector (permutations that only move extent-1 dims are the same layout)
  std::unordered_map<const flow::Region *, std::vector<Layout>> cand;
  auto candidates = [&](const flow::RegionPtr &r) -> const std::vector<Layout> & {
    auto it = cand.find(r.get());
    if (it != cand.end()) return it->second;
    std::vector<Layout> list;
    const size_t rank = r->meta.GetRank();
    if (r->kind != flow::Region::kInner || rank > 5) {
      list.push_back(utils::GenDefaultLayout(rank));  // interface tensors are caller buffers
    } else {
      std::vector<Layout> all = utils::GenAllOrders(rank);
      std::stable_partition(all.begin(), all.end(), [](const Layout &l) { return utils::IsDefaultLayout(l); });
      std::set<std::vector<int64_t>> seen;
      for (const Layout &l : all) {
        std::vector<int64_t> s = utils::GenStrides(r->meta.GetShape(), l);
        for (size_t i = 0; i < rank; ++i) if (r->meta.GetShape()[i] == 1) s[i] = 0;
        if (seen.insert(s).second) list.push_back(l);
      }
    }
    return cand.emplace(r.get(), std::move(list)).first->second;
  };

  // current assignment (regions start at their default layout)
  std::unordered_map<const flow::Region *, Layout> cur;
  for (const auto &r : flow.regions) cur[r.get()] = utils::GenDefaultLayout(r->meta.GetRank());
  auto layout_of = [&](const flow::RegionPtr &r) -> const Layout & { return cur.at(r.get()); };

  // cost of node i with region `var` (if any) forced to `lv` and its output to `lo`
  auto node_cost = [&](size_t i, const flow::Region *var, const Layout *lv, const Layout *lo) {
    const flow::Node &nd = *flow.nodes[i];
    std::vector<Layout> ins;
    for (const auto &r : nd.inputs) ins.push_back(var && r.get() == var ? *lv : layout_of(r));
    const Layout &out = lo ? *lo : (var && nd.output.get() == var ? *lv : layout_of(nd.output));
    return cost_.GetTimeCost(nd, ins, out);
  };

  for (int round = 0; round < 4; ++round) {
    bool changed = false;
    for (const std::vector<size_t> &chain : chains) {
      std::unordered_set<size_t> in_chain(chain.begin(), chain.end());
      const size_t m = chain.size();
      // f[j][a] = best cost of the chain prefix ending with output j in candidate a
      std::vector<std::vector<double>> f(m);
      std::vector<std::vector<int>> back(m);
      for (size_t j = 0; j < m; ++j) {
        const size_t i = chain[j];
        const flow::RegionPtr &out = flow.nodes[i]->output;
        const std::vector<Layout> &oc = candidates(out);
        f[j].assign(oc.size(), std::numeric_limits<double>::max());
        back[j].assign(oc.size(), -1);
        const flow::Region *prev = j ? flow.nodes[chain[j - 1]]->output.get() : nullptr;
        for (size_t a = 0; a < oc.size(); ++a) {
          // consumers of this tensor outside the chain pay for its layout too
          double ext = 0;
          auto cit = consumers.find(out.get());
          if (cit != consumers.end())
            for (size_t c : cit->second) {
              if (j + 1 < m && c == chain[j + 1]) continue;  // priced by the recursion itself
              ext += (double)node_cost(c, out.get(), &oc[a], nullptr);
            }
          if (!prev) {
            f[j][a] = (double)node_cost(i, nullptr, nullptr, &oc[a]) + ext;
            continue;
          }
          const std::vector<Layout> &pc = candidates(flow.nodes[chain[j - 1]]->output);
          for (size_t b = 0; b < pc.size(); ++b) {
            const double c = f[j - 1][b] + (double)node_cost(i, prev, &pc[b], &oc[a]) + ext;
            if (c < f[j][a]) { f[j][a] = c; back[j][a] = (int)b; }
          }
        }
      }
      // arg-min terminal layout, then walk back
      int a = (int)(std::min_element(f[m - 1].begin(), f[m - 1].end()) - f[m - 1].begin());
      for (size_t j = m; j-- > 0;) {
        const flow::RegionPtr &out = flow.nodes[chain[j]]->output;
        const Layout &l = candidates(out)[a];
        if (cur[out.get()] != l) { cur[out.get()] = l; changed = true; }
        a = back[j][a];
      }
    }
    if (!changed) break;
  }

  DynamicProgrammingPlan plan;
  for (const auto &r : flow.regions)
    if (r->kind == flow::Region::kInner) plan.Insert(r->name, cur.at(r.get()));
  return plan;
}

}  // namespace evaluation
}  // namespace fluidml
