// C entry points over the host helpers (layout/stride utilities, shape rules, memory plans).
#include "base.h"
#include "dp.h"
#include "fluidml_executor.h"
#include "memory.h"

using namespace fluidml;

extern "C" {

int fml_host_gen_strides(const long long *shape, const long long *layout, int rank, long long *strides) {
  if (rank < 0 || (rank && (!shape || !strides))) return 1;
  std::vector<int64_t> sh(shape, shape + rank);
  std::vector<size_t> l = utils::GenDefaultLayout((size_t)rank);
  if (layout)
    for (int i = 0; i < rank; ++i) {
      if (layout[i] < 0 || layout[i] >= rank) return 1;
      l[i] = (size_t)layout[i];
    }
  const std::vector<int64_t> s = utils::GenStrides(sh, l);
  for (int i = 0; i < rank; ++i) strides[i] = s[i];
  return 0;
}

long long fml_host_gen_all_orders(int len, long long *out) {
  if (len < 0 || len > 10) return -1;
  const auto orders = utils::GenAllOrders((size_t)len);
  if (out)
    for (size_t r = 0; r < orders.size(); ++r)
      for (int i = 0; i < len; ++i) out[r * len + i] = (long long)orders[r][i];
  return (long long)orders.size();
}

int fml_host_broadcast_shape(const long long *a, int ra, const long long *b, int rb, int matmul, long long *out) {
  Meta ma(Type::kFloat32, std::vector<int64_t>(a, a + ra)), mb(Type::kFloat32, std::vector<int64_t>(b, b + rb));
  std::optional<Meta> r = matmul ? BroadcastMatMulShape(ma, mb, Type::kFloat32) : BroadcastShape(ma, mb, Type::kFloat32);
  if (!r) return -1;
  for (size_t i = 0; i < r->GetRank(); ++i) out[i] = r->GetShape()[i];
  return (int)r->GetRank();
}

int fml_host_memory_plan(int greedy, int n, const char *const *names, const size_t *start, const size_t *end,
                         const size_t *size, size_t alignment, size_t *offset_out, size_t *maximum_out) {
  if (n < 0 || (n && (!names || !start || !end || !size || !offset_out)) || !maximum_out) return 1;
  std::unique_ptr<memory::Infos> infos;
  std::unique_ptr<memory::Plan> plan;
  if (greedy) { infos = std::make_unique<memory::GreedyInfos>(); plan = std::make_unique<memory::GreedyPlan>(alignment); }
  else { infos = std::make_unique<memory::PlainInfos>(); plan = std::make_unique<memory::LinearPlan>(alignment); }
  for (int i = 0; i < n; ++i) infos->Push({names[i], start[i], end[i], size[i]});
  const memory::Index index = plan->Run(*infos);
  for (int i = 0; i < n; ++i) offset_out[i] = index.Get(names[i]);
  *maximum_out = index.GetMaximum();
  return 0;
}

namespace {
bool ReadLayout(const long long *layout, size_t rank, std::vector<size_t> *out) {
  *out = utils::GenDefaultLayout(rank);
  if (!layout) return true;
  std::vector<bool> seen(rank, false);
  for (size_t i = 0; i < rank; ++i) {
    if (layout[i] < 0 || layout[i] >= (long long)rank || seen[(size_t)layout[i]]) return false;
    seen[(size_t)layout[i]] = true;
    (*out)[i] = (size_t)layout[i];
  }
  return true;
}
flow::RegionPtr MakeRegion(const char *name, flow::Region::Kind kind, std::vector<int64_t> shape) {
  auto r = std::make_shared<flow::Region>();
  r->kind = kind;
  r->name = name;
  r->meta = Meta(Type::kFloat32, std::move(shape));
  r->layout = utils::GenDefaultLayout(r->meta.GetRank());
  return r;
}
}  // namespace

int fml_host_model_gemm_cost(long long m, long long k, long long n, const long long *a_layout,
                             const long long *c_layout, int precision, double *ns) {
  if (m <= 0 || k <= 0 || n <= 0 || !ns) return 1;
  std::vector<size_t> la, lc;
  if (!ReadLayout(a_layout, 2, &la) || !ReadLayout(c_layout, 2, &lc)) return 1;
  flow::Node node;
  node.kind = flow::Kind::MatMul;
  node.name = "probe";
  node.inputs = {MakeRegion("a", flow::Region::kInner, {m, k}), MakeRegion("b", flow::Region::kConstant, {k, n})};
  node.output = MakeRegion("c", flow::Region::kInner, {m, n});
  evaluation::CostModel model(false, precision);
  *ns = (double)model.GetTimeCost(node, {la, node.inputs[1]->layout}, lc);
  return 0;
}

int fml_host_model_layernorm_cost(long long rows, long long cols, const long long *in_layout,
                                  const long long *out_layout, double *ns) {
  if (rows <= 0 || cols <= 0 || !ns) return 1;
  std::vector<size_t> li, lo;
  if (!ReadLayout(in_layout, 2, &li) || !ReadLayout(out_layout, 2, &lo)) return 1;
  flow::Node node;
  node.kind = flow::Kind::LayerNormalizationConstantScaleBias;
  node.name = "probe";
  node.axis = 1;
  node.inputs = {MakeRegion("x", flow::Region::kInner, {rows, cols})};
  node.consts = {MakeRegion("scale", flow::Region::kConstant, {cols}), MakeRegion("bias", flow::Region::kConstant, {cols})};
  node.output = MakeRegion("y", flow::Region::kInner, {rows, cols});
  evaluation::CostModel model(false, 0);
  *ns = (double)model.GetTimeCost(node, {li}, lo);
  return 0;
}

}  // extern "C"
