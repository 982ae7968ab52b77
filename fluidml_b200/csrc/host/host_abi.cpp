// C entry points over the host helpers (layout/stride utilities, shape rules, memory plans).
#include "base.h"
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

}  // extern "C"
