#include "base.h"
#include <algorithm>

namespace fluidml {

const char *GetStringFromType(Type t) {
  switch (t) {
  case Type::kFloat32: return "f32";
  case Type::kInt32: return "i32";
  case Type::kInt64: return "i64";
  case Type::kBool: return "i1";
  case Type::kFloat16: return "f16";
  case Type::kFloat64: return "f64";
  default: return "unknown";
  }
}

static std::vector<int64_t> align_left(const std::vector<int64_t> &s, size_t rank) {
  std::vector<int64_t> r(rank - s.size(), 1);
  r.insert(r.end(), s.begin(), s.end());
  return r;
}

std::optional<Meta> BroadcastShape(const Meta &lhs, const Meta &rhs, Type type) {
  const size_t rank = std::max(lhs.GetRank(), rhs.GetRank());
  const std::vector<int64_t> a = align_left(lhs.GetShape(), rank), b = align_left(rhs.GetShape(), rank);
  std::vector<int64_t> out(rank);
  for (size_t i = 0; i < rank; ++i) {
    if (a[i] == b[i]) out[i] = a[i];
    else if (a[i] == 1) out[i] = b[i];
    else if (b[i] == 1) out[i] = a[i];
    else return std::nullopt;
  }
  return Meta(type, std::move(out));
}

std::optional<Meta> BroadcastMatMulShape(const Meta &lhs, const Meta &rhs, Type type) {
  if (lhs.GetRank() < 2 || rhs.GetRank() < 2) return std::nullopt;
  const size_t rank = std::max(lhs.GetRank(), rhs.GetRank());
  const std::vector<int64_t> a = align_left(lhs.GetShape(), rank), b = align_left(rhs.GetShape(), rank);
  if (a[rank - 1] != b[rank - 2]) return std::nullopt;
  std::vector<int64_t> out(rank);
  for (size_t i = 0; i + 2 < rank; ++i) {
    if (a[i] == b[i]) out[i] = a[i];
    else if (a[i] == 1) out[i] = b[i];
    else if (b[i] == 1) out[i] = a[i];
    else return std::nullopt;
  }
  out[rank - 2] = a[rank - 2];
  out[rank - 1] = b[rank - 1];
  return Meta(type, std::move(out));
}

double Tensor::AsDouble(int64_t i) const {
  const uint8_t *p = bytes_.data();
  switch (meta_.GetType()) {
  case Type::kFloat32: { float v; memcpy(&v, p + 4 * i, 4); return v; }
  case Type::kFloat64: { double v; memcpy(&v, p + 8 * i, 8); return v; }
  case Type::kInt32: { int32_t v; memcpy(&v, p + 4 * i, 4); return v; }
  case Type::kInt64: { int64_t v; memcpy(&v, p + 8 * i, 8); return (double)v; }
  case Type::kBool: return p[i] ? 1.0 : 0.0;
  default: throw Error("constant tensor has an unsupported dtype");
  }
}

int64_t Tensor::AsInt(int64_t i) const {
  if (meta_.GetType() == Type::kInt64) { int64_t v; memcpy(&v, bytes_.data() + 8 * i, 8); return v; }
  return (int64_t)AsDouble(i);
}

std::vector<int64_t> Tensor::AsInts() const {
  std::vector<int64_t> r((size_t)meta_.GetElementsNum());
  for (size_t i = 0; i < r.size(); ++i) r[i] = AsInt((int64_t)i);
  return r;
}

namespace utils {

// Every permutation of len-1 with the value len-1 inserted at each position, in that order:
// the enumeration order decides which plan a first-wins merge keeps.
std::vector<std::vector<size_t>> GenAllOrders(size_t len) {
  std::vector<std::vector<size_t>> orders;
  if (len == 0) { orders.push_back({}); return orders; }
  for (const auto &prev : GenAllOrders(len - 1))
    for (size_t pos = 0; pos < len; ++pos) {
      std::vector<size_t> o = prev;
      o.insert(o.begin() + pos, len - 1);
      orders.push_back(std::move(o));
    }
  return orders;
}

std::vector<std::vector<size_t>> GenAllIndicesInOrder(const std::vector<int64_t> &shape) {
  std::vector<std::vector<size_t>> res = {{}};
  for (int64_t d : shape) {
    std::vector<std::vector<size_t>> next;
    for (const auto &p : res)
      for (int64_t i = 0; i < d; ++i) { auto q = p; q.push_back((size_t)i); next.push_back(std::move(q)); }
    res = std::move(next);
  }
  return res;
}

std::vector<int64_t> GenPhysicalShape(const std::vector<int64_t> &shape, const std::vector<size_t> &layout) {
  std::vector<int64_t> phys(shape.size());
  for (size_t i = 0; i < shape.size(); ++i) phys.at(layout.at(i)) = shape[i];
  return phys;
}

std::vector<int64_t> GenStrides(const std::vector<int64_t> &shape) {
  std::vector<int64_t> s(shape.size());
  if (shape.empty()) return s;
  s.back() = 1;
  for (size_t i = shape.size() - 1; i > 0; --i) s[i - 1] = s[i] * shape[i];
  return s;
}

std::vector<int64_t> GenStrides(const std::vector<int64_t> &shape, const std::vector<size_t> &layout) {
  const std::vector<int64_t> ps = GenStrides(GenPhysicalShape(shape, layout));
  std::vector<int64_t> s(shape.size());
  for (size_t i = 0; i < shape.size(); ++i) s[i] = ps[layout[i]];
  return s;
}

std::vector<size_t> GenDefaultLayout(size_t rank) {
  std::vector<size_t> l(rank);
  for (size_t i = 0; i < rank; ++i) l[i] = i;
  return l;
}

bool IsDefaultLayout(const std::vector<size_t> &layout) {
  for (size_t i = 0; i < layout.size(); ++i)
    if (layout[i] != i) return false;
  return true;
}

}  // namespace utils
}  // namespace fluidml
