// Host data model shared by every stage: element types, Meta, constant tensors, the
// layout/stride helpers and the broadcast shape rules.
//
// Mirrors (by behaviour, not code) src/utils/type.cpp, src/utils/utils.cpp and
// src/structure/tensor/{meta,tensor}.cpp of the reference.  Constants keep their native
// dtype here; the reference holds every constant as vector<double> (tensor.h:36-37).
#pragma once
#include <cstdint>
#include <cstring>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace fluidml {

enum class Type : int32_t {
  kUnknown = 0,
  kFloat32 = 1,  // codes are the ONNX TensorProto codes (src/utils/type.cpp:8-23)
  kInt32 = 6,
  kInt64 = 7,
  kBool = 9,
  kFloat16 = 10,
  kFloat64 = 11,
};

inline size_t GetSizeFromType(Type t) {
  switch (t) {
  case Type::kFloat32: case Type::kInt32: return 4;
  case Type::kInt64: case Type::kFloat64: return 8;
  case Type::kFloat16: return 2;
  case Type::kBool: return 1;
  default: return 0;
  }
}

const char *GetStringFromType(Type t);

class Error : public std::runtime_error {
public:
  using std::runtime_error::runtime_error;
};

class Meta {
public:
  Meta() = default;
  Meta(Type type, std::vector<int64_t> shape) : type_(type), shape_(std::move(shape)) {}
  Type GetType() const { return type_; }
  const std::vector<int64_t> &GetShape() const { return shape_; }
  size_t GetRank() const { return shape_.size(); }
  int64_t GetElementsNum() const {
    int64_t n = 1;
    for (int64_t d : shape_) n *= d;
    return n;
  }
  size_t GetSize() const { return (size_t)GetElementsNum() * GetSizeFromType(type_); }
  bool operator==(const Meta &o) const { return type_ == o.type_ && shape_ == o.shape_; }
  bool operator!=(const Meta &o) const { return !(*this == o); }

private:
  Type type_ = Type::kUnknown;
  std::vector<int64_t> shape_;
};

// meta.cpp:59-137
std::optional<Meta> BroadcastShape(const Meta &lhs, const Meta &rhs, Type type);
std::optional<Meta> BroadcastMatMulShape(const Meta &lhs, const Meta &rhs, Type type);

// A constant: row-major bytes in its native dtype.
class Tensor {
public:
  Tensor() = default;
  Tensor(Meta meta, std::vector<uint8_t> bytes) : meta_(std::move(meta)), bytes_(std::move(bytes)) {}
  const Meta &GetMeta() const { return meta_; }
  const std::vector<uint8_t> &Bytes() const { return bytes_; }
  std::vector<uint8_t> &Bytes() { return bytes_; }
  // Element `i` (row-major) converted to double / int64, whatever the dtype.
  double AsDouble(int64_t i = 0) const;
  int64_t AsInt(int64_t i = 0) const;
  std::vector<int64_t> AsInts() const;

private:
  Meta meta_;
  std::vector<uint8_t> bytes_;
};

namespace utils {
// utils.cpp:26-41, :64-125.  layout[i] = physical position of logical dim i.
std::vector<std::vector<size_t>> GenAllOrders(size_t len);
std::vector<std::vector<size_t>> GenAllIndicesInOrder(const std::vector<int64_t> &shape);
std::vector<int64_t> GenPhysicalShape(const std::vector<int64_t> &shape, const std::vector<size_t> &layout);
std::vector<int64_t> GenStrides(const std::vector<int64_t> &shape);
std::vector<int64_t> GenStrides(const std::vector<int64_t> &shape, const std::vector<size_t> &layout);
std::vector<size_t> GenDefaultLayout(size_t rank);
bool IsDefaultLayout(const std::vector<size_t> &layout);
}  // namespace utils

}  // namespace fluidml
