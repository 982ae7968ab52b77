// ONNX-level graph produced by the parser: untyped nodes with an attribute map, named values
// with static metas, constants as tensors.  Plays the role of structure/graph/ in the
// reference (include/structure/graph/{graph,node,edge,attribute}.h) with only what the
// parser and converter touch.
#pragma once
#include "base.h"
#include <map>
#include <unordered_map>

namespace fluidml {
namespace graph {

struct Attribute {
  enum Kind { kNone, kInt, kFloat, kInts, kFloats, kTensor, kString } kind = kNone;
  int64_t i = 0;
  float f = 0.0f;
  std::vector<int64_t> ints;
  std::vector<float> floats;
  std::shared_ptr<Tensor> tensor;
  std::string s;
};

struct Node {
  std::string name, op_type;
  std::vector<std::string> inputs, outputs;
  std::map<std::string, Attribute> attrs;
  bool HasAttr(const std::string &k) const { return attrs.count(k) != 0; }
  int64_t Int(const std::string &k, int64_t dflt) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? dflt : it->second.i;
  }
  float Float(const std::string &k, float dflt) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? dflt : it->second.f;
  }
  std::vector<int64_t> Ints(const std::string &k) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? std::vector<int64_t>{} : it->second.ints;
  }
};

struct Value {
  enum Kind { kInner, kInput, kOutput, kConstant } kind = kInner;
  std::string name;
  Meta meta;
  std::shared_ptr<Tensor> constant;  // kConstant only
  bool IsScalarConstant() const { return kind == kConstant && meta.GetRank() == 0; }
  bool IsTensorConstant() const { return kind == kConstant && meta.GetRank() >= 1; }
};

struct Graph {
  std::string name;
  std::vector<Node> nodes;
  std::unordered_map<std::string, Value> values;
  std::vector<std::string> inputs, outputs;  // declaration order
  const Value &Get(const std::string &n) const {
    auto it = values.find(n);
    if (it == values.end()) throw Error("value '" + n + "' has no shape information (every intermediate "
                                        "tensor needs a value_info entry)");
    return it->second;
  }
};

}  // namespace graph
}  // namespace fluidml
