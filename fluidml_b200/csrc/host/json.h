// Minimal JSON value (build + dump) for the compile-time dumps; the reference uses
// nlohmann::json for the same purpose (src/worker/executor.cpp:102-104).
#pragma once
#include <cmath>
#include <cstdio>
#include <string>
#include <utility>
#include <vector>

namespace fluidml {
namespace json {

class Value {
public:
  enum Kind { kNull, kNumber, kString, kBool, kArray, kObject };
  Value() : kind_(kNull) {}
  explicit Value(double n) : kind_(kNumber), num_(n) {}
  explicit Value(const std::string &s) : kind_(kString), str_(s) {}
  explicit Value(const char *s) : kind_(kString), str_(s) {}
  explicit Value(bool b) : kind_(kBool), num_(b ? 1 : 0) {}
  static Value Array() { Value v; v.kind_ = kArray; return v; }
  static Value Object() { Value v; v.kind_ = kObject; return v; }
  void Push(Value v) { items_.emplace_back(std::string(), std::move(v)); }
  void Set(const std::string &k, Value v) {
    for (auto &kv : items_) if (kv.first == k) { kv.second = std::move(v); return; }
    items_.emplace_back(k, std::move(v));
  }
  std::string Dump() const { std::string s; DumpTo(s); return s; }

private:
  static void Quote(const std::string &in, std::string &out) {
    out += '"';
    for (char c : in) {
      if (c == '"' || c == '\\') { out += '\\'; out += c; }
      else if (c == '\n') out += "\\n";
      else if ((unsigned char)c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
      else out += c;
    }
    out += '"';
  }
  void DumpTo(std::string &s) const {
    switch (kind_) {
    case kNull: s += "null"; break;
    case kBool: s += num_ ? "true" : "false"; break;
    case kString: Quote(str_, s); break;
    case kNumber: {
      char b[40];
      if (std::floor(num_) == num_ && std::fabs(num_) < 9e15) snprintf(b, sizeof b, "%.0f", num_);
      else snprintf(b, sizeof b, "%.9g", num_);
      s += b;
      break;
    }
    case kArray:
      s += '[';
      for (size_t i = 0; i < items_.size(); ++i) { if (i) s += ','; items_[i].second.DumpTo(s); }
      s += ']';
      break;
    case kObject:
      s += '{';
      for (size_t i = 0; i < items_.size(); ++i) {
        if (i) s += ',';
        Quote(items_[i].first, s);
        s += ':';
        items_[i].second.DumpTo(s);
      }
      s += '}';
      break;
    }
  }
  Kind kind_;
  double num_ = 0;
  std::string str_;
  std::vector<std::pair<std::string, Value>> items_;
};

}  // namespace json
}  // namespace fluidml
