// worker::Parser -- ONNX bytes -> graph::Graph (reference: include/worker/parser.h,
// src/worker/parser.cpp:193-332).
#pragma once
#include "graph.h"
#include <iosfwd>

namespace fluidml {
namespace worker {

class Parser {
public:
  static graph::Graph Run(const std::string &path);
  static graph::Graph Run(std::istream &input);
  static graph::Graph Run(const uint8_t *data, size_t size);
};

}  // namespace worker
}  // namespace fluidml
