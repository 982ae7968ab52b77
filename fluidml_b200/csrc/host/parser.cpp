// Parser: ONNX ModelProto bytes -> graph::Graph.
//
// Does what worker::Parser does (src/worker/parser.cpp:193-332): initialisers become
// constants (rank 0 -> scalar constants, :226-237), graph inputs / outputs / value_info
// become values with static metas (:240-248), nodes keep their op_type, inputs, outputs and
// attributes (:249-327).  The reference links the onnx protobuf library; this is a
// hand-written reader of the protobuf wire format for exactly the fields that parser
// touches (field numbers from the public onnx.proto3):
//   ModelProto.graph=7; GraphProto node=1 name=2 initializer=5 input=11 output=12
//   value_info=13; NodeProto input=1 output=2 name=3 op_type=4 attribute=5;
//   AttributeProto name=1 f=2 i=3 s=4 t=5 floats=7 ints=8 type=20;
//   TensorProto dims=1 data_type=2 float_data=4 int32_data=5 int64_data=7 name=8
//   raw_data=9 double_data=10; ValueInfoProto name=1 type=2; TypeProto.tensor_type=1;
//   Tensor elem_type=1 shape=2; TensorShapeProto.dim=1; Dimension.dim_value=1.
#include "parser.h"
#include <fstream>
#include <istream>
#include <iterator>
#include <set>

namespace fluidml {
namespace worker {
namespace {

struct Reader {
  const uint8_t *p, *end;
  bool Done() const { return p >= end; }
  uint64_t Varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 70; shift += 7) {
      if (p >= end) throw Error("ONNX file is truncated (varint)");
      uint8_t b = *p++;
      v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
    }
    throw Error("ONNX file is corrupt (varint too long)");
  }
  Reader Sub() {
    uint64_t n = Varint();
    if ((uint64_t)(end - p) < n) throw Error("ONNX file is truncated (length-delimited field)");
    Reader r{p, p + n};
    p += n;
    return r;
  }
  void Skip(int wire) {
    switch (wire) {
    case 0: Varint(); break;
    case 1: Need(8); p += 8; break;
    case 2: Sub(); break;
    case 5: Need(4); p += 4; break;
    default: throw Error("ONNX file uses an unsupported protobuf wire type");
    }
  }
  void Need(size_t n) { if ((size_t)(end - p) < n) throw Error("ONNX file is truncated"); }
  std::string Str() { Reader r = Sub(); return std::string((const char *)r.p, (size_t)(r.end - r.p)); }
  float F32() { Need(4); float v; memcpy(&v, p, 4); p += 4; return v; }
  double F64() { Need(8); double v; memcpy(&v, p, 8); p += 8; return v; }
};

void ReadPackedInts(Reader &r, int wire, std::vector<int64_t> &out) {
  if (wire == 0) { out.push_back((int64_t)r.Varint()); return; }
  Reader s = r.Sub();
  while (!s.Done()) out.push_back((int64_t)s.Varint());
}

std::pair<std::string, std::shared_ptr<Tensor>> ReadTensor(Reader r) {
  std::vector<int64_t> dims, ints;
  std::vector<float> floats;
  std::vector<double> doubles;
  std::string name, raw;
  bool has_raw = false;
  int64_t code = 1;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 1) ReadPackedInts(r, w, dims);
    else if (f == 2) code = (int64_t)r.Varint();
    else if (f == 8) name = r.Str();
    else if (f == 9) { raw = r.Str(); has_raw = true; }
    else if (f == 4) { if (w == 2) { Reader s = r.Sub(); while (!s.Done()) floats.push_back(s.F32()); } else floats.push_back(r.F32()); }
    else if (f == 10) { if (w == 2) { Reader s = r.Sub(); while (!s.Done()) doubles.push_back(s.F64()); } else doubles.push_back(r.F64()); }
    else if (f == 5 || f == 7) ReadPackedInts(r, w, ints);
    else r.Skip(w);
  }
  Type type = (Type)code;
  const size_t es = GetSizeFromType(type);
  if (es == 0) throw Error("initializer '" + name + "' has unsupported data_type " + std::to_string(code));
  Meta meta(type, dims);
  const size_t n = (size_t)meta.GetElementsNum();
  std::vector<uint8_t> bytes(n * es);
  if (has_raw) {
    if (raw.size() != bytes.size()) throw Error("initializer '" + name + "': raw_data size does not match its dims");
    memcpy(bytes.data(), raw.data(), raw.size());
  } else {
    auto put = [&](size_t i, double v) {
      switch (type) {
      case Type::kFloat32: { float x = (float)v; memcpy(bytes.data() + 4 * i, &x, 4); break; }
      case Type::kFloat64: memcpy(bytes.data() + 8 * i, &v, 8); break;
      case Type::kInt32: { int32_t x = (int32_t)v; memcpy(bytes.data() + 4 * i, &x, 4); break; }
      case Type::kInt64: { int64_t x = (int64_t)v; memcpy(bytes.data() + 8 * i, &x, 8); break; }
      case Type::kBool: bytes[i] = v != 0; break;
      default: throw Error("initializer '" + name + "': typed data for this dtype is not supported");
      }
    };
    size_t have = !floats.empty() ? floats.size() : !doubles.empty() ? doubles.size() : ints.size();
    if (have != n) throw Error("initializer '" + name + "': element count does not match its dims");
    for (size_t i = 0; i < n; ++i) {
      if (!floats.empty()) put(i, floats[i]);
      else if (!doubles.empty()) put(i, doubles[i]);
      else if (type == Type::kInt64) { memcpy(bytes.data() + 8 * i, &ints[i], 8); }
      else put(i, (double)ints[i]);
    }
  }
  return {name, std::make_shared<Tensor>(std::move(meta), std::move(bytes))};
}

void ReadValueInfo(Reader r, std::string &name, Meta &meta) {
  int64_t code = 1;
  std::vector<int64_t> shape;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 1) name = r.Str();
    else if (f == 2) {
      Reader t = r.Sub();
      while (!t.Done()) {
        uint64_t k2 = t.Varint();
        if ((k2 >> 3) != 1) { t.Skip((int)(k2 & 7)); continue; }
        Reader tt = t.Sub();  // TypeProto.Tensor
        while (!tt.Done()) {
          uint64_t k3 = tt.Varint();
          int f3 = (int)(k3 >> 3);
          if (f3 == 1) code = (int64_t)tt.Varint();
          else if (f3 == 2) {
            Reader sh = tt.Sub();
            while (!sh.Done()) {
              uint64_t k4 = sh.Varint();
              if ((k4 >> 3) != 1) { sh.Skip((int)(k4 & 7)); continue; }
              Reader dim = sh.Sub();
              int64_t dv = -1;
              while (!dim.Done()) {
                uint64_t k5 = dim.Varint();
                if ((k5 >> 3) == 1) dv = (int64_t)dim.Varint();
                else dim.Skip((int)(k5 & 7));
              }
              if (dv < 0) throw Error("value '" + name + "' has a symbolic or missing dimension; shapes must be static");
              shape.push_back(dv);
            }
          } else tt.Skip((int)(k3 & 7));
        }
      }
    } else r.Skip(w);
  }
  meta = Meta((Type)code, std::move(shape));
}

std::pair<std::string, graph::Attribute> ReadAttribute(Reader r) {
  graph::Attribute a;
  std::string name;
  int64_t type = 0;
  bool has_i = false, has_f = false, has_s = false;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 1) name = r.Str();
    else if (f == 2) { a.f = r.F32(); has_f = true; }
    else if (f == 3) { a.i = (int64_t)r.Varint(); has_i = true; }
    else if (f == 4) { a.s = r.Str(); has_s = true; }
    else if (f == 5) a.tensor = ReadTensor(r.Sub()).second;
    else if (f == 7) { if (w == 2) { Reader s = r.Sub(); while (!s.Done()) a.floats.push_back(s.F32()); } else a.floats.push_back(r.F32()); }
    else if (f == 8) ReadPackedInts(r, w, a.ints);
    else if (f == 20) type = (int64_t)r.Varint();
    else r.Skip(w);
  }
  using A = graph::Attribute;
  switch (type) {
  case 1: a.kind = A::kFloat; break;
  case 2: a.kind = A::kInt; break;
  case 3: a.kind = A::kString; break;
  case 4: a.kind = A::kTensor; break;
  case 6: a.kind = A::kFloats; break;
  case 7: a.kind = A::kInts; break;
  default:
    a.kind = a.tensor ? A::kTensor : !a.ints.empty() ? A::kInts : !a.floats.empty() ? A::kFloats
             : has_i ? A::kInt : has_f ? A::kFloat : has_s ? A::kString : A::kNone;
  }
  if (a.kind == A::kInt) a.f = (float)a.i;
  if (a.kind == A::kFloat) a.i = (int64_t)a.f;
  return {name, std::move(a)};
}

graph::Node ReadNode(Reader r) {
  graph::Node n;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 1) n.inputs.push_back(r.Str());
    else if (f == 2) n.outputs.push_back(r.Str());
    else if (f == 3) n.name = r.Str();
    else if (f == 4) n.op_type = r.Str();
    else if (f == 5) { auto kv = ReadAttribute(r.Sub()); n.attrs[kv.first] = std::move(kv.second); }
    else r.Skip(w);
  }
  return n;
}

// Operators the reference parser accepts (parser.cpp:249-327) plus Sigmoid, which the
// reference rejects (:320-326) but the EfficientNet configuration needs.
const std::set<std::string> kKnownOps = {
    "Add", "AveragePool", "Cast", "Clip", "Concat", "ConstantOfShape", "Conv", "CumSum", "Div",
    "Dropout", "Equal", "Erf", "Flatten", "Gather", "Gemm", "LayerNormalization", "MatMul",
    "MaxPool", "Mul", "Neg", "Not", "Pad", "Pow", "ReduceMean", "Relu", "Reshape", "Slice",
    "Softmax", "Sqrt", "Squeeze", "Sub", "Tanh", "Transpose", "Unsqueeze", "Where", "Sigmoid",
    "Identity"};

void ReadGraph(Reader r, graph::Graph &g) {
  std::vector<std::pair<std::string, Meta>> ins, outs, infos;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 1) g.nodes.push_back(ReadNode(r.Sub()));
    else if (f == 2) g.name = r.Str();
    else if (f == 5) {
      auto kv = ReadTensor(r.Sub());
      graph::Value v;
      v.kind = graph::Value::kConstant;
      v.name = kv.first;
      v.meta = kv.second->GetMeta();
      v.constant = kv.second;
      g.values[v.name] = std::move(v);
    } else if (f == 11 || f == 12 || f == 13) {
      std::string name;
      Meta meta;
      ReadValueInfo(r.Sub(), name, meta);
      (f == 11 ? ins : f == 12 ? outs : infos).emplace_back(std::move(name), std::move(meta));
    } else r.Skip(w);
  }
  auto put = [&](const std::pair<std::string, Meta> &vi, graph::Value::Kind kind) {
    auto it = g.values.find(vi.first);
    if (it != g.values.end() && it->second.kind == graph::Value::kConstant) return false;  // input shadowed by an initialiser
    graph::Value v;
    v.kind = kind;
    v.name = vi.first;
    v.meta = vi.second;
    g.values[v.name] = std::move(v);
    return true;
  };
  for (auto &vi : infos) put(vi, graph::Value::kInner);
  for (auto &vi : ins) if (put(vi, graph::Value::kInput)) g.inputs.push_back(vi.first);
  for (auto &vi : outs) { put(vi, graph::Value::kOutput); g.outputs.push_back(vi.first); }
  size_t k = 0;
  for (auto &n : g.nodes) {
    if (!kKnownOps.count(n.op_type)) throw Error("unsupported ONNX operator '" + n.op_type + "' (node '" + n.name + "')");
    if (n.name.empty()) n.name = n.op_type + "_" + std::to_string(k);
    ++k;
  }
}

}  // namespace

graph::Graph Parser::Run(const uint8_t *data, size_t size) {
  graph::Graph g;
  Reader r{data, data + size};
  bool seen = false;
  while (!r.Done()) {
    uint64_t key = r.Varint();
    int f = (int)(key >> 3), w = (int)(key & 7);
    if (f == 7 && w == 2) { ReadGraph(r.Sub(), g); seen = true; }
    else r.Skip(w);
  }
  if (!seen) throw Error("not an ONNX model: no graph found");
  return g;
}

graph::Graph Parser::Run(std::istream &input) {
  std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(input)), std::istreambuf_iterator<char>());
  if (bytes.empty()) throw Error("ONNX input stream is empty or unreadable");
  return Run(bytes.data(), bytes.size());
}

graph::Graph Parser::Run(const std::string &path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw Error("cannot open ONNX file '" + path + "'");
  return Run(f);
}

}  // namespace worker
}  // namespace fluidml
