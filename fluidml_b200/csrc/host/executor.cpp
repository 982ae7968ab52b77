// Executor: the public facade (include/worker/executor.h) and its C ABI
// (include/fluidml_executor.h).  Compile = Parser -> Converter -> fusion passes ->
// TopologicalSort -> (DP layout search) -> lowering -> memory plan -> Builder -> Runner,
// the same stage order as src/worker/executor.cpp:91-133.
#include <algorithm>
#include <iterator>
#include <cstdio>
#include <fstream>
#include "worker/executor.h"
#include "converter.h"
#include "dp.h"
#include "fluidml_executor.h"
#include "fusion.h"
#include "json.h"
#include "parser.h"
#include "planner.h"
#include "program.h"
#include <cstdlib>
#include <set>
#include <sstream>

namespace fluidml {
namespace worker {
namespace {

enum class LayoutMode { kPlain, kDP };

std::string EnvOr(const char *key, const std::string &dflt) {
  const char *v = std::getenv(key);
  return v && *v ? std::string(v) : dflt;
}

int ParsePrecision(const std::string &v) {
  if (v == "auto") return FML_GEMM_AUTO;
  if (v == "fp32") return FML_GEMM_FP32;
  if (v == "3xtf32") return FML_GEMM_3XTF32;
  if (v == "tf32") return FML_GEMM_TF32;
  throw Error("gemm_precision must be one of auto, fp32, 3xtf32, tf32 (got '" + v + "')");
}

class ExecutorImpl : public Executor {
public:
  ExecutorImpl(std::string &&name, size_t epoch, LayoutMode layout, MemoryPlanKind plan)
      : name_(std::move(name)), epoch_(epoch ? epoch : 1), layout_(layout), plan_(plan) {
    SetOption("device", EnvOr("FLUIDML_DEVICE", "0"));
    SetOption("gemm_precision", EnvOr("FLUIDML_GEMM_PRECISION", "auto"));
    SetOption("fusion", EnvOr("FLUIDML_FUSION", "1"));
    SetOption("cuda_graph", EnvOr("FLUIDML_CUDA_GRAPH", "1"));
    SetOption("alignment", EnvOr("FLUIDML_ALIGNMENT", "256"));
    SetOption("dp_cost", EnvOr("FLUIDML_DP_COST", "model"));
    SetOption("autotune", EnvOr("FLUIDML_AUTOTUNE", "1"));
    SetOption("weight_prefetch", EnvOr("FLUIDML_WEIGHT_PREFETCH", "1"));
    SetOption("plan_cache", EnvOr("FLUIDML_PLAN_CACHE", ""));
    SetOption("resident", EnvOr("FLUIDML_RESIDENT", "0"));
  }

  void SetOption(const std::string &key, const std::string &value) override {
    if (key == "device") options_.device = std::stoi(value);
    else if (key == "gemm_precision") options_.gemm_precision = ParsePrecision(value);
    else if (key == "fusion") options_.fusion = value != "0";
    else if (key == "cuda_graph") options_.cuda_graph = value != "0";
    else if (key == "autotune") options_.autotune = value != "0";
    else if (key == "weight_prefetch") options_.weight_prefetch = value != "0";
    else if (key == "plan_cache") options_.plan_cache = value;
    else if (key == "resident") options_.resident = value != "0";
    else if (key == "alignment") {
      options_.alignment = (size_t)std::stoul(value);
      if (options_.alignment < 16 || (options_.alignment & (options_.alignment - 1)))
        throw Error("alignment must be a power of two >= 16");
    } else if (key == "dp_cost") {
      if (value != "model" && value != "constant") throw Error("dp_cost must be 'model' or 'constant'");
      options_.dp_constant_cost = value == "constant";
    } else throw Error("unknown option '" + key + "'");
  }

  void Compile(std::istream &input, std::ofstream *mlir, std::ofstream *llvm, std::ofstream *json) override {
    const std::string bytes((std::istreambuf_iterator<char>(input)), std::istreambuf_iterator<char>());
    CompileBuffer(bytes.data(), bytes.size(), mlir, llvm, json);
  }

  void Compile(std::string_view input, std::optional<std::string_view> mlir,
               std::optional<std::string_view> llvm, std::optional<std::string_view> json) override {
    std::ofstream fm, fl, fj;
    auto open = [](std::ofstream &f, const std::optional<std::string_view> &p) -> std::ofstream * {
      if (!p) return nullptr;
      f.open(std::string(*p));
      if (!f) throw Error("cannot write '" + std::string(*p) + "'");
      return &f;
    };
    std::ofstream *pm = open(fm, mlir), *pl = open(fl, llvm), *pj = open(fj, json);
    std::ifstream in{std::string(input), std::ios::binary};
    if (!in) throw Error("cannot open '" + std::string(input) + "'");
    Compile(in, pm, pl, pj);
  }

  void CompileBuffer(const void *data, size_t size, std::ofstream *mlir, std::ofstream *llvm, std::ofstream *json,
                     bool dry_run = false) {
    // FNV-1a over the model bytes: the key of the plan cache
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < size; ++i) h = (h ^ ((const uint8_t *)data)[i]) * 1099511628211ull;
    model_hash_ = h;
    CompileGraph(Parser::Run((const uint8_t *)data, size), mlir, llvm, json, dry_run);
  }

  size_t Invoke(const std::unordered_map<std::string, void *> &args) override {
    if (!runner_) throw Error("Invoke called before Compile");
    return runner_->Run(args, epoch_);
  }

  std::string GetStatsJson() const override { return stats_.Dump(); }

  std::string ProfileJson(const std::unordered_map<std::string, void *> &args, size_t passes) {
    if (!runner_) throw Error("Profile called before Compile");
    json::Value o = json::Value::Object();
    for (const auto &kv : runner_->Profile(args, passes ? passes : 1)) {
      json::Value e = json::Value::Object();
      e.Set("us", json::Value(kv.second.us));
      e.Set("launches", json::Value((double)kv.second.launches));
      o.Set(kv.first, e);
    }
    return o.Dump();
  }

  std::string TraceJson(const std::unordered_map<std::string, void *> &args, size_t passes) {
    if (!runner_) throw Error("Trace called before Compile");
    double pass_us = 0.0;
    json::Value kernels = json::Value::Object();
    std::vector<double> per_launch;
    for (const auto &kv : runner_->Trace(args, passes ? passes : 1, &pass_us, &per_launch)) {
      json::Value e = json::Value::Object();
      e.Set("us", json::Value(kv.second.us));
      e.Set("launches", json::Value((double)kv.second.launches));
      kernels.Set(kv.first, e);
    }
    json::Value list = json::Value::Array();
    const auto &launches = runner_->GetProgram().launches;
    for (size_t i = 0; i < launches.size() && i < per_launch.size(); ++i) {
      json::Value e = json::Value::Object();
      e.Set("node", json::Value(launches[i].node));
      e.Set("kernel", json::Value(launches[i].kernel));
      e.Set("us", json::Value(per_launch[i]));
      list.Push(e);
    }
    json::Value o = json::Value::Object();
    o.Set("pass_us", json::Value(pass_us));
    o.Set("kernels", kernels);
    o.Set("launch_list", list);
    return o.Dump();
  }

private:
  // One file per (model bytes, mode, options that shape the plan): text lines
  //   layout <tensor> <p0> <p1> ...      physical position of every logical dim
  //   tiles <node> <tile_n> <split_k>    tuned GEMM tiles
  struct PlanCacheEntry {
    std::map<std::string, std::vector<size_t>> layouts;
    std::map<std::string, std::pair<int, int>> tiles;
    bool Load(const std::string &path) {
      std::ifstream in(path);
      if (!in) return false;
      std::string line;
      bool complete = false;
      while (std::getline(in, line)) {
        std::istringstream ls(line);
        std::string tag, name;
        ls >> tag;
        if (tag == "end") { complete = true; break; }
        ls >> name;
        if (tag == "layout") {
          std::vector<size_t> l;
          size_t v;
          while (ls >> v) l.push_back(v);
          layouts[name] = l;
        } else if (tag == "tiles") {
          int tn = 0, sk = 0;
          ls >> tn >> sk;
          if (tn > 0 && sk > 0) tiles[name] = {tn, sk};
        }
      }
      return complete;  // a truncated file (interrupted writer) is a miss
    }
    void Store(const std::string &path) const {
      const std::string tmp = path + ".tmp";
      {
        std::ofstream out(tmp);
        if (!out) return;
        for (const auto &kv : layouts) {
          out << "layout " << kv.first;
          for (size_t v : kv.second) out << " " << v;
          out << "\n";
        }
        for (const auto &kv : tiles) out << "tiles " << kv.first << " " << kv.second.first << " " << kv.second.second << "\n";
        out << "end\n";
      }
      std::rename(tmp.c_str(), path.c_str());
    }
  };

  std::string PlanCachePath() const {
    if (options_.plan_cache.empty() || model_hash_ == 0) return std::string();
    char buf[160];
    snprintf(buf, sizeof(buf), "/%016llx-%s-%s-p%d-f%d-c%d-a%d-t%d-r%d.plan", (unsigned long long)model_hash_,
             layout_ == LayoutMode::kDP ? "dp" : "plain", plan_ == MemoryPlanKind::kGreedy ? "greedy" : "linear",
             options_.gemm_precision, options_.fusion ? 1 : 0, options_.dp_constant_cost ? 1 : 0, (int)options_.alignment,
             options_.autotune ? 1 : 0, options_.resident ? 1 : 0);
    return options_.plan_cache + buf;
  }

  // `dry_run`: stop before anything touches the device (planning only).
  void CompileGraph(graph::Graph graph, std::ofstream *mlir, std::ofstream *llvm, std::ofstream *json,
                    bool dry_run = false) {
    runner_.reset();
    flow::Flow flow = Converter::Run(graph);
    graph = graph::Graph();  // constants now live in the flow's regions

    // Arena the reference would plan for this model: unfused flow, default layouts, its own
    // kernels' scratch sizes, no alignment (src/worker/planner.cpp:236-293).
    size_t reference_greedy = 0, reference_linear = 0;
    {
      const flow::Sequence seq = Planner::TopologicalSort(flow);
      const std::vector<memory::Info> infos = Planner::Lifetimes(seq, /*reference_scratch=*/true);
      reference_greedy = Planner::Plan(infos, MemoryPlanKind::kGreedy, 1).GetMaximum();
      reference_linear = Planner::Plan(infos, MemoryPlanKind::kLinear, 1).GetMaximum();
    }
    const size_t nodes_before_fusion = flow.nodes.size();
    if (options_.fusion) FusionPasses::Run(flow);

    flow::Sequence sequence = Planner::TopologicalSort(flow);
    json::Value dp_json = json::Value::Object();
    json::Value plan_json = json::Value::Object();
    // Plan cache: layouts and GEMM tiles of an earlier Compile of the same bytes and options.
    PlanCacheEntry cached;
    const std::string cache_path = PlanCachePath();  // a planning-only run reads the cache too, but never writes it
    bool cache_hit = !cache_path.empty() && cached.Load(cache_path);
    if (cache_hit) {
      // A stale, hand-edited or corrupt file must not reach the stride computation: every layout
      // it names has to be a permutation of 0..rank-1 of a tensor of this model.  Anything else
      // makes the whole file a miss and the model is planned afresh.
      for (const auto &r : sequence.regions) {
        auto it = cached.layouts.find(r->name);
        if (it == cached.layouts.end()) continue;
        const size_t rank = r->meta.GetRank();
        std::vector<bool> seen(rank, false);
        bool ok = it->second.size() == rank;
        for (size_t v : it->second) {
          if (!ok) break;
          if (v >= rank || seen[v]) ok = false;
          else seen[v] = true;
        }
        if (!ok) { cache_hit = false; break; }
      }
      if (!cache_hit) cached = PlanCacheEntry();
    }
    options_.gemm_tiles = std::make_shared<std::map<std::string, std::pair<int, int>>>();
    if (cache_hit) {
      for (const auto &r : sequence.regions) {
        auto it = cached.layouts.find(r->name);
        if (it != cached.layouts.end()) r->layout = it->second;
      }
      *options_.gemm_tiles = cached.tiles;
      dp_json.Set("plan_cache", json::Value(cache_path));
    } else if (layout_ == LayoutMode::kDP) {
      evaluation::DynamicProgrammingTable table(options_.dp_constant_cost, options_.gemm_precision);
      evaluation::DynamicProgrammingPlan plan = table.Run(flow);
      for (const auto &r : sequence.regions)
        if (plan.HasLayout(r->name)) r->layout = plan.GetLayout(r->name);
      dp_json = table.ToJson();
      plan_json = plan.ToJson();
    }

    // Convolution weights the tensor-core kernel can take are baked tap-major with the output
    // channel innermost ([KH][KW][IC][OC]): layout (3, 2, 0, 1) of the OIHW constant.  The
    // CUDA-core kernel reads any strides, so the choice is safe whichever path runs.
    for (const auto &n : sequence.nodes) {
      if (n->kind != flow::Kind::ConvWithPadding && n->kind != flow::Kind::ConvWithoutPadding) continue;
      if (n->group != 1 || n->consts.empty() || n->consts[0]->meta.GetRank() != 4) continue;
      const auto unit = [](const std::vector<int64_t> &v) { return std::all_of(v.begin(), v.end(), [](int64_t x) { return x == 1; }); };
      if (!unit(n->strides) || !unit(n->dilations)) continue;
      // a convolution over a single pixel (squeeze-and-excite) is a weight-streaming product:
      // [OC][IC] as stored is its K-major right-hand side, read with 16-byte loads along k
      const auto &xs = n->inputs[0]->meta.GetShape();
      if (xs.size() == 4 && xs[2] * xs[3] == 1) continue;
      n->consts[0]->layout = {3, 2, 0, 1};
    }

    // A constant right-hand side [K, N] whose N is not a multiple of 4 has rows that do not start
    // on 16-byte steps, which the tensor-core GEMM's loads need; stored K-major ([N][K], layout
    // (1, 0)) it qualifies whenever K is a multiple of 4.  (ConvBERT's 384 x 54 kernel generator:
    // 40 us on the CUDA-core path, 10 us on tensor cores.)
    if (!cache_hit)
      for (const auto &n : sequence.nodes) {
        if (n->kind != flow::Kind::MatMul && n->kind != flow::Kind::FusedGemm && n->kind != flow::Kind::GemmConstantBias) continue;
        const bool captured = n->kind == flow::Kind::GemmConstantBias || (n->kind == flow::Kind::FusedGemm && n->b_is_const);
        flow::RegionPtr b = captured ? (n->consts.empty() ? nullptr : n->consts[0]) : (n->inputs.size() > 1 ? n->inputs[1] : nullptr);
        if (!b || b->kind != flow::Region::kConstant || b->meta.GetRank() != 2 || n->trans_b) continue;
        const int64_t K = b->meta.GetShape()[0], N = b->meta.GetShape()[1];
        if (N % 4 != 0 && K % 4 == 0 && utils::IsDefaultLayout(b->layout)) b->layout = {1, 0};
      }

    kernel::KernelOptions ko;
    ko.gemm_precision = options_.gemm_precision;
    const AliasMap aliases = Lowering::ComputeAliases(sequence, ko);
    Lowering::ComputeScratch(sequence, ko);
    const std::vector<memory::Info> infos = Lowering::Lifetimes(sequence, aliases);
    const memory::Index index = Planner::Plan(infos, plan_, options_.alignment);
    const size_t unaligned = Planner::Plan(infos, plan_, 1).GetMaximum();

    std::unique_ptr<Program> program;
    if (!dry_run) program = Builder::Run(flow, sequence, index, aliases, options_);
    if (program && !cache_path.empty() && !cache_hit) {
      PlanCacheEntry fresh;
      for (const auto &r : sequence.regions) fresh.layouts[r->name] = r->layout;
      fresh.tiles = *options_.gemm_tiles;
      fresh.Store(cache_path);  // best effort: an unwritable directory only costs the next Compile its time
    }

    stats_ = json::Value::Object();
    stats_.Set("name", json::Value(name_));
    stats_.Set("mode", json::Value(std::string(layout_ == LayoutMode::kDP ? "dp" : "plain") +
                                   (plan_ == MemoryPlanKind::kGreedy ? "_greedy" : "_linear")));
    stats_.Set("peak_arena_bytes", json::Value((double)index.GetMaximum()));
    stats_.Set("peak_arena_bytes_unaligned", json::Value((double)unaligned));
    stats_.Set("reference_arena_bytes_greedy", json::Value((double)reference_greedy));
    stats_.Set("reference_arena_bytes_linear", json::Value((double)reference_linear));
    stats_.Set("graph_nodes", json::Value((double)nodes_before_fusion));
    stats_.Set("flow_nodes", json::Value((double)flow.nodes.size()));
    stats_.Set("aliased_nodes", json::Value((double)aliases.size()));
    stats_.Set("plan_cache", json::Value(std::string(cache_path.empty() ? "off" : cache_hit ? "hit" : "miss")));
    stats_.Set("plan_cache_file", json::Value(cache_path));
    json::Value seq = json::Value::Array();
    for (const auto &n : sequence.nodes) {
      json::Value e = json::Value::Object();
      e.Set("name", json::Value(n->name));
      e.Set("kind", json::Value(flow::KindName(n->kind)));
      e.Set("alias", json::Value(aliases.count(n->output.get()) != 0));
      e.Set("output", json::Value(n->output->name));
      json::Value ins = json::Value::Array();
      for (const auto &r : n->inputs) ins.Push(json::Value(r->name));
      e.Set("inputs", ins);
      e.Set("scratch", json::Value((double)n->buffer_size));
      seq.Push(e);
    }
    stats_.Set("sequence", seq);
    if (program) {
      stats_.Set("weight_bytes", json::Value((double)program->weight_bytes));
      stats_.Set("interface_bytes", json::Value((double)program->io_bytes));
      stats_.Set("launches", json::Value((double)program->launches.size()));
      stats_.Set("resident_programs", json::Value((double)program->resident_programs.size()));
      stats_.Set("resident_stages", json::Value((double)program->resident_stages));
      stats_.Set("resident_bytes", json::Value((double)program->resident_scratch_bytes));
      json::Value iface = json::Value::Object();  // host buffer size of every argument of Invoke
      for (const auto &b : program->inputs) iface.Set(b.name, json::Value((double)b.bytes));
      for (const auto &b : program->outputs) iface.Set(b.name, json::Value((double)b.bytes));
      stats_.Set("interface", iface);
      json::Value hist = json::Value::Object();
      for (const auto &kv : program->kernel_histogram) hist.Set(kv.first, json::Value((double)kv.second));
      stats_.Set("kernels", hist);
    }

    if (mlir && program) {  // the launch plan, one line per launch
      for (const auto &l : program->launches) *mlir << l.kernel << "  // node " << l.node << "\n";
    }
    if (llvm) {  // region table: where every tensor lives and how it is laid out
      for (const auto &r : sequence.regions) {
        *llvm << r->name << " " << GetStringFromType(r->meta.GetType()) << " [";
        for (size_t i = 0; i < r->meta.GetRank(); ++i) *llvm << (i ? "," : "") << r->meta.GetShape()[i];
        *llvm << "] layout [";
        for (size_t i = 0; i < r->layout.size(); ++i) *llvm << (i ? "," : "") << r->layout[i];
        *llvm << "] ";
        auto it = aliases.find(r.get());
        if (it != aliases.end()) *llvm << "alias-of " << it->second->name;
        else if (r->kind == flow::Region::kInner && index.Has(r->name)) *llvm << "arena+" << index.Get(r->name);
        else *llvm << (r->kind == flow::Region::kConstant ? "constant" : r->kind == flow::Region::kInput ? "input" : r->kind == flow::Region::kOutput ? "output" : "unused");
        *llvm << "\n";
      }
    }
    if (json) {
      json::Value root = json::Value::Object();
      root.Set("dp_table", dp_json);
      root.Set("plan", plan_json);
      // logical shape of every tensor the sequence touches: what the reference's analyzer
      // (tools/analyzer.py:96-112) reads from the ONNX file's value_info
      json::Value shapes = json::Value::Object();
      for (const auto &r : sequence.regions) {
        json::Value sh = json::Value::Array();
        for (int64_t d : r->meta.GetShape()) sh.Push(json::Value((double)d));
        shapes.Set(r->name, sh);
      }
      root.Set("infos", shapes);
      json::Value arena = json::Value::Object();
      for (const auto &kv : index.All()) {
        json::Value e = json::Value::Array();
        e.Push(json::Value((double)kv.second.first));
        e.Push(json::Value((double)kv.second.second));
        arena.Set(kv.first, e);
      }
      json::Value a = json::Value::Object();
      a.Set("tenants", arena);
      json::Value lives = json::Value::Object();
      for (const memory::Info &i : infos) {
        json::Value e = json::Value::Array();
        e.Push(json::Value((double)i.start));
        e.Push(json::Value((double)i.end));
        e.Push(json::Value((double)i.size));
        lives.Set(i.name, e);
      }
      a.Set("lifetimes", lives);
      a.Set("stats", stats_);
      root.Set("arena", a);
      *json << root.Dump();
    }
    if (program) runner_ = std::make_unique<Runner>(std::move(program), options_);
    if (runner_ && options_.autotune && !options_.dp_constant_cost) ReportCostModel(sequence, aliases);
  }

  // The reference's layout search runs on MEASURED kernel times (src/evaluation/eval.cpp:64-100,
  // :261-302); this back end plans with a model.  After Compile the two are put side by side:
  // per kernel class the modelled cost of its nodes under the chosen layouts and the time the
  // same launches take inside the replayed graph (kernel-start stamps), so that a model that has
  // drifted from the hardware shows in the stats ("cost_model").
  void ReportCostModel(const flow::Sequence &sequence, const AliasMap &aliases) {
    try {
      double pass_us = 0.0;
      const auto measured = runner_->Trace({}, 5, &pass_us);
      evaluation::CostModel model(false, options_.gemm_precision);
      std::unordered_map<std::string, const flow::Node *> by_name;
      for (const auto &n : sequence.nodes)
        if (!aliases.count(n->output.get())) by_name[n->name] = n.get();
      std::map<std::string, double> modelled;
      std::set<std::string> seen;
      for (const auto &l : runner_->GetProgram().launches) {
        if (!seen.insert(l.node).second) continue;  // a node with several launches is modelled once
        auto it = by_name.find(l.node);
        if (it == by_name.end()) continue;
        std::vector<std::vector<size_t>> ins;
        for (const auto &r : it->second->inputs) ins.push_back(r->layout);
        modelled[l.kernel] += (double)model.GetTimeCost(*it->second, ins, it->second->output->layout) * 1e-3;
      }
      json::Value o = json::Value::Object();
      for (const auto &kv : measured) {
        json::Value e = json::Value::Object();
        e.Set("measured_us", json::Value(kv.second.us));
        e.Set("modelled_us", json::Value(modelled.count(kv.first) ? modelled[kv.first] : 0.0));
        e.Set("launches", json::Value((double)kv.second.launches));
        o.Set(kv.first, e);
      }
      stats_.Set("cost_model", o);
      stats_.Set("cost_model_pass_us", json::Value(pass_us));
    } catch (const std::exception &e) {
      stats_.Set("cost_model", json::Value(std::string("not measured: ") + e.what()));
    }
  }


  std::string name_;
  size_t epoch_;
  LayoutMode layout_;
  MemoryPlanKind plan_;
  Options options_;
  std::unique_ptr<Runner> runner_;
  json::Value stats_ = json::Value::Object();
  uint64_t model_hash_ = 0;

};

}  // namespace

std::unique_ptr<Executor> Executor::MakePlainLinear(std::string &&name, size_t epoch) {
  return std::make_unique<ExecutorImpl>(std::move(name), epoch, LayoutMode::kPlain, MemoryPlanKind::kLinear);
}
std::unique_ptr<Executor> Executor::MakePlainGreedy(std::string &&name, size_t epoch) {
  return std::make_unique<ExecutorImpl>(std::move(name), epoch, LayoutMode::kPlain, MemoryPlanKind::kGreedy);
}
std::unique_ptr<Executor> Executor::MakeDPGreedy(std::string &&name, size_t epoch) {
  return std::make_unique<ExecutorImpl>(std::move(name), epoch, LayoutMode::kDP, MemoryPlanKind::kGreedy);
}

}  // namespace worker
}  // namespace fluidml

// ------------------------------------------------------------------------------ C ABI
struct fml_executor {
  std::unique_ptr<fluidml::worker::Executor> impl;
  std::string error, stats;
};

namespace {
template <typename F> int Guard(fml_executor *e, F &&f) {
  try {
    f();
    if (e) e->error.clear();
    return 0;
  } catch (const std::out_of_range &ex) {
    if (e) e->error = std::string("missing argument: ") + ex.what();
    return 2;
  } catch (const std::exception &ex) {
    if (e) e->error = ex.what();
    return 1;
  }
}
std::ofstream *OpenOpt(std::ofstream &f, const char *path) {
  if (!path) return nullptr;
  f.open(path);
  if (!f) throw fluidml::Error(std::string("cannot write '") + path + "'");
  return &f;
}
}  // namespace

extern "C" {

int fml_executor_create(const char *name, int mode, size_t epoch, fml_executor **out) {
  if (!out || !name) return 1;
  *out = nullptr;
  auto *e = new fml_executor();
  int st = Guard(e, [&] {
    using fluidml::worker::Executor;
    switch (mode) {
    case FML_EXECUTOR_PLAIN_LINEAR: e->impl = Executor::MakePlainLinear(std::string(name), epoch); break;
    case FML_EXECUTOR_PLAIN_GREEDY: e->impl = Executor::MakePlainGreedy(std::string(name), epoch); break;
    case FML_EXECUTOR_DP_GREEDY: e->impl = Executor::MakeDPGreedy(std::string(name), epoch); break;
    default: throw fluidml::Error("unknown executor mode");
    }
  });
  *out = e;  // returned even on failure so the message can be read; destroy it either way
  return st;
}

void fml_executor_destroy(fml_executor *e) { delete e; }

const char *fml_executor_last_error(const fml_executor *e) { return e ? e->error.c_str() : "null executor"; }

int fml_executor_set_option(fml_executor *e, const char *key, const char *value) {
  if (!e || !e->impl || !key || !value) return 1;
  return Guard(e, [&] { e->impl->SetOption(key, value); });
}

int fml_executor_compile_file(fml_executor *e, const char *onnx_path, const char *mlir_path,
                              const char *llvm_path, const char *json_path) {
  if (!e || !e->impl || !onnx_path) return 1;
  return Guard(e, [&] {
    e->impl->Compile(std::string_view(onnx_path),
                     mlir_path ? std::optional<std::string_view>(mlir_path) : std::nullopt,
                     llvm_path ? std::optional<std::string_view>(llvm_path) : std::nullopt,
                     json_path ? std::optional<std::string_view>(json_path) : std::nullopt);
  });
}

int fml_executor_compile_buffer(fml_executor *e, const void *onnx_bytes, size_t size,
                                const char *mlir_path, const char *llvm_path, const char *json_path) {
  if (!e || !e->impl || !onnx_bytes) return 1;
  return Guard(e, [&] {
    std::ofstream fm, fl, fj;
    std::ofstream *pm = OpenOpt(fm, mlir_path), *pl = OpenOpt(fl, llvm_path), *pj = OpenOpt(fj, json_path);
    static_cast<fluidml::worker::ExecutorImpl *>(e->impl.get())->CompileBuffer(onnx_bytes, size, pm, pl, pj);
  });
}

int fml_executor_invoke(fml_executor *e, const char *const *names, void *const *buffers, size_t count,
                        size_t *ns_per_epoch) {
  if (!e || !e->impl || (count && (!names || !buffers))) return 1;
  return Guard(e, [&] {
    std::unordered_map<std::string, void *> args;
    for (size_t i = 0; i < count; ++i) args[names[i]] = buffers[i];
    size_t ns = e->impl->Invoke(args);
    if (ns_per_epoch) *ns_per_epoch = ns;
  });
}

int fml_executor_plan_buffer(fml_executor *e, const void *onnx_bytes, size_t size, const char *llvm_path,
                             const char *json_path) {
  if (!e || !e->impl || !onnx_bytes) return 1;
  return Guard(e, [&] {
    std::ofstream fl, fj;
    std::ofstream *pl = OpenOpt(fl, llvm_path), *pj = OpenOpt(fj, json_path);
    static_cast<fluidml::worker::ExecutorImpl *>(e->impl.get())->CompileBuffer(onnx_bytes, size, nullptr, pl, pj, true);
  });
}

int fml_executor_profile(fml_executor *e, const char *const *names, void *const *buffers, size_t count,
                         size_t passes, const char **json_out) {
  if (!e || !e->impl || !json_out || (count && (!names || !buffers))) return 1;
  return Guard(e, [&] {
    std::unordered_map<std::string, void *> args;
    for (size_t i = 0; i < count; ++i) args[names[i]] = buffers[i];
    e->stats = static_cast<fluidml::worker::ExecutorImpl *>(e->impl.get())->ProfileJson(args, passes);
    *json_out = e->stats.c_str();
  });
}

int fml_executor_trace(fml_executor *e, const char *const *names, void *const *buffers, size_t count,
                       size_t passes, const char **json_out) {
  if (!e || !e->impl || !json_out || (count && (!names || !buffers))) return 1;
  return Guard(e, [&] {
    std::unordered_map<std::string, void *> args;
    for (size_t i = 0; i < count; ++i) args[names[i]] = buffers[i];
    e->stats = static_cast<fluidml::worker::ExecutorImpl *>(e->impl.get())->TraceJson(args, passes);
    *json_out = e->stats.c_str();
  });
}

const char *fml_executor_stats_json(fml_executor *e) {
  if (!e || !e->impl) return "{}";
  e->stats = e->impl->GetStatsJson();
  return e->stats.c_str();
}

}  // extern "C"
