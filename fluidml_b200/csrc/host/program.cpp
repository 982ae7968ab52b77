#include "program.h"
#include <algorithm>
#include <unordered_set>
#include <cstdio>
#include <cstdlib>
#include <vector>

namespace fluidml {
namespace worker {

namespace {

void Check(int status, const std::string &what) {
  if (status != FML_OK) throw Error(what + ": " + fml_last_error());
}

size_t AlignUp(size_t v, size_t a) { return a <= 1 ? v : (v + a - 1) / a * a; }

// A placeholder base address with the alignment every planned tenant has.
void *const kPlaceholder = reinterpret_cast<void *>(static_cast<uintptr_t>(1) << 20);

kernel::ConstResolver PlaceholderResolver() {
  return [](const flow::RegionPtr &r) { return kernel::MakeTensor(*r, kPlaceholder); };
}

const flow::RegionPtr &Owner(const AliasMap &aliases, const flow::RegionPtr &r) {
  auto it = aliases.find(r.get());
  return it == aliases.end() ? r : it->second;
}

// Row-major logical bytes -> bytes in the region's physical order (builder.cpp:280-296).
std::vector<uint8_t> PermuteConstant(const flow::Region &r) {
  const std::vector<uint8_t> &src = r.constant->Bytes();
  if (utils::IsDefaultLayout(r.layout)) return src;
  const size_t es = GetSizeFromType(r.meta.GetType());
  const std::vector<int64_t> &shape = r.meta.GetShape();
  const std::vector<int64_t> strides = r.GetStrides();
  std::vector<uint8_t> dst(src.size());
  const size_t rank = shape.size();
  std::vector<int64_t> idx(rank, 0);
  const int64_t n = r.meta.GetElementsNum();
  for (int64_t e = 0; e < n; ++e) {
    int64_t off = 0;
    for (size_t d = 0; d < rank; ++d) off += idx[d] * strides[d];
    memcpy(dst.data() + off * es, src.data() + e * es, es);
    for (size_t d = rank; d-- > 0;) {
      if (++idx[d] < shape[d]) break;
      idx[d] = 0;
    }
  }
  return dst;
}

}  // namespace

AliasMap Lowering::ComputeAliases(const flow::Sequence &sequence, const kernel::KernelOptions &ko) {
  AliasMap aliases;
  const kernel::ConstResolver resolve = PlaceholderResolver();
  for (const auto &node : sequence.nodes) {
    if (node->inputs.size() != 1 || node->output->kind != flow::Region::kInner) continue;
    std::unique_ptr<kernel::Kernel> k = kernel::SelectKernel(*node, resolve, ko);
    // the input as it will really be addressed (it may itself be a view)
    const fml_tensor in = kernel::MakeTensor(*node->inputs[0], kPlaceholder);
    flow::Region plain = *node->output;
    plain.is_view = false;
    const fml_tensor out = kernel::MakeTensor(plain, kPlaceholder);
    fml_tensor view;
    if (!k->GetView(in, out, &view)) continue;
    // the output becomes a view over the owner's bytes: same element type, explicit strides,
    // offset measured from the owner's base
    const flow::RegionPtr &owner = Owner(aliases, node->inputs[0]);
    const int64_t es = (int64_t)GetSizeFromType(node->output->meta.GetType());
    flow::Region &o = *node->output;
    o.is_view = true;
    o.view_strides.assign(view.stride, view.stride + view.rank);
    o.view_offset = ((char *)view.data - (char *)kPlaceholder) / es;
    aliases[node->output.get()] = owner;
  }
  return aliases;
}

void Lowering::ComputeScratch(const flow::Sequence &sequence, const kernel::KernelOptions &ko) {
  const kernel::ConstResolver resolve = PlaceholderResolver();
  for (const auto &node : sequence.nodes) {
    std::unique_ptr<kernel::Kernel> k = kernel::SelectKernel(*node, resolve, ko);
    std::vector<fml_tensor> ins;
    for (const auto &r : node->inputs) ins.push_back(kernel::MakeTensor(*r, kPlaceholder));
    node->buffer_size = k->GetBufferSize(ins, kernel::MakeTensor(*node->output, kPlaceholder));
  }
}

std::vector<memory::Info> Lowering::Lifetimes(const flow::Sequence &sequence, const AliasMap &aliases) {
  std::unordered_map<const flow::Region *, std::pair<size_t, size_t>> life;
  auto touch = [&](const flow::RegionPtr &r0, size_t i) {
    const flow::RegionPtr &r = Owner(aliases, r0);
    if (!r->NeedMemoryAllocation()) return;
    auto it = life.find(r.get());
    if (it == life.end()) life[r.get()] = {i, i};
    else { it->second.first = std::min(it->second.first, i); it->second.second = std::max(it->second.second, i); }
  };
  for (size_t i = 0; i < sequence.nodes.size(); ++i) {
    for (const auto &r : sequence.nodes[i]->inputs) touch(r, i);
    touch(sequence.nodes[i]->output, i);
  }
  std::vector<memory::Info> infos;
  for (const auto &r : sequence.regions) {
    auto it = life.find(r.get());
    if (it == life.end()) continue;
    infos.push_back({r->name, it->second.first, it->second.second, r->meta.GetSize()});
  }
  for (size_t i = 0; i < sequence.nodes.size(); ++i)
    if (sequence.nodes[i]->buffer_size > 0)
      infos.push_back({sequence.nodes[i]->name, i, i, sequence.nodes[i]->buffer_size});
  return infos;
}

Program::~Program() {
  for (fml_resident *r : resident_programs) fml_resident_destroy(r);
  if (arena) fml_free(arena);
  if (weights) fml_free(weights);
  if (io) fml_free(io);
}

std::unique_ptr<Program> Builder::Run(const flow::Flow &flow, const flow::Sequence &sequence,
                                      const memory::Index &index, const AliasMap &aliases,
                                      const Options &options) {
  auto prog = std::make_unique<Program>();
  Check(fml_set_device(options.device), "selecting the device");
  Check(fml_warmup(), "initialising the kernel library");

  // ---- constants referenced by any node: one blob, each at a 256-byte boundary
  std::unordered_map<const flow::Region *, size_t> const_offset;
  std::vector<uint8_t> blob;
  auto add_const = [&](const flow::RegionPtr &r) {
    if (r->kind != flow::Region::kConstant || const_offset.count(r.get())) return;
    const size_t off = AlignUp(blob.size(), 256);
    const std::vector<uint8_t> bytes = PermuteConstant(*r);
    blob.resize(off + std::max<size_t>(bytes.size(), 1));
    memcpy(blob.data() + off, bytes.data(), bytes.size());
    const_offset[r.get()] = off;
  };
  for (const auto &node : sequence.nodes) {
    for (const auto &r : node->inputs) add_const(r);
    for (const auto &r : node->consts) add_const(r);
  }
  prog->weight_bytes = blob.size();
  Check(fml_malloc(&prog->weights, blob.size()), "allocating the weight blob");
  if (!blob.empty()) {
    Check(fml_memcpy_h2d(prog->weights, blob.data(), blob.size(), nullptr), "uploading the weights");
    Check(fml_stream_sync(nullptr), "uploading the weights");
  }

  // ---- arena (zeroed once) and interface buffers
  prog->arena_bytes = index.GetMaximum();
  Check(fml_malloc(&prog->arena, prog->arena_bytes), "allocating the arena");
  Check(fml_memset(prog->arena, 0, prog->arena_bytes, nullptr), "clearing the arena");
  std::unordered_map<const flow::Region *, size_t> io_offset;
  size_t io_bytes = 0;
  for (const auto &r : flow.regions) {
    if (r->kind != flow::Region::kInput && r->kind != flow::Region::kOutput) continue;
    io_offset[r.get()] = io_bytes;
    io_bytes = AlignUp(io_bytes + r->meta.GetSize(), 256);
  }
  prog->io_bytes = io_bytes;
  Check(fml_malloc(&prog->io, io_bytes), "allocating the interface buffers");
  Check(fml_memset(prog->io, 0, io_bytes, nullptr), "clearing the interface buffers");
  Check(fml_stream_sync(nullptr), "initialising device memory");

  auto base_of = [&](const flow::RegionPtr &r0) -> void * {
    const flow::RegionPtr &r = Owner(aliases, r0);
    switch (r->kind) {
    case flow::Region::kConstant: {
      auto it = const_offset.find(r.get());
      if (it == const_offset.end()) throw Error("constant '" + r->name + "' was never uploaded");
      return (char *)prog->weights + it->second;
    }
    case flow::Region::kInput:
    case flow::Region::kOutput: return (char *)prog->io + io_offset.at(r.get());
    default:
      if (!index.Has(r->name)) throw Error("tensor '" + r->name + "' has no place in the arena");
      return (char *)prog->arena + index.Get(r->name);
    }
  };
  // An aliased region keeps its own shape and layout over its owner's bytes.
  auto tensor_of = [&](const flow::RegionPtr &r) { return kernel::MakeTensor(*r, base_of(r)); };
  const kernel::ConstResolver resolve = [&](const flow::RegionPtr &r) { return tensor_of(r); };

  for (const std::string &name : flow.inputs) {
    const flow::RegionPtr r = flow.Get(name);
    prog->inputs.push_back({name, base_of(r), r->meta.GetSize()});
  }
  for (const std::string &name : flow.outputs) {
    const flow::RegionPtr r = flow.Get(name);
    prog->outputs.push_back({name, base_of(r), r->meta.GetSize()});
  }

  kernel::KernelOptions ko;
  ko.gemm_precision = options.gemm_precision;
  ko.autotune = options.autotune;
  kernel::LaunchRecorder rec;
  std::vector<std::pair<flow::NodePtr, std::unique_ptr<kernel::Kernel>>> kernels;
  for (const auto &node : sequence.nodes) {
    if (aliases.count(node->output.get())) { ++prog->aliased_nodes; continue; }
    kernels.emplace_back(node, kernel::SelectKernel(*node, resolve, ko));
  }
  // Weight prefetch chain: every kernel that streams constant weights is told about the next
  // such kernel's bytes (circularly: the last one names the first, for the next pass), so
  // that HBM keeps streaming weights into L2 between the launches of a latency-bound pass.
  if (options.weight_prefetch) {
    const void *next_ptr = nullptr;
    size_t next_bytes = 0;
    for (const auto &kv : kernels)
      if (kv.second->StreamedConstant(&next_ptr, &next_bytes)) break;  // the first: target of the last
    for (size_t i = kernels.size(); i-- > 0;) {
      const void *own = nullptr;
      size_t own_bytes = 0;
      if (!kernels[i].second->StreamedConstant(&own, &own_bytes)) continue;
      if (next_ptr && next_ptr != own) kernels[i].second->SetPrefetch(next_ptr, next_bytes);
      next_ptr = own;
      next_bytes = own_bytes;
    }
  }
  // ---- resident programs: maximal runs of nodes that have a resident stage form
  std::vector<int> run_of(kernels.size(), -1);             // kernel index -> run index
  std::vector<std::vector<fml_resident_stage>> run_stages;  // per run
  std::vector<size_t> run_first;
  if (options.resident) {
    // regions read by nodes outside a run (through views as well) must be stored for them
    auto consumers_outside = [&](const flow::Region *r, size_t lo, size_t hi) {
      // kernels[lo..hi) is the run; any other node of the sequence reading r (or a view of it)?
      std::unordered_set<const flow::Node *> inside;
      for (size_t i = lo; i < hi; ++i) inside.insert(kernels[i].first.get());
      if (r->kind != flow::Region::kInner) return true;
      for (const auto &n : sequence.nodes) {
        if (inside.count(n.get()) || aliases.count(n->output.get())) continue;
        for (const auto &in : n->inputs)
          if (Owner(aliases, in).get() == r) return true;
      }
      return false;
    };
    auto consumers_total = [&](const flow::Region *r) {
      int count = 0;
      for (const auto &n : sequence.nodes) {
        if (aliases.count(n->output.get())) continue;
        for (const auto &in : n->inputs)
          if (Owner(aliases, in).get() == r) ++count;
      }
      return count;
    };
    auto inputs_of = [&](const flow::NodePtr &node) {
      std::vector<fml_tensor> ins;
      for (const auto &r : node->inputs) ins.push_back(tensor_of(r));
      return ins;
    };
    size_t i = 0;
    while (i < kernels.size()) {
      std::vector<fml_resident_stage> stages;
      std::vector<std::pair<size_t, size_t>> span;  // kernels covered by each stage: [first, last]
      size_t j = i;
      while (j < kernels.size()) {
        fml_resident_stage st;
        if (!kernels[j].second->DescribeResident(inputs_of(kernels[j].first), tensor_of(kernels[j].first->output), &st)) break;
        size_t last = j;
        if (st.kind == FML_RESIDENT_GEMM && j + 1 < kernels.size()) {
          // a LayerNorm that is the only reader of this product rides in its epilogue
          const flow::NodePtr &ln = kernels[j + 1].first;
          fml_tensor scale, bias;
          float eps = 0.0f;
          if (!ln->inputs.empty() && ln->inputs[0].get() == kernels[j].first->output.get() &&
              kernels[j].first->output->kind == flow::Region::kInner && consumers_total(kernels[j].first->output.get()) == 1 &&
              kernels[j + 1].second->DescribeLayerNorm(tensor_of(ln->inputs[0]), &scale, &bias, &eps)) {
            st.layernorm = 1; st.ln_scale = scale; st.ln_bias = bias; st.ln_eps = eps;
            st.out = tensor_of(ln->output);
            last = j + 1;
          }
        }
        stages.push_back(st);
        span.push_back({j, last});
        j = last + 1;
      }
      if (getenv("FLUIDML_RESIDENT_VERBOSE") && !stages.empty())
        fprintf(stderr, "resident: run of %zu stages starting at node '%s'\n", stages.size(), kernels[i].first->name.c_str());
      // the longest prefix of the run the library accepts (a stage it cannot take, such as a
      // product with fewer than 128 rows, ends the run there)
      while (stages.size() >= 2) {
        j = span.back().second + 1;
        for (size_t s = 0; s < stages.size(); ++s) {
          const flow::Region *out = kernels[span[s].second].first->output.get();
          stages[s].out_external = consumers_outside(out, i, j) ? 1 : 0;
        }
        fml_resident_info info;
        if (fml_resident_plan(stages.data(), (int32_t)stages.size(), 0, &info) == FML_OK) break;
        if (getenv("FLUIDML_RESIDENT_VERBOSE"))
          fprintf(stderr, "resident: %zu stages from node '%s' refused: %s\n", stages.size(), kernels[i].first->name.c_str(), fml_last_error());
        stages.pop_back();
        span.pop_back();
      }
      if (stages.size() >= 2) {
        j = span.back().second + 1;
        fml_resident *prog_r = nullptr;
        const int st = fml_resident_create(stages.data(), (int32_t)stages.size(), &prog_r);
        if (st == FML_OK) {
          for (size_t k = i; k < j; ++k) run_of[k] = (int)run_stages.size();
          run_stages.push_back(stages);
          run_first.push_back(i);
          prog->resident_programs.push_back(prog_r);
          prog->resident_stages += stages.size();
          fml_resident_info info;
          if (fml_resident_info_of(prog_r, &info) == FML_OK) prog->resident_scratch_bytes += info.scratch_bytes + info.packed_weight_bytes;
        } else if (st != FML_UNSUPPORTED) {
          throw Error(std::string("creating a resident program: ") + fml_last_error());
        } else if (getenv("FLUIDML_RESIDENT_VERBOSE")) {
          fprintf(stderr, "resident: %zu stages from node '%s' stay separate launches: %s\n", stages.size(),
                  kernels[i].first->name.c_str(), fml_last_error());
        }
        i = j;
      } else {
        i = std::max(j, i + 1);
      }
    }
  }
  for (size_t ki = 0; ki < kernels.size(); ++ki) {
    const auto &kv = kernels[ki];
    const flow::NodePtr &node = kv.first;
    const std::unique_ptr<kernel::Kernel> &k = kv.second;
    if (run_of[ki] >= 0) {
      if (run_first[run_of[ki]] == ki) {
        fml_resident *r = prog->resident_programs[run_of[ki]];
        rec.SetNode(node->name);
        rec.Add("ResidentProgramKernel", [r](void *s) { return fml_resident_launch(r, s); });
      }
      continue;
    }
    std::vector<fml_tensor> ins;
    for (const auto &r : node->inputs) ins.push_back(tensor_of(r));
    const fml_tensor out = tensor_of(node->output);
    kernel::Buffer buf;
    const size_t need = k->GetBufferSize(ins, out);
    if (need > node->buffer_size)
      throw Error("node '" + node->name + "' needs more scratch than was planned for it");
    if (need > 0) {
      buf.data = (char *)prog->arena + index.Get(node->name);
      buf.bytes = node->buffer_size;
    }
    if (options.gemm_tiles) {
      auto it = options.gemm_tiles->find(node->name);
      if (it != options.gemm_tiles->end()) k->PresetTiles(it->second.first, it->second.second);
    }
    rec.SetNode(node->name);
    k->Launch(rec, ins, out, buf);
    int tn = 0, sk = 0;
    if (options.gemm_tiles && k->TunedTiles(&tn, &sk)) (*options.gemm_tiles)[node->name] = {tn, sk};
  }
  prog->launches = rec.Launches();
  for (const auto &l : prog->launches) ++prog->kernel_histogram[l.kernel];
  return prog;
}

// ------------------------------------------------------------------------------ Runner
Runner::Runner(std::unique_ptr<Program> program, const Options &options)
    : program_(std::move(program)), options_(options) {
  Check(fml_set_device(options_.device), "selecting the device");
  Check(fml_stream_create(&stream_), "creating the stream");
  Check(fml_event_create(&ev_start_), "creating an event");
  Check(fml_event_create(&ev_stop_), "creating an event");
  // One eager pass: validates every launch and lets the library do its lazy set-up before
  // anything is captured.
  for (const auto &l : program_->launches) {
    int st = l.fn(stream_);
    if (st != FML_OK) throw Error("node '" + l.node + "' (" + l.kernel + "): " + fml_last_error());
  }
  Check(fml_check_device(stream_), "first forward pass");
  if (options_.cuda_graph && !program_->launches.empty()) {
    Check(fml_graph_begin_capture(stream_), "starting the graph capture");
    for (const auto &l : program_->launches) {
      int st = l.fn(stream_);
      if (st != FML_OK) {
        const std::string msg = fml_last_error();
        fml_graph_abort_capture(stream_);
        throw Error("capturing node '" + l.node + "' (" + l.kernel + "): " + msg);
      }
    }
    Check(fml_graph_end_capture(stream_, &graph_exec_), "instantiating the graph");
  }
}

Runner::~Runner() {
  if (stream_) fml_stream_sync(stream_);
  if (graph_exec_) fml_graph_destroy(graph_exec_);
  if (ev_start_) fml_event_destroy(ev_start_);
  if (ev_stop_) fml_event_destroy(ev_stop_);
  if (stream_) fml_stream_destroy(stream_);
}

void Runner::Replay() {
  if (graph_exec_) {
    Check(fml_graph_launch(graph_exec_, stream_), "launching the graph");
    return;
  }
  for (const auto &l : program_->launches) {
    int st = l.fn(stream_);
    if (st != FML_OK) throw Error("node '" + l.node + "' (" + l.kernel + "): " + fml_last_error());
  }
}

size_t Runner::Run(const std::unordered_map<std::string, void *> &args, size_t epoch) {
  if (epoch == 0) epoch = 1;
  Check(fml_set_device(options_.device), "selecting the device");
  // args.at() throws std::out_of_range for a missing name, as the reference does
  // (src/worker/runner.cpp:70); look everything up before touching the device.
  std::vector<void *> in_host, out_host;
  for (const auto &b : program_->inputs) in_host.push_back(args.at(b.name));
  for (const auto &b : program_->outputs) out_host.push_back(args.at(b.name));
  for (size_t i = 0; i < in_host.size(); ++i) {
    if (!in_host[i]) throw Error("input '" + program_->inputs[i].name + "' is a null pointer");
    Check(fml_memcpy_h2d(program_->inputs[i].device, in_host[i], program_->inputs[i].bytes, stream_), "copying an input");
  }
  Check(fml_event_record(ev_start_, stream_), "recording an event");
  for (size_t e = 0; e < epoch; ++e) Replay();
  Check(fml_event_record(ev_stop_, stream_), "recording an event");
  for (size_t i = 0; i < out_host.size(); ++i) {
    if (!out_host[i]) throw Error("output '" + program_->outputs[i].name + "' is a null pointer");
    Check(fml_memcpy_d2h(out_host[i], program_->outputs[i].device, program_->outputs[i].bytes, stream_), "copying an output");
  }
  const int status = fml_check_device(stream_);
  if (status == FML_DEVICE_TIMEOUT)  // a resident program's buffers hold mixed generations after an abandoned pass
    for (fml_resident *r : program_->resident_programs) fml_resident_reset(r, stream_);
  Check(status, "forward pass");
  float ms = 0.0f;
  Check(fml_event_elapsed_ms(ev_start_, ev_stop_, &ms), "reading the timer");
  return (size_t)((double)ms * 1e6 / (double)epoch);
}

std::map<std::string, Runner::KernelTime> Runner::Profile(const std::unordered_map<std::string, void *> &args,
                                                          size_t passes) {
  Check(fml_set_device(options_.device), "selecting the device");
  for (const auto &b : program_->inputs)
    Check(fml_memcpy_h2d(b.device, args.at(b.name), b.bytes, stream_), "copying an input");
  const size_t n = program_->launches.size();
  std::vector<void *> events(2 * (n + 1), nullptr);
  for (auto &e : events) Check(fml_event_create(&e), "creating an event");
  std::map<std::string, KernelTime> out;
  for (size_t p = 0; p < passes; ++p) {
    for (size_t i = 0; i < n; ++i) {
      Check(fml_event_record(events[2 * i], stream_), "recording an event");
      int st = program_->launches[i].fn(stream_);
      if (st != FML_OK) throw Error("node '" + program_->launches[i].node + "': " + fml_last_error());
      Check(fml_event_record(events[2 * i + 1], stream_), "recording an event");
    }
    Check(fml_event_record(events[2 * n], stream_), "recording an event");
    Check(fml_event_record(events[2 * n + 1], stream_), "recording an event");
    Check(fml_check_device(stream_), "profiled forward pass");
    for (size_t i = 0; i <= n; ++i) {
      float ms = 0;
      Check(fml_event_elapsed_ms(events[2 * i], events[2 * i + 1], &ms), "reading the timer");
      KernelTime &k = out[i < n ? program_->launches[i].kernel : std::string("(empty event pair)")];
      k.us += (double)ms * 1e3;
      k.launches += 1;
      // FLUIDML_PROFILE_NODES=1: one more entry per launch, keyed "node <name>"
      static const bool per_node = [] { const char *e = getenv("FLUIDML_PROFILE_NODES"); return e && e[0] == '1'; }();
      if (per_node && i < n) {
        KernelTime &pn = out["node " + program_->launches[i].node];
        pn.us += (double)ms * 1e3;
        pn.launches += 1;
      }
    }
  }
  for (auto &e : events) fml_event_destroy(e);
  return out;
}

std::map<std::string, Runner::KernelTime> Runner::Trace(const std::unordered_map<std::string, void *> &args,
                                                        size_t passes, double *pass_us,
                                                        std::vector<double> *per_launch_us) {
  Check(fml_set_device(options_.device), "selecting the device");
  if (passes < 1) passes = 1;
  if (!args.empty())  // with no arguments the interface buffers are traced as they are
    for (const auto &b : program_->inputs)
      Check(fml_memcpy_h2d(b.device, args.at(b.name), b.bytes, stream_), "copying an input");
  const size_t n = program_->launches.size(), reps = passes + 2, cap = n * reps;
  std::map<std::string, KernelTime> out;
  if (n == 0) return out;
  void *buf = nullptr, *cursor = nullptr;
  Check(fml_malloc(&buf, cap * 8), "allocating the trace buffer");
  Check(fml_malloc(&cursor, 4), "allocating the trace cursor");
  Check(fml_memset(cursor, 0, 4, stream_), "clearing the trace cursor");
  Check(fml_stream_sync(stream_), "clearing the trace cursor");
  std::vector<unsigned long long> stamps(cap, 0);
  unsigned stamped = 0;
  int st = fml_set_kernel_trace(buf, cursor, (unsigned)cap);
  if (st == FML_OK) {
    for (size_t r = 0; r < reps && st == FML_OK; ++r) {
      if (graph_exec_) st = fml_graph_launch(graph_exec_, stream_);
      else for (const auto &l : program_->launches) { st = l.fn(stream_); if (st != FML_OK) break; }
    }
    if (st == FML_OK) st = fml_check_device(stream_);
    fml_set_kernel_trace(nullptr, nullptr, 0);
    if (st == FML_OK) st = fml_memcpy_d2h(stamps.data(), buf, cap * 8, stream_);
    if (st == FML_OK) st = fml_memcpy_d2h(&stamped, cursor, 4, stream_);
    if (st == FML_OK) st = fml_stream_sync(stream_);
  }
  fml_free(buf);
  fml_free(cursor);
  Check(st, "tracing the forward pass");
  if (stamped != cap)
    throw Error("the launch list does not stamp once per launch (" + std::to_string(stamped) + " stamps for " +
                std::to_string(cap) + " launches): use Profile for this model");
  // every launch stamps once: launch i of replay r is entry r * n + i
  std::vector<double> period(n, 0.0);
  std::vector<unsigned long long> v(passes);
  for (size_t i = 0; i < n; ++i) {
    for (size_t r = 0; r < passes; ++r) {
      const size_t at = (r + 1) * n + i;
      v[r] = stamps[at + 1] - stamps[at];
    }
    std::sort(v.begin(), v.end());
    period[i] = (double)v[passes / 2] * 1e-3;
  }
  double total = 0.0;
  for (size_t i = 0; i < n; ++i) {
    KernelTime &k = out[program_->launches[i].kernel];
    k.us += period[i];
    k.launches += 1;
    total += period[i];
  }
  if (pass_us) *pass_us = total;
  if (per_launch_us) *per_launch_us = period;
  return out;
}

}  // namespace worker
}  // namespace fluidml
