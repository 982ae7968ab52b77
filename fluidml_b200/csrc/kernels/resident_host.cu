// Planner, plan checker, weight packer and C ABI of the resident stage program (the persistent
// kernel itself is in resident.cu, the data model in resident.cuh).
//
// Planning.  Every GEMM stage [128 x K] x [K x N] is cut into units (column slab of tile_n,
// k split): one unit per CTA, so that every SM streams about 1 / ctas of every weight matrix.
// tile_n and the number of splits S are chosen per stage with a small time model (the cost of
// a tcgen05.mma does not fall below ~104 cycles however narrow the tile, and the S partial
// tiles of a slab cross L2 twice), or given by the caller.  After its unit a CTA "finishes"
// part of the stage: without LayerNorm the rows [s * 128 / S, (s + 1) * 128 / S) of its own
// slab (it only needs the S partial tiles of that slab), with LayerNorm whole rows (it needs
// every slab).  An attention stage is cut into (head, 16 query rows) steps.
//
// Buffers.  Stage outputs and split-K partial tiles live in buffers the program owns; every
// word in them carries the parity of the buffer's write generation (resident.cuh), which is all
// the synchronisation there is.  A buffer is handed to a later stage once its last reader is a
// given number of stages back; the plan is then checked and the distance doubled until it
// passes.
//
// Checking.  The plan is executed symbolically: a step can run once every step that writes
// words it reads (same buffer, same generation, overlapping region) has run; each step gets a
// vector clock (how many steps of every CTA must be complete before it can start, by program
// order and by those read-after-write edges alone).  The check demands that every read is
// covered exactly by writes of its generation, that no two steps write the same word of one
// generation, and that every step that overwrites a buffer region is ordered, by those clocks,
// after every reader and writer of the region's previous generation.  A plan that fails is not
// created.
#include "resident_host.h"
#include <algorithm>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

struct fml_resident {
  fml::res::KernelArgs args{};
  int ctas = 0;
  size_t smem_bytes = 0;
  void *scratch = nullptr, *packed = nullptr;
  size_t tagged_offset = 0, tagged_bytes = 0;  // the tagged buffers inside scratch
  bool trace = false;
  size_t trace_entries = 0;
  fml_resident_info info{};
  int device = 0;
};

namespace fml {
namespace res {
namespace {

struct Rows {  // a tensor seen as [rows x cols] with unit column stride
  int64_t rows = 0, cols = 0, ld = 0;
};
bool as_rows(const fml_tensor &t, Rows &r) {
  if (t.rank < 1 || t.dtype != FML_F32 || t.stride[t.rank - 1] != 1) return false;
  r.cols = t.shape[t.rank - 1];
  r.rows = 1;
  r.ld = r.cols;
  int64_t expect = 0;  // stride the next outer dim must have for rows to be evenly spaced
  for (int d = t.rank - 2; d >= 0; --d) {
    if (t.shape[d] == 1) continue;
    if (expect == 0) { r.ld = t.stride[d]; expect = t.stride[d] * t.shape[d]; }
    else { if (t.stride[d] != expect) return false; expect *= t.shape[d]; }
    r.rows *= t.shape[d];
  }
  return r.ld >= r.cols;
}

struct PackDesc {
  unsigned long long dst;
  int n0, k0, tile_n, pad;
};

constexpr size_t kSmemMax = 227 * 1024;

size_t attention_smem(int D, int Dv, int Sk) {
  return (size_t)(kAttnRows * (D + 4) + Sk * (D + 4) + Sk * Dv + 8 * kAttnRows * Dv + kAttnRows * (Sk | 1) +
                  kAttnRows * Sk) * sizeof(float);
}

// Time model of one GEMM stage in microseconds (see the header comment).
double stage_cost(int K, int N, int tile_n, int S, bool ln) {
  const int nkb = (K / kBK + S - 1) / S;
  const double mma = nkb * 12.0 * std::max(104.0, 0.54 * tile_n) / 1900.0;
  const double tile_bytes = 128.0 * tile_n * 4;
  const double exchange = 0.55 + tile_bytes / 55e3 + 0.4 + tile_bytes / 65e3;
  const double a_load = 0.7 + nkb * 0.05;
  return mma + exchange + a_load + (ln ? 0.03 * S : 0.0);
}

struct TileChoice { int tile_n = 0, S = 0; };
TileChoice choose_tiles(int K, int N, bool ln, int ctas, int want_tn, int want_s) {
  TileChoice best;
  double best_t = 1e30;
  const int nkb = K / kBK;
  for (int tn = 16; tn <= kMaxTileN; tn += 16) {
    if (want_tn && tn != want_tn) continue;
    if (N % tn) continue;
    const int slabs = N / tn;
    if (slabs > ctas) continue;
    for (int S = 1; S <= nkb && S <= kRows; ++S) {
      if (want_s && S != want_s) continue;
      if ((long long)slabs * S > ctas) break;
      const double t = stage_cost(K, N, tn, S, ln);
      if (t < best_t) { best_t = t; best.tile_n = tn; best.S = S; }
    }
  }
  return best;
}

// FLUIDML_RESIDENT_TILES="64x4,64x12,128x6,64x12": tile_n x splits for the GEMM stages in order,
// repeated cyclically (an experiment knob; stages the list does not fit fall back to the model).
bool env_tiles(int gemm_index, int &tn, int &s) {
  static const std::vector<std::pair<int, int>> list = [] {
    std::vector<std::pair<int, int>> v;
    const char *e = getenv("FLUIDML_RESIDENT_TILES");
    if (!e) return v;
    std::string str(e);
    size_t pos = 0;
    while (pos < str.size()) {
      size_t end = str.find(',', pos);
      if (end == std::string::npos) end = str.size();
      const std::string item = str.substr(pos, end - pos);
      const size_t x = item.find('x');
      if (x != std::string::npos) v.push_back({atoi(item.substr(0, x).c_str()), atoi(item.substr(x + 1).c_str())});
      pos = end + 1;
    }
    return v;
  }();
  if (list.empty()) return false;
  tn = list[gemm_index % list.size()].first;
  s = list[gemm_index % list.size()].second;
  return true;
}


struct Buffer {
  size_t bytes = 0, offset = 0;
  int uses = 0;          // stages that write it in one pass
  int free_after = -1;   // last stage that reads the current content
};

struct Access {
  int buffer, gen;       // gen < 0: an input from outside the program (never written here)
  int r0, r1, c0, c1;    // rows, quads
  bool write;
  int cta, index;        // the step
};

struct OutInfo {
  const char *base = nullptr;  // out.data: bytes [base, base + 128 * N * 4) identify the tensor
  int N = 0;
  bool external = false;
  int buffer = -1, gen = 0;    // tiled copy inside the program (absent for an external output nobody reads)
};

struct Plan {
  int ctas = 0;
  std::vector<std::vector<Step>> steps;           // per CTA (without the end marker)
  std::vector<GemmStage> gemm;                    // buffer pointers are resolved at creation
  std::vector<AttnStage> attn;
  std::vector<int> stage_to_gemm, stage_to_attn;  // stage index -> index in gemm / attn
  std::vector<std::vector<PackDesc>> pack;        // per GEMM stage
  std::vector<unsigned long long> weight_begin;   // per CTA
  size_t packed_bytes = 0;
  std::vector<Buffer> buffers;
  size_t buffer_bytes = 0;
  int slot_bytes = 0, nslots = 0, overlay_bytes = 0, max_steps = 0;
  std::vector<OutInfo> outs;
  std::vector<Access> accesses;
  std::string error;
};

struct Operand {  // a [128 x cols] input of a stage
  bool tiled = false;
  int producer = -1, col0 = 0;
  const float *ptr = nullptr;  // row-major: element (0, 0)
  int64_t ld = 0;
};
struct GemmOperands { Operand a, res; bool has_res = false; int part_buffer = -1, part_gen = 0; };
struct AttnSources { int producer[3]; };

struct Planner {
  const fml_resident_stage *stages;
  int count, ctas;
  int lag;  // stages between a buffer's last reader and its next writer
  Plan plan;
  std::vector<GemmOperands> gemm_operands;
  std::vector<AttnSources> attn_sources;
  std::vector<int> last_reader;  // per stage: last stage that reads its output

  bool fail(const std::string &msg) { plan.error = msg; return false; }

  int producer_of(const void *p, int before, int64_t *elem) const {
    const char *c = (const char *)p;
    for (int j = before - 1; j >= 0; --j) {
      const OutInfo &o = plan.outs[j];
      if (c >= o.base && c < o.base + (size_t)kRows * o.N * 4) {
        *elem = (c - o.base) / 4;
        return j;
      }
    }
    return -1;
  }
  // same lookup before plan.outs exists (first pass over the stages)
  static bool out_extent(const fml_resident_stage &st, const char **base, int64_t *n) {
    if (!st.out.data || st.out.rank < 2) return false;
    *base = (const char *)st.out.data;
    if (st.kind == FML_RESIDENT_GEMM) *n = st.out.shape[st.out.rank - 1];
    else *n = st.out.stride[st.out.rank - 2];
    return *n > 0;
  }
  void find_last_readers() {
    last_reader.assign(count, -1);
    for (int i = 0; i < count; ++i) {
      const fml_resident_stage &st = stages[i];
      const fml_tensor *ins[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
      if (st.kind == FML_RESIDENT_GEMM) { ins[0] = &st.a; ins[1] = &st.residual; }
      else { ins[0] = &st.q; ins[1] = &st.kt; ins[2] = &st.v; }
      for (const fml_tensor *t : ins) {
        if (!t || !t->data) continue;
        for (int j = i - 1; j >= 0; --j) {
          const char *base; int64_t n;
          if (!out_extent(stages[j], &base, &n)) continue;
          const char *c = (const char *)t->data;
          if (c >= base && c < base + (size_t)kRows * n * 4) { last_reader[j] = std::max(last_reader[j], i); break; }
        }
      }
    }
  }
  // a buffer of `bytes` for stage `stage`, whose content is last read by stage `free_after`
  int take_buffer(size_t bytes, int stage, int free_after, int *gen) {
    int best = -1;
    for (size_t b = 0; b < plan.buffers.size(); ++b) {
      Buffer &bf = plan.buffers[b];
      if (bf.bytes == bytes && bf.free_after + lag <= stage) { best = (int)b; break; }
    }
    if (best < 0) {
      Buffer bf;
      bf.bytes = bytes;
      plan.buffers.push_back(bf);
      best = (int)plan.buffers.size() - 1;
    }
    Buffer &bf = plan.buffers[best];
    *gen = bf.uses++;
    bf.free_after = free_after;
    return best;
  }
  void access(int buffer, int gen, int r0, int r1, int c0, int c1, bool write, int cta) {
    plan.accesses.push_back({buffer, gen, r0, r1, c0, c1, write, cta, (int)plan.steps[cta].size()});
  }

  bool operand(const fml_tensor &t, int i, int64_t cols, Operand &op, const char *what) {
    Rows r;
    if (!as_rows(t, r) || r.rows != kRows || r.cols != cols)
      return fail(std::string(what) + ": expected a [128 x n] fp32 block with unit column stride");
    int64_t e = 0;
    const int j = producer_of(t.data, i, &e);
    if (j >= 0) {
      const OutInfo &o = plan.outs[j];
      if (r.ld != o.N || e >= o.N || (e & 3) || e + cols > o.N)
        return fail(std::string(what) + ": not a column range of the producing stage's rows");
      op.tiled = true; op.producer = j; op.col0 = (int)e;
      return true;
    }
    if (((uintptr_t)t.data & 15) || (r.ld & 3)) return fail(std::string(what) + ": external operand is not 16-byte aligned");
    op.tiled = false; op.ptr = (const float *)t.data; op.ld = r.ld;
    return true;
  }
  static int tagsel(int gen, int uses) { return (gen & 1) | ((uses & 1) << 1); }

  bool run() {
    plan = Plan();
    gemm_operands.clear();
    attn_sources.clear();
    plan.ctas = ctas;
    plan.steps.assign(ctas, {});
    plan.weight_begin.assign(ctas, 0);
    plan.stage_to_gemm.assign(count, -1);
    plan.stage_to_attn.assign(count, -1);
    if (count < 1) return fail("no stages");
    if (ctas < 1) return fail("no CTAs");
    find_last_readers();
    std::vector<std::vector<std::pair<int, PackDesc>>> cta_chunks(ctas);
    int max_tile_n = 16;
    size_t attn_bytes = 0;
    int max_finish_slots = 1;

    for (int i = 0; i < count; ++i) {
      const fml_resident_stage &st = stages[i];
      OutInfo o;
      o.external = st.out_external != 0;
      o.base = (const char *)st.out.data;
      if (!st.out.data || ((uintptr_t)st.out.data & 15)) return fail("stage output is null or not 16-byte aligned");
      const bool read_inside = last_reader[i] >= 0;
      if (!o.external && !read_inside) return fail("a stage output that nothing reads");

      if (st.kind == FML_RESIDENT_GEMM) {
        Rows ro;
        if (!as_rows(st.out, ro) || ro.rows != kRows) return fail("GEMM output must be a [128 x N] fp32 block");
        const int N = (int)ro.cols;
        if (st.w.rank != 2 || st.w.dtype != FML_F32 || !st.w.data || st.w.shape[1] != N) return fail("GEMM weights must be a [K, N] fp32 matrix");
        const int K = (int)st.w.shape[0];
        if (K < kBK || K % kBK || N % 16 || N > 4096) return fail("GEMM needs K a multiple of 32 and N a multiple of 16 up to 4096");
        if (!o.external && ro.ld != N) return fail("an internal GEMM output must be dense");
        if (o.external && (ro.ld & 3)) return fail("external GEMM output rows must be 16-byte multiples");
        if (st.act < FML_ACT_NONE || st.act > FML_ACT_SIGMOID) return fail("unsupported activation");
        o.N = N;
        if (read_inside) o.buffer = take_buffer((size_t)kRows * N * 4, i, last_reader[i], &o.gen);
        plan.outs.push_back(o);
        GemmOperands ops;
        if (!operand(st.a, i, K, ops.a, "GEMM input")) return false;
        ops.has_res = st.residual.data != nullptr;
        if (ops.has_res && !operand(st.residual, i, N, ops.res, "GEMM residual")) return false;
        if (st.bias.data && (st.bias.dtype != FML_F32 || st.bias.shape[st.bias.rank - 1] != N || st.bias.stride[st.bias.rank - 1] != 1 ||
                             ((uintptr_t)st.bias.data & 15)))
          return fail("GEMM bias must be a dense, aligned [N] vector");
        if (st.layernorm) {
          for (const fml_tensor *t : {&st.ln_scale, &st.ln_bias})
            if (!t->data || t->dtype != FML_F32 || t->shape[t->rank - 1] != N || t->stride[t->rank - 1] != 1 || ((uintptr_t)t->data & 15))
              return fail("LayerNorm scale / bias must be dense, aligned [N] vectors");
        }
        const int gi = (int)plan.gemm.size();
        int want_tn = st.tile_n, want_s = st.split_k;
        if (!want_tn && !want_s) env_tiles(gi, want_tn, want_s);
        TileChoice tc = choose_tiles(K, N, st.layernorm != 0, ctas, want_tn, want_s);
        if (!tc.tile_n && (want_tn || want_s)) tc = choose_tiles(K, N, st.layernorm != 0, ctas, 0, 0);
        if (!tc.tile_n) return fail("no tiling of this GEMM fits the grid");
        max_tile_n = std::max(max_tile_n, tc.tile_n);
        if (getenv("FLUIDML_RESIDENT_VERBOSE"))
          fprintf(stderr, "resident: stage %d GEMM K=%d N=%d -> tile_n %d x %d splits (%d units, model %.2f us)\n", i, K, N,
                  tc.tile_n, tc.S, N / tc.tile_n * tc.S, stage_cost(K, N, tc.tile_n, tc.S, st.layernorm != 0));
        const int slabs = N / tc.tile_n, S = tc.S, nkb_total = K / kBK, NC = N / 4;
        const bool ln = st.layernorm != 0;
        const bool res_tagged = ops.has_res && ops.res.tiled;
        // fetch slots a finishing thread needs at once: LayerNorm keeps all its quads of a row
        const int per = S + (res_tagged ? 1 : 0);
        max_finish_slots = std::max(max_finish_slots, ln ? ((NC + kWorkers - 1) / kWorkers) * per : per);
        if (ln && (NC + kWorkers - 1) / kWorkers > 4) return fail("LayerNorm rows longer than 4096");
        ops.part_buffer = take_buffer((size_t)S * N * kRows * 4, i, i, &ops.part_gen);

        GemmStage g{};
        g.N = N; g.K = K; g.S = S; g.tile_n = tc.tile_n;
        g.a_tiled = ops.a.tiled; g.a_ld = ops.a.ld; g.a = ops.a.ptr;
        g.a_tag = ops.a.tiled ? 0 : -1;  // selectors are filled in once every buffer's use count is known
        g.bias = (const float *)st.bias.data;
        g.res_tiled = res_tagged; g.res_ld = ops.res.ld; g.res = ops.has_res ? ops.res.ptr : nullptr;
        g.res_tag = res_tagged ? 0 : -1;
        g.act = st.act; g.c0 = st.act_param[0]; g.c1 = st.act_param[1]; g.c2 = st.act_param[2];
        g.ln = ln; g.gamma = (const float *)st.ln_scale.data; g.beta = (const float *)st.ln_bias.data; g.eps = st.ln_eps;
        g.out_rm = o.external ? (float *)st.out.data : nullptr;
        g.out_ld = ro.ld;
        plan.gemm.push_back(g);
        plan.stage_to_gemm[i] = gi;
        gemm_operands.push_back(ops);
        plan.pack.push_back({});

        // ---- units: read A columns [kb0 * 32, kb1 * 32), write their partial tile
        for (int n = 0; n < slabs; ++n)
          for (int s = 0; s < S; ++s) {
            const int cta = (n * S + s) % ctas;
            const int kb0 = (int)((long long)s * nkb_total / S), kb1 = (int)((long long)(s + 1) * nkb_total / S);
            Step u{};
            u.kind = kUnit; u.stage = gi; u.p0 = n; u.p1 = s; u.p2 = kb0; u.p3 = kb1 - kb0;
            if (ops.a.tiled)
              access(plan.outs[ops.a.producer].buffer, plan.outs[ops.a.producer].gen, 0, kRows, (ops.a.col0 + kb0 * kBK) / 4,
                     (ops.a.col0 + kb1 * kBK) / 4, false, cta);
            access(ops.part_buffer, ops.part_gen, 0, kRows, s * NC + n * tc.tile_n / 4, s * NC + (n + 1) * tc.tile_n / 4, true, cta);
            plan.steps[cta].push_back(u);
            for (int kb = kb0; kb < kb1; ++kb) cta_chunks[cta].push_back({gi, PackDesc{0, n * tc.tile_n, kb * kBK, tc.tile_n, 0}});
          }
        // ---- finish steps
        auto finish = [&](int cta, int r0, int r1, int q0, int q1) {
          Step f{};
          f.kind = kFinish; f.stage = gi; f.p0 = r0; f.p1 = r1; f.p2 = q0; f.p3 = q1;
          for (int s = 0; s < S; ++s) access(ops.part_buffer, ops.part_gen, r0, r1, s * NC + q0, s * NC + q1, false, cta);
          if (res_tagged)
            access(plan.outs[ops.res.producer].buffer, plan.outs[ops.res.producer].gen, r0, r1, ops.res.col0 / 4 + q0, ops.res.col0 / 4 + q1, false, cta);
          if (o.buffer >= 0) access(o.buffer, o.gen, r0, r1, q0, q1, true, cta);
          plan.steps[cta].push_back(f);
        };
        if (ln) {
          const int owners = std::min(ctas, kRows);
          for (int k = 0; k < owners; ++k) finish(k, k * kRows / owners, (k + 1) * kRows / owners, 0, NC);
        } else {
          for (int n = 0; n < slabs; ++n)
            for (int s = 0; s < S; ++s)
              finish((n * S + s) % ctas, s * kRows / S, (s + 1) * kRows / S, n * tc.tile_n / 4, (n + 1) * tc.tile_n / 4);
        }
      } else if (st.kind == FML_RESIDENT_ATTENTION) {
        // q [.., H, 128, D], kt [.., H, D, 128], v [.., H, 128, Dv], out [.., H, 128, Dv]
        const fml_tensor &q = st.q, &kt = st.kt, &v = st.v, &out = st.out;
        for (const fml_tensor *t : {&q, &kt, &v, &out})
          if (t->rank < 3 || t->dtype != FML_F32 || !t->data) return fail("attention operands must be fp32 tensors of rank >= 3");
        auto lead_one = [](const fml_tensor &t) { for (int d = 0; d < t.rank - 3; ++d) if (t.shape[d] != 1) return false; return true; };
        if (!lead_one(q) || !lead_one(kt) || !lead_one(v) || !lead_one(out)) return fail("attention over more than one batch entry");
        const int H = (int)q.shape[q.rank - 3], D = (int)q.shape[q.rank - 1], Dv = (int)v.shape[v.rank - 1];
        const int Sq = (int)q.shape[q.rank - 2], Sk = (int)kt.shape[kt.rank - 1];
        if (Sq != kRows || Sk != kRows || kt.shape[kt.rank - 2] != D || kt.shape[kt.rank - 3] != H || v.shape[v.rank - 3] != H ||
            v.shape[v.rank - 2] != Sk || out.shape[out.rank - 3] != H || out.shape[out.rank - 2] != Sq || out.shape[out.rank - 1] != Dv)
          return fail("attention shapes do not chain over 128 rows");
        if (D < 4 || Dv < 4 || D > 128 || Dv > 128 || (D & 3) || (Dv & 3)) return fail("attention head sizes must be multiples of 4 up to 128");
        if (st.divisor == 0.0f) return fail("attention divisor is zero");
        // the output: element (h, r, d) at r * ld + h * hs + d
        if (out.stride[out.rank - 1] != 1) return fail("attention output columns must be contiguous");
        const int64_t o_ld = out.stride[out.rank - 2], o_hs = H > 1 ? out.stride[out.rank - 3] : Dv;
        if (o_ld < (int64_t)(H - 1) * o_hs + Dv || (o_hs & 3) || (o_ld & 3) || o_hs < Dv) return fail("attention output heads overlap or are misaligned");
        if (!o.external && o_ld != (int64_t)H * o_hs) return fail("an internal attention output must be dense");
        o.N = (int)o_ld;
        if (read_inside) o.buffer = take_buffer((size_t)kRows * o.N * 4, i, last_reader[i], &o.gen);
        plan.outs.push_back(o);
        AttnStage A{};
        A.heads = H; A.D = D; A.Dv = Dv; A.Sk = Sk; A.divisor = st.divisor;
        A.o_col = 0; A.o_hs = (int)o_hs; A.out_ld = o_ld;
        A.out_rm = o.external ? (float *)out.data : nullptr;
        // q / k / v: column ranges of earlier stages' tiled outputs
        struct Src { int producer, col0, hs; } src[3];
        const fml_tensor *ts[3] = {&q, &kt, &v};
        for (int k = 0; k < 3; ++k) {
          const fml_tensor &t = *ts[k];
          const int row_dim = k == 1 ? t.rank - 1 : t.rank - 2, col_dim = k == 1 ? t.rank - 2 : t.rank - 1;
          int64_t e = 0;
          const int j = producer_of(t.data, i, &e);
          if (j < 0) return fail("attention inputs must come from an earlier stage of the program");
          const OutInfo &p = plan.outs[j];
          const int64_t hs = H > 1 ? t.stride[t.rank - 3] : 0;
          const int width = (int)t.shape[col_dim];
          if (t.stride[col_dim] != 1 || t.stride[row_dim] != p.N || e >= p.N || (e & 3) || (hs & 3) || hs < 0 ||
              e + (int64_t)(H - 1) * hs + width > p.N)
            return fail("attention input is not a per-head column range of the producing stage's rows");
          src[k] = {j, (int)e, (int)hs};
        }
        A.q_col = src[0].col0; A.q_hs = src[0].hs; A.k_col = src[1].col0; A.k_hs = src[1].hs; A.v_col = src[2].col0; A.v_hs = src[2].hs;
        if (st.mask.data) {
          const fml_tensor &m = st.mask;
          int64_t e = 0;
          if (m.dtype != FML_F32 || producer_of(m.data, i, &e) >= 0) return fail("attention mask must be an fp32 tensor from outside the program");
          const int64_t want[3] = {H, Sq, Sk};
          int64_t strides[3] = {0, 0, 0};
          for (int d = 0; d < m.rank; ++d) {
            const int pos = d - (m.rank - 3);  // 0: head, 1: query row, 2: key
            if (pos < 0) { if (m.shape[d] != 1) return fail("attention mask has a batch dimension"); continue; }
            if (m.shape[d] == want[pos]) strides[pos] = m.shape[d] == 1 ? 0 : m.stride[d];
            else if (m.shape[d] != 1) return fail("attention mask does not broadcast to the scores");
          }
          A.mask = (const float *)m.data; A.m_sh = strides[0]; A.m_sr = strides[1]; A.m_sk = strides[2];
        }
        attn_bytes = std::max(attn_bytes, attention_smem(D, Dv, Sk));
        const int ai = (int)plan.attn.size();
        plan.attn.push_back(A);
        plan.stage_to_attn[i] = ai;
        attn_sources.push_back({{src[0].producer, src[1].producer, src[2].producer}});
        const int rowblocks = kRows / kAttnRows;
        for (int h = 0; h < H; ++h)
          for (int rb = 0; rb < rowblocks; ++rb) {
            const int cta = (h * rowblocks + rb) % ctas;
            Step a{};
            a.kind = kAttention; a.stage = ai; a.p0 = h; a.p1 = rb * kAttnRows;
            const int widths[3] = {D, D, Dv};
            for (int k = 0; k < 3; ++k) {
              const int c0 = (src[k].col0 + h * src[k].hs) / 4, c1 = c0 + widths[k] / 4;
              const int r0 = k == 0 ? rb * kAttnRows : 0, r1 = k == 0 ? r0 + kAttnRows : kRows;
              access(plan.outs[src[k].producer].buffer, plan.outs[src[k].producer].gen, r0, r1, c0, c1, false, cta);
            }
            if (o.buffer >= 0)
              access(o.buffer, o.gen, rb * kAttnRows, (rb + 1) * kAttnRows, (int)(h * o_hs / 4), (int)((h * o_hs + Dv) / 4), true, cta);
            plan.steps[cta].push_back(a);
          }
      } else {
        return fail("unknown stage kind");
      }
    }

    // ---- tag selectors, now that every buffer's number of generations per pass is known
    for (int i = 0; i < count; ++i) {
      const OutInfo &o = plan.outs[i];
      const int out_tag = o.buffer >= 0 ? tagsel(o.gen, plan.buffers[o.buffer].uses) : 0;
      auto tag_of = [&](int producer) { const OutInfo &p = plan.outs[producer]; return tagsel(p.gen, plan.buffers[p.buffer].uses); };
      if (plan.stage_to_gemm[i] >= 0) {
        const int gi = plan.stage_to_gemm[i];
        GemmStage &g = plan.gemm[gi];
        const GemmOperands &ops = gemm_operands[gi];
        if (ops.a.tiled) g.a_tag = tag_of(ops.a.producer);
        if (ops.has_res && ops.res.tiled) g.res_tag = tag_of(ops.res.producer);
        g.part_tag = tagsel(ops.part_gen, plan.buffers[ops.part_buffer].uses);
        g.out_tag = out_tag;
      } else {
        const int ai = plan.stage_to_attn[i];
        AttnStage &a = plan.attn[ai];
        a.q_tag = tag_of(attn_sources[ai].producer[0]);
        a.k_tag = tag_of(attn_sources[ai].producer[1]);
        a.v_tag = tag_of(attn_sources[ai].producer[2]);
        a.out_tag = out_tag;
      }
    }

    // ---- shared memory: ring slots sized for the widest tile; the overlay holds the lo(B) slots
    // and staged A rows of a unit, the fetch slots of a finish step, or the attention tiles
    plan.slot_bytes = max_tile_n * 128;
    size_t overlay = (size_t)kConvDepth * plan.slot_bytes + (size_t)kAStages * kRows * kAPitch * 4;
    overlay = std::max(overlay, attn_bytes);
    overlay = std::max(overlay, (size_t)max_finish_slots * kWorkers * 16);
    overlay = (overlay + 1023) / 1024 * 1024;
    plan.overlay_bytes = (int)overlay;
    int nslots = 8;
    while (nslots >= 2 && kernel_smem_bytes(nslots, plan.slot_bytes, plan.overlay_bytes) > kSmemMax) --nslots;
    if (nslots < 2) return fail("the stages do not fit in shared memory");
    plan.nslots = nslots;

    // ---- weight streams: each CTA's chunks back to back, streams 1024-byte aligned
    size_t off = 0;
    for (int c = 0; c < ctas; ++c) {
      off = (off + 1023) / 1024 * 1024;
      plan.weight_begin[c] = off;
      for (auto &ch : cta_chunks[c]) {
        ch.second.dst = off;
        plan.pack[ch.first].push_back(ch.second);
        off += (size_t)ch.second.tile_n * 128;
      }
    }
    plan.packed_bytes = std::max<size_t>(off, 1024);
    for (int c = 0; c < ctas; ++c) plan.max_steps = std::max(plan.max_steps, (int)plan.steps[c].size());
    size_t boff = 0;
    for (Buffer &b : plan.buffers) { b.offset = boff; boff += (b.bytes + 1023) / 1024 * 1024; }
    plan.buffer_bytes = std::max<size_t>(boff, 1024);
    std::string why;
    if (!check(why)) return fail("plan check failed: " + why);
    return true;
  }

  // Symbolic execution over read-after-write edges with vector clocks, then the ordering checks.
  bool check(std::string &why) const {
    const int C = ctas;
    // accesses of each (buffer, generation)
    std::map<std::pair<int, int>, std::vector<const Access *>> by_gen;
    std::vector<std::vector<std::vector<const Access *>>> of_step(C);
    for (int c = 0; c < C; ++c) of_step[c].resize(plan.steps[c].size());
    for (const Access &a : plan.accesses) {
      by_gen[{a.buffer, a.gen}].push_back(&a);
      of_step[a.cta][a.index].push_back(&a);
    }
    auto overlap = [](const Access &x, const Access &y) {
      const long long r = std::min(x.r1, y.r1) - std::max(x.r0, y.r0), c = std::min(x.c1, y.c1) - std::max(x.c0, y.c0);
      return r > 0 && c > 0 ? r * c : 0ll;
    };
    // coverage and write-write exclusion inside a generation
    for (const auto &kv : by_gen) {
      const auto &v = kv.second;
      for (size_t i = 0; i < v.size(); ++i) {
        if (v[i]->write) {
          for (size_t j = i + 1; j < v.size(); ++j)
            if (v[j]->write && overlap(*v[i], *v[j])) { why = "two steps write the same word of one generation"; return false; }
        } else {
          long long covered = 0;
          for (const Access *w : v)
            if (w->write) covered += overlap(*v[i], *w);
          if (covered != (long long)(v[i]->r1 - v[i]->r0) * (v[i]->c1 - v[i]->c0)) { why = "a read that no write of its generation covers"; return false; }
        }
      }
    }
    // run: a step is ready when every write its reads overlap has run
    std::vector<std::vector<char>> done(C);
    std::vector<std::vector<std::vector<int>>> clock(C);  // clock[cta][step] at step start
    for (int c = 0; c < C; ++c) { done[c].assign(plan.steps[c].size(), 0); clock[c].resize(plan.steps[c].size()); }
    std::vector<size_t> pc(C, 0);
    std::vector<std::vector<int>> last(C, std::vector<int>(C, 0));
    size_t finished = 0, total = 0;
    for (int c = 0; c < C; ++c) total += plan.steps[c].size();
    bool progress = true;
    while (progress) {
      progress = false;
      for (int c = 0; c < C; ++c) {
        while (pc[c] < plan.steps[c].size()) {
          const size_t k = pc[c];
          bool ready = true;
          std::vector<int> clk = last[c];
          for (const Access *r : of_step[c][k]) {
            if (r->write) continue;
            for (const Access *w : by_gen.at({r->buffer, r->gen})) {
              if (!w->write || !overlap(*r, *w)) continue;
              if (w->cta == c && (size_t)w->index == k) continue;
              if (!done[w->cta][w->index]) { ready = false; break; }
              // everything known at the writer's start, plus the writer itself
              const std::vector<int> &wc = clock[w->cta][w->index];
              for (int x = 0; x < C; ++x) clk[x] = std::max(clk[x], wc[x]);
              clk[w->cta] = std::max(clk[w->cta], w->index + 1);
            }
            if (!ready) break;
          }
          if (!ready) break;
          clock[c][k] = clk;
          last[c] = clk;
          last[c][c] = (int)k + 1;
          done[c][k] = 1;
          ++pc[c];
          ++finished;
          progress = true;
        }
      }
    }
    if (finished != total) { why = "the step lists cannot all run (a step waits for data written after it)"; return false; }
    // every overwrite is ordered after the readers and writers of the previous generation
    auto before = [&](const Access &x, const Access &y) {  // x's step is complete when y's may start
      if (x.cta == y.cta) return x.index < y.index;
      return clock[y.cta][y.index][x.cta] > x.index;
    };
    for (const auto &kv : by_gen) {
      if (kv.first.second == 0) continue;
      auto prev = by_gen.find({kv.first.first, kv.first.second - 1});
      if (prev == by_gen.end()) continue;
      for (const Access *w : kv.second) {
        if (!w->write) continue;
        for (const Access *p : prev->second) {
          if (!overlap(*w, *p)) continue;
          if (!before(*p, *w)) {
            char buf[220];
            snprintf(buf, sizeof(buf), "buffer %d reused too early: cta %d step %d writes generation %d while cta %d step %d may still %s generation %d",
                     w->buffer, w->cta, w->index, w->gen, p->cta, p->index, p->write ? "write" : "read", p->gen);
            why = buf;
            return false;
          }
        }
      }
    }
    return true;
  }
};

// Plans with the shortest buffer-reuse distance that passes the check.
bool plan_program(const fml_resident_stage *stages, int count, int ctas, Planner &pl) {
  std::string first_error;
  for (int lag = 4; lag <= std::max(8, 2 * count); lag *= 2) {
    pl = Planner{stages, count, ctas, lag};
    if (pl.run()) return true;
    if (pl.plan.error.find("reused too early") == std::string::npos) return false;  // nothing a longer distance would cure
    if (first_error.empty()) first_error = pl.plan.error;
  }
  return false;
}

void fill_info(const Plan &p, fml_resident_info *info) {
  memset(info, 0, sizeof(*info));
  info->ctas = p.ctas;
  info->stages = (int)(p.gemm.size() + p.attn.size());
  for (const auto &s : p.steps) info->steps += (int)s.size();
  info->buffers = (int)p.buffers.size();
  info->ring_slots = p.nslots;
  info->slot_bytes = p.slot_bytes;
  info->packed_weight_bytes = p.packed_bytes;
  info->scratch_bytes = p.buffer_bytes;
  info->shared_memory_bytes = kernel_smem_bytes(p.nslots, p.slot_bytes, p.overlay_bytes);
}

__global__ void pack_weights_kernel(const float *w, long long sk, long long sn, const PackDesc *descs, int count,
                                    uint8_t *packed) {
  for (int d = blockIdx.x; d < count; d += gridDim.x) {
    const PackDesc pd = descs[d];
    // element (n, k) of the tile -> K-major row n of 128 bytes, 16-byte units XOR-swizzled by (n & 7),
    // eight rows per 1024-byte group: the image a 128-byte-swizzle shared-memory descriptor expects
    for (int e = threadIdx.x; e < pd.tile_n * kBK; e += blockDim.x) {
      const int k = e / pd.tile_n, n = e - k * pd.tile_n;
      const float v = w[(long long)(pd.k0 + k) * sk + (long long)(pd.n0 + n) * sn];
      const size_t at = (size_t)(n >> 3) * 1024 + (size_t)(n & 7) * 128 + (size_t)((((k >> 2) ^ (n & 7)) & 7) << 4) + (size_t)(k & 3) * 4;
      *reinterpret_cast<float *>(packed + pd.dst + at) = v;
    }
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }



}  // namespace
}  // namespace res
}  // namespace fml

using namespace fml;
using namespace fml::res;

extern "C" int fml_resident_plan(const fml_resident_stage *stages, int32_t count, int32_t ctas,
                                 fml_resident_info *info) {
  FML_REQUIRE(stages && count > 0 && info, FML_BAD_ARG, "fml_resident_plan: bad argument");
  if (ctas <= 0) {
    int dev = 0;
    FML_CUDA(cudaGetDevice(&dev));
    FML_CUDA(cudaDeviceGetAttribute(&ctas, cudaDevAttrMultiProcessorCount, dev));
  }
  Planner pl{stages, count, ctas, 4};
  FML_REQUIRE(plan_program(stages, count, ctas, pl), FML_UNSUPPORTED, "fml_resident_plan: %s", pl.plan.error.c_str());
  fill_info(pl.plan, info);
  return FML_OK;
}

extern "C" int fml_resident_create(const fml_resident_stage *stages, int32_t count, fml_resident **out) {
  FML_REQUIRE(stages && count > 0 && out, FML_BAD_ARG, "fml_resident_create: bad argument");
  *out = nullptr;
  int dev = 0, ctas = 0;
  FML_CUDA(cudaGetDevice(&dev));
  FML_CUDA(cudaDeviceGetAttribute(&ctas, cudaDevAttrMultiProcessorCount, dev));
  Planner pl{stages, count, ctas, 4};
  FML_REQUIRE(plan_program(stages, count, ctas, pl), FML_UNSUPPORTED, "fml_resident_create: %s", pl.plan.error.c_str());
  Plan &p = pl.plan;
  int *status = device_status_word();
  FML_REQUIRE(status, FML_CUDA_ERROR, "fml_resident_create: no device status word");

  // ---- scratch layout
  size_t off = 0;
  auto take = [&](size_t bytes, size_t align) { off = align_up(off, align); const size_t at = off; off += bytes; return at; };
  size_t total_steps = 0;
  for (const auto &s : p.steps) total_steps += s.size() + 1;
  const size_t o_steps = take(total_steps * sizeof(Step), 256);
  const size_t o_begin = take((size_t)p.ctas * sizeof(int32_t), 256);
  const size_t o_gemm = take(std::max<size_t>(1, p.gemm.size()) * sizeof(GemmStage), 256);
  const size_t o_attn = take(std::max<size_t>(1, p.attn.size()) * sizeof(AttnStage), 256);
  const size_t o_wbegin = take((size_t)p.ctas * sizeof(unsigned long long), 256);
  const size_t o_words = take(256, 256);  // [0] pass number, [32] abort word
  const size_t o_buffers = take(p.buffer_bytes, 1024);
  const size_t trace_entries = (size_t)p.ctas * p.max_steps * kTraceSlots;
  const size_t o_trace = take(trace_entries * 8, 256);
  size_t pack_descs = 0;
  for (const auto &v : p.pack) pack_descs = std::max(pack_descs, v.size());
  const size_t o_pack = take(pack_descs * sizeof(PackDesc), 256);

  fml_resident *r = new fml_resident();
  r->device = dev;
  cudaError_t e = cudaMalloc(&r->scratch, off);
  if (e == cudaSuccess) e = cudaMalloc(&r->packed, p.packed_bytes);
  if (e != cudaSuccess) {
    if (r->scratch) cudaFree(r->scratch);
    delete r;
    set_error("fml_resident_create: cannot allocate %zu + %zu bytes", off, p.packed_bytes);
    cudaGetLastError();
    return FML_OUT_OF_MEMORY;
  }
  char *base = (char *)r->scratch;
  auto fail_free = [&](int st) { cudaFree(r->scratch); cudaFree(r->packed); delete r; return st; };
#define FML_TRY(call) do { cudaError_t e__ = (call); if (e__ != cudaSuccess) return fail_free(cuda_fail(e__, #call)); } while (0)
  FML_TRY(cudaMemset(r->scratch, 0, off));
  FML_TRY(cudaMemset(base + o_buffers, 0x01, p.buffer_bytes));  // every word's generation bit starts at 1
  FML_TRY(cudaMemset(r->packed, 0, p.packed_bytes));

  // ---- resolve buffer addresses
  auto buffer_ptr = [&](int b) -> float * { return (float *)(base + o_buffers + p.buffers[b].offset); };
  auto tiled_ptr = [&](int stage) -> float * { return p.outs[stage].buffer >= 0 ? buffer_ptr(p.outs[stage].buffer) : nullptr; };
  for (int i = 0; i < count; ++i) {
    if (p.stage_to_gemm[i] >= 0) {
      const int gi = p.stage_to_gemm[i];
      GemmStage &g = p.gemm[gi];
      const GemmOperands &ops = pl.gemm_operands[gi];
      if (ops.a.tiled) g.a = tiled_ptr(ops.a.producer) + (size_t)(ops.a.col0 / 4) * kRows * 4;
      if (ops.has_res && ops.res.tiled) g.res = tiled_ptr(ops.res.producer) + (size_t)(ops.res.col0 / 4) * kRows * 4;
      g.partial = buffer_ptr(ops.part_buffer);
      g.out_tiled = tiled_ptr(i);
    } else {
      const int ai = p.stage_to_attn[i];
      AttnStage &a = p.attn[ai];
      a.q = tiled_ptr(pl.attn_sources[ai].producer[0]);
      a.k = tiled_ptr(pl.attn_sources[ai].producer[1]);
      a.v = tiled_ptr(pl.attn_sources[ai].producer[2]);
      a.out_tiled = tiled_ptr(i);
    }
  }
  // ---- upload tables
  std::vector<Step> flat;
  std::vector<int32_t> begin(p.ctas);
  for (int c = 0; c < p.ctas; ++c) {
    begin[c] = (int32_t)flat.size();
    flat.insert(flat.end(), p.steps[c].begin(), p.steps[c].end());
    Step end{};
    end.kind = kEnd;
    flat.push_back(end);
  }
  FML_TRY(cudaMemcpy(base + o_steps, flat.data(), flat.size() * sizeof(Step), cudaMemcpyHostToDevice));
  FML_TRY(cudaMemcpy(base + o_begin, begin.data(), begin.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
  if (!p.gemm.empty()) FML_TRY(cudaMemcpy(base + o_gemm, p.gemm.data(), p.gemm.size() * sizeof(GemmStage), cudaMemcpyHostToDevice));
  if (!p.attn.empty()) FML_TRY(cudaMemcpy(base + o_attn, p.attn.data(), p.attn.size() * sizeof(AttnStage), cudaMemcpyHostToDevice));
  FML_TRY(cudaMemcpy(base + o_wbegin, p.weight_begin.data(), p.weight_begin.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
  // ---- pack the weights, one GEMM stage at a time
  for (int i = 0; i < count; ++i) {
    const int gi = p.stage_to_gemm[i];
    if (gi < 0 || p.pack[gi].empty()) continue;
    const fml_tensor &w = stages[i].w;
    FML_TRY(cudaMemcpy(base + o_pack, p.pack[gi].data(), p.pack[gi].size() * sizeof(PackDesc), cudaMemcpyHostToDevice));
    pack_weights_kernel<<<(unsigned)std::min<size_t>(p.pack[gi].size(), 4096), 256>>>(
        (const float *)w.data, (long long)w.stride[0], (long long)w.stride[1], (const PackDesc *)(base + o_pack),
        (int)p.pack[gi].size(), (uint8_t *)r->packed);
    FML_TRY(cudaGetLastError());
    FML_TRY(cudaDeviceSynchronize());  // the descriptor buffer is reused by the next stage
  }
#undef FML_TRY
  r->ctas = p.ctas;
  r->tagged_offset = o_buffers;
  r->tagged_bytes = p.buffer_bytes;
  r->trace_entries = trace_entries;
  r->smem_bytes = kernel_smem_bytes(p.nslots, p.slot_bytes, p.overlay_bytes);
  KernelArgs &a = r->args;
  a.steps = (const Step *)(base + o_steps);
  a.step_begin = (const int32_t *)(base + o_begin);
  a.gemm = (const GemmStage *)(base + o_gemm);
  a.attn = (const AttnStage *)(base + o_attn);
  a.weights = (const uint8_t *)r->packed;
  a.weight_begin = (const unsigned long long *)(base + o_wbegin);
  a.epoch = (unsigned *)(base + o_words);
  a.abort_word = a.epoch + 32;
  a.status = status;
  a.trace = (unsigned long long *)(base + o_trace);
  a.nslots = p.nslots; a.slot_bytes = p.slot_bytes; a.overlay_bytes = p.overlay_bytes; a.max_steps = p.max_steps;
  fill_info(p, &r->info);
  r->info.scratch_bytes = off;
  *out = r;
  return FML_OK;
}

extern "C" int fml_resident_launch(fml_resident *r, void *stream) {
  FML_REQUIRE(r, FML_BAD_ARG, "fml_resident_launch: null program");
  return launch_resident_kernel(r->args, r->ctas, r->smem_bytes, r->trace, as_stream(stream));
}

extern "C" int fml_resident_reset(fml_resident *r, void *stream) {
  FML_REQUIRE(r, FML_BAD_ARG, "fml_resident_reset: null program");
  cudaStream_t s = as_stream(stream);
  FML_CUDA(cudaMemsetAsync((char *)r->scratch + r->tagged_offset, 0x01, r->tagged_bytes, s));
  FML_CUDA(cudaMemsetAsync(r->args.epoch, 0, 256, s));  // pass number and abort word
  return FML_OK;
}

extern "C" int fml_resident_info_of(const fml_resident *r, fml_resident_info *info) {
  FML_REQUIRE(r && info, FML_BAD_ARG, "fml_resident_info_of: null argument");
  *info = r->info;
  return FML_OK;
}

extern "C" int fml_resident_destroy(fml_resident *r) {
  if (!r) return FML_OK;
  cudaFree(r->scratch);
  cudaFree(r->packed);
  delete r;
  return FML_OK;
}

extern "C" int fml_resident_set_trace(fml_resident *r, int32_t on) {
  FML_REQUIRE(r, FML_BAD_ARG, "fml_resident_set_trace: null program");
  r->trace = on != 0;
  return FML_OK;
}

extern "C" int fml_resident_read_trace(fml_resident *r, uint64_t *host, uint64_t capacity, int32_t *ctas,
                                       int32_t *max_steps) {
  FML_REQUIRE(r && host && ctas && max_steps, FML_BAD_ARG, "fml_resident_read_trace: null argument");
  FML_REQUIRE(capacity >= r->trace_entries, FML_BAD_ARG, "fml_resident_read_trace: the buffer needs %zu entries", r->trace_entries);
  FML_CUDA(cudaMemcpy(host, r->args.trace, r->trace_entries * 8, cudaMemcpyDeviceToHost));
  *ctas = r->ctas;
  *max_steps = r->args.max_steps;
  return FML_OK;
}
