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
// every slab).  An attention stage is cut into (head, 16 query rows) steps.  Steps name the
// counters they wait for and the counters they bump; a counter's target is always the number of
// steps that bump it, so "counter reached" means "all of them are done".
//
// Checking.  The plan is executed symbolically with a vector clock per step (how many steps of
// each CTA are known to be complete when it starts).  Every pair of accesses to overlapping
// memory, at least one of them a write, must be ordered by those clocks in stage order; the
// partial-tile buffers are shared between stages only as far as that holds.  A plan that fails
// the check is not created.
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
  size_t counter_bytes = 0;
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

struct OutInfo {
  const char *base = nullptr;  // out.data: bytes [base, base + 128 * N * 4) when internal
  int N = 0;
  bool external = false;
  size_t tiled_offset = 0;     // external: offset of the tiled shadow in scratch
  bool needs_shadow = false;   // external and read by a later stage
  int matrix = -1;             // access-tracking id of the tiled matrix
  int matrix_rm = -1;          // ... of the row-major copy
};

struct Access {
  int matrix;            // tracking id
  int r0, r1, c0, c1;    // rows, quads (or columns / 4) touched
  uintptr_t lo, hi;      // conservative byte range
  bool write;
  int cta, index;        // the step
  int order;             // stage order key: earlier must happen-before later
};

struct PackDesc {
  unsigned long long dst;
  int n0, k0, tile_n, pad;
};

struct Plan {
  int ctas = 0;
  std::vector<std::vector<Step>> steps;           // per CTA (without the end marker)
  std::vector<GemmStage> gemm;                    // pointers into scratch are OFFSETS until resolved
  std::vector<AttnStage> attn;
  std::vector<int> stage_to_gemm, stage_to_attn;  // stage index -> index in gemm / attn
  std::vector<std::vector<PackDesc>> pack;        // per GEMM stage
  std::vector<unsigned long long> weight_begin;   // per CTA
  size_t packed_bytes = 0;
  int counters = 0;
  std::vector<uint32_t> counter_total;
  std::vector<size_t> partial_offset;             // per partial slot
  std::vector<size_t> partial_bytes;
  std::vector<int> gemm_partial_slot;
  size_t shadow_bytes = 0;
  int slot_bytes = 0, nslots = 0, overlay_bytes = 0, max_steps = 0;
  std::vector<OutInfo> outs;
  std::vector<Access> accesses;
  std::string error;
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

struct Planner {
  const fml_resident_stage *stages;
  int count, ctas;
  Plan plan;
  // counters of each stage
  struct StageCounters {
    std::vector<int> unit_slab;  // per slab: units done (non-LN)
    int unit_all = -1;           // all units done (LN)
    std::vector<int> fin_slab;   // per slab: finish tiles done (non-LN)
    int fin_all = -1;            // all finish steps done
    int fin_all_total = 0;
    std::vector<int> head;       // attention: per head
    int head_all = -1, head_all_total = 0;
    int tile_n = 0, S = 0, rowblocks = 0;
    bool ln = false;
  };
  std::vector<StageCounters> sc;
  int next_matrix = 0;

  bool fail(const std::string &msg) { plan.error = msg; return false; }
  int new_counter() { plan.counter_total.push_back(0); return plan.counters++; }

  // operand lookup: which earlier stage's output contains this address
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
  // counters a reader of columns [c0, c1) of stage j's output has to wait for
  void deps_for(int j, int c0, int c1, std::vector<std::pair<int, uint32_t>> &w, bool coarse = false) const {
    const StageCounters &s = sc[j];
    if (stages[j].kind == FML_RESIDENT_GEMM) {
      if (!s.ln && !coarse) {
        const int n0 = c0 / s.tile_n, n1 = (c1 - 1) / s.tile_n;
        if (n1 - n0 + 1 <= 2) {
          for (int n = n0; n <= n1; ++n) w.push_back({s.fin_slab[n], (uint32_t)s.S});
          return;
        }
      }
      w.push_back({s.fin_all, (uint32_t)s.fin_all_total});
    } else {
      const fml_resident_stage &st = stages[j];
      const int dv = (int)st.v.shape[st.v.rank - 1];
      const int hs = plan.attn[plan.stage_to_attn[j]].o_hs, oc = plan.attn[plan.stage_to_attn[j]].o_col;
      // heads whose output columns [oc + h * hs, oc + h * hs + dv) meet [c0, c1)
      std::vector<int> hit;
      for (int h = 0; h < (int)s.head.size(); ++h)
        if (oc + h * hs < c1 && oc + h * hs + dv > c0) hit.push_back(h);
      if (hit.size() <= 2 && !coarse) for (int h : hit) w.push_back({s.head[h], (uint32_t)s.rowblocks});
      else w.push_back({s.head_all, (uint32_t)s.head_all_total});
    }
  }
  void set_waits(Step &st, std::vector<std::pair<int, uint32_t>> w) {
    std::sort(w.begin(), w.end());
    w.erase(std::unique(w.begin(), w.end()), w.end());
    st.nwait = 0;
    for (auto &p : w) {
      if (st.nwait == kMaxWait) break;  // cannot happen: callers keep the lists short
      st.wait_ctr[st.nwait] = p.first;
      st.wait_target[st.nwait] = p.second;
      ++st.nwait;
    }
  }
  void access(int matrix, int r0, int r1, int c0, int c1, uintptr_t lo, uintptr_t hi, bool write, int cta, int order) {
    plan.accesses.push_back({matrix, r0, r1, c0, c1, lo, hi, write, cta, (int)plan.steps[cta].size(), order});
  }
  // a tiled matrix at `base`: byte range of quads [c0, c1)
  void access_tiled(int matrix, const void *base, int r0, int r1, int c0, int c1, bool write, int cta, int order) {
    const uintptr_t b = (uintptr_t)base;
    access(matrix, r0, r1, c0, c1, b + (uintptr_t)c0 * kRows * 16, b + (uintptr_t)c1 * kRows * 16, write, cta, order);
  }
  void access_rm(int matrix, const void *base, int64_t ld, int r0, int r1, int c0, int c1, bool write, int cta, int order) {
    const uintptr_t b = (uintptr_t)base;
    access(matrix, r0, r1, c0, c1, b + (uintptr_t)r0 * ld * 4 + (uintptr_t)c0 * 16, b + (uintptr_t)(r1 - 1) * ld * 4 + (uintptr_t)c1 * 16, write, cta, order);
  }

  struct Operand {  // a [128 x cols] input
    bool tiled = false;
    int producer = -1, col0 = 0;
    const float *ptr = nullptr;  // row-major: element (0, 0); tiled: resolved later from the producer
    int64_t ld = 0;
    int matrix = -1;
  };
  std::map<const void *, int> external_ids;  // row-major inputs nobody in the program writes

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
      op.tiled = true; op.producer = j; op.col0 = (int)e; op.matrix = o.matrix;
      plan.outs[j].needs_shadow = plan.outs[j].external;
      return true;
    }
    if (((uintptr_t)t.data & 15) || (r.ld & 3)) return fail(std::string(what) + ": external operand is not 16-byte aligned");
    op.tiled = false; op.ptr = (const float *)t.data; op.ld = r.ld;
    auto it = external_ids.find(t.data);
    if (it == external_ids.end()) it = external_ids.insert({t.data, next_matrix++}).first;
    op.matrix = it->second;
    return true;
  }

  bool run() {
    plan.ctas = ctas;
    plan.steps.assign(ctas, {});
    plan.weight_begin.assign(ctas, 0);
    plan.stage_to_gemm.assign(count, -1);
    plan.stage_to_attn.assign(count, -1);
    sc.assign(count, {});
    if (count < 1) return fail("no stages");
    if (ctas < 1) return fail("no CTAs");
    std::vector<std::vector<uint32_t>> cta_bytes(ctas);  // chunk sizes per CTA in stream order
    std::vector<std::vector<std::pair<int, PackDesc>>> cta_chunks(ctas);
    int max_tile_n = 16;
    size_t attn_bytes = 0;

    for (int i = 0; i < count; ++i) {
      const fml_resident_stage &st = stages[i];
      OutInfo o;
      o.external = st.out_external != 0;
      o.base = (const char *)st.out.data;
      o.matrix = next_matrix++;
      o.matrix_rm = o.external ? next_matrix++ : -1;
      if (!st.out.data || ((uintptr_t)st.out.data & 15)) return fail("stage output is null or not 16-byte aligned");
      const int order_unit = 3 * i, order_fin = 3 * i + 1;

      if (st.kind == FML_RESIDENT_GEMM) {
        Rows ro;
        if (!as_rows(st.out, ro) || ro.rows != kRows) return fail("GEMM output must be a [128 x N] fp32 block");
        const int N = (int)ro.cols;
        if (st.w.rank != 2 || st.w.dtype != FML_F32 || !st.w.data || st.w.shape[1] != N) return fail("GEMM weights must be a [K, N] fp32 matrix");
        const int K = (int)st.w.shape[0];
        if (K < kBK || K % kBK || N % 16 || N > 4096 * 4) return fail("GEMM needs K a multiple of 32 and N a multiple of 16");
        if (!o.external && ro.ld != N) return fail("an internal GEMM output must be dense");
        if (o.external && (ro.ld & 3)) return fail("external GEMM output rows must be 16-byte multiples");
        if (st.layernorm && N > 4096) return fail("LayerNorm rows longer than 4096");
        if (st.act < FML_ACT_NONE || st.act > FML_ACT_SIGMOID) return fail("unsupported activation");
        o.N = N;
        plan.outs.push_back(o);
        Operand a, res;
        if (!operand(st.a, i, K, a, "GEMM input")) return false;
        const bool has_res = st.residual.data != nullptr;
        if (has_res && !operand(st.residual, i, N, res, "GEMM residual")) return false;
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

        StageCounters &c = sc[i];
        c.tile_n = tc.tile_n; c.S = S; c.ln = st.layernorm != 0;
        if (c.ln) c.unit_all = new_counter();
        else { c.unit_slab.resize(slabs); for (int &x : c.unit_slab) x = new_counter(); }
        if (!c.ln) { c.fin_slab.resize(slabs); for (int &x : c.fin_slab) x = new_counter(); }
        c.fin_all = new_counter();

        GemmStage g{};
        g.N = N; g.K = K; g.S = S; g.tile_n = tc.tile_n;
        g.a_tiled = a.tiled; g.a_ld = a.ld;
        g.a = a.tiled ? (const float *)(uintptr_t)a.col0 : a.ptr;  // tiled: resolved in resolve()
        g.bias = (const float *)st.bias.data;
        g.res_tiled = has_res && res.tiled; g.res_ld = res.ld;
        g.res = has_res ? (res.tiled ? (const float *)(uintptr_t)res.col0 : res.ptr) : nullptr;
        g.act = st.act; g.c0 = st.act_param[0]; g.c1 = st.act_param[1]; g.c2 = st.act_param[2];
        g.ln = c.ln; g.gamma = (const float *)st.ln_scale.data; g.beta = (const float *)st.ln_bias.data; g.eps = st.ln_eps;
        g.out_rm = o.external ? (float *)st.out.data : nullptr;
        g.out_ld = ro.ld;
        plan.gemm.push_back(g);
        plan.stage_to_gemm[i] = gi;
        gemm_operands.push_back({a, res, has_res});
        plan.pack.push_back({});
        plan.gemm_partial_slot.push_back(-1);  // assigned by assign_partials()

        // ---- units
        const int partial_matrix = next_matrix++;
        partial_matrix_of.push_back(partial_matrix);
        for (int n = 0; n < slabs; ++n)
          for (int s = 0; s < S; ++s) {
            const int cta = (n * S + s) % ctas;
            const int kb0 = (int)((long long)s * nkb_total / S), kb1 = (int)((long long)(s + 1) * nkb_total / S);
            Step u{};
            u.kind = kUnit; u.stage = gi; u.p0 = n; u.p1 = s; u.p2 = kb0; u.p3 = kb1 - kb0;
            u.sig[0] = c.ln ? c.unit_all : c.unit_slab[n];
            u.sig[1] = -1;
            ++plan.counter_total[u.sig[0]];
            std::vector<std::pair<int, uint32_t>> w;
            if (a.tiled) deps_for(a.producer, a.col0 + kb0 * kBK, a.col0 + kb1 * kBK, w);
            set_waits(u, w);
            // reads A columns [kb0*32, kb1*32), writes its partial tile
            if (a.tiled) access_tiled(a.matrix, tiled_base_key(a.producer), 0, kRows, (a.col0 + kb0 * kBK) / 4, (a.col0 + kb1 * kBK) / 4, false, cta, order_unit);
            else access_rm(a.matrix, a.ptr, a.ld, 0, kRows, kb0 * 8, kb1 * 8, false, cta, order_unit);
            pending_partial.push_back({(int)plan.accesses.size(), gi});
            access(partial_matrix, 0, kRows, s * NC + n * tc.tile_n / 4, s * NC + (n + 1) * tc.tile_n / 4, 0, 0, true, cta, order_unit);
            plan.steps[cta].push_back(u);
            for (int kb = kb0; kb < kb1; ++kb) {
              cta_chunks[cta].push_back({gi, PackDesc{0, n * tc.tile_n, kb * kBK, tc.tile_n, 0}});
              cta_bytes[cta].push_back((uint32_t)tc.tile_n * 128u);
            }
          }
        // ---- finish steps
        auto finish = [&](int cta, int r0, int r1, int q0, int q1, int n) {
          Step f{};
          f.kind = kFinish; f.stage = gi; f.p0 = r0; f.p1 = r1; f.p2 = q0; f.p3 = q1;
          f.sig[0] = c.fin_all; f.sig[1] = c.ln ? -1 : c.fin_slab[n];
          ++plan.counter_total[c.fin_all];
          if (f.sig[1] >= 0) ++plan.counter_total[f.sig[1]];
          std::vector<std::pair<int, uint32_t>> w;
          if (c.ln) w.push_back({c.unit_all, (uint32_t)(slabs * S)});
          else w.push_back({c.unit_slab[n], (uint32_t)S});
          if (has_res && res.tiled) {
            std::vector<std::pair<int, uint32_t>> wr;
            deps_for(res.producer, res.col0 + q0 * 4, res.col0 + q1 * 4, wr);
            for (auto &p : wr) w.push_back(p);
          }
          set_waits(f, w);
          for (int s = 0; s < S; ++s) {
            pending_partial.push_back({(int)plan.accesses.size(), gi});
            access(partial_matrix, r0, r1, s * NC + q0, s * NC + q1, 0, 0, false, cta, order_fin);
          }
          if (has_res) {
            if (res.tiled) access_tiled(res.matrix, tiled_base_key(res.producer), r0, r1, res.col0 / 4 + q0, res.col0 / 4 + q1, false, cta, order_fin);
            else access_rm(res.matrix, res.ptr, res.ld, r0, r1, q0, q1, false, cta, order_fin);
          }
          pending_out.push_back({(int)plan.accesses.size(), i});
          access(o.matrix, r0, r1, q0, q1, 0, 0, true, cta, order_fin);
          if (o.external) access_rm(o.matrix_rm, st.out.data, ro.ld, r0, r1, q0, q1, true, cta, order_fin);
          plan.steps[cta].push_back(f);
        };
        if (c.ln) {
          const int owners = std::min(ctas, kRows);
          for (int k = 0; k < owners; ++k) {
            const int r0 = k * kRows / owners, r1 = (k + 1) * kRows / owners;
            finish(k, r0, r1, 0, NC, -1);
          }
          c.fin_all_total = owners;
        } else {
          for (int n = 0; n < slabs; ++n)
            for (int s = 0; s < S; ++s) {
              const int r0 = s * kRows / S, r1 = (s + 1) * kRows / S;
              finish((n * S + s) % ctas, r0, r1, n * tc.tile_n / 4, (n + 1) * tc.tile_n / 4, n);
            }
          c.fin_all_total = slabs * S;
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
        plan.outs.push_back(o);
        AttnStage A{};
        A.heads = H; A.D = D; A.Dv = Dv; A.Sk = Sk; A.divisor = st.divisor;
        A.o_col = 0; A.o_hs = (int)o_hs; A.out_ld = o_ld;
        A.out_rm = o.external ? (float *)out.data : nullptr;
        // q / k / v: column ranges of earlier stages' tiled outputs
        struct Src { int producer, col0, hs, matrix; } src[3];
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
          src[k] = {j, (int)e, (int)hs, p.matrix};
          plan.outs[j].needs_shadow = plan.outs[j].external;
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
        attn_sources.push_back({src[0].producer, src[1].producer, src[2].producer});
        StageCounters &c = sc[i];
        c.rowblocks = kRows / kAttnRows;
        c.head.resize(H);
        for (int &x : c.head) x = new_counter();
        c.head_all = new_counter();
        c.head_all_total = H * c.rowblocks;
        for (int h = 0; h < H; ++h)
          for (int rb = 0; rb < c.rowblocks; ++rb) {
            const int cta = (h * c.rowblocks + rb) % ctas;
            Step a{};
            a.kind = kAttention; a.stage = ai; a.p0 = h; a.p1 = rb * kAttnRows;
            a.sig[0] = c.head[h]; a.sig[1] = c.head_all;
            ++plan.counter_total[a.sig[0]];
            ++plan.counter_total[a.sig[1]];
            std::vector<std::pair<int, uint32_t>> w;
            const int widths[3] = {D, D, Dv};
            for (int pass = 0; pass < 2; ++pass) {  // per-slab counters first, whole-stage counters if those are too many
              w.clear();
              for (int k = 0; k < 3; ++k)
                deps_for(src[k].producer, src[k].col0 + h * src[k].hs, src[k].col0 + h * src[k].hs + widths[k], w, pass == 1);
              std::sort(w.begin(), w.end());
              w.erase(std::unique(w.begin(), w.end()), w.end());
              if (w.size() <= (size_t)kMaxWait) break;
            }
            if (w.size() > (size_t)kMaxWait) return fail("attention step depends on too many counters");
            set_waits(a, w);
            for (int k = 0; k < 3; ++k) {
              const int c0 = (src[k].col0 + h * src[k].hs) / 4, c1 = c0 + widths[k] / 4;
              const int r0 = k == 0 ? rb * kAttnRows : 0, r1 = k == 0 ? r0 + kAttnRows : kRows;
              access_tiled(src[k].matrix, tiled_base_key(src[k].producer), r0, r1, c0, c1, false, cta, order_unit);
            }
            pending_out.push_back({(int)plan.accesses.size(), i});
            access(o.matrix, rb * kAttnRows, (rb + 1) * kAttnRows, (int)(h * o_hs / 4), (int)((h * o_hs + Dv) / 4), 0, 0, true, cta, order_unit);
            if (o.external) access_rm(o.matrix_rm, out.data, o_ld, rb * kAttnRows, (rb + 1) * kAttnRows, (int)(h * o_hs / 4), (int)((h * o_hs + Dv) / 4), true, cta, order_unit);
            plan.steps[cta].push_back(a);
          }
      } else {
        return fail("unknown stage kind");
      }
    }

    // ---- shared memory: ring slots sized for the widest tile, overlay for lo(B) / attention
    plan.slot_bytes = max_tile_n * 128;
    size_t overlay = std::max((size_t)kConvDepth * plan.slot_bytes, attn_bytes);
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

    // ---- tiled shadows of external outputs that later stages read
    for (int i = 0; i < count; ++i)
      if (plan.outs[i].external && plan.outs[i].needs_shadow) {
        plan.outs[i].tiled_offset = plan.shadow_bytes;
        plan.shadow_bytes += (size_t)kRows * plan.outs[i].N * 4;
      }
    return assign_partials();
  }

  // bookkeeping for addresses that are only known once scratch is laid out
  struct GemmOperands { Operand a, res; bool has_res; };
  std::vector<GemmOperands> gemm_operands;
  std::vector<std::vector<int>> attn_sources;
  std::vector<int> partial_matrix_of;
  std::vector<std::pair<int, int>> pending_partial;  // (access index, gemm index)
  std::vector<std::pair<int, int>> pending_out;      // (access index, stage index)

  // Address key of stage j's tiled output for the alias check: its own bytes when internal, a
  // private range (never aliasing anything else) when it is a shadow in scratch.
  const void *tiled_base_key(int j) const {
    const OutInfo &o = plan.outs[j];
    return o.external ? (const void *)((uintptr_t)1 << 60 | ((uintptr_t)j << 40)) : (const void *)o.base;
  }

  // Partial-tile buffers: stages share `period` buffers round robin; the smallest period whose
  // plan passes the ordering check is taken.
  bool assign_partials() {
    const int ng = (int)plan.gemm.size();
    std::vector<int> periods;
    for (int x = 2; x < ng; x *= 2) periods.push_back(x);
    periods.push_back(std::max(ng, 1));
    for (int period : periods) {
      plan.partial_bytes.assign(std::max(period, 1), 0);
      for (int g = 0; g < ng; ++g) {
        plan.gemm_partial_slot[g] = g % period;
        plan.partial_bytes[g % period] = std::max(plan.partial_bytes[g % period], (size_t)plan.gemm[g].S * plan.gemm[g].N * kRows * 4);
      }
      // address keys for the check: partial slot p lives in its own private range
      for (auto &pa : pending_partial) {
        Access &a = plan.accesses[pa.first];
        const uintptr_t base = ((uintptr_t)2 << 60) | ((uintptr_t)plan.gemm_partial_slot[pa.second] << 40);
        a.lo = base + (uintptr_t)a.c0 * kRows * 16;
        a.hi = base + (uintptr_t)a.c1 * kRows * 16;
      }
      for (auto &po : pending_out) {
        Access &a = plan.accesses[po.first];
        const uintptr_t base = (uintptr_t)tiled_base_key(po.second);
        a.lo = base + (uintptr_t)a.c0 * kRows * 16;
        a.hi = base + (uintptr_t)a.c1 * kRows * 16;
      }
      std::string why;
      if (check(why)) return true;
      if (ng == 0 || period >= ng) return fail("plan check failed: " + why);
    }
    return fail("plan check failed");
  }

  // Symbolic execution with vector clocks, then the pairwise ordering check.
  bool check(std::string &why) const {
    const int C = ctas;
    std::vector<size_t> pc(C, 0);
    std::vector<uint32_t> value(plan.counters, 0);
    std::vector<std::vector<int>> closure(plan.counters, std::vector<int>(C, 0));  // clock implied by "counter complete"
    std::vector<std::vector<std::vector<int>>> clock(C);  // clock[cta][step] at step start
    for (int c = 0; c < C; ++c) clock[c].resize(plan.steps[c].size());
    std::vector<std::vector<int>> last(C, std::vector<int>(C, 0));  // running clock of each CTA
    for (int c = 0; c < plan.counters; ++c)
      if (plan.counter_total[c] == 0) { why = "a counter nobody bumps"; return false; }
    bool progress = true;
    size_t done = 0, total = 0;
    for (int c = 0; c < C; ++c) total += plan.steps[c].size();
    while (progress) {
      progress = false;
      for (int c = 0; c < C; ++c) {
        while (pc[c] < plan.steps[c].size()) {
          const Step &st = plan.steps[c][pc[c]];
          bool ready = true;
          for (int w = 0; w < st.nwait; ++w) {
            if (st.wait_target[w] != plan.counter_total[st.wait_ctr[w]]) { why = "a wait target differs from the counter's total"; return false; }
            if (value[st.wait_ctr[w]] < st.wait_target[w]) ready = false;
          }
          if (!ready) break;
          std::vector<int> &k = last[c];
          for (int w = 0; w < st.nwait; ++w)
            for (int x = 0; x < C; ++x) k[x] = std::max(k[x], closure[st.wait_ctr[w]][x]);
          clock[c][pc[c]] = k;
          k[c] = (int)pc[c] + 1;  // at its end the step itself is complete
          for (int sgi = 0; sgi < 2; ++sgi)
            if (st.sig[sgi] >= 0) {
              ++value[st.sig[sgi]];
              for (int x = 0; x < C; ++x) closure[st.sig[sgi]][x] = std::max(closure[st.sig[sgi]][x], k[x]);
            }
          ++pc[c];
          ++done;
          progress = true;
        }
      }
    }
    if (done != total) { why = "the step lists deadlock"; return false; }
    // pairwise: group by matrix; different matrices only where byte ranges overlap
    std::vector<const Access *> acc;
    for (const Access &a : plan.accesses) acc.push_back(&a);
    std::sort(acc.begin(), acc.end(), [](const Access *x, const Access *y) { return x->lo < y->lo; });
    auto before = [&](const Access &x, const Access &y) {  // x's step complete when y's starts
      if (x.cta == y.cta) return x.index < y.index;
      return clock[y.cta][y.index][x.cta] > x.index;
    };
    for (size_t i = 0; i < acc.size(); ++i) {
      const Access &x = *acc[i];
      for (size_t j = i + 1; j < acc.size() && acc[j]->lo < x.hi; ++j) {
        const Access &y = *acc[j];
        if (!x.write && !y.write) continue;
        if (x.cta == y.cta && x.index == y.index) continue;
        if (x.matrix == y.matrix) {
          if (x.r1 <= y.r0 || y.r1 <= x.r0 || x.c1 <= y.c0 || y.c1 <= x.c0) continue;
        }
        const Access &first = (x.order < y.order || (x.order == y.order && !y.write)) ? x : y;
        const Access &second = &first == &x ? y : x;
        if (first.order == second.order && x.matrix == y.matrix && x.write && y.write) { why = "two steps of one stage write the same element"; return false; }
        if (!before(first, second)) {
          char buf[200];
          snprintf(buf, sizeof(buf), "unordered accesses: cta %d step %d (%s, order %d) and cta %d step %d (%s, order %d), matrices %d / %d",
                   first.cta, first.index, first.write ? "write" : "read", first.order, second.cta, second.index,
                   second.write ? "write" : "read", second.order, first.matrix, second.matrix);
          why = buf;
          return false;
        }
      }
    }
    return true;
  }
};

void fill_info(const Plan &p, fml_resident_info *info) {
  memset(info, 0, sizeof(*info));
  info->ctas = p.ctas;
  info->stages = (int)(p.gemm.size() + p.attn.size());
  for (const auto &s : p.steps) info->steps += (int)s.size();
  info->counters = p.counters;
  info->ring_slots = p.nslots;
  info->slot_bytes = p.slot_bytes;
  info->packed_weight_bytes = p.packed_bytes;
  size_t scratch = p.shadow_bytes;
  for (size_t b : p.partial_bytes) scratch += b;
  info->scratch_bytes = scratch;
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
  Planner pl{stages, count, ctas};
  FML_REQUIRE(pl.run(), FML_UNSUPPORTED, "fml_resident_plan: %s", pl.plan.error.c_str());
  fill_info(pl.plan, info);
  return FML_OK;
}

extern "C" int fml_resident_create(const fml_resident_stage *stages, int32_t count, fml_resident **out) {
  FML_REQUIRE(stages && count > 0 && out, FML_BAD_ARG, "fml_resident_create: bad argument");
  *out = nullptr;
  int dev = 0, ctas = 0;
  FML_CUDA(cudaGetDevice(&dev));
  FML_CUDA(cudaDeviceGetAttribute(&ctas, cudaDevAttrMultiProcessorCount, dev));
  Planner pl{stages, count, ctas};
  FML_REQUIRE(pl.run(), FML_UNSUPPORTED, "fml_resident_create: %s", pl.plan.error.c_str());
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
  const size_t counter_bytes = align_up((size_t)(p.counters + 1) * 4, 256);  // + the abort word
  const size_t o_counters = take(counter_bytes, 256);
  std::vector<size_t> o_partial(p.partial_bytes.size());
  for (size_t i = 0; i < p.partial_bytes.size(); ++i) o_partial[i] = take(p.partial_bytes[i], 1024);
  const size_t o_shadow = take(p.shadow_bytes, 1024);
  const size_t trace_entries = (size_t)p.ctas * p.max_steps * 2;
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
  FML_TRY(cudaMemset(r->packed, 0, p.packed_bytes));

  // ---- resolve addresses
  auto tiled_ptr = [&](int stage) -> float * {
    const OutInfo &o = p.outs[stage];
    return o.external ? (o.needs_shadow ? (float *)(base + o_shadow + o.tiled_offset) : nullptr) : (float *)o.base;
  };
  for (int i = 0; i < count; ++i) {
    if (p.stage_to_gemm[i] >= 0) {
      const int gi = p.stage_to_gemm[i];
      GemmStage &g = p.gemm[gi];
      const auto &ops = pl.gemm_operands[gi];
      if (ops.a.tiled) g.a = tiled_ptr(ops.a.producer) + (size_t)(ops.a.col0 / 4) * kRows * 4;
      if (ops.has_res && ops.res.tiled) g.res = tiled_ptr(ops.res.producer) + (size_t)(ops.res.col0 / 4) * kRows * 4;
      g.partial = (float *)(base + o_partial[p.gemm_partial_slot[gi]]);
      g.out_tiled = tiled_ptr(i);
    } else {
      const int ai = p.stage_to_attn[i];
      AttnStage &a = p.attn[ai];
      a.q = tiled_ptr(pl.attn_sources[ai][0]);
      a.k = tiled_ptr(pl.attn_sources[ai][1]);
      a.v = tiled_ptr(pl.attn_sources[ai][2]);
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
  r->counter_bytes = counter_bytes;
  r->trace_entries = trace_entries;
  r->smem_bytes = kernel_smem_bytes(p.nslots, p.slot_bytes, p.overlay_bytes);
  KernelArgs &a = r->args;
  a.steps = (const Step *)(base + o_steps);
  a.step_begin = (const int32_t *)(base + o_begin);
  a.gemm = (const GemmStage *)(base + o_gemm);
  a.attn = (const AttnStage *)(base + o_attn);
  a.weights = (const uint8_t *)r->packed;
  a.weight_begin = (const unsigned long long *)(base + o_wbegin);
  a.counters = (unsigned *)(base + o_counters);
  a.abort_word = a.counters + p.counters;
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
  cudaStream_t s = as_stream(stream);
  FML_CUDA(cudaMemsetAsync(r->args.counters, 0, r->counter_bytes, s));
  return launch_resident_kernel(r->args, r->ctas, r->smem_bytes, r->trace, s);
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
