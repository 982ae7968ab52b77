// GEMM front end: shape analysis, the fp32 FMA kernel for operands the tensor-core path
// cannot take (arbitrary strides, tiny or unaligned shapes), and the C-ABI entry points.
#include "gemm_common.cuh"
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace fml {

int analyse_gemm(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                 const fml_tensor *bias, const fml_tensor *res, GemmProblem &p) {
  FML_REQUIRE(valid_tensor(a) && valid_tensor(b) && valid_tensor(c), FML_BAD_ARG, "fml_gemm: bad tensor");
  FML_REQUIRE(a->dtype == FML_F32 && b->dtype == FML_F32 && c->dtype == FML_F32, FML_UNSUPPORTED,
              "fml_gemm: fp32 only");
  FML_REQUIRE(a->rank >= 2 && b->rank >= 2 && c->rank >= 2 && a->rank <= c->rank && b->rank <= c->rank,
              FML_BAD_ARG, "fml_gemm: operand ranks");
  const int r = c->rank;
  p.prefetch = nullptr;
  p.prefetch_bytes = 0;
  p.b_constant = 0;
  p.M = c->shape[r - 2];
  p.N = c->shape[r - 1];
  p.K = a->shape[a->rank - 1];
  FML_REQUIRE(a->shape[a->rank - 2] == p.M && b->shape[b->rank - 2] == p.K && b->shape[b->rank - 1] == p.N,
              FML_BAD_ARG, "fml_gemm: inner dimensions do not match");
  p.a = (const float *)a->data; p.b = (const float *)b->data; p.c = (float *)c->data;
  p.bias = bias ? (const float *)bias->data : nullptr;
  p.res = res ? (const float *)res->data : nullptr;
  p.a_sm = a->stride[a->rank - 2]; p.a_sk = a->stride[a->rank - 1];
  p.b_sk = b->stride[b->rank - 2]; p.b_sn = b->stride[b->rank - 1];
  p.c_sm = c->stride[r - 2]; p.c_sn = c->stride[r - 1];
  int64_t bias_s[kMaxDims] = {0}, res_s[kMaxDims] = {0};
  if (bias) {
    FML_REQUIRE(valid_tensor(bias) && bias->dtype == FML_F32 && broadcast_strides(bias, c, bias_s),
                FML_BAD_ARG, "fml_gemm: bias does not broadcast to the output");
  }
  if (res) {
    FML_REQUIRE(valid_tensor(res) && res->dtype == FML_F32 && broadcast_strides(res, c, res_s),
                FML_BAD_ARG, "fml_gemm: residual does not broadcast to the output");
  }
  p.bias_sm = bias_s[r - 2]; p.bias_sn = bias_s[r - 1];
  p.res_sm = res_s[r - 2]; p.res_sn = res_s[r - 1];

  // batch dims, outermost first; operand 0..4 = c, a, b, bias, res
  Iter<5> it;
  it.rank = r - 2;
  for (int i = 0; i < r - 2; ++i) {
    it.shape[i] = c->shape[i];
    it.stride[0][i] = c->stride[i];
    const int ia = i - (r - a->rank), ib = i - (r - b->rank);
    if (ia >= 0) FML_REQUIRE(a->shape[ia] == c->shape[i] || a->shape[ia] == 1, FML_BAD_ARG, "fml_gemm: batch dims of A");
    if (ib >= 0) FML_REQUIRE(b->shape[ib] == c->shape[i] || b->shape[ib] == 1, FML_BAD_ARG, "fml_gemm: batch dims of B");
    it.stride[1][i] = (ia >= 0 && a->shape[ia] != 1) ? a->stride[ia] : 0;
    it.stride[2][i] = (ib >= 0 && b->shape[ib] != 1) ? b->stride[ib] : 0;
    it.stride[3][i] = bias_s[i];
    it.stride[4][i] = res_s[i];
  }
  if (it.rank == 0) { it.rank = 1; it.shape[0] = 1; for (int o = 0; o < 5; ++o) it.stride[o][0] = 0; }
  collapse(it);
  // fold the innermost batch dim into M when B does not vary over it and rows continue
  while (it.rank >= 1 && it.shape[it.rank - 1] > 1) {
    const int l = it.rank - 1;
    const bool ok = it.stride[2][l] == 0 && it.stride[0][l] == p.M * p.c_sm &&
                    it.stride[1][l] == p.M * p.a_sm &&
                    (!bias || it.stride[3][l] == p.M * p.bias_sm) &&
                    (!res || it.stride[4][l] == p.M * p.res_sm);
    if (!ok) break;
    p.M *= it.shape[l];
    if (it.rank == 1) { it.shape[0] = 1; for (int o = 0; o < 5; ++o) it.stride[o][0] = 0; }
    else --it.rank;
  }
  FML_REQUIRE(it.rank <= 2, FML_UNSUPPORTED, "fml_gemm: more than two independent batch dims");
  const int l = it.rank - 1;
  p.nb0 = it.shape[l];
  p.c_b0 = it.stride[0][l]; p.a_b0 = it.stride[1][l]; p.b_b0 = it.stride[2][l];
  p.bias_b0 = it.stride[3][l]; p.res_b0 = it.stride[4][l];
  if (it.rank == 2) {
    p.nb1 = it.shape[0];
    p.c_b1 = it.stride[0][0]; p.a_b1 = it.stride[1][0]; p.b_b1 = it.stride[2][0];
    p.bias_b1 = it.stride[3][0]; p.res_b1 = it.stride[4][0];
  } else {
    p.nb1 = 1;
    p.c_b1 = p.a_b1 = p.b_b1 = p.bias_b1 = p.res_b1 = 0;
  }
  return FML_OK;
}

namespace {

// 64x64 output tile, 16-deep k slab, 256 threads with a 4x4 micro-tile each.  Operands are
// read with their element strides, so any layout works; the k-fast / m-fast thread mapping
// of the loads follows whichever stride is 1.
constexpr int SB = 64, SK = 16;

__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmProblem p, GemmEpilogue e) {
  pdl_prologue();
  __shared__ float As[SK][SB + 4];
  __shared__ float Bs[SK][SB + 4];
  const int64_t z = blockIdx.z, z0 = z % p.nb0, z1 = z / p.nb0;
  const float *A = p.a + z0 * p.a_b0 + z1 * p.a_b1;
  const float *B = p.b + z0 * p.b_b0 + z1 * p.b_b1;
  const int64_t m0 = (int64_t)blockIdx.y * SB, n0 = (int64_t)blockIdx.x * SB;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  float acc[4][4] = {};
  const bool a_kfast = p.a_sk == 1, b_nfast = p.b_sn == 1;
  for (int64_t k0 = 0; k0 < p.K; k0 += SK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e_ = t + i * 256;
      int mm, kk;
      if (a_kfast) { kk = e_ & 15; mm = e_ >> 4; } else { mm = e_ & 63; kk = e_ >> 6; }
      const int64_t gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < p.M && gk < p.K) ? A[gm * p.a_sm + gk * p.a_sk] : 0.0f;
      int nn, kb;
      if (b_nfast) { nn = e_ & 63; kb = e_ >> 6; } else { kb = e_ & 15; nn = e_ >> 4; }
      const int64_t gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < p.N && gkb < p.K) ? B[gkb * p.b_sk + gn * p.b_sn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  float *C = p.c + z0 * p.c_b0 + z1 * p.c_b1;
  const float *bias = p.bias ? p.bias + z0 * p.bias_b0 + z1 * p.bias_b1 : nullptr;
  const float *res = p.res ? p.res + z0 * p.res_b0 + z1 * p.res_b1 : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < p.M && n < p.N) {
        const float bv = bias ? bias[m * p.bias_sm + n * p.bias_sn] : 0.0f;
        const float rv = res ? res[m * p.res_sm + n * p.res_sn] : 0.0f;
        C[m * p.c_sm + n * p.c_sn] = gemm_epilogue(e, acc[i][j], bv, rv);
      }
    }
}

}  // namespace

int launch_gemm_simt(const GemmProblem &p, const GemmEpilogue &e, cudaStream_t s) {
  const int64_t batch = p.nb0 * p.nb1;
  FML_REQUIRE(batch <= 65535 && (p.M + SB - 1) / SB <= 65535, FML_UNSUPPORTED,
              "fml_gemm: batch or M too large for the fp32 kernel grid");
  dim3 grid((unsigned)((p.N + SB - 1) / SB), (unsigned)((p.M + SB - 1) / SB), (unsigned)batch);
  FML_LAUNCH((gemm_simt_kernel), grid, 256, 0, s, p, e);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

static GemmEpilogue make_epilogue(const fml_gemm_params &gp, bool has_bias, bool has_res) {
  GemmEpilogue e;
  e.divisor = gp.divisor == 0.0f ? 1.0f : gp.divisor;
  e.alpha = gp.alpha; e.beta = gp.beta; e.act = gp.act;
  e.c0 = gp.act_param[0]; e.c1 = gp.act_param[1]; e.c2 = gp.act_param[2];
  e.has_bias = has_bias; e.has_res = has_res;
  return e;
}

}  // namespace fml

using namespace fml;

extern "C" void fml_gemm_default_params(fml_gemm_params *p) {
  if (!p) return;
  memset(p, 0, sizeof(*p));
  p->precision = FML_GEMM_AUTO;
  p->act = FML_ACT_NONE;
  p->divisor = 1.0f;
  p->alpha = 1.0f;
  p->beta = 1.0f;
  p->act_param[0] = 1.4142135381698608f;  // sqrt(2) in fp32
  p->act_param[1] = 1.0f;
  p->act_param[2] = 0.5f;
}

static int resolve(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                   const fml_tensor *bias, const fml_tensor *res, const fml_gemm_params *gp,
                   GemmProblem &p, TcPlan &plan, bool &use_tc) {
  FML_REQUIRE(gp, FML_BAD_ARG, "fml_gemm: null params");
  int st = analyse_gemm(a, b, c, bias, res, p);
  if (st != FML_OK) return st;
  use_tc = gp->precision != FML_GEMM_FP32 && plan_gemm_tc(p, *gp, plan);
  FML_REQUIRE(use_tc || gp->precision == FML_GEMM_AUTO || gp->precision == FML_GEMM_FP32,
              FML_MISALIGNED,
              "fml_gemm: a tensor-core precision was requested but the operands cannot be fed to "
              "TMA (need a unit-stride k or n dim, 16-byte aligned bases and row strides)");
  return FML_OK;
}

extern "C" int fml_gemm_plan(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                             const fml_gemm_params *gp, fml_gemm_plan_info *info) {
  FML_REQUIRE(info, FML_BAD_ARG, "fml_gemm_plan: null argument");
  GemmProblem p;
  TcPlan plan;
  bool use_tc = false;
  int st = resolve(a, b, c, nullptr, nullptr, gp, p, plan, use_tc);
  if (st != FML_OK) return st;
  memset(info, 0, sizeof(*info));
  info->uses_tensor_cores = use_tc ? 1 : 0;
  if (use_tc) {
    info->tile_n = plan.tile_n; info->split_k = plan.split_k; info->stages = plan.stages;
    info->b_mn_major = plan.b_mn_major; info->three_pass = plan.three_pass;
    info->shared_memory_bytes = plan.smem_bytes;
  }
  return FML_OK;
}

extern "C" int fml_gemm_uses_tensor_cores(const fml_tensor *a, const fml_tensor *b,
                                          const fml_tensor *c, const fml_gemm_params *gp, int *uses) {
  FML_REQUIRE(uses, FML_BAD_ARG, "fml_gemm_uses_tensor_cores: null argument");
  GemmProblem p;
  TcPlan plan;
  bool use_tc = false;
  int st = resolve(a, b, c, nullptr, nullptr, gp, p, plan, use_tc);
  if (st != FML_OK) return st;
  *uses = use_tc ? 1 : 0;
  return FML_OK;
}

extern "C" int fml_gemm(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                        const fml_tensor *bias, const fml_tensor *residual,
                        const fml_gemm_params *gp, void *stream) {
  GemmProblem p;
  TcPlan plan;
  bool use_tc = false;
  int st = resolve(a, b, c, bias, residual, gp, p, plan, use_tc);
  if (st != FML_OK) return st;
  if (p.M == 0 || p.N == 0 || p.nb0 * p.nb1 == 0) return FML_OK;
  GemmEpilogue e = make_epilogue(*gp, bias != nullptr, residual != nullptr);
  p.b_constant = gp->b_constant ? 1 : 0;
  if (gp->l2_prefetch && gp->l2_prefetch_bytes) {
    FML_REQUIRE((reinterpret_cast<uintptr_t>(gp->l2_prefetch) & 15) == 0, FML_MISALIGNED,
                "fml_gemm: the L2 prefetch hint must be 16-byte aligned");
    p.prefetch = static_cast<const char *>(gp->l2_prefetch);
    p.prefetch_bytes = gp->l2_prefetch_bytes;
  }
  if (use_tc) return launch_gemm_tc(p, e, plan, as_stream(stream));
  if (skinny_eligible(p)) return launch_gemm_skinny(p, e, as_stream(stream));
  return launch_gemm_simt(p, e, as_stream(stream));
}

// One-off on-device tuning of (tile_n, split_k) for one GEMM, cached per problem signature.
// The reference tunes its MatMul / Gemm kernels the same way -- by running the candidates
// (there: six loop orders on the CPU, src/structure/kernel/generator/matmul.cpp:100-123) and
// keeping the fastest per layout triple.
extern "C" int fml_gemm_autotune(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                                 const fml_tensor *bias, const fml_tensor *residual,
                                 const fml_gemm_params *gp, void *stream, fml_gemm_params *tuned) {
  FML_REQUIRE(gp && tuned, FML_BAD_ARG, "fml_gemm_autotune: null argument");
  *tuned = *gp;
  GemmProblem p;
  TcPlan plan;
  bool use_tc = false;
  int st = resolve(a, b, c, bias, residual, gp, p, plan, use_tc);
  if (st != FML_OK) return st;
  if (!use_tc || gp->tile_n != 0 || gp->split_k != 0) return FML_OK;  // nothing to choose
  char key[256];
  snprintf(key, sizeof(key), "%lld,%lld,%lld,%lld,%lld|%d%d|%d,%d,%d,%d|%lld,%lld", (long long)p.M, (long long)p.N,
           (long long)p.K, (long long)p.nb0, (long long)p.nb1, plan.b_mn_major, plan.three_pass, gp->act,
           bias != nullptr, residual != nullptr, gp->divisor != 1.0f, (long long)p.c_sm, (long long)p.c_sn);
  static std::map<std::string, std::pair<int, int>> cache;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { tuned->tile_n = it->second.first; tuned->split_k = it->second.second; return FML_OK; }
  }
  cudaStream_t s = as_stream(stream);
  cudaEvent_t e0, e1;
  FML_CUDA(cudaEventCreate(&e0));
  FML_CUDA(cudaEventCreate(&e1));
  const GemmEpilogue epi = make_epilogue(*gp, bias != nullptr, residual != nullptr);
  const int tn_opts[] = {32, 48, 64, 96, 128, 192, 256};
  const int sk_opts[] = {1, 2, 4, 8};
  float best = 1e30f;
  int best_tn = plan.tile_n, best_sk = plan.split_k;
  std::vector<std::pair<int, int>> seen;
  for (int tn : tn_opts)
    for (int sk : sk_opts) {
      fml_gemm_params q = *gp;
      q.tile_n = tn;
      q.split_k = sk;
      TcPlan cand;
      if (!plan_gemm_tc(p, q, cand)) continue;
      const std::pair<int, int> id(cand.tile_n, cand.split_k);
      bool dup = false;
      for (const auto &x : seen) dup = dup || x == id;
      if (dup) continue;
      seen.push_back(id);
      const int reps = 6;
      if (launch_gemm_tc(p, epi, cand, s) != FML_OK) { cudaGetLastError(); continue; }  // warm-up; skip what cannot launch
      cudaEventRecord(e0, s);
      bool ok = true;
      for (int r = 0; r < reps && ok; ++r) ok = launch_gemm_tc(p, epi, cand, s) == FML_OK;
      cudaEventRecord(e1, s);
      if (cudaEventSynchronize(e1) != cudaSuccess || !ok) { cudaGetLastError(); continue; }
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      if (ms < best) { best = ms; best_tn = cand.tile_n; best_sk = cand.split_k; }
    }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  tuned->tile_n = best_tn;
  tuned->split_k = best_sk;
  std::lock_guard<std::mutex> lock(mu);
  cache[key] = {best_tn, best_sk};
  return FML_OK;
}
