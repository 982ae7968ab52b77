// Shape analysis and epilogue shared by the two GEMM kernels (fp32 FMA and tcgen05).
#pragma once
#include "common.cuh"

namespace fml {

// C[z, m, n] = sum_k A[z, m, k] * B[z, k, n]; z runs over at most two collapsed batch dims
// (inner = fastest).  All strides in elements; a batch stride of 0 means broadcast.
struct GemmProblem {
  int64_t M, N, K;
  int64_t nb0, nb1;  // inner / outer batch extents (1 when absent)
  int64_t a_sm, a_sk, a_b0, a_b1;
  int64_t b_sk, b_sn, b_b0, b_b1;
  int64_t c_sm, c_sn, c_b0, c_b1;
  int64_t bias_sm, bias_sn, bias_b0, bias_b1;
  int64_t res_sm, res_sn, res_b0, res_b1;
  const float *a, *b, *bias, *res;
  float *c;
  const char *prefetch;  // optional L2 prefetch hint (fml_gemm_params::l2_prefetch)
  unsigned long long prefetch_bytes;
  int b_constant;  // B is not written by earlier launches on the stream (fml_gemm_params::b_constant)
};

struct GemmEpilogue {
  float divisor, alpha, beta;
  int act;
  float c0, c1, c2;
  int has_bias, has_res;
};

__device__ __forceinline__ float gemm_epilogue(const GemmEpilogue &e, float acc, float bias,
                                               float res) {
  float v = acc;
  if (e.divisor != 1.0f) v = v / e.divisor;
  if (e.has_bias) v = e.alpha * v + e.beta * bias;
  else if (e.alpha != 1.0f) v = e.alpha * v;
  switch (e.act) {
  case FML_ACT_GELU_ERF: v = v * (erff(v / e.c0) + e.c1) * e.c2; break;
  case FML_ACT_RELU: v = fmaxf(v, 0.0f); break;
  case FML_ACT_TANH: v = tanhf(v); break;
  case FML_ACT_SIGMOID: v = 1.0f / (1.0f + expf(-v)); break;
  case FML_ACT_SILU: v = v * (1.0f / (1.0f + expf(-v))); break;
  default: break;
  }
  if (e.has_res) v += res;
  return v;
}

// Fills `p` from the tensors; returns FML_UNSUPPORTED when more than two batch dims remain
// after collapsing (the caller then loops or falls back).
int analyse_gemm(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                 const fml_tensor *bias, const fml_tensor *res, GemmProblem &p);

int launch_gemm_simt(const GemmProblem &p, const GemmEpilogue &e, cudaStream_t s);

// Products with at most 32 rows: a weight-streaming kernel with split-K partials in
// library-owned scratch memory (one buffer per device and stream).
bool skinny_eligible(const GemmProblem &p);
int launch_gemm_skinny(const GemmProblem &p, const GemmEpilogue &e, cudaStream_t s);

// tcgen05 path -------------------------------------------------------------------------
struct TcPlan {
  int tile_n;     // 16..256, multiple of 16
  int split_k;    // >= 1
  int stages;
  int b_mn_major; // 0: B tile is K-major (b_sk == 1), 1: MN-major (b_sn == 1)
  int three_pass; // 1: 3xTF32, 0: single TF32
  int a_tmem;     // 3xTF32 only: A's hi / lo parts live in tensor memory instead of shared memory
  size_t smem_bytes;
};

// Whether the operands can be fed to TMA/UMMA directly, and with which plan.
bool plan_gemm_tc(const GemmProblem &p, const fml_gemm_params &gp, TcPlan &plan);
int launch_gemm_tc(const GemmProblem &p, const GemmEpilogue &e, const TcPlan &plan, cudaStream_t s);

// pipelined depthwise convolution over dense NCHW planes (conv_depthwise_tma.cu); false = not taken
bool launch_depthwise_tma(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias, const fml_tensor *y,
                          const fml_conv_params *p, cudaStream_t s, int *status);

// tcgen05 implicit-GEMM convolution (conv_tc.cu)
bool conv_tc_eligible(const fml_tensor *x, const fml_tensor *w, const fml_tensor *y, const fml_conv_params *p);
int launch_conv_tc(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias, const fml_tensor *y,
                   const fml_conv_params *p, cudaStream_t s, const float *x_scale = nullptr, int64_t x_scale_sn = 0,
                   int64_t x_scale_sc = 0);

}  // namespace fml
