// Convolution and pooling.
//
// group == 1: implicit GEMM (M = N*OH*OW output pixels, N = OC, K = IC*KH*KW) on a 64x64
// output tile; the im2col gather happens while filling the shared-memory A tile, so padding
// is implicit (out-of-image taps read as zero) and no padded copy or scratch is needed.
// group == C (depthwise, multiplier 1): one thread per output element.
// 1-D convolutions are the 2-D kernels with H = 1.
#include "gemm_common.cuh"

namespace fml {
namespace {

struct ConvArgs {
  int64_t N, IC, IH, IW, OC, OH, OW, KH, KW;
  int64_t ph, pw, sh, sw, dh, dw;
  int64_t xs[4], ws[4], ys[4];  // element strides n/c/h/w, o/i/h/w, n/c/h/w
  int64_t bias_stride;
  int64_t w_span, bias_span;  // bytes from the first to the last element of w / bias
  const float *x, *w, *bias;
  float *y;
  int act;
};

__device__ __forceinline__ float conv_act(int act, float v) {
  switch (act) {
  case FML_ACT_RELU: return fmaxf(v, 0.0f);
  case FML_ACT_TANH: return tanhf(v);
  // exp2-based exponential and approximate reciprocal (about 2 ulp each): the exact forms are
  // ~40 dependent instructions per element, which a TMEM-lane-per-thread epilogue with two warps
  // per scheduler cannot hide (measured: 8.6 us of a 128x96 tile's epilogue against 1.x us)
  case FML_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
  case FML_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
  default: return v;
  }
}

constexpr int CB = 64, CK = 16;

__global__ void __launch_bounds__(256) conv_igemm_kernel(ConvArgs a) {
  pdl_launch_dependents();
  l2_prefetch_span(a.w, a.w_span);
  l2_prefetch_span(a.bias, a.bias_span);
  pdl_wait();
  __shared__ float As[CK][CB + 4];
  __shared__ float Bs[CK][CB + 4];
  const int64_t Mtot = a.N * a.OH * a.OW, Ktot = a.IC * a.KH * a.KW;
  const int64_t m0 = (int64_t)blockIdx.y * CB, n0 = (int64_t)blockIdx.x * CB;
  const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < Ktot; k0 += CK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = t + i * 256;
      {  // A: pixel-fast mapping (consecutive threads = consecutive output pixels)
        const int mm = e & 63, kk = e >> 6;
        const int64_t gm = m0 + mm, gk = k0 + kk;
        float v = 0.0f;
        if (gm < Mtot && gk < Ktot) {
          const int64_t ow = gm % a.OW, oh = (gm / a.OW) % a.OH, n = gm / (a.OW * a.OH);
          const int64_t kw = gk % a.KW, kh = (gk / a.KW) % a.KH, ic = gk / (a.KW * a.KH);
          const int64_t ih = oh * a.sh - a.ph + kh * a.dh, iw = ow * a.sw - a.pw + kw * a.dw;
          if (ih >= 0 && ih < a.IH && iw >= 0 && iw < a.IW)
            v = a.x[n * a.xs[0] + ic * a.xs[1] + ih * a.xs[2] + iw * a.xs[3]];
        }
        As[kk][mm] = v;
      }
      {  // B: k-fast mapping (OIHW weights are contiguous in k for one output channel)
        const int kk = e & 15, nn = e >> 4;
        const int64_t gn = n0 + nn, gk = k0 + kk;
        float v = 0.0f;
        if (gn < a.OC && gk < Ktot) {
          const int64_t kw = gk % a.KW, kh = (gk / a.KW) % a.KH, ic = gk / (a.KW * a.KH);
          v = a.w[gn * a.ws[0] + ic * a.ws[1] + kh * a.ws[2] + kw * a.ws[3]];
        }
        Bs[kk][nn] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < CK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[kk][tx * 4 + i]; bv[i] = Bs[kk][ty * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  // threads along tx own consecutive pixels: stores to NCHW are contiguous in ow
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t gm = m0 + tx * 4 + i, oc = n0 + ty * 4 + j;
      if (gm < Mtot && oc < a.OC) {
        const int64_t ow = gm % a.OW, oh = (gm / a.OW) % a.OH, n = gm / (a.OW * a.OH);
        float v = acc[i][j];
        if (a.bias) v += a.bias[oc * a.bias_stride];
        a.y[n * a.ys[0] + oc * a.ys[1] + oh * a.ys[2] + ow * a.ys[3]] = conv_act(a.act, v);
      }
    }
}

__global__ void conv_depthwise_kernel(ConvArgs a) {
  pdl_launch_dependents();
  l2_prefetch_span(a.w, a.w_span);
  l2_prefetch_span(a.bias, a.bias_span);
  pdl_wait();
  const int64_t total = a.N * a.OC * a.OH * a.OW;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t ow = e % a.OW, oh = (e / a.OW) % a.OH, c = (e / (a.OW * a.OH)) % a.OC,
                  n = e / (a.OW * a.OH * a.OC);
    float s = 0.0f;
    for (int64_t kh = 0; kh < a.KH; ++kh) {
      const int64_t ih = oh * a.sh - a.ph + kh * a.dh;
      if (ih < 0 || ih >= a.IH) continue;
      for (int64_t kw = 0; kw < a.KW; ++kw) {
        const int64_t iw = ow * a.sw - a.pw + kw * a.dw;
        if (iw < 0 || iw >= a.IW) continue;
        s = fmaf(a.x[n * a.xs[0] + c * a.xs[1] + ih * a.xs[2] + iw * a.xs[3]],
                 a.w[c * a.ws[0] + kh * a.ws[2] + kw * a.ws[3]], s);
      }
    }
    if (a.bias) s += a.bias[c * a.bias_stride];
    a.y[n * a.ys[0] + c * a.ys[1] + oh * a.ys[2] + ow * a.ys[3]] = conv_act(a.act, s);
  }
}

// Depthwise convolution, tiled (dilation 1, stride 1 or 2, compile-time window).  A depthwise
// layer does KH*KW multiply-adds per element it moves, so it is bound by HBM, not by arithmetic,
// and the kernel is built around the memory system: a CTA stages the input patch of its output
// tile in shared memory with coalesced loads (rows and columns outside the image become the zero
// padding there), every thread then produces a strip of four adjacent outputs from 16-byte
// shared-memory loads with the window's weights in registers, and stores the strip as one float4
// where the row length allows.  Each input element is read from global memory once per tile
// (plus the halo rows between row tiles).  Planes too small to fill a CTA are batched: a CTA takes
// PP whole planes of TH = OH rows, otherwise one plane and TH rows of it.
struct DwArgs {
  ConvArgs c;
  int TH, PP, SW;       // output rows per tile, planes per CTA, four-wide strips per output row
  int PH, PWn, pitch;   // patch rows, patch columns that are loaded, shared-memory row pitch (floats)
  int row_tiles;        // ceil(OH / TH)
  int64_t planes;       // N * C
};

template <int KH, int KW, int S>
__global__ void __launch_bounds__(256) conv_depthwise_tiled_kernel(const DwArgs d) {
  extern __shared__ __align__(16) float dw_smem[];
  const ConvArgs &a = d.c;
  float *patch = dw_smem;                                            // [PP][PH][pitch]
  float *wts = dw_smem + (size_t)d.PP * d.PH * d.pitch;              // [PP][KH*KW + 1]: window, bias
  pdl_launch_dependents();
  l2_prefetch_span(a.w, a.w_span);
  l2_prefetch_span(a.bias, a.bias_span);
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t plane0 = (int64_t)(blockIdx.x / d.row_tiles) * d.PP;
  const int oh0 = (int)(blockIdx.x % d.row_tiles) * d.TH;
  const int ih0 = oh0 * S - (int)a.ph;
  // ---- stage weights and bias of the CTA's planes
  for (int i = tid; i < d.PP * (KH * KW + 1); i += 256) {
    const int pl = i / (KH * KW + 1), k = i - pl * (KH * KW + 1);
    const int64_t plane = plane0 + pl;
    float v = 0.0f;
    if (plane < d.planes) {
      const int64_t ch = plane % a.OC;
      if (k < KH * KW) v = a.w[ch * a.ws[0] + (k / KW) * a.ws[2] + (k % KW) * a.ws[3]];
      else if (a.bias) v = a.bias[ch * a.bias_stride];
    }
    wts[i] = v;
  }
  // ---- stage the patch: lanes run along a patch row (sub-warps share a warp when rows are short)
  {
    int p2 = 32;
    while (p2 > 1 && (p2 >> 1) >= d.PWn) p2 >>= 1;  // smallest power of two >= PWn, at most 32
    const int sub = lane / p2, pc0 = lane - sub * p2, rows_per_iter = 8 * (32 / p2);
    const int total_rows = d.PP * d.PH;
    for (int row = warp * (32 / p2) + sub; row < total_rows; row += rows_per_iter) {
      const int pl = row / d.PH, pr = row - pl * d.PH;
      const int64_t plane = plane0 + pl;
      const int ih = ih0 + pr;
      const bool row_ok = plane < d.planes && ih >= 0 && ih < a.IH;
      const float *src = a.x + (plane / a.IC) * a.xs[0] + (plane % a.IC) * a.xs[1] + (int64_t)ih * a.xs[2];
      float *dst = patch + (size_t)row * d.pitch;
      for (int pc = pc0; pc < d.PWn; pc += p2) {
        const int iw = pc - (int)a.pw;
        dst[pc] = (row_ok && iw >= 0 && iw < a.IW) ? src[(int64_t)iw * a.xs[3]] : 0.0f;
      }
    }
  }
  __syncthreads();
  // ---- compute: thread -> (plane, output row, strip of four outputs)
  const int per_plane = d.TH * d.SW;
  const int pl = tid / per_plane, rem = tid - pl * per_plane;
  const int r = rem / d.SW, j = rem - r * d.SW;
  const int64_t plane = plane0 + pl;
  const int oh = oh0 + r, ow0 = j * 4;
  if (pl >= d.PP || plane >= d.planes || oh >= a.OH) return;
  constexpr int IN_W = 3 * S + KW;            // inputs a strip of four outputs reads per row
  constexpr int IN_V = (IN_W + 3) / 4;        // ... as 16-byte loads
  float w[KH * KW];
  const float *wp = wts + pl * (KH * KW + 1);
#pragma unroll
  for (int k = 0; k < KH * KW; ++k) w[k] = wp[k];
  const float bias = wp[KH * KW];
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // window first, bias last: the reference's order
  const float *prow = patch + ((size_t)pl * d.PH + (size_t)r * S) * d.pitch + (size_t)ow0 * S;
#pragma unroll
  for (int kh = 0; kh < KH; ++kh) {
    float in[IN_V * 4];
#pragma unroll
    for (int v = 0; v < IN_V; ++v) {
      const float4 t = *reinterpret_cast<const float4 *>(prow + (size_t)kh * d.pitch + v * 4);
      in[4 * v] = t.x; in[4 * v + 1] = t.y; in[4 * v + 2] = t.z; in[4 * v + 3] = t.w;
    }
#pragma unroll
    for (int kw = 0; kw < KW; ++kw)
#pragma unroll
      for (int o = 0; o < 4; ++o) acc[o] = fmaf(in[o * S + kw], w[kh * KW + kw], acc[o]);
  }
  float *yp = a.y + (plane / a.OC) * a.ys[0] + (plane % a.OC) * a.ys[1] + (int64_t)oh * a.ys[2] + (int64_t)ow0 * a.ys[3];
  if (a.ys[3] == 1 && ow0 + 4 <= a.OW && ((reinterpret_cast<uintptr_t>(yp) & 15) == 0)) {
    *reinterpret_cast<float4 *>(yp) = make_float4(conv_act(a.act, acc[0] + bias), conv_act(a.act, acc[1] + bias),
                                                  conv_act(a.act, acc[2] + bias), conv_act(a.act, acc[3] + bias));
  } else {
#pragma unroll
    for (int o = 0; o < 4; ++o)
      if (ow0 + o < a.OW) yp[(int64_t)o * a.ys[3]] = conv_act(a.act, acc[o] + bias);
  }
}

// Launches the tiled depthwise kernel when it has a variant for the window and stride; returns
// false (nothing launched) otherwise.
template <int KH, int KW, int S>
static bool launch_depthwise_tiled(const ConvArgs &a, cudaStream_t s, int *status) {
  DwArgs d;
  d.c = a;
  d.SW = (int)((a.OW + 3) / 4);
  if (d.SW > 256) return false;
  const int per_plane = (int)a.OH * d.SW;
  if (per_plane <= 256) { d.TH = (int)a.OH; d.PP = 256 / per_plane; }
  else { d.TH = 256 / d.SW; d.PP = 1; }
  d.planes = a.N * a.OC;
  if (d.PP > d.planes) d.PP = (int)d.planes;
  d.PH = (d.TH - 1) * S + KH;
  // columns a row of strips reads: the last strip starts at (SW - 1) * 4 * S and reads IN_V float4
  const int in_v = (3 * S + KW + 3) / 4;
  d.PWn = (d.SW - 1) * 4 * S + in_v * 4;
  d.pitch = d.PWn + 4;  // rows 16 bytes apart modulo the bank cycle
  d.row_tiles = (int)((a.OH + d.TH - 1) / d.TH);
  const size_t smem = ((size_t)d.PP * d.PH * d.pitch + (size_t)d.PP * (KH * KW + 1)) * sizeof(float);
  if (smem > 48 * 1024) return false;
  const int64_t ctas = (d.planes + d.PP - 1) / d.PP * d.row_tiles;
  if (ctas > 0x7fffffff) return false;
  *status = launch_kernel(conv_depthwise_tiled_kernel<KH, KW, S>, dim3((unsigned)ctas), dim3(256), smem, s, d) == cudaSuccess
                ? FML_OK : FML_CUDA_ERROR;
  return true;
}

struct PoolArgs {
  int64_t N, C, OH, OW, KH, KW, sh, sw;
  int64_t xs[4], ys[4];
  const float *x;
  float *y;
  int mode;
};

__global__ void pool2d_kernel(PoolArgs a) {
  pdl_prologue();
  const int64_t total = a.N * a.C * a.OH * a.OW;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t ow = e % a.OW, oh = (e / a.OW) % a.OH, c = (e / (a.OW * a.OH)) % a.C,
                  n = e / (a.OW * a.OH * a.C);
    const float *src = a.x + n * a.xs[0] + c * a.xs[1] + oh * a.sh * a.xs[2] + ow * a.sw * a.xs[3];
    float r = a.mode ? 0.0f : -3.402823466e+38f;
    for (int64_t kh = 0; kh < a.KH; ++kh)
      for (int64_t kw = 0; kw < a.KW; ++kw) {
        const float v = src[kh * a.xs[2] + kw * a.xs[3]];
        r = a.mode ? r + v : fmaxf(r, v);
      }
    if (a.mode) r = r / (float)(a.KH * a.KW);
    a.y[n * a.ys[0] + c * a.ys[1] + oh * a.ys[2] + ow * a.ys[3]] = r;
  }
}

}  // namespace
}  // namespace fml

using namespace fml;

extern "C" int fml_conv(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias,
                        const fml_tensor *y, const fml_conv_params *p, void *stream) {
  FML_REQUIRE(valid_tensor(x) && valid_tensor(w) && valid_tensor(y) && p, FML_BAD_ARG, "fml_conv: bad argument");
  FML_REQUIRE(x->dtype == FML_F32 && w->dtype == FML_F32 && y->dtype == FML_F32, FML_UNSUPPORTED, "fml_conv: fp32 only");
  FML_REQUIRE((x->rank == 3 || x->rank == 4) && w->rank == x->rank && y->rank == x->rank, FML_BAD_ARG,
              "fml_conv: 1-D or 2-D NCHW/OIHW tensors expected");
  const int nd = x->rank - 2;
  ConvArgs a;
  a.N = x->shape[0]; a.IC = x->shape[1]; a.OC = w->shape[0];
  a.IH = nd == 2 ? x->shape[2] : 1; a.IW = x->shape[nd + 1];
  a.OH = nd == 2 ? y->shape[2] : 1; a.OW = y->shape[nd + 1];
  a.KH = nd == 2 ? w->shape[2] : 1; a.KW = w->shape[nd + 1];
  a.ph = nd == 2 ? p->pads_begin[0] : 0; a.pw = nd == 2 ? p->pads_begin[1] : p->pads_begin[0];
  a.sh = nd == 2 ? p->strides[0] : 1; a.sw = nd == 2 ? p->strides[1] : p->strides[0];
  a.dh = nd == 2 ? p->dilations[0] : 1; a.dw = nd == 2 ? p->dilations[1] : p->dilations[0];
  FML_REQUIRE(a.sh >= 1 && a.sw >= 1 && a.dh >= 1 && a.dw >= 1, FML_BAD_ARG, "fml_conv: strides/dilations must be >= 1");
  FML_REQUIRE(y->shape[0] == a.N && y->shape[1] == a.OC, FML_BAD_ARG, "fml_conv: output shape");
  const int64_t group = p->group <= 0 ? 1 : p->group;
  FML_REQUIRE(group == 1 || (group == a.IC && a.OC == a.IC && w->shape[1] == 1), FML_UNSUPPORTED,
              "fml_conv: group must be 1 or depthwise with multiplier 1");
  FML_REQUIRE(group != 1 || w->shape[1] == a.IC, FML_BAD_ARG, "fml_conv: weight input channels");
  a.xs[0] = x->stride[0]; a.xs[1] = x->stride[1]; a.xs[2] = nd == 2 ? x->stride[2] : 0; a.xs[3] = x->stride[nd + 1];
  a.ws[0] = w->stride[0]; a.ws[1] = w->stride[1]; a.ws[2] = nd == 2 ? w->stride[2] : 0; a.ws[3] = w->stride[nd + 1];
  a.ys[0] = y->stride[0]; a.ys[1] = y->stride[1]; a.ys[2] = nd == 2 ? y->stride[2] : 0; a.ys[3] = y->stride[nd + 1];
  a.x = (const float *)x->data; a.w = (const float *)w->data; a.y = (float *)y->data;
  a.bias = nullptr; a.bias_stride = 0;
  if (bias) {
    FML_REQUIRE(valid_tensor(bias) && bias->dtype == FML_F32 && numel(bias) == a.OC, FML_BAD_ARG,
                "fml_conv: bias must hold one value per output channel");
    a.bias = (const float *)bias->data;
    for (int i = 0; i < bias->rank; ++i) if (bias->shape[i] != 1) a.bias_stride = bias->stride[i];
  }
  {
    int64_t last = 0;
    for (int i = 0; i < w->rank; ++i) last += (w->shape[i] - 1) * (w->stride[i] > 0 ? w->stride[i] : 0);
    a.w_span = (last + 1) * (int64_t)sizeof(float);
    a.bias_span = a.bias ? ((a.OC - 1) * (a.bias_stride > 0 ? a.bias_stride : 0) + 1) * (int64_t)sizeof(float) : 0;
  }
  a.act = p->act;
  const int64_t M = a.N * a.OH * a.OW;
  if (M == 0 || a.OC == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  if (group == 1 && a.IH == 1 && a.IW == 1 && a.OH == 1 && a.OW == 1 && a.ph < a.KH && a.pw < a.KW) {
    // One pixel in, one pixel out (the squeeze-and-excite convolutions): only the tap under the
    // pixel contributes, and the convolution is the product [N, IC] x [IC, OC] -- rows = images,
    // so the weight-streaming kernel takes it (up to 32 images), with the bias and activation in
    // its epilogue.
    GemmProblem g;
    memset(&g, 0, sizeof(g));
    g.M = a.N; g.N = a.OC; g.K = a.IC; g.nb0 = g.nb1 = 1;
    g.a = a.x; g.a_sm = a.xs[0]; g.a_sk = a.xs[1];
    g.b = a.w + a.ph * a.ws[2] + a.pw * a.ws[3]; g.b_sk = a.ws[1]; g.b_sn = a.ws[0];
    g.c = a.y; g.c_sm = a.ys[0]; g.c_sn = a.ys[1];
    g.bias = a.bias; g.bias_sm = 0; g.bias_sn = a.bias_stride;
    GemmEpilogue e;
    e.divisor = 1.0f; e.alpha = 1.0f; e.beta = 1.0f; e.act = a.act;
    e.c0 = 1.4142135381698608f; e.c1 = 1.0f; e.c2 = 0.5f;
    e.has_bias = a.bias != nullptr; e.has_res = 0;
    return skinny_eligible(g) ? launch_gemm_skinny(g, e, s) : launch_gemm_simt(g, e, s);
  }
  if (group == 1 && nd == 2 && conv_tc_eligible(x, w, y, p)) return launch_conv_tc(x, w, bias, y, p, s);
  if (group == 1 && a.KH == 1 && a.KW == 1 && a.ph == 0 && a.pw == 0 && a.sh == 1 && a.sw == 1 && a.ws[1] == 1 &&
      a.xs[3] == 1 && (nd == 1 || a.xs[2] == a.IW) && a.ys[3] == 1 && (nd == 1 || a.ys[2] == a.OW) &&
      a.act <= FML_ACT_SIGMOID && a.OH == a.IH && a.OW == a.IW) {
    // A pointwise convolution with channel-contiguous weights is, per image, the product
    // W [OC, IC] x X [IC, H*W] (pixels contiguous: an MN-major B operand): fml_gemm takes it, on
    // tensor cores when the pixel count is a multiple of 4, with the bias per output row.
    fml_tensor A, B, C, bias_t;
    memset(&A, 0, sizeof(A)); memset(&B, 0, sizeof(B)); memset(&C, 0, sizeof(C)); memset(&bias_t, 0, sizeof(bias_t));
    const int64_t HW = a.IH * a.IW;
    A.data = const_cast<float *>(a.w); A.dtype = FML_F32; A.rank = 2;
    A.shape[0] = a.OC; A.shape[1] = a.IC; A.stride[0] = a.ws[0]; A.stride[1] = 1;
    B.data = const_cast<float *>(a.x); B.dtype = FML_F32; B.rank = 3;
    B.shape[0] = a.N; B.shape[1] = a.IC; B.shape[2] = HW; B.stride[0] = a.xs[0]; B.stride[1] = a.xs[1]; B.stride[2] = 1;
    C.data = a.y; C.dtype = FML_F32; C.rank = 3;
    C.shape[0] = a.N; C.shape[1] = a.OC; C.shape[2] = HW; C.stride[0] = a.ys[0]; C.stride[1] = a.ys[1]; C.stride[2] = 1;
    bias_t.data = const_cast<float *>(a.bias); bias_t.dtype = FML_F32; bias_t.rank = 2;
    bias_t.shape[0] = a.OC; bias_t.shape[1] = 1; bias_t.stride[0] = a.bias_stride; bias_t.stride[1] = 0;
    fml_gemm_params gp;
    fml_gemm_default_params(&gp);
    gp.precision = p->precision;
    gp.act = a.act;
    gp.b_constant = 0;
    const int st = fml_gemm(&A, &B, &C, a.bias ? &bias_t : nullptr, nullptr, &gp, stream);
    if (st != FML_MISALIGNED) return st;  // a forced tensor-core precision on unaligned planes: CUDA cores below
  }
  if (group == 1) {
    FML_REQUIRE((M + CB - 1) / CB <= 65535 * 32768ll, FML_UNSUPPORTED, "fml_conv: too many output pixels");
    dim3 grid((unsigned)((a.OC + CB - 1) / CB), (unsigned)((M + CB - 1) / CB));
    FML_REQUIRE(grid.y <= 65535, FML_UNSUPPORTED, "fml_conv: too many output pixels for one launch");
    FML_LAUNCH((conv_igemm_kernel), grid, 256, 0, s, a);
  } else {
    if (a.dh == 1 && a.dw == 1 && a.sh == a.sw && (a.sh == 1 || a.sh == 2) && a.xs[3] == 1) {
      int st = FML_OK;
      bool done = false;
      const int key = (int)(a.KH * 100 + a.KW * 10 + a.sh);
      switch (key) {
      case 331: done = launch_depthwise_tiled<3, 3, 1>(a, s, &st); break;
      case 332: done = launch_depthwise_tiled<3, 3, 2>(a, s, &st); break;
      case 551: done = launch_depthwise_tiled<5, 5, 1>(a, s, &st); break;
      case 552: done = launch_depthwise_tiled<5, 5, 2>(a, s, &st); break;
      case 191: done = launch_depthwise_tiled<1, 9, 1>(a, s, &st); break;
      case 131: done = launch_depthwise_tiled<1, 3, 1>(a, s, &st); break;
      case 771: done = launch_depthwise_tiled<7, 7, 1>(a, s, &st); break;
      default: break;
      }
      if (done) {
        FML_REQUIRE(st == FML_OK, FML_CUDA_ERROR, "fml_conv: depthwise launch failed (%s)", cudaGetErrorString(cudaGetLastError()));
        return FML_OK;
      }
    }
    FML_LAUNCH((conv_depthwise_kernel), grid_for(M * a.OC, 256), 256, 0, s, a);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_conv_uses_tensor_cores(const fml_tensor *x, const fml_tensor *w, const fml_tensor *y,
                                          const fml_conv_params *p, int *uses) {
  FML_REQUIRE(valid_tensor(x) && valid_tensor(w) && valid_tensor(y) && p && uses, FML_BAD_ARG,
              "fml_conv_uses_tensor_cores: bad argument");
  *uses = x->rank == 4 && w->rank == 4 && y->rank == 4 && x->dtype == FML_F32 && w->dtype == FML_F32 &&
                  y->dtype == FML_F32 && p->group <= 1 && conv_tc_eligible(x, w, y, p)
              ? 1 : 0;
  return FML_OK;
}

extern "C" int fml_pool2d(const fml_tensor *x, const fml_tensor *y, int mode, const int64_t *kernel,
                          const int64_t *strides, void *stream) {
  FML_REQUIRE(valid_tensor(x) && valid_tensor(y) && kernel && strides, FML_BAD_ARG, "fml_pool2d: bad argument");
  FML_REQUIRE(x->dtype == FML_F32 && y->dtype == FML_F32 && x->rank == 4 && y->rank == 4, FML_UNSUPPORTED,
              "fml_pool2d: fp32 NCHW only");
  PoolArgs a;
  a.N = y->shape[0]; a.C = y->shape[1]; a.OH = y->shape[2]; a.OW = y->shape[3];
  a.KH = kernel[0]; a.KW = kernel[1]; a.sh = strides[0]; a.sw = strides[1];
  FML_REQUIRE(a.KH >= 1 && a.KW >= 1 && a.sh >= 1 && a.sw >= 1, FML_BAD_ARG, "fml_pool2d: kernel/strides");
  FML_REQUIRE((a.OH - 1) * a.sh + a.KH <= x->shape[2] && (a.OW - 1) * a.sw + a.KW <= x->shape[3] &&
                  x->shape[0] == a.N && x->shape[1] == a.C,
              FML_BAD_ARG, "fml_pool2d: window leaves the input (pools take no padding)");
  for (int i = 0; i < 4; ++i) { a.xs[i] = x->stride[i]; a.ys[i] = y->stride[i]; }
  a.x = (const float *)x->data; a.y = (float *)y->data; a.mode = mode;
  const int64_t total = a.N * a.C * a.OH * a.OW;
  if (total == 0) return FML_OK;
  FML_LAUNCH((pool2d_kernel), grid_for(total, 256), 256, 0, as_stream(stream), a);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}
