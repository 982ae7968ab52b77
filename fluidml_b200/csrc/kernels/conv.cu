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
  // optional per-(image, input channel) scale of x, applied (one fp32 rounding, as a separate
  // Mul kernel would) while the operand is gathered
  const float *scale;
  int64_t scale_sn, scale_sc;
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
          if (ih >= 0 && ih < a.IH && iw >= 0 && iw < a.IW) {
            v = a.x[n * a.xs[0] + ic * a.xs[1] + ih * a.xs[2] + iw * a.xs[3]];
            if (a.scale) v = __fmul_rn(v, a.scale[n * a.scale_sn + ic * a.scale_sc]);
          }
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

// Direct convolution for a short reduction (IC * KH * KW <= 64: the strided first layer of an
// image network, 3 x 3 x 3 = 27).  The implicit GEMM above spends its time on index arithmetic
// when K is two k blocks long.  Here a thread owns one output pixel and OCB output channels:
// the CTA's weights [K][OCB] and a table of the K taps' input offsets sit in shared memory, each
// tap is one bounds-checked input load (lanes = consecutive pixels of a row) and OCB
// multiply-adds against broadcast 16-byte weight loads, and for every channel a warp stores 32
// consecutive pixels.  Any stride, dilation and padding.
struct DirectArgs {
  ConvArgs c;
  int K;
  int64_t M;
};

template <int OCB>
__global__ void __launch_bounds__(128) conv_direct_small_kernel(const DirectArgs d) {
  extern __shared__ __align__(16) float dc_smem[];
  const ConvArgs &a = d.c;
  float *w_s = dc_smem;                                   // [K][OCB]
  float *b_s = dc_smem + d.K * OCB;                       // [OCB]: on chip, so that no global load sits between the stores
  int *tab = reinterpret_cast<int *>(b_s + OCB);          // [K][3]: dy, dx, element offset
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int oc0 = (int)blockIdx.y * OCB;
  const int taps = (int)(a.KH * a.KW), KW = (int)a.KW;
  for (int i = tid; i < d.K * OCB; i += 128) {
    const int k = i / OCB, o = i - k * OCB;
    const int ic = k / taps, t = k - ic * taps, kh = t / KW, kw = t - kh * KW;
    const int oc = oc0 + o;
    w_s[i] = oc < (int)a.OC ? a.w[oc * a.ws[0] + ic * a.ws[1] + kh * a.ws[2] + kw * a.ws[3]] : 0.0f;
  }
  if (tid < OCB) b_s[tid] = (a.bias && oc0 + tid < (int)a.OC) ? a.bias[(oc0 + tid) * a.bias_stride] : 0.0f;
  for (int k = tid; k < d.K; k += 128) {
    const int ic = k / taps, t = k - ic * taps, kh = t / KW, kw = t - kh * KW;
    tab[3 * k] = kh * (int)a.dh;
    tab[3 * k + 1] = kw * (int)a.dw;
    tab[3 * k + 2] = (int)(ic * a.xs[1] + kh * a.dh * a.xs[2] + kw * a.dw * a.xs[3]);
  }
  __syncthreads();
  const int64_t m = (int64_t)blockIdx.x * 128 + tid;
  if (m >= d.M) return;
  const int OW = (int)a.OW, OH = (int)a.OH, IH = (int)a.IH, IW = (int)a.IW;
  const int64_t row = m / OW;
  const int ow = (int)(m - row * OW);
  const int64_t n = row / OH;
  const int oh = (int)(row - n * OH);
  const int ih0 = oh * (int)a.sh - (int)a.ph, iw0 = ow * (int)a.sw - (int)a.pw;
  const float *base = a.x + n * a.xs[0] + (int64_t)ih0 * a.xs[2] + (int64_t)iw0 * a.xs[3];
  float acc[OCB];
#pragma unroll
  for (int o = 0; o < OCB; ++o) acc[o] = 0.0f;
  for (int k = 0; k < d.K; ++k) {
    const int ih = ih0 + tab[3 * k], iw = iw0 + tab[3 * k + 1];
    const float v = ((unsigned)ih < (unsigned)IH && (unsigned)iw < (unsigned)IW) ? base[tab[3 * k + 2]] : 0.0f;
    const float4 *wr = reinterpret_cast<const float4 *>(w_s + k * OCB);
#pragma unroll
    for (int q = 0; q < OCB / 4; ++q) {
      const float4 w4 = wr[q];
      acc[4 * q] = fmaf(v, w4.x, acc[4 * q]);
      acc[4 * q + 1] = fmaf(v, w4.y, acc[4 * q + 1]);
      acc[4 * q + 2] = fmaf(v, w4.z, acc[4 * q + 2]);
      acc[4 * q + 3] = fmaf(v, w4.w, acc[4 * q + 3]);
    }
  }
  float *yp = a.y + n * a.ys[0] + (int64_t)oc0 * a.ys[1] + (int64_t)oh * a.ys[2] + (int64_t)ow * a.ys[3];
  const int nb = min(OCB, (int)a.OC - oc0);
  switch (a.act) {  // one dispatch per thread, outside the store loop
#define FML_DC_STORE(ACT)                                                                   \
  _Pragma("unroll") for (int o = 0; o < OCB; ++o)                                           \
    if (o < nb) yp[o * a.ys[1]] = conv_act(ACT, acc[o] + b_s[o]);
  case FML_ACT_RELU: FML_DC_STORE(FML_ACT_RELU) break;
  case FML_ACT_TANH: FML_DC_STORE(FML_ACT_TANH) break;
  case FML_ACT_SIGMOID: FML_DC_STORE(FML_ACT_SIGMOID) break;
  case FML_ACT_SILU: FML_DC_STORE(FML_ACT_SILU) break;
  default: FML_DC_STORE(FML_ACT_NONE) break;
#undef FML_DC_STORE
  }
}

// Depthwise convolution, tiled (dilation 1, stride 1 or 2, compile-time window).  A depthwise
// layer does KH*KW multiply-adds per element it moves, so it is bound by HBM -- and, on the way
// there, by the instructions issued per output, not by arithmetic.  The kernel is built around
// both: a CTA stages the input patch of its output tile in shared memory with coalesced 16-byte
// loads (rows and columns outside the image become the zero padding there); every thread then
// produces a micro-tile of 4 x 4 outputs, reading each input row of the micro-tile once as
// 16-byte shared-memory loads with the window's weights in registers (about 20 instructions per
// output, against ~140 with one strip per thread), and stores rows as float4 where the row
// length allows.  No index division sits inside a loop.  Planes too small to fill a CTA are
// batched: a CTA takes PP whole planes, otherwise one plane and a band of its rows.
struct DwArgs {
  ConvArgs c;
  int TR, PP, SW;       // thread rows (of 4 output rows) per tile, planes per CTA, strips per output row
  int PH, PWn, pitch;   // patch rows, patch columns, shared-memory row pitch (floats)
  int row_tiles;        // bands per plane
  int vec;              // input rows can be fetched as aligned float4
  int planes;           // N * C
  // ceil(2^32 / d) for d = PH * PWn, PWn and C: exact quotients by one multiply for dividends
  // below 2^16 (the flat staging walk divides every element index three times; with hardware
  // division the reciprocal unit was the busiest pipe of the kernel)
  uint32_t m_plane, m_pwn, m_c;
};

__device__ __forceinline__ uint32_t div_magic(uint32_t n, uint32_t d, uint32_t magic) { return d == 1 ? n : __umulhi(n, magic); }

template <int ACT>
__device__ __forceinline__ void dw_store_row(float *yp, const float *v, float bias, bool vec, int valid, int64_t ys3) {
  if (vec) {
    *reinterpret_cast<float4 *>(yp) = make_float4(conv_act(ACT, v[0] + bias), conv_act(ACT, v[1] + bias),
                                                  conv_act(ACT, v[2] + bias), conv_act(ACT, v[3] + bias));
  } else {
#pragma unroll
    for (int o = 0; o < 4; ++o)
      if (o < valid) yp[o * ys3] = conv_act(ACT, v[o] + bias);
  }
}

// RT: output rows per thread (4; 1 for one-row images, i.e. 1-D convolutions)
template <int KH, int KW, int S, int RT>
__global__ void __launch_bounds__(256) conv_depthwise_tiled_kernel(const DwArgs d) {
  extern __shared__ __align__(16) float dw_smem[];
  const ConvArgs &a = d.c;
  float *patch = dw_smem;                          // [PP][PH][pitch]
  float *wts = dw_smem + d.PP * d.PH * d.pitch;    // [PP][KH*KW + 1]: window, bias
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = (int)blockIdx.x / d.row_tiles;
  const int plane0 = tile * d.PP;
  const int oh0 = ((int)blockIdx.x - tile * d.row_tiles) * d.TR * RT;
  const int ih0 = oh0 * S - (int)a.ph;
  const int C = (int)a.OC, IH = (int)a.IH, IW = (int)a.IW, pw = (int)a.pw;
  const int n0 = plane0 / C, c0 = plane0 - n0 * C;  // the only division by a tensor extent
  // ---- weights and bias of the CTA's planes
  for (int i = tid; i < d.PP * (KH * KW + 1); i += 256) {
    const int pl = i / (KH * KW + 1), k = i - pl * (KH * KW + 1);
    float v = 0.0f;
    if (plane0 + pl < d.planes) {
      const int ch = (c0 + pl) % C;
      if (k < KH * KW) v = a.w[ch * a.ws[0] + (k / KW) * a.ws[2] + (k % KW) * a.ws[3]];
      else if (a.bias) v = a.bias[ch * a.bias_stride];
    }
    wts[i] = v;
  }
  // ---- patch.  Rows that cannot be fetched as aligned float4 (14- and 7-wide planes): a flat
  // walk over the patch, four independent elements per thread and step, loads before stores, so
  // that a CTA's few dozen loads per thread overlap instead of queueing behind each other's latency.
  if (!d.vec) {
    const int per_plane_elems = d.PH * d.PWn, total = d.PP * per_plane_elems;
    const int xs0 = (int)a.xs[0], xs1 = (int)a.xs[1], xs2 = (int)a.xs[2];  // the launcher checked that offsets fit 31 bits
    for (int base = tid; base < total; base += 1024) {
      float v[4];
      int at[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = base + 256 * u;
        v[u] = 0.0f;
        at[u] = -1;
        if (e < total) {
          const int pl = (int)div_magic((uint32_t)e, (uint32_t)per_plane_elems, d.m_plane), rem = e - pl * per_plane_elems;
          const int pr = (int)div_magic((uint32_t)rem, (uint32_t)d.PWn, d.m_pwn), pc = rem - pr * d.PWn;
          const int lin = c0 + pl, dn = (int)div_magic((uint32_t)lin, (uint32_t)C, d.m_c);
          const int ih = ih0 + pr, iw = pc - pw, nn = n0 + dn, ch = lin - dn * C;
          at[u] = (pl * d.PH + pr) * d.pitch + pc;
          if (plane0 + pl < d.planes && ih >= 0 && ih < IH && iw >= 0 && iw < IW)
            v[u] = a.x[nn * xs0 + ch * xs1 + ih * xs2 + iw];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (at[u] >= 0) patch[at[u]] = v[u];
    }
  } else {
    const int units = IW >> 2;                     // float4 chunks of the image row
    int p2 = 32, sh = 5;
    while (p2 > 1 && (p2 >> 1) >= units) { p2 >>= 1; --sh; }
    const int sub = lane >> sh, u0 = lane & (p2 - 1), step = 8 << (5 - sh);
    const int total_rows = d.PP * d.PH;
    int row = (warp << (5 - sh)) + sub;
    int pl = row / d.PH, pr = row - pl * d.PH;     // once per thread
    int n = n0, ch = c0 + pl;
    while (ch >= C) { ch -= C; ++n; }
    for (; row < total_rows; row += step) {
      const int ih = ih0 + pr;
      const bool row_ok = plane0 + pl < d.planes && ih >= 0 && ih < IH;
      const float *src = a.x + n * a.xs[0] + ch * a.xs[1] + ih * a.xs[2];
      float *dst = patch + row * d.pitch;
      {
        if (row_ok) {
          for (int u = u0; u < units; u += p2) {
            const float4 t = *reinterpret_cast<const float4 *>(src + 4 * u);
            float *q = dst + pw + 4 * u;
            q[0] = t.x; q[1] = t.y; q[2] = t.z; q[3] = t.w;
          }
          for (int c = u0; c < pw; c += p2) dst[c] = 0.0f;
          for (int c = pw + IW + u0; c < d.PWn; c += p2) dst[c] = 0.0f;
        } else {
          for (int c = u0; c < d.PWn; c += p2) dst[c] = 0.0f;
        }
      }
      pr += step;
      while (pr >= d.PH) { pr -= d.PH; ++pl; if (++ch == C) { ch = 0; ++n; } }
    }
  }
  __syncthreads();
  // ---- compute: thread -> (plane, thread row, strip): RT output rows x 4 output columns
  const int per_plane = d.TR * d.SW;
  const int pl = d.PP == 1 ? 0 : tid / per_plane, rem = tid - pl * per_plane;
  const int tr = rem / d.SW, j = rem - tr * d.SW;
  const int oh = oh0 + tr * RT, ow0 = j * 4;
  if (pl >= d.PP || tr >= d.TR || plane0 + pl >= d.planes || oh >= (int)a.OH) return;
  constexpr int IN_V = (3 * S + KW + 3) / 4;   // 16-byte loads per input row of the micro-tile
  constexpr int ROWS = (RT - 1) * S + KH;      // input rows of the micro-tile
  float w[KH * KW];
  const float *wp = wts + pl * (KH * KW + 1);
#pragma unroll
  for (int k = 0; k < KH * KW; ++k) w[k] = wp[k];
  const float bias = wp[KH * KW];
  float acc[RT][4];
#pragma unroll
  for (int i = 0; i < RT; ++i)
#pragma unroll
    for (int o = 0; o < 4; ++o) acc[i][o] = 0.0f;  // window first, bias last: the reference's order
  const float *prow = patch + (pl * d.PH + tr * RT * S) * d.pitch + ow0 * S;
#pragma unroll
  for (int ir = 0; ir < ROWS; ++ir) {
    float in[IN_V * 4];
#pragma unroll
    for (int v = 0; v < IN_V; ++v) {
      const float4 t = *reinterpret_cast<const float4 *>(prow + ir * d.pitch + v * 4);
      in[4 * v] = t.x; in[4 * v + 1] = t.y; in[4 * v + 2] = t.z; in[4 * v + 3] = t.w;
    }
#pragma unroll
    for (int rr = 0; rr < RT; ++rr) {
      const int kh = ir - rr * S;  // compile-time after unrolling
      if (kh >= 0 && kh < KH) {
#pragma unroll
        for (int kw = 0; kw < KW; ++kw)
#pragma unroll
          for (int o = 0; o < 4; ++o) acc[rr][o] = fmaf(in[o * S + kw], w[kh * KW + kw], acc[rr][o]);
      }
    }
  }
  int n = n0, ch = c0 + pl;
  while (ch >= C) { ch -= C; ++n; }
  float *yp = a.y + n * a.ys[0] + ch * a.ys[1] + oh * a.ys[2] + ow0 * a.ys[3];
  const int valid = (int)a.OW - ow0;
  const bool vec = a.ys[3] == 1 && valid >= 4 && ((reinterpret_cast<uintptr_t>(yp) & 15) == 0) && (a.ys[2] & 3) == 0;
  const int rows = min(RT, (int)a.OH - oh);
  switch (a.act) {  // one dispatch per thread, outside the store loops
#define FML_DW_ROWS(ACT)                                                                  \
  _Pragma("unroll") for (int rr = 0; rr < RT; ++rr)                                          \
    if (rr < rows) dw_store_row<ACT>(yp + rr * a.ys[2], acc[rr], bias, vec, valid, a.ys[3]);
  case FML_ACT_RELU: FML_DW_ROWS(FML_ACT_RELU) break;
  case FML_ACT_TANH: FML_DW_ROWS(FML_ACT_TANH) break;
  case FML_ACT_SIGMOID: FML_DW_ROWS(FML_ACT_SIGMOID) break;
  case FML_ACT_SILU: FML_DW_ROWS(FML_ACT_SILU) break;
  default: FML_DW_ROWS(FML_ACT_NONE) break;
#undef FML_DW_ROWS
  }
}

// Launches the tiled depthwise kernel when it has a variant for the window and stride; returns
// false (nothing launched) otherwise.
template <int KH, int KW, int S, int RT>
static bool launch_depthwise_tiled(const ConvArgs &a, const void *x_base, cudaStream_t s, int *status) {
  DwArgs d;
  d.c = a;
  d.SW = (int)((a.OW + 3) / 4);
  const int RW = (int)((a.OH + RT - 1) / RT);  // thread rows per plane
  if (d.SW > 256 || a.N * a.OC >= (1ll << 30) || a.IH * a.IW >= (1ll << 30)) return false;
  const int in_v = (3 * S + KW + 3) / 4;
  d.PWn = (d.SW - 1) * 4 * S + in_v * 4;  // the last strip starts at (SW - 1) * 4 * S and reads in_v float4
  if (d.PWn < (int)(a.pw + a.IW)) d.PWn = (int)(a.pw + a.IW + 3) / 4 * 4;  // the staged row always fits
  d.pitch = d.PWn + 4;  // rows 16 bytes apart modulo the bank cycle
  const int per_plane = RW * d.SW;
  d.row_tiles = 1;
  if (per_plane <= 256) {
    d.TR = RW; d.PP = 256 / per_plane;
  } else {  // bands of equal height
    const int tr_max = 256 / d.SW;
    d.row_tiles = (RW + tr_max - 1) / tr_max;
    d.TR = (RW + d.row_tiles - 1) / d.row_tiles;
    d.PP = 1;
  }
  d.planes = (int)(a.N * a.OC);
  if (d.PP > d.planes) d.PP = d.planes;
  auto smem_of = [&]() {
    d.PH = (d.TR * RT - 1) * S + KH;
    return ((size_t)d.PP * d.PH * d.pitch + (size_t)d.PP * (KH * KW + 1)) * sizeof(float);
  };
  while (smem_of() > 48 * 1024) {  // fewer planes, then shorter bands
    if (d.PP > 1) { d.PP = (d.PP + 1) / 2; continue; }
    if (d.TR == 1) return false;
    d.row_tiles += 1;
    d.TR = (RW + d.row_tiles - 1) / d.row_tiles;
  }
  d.row_tiles = (RW + d.TR - 1) / d.TR;
  const size_t smem = smem_of();
  auto magic = [](int64_t dv) { return (uint32_t)((0x100000000ull + (uint64_t)dv - 1) / (uint64_t)dv); };
  d.m_plane = magic((int64_t)d.PH * d.PWn); d.m_pwn = magic(d.PWn); d.m_c = magic(a.OC);
  if ((int64_t)d.PP * d.PH * d.PWn >= 65536 || a.OC + d.PP >= 65536) return false;  // the magic division's range
  if (a.N * a.xs[0] >= (1ll << 31) || a.xs[0] < 0 || a.xs[1] < 0 || a.xs[2] < 0) return false;  // 31-bit input offsets
  d.vec = (a.IW % 4 == 0) && (a.xs[2] % 4 == 0) && (a.xs[1] % 4 == 0) && (a.xs[0] % 4 == 0) &&
          ((reinterpret_cast<uintptr_t>(x_base) & 15) == 0) ? 1 : 0;
  const int64_t ctas = (int64_t)((d.planes + d.PP - 1) / d.PP) * d.row_tiles;
  if (ctas > 0x7fffffff) return false;
  *status = launch_kernel(conv_depthwise_tiled_kernel<KH, KW, S, RT>, dim3((unsigned)ctas), dim3(256), smem, s, d) == cudaSuccess
                ? FML_OK : FML_CUDA_ERROR;
  return true;
}

// Depthwise convolution over channel-innermost operands (x and y with channel stride 1: what a
// [batch, length, channels] activation looks like through the transposed view a Conv node reads
// it by).  Threads run along the channels, so every tap is one coalesced load and the weights of
// a thread's channels stay in L1; V channels per thread (4 when the channel count and the
// addresses allow 16-byte accesses).
template <int V>
__global__ void __launch_bounds__(256) conv_depthwise_cl_kernel(const ConvArgs a) {
  pdl_prologue();
  const unsigned CV = (unsigned)(a.OC / V), OW = (unsigned)a.OW, OH = (unsigned)a.OH;
  const unsigned total = (unsigned)a.N * OH * OW * CV;
  for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
    const unsigned pix = e / CV, c = (e - pix * CV) * V;
    const unsigned row = pix / OW, ow = pix - row * OW;
    const unsigned n = row / OH, oh = row - n * OH;
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.0f;
    const float *xn = a.x + n * a.xs[0] + c;
    for (int kh = 0; kh < (int)a.KH; ++kh) {
      const int ih = (int)oh * (int)a.sh - (int)a.ph + kh * (int)a.dh;
      if (ih < 0 || ih >= (int)a.IH) continue;
      for (int kw = 0; kw < (int)a.KW; ++kw) {
        const int iw = (int)ow * (int)a.sw - (int)a.pw + kw * (int)a.dw;
        if (iw < 0 || iw >= (int)a.IW) continue;
        const float *xp = xn + ih * a.xs[2] + iw * a.xs[3];
        const float *wp = a.w + c * a.ws[0] + kh * a.ws[2] + kw * a.ws[3];
        float xv[V];
        if (V == 4) {
          const float4 t = *reinterpret_cast<const float4 *>(xp);
          xv[0] = t.x; xv[1] = t.y; xv[2] = t.z; xv[3] = t.w;
        } else {
          xv[0] = xp[0];
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = fmaf(xv[v], __ldg(wp + v * a.ws[0]), acc[v]);
      }
    }
    float r[V];
#pragma unroll
    for (int v = 0; v < V; ++v) r[v] = conv_act(a.act, acc[v] + (a.bias ? __ldg(a.bias + (c + v) * a.bias_stride) : 0.0f));
    float *yp = a.y + n * a.ys[0] + oh * a.ys[2] + ow * a.ys[3] + c;
    if (V == 4) *reinterpret_cast<float4 *>(yp) = make_float4(r[0], r[1], r[2], r[3]);
    else yp[0] = r[0];
  }
}

// 1-D depthwise convolution, unit stride, reading a channel-innermost input ([batch, length,
// channels] through a transposed view) and writing a length-innermost output: a 32-channel x
// 32-position tile goes through shared memory, loaded with lanes along the channels and consumed
// with lanes along the positions, so both sides are coalesced (pitch 33: conflict-free).
constexpr int kDwT = 32, kDwSpanMax = 64;
__global__ void __launch_bounds__(256) conv_depthwise_1d_transposing_kernel(const ConvArgs a) {
  __shared__ float tile[kDwT + kDwSpanMax][kDwT + 1];
  pdl_prologue();
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int ow0 = (int)blockIdx.x * kDwT, c0 = (int)blockIdx.y * kDwT, n = (int)blockIdx.z;
  const int span = ((int)a.KW - 1) * (int)a.dw + 1, rows = kDwT + span - 1;
  const int C = (int)a.OC, IW = (int)a.IW, OW = (int)a.OW;
  for (int r = ty; r < rows; r += 8) {
    const int iw = ow0 - (int)a.pw + r, c = c0 + tx;
    tile[r][tx] = (iw >= 0 && iw < IW && c < C) ? a.x[n * a.xs[0] + iw * a.xs[3] + c] : 0.0f;
  }
  __syncthreads();
  const int ow = ow0 + tx;
  for (int cc = ty; cc < kDwT; cc += 8) {
    const int c = c0 + cc;
    if (c >= C) break;
    float acc = 0.0f;
    const float *wp = a.w + c * a.ws[0];
    for (int k = 0; k < (int)a.KW; ++k) acc = fmaf(tile[tx + k * (int)a.dw][cc], __ldg(wp + k * a.ws[3]), acc);
    if (a.bias) acc += __ldg(a.bias + c * a.bias_stride);
    if (ow < OW) a.y[n * a.ys[0] + c * a.ys[1] + ow * a.ys[3]] = conv_act(a.act, acc);
  }
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

// 2 x 2 / stride 2 pooling over dense NCHW planes whose rows are a multiple of 4 long (every
// pooling layer of VGG-16): a thread reads 16 bytes from each of the two input rows and writes two
// outputs; 32-bit index arithmetic with two divisions per thread.
__global__ void __launch_bounds__(256) pool2x2_kernel(const float *__restrict__ x, float *__restrict__ y, unsigned planes,
                                                     unsigned OH, unsigned OW2, unsigned IW, unsigned in_plane, int mode) {
  pdl_prologue();
  const unsigned total = planes * OH * OW2;
  for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
    const unsigned row = e / OW2, j = e - row * OW2;
    const unsigned plane = row / OH, oh = row - plane * OH;
    const float *src = x + (size_t)plane * in_plane + (size_t)(2 * oh) * IW + 4 * j;
    const float4 r0 = *reinterpret_cast<const float4 *>(src), r1 = *reinterpret_cast<const float4 *>(src + IW);
    float2 o;
    if (mode) {
      o.x = (((r0.x + r0.y) + r1.x) + r1.y) / 4.0f;  // the window's elements in row-major order
      o.y = (((r0.z + r0.w) + r1.z) + r1.w) / 4.0f;
    } else {
      o.x = fmaxf(fmaxf(r0.x, r0.y), fmaxf(r1.x, r1.y));
      o.y = fmaxf(fmaxf(r0.z, r0.w), fmaxf(r1.z, r1.w));
    }
    *reinterpret_cast<float2 *>(y + (size_t)row * (2 * OW2) + 2 * j) = o;
  }
}

}  // namespace
}  // namespace fml

using namespace fml;

// x_scale: nullptr, or a tensor broadcastable to [N, IC, 1, 1] that multiplies x (fml_conv_scaled)
static int conv_impl(const fml_tensor *x, const fml_tensor *x_scale, const fml_tensor *w, const fml_tensor *bias,
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
  a.scale = nullptr; a.scale_sn = a.scale_sc = 0;
  if (x_scale) {
    FML_REQUIRE(valid_tensor(x_scale) && x_scale->dtype == FML_F32 && x_scale->rank == x->rank, FML_BAD_ARG,
                "fml_conv_scaled: the scale must be an fp32 tensor of x's rank");
    FML_REQUIRE(group == 1, FML_UNSUPPORTED, "fml_conv_scaled: group must be 1");
    for (int i = 0; i < x_scale->rank; ++i) {
      const int64_t want = i < 2 ? x->shape[i] : 1;
      FML_REQUIRE(x_scale->shape[i] == want || (i < 2 && x_scale->shape[i] == 1), FML_BAD_ARG,
                  "fml_conv_scaled: the scale must broadcast to [N, IC, 1, 1]");
    }
    a.scale = (const float *)x_scale->data;
    a.scale_sn = x_scale->shape[0] == 1 ? 0 : x_scale->stride[0];
    a.scale_sc = x_scale->shape[1] == 1 ? 0 : x_scale->stride[1];
  }
  const int64_t M = a.N * a.OH * a.OW;
  if (M == 0 || a.OC == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  if (a.scale) {
    // the tensor-core kernel applies the scale while it splits the operand; every other case
    // takes the general implicit GEMM (the specialised CUDA-core paths below read x unscaled)
    if (nd == 2 && a.IC <= 4096 && conv_tc_eligible(x, w, y, p))
      return launch_conv_tc(x, w, bias, y, p, s, a.scale, a.scale_sn, a.scale_sc);
    FML_REQUIRE((M + CB - 1) / CB <= 65535, FML_UNSUPPORTED, "fml_conv_scaled: too many output pixels for one launch");
    dim3 grid((unsigned)((a.OC + CB - 1) / CB), (unsigned)((M + CB - 1) / CB));
    FML_LAUNCH((conv_igemm_kernel), grid, 256, 0, s, a);
    return FML_OK;
  }
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
    if (skinny_eligible(g)) return launch_gemm_skinny(g, e, s);
    // more images than the weight-streaming kernel takes: the general product, on tensor cores
    // when the shapes and alignments allow
    fml_tensor A, B, Cc, bias_t;
    memset(&A, 0, sizeof(A)); memset(&B, 0, sizeof(B)); memset(&Cc, 0, sizeof(Cc)); memset(&bias_t, 0, sizeof(bias_t));
    A.data = const_cast<float *>(g.a); A.dtype = FML_F32; A.rank = 2;
    A.shape[0] = g.M; A.shape[1] = g.K; A.stride[0] = g.a_sm; A.stride[1] = g.a_sk;
    B.data = const_cast<float *>(g.b); B.dtype = FML_F32; B.rank = 2;
    B.shape[0] = g.K; B.shape[1] = g.N; B.stride[0] = g.b_sk; B.stride[1] = g.b_sn;
    Cc.data = g.c; Cc.dtype = FML_F32; Cc.rank = 2;
    Cc.shape[0] = g.M; Cc.shape[1] = g.N; Cc.stride[0] = g.c_sm; Cc.stride[1] = g.c_sn;
    bias_t.data = const_cast<float *>(a.bias); bias_t.dtype = FML_F32; bias_t.rank = 1;
    bias_t.shape[0] = g.N; bias_t.stride[0] = a.bias_stride;
    fml_gemm_params gp;
    fml_gemm_default_params(&gp);
    gp.precision = p->precision;
    gp.act = a.act;
    return fml_gemm(&A, &B, &Cc, a.bias ? &bias_t : nullptr, nullptr, &gp, stream);
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
  if (group == 1 && a.IC * a.KH * a.KW <= 64 && a.IC * a.IH * a.IW < (1ll << 31) / 4 && (a.OC + 31) / 32 <= 65535 &&
      (M + 127) / 128 <= 0x7fffffff) {
    DirectArgs d;
    d.c = a; d.K = (int)(a.IC * a.KH * a.KW); d.M = M;
    const dim3 grid((unsigned)((M + 127) / 128), (unsigned)((a.OC + 31) / 32));
    const size_t smem = ((size_t)d.K * 32 + 32) * sizeof(float) + (size_t)d.K * 3 * sizeof(int);
    FML_LAUNCH((conv_direct_small_kernel<32>), grid, 128, smem, s, d);
    return FML_OK;
  }
  if (group == 1) {
    FML_REQUIRE((M + CB - 1) / CB <= 65535 * 32768ll, FML_UNSUPPORTED, "fml_conv: too many output pixels");
    dim3 grid((unsigned)((a.OC + CB - 1) / CB), (unsigned)((M + CB - 1) / CB));
    FML_REQUIRE(grid.y <= 65535, FML_UNSUPPORTED, "fml_conv: too many output pixels for one launch");
    FML_LAUNCH((conv_igemm_kernel), grid, 256, 0, s, a);
  } else {
    if (a.xs[1] == 1 && a.ys[1] == 1 && a.OC > 1 && M * a.OC < (1ll << 31)) {  // channel-innermost operands
      bool narrow = true;  // 32-bit offsets
      for (int i = 0; i < 4; ++i) narrow = narrow && a.xs[i] >= 0 && a.ys[i] >= 0;
      narrow = narrow && a.N * a.xs[0] < (1ll << 31) && a.N * a.ys[0] < (1ll << 31);
      if (narrow) {
        const bool v4 = a.OC % 4 == 0 && aligned16(a.x) && aligned16(a.y) && a.xs[0] % 4 == 0 && a.xs[2] % 4 == 0 &&
                        a.xs[3] % 4 == 0 && a.ys[0] % 4 == 0 && a.ys[2] % 4 == 0 && a.ys[3] % 4 == 0;
        if (v4) FML_LAUNCH((conv_depthwise_cl_kernel<4>), grid_for(M * a.OC / 4, 256), 256, 0, s, a);
        else FML_LAUNCH((conv_depthwise_cl_kernel<1>), grid_for(M * a.OC, 256), 256, 0, s, a);
        return FML_OK;
      }
    }
    if (a.IH == 1 && a.OH == 1 && a.KH == 1 && a.sw == 1 && a.xs[1] == 1 && a.ys[3] == 1 && a.OC > 1 &&
        (a.KW - 1) * a.dw + 1 <= kDwSpanMax && a.N <= 65535 && (a.OC + kDwT - 1) / kDwT <= 65535) {
      const dim3 grid((unsigned)((a.OW + kDwT - 1) / kDwT), (unsigned)((a.OC + kDwT - 1) / kDwT), (unsigned)a.N);
      FML_LAUNCH((conv_depthwise_1d_transposing_kernel), grid, 256, 0, s, a);
      return FML_OK;
    }
    if (nd == 2) {
      int st = FML_OK;
      if (launch_depthwise_tma(x, w, bias, y, p, s, &st)) return st;
    }
    if (a.dh == 1 && a.dw == 1 && a.sh == a.sw && (a.sh == 1 || a.sh == 2) && a.xs[3] == 1) {
      int st = FML_OK;
      bool done = false;
      const int key = (int)(a.KH * 100 + a.KW * 10 + a.sh);
      switch (key) {
      case 331: done = launch_depthwise_tiled<3, 3, 1, 4>(a, a.x, s, &st); break;
      case 332: done = launch_depthwise_tiled<3, 3, 2, 4>(a, a.x, s, &st); break;
      case 551: done = launch_depthwise_tiled<5, 5, 1, 4>(a, a.x, s, &st); break;
      case 552: done = launch_depthwise_tiled<5, 5, 2, 4>(a, a.x, s, &st); break;
      case 191: done = launch_depthwise_tiled<1, 9, 1, 1>(a, a.x, s, &st); break;
      case 131: done = launch_depthwise_tiled<1, 3, 1, 1>(a, a.x, s, &st); break;
      case 771: done = launch_depthwise_tiled<7, 7, 1, 4>(a, a.x, s, &st); break;
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

extern "C" int fml_conv(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias,
                        const fml_tensor *y, const fml_conv_params *p, void *stream) {
  return conv_impl(x, nullptr, w, bias, y, p, stream);
}

extern "C" int fml_conv_scaled(const fml_tensor *x, const fml_tensor *x_scale, const fml_tensor *w,
                               const fml_tensor *bias, const fml_tensor *y, const fml_conv_params *p, void *stream) {
  FML_REQUIRE(x_scale, FML_BAD_ARG, "fml_conv_scaled: no scale");
  return conv_impl(x, x_scale, w, bias, y, p, stream);
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
  if (mode == 1 && a.OH == 1 && a.OW == 1 && a.KH == x->shape[2] && a.KW == x->shape[3]) {
    // global average pooling is the mean over the two spatial axes: one warp per plane with
    // coalesced loads (the window kernel below gives a thread a whole plane, 196 bytes from its
    // neighbour's)
    const int32_t spatial[4] = {0, 0, 1, 1};
    return fml_reduce_mean(x, y, spatial, stream);
  }
  {
    const int64_t IH = x->shape[2], IW = x->shape[3];
    const bool dense_in = x->stride[3] == 1 && x->stride[2] == IW && x->stride[1] == IH * IW && x->stride[0] == a.C * IH * IW;
    const bool dense_out = y->stride[3] == 1 && y->stride[2] == a.OW && y->stride[1] == a.OH * a.OW &&
                           y->stride[0] == a.C * a.OH * a.OW;
    if (a.KH == 2 && a.KW == 2 && a.sh == 2 && a.sw == 2 && dense_in && dense_out && IW % 4 == 0 && 2 * a.OW == IW &&
        (IH * IW) % 4 == 0 && aligned16(x->data) && (reinterpret_cast<uintptr_t>(y->data) & 7) == 0 &&
        total < (1ll << 31) && a.N * a.C * IH * IW < (1ll << 40)) {
      FML_LAUNCH((pool2x2_kernel), grid_for(total / 2, 256), 256, 0, as_stream(stream), (const float *)x->data,
                 (float *)y->data, (unsigned)(a.N * a.C), (unsigned)a.OH, (unsigned)(a.OW / 2), (unsigned)IW,
                 (unsigned)(IH * IW), mode);
      return FML_OK;
    }
  }
  FML_LAUNCH((pool2d_kernel), grid_for(total, 256), 256, 0, as_stream(stream), a);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}
