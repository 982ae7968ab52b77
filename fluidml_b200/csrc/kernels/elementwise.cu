// Strided N-ary elementwise kernels: Add/Mul/Div/Sub/Pow/Equal (broadcast), their
// scalar-constant variants, the unary math ops, bias+GELU and Where.
//
// HBM-bound: each output element is read-modify-written once.  When every operand's
// innermost collapsed dimension is contiguous (or broadcast) and 16-byte aligned the kernel
// moves float4 per thread; otherwise it falls back to one element per thread with the
// offsets rebuilt from the collapsed shape.
#include "common.cuh"

namespace fml {
namespace {

__device__ __forceinline__ float gelu_erf(float t, float c0, float c1, float c2) {
  return t * (erff(t / c0) + c1) * c2;
}

__device__ __forceinline__ float ew_apply(int op, float a, float b, float p0, float p1) {
  switch (op) {
  case FML_ADD: return a + b;
  case FML_MUL: return a * b;
  case FML_DIV: return a / b;
  case FML_SUB: return a - b;
  case FML_POW: return powf(a, b);
  case FML_ADD_SCALAR: return a + p0;
  case FML_MUL_SCALAR: return a * p0;
  case FML_DIV_SCALAR: return a / p0;
  case FML_RSUB_SCALAR: return p0 - a;
  case FML_POW_SCALAR: return powf(a, p0);
  case FML_CLIP: return fminf(fmaxf(a, p0), p1);
  case FML_RSUB_MUL_SCALAR: return (p0 - a) * p1;
  case FML_ERF: return erff(a);
  case FML_TANH: return tanhf(a);
  case FML_SQRT: return sqrtf(a);
  case FML_NEG: return -a;
  case FML_RELU: return fmaxf(a, 0.0f);
  case FML_SIGMOID: return 1.0f / (1.0f + expf(-a));
  case FML_EXP: return expf(a);
  case FML_SILU: return a / (1.0f + expf(-a));
  default: return a;
  }
}

__device__ __forceinline__ int64_t ew_apply_i64(int op, int64_t a, int64_t b, int64_t p0) {
  switch (op) {
  case FML_ADD: return a + b;
  case FML_MUL: return a * b;
  case FML_SUB: return a - b;
  case FML_ADD_SCALAR: return a + p0;
  case FML_MUL_SCALAR: return a * p0;
  case FML_RSUB_SCALAR: return p0 - a;
  default: return a;
  }
}

// operand 0 = out, 1 = a, 2 = b
// I: index type.  Every tensor of a model fits 32-bit offsets, and a 64-bit division costs about
// five times a 32-bit one: with the 64-bit walk the broadcast multiply of EfficientNet's
// squeeze-and-excite blocks issued ~200 instructions per float4 and ran at a fifth of the copy
// bandwidth.  The outermost dim needs no division at all.
template <typename I>
__global__ void ew_f32_generic(Iter<3> it, int op, float *out, const float *a, const float *b,
                               float p0, float p1) {
  pdl_prologue();
  const I total = (I)it.total;
  for (I i = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x; i < total; i += (I)gridDim.x * (I)blockDim.x) {
    I lin = i, off[3] = {0, 0, 0};
    for (int d = it.rank - 1; d >= 0; --d) {
      I c = lin;
      if (d > 0) { const I q = lin / (I)it.shape[d]; c = lin - q * (I)it.shape[d]; lin = q; }
      off[0] += c * (I)it.stride[0][d];
      off[1] += c * (I)it.stride[1][d];
      off[2] += c * (I)it.stride[2][d];
    }
    float bv = b ? b[off[2]] : 0.0f;
    out[off[0]] = ew_apply(op, a[off[1]], bv, p0, p1);
  }
}

// Innermost dim: out stride 1, a/b stride 1 or 0; inner extent a multiple of 4.
template <typename I>
__global__ void ew_f32_vec4(Iter<3> it, int op, float *out, const float *a, const float *b,
                            float p0, float p1) {
  pdl_prologue();
  const I inner4 = (I)(it.shape[it.rank - 1] >> 2);
  const I total4 = (I)(it.total >> 2);
  const bool a_vec = it.stride[1][it.rank - 1] == 1, b_vec = b && it.stride[2][it.rank - 1] == 1;
  const I stride = (I)gridDim.x * (I)blockDim.x;
  // two float4 per thread and step, both loaded before either is used: with one in flight per
  // thread the broadcast forms (a division and a scalar load beside the 16-byte one) ran at a
  // third of the copy bandwidth
  for (I i0 = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x; i0 < total4; i0 += 2 * stride) {
    float4 av[2], bv[2];
    I oo[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const I i = i0 + (I)u * stride;
      live[u] = i < total4;
      bv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      av[u] = bv[u];
      oo[u] = 0;
      if (!live[u]) continue;
      I row = it.rank > 1 ? i / inner4 : 0;
      const I c4 = i - row * inner4;
      I off[3] = {c4 * 4, a_vec ? c4 * 4 : 0, b_vec ? c4 * 4 : 0};
      for (int d = it.rank - 2; d >= 0; --d) {
        I c = row;
        if (d > 0) { const I q = row / (I)it.shape[d]; c = row - q * (I)it.shape[d]; row = q; }
        off[0] += c * (I)it.stride[0][d];
        off[1] += c * (I)it.stride[1][d];
        off[2] += c * (I)it.stride[2][d];
      }
      oo[u] = off[0];
      if (a_vec) av[u] = *reinterpret_cast<const float4 *>(a + off[1]);
      else { float s = a[off[1]]; av[u] = make_float4(s, s, s, s); }
      if (b) {
        if (b_vec) bv[u] = *reinterpret_cast<const float4 *>(b + off[2]);
        else { float s = b[off[2]]; bv[u] = make_float4(s, s, s, s); }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!live[u]) continue;
      float4 r;
      r.x = ew_apply(op, av[u].x, bv[u].x, p0, p1);
      r.y = ew_apply(op, av[u].y, bv[u].y, p0, p1);
      r.z = ew_apply(op, av[u].z, bv[u].z, p0, p1);
      r.w = ew_apply(op, av[u].w, bv[u].w, p0, p1);
      *reinterpret_cast<float4 *>(out + oo[u]) = r;
    }
  }
}


__global__ void ew_i64_generic(Iter<3> it, int op, int64_t *out, const int64_t *a,
                               const int64_t *b, int64_t p0) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    offsets_of(it, i, off);
    out[off[0]] = ew_apply_i64(op, a[off[1]], b ? b[off[2]] : 0, p0);
  }
}

__global__ void ew_equal_i64(Iter<3> it, uint8_t *out, const int64_t *a, const int64_t *b,
                             int64_t p0) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    offsets_of(it, i, off);
    out[off[0]] = a[off[1]] == (b ? b[off[2]] : p0);
  }
}

__global__ void ew_not(Iter<3> it, uint8_t *out, const uint8_t *a) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    offsets_of(it, i, off);
    out[off[0]] = !a[off[1]];
  }
}

template <typename TI, typename TO>
__global__ void ew_cast(Iter<3> it, TO *out, const TI *a) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    offsets_of(it, i, off);
    out[off[0]] = static_cast<TO>(a[off[1]]);
  }
}

// operand 0 = out, 1 = x, 2 = bias
__global__ void bias_gelu_generic(Iter<3> it, float *out, const float *x, const float *bias,
                                  float c0, float c1, float c2) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    offsets_of(it, i, off);
    out[off[0]] = gelu_erf(x[off[1]] + bias[off[2]], c0, c1, c2);
  }
}

// Offsets of the float4 with linear index i when the innermost dim is walked 4 elements at a
// time: operand o advances 4 * c4 elements when its innermost stride is 1, nothing when it is 0.
template <int N>
__device__ __forceinline__ void vec4_offsets(const Iter<N> &it, int64_t i, int64_t inner4, int64_t off[N]) {
  int64_t row = i / inner4;
  const int64_t c4 = i - row * inner4;
#pragma unroll
  for (int o = 0; o < N; ++o) off[o] = it.stride[o][it.rank - 1] == 1 ? c4 * 4 : 0;
  for (int d = it.rank - 2; d >= 0; --d) {
    const int64_t q = row / it.shape[d], c = row - q * it.shape[d];
    row = q;
#pragma unroll
    for (int o = 0; o < N; ++o) off[o] += c * it.stride[o][d];
  }
}

// 16-byte variants of the two kernels above (innermost dim: out stride 1, inputs stride 1 or 0,
// extent a multiple of 4, everything 16-byte aligned).
__global__ void bias_gelu_vec4(Iter<3> it, float *out, const float *x, const float *bias, float c0, float c1, float c2) {
  pdl_prologue();
  const int64_t inner4 = it.shape[it.rank - 1] >> 2, total4 = it.total >> 2;
  const bool x_vec = it.stride[1][it.rank - 1] == 1, b_vec = it.stride[2][it.rank - 1] == 1;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[3];
    vec4_offsets<3>(it, i, inner4, off);
    float4 xv, bv;
    if (x_vec) xv = *reinterpret_cast<const float4 *>(x + off[1]);
    else { const float t = x[off[1]]; xv = make_float4(t, t, t, t); }
    if (b_vec) bv = *reinterpret_cast<const float4 *>(bias + off[2]);
    else { const float t = bias[off[2]]; bv = make_float4(t, t, t, t); }
    *reinterpret_cast<float4 *>(out + off[0]) =
        make_float4(gelu_erf(xv.x + bv.x, c0, c1, c2), gelu_erf(xv.y + bv.y, c0, c1, c2),
                    gelu_erf(xv.z + bv.z, c0, c1, c2), gelu_erf(xv.w + bv.w, c0, c1, c2));
  }
}

__global__ void where_vec4(Iter<4> it, float *out, const uint8_t *cond, const float *x, const float *y, float y_scalar) {
  pdl_prologue();
  const int64_t inner4 = it.shape[it.rank - 1] >> 2, total4 = it.total >> 2;
  const int l = it.rank - 1;
  const bool c_vec = it.stride[1][l] == 1, x_vec = it.stride[2][l] == 1, y_vec = y && it.stride[3][l] == 1;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[4];
    vec4_offsets<4>(it, i, inner4, off);
    uchar4 cv;
    if (c_vec) cv = *reinterpret_cast<const uchar4 *>(cond + off[1]);
    else { const uint8_t t = cond[off[1]]; cv = make_uchar4(t, t, t, t); }
    float4 xv, yv = make_float4(y_scalar, y_scalar, y_scalar, y_scalar);
    if (x_vec) xv = *reinterpret_cast<const float4 *>(x + off[2]);
    else { const float t = x[off[2]]; xv = make_float4(t, t, t, t); }
    if (y) {
      if (y_vec) yv = *reinterpret_cast<const float4 *>(y + off[3]);
      else { const float t = y[off[3]]; yv = make_float4(t, t, t, t); }
    }
    *reinterpret_cast<float4 *>(out + off[0]) =
        make_float4(cv.x ? xv.x : yv.x, cv.y ? xv.y : yv.y, cv.z ? xv.z : yv.z, cv.w ? xv.w : yv.w);
  }
}

// operand 0 = out, 1 = cond, 2 = x, 3 = y
__global__ void where_generic(Iter<4> it, float *out, const uint8_t *cond, const float *x,
                              const float *y, float y_scalar) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[4];
    offsets_of(it, i, off);
    out[off[0]] = cond[off[1]] ? x[off[2]] : (y ? y[off[3]] : y_scalar);
  }
}

template <int N>
int make_iter(Iter<N> &it, const fml_tensor *out, const fml_tensor *const *ins, const char *who) {
  FML_REQUIRE(valid_tensor(out), FML_BAD_ARG, "%s: bad output tensor", who);
  it.rank = out->rank;
  for (int i = 0; i < out->rank; ++i) {
    it.shape[i] = out->shape[i];
    it.stride[0][i] = out->stride[i];
  }
  for (int o = 1; o < N; ++o) {
    if (!ins[o - 1]) {
      for (int i = 0; i < out->rank; ++i) it.stride[o][i] = 0;
      continue;
    }
    FML_REQUIRE(valid_tensor(ins[o - 1]), FML_BAD_ARG, "%s: bad input tensor %d", who, o - 1);
    FML_REQUIRE(broadcast_strides(ins[o - 1], out, it.stride[o]), FML_BAD_ARG,
                "%s: input %d does not broadcast to the output shape", who, o - 1);
  }
  collapse(it);
  return FML_OK;
}

// out = a * b + c, all broadcast to out: the multiply and the add as two IEEE operations (no
// fused multiply-add: the result is what MulCommon followed by AddCommon gives, bit for bit).
__global__ void mul_add_vec4(Iter<4> it, float *out, const float *a, const float *b, const float *c) {
  pdl_prologue();
  const uint32_t inner4 = (uint32_t)(it.shape[it.rank - 1] >> 2), total4 = (uint32_t)(it.total >> 2);
  const int l = it.rank - 1;
  const bool av = it.stride[1][l] == 1, bv = it.stride[2][l] == 1, cv = it.stride[3][l] == 1;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
    uint32_t row = it.rank > 1 ? i / inner4 : 0;
    const uint32_t c4 = i - row * inner4;
    uint32_t off[4] = {c4 * 4, av ? c4 * 4 : 0, bv ? c4 * 4 : 0, cv ? c4 * 4 : 0};
    for (int d = it.rank - 2; d >= 0; --d) {
      uint32_t cc = row;
      if (d > 0) { const uint32_t q = row / (uint32_t)it.shape[d]; cc = row - q * (uint32_t)it.shape[d]; row = q; }
#pragma unroll
      for (int o = 0; o < 4; ++o) off[o] += cc * (uint32_t)it.stride[o][d];
    }
    auto load = [](const float *p, uint32_t o, bool vec) {
      if (vec) return *reinterpret_cast<const float4 *>(p + o);
      const float t = p[o];
      return make_float4(t, t, t, t);
    };
    const float4 x = load(a, off[1], av), y = load(b, off[2], bv), z = load(c, off[3], cv);
    *reinterpret_cast<float4 *>(out + off[0]) =
        make_float4(__fadd_rn(__fmul_rn(x.x, y.x), z.x), __fadd_rn(__fmul_rn(x.y, y.y), z.y),
                    __fadd_rn(__fmul_rn(x.z, y.z), z.z), __fadd_rn(__fmul_rn(x.w, y.w), z.w));
  }
}
__global__ void mul_add_generic(Iter<4> it, float *out, const float *a, const float *b, const float *c) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[4];
    offsets_of(it, i, off);
    out[off[0]] = __fadd_rn(__fmul_rn(a[off[1]], b[off[2]]), c[off[3]]);
  }
}

// out = a0*b0 + a1*b1 + ... + a(n-1)*b(n-1), all broadcast to out, evaluated as the chain of
// MulCommon / AddCommon kernels it replaces: acc = rn(a0*b0); acc = rn(rn(ai*bi) + acc) for
// i = 1 .. n-1 (every product and every sum rounded to fp32, no fused multiply-add), so the result
// is theirs bit for bit.  One pass: every operand read once, nothing written in between.
constexpr int kMaxPairs = 12;
struct PairPtrs { const float *a[kMaxPairs], *b[kMaxPairs]; };

__global__ void sum_products_vec4(Iter<2 * kMaxPairs + 1> it, float *out, PairPtrs ptr, int n) {
  pdl_prologue();
  constexpr int NO = 2 * kMaxPairs + 1;
  const uint32_t inner4 = (uint32_t)(it.shape[it.rank - 1] >> 2), total4 = (uint32_t)(it.total >> 2);
  const int l = it.rank - 1;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
    uint32_t row = it.rank > 1 ? i / inner4 : 0;
    const uint32_t c4 = i - row * inner4;
    uint32_t off[NO];
#pragma unroll
    for (int o = 0; o < NO; ++o) off[o] = it.stride[o][l] == 1 ? c4 * 4 : 0;
    for (int d = it.rank - 2; d >= 0; --d) {
      uint32_t cc = row;
      if (d > 0) { const uint32_t q = row / (uint32_t)it.shape[d]; cc = row - q * (uint32_t)it.shape[d]; row = q; }
#pragma unroll
      for (int o = 0; o < NO; ++o)
        if (o <= 2 * n) off[o] += cc * (uint32_t)it.stride[o][d];
    }
    auto load = [](const float *p, uint32_t o, bool vec) {
      if (vec) return *reinterpret_cast<const float4 *>(p + o);
      const float t = p[o];
      return make_float4(t, t, t, t);
    };
    float4 x[kMaxPairs], y[kMaxPairs];
#pragma unroll
    for (int p = 0; p < kMaxPairs; ++p)
      if (p < n) {
        x[p] = load(ptr.a[p], off[1 + 2 * p], it.stride[1 + 2 * p][l] == 1);
        y[p] = load(ptr.b[p], off[2 + 2 * p], it.stride[2 + 2 * p][l] == 1);
      }
    float4 acc = make_float4(__fmul_rn(x[0].x, y[0].x), __fmul_rn(x[0].y, y[0].y), __fmul_rn(x[0].z, y[0].z), __fmul_rn(x[0].w, y[0].w));
#pragma unroll
    for (int p = 1; p < kMaxPairs; ++p)
      if (p < n) {
        acc.x = __fadd_rn(__fmul_rn(x[p].x, y[p].x), acc.x);
        acc.y = __fadd_rn(__fmul_rn(x[p].y, y[p].y), acc.y);
        acc.z = __fadd_rn(__fmul_rn(x[p].z, y[p].z), acc.z);
        acc.w = __fadd_rn(__fmul_rn(x[p].w, y[p].w), acc.w);
      }
    *reinterpret_cast<float4 *>(out + off[0]) = acc;
  }
}
__global__ void sum_products_generic(Iter<2 * kMaxPairs + 1> it, float *out, PairPtrs ptr, int n) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[2 * kMaxPairs + 1];
    offsets_of(it, i, off);
    float acc = __fmul_rn(ptr.a[0][off[1]], ptr.b[0][off[2]]);
    for (int p = 1; p < n; ++p) acc = __fadd_rn(__fmul_rn(ptr.a[p][off[1 + 2 * p]], ptr.b[p][off[2 + 2 * p]]), acc);
    out[off[0]] = acc;
  }
}

// Rotary position embedding over the first `rot` of D features (GPT-NeoX style halves), the
// operator chain Slice, Slice, Neg, Concat, Mul, Mul, Add, Concat in one pass:
//   j < rot/2        : out[j] = rn(rn(x[j] * cos[j]) + rn(-x[j + rot/2] * sin[j]))
//   rot/2 <= j < rot : out[j] = rn(rn(x[j] * cos[j]) + rn( x[j - rot/2] * sin[j]))
//   j >= rot         : out[j] = x[j]
// with the chain's roundings (two products, one sum, no fused multiply-add): bit-equal to it.
struct RotaryArgs {
  int rank;                 // dims before the feature dim
  int64_t shape[kMaxDims];  // their extents
  int64_t xs[kMaxDims], os[kMaxDims], cs[kMaxDims], ss[kMaxDims];  // element strides of x, out, cos, sin over them
  int64_t x_last, o_last, c_last, s_last;                          // strides along the features
  int64_t rows;
  int D, rot;
  const float *x, *cosv, *sinv;
  float *out;
};
template <int V>  // features per thread: 4 (16-byte accesses) or 1
__global__ void rotary_kernel(const RotaryArgs a) {
  pdl_prologue();
  const int per_row = a.D / V, half = a.rot >> 1;
  const int64_t total = a.rows * per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = i / per_row;
    const int j = (int)(i - row * per_row) * V;
    int64_t xo = 0, oo = 0, co = 0, so = 0;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t q = row / a.shape[d], c = row - q * a.shape[d];
      row = q;
      xo += c * a.xs[d]; oo += c * a.os[d]; co += c * a.cs[d]; so += c * a.ss[d];
    }
    if (V == 4) {
      const float4 xv = *reinterpret_cast<const float4 *>(a.x + xo + j);
      float4 r = xv;
      if (j < a.rot) {
        const int pj = j < half ? j + half : j - half;
        const float sgn = j < half ? -1.0f : 1.0f;
        const float4 pv = *reinterpret_cast<const float4 *>(a.x + xo + pj);
        const float4 cv = *reinterpret_cast<const float4 *>(a.cosv + co + j);
        const float4 sv = *reinterpret_cast<const float4 *>(a.sinv + so + j);
        r.x = __fadd_rn(__fmul_rn(xv.x, cv.x), __fmul_rn(sgn * pv.x, sv.x));
        r.y = __fadd_rn(__fmul_rn(xv.y, cv.y), __fmul_rn(sgn * pv.y, sv.y));
        r.z = __fadd_rn(__fmul_rn(xv.z, cv.z), __fmul_rn(sgn * pv.z, sv.z));
        r.w = __fadd_rn(__fmul_rn(xv.w, cv.w), __fmul_rn(sgn * pv.w, sv.w));
      }
      *reinterpret_cast<float4 *>(a.out + oo + j) = r;
    } else {
      const float xv = a.x[xo + j * a.x_last];
      float r = xv;
      if (j < a.rot) {
        const int pj = j < half ? j + half : j - half;
        const float pv = a.x[xo + pj * a.x_last];
        r = __fadd_rn(__fmul_rn(xv, a.cosv[co + j * a.c_last]), __fmul_rn(j < half ? -pv : pv, a.sinv[so + j * a.s_last]));
      }
      a.out[oo + j * a.o_last] = r;
    }
  }
}

bool vec4_ok(const Iter<3> &it, const void *out, const void *a, const void *b) {
  int l = it.rank - 1;
  if (it.shape[l] % 4 != 0 || it.stride[0][l] != 1) return false;
  if (!aligned16(out) || !aligned16(a) || (b && !aligned16(b))) return false;
  if (it.stride[1][l] != 1 && it.stride[1][l] != 0) return false;
  if (b && it.stride[2][l] != 1 && it.stride[2][l] != 0) return false;
  // outer strides must keep 16-byte alignment only for operands that are read 16 bytes at a time; an
  // operand broadcast along the innermost dim (a per-row scale) is read as one scalar per float4
  for (int d = 0; d < l; ++d)
    for (int o = 0; o < 3; ++o)
      if (it.stride[o][l] != 0 && it.stride[o][d] % 4 != 0) return false;
  return true;
}

}  // namespace
}  // namespace fml

using namespace fml;

extern "C" int fml_elementwise(int op, const fml_tensor *a, const fml_tensor *b,
                               const fml_tensor *out, double p0, double p1, void *stream) {
  FML_REQUIRE(a && out, FML_BAD_ARG, "fml_elementwise: null tensor");
  const bool binary = op <= FML_EQUAL;
  FML_REQUIRE(!binary || b, FML_BAD_ARG, "fml_elementwise: binary op %d needs two inputs", op);
  if (!binary) b = nullptr;
  Iter<3> it;
  const fml_tensor *ins[2] = {a, b};
  int st = make_iter(it, out, ins, "fml_elementwise");
  if (st != FML_OK) return st;
  if (it.total == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  const int block = 256;
  const int grid = grid_for(it.total, block);

  if (op == FML_CAST) {
#define CAST_CASE(TI, CI, TO, CO)                                                          \
  if (a->dtype == CI && out->dtype == CO) {                                                \
    FML_LAUNCH((ew_cast<TI, TO>), grid, block, 0, s, it, (TO *)out->data, (const TI *)a->data);      \
    FML_CUDA(cudaGetLastError());                                                          \
    return FML_OK;                                                                         \
  }
    CAST_CASE(int64_t, FML_I64, float, FML_F32)
    CAST_CASE(int32_t, FML_I32, float, FML_F32)
    CAST_CASE(uint8_t, FML_BOOL, float, FML_F32)
    CAST_CASE(int64_t, FML_I64, int32_t, FML_I32)
    CAST_CASE(int32_t, FML_I32, int64_t, FML_I64)
    CAST_CASE(uint8_t, FML_BOOL, int64_t, FML_I64)
    CAST_CASE(uint8_t, FML_BOOL, int32_t, FML_I32)
    CAST_CASE(float, FML_F32, int64_t, FML_I64)
    CAST_CASE(float, FML_F32, int32_t, FML_I32)
    CAST_CASE(int64_t, FML_I64, int64_t, FML_I64)
    CAST_CASE(float, FML_F32, float, FML_F32)
#undef CAST_CASE
    FML_REQUIRE(false, FML_UNSUPPORTED, "fml_elementwise: cast %d -> %d", a->dtype, out->dtype);
  }
  if (op == FML_COPY) {
    FML_REQUIRE(a->dtype == out->dtype, FML_BAD_ARG, "fml_elementwise: copy changes dtype");
    return fml_copy_strided(a, out, stream);
  }
  if (op == FML_NOT) {
    FML_REQUIRE(a->dtype == FML_BOOL && out->dtype == FML_BOOL, FML_UNSUPPORTED,
                "fml_elementwise: Not takes bool");
    FML_LAUNCH((ew_not), grid, block, 0, s, it, (uint8_t *)out->data, (const uint8_t *)a->data);
    FML_CUDA(cudaGetLastError());
    return FML_OK;
  }
  if (op == FML_EQUAL || op == FML_EQUAL_SCALAR) {
    FML_REQUIRE(a->dtype == FML_I64 && out->dtype == FML_BOOL && (!b || b->dtype == FML_I64),
                FML_UNSUPPORTED, "fml_elementwise: Equal takes int64 and yields bool");
    FML_LAUNCH((ew_equal_i64), grid, block, 0, s, it, (uint8_t *)out->data, (const int64_t *)a->data,
                                        b ? (const int64_t *)b->data : nullptr, (int64_t)p0);
    FML_CUDA(cudaGetLastError());
    return FML_OK;
  }
  FML_REQUIRE(a->dtype == out->dtype && (!b || b->dtype == a->dtype), FML_BAD_ARG,
              "fml_elementwise: operand dtypes differ");
  if (a->dtype == FML_I64) {
    FML_REQUIRE(op == FML_ADD || op == FML_MUL || op == FML_SUB || op == FML_ADD_SCALAR ||
                    op == FML_MUL_SCALAR || op == FML_RSUB_SCALAR,
                FML_UNSUPPORTED, "fml_elementwise: op %d has no int64 kernel", op);
    FML_LAUNCH((ew_i64_generic), grid, block, 0, s, it, op, (int64_t *)out->data, (const int64_t *)a->data,
                                          b ? (const int64_t *)b->data : nullptr, (int64_t)p0);
    FML_CUDA(cudaGetLastError());
    return FML_OK;
  }
  FML_REQUIRE(a->dtype == FML_F32, FML_UNSUPPORTED, "fml_elementwise: dtype %d", a->dtype);
  FML_REQUIRE(op != FML_EQUAL && (op <= FML_POW || (op >= FML_ADD_SCALAR && op <= FML_RSUB_MUL_SCALAR) ||
                                  (op >= FML_ERF && op <= FML_SILU)),
              FML_UNSUPPORTED, "fml_elementwise: unknown op %d", op);
  const float *bp = b ? (const float *)b->data : nullptr;
  // 32-bit index arithmetic whenever every offset (and the grid-stride loop's last step) fits
  bool narrow = it.total < (1ll << 30);
  for (int o = 0; o < 3 && narrow; ++o) {
    int64_t last = 0;
    for (int d = 0; d < it.rank; ++d) {
      if (it.stride[o][d] < 0) narrow = false;
      last += (it.shape[d] - 1) * it.stride[o][d];
    }
    narrow = narrow && last < (1ll << 31) - 8;
  }
  if (vec4_ok(it, out->data, a->data, bp)) {
    if (narrow)
      FML_LAUNCH((ew_f32_vec4<uint32_t>), grid_for(it.total / 4, block), block, 0, s,
                 it, op, (float *)out->data, (const float *)a->data, bp, (float)p0, (float)p1);
    else
      FML_LAUNCH((ew_f32_vec4<int64_t>), grid_for(it.total / 4, block), block, 0, s,
                 it, op, (float *)out->data, (const float *)a->data, bp, (float)p0, (float)p1);
  } else if (narrow) {
    FML_LAUNCH((ew_f32_generic<uint32_t>), grid, block, 0, s, it, op, (float *)out->data, (const float *)a->data, bp,
               (float)p0, (float)p1);
  } else {
    FML_LAUNCH((ew_f32_generic<int64_t>), grid, block, 0, s, it, op, (float *)out->data, (const float *)a->data, bp,
               (float)p0, (float)p1);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_bias_gelu(const fml_tensor *x, const fml_tensor *bias, const fml_tensor *out,
                             float c0, float c1, float c2, void *stream) {
  FML_REQUIRE(x && bias && out, FML_BAD_ARG, "fml_bias_gelu: null tensor");
  FML_REQUIRE(x->dtype == FML_F32 && bias->dtype == FML_F32 && out->dtype == FML_F32,
              FML_UNSUPPORTED, "fml_bias_gelu: fp32 only");
  Iter<3> it;
  const fml_tensor *ins[2] = {x, bias};
  int st = make_iter(it, out, ins, "fml_bias_gelu");
  if (st != FML_OK) return st;
  if (it.total == 0) return FML_OK;
  if (vec4_ok(it, out->data, x->data, (const float *)bias->data))
    FML_LAUNCH((bias_gelu_vec4), grid_for(it.total / 4, 256), 256, 0, as_stream(stream),
        it, (float *)out->data, (const float *)x->data, (const float *)bias->data, c0, c1, c2);
  else
    FML_LAUNCH((bias_gelu_generic), grid_for(it.total, 256), 256, 0, as_stream(stream),
        it, (float *)out->data, (const float *)x->data, (const float *)bias->data, c0, c1, c2);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_where(const fml_tensor *cond, const fml_tensor *x, const fml_tensor *y,
                         float y_scalar, const fml_tensor *out, void *stream) {
  FML_REQUIRE(cond && x && out, FML_BAD_ARG, "fml_where: null tensor");
  FML_REQUIRE(cond->dtype == FML_BOOL && x->dtype == FML_F32 && out->dtype == FML_F32 &&
                  (!y || y->dtype == FML_F32),
              FML_UNSUPPORTED, "fml_where: cond bool, x/y/out fp32");
  Iter<4> it;
  const fml_tensor *ins[3] = {cond, x, y};
  int st = make_iter(it, out, ins, "fml_where");
  if (st != FML_OK) return st;
  if (it.total == 0) return FML_OK;
  {
    // the 16-byte path: out / x / y as for the binary kernels, the condition bytes on 4-byte steps
    const int l = it.rank - 1;
    bool ok = it.rank >= 1 && (it.shape[l] & 3) == 0 && it.stride[0][l] == 1 && aligned16(out->data) && aligned16(x->data) &&
              (!y || aligned16(y->data)) && (reinterpret_cast<uintptr_t>(cond->data) & 3) == 0;
    for (int o = 1; o < 4 && ok; ++o) ok = it.stride[o][l] == 1 || it.stride[o][l] == 0 || (o == 3 && !y);
    for (int d = 0; d < l && ok; ++d)
      for (int o = 0; o < 4; ++o)
        if (it.stride[o][d] % 4 != 0 && !(o == 3 && !y)) ok = false;
    if (ok) {
      FML_LAUNCH((where_vec4), grid_for(it.total / 4, 256), 256, 0, as_stream(stream),
          it, (float *)out->data, (const uint8_t *)cond->data, (const float *)x->data,
          y ? (const float *)y->data : nullptr, y_scalar);
      FML_CUDA(cudaGetLastError());
      return FML_OK;
    }
  }
  FML_LAUNCH((where_generic), grid_for(it.total, 256), 256, 0, as_stream(stream), 
      it, (float *)out->data, (const uint8_t *)cond->data, (const float *)x->data,
      y ? (const float *)y->data : nullptr, y_scalar);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_rotary(const fml_tensor *x, const fml_tensor *cosv, const fml_tensor *sinv, int64_t rot,
                          const fml_tensor *out, void *stream) {
  FML_REQUIRE(valid_tensor(x) && valid_tensor(cosv) && valid_tensor(sinv) && valid_tensor(out), FML_BAD_ARG, "fml_rotary: bad tensor");
  FML_REQUIRE(x->dtype == FML_F32 && cosv->dtype == FML_F32 && sinv->dtype == FML_F32 && out->dtype == FML_F32, FML_UNSUPPORTED,
              "fml_rotary: fp32 only");
  FML_REQUIRE(x->rank >= 1 && out->rank == x->rank && cosv->rank <= x->rank && sinv->rank <= x->rank, FML_BAD_ARG,
              "fml_rotary: ranks");
  const int r = x->rank - 1;
  RotaryArgs a;
  memset(&a, 0, sizeof(a));
  a.D = (int)x->shape[r];
  FML_REQUIRE(rot >= 2 && (rot & 1) == 0 && rot <= a.D && x->shape[r] < (1ll << 30), FML_BAD_ARG,
              "fml_rotary: the rotated width must be even and at most the feature count");
  a.rot = (int)rot;
  a.rank = r;
  a.rows = 1;
  // cos / sin: [..., rot], leading dims broadcast to x's (numpy rules, right-aligned)
  auto lead_strides = [&](const fml_tensor *t, int64_t *st, int64_t *last) {
    if (t->rank < 1 || t->shape[t->rank - 1] != rot) return false;
    *last = t->stride[t->rank - 1];
    for (int i = 0; i < r; ++i) {
      const int ti = i - (x->rank - t->rank);
      if (ti < 0) { st[i] = 0; continue; }
      if (t->shape[ti] == x->shape[i]) st[i] = t->shape[ti] == 1 ? 0 : t->stride[ti];
      else if (t->shape[ti] == 1) st[i] = 0;
      else return false;
    }
    return true;
  };
  for (int i = 0; i <= r; ++i) FML_REQUIRE(out->shape[i] == x->shape[i], FML_BAD_ARG, "fml_rotary: output shape");
  for (int i = 0; i < r; ++i) {
    a.shape[i] = x->shape[i]; a.xs[i] = x->stride[i]; a.os[i] = out->stride[i];
    a.rows *= x->shape[i];
  }
  FML_REQUIRE(lead_strides(cosv, a.cs, &a.c_last) && lead_strides(sinv, a.ss, &a.s_last), FML_BAD_ARG,
              "fml_rotary: cos / sin must be [..., rot] and broadcast to x's leading dims");
  a.x_last = x->stride[r]; a.o_last = out->stride[r];
  a.x = (const float *)x->data; a.cosv = (const float *)cosv->data; a.sinv = (const float *)sinv->data;
  a.out = (float *)out->data;
  if (a.rows == 0 || a.D == 0) return FML_OK;
  bool vec = a.x_last == 1 && a.o_last == 1 && a.c_last == 1 && a.s_last == 1 && (a.D & 3) == 0 && (a.rot & 7) == 0 &&
             aligned16(a.x) && aligned16(a.out) && aligned16(a.cosv) && aligned16(a.sinv);
  for (int i = 0; i < r && vec; ++i) vec = (a.xs[i] & 3) == 0 && (a.os[i] & 3) == 0 && (a.cs[i] & 3) == 0 && (a.ss[i] & 3) == 0;
  const int64_t work = a.rows * (vec ? a.D / 4 : a.D);
  if (vec) FML_LAUNCH((rotary_kernel<4>), grid_for(work, 256), 256, 0, as_stream(stream), a);
  else FML_LAUNCH((rotary_kernel<1>), grid_for(work, 256), 256, 0, as_stream(stream), a);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_sum_of_products(int n, const fml_tensor *const *a, const fml_tensor *const *b, const fml_tensor *out,
                                   void *stream) {
  FML_REQUIRE(a && b && out && n >= 1 && n <= kMaxPairs, FML_BAD_ARG, "fml_sum_of_products: 1 to %d pairs", kMaxPairs);
  FML_REQUIRE(out->dtype == FML_F32, FML_UNSUPPORTED, "fml_sum_of_products: fp32 only");
  constexpr int NO = 2 * kMaxPairs + 1;
  Iter<NO> it;
  const fml_tensor *ins[NO - 1];
  PairPtrs ptr;
  for (int p = 0; p < kMaxPairs; ++p) {
    ins[2 * p] = p < n ? a[p] : nullptr;
    ins[2 * p + 1] = p < n ? b[p] : nullptr;
    if (p < n) {
      FML_REQUIRE(a[p] && b[p] && a[p]->dtype == FML_F32 && b[p]->dtype == FML_F32, FML_BAD_ARG,
                  "fml_sum_of_products: pair %d must be two fp32 tensors", p);
      ptr.a[p] = (const float *)a[p]->data;
      ptr.b[p] = (const float *)b[p]->data;
    } else {
      ptr.a[p] = ptr.b[p] = nullptr;
    }
  }
  int st = make_iter(it, out, ins, "fml_sum_of_products");
  if (st != FML_OK) return st;
  if (it.total == 0) return FML_OK;
  const int l = it.rank - 1;
  bool ok = (it.shape[l] & 3) == 0 && it.stride[0][l] == 1 && aligned16(out->data) && it.total < (1ll << 30);
  for (int o = 1; o <= 2 * n && ok; ++o) {
    ok = (it.stride[o][l] == 1 || it.stride[o][l] == 0) && aligned16(o & 1 ? ptr.a[(o - 1) / 2] : ptr.b[(o - 2) / 2]);
    int64_t last = 0;
    for (int d = 0; d < it.rank && ok; ++d) {
      if (it.stride[o][d] < 0) ok = false;
      last += (it.shape[d] - 1) * it.stride[o][d];
      if (d < l && it.stride[o][l] != 0 && it.stride[o][d] % 4 != 0) ok = false;  // 16-byte rows for vector operands
    }
    ok = ok && last < (1ll << 31) - 8;
  }
  for (int d = 0; d < l && ok; ++d) ok = it.stride[0][d] % 4 == 0 && it.stride[0][d] >= 0;
  if (ok) {
    FML_LAUNCH((sum_products_vec4), grid_for(it.total / 4, 256), 256, 0, as_stream(stream), it, (float *)out->data, ptr, n);
  } else {
    FML_LAUNCH((sum_products_generic), grid_for(it.total, 256), 256, 0, as_stream(stream), it, (float *)out->data, ptr, n);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_mul_add(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c, const fml_tensor *out,
                           void *stream) {
  FML_REQUIRE(a && b && c && out, FML_BAD_ARG, "fml_mul_add: null tensor");
  FML_REQUIRE(a->dtype == FML_F32 && b->dtype == FML_F32 && c->dtype == FML_F32 && out->dtype == FML_F32, FML_UNSUPPORTED,
              "fml_mul_add: fp32 only");
  Iter<4> it;
  const fml_tensor *ins[3] = {a, b, c};
  int st = make_iter(it, out, ins, "fml_mul_add");
  if (st != FML_OK) return st;
  if (it.total == 0) return FML_OK;
  const int l = it.rank - 1;
  bool ok = (it.shape[l] & 3) == 0 && it.stride[0][l] == 1 && aligned16(out->data) && aligned16(a->data) &&
            aligned16(b->data) && aligned16(c->data) && it.total < (1ll << 30);
  for (int o = 1; o < 4 && ok; ++o) {
    ok = it.stride[o][l] == 1 || it.stride[o][l] == 0;
    int64_t last = 0;
    for (int d = 0; d < it.rank && ok; ++d) {
      if (it.stride[o][d] < 0) ok = false;
      last += (it.shape[d] - 1) * it.stride[o][d];
      if (d < l && it.stride[o][l] != 0 && it.stride[o][d] % 4 != 0) ok = false;  // 16-byte rows for vector operands
    }
    ok = ok && last < (1ll << 31) - 8;
  }
  for (int d = 0; d < l && ok; ++d) ok = it.stride[0][d] % 4 == 0 && it.stride[0][d] >= 0;
  if (ok) {
    FML_LAUNCH((mul_add_vec4), grid_for(it.total / 4, 256), 256, 0, as_stream(stream), it, (float *)out->data,
               (const float *)a->data, (const float *)b->data, (const float *)c->data);
  } else {
    FML_LAUNCH((mul_add_generic), grid_for(it.total, 256), 256, 0, as_stream(stream), it, (float *)out->data,
               (const float *)a->data, (const float *)b->data, (const float *)c->data);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}
