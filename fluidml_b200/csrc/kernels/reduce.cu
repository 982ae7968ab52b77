// Row reductions: Softmax (optionally fused with the attention-score divide and mask add),
// LayerNormalization (optionally fused with the residual add), ReduceMean, CumSum.
//
// HBM-bound.  One warp owns one row; when the reduced axis is contiguous and a multiple of
// four floats the row is read once with 16-byte loads and kept in registers for the
// max/sum (softmax) or mean/variance (LayerNorm) passes, then written once.  Reductions
// use warp shuffles only; no shared memory and no scratch buffer is needed.
#include "common.cuh"

namespace fml {
namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Row iteration: operand 0 = out, 1 = in, 2 = aux0 (mask / residual).  The reduced axis is
// removed from `rows`; its extent and per-operand strides are passed separately.
struct RowArgs {
  Iter<3> rows;
  int64_t len;
  int64_t axis_stride[3];
};

// ---- softmax -----------------------------------------------------------------------
template <int NV>  // float4 per lane
__global__ void softmax_rows_vec(RowArgs a, float *out, const float *in, const float *mask,
                                 float divisor) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (row >= a.rows.total) return;
  int64_t off[3];
  offsets_of(a.rows, row, off);
  const int64_t n4 = a.len >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(in + off[1]);
  const bool mvec = mask && a.axis_stride[2] == 1;
  const ExactDivisor div(divisor);
  float4 v[NV];
  float mx = -3.402823466e+38f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int64_t c = lane + 32 * i;
    if (c < n4) {
      float4 t = x4[c];
      if (divisor != 1.0f) { t.x = div(t.x); t.y = div(t.y); t.z = div(t.z); t.w = div(t.w); }
      if (mask) {
        float4 m;
        if (mvec) m = *reinterpret_cast<const float4 *>(mask + off[2] + c * 4);
        else { float s = mask[off[2]]; m = make_float4(s, s, s, s); }
        t.x += m.x; t.y += m.y; t.z += m.z; t.w += m.w;
      }
      v[i] = t;
      mx = fmaxf(mx, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
    }
  }
  mx = warp_max(mx);
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < n4) {
      v[i].x = expf(v[i].x - mx); v[i].y = expf(v[i].y - mx);
      v[i].z = expf(v[i].z - mx); v[i].w = expf(v[i].w - mx);
      sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  sum = warp_sum(sum);
  // one correctly rounded reciprocal per row, then multiplies: within 1.5 ulp of the division
  const float inv = 1.0f / sum;
  float4 *y4 = reinterpret_cast<float4 *>(out + off[0]);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int64_t c = lane + 32 * i;
    if (c < n4) y4[c] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
  }
}

__global__ void softmax_rows_generic(RowArgs a, float *out, const float *in, const float *mask,
                                     float divisor) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (row >= a.rows.total) return;
  int64_t off[3];
  offsets_of(a.rows, row, off);
  const ExactDivisor div(divisor);
  auto load = [&](int64_t c) {
    float t = in[off[1] + c * a.axis_stride[1]];
    if (divisor != 1.0f) t = div(t);
    if (mask) t += mask[off[2] + c * a.axis_stride[2]];
    return t;
  };
  float mx = -3.402823466e+38f;
  for (int64_t c = lane; c < a.len; c += 32) mx = fmaxf(mx, load(c));
  mx = warp_max(mx);
  float sum = 0.0f;
  for (int64_t c = lane; c < a.len; c += 32) sum += expf(load(c) - mx);
  sum = warp_sum(sum);
  for (int64_t c = lane; c < a.len; c += 32)
    out[off[0] + c * a.axis_stride[0]] = expf(load(c) - mx) / sum;
}

// ---- LayerNorm ---------------------------------------------------------------------
// EARLY: for a few rows (a latency-bound launch) gamma and beta are fetched together with the
// row instead of after the two reductions, so that their latency overlaps the row's; with many
// rows the 8 * NV extra registers would cost occupancy and the vectors are cache hits anyway.
template <int NV, bool EARLY>
__global__ void layernorm_rows_vec(RowArgs a, float *out, const float *in, const float *res,
                                   const float *gamma, const float *beta, float eps) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int64_t n4 = a.len >> 2;
  const float4 *g4 = reinterpret_cast<const float4 *>(gamma), *b4 = reinterpret_cast<const float4 *>(beta);
  // While the preceding kernel drains: pull gamma and beta (weights: cold in a pass that
  // streams more weights than L2 holds) into L2.  A prefetch reads nothing into the SM, so it
  // is harmless even when that kernel is still producing them.
  if (blockIdx.x == 0 && threadIdx.x < 32) {
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + 32 * i < n4) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(g4 + lane + 32 * i));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(b4 + lane + 32 * i));
      }
  }
  pdl_wait();
  const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (row >= a.rows.total) return;
  int64_t off[3];
  offsets_of(a.rows, row, off);
  const float4 *x4 = reinterpret_cast<const float4 *>(in + off[1]);
  const float4 *r4 = res ? reinterpret_cast<const float4 *>(res + off[2]) : nullptr;
  float4 v[NV];
  float4 ge[EARLY ? NV : 1], be[EARLY ? NV : 1];
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int64_t c = lane + 32 * i;
    if (c < n4) {
      float4 t = x4[c];
      if (r4) { float4 r = r4[c]; t.x += r.x; t.y += r.y; t.z += r.z; t.w += r.w; }
      if (EARLY) { ge[EARLY ? i : 0] = g4[c]; be[EARLY ? i : 0] = b4[c]; }
      v[i] = t;
      s += (t.x + t.y) + (t.z + t.w);
    }
  }
  const float mean = warp_sum(s) / (float)a.len;
  float q = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < n4) {
      v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
      q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
  }
  const float var = warp_sum(q) / (float)a.len;
  const float inv = 1.0f / sqrtf(var + eps);
  float4 *y4 = reinterpret_cast<float4 *>(out + off[0]);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    int64_t c = lane + 32 * i;
    if (c < n4) {
      const float4 g = EARLY ? ge[EARLY ? i : 0] : g4[c], b = EARLY ? be[EARLY ? i : 0] : b4[c];
      y4[c] = make_float4(v[i].x * inv * g.x + b.x, v[i].y * inv * g.y + b.y,
                          v[i].z * inv * g.z + b.z, v[i].w * inv * g.w + b.w);
    }
  }
}

__global__ void layernorm_rows_generic(RowArgs a, float *out, const float *in, const float *res,
                                       const float *gamma, int64_t gstride, const float *beta,
                                       int64_t bstride, float eps) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t row = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (row >= a.rows.total) return;
  int64_t off[3];
  offsets_of(a.rows, row, off);
  auto load = [&](int64_t c) {
    float t = in[off[1] + c * a.axis_stride[1]];
    if (res) t += res[off[2] + c * a.axis_stride[2]];
    return t;
  };
  float s = 0.0f;
  for (int64_t c = lane; c < a.len; c += 32) s += load(c);
  const float mean = warp_sum(s) / (float)a.len;
  float q = 0.0f;
  for (int64_t c = lane; c < a.len; c += 32) { float d = load(c) - mean; q += d * d; }
  const float inv = 1.0f / sqrtf(warp_sum(q) / (float)a.len + eps);
  for (int64_t c = lane; c < a.len; c += 32)
    out[off[0] + c * a.axis_stride[0]] = (load(c) - mean) * inv * gamma[c * gstride] + beta[c * bstride];
}

// ---- ReduceMean / CumSum -------------------------------------------------------------
struct ReduceArgs {
  Iter<2> keep;    // over the output shape: operand 0 = out, 1 = in (reduced axes stride 0 in out view)
  int rrank;
  int64_t rshape[kMaxDims], rstride[kMaxDims];
  int64_t count;
};

__global__ void reduce_mean_kernel(ReduceArgs a, float *out, const float *in) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t o = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (o >= a.keep.total) return;
  int64_t off[2];
  offsets_of(a.keep, o, off);
  float s = 0.0f;
  for (int64_t r = lane; r < a.count; r += 32) {
    int64_t l = r, io = off[1];
    for (int d = a.rrank - 1; d >= 0; --d) {
      int64_t q = l / a.rshape[d];
      io += (l - q * a.rshape[d]) * a.rstride[d];
      l = q;
    }
    s += in[io];
  }
  s = warp_sum(s);
  if (lane == 0) out[off[0]] = s / (float)a.count;
}

// The reduced dims form one contiguous run of `count` floats (a global average pool over
// H x W in NCHW): one CTA per output, 16-byte loads when the run is aligned, shuffle + shared
// memory reduction in a fixed order.
__global__ void __launch_bounds__(256) reduce_mean_contig_kernel(ReduceArgs a, float *out, const float *in) {
  pdl_prologue();
  __shared__ float part[8];
  const int64_t o = blockIdx.x;
  int64_t off[2];
  offsets_of(a.keep, o, off);
  const float *src = in + off[1];
  float s = 0.0f;
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int64_t n4 = a.count >> 2;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    for (int64_t i = threadIdx.x; i < n4; i += 256) {
      const float4 v = s4[i];
      s += (v.x + v.y) + (v.z + v.w);
    }
    for (int64_t i = (n4 << 2) + threadIdx.x; i < a.count; i += 256) s += src[i];
  } else {
    for (int64_t i = threadIdx.x; i < a.count; i += 256) s += src[i];
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
    for (int w = 0; w < 8; ++w) t += part[w];
    out[off[0]] = t / (float)a.count;
  }
}

// The same contiguous run, one WARP per output: for runs of a few thousand floats or fewer (the
// squeeze-and-excite pools over 56 x 56 ... 7 x 7 planes) a CTA per output spends more on its
// set-up and barrier than on the run.  Lanes take 16-byte pieces when the run is aligned and a
// multiple of four long; the sum order is fixed (lane-strided, then the shuffle tree).
__global__ void __launch_bounds__(256) reduce_mean_rows_kernel(ReduceArgs a, float *out, const float *in) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t o = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (o >= a.keep.total) return;
  int64_t off[2];
  offsets_of(a.keep, o, off);
  const float *src = in + off[1];
  const int count = (int)a.count;
  float s = 0.0f;
  if ((count & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    const int n4 = count >> 2;
    float t0 = 0.0f, t1 = 0.0f;  // two chains: the loads of consecutive pieces overlap
    int i = lane;
    for (; i + 32 < n4; i += 64) {
      const float4 u = s4[i], v = s4[i + 32];
      t0 += (u.x + u.y) + (u.z + u.w);
      t1 += (v.x + v.y) + (v.z + v.w);
    }
    if (i < n4) { const float4 u = s4[i]; t0 += (u.x + u.y) + (u.z + u.w); }
    s = t0 + t1;
  } else {
    for (int i = lane; i < count; i += 32) s += src[i];
  }
  s = warp_sum(s);
  if (lane == 0) out[off[0]] = s / (float)a.count;
}

__global__ void cumsum_kernel(RowArgs a, int64_t *out, const int64_t *in) {
  pdl_prologue();
  const int64_t row = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (row >= a.rows.total) return;
  int64_t off[3];
  offsets_of(a.rows, row, off);
  int64_t s = 0;
  for (int64_t c = 0; c < a.len; ++c) {
    s += in[off[1] + c * a.axis_stride[1]];
    out[off[0] + c * a.axis_stride[0]] = s;
  }
}

int make_rows(RowArgs &a, const fml_tensor *out, const fml_tensor *in, const fml_tensor *aux,
              int axis, const char *who) {
  FML_REQUIRE(valid_tensor(in) && valid_tensor(out), FML_BAD_ARG, "%s: bad tensor", who);
  FML_REQUIRE(in->rank == out->rank && in->rank >= 1, FML_BAD_ARG, "%s: rank mismatch", who);
  if (axis < 0) axis += in->rank;
  FML_REQUIRE(axis >= 0 && axis < in->rank, FML_BAD_ARG, "%s: axis out of range", who);
  for (int i = 0; i < in->rank; ++i)
    FML_REQUIRE(in->shape[i] == out->shape[i], FML_BAD_ARG, "%s: shape mismatch", who);
  int64_t aux_stride[kMaxDims] = {0};
  if (aux) {
    FML_REQUIRE(valid_tensor(aux) && aux->dtype == in->dtype, FML_BAD_ARG, "%s: bad auxiliary tensor", who);
    FML_REQUIRE(broadcast_strides(aux, in, aux_stride), FML_BAD_ARG,
                "%s: auxiliary tensor does not broadcast to the input", who);
  }
  a.len = in->shape[axis];
  a.axis_stride[0] = out->stride[axis];
  a.axis_stride[1] = in->stride[axis];
  a.axis_stride[2] = aux_stride[axis];
  a.rows.rank = in->rank;
  for (int i = 0; i < in->rank; ++i) {
    a.rows.shape[i] = i == axis ? 1 : in->shape[i];
    a.rows.stride[0][i] = out->stride[i];
    a.rows.stride[1][i] = in->stride[i];
    a.rows.stride[2][i] = aux_stride[i];
  }
  collapse(a.rows);
  return FML_OK;
}

bool rows_vec_ok(const RowArgs &a, const void *out, const void *in, const void *aux) {
  if (a.len % 4 != 0 || a.len > 4096) return false;
  if (a.axis_stride[0] != 1 || a.axis_stride[1] != 1) return false;
  if (aux && a.axis_stride[2] != 1 && a.axis_stride[2] != 0) return false;
  if (!aligned16(out) || !aligned16(in) || (aux && !aligned16(aux))) return false;
  for (int d = 0; d < a.rows.rank; ++d)
    for (int o = 0; o < 3; ++o)
      if (a.rows.stride[o][d] % 4 != 0) return false;
  return true;
}

}  // namespace
}  // namespace fml

using namespace fml;

#define DISPATCH_NV(len, KERNEL, grid, stream, ...)                                        \
  do {                                                                                     \
    int64_t per_lane = ((len) / 4 + 31) / 32;                                              \
    if (per_lane <= 1) FML_LAUNCH((KERNEL<1>), grid, 256, 0, stream, __VA_ARGS__);         \
    else if (per_lane <= 2) FML_LAUNCH((KERNEL<2>), grid, 256, 0, stream, __VA_ARGS__);    \
    else if (per_lane <= 4) FML_LAUNCH((KERNEL<4>), grid, 256, 0, stream, __VA_ARGS__);    \
    else if (per_lane <= 8) FML_LAUNCH((KERNEL<8>), grid, 256, 0, stream, __VA_ARGS__);    \
    else if (per_lane <= 16) FML_LAUNCH((KERNEL<16>), grid, 256, 0, stream, __VA_ARGS__);  \
    else FML_LAUNCH((KERNEL<32>), grid, 256, 0, stream, __VA_ARGS__);                      \
  } while (0)

// The same ladder for a kernel family named through a macro K(NV).
#define DISPATCH_NV_FN(per_lane, K, grid, stream, ...)                                     \
  do {                                                                                     \
    if ((per_lane) <= 1) FML_LAUNCH((K(1)), grid, 256, 0, stream, __VA_ARGS__);            \
    else if ((per_lane) <= 2) FML_LAUNCH((K(2)), grid, 256, 0, stream, __VA_ARGS__);       \
    else if ((per_lane) <= 4) FML_LAUNCH((K(4)), grid, 256, 0, stream, __VA_ARGS__);       \
    else if ((per_lane) <= 8) FML_LAUNCH((K(8)), grid, 256, 0, stream, __VA_ARGS__);       \
    else if ((per_lane) <= 16) FML_LAUNCH((K(16)), grid, 256, 0, stream, __VA_ARGS__);     \
    else FML_LAUNCH((K(32)), grid, 256, 0, stream, __VA_ARGS__);                           \
  } while (0)

extern "C" int fml_softmax(const fml_tensor *in, const fml_tensor *mask, float divisor,
                           const fml_tensor *out, int axis, void *stream) {
  FML_REQUIRE(in && out, FML_BAD_ARG, "fml_softmax: null tensor");
  FML_REQUIRE(in->dtype == FML_F32 && out->dtype == FML_F32, FML_UNSUPPORTED, "fml_softmax: fp32 only");
  FML_REQUIRE(divisor != 0.0f, FML_BAD_ARG, "fml_softmax: divisor is zero");
  RowArgs a;
  int st = make_rows(a, out, in, mask, axis, "fml_softmax");
  if (st != FML_OK) return st;
  if (a.rows.total == 0 || a.len == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  const unsigned grid = (unsigned)((a.rows.total * 32 + 255) / 256);
  const float *mp = mask ? (const float *)mask->data : nullptr;
  if (rows_vec_ok(a, out->data, in->data, mp)) {
    DISPATCH_NV(a.len, softmax_rows_vec, grid, s, a, (float *)out->data, (const float *)in->data, mp, divisor);
  } else {
    FML_LAUNCH((softmax_rows_generic), grid, 256, 0, s, a, (float *)out->data, (const float *)in->data, mp, divisor);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_layernorm(const fml_tensor *in, const fml_tensor *residual,
                             const fml_tensor *scale, const fml_tensor *bias, const fml_tensor *out,
                             int axis, float eps, void *stream) {
  FML_REQUIRE(in && out && scale && bias, FML_BAD_ARG, "fml_layernorm: null tensor");
  FML_REQUIRE(in->dtype == FML_F32 && out->dtype == FML_F32 && scale->dtype == FML_F32 &&
                  bias->dtype == FML_F32, FML_UNSUPPORTED, "fml_layernorm: fp32 only");
  RowArgs a;
  int st = make_rows(a, out, in, residual, axis, "fml_layernorm");
  if (st != FML_OK) return st;
  FML_REQUIRE(valid_tensor(scale) && valid_tensor(bias) && numel(scale) == a.len && numel(bias) == a.len,
              FML_BAD_ARG, "fml_layernorm: scale/bias must hold one value per normalised element");
  if (a.rows.total == 0 || a.len == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  const unsigned grid = (unsigned)((a.rows.total * 32 + 255) / 256);
  const float *rp = residual ? (const float *)residual->data : nullptr;
  // stride of the (single) non-unit dim of scale / bias
  auto vec_stride = [](const fml_tensor *t) {
    for (int i = 0; i < t->rank; ++i) if (t->shape[i] != 1) return t->stride[i];
    return (int64_t)1;
  };
  const int64_t gs = vec_stride(scale), bs = vec_stride(bias);
  const bool res_vec = !residual || a.axis_stride[2] == 1;
  if (rows_vec_ok(a, out->data, in->data, rp) && res_vec && gs == 1 && bs == 1 &&
      aligned16(scale->data) && aligned16(bias->data)) {
#define LN_EARLY(NV) layernorm_rows_vec<NV, true>
#define LN_LATE(NV) layernorm_rows_vec<NV, false>
    const int64_t per_lane = (a.len / 4 + 31) / 32;
    if (a.rows.total <= 4096 && per_lane <= 8)
      DISPATCH_NV_FN(per_lane, LN_EARLY, grid, s, a, (float *)out->data, (const float *)in->data, rp, (const float *)scale->data, (const float *)bias->data, eps);
    else
      DISPATCH_NV_FN(per_lane, LN_LATE, grid, s, a, (float *)out->data, (const float *)in->data, rp, (const float *)scale->data, (const float *)bias->data, eps);
#undef LN_EARLY
#undef LN_LATE
  } else {
    FML_LAUNCH((layernorm_rows_generic), grid, 256, 0, s, a, (float *)out->data, (const float *)in->data, rp,
                                                (const float *)scale->data, gs,
                                                (const float *)bias->data, bs, eps);
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_reduce_mean(const fml_tensor *in, const fml_tensor *out, const int32_t *reduce,
                               void *stream) {
  FML_REQUIRE(valid_tensor(in) && valid_tensor(out) && reduce, FML_BAD_ARG, "fml_reduce_mean: bad argument");
  FML_REQUIRE(in->dtype == FML_F32 && out->dtype == FML_F32 && in->rank == out->rank, FML_BAD_ARG,
              "fml_reduce_mean: fp32, keepdims layout");
  ReduceArgs a;
  a.keep.rank = in->rank;
  a.rrank = 0;
  a.count = 1;
  for (int i = 0; i < in->rank; ++i) {
    if (reduce[i]) {
      FML_REQUIRE(out->shape[i] == 1, FML_BAD_ARG, "fml_reduce_mean: reduced dims must be 1 in the output");
      a.keep.shape[i] = 1;
      a.keep.stride[0][i] = 0;
      a.keep.stride[1][i] = 0;
      a.rshape[a.rrank] = in->shape[i];
      a.rstride[a.rrank++] = in->stride[i];
      a.count *= in->shape[i];
    } else {
      FML_REQUIRE(out->shape[i] == in->shape[i], FML_BAD_ARG, "fml_reduce_mean: shape mismatch");
      a.keep.shape[i] = in->shape[i];
      a.keep.stride[0][i] = out->stride[i];
      a.keep.stride[1][i] = in->stride[i];
    }
  }
  collapse(a.keep);
  if (a.keep.total == 0 || a.count == 0) return FML_OK;
  // contiguous run? (reduced dims in memory order, each stride = the product of the later extents)
  bool contig = a.rrank > 0;
  {
    int64_t expect = 1;
    for (int d = a.rrank - 1; d >= 0 && contig; --d) {
      if (a.rshape[d] != 1 && a.rstride[d] != expect) contig = false;
      expect *= a.rshape[d];
    }
  }
  if (contig && a.count < 8192 && a.keep.total * 32 < (1ll << 40)) {
    FML_LAUNCH((reduce_mean_rows_kernel), (unsigned)((a.keep.total * 32 + 255) / 256), 256, 0, as_stream(stream), a,
               (float *)out->data, (const float *)in->data);
    return FML_OK;
  }
  if (contig && a.count >= 256 && a.keep.total <= 0x7fffffff) {
    FML_LAUNCH((reduce_mean_contig_kernel), (unsigned)a.keep.total, 256, 0, as_stream(stream), a, (float *)out->data,
               (const float *)in->data);
    return FML_OK;
  }
  FML_LAUNCH((reduce_mean_kernel), (unsigned)((a.keep.total * 32 + 255) / 256), 256, 0, as_stream(stream), 
      a, (float *)out->data, (const float *)in->data);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_cumsum(const fml_tensor *in, const fml_tensor *out, int axis, void *stream) {
  FML_REQUIRE(in && out, FML_BAD_ARG, "fml_cumsum: null tensor");
  FML_REQUIRE(in->dtype == FML_I64 && out->dtype == FML_I64, FML_UNSUPPORTED, "fml_cumsum: int64 only");
  RowArgs a;
  int st = make_rows(a, out, in, nullptr, axis, "fml_cumsum");
  if (st != FML_OK) return st;
  if (a.rows.total == 0) return FML_OK;
  FML_LAUNCH((cumsum_kernel), grid_for(a.rows.total, 128, 1 << 20), 128, 0, as_stream(stream), 
      a, (int64_t *)out->data, (const int64_t *)in->data);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}
