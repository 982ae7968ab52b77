/*
 * CPU oracle for the FluidML operator hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of what each reference kernel computes
 * (src/structure/kernel/kernel/<op>.cpp of sgjzfzzf/FluidML).  The reference emits MLIR
 * linalg.generic ops that LLVM turns into scalar single-thread loop nests over strided
 * memrefs; the loops below are those loop nests written by hand, one full pass per
 * generic op, fp32 storage, and the same libm calls the reference lowers to
 * (src/worker/lower.cpp:45).  Nothing in the shipped library links or calls this file:
 * it is the checker for the CUDA kernels and the timed CPU baseline.
 *
 * Parity status: the reference stores no golden vectors for these operators (its node
 * tests compare against onnxruntime on unseeded inputs, test/python/node/node_test.py), so
 * the arithmetic here is pinned to ONNX operator semantics by cross-checks against torch
 * CPU (committed fixtures under tests/golden) and is otherwise "parity unpinned" against
 * the reference binary, which cannot be built without LLVM/MLIR 18.  Where the reference
 * departs from ONNX (Gemm alpha/beta placement, Conv strides/dilations/bias, LayerNorm
 * scratch initialisation, Pad border) this file follows ONNX; each place says so.
 *
 * Every tensor is (data, dtype, rank, shape[], stride[]) with strides in ELEMENTS, which
 * is how the reference addresses every operand (layout permutation -> strides,
 * src/utils/utils.cpp:64-102).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_RANK 8
enum { ORC_F32 = 1, ORC_I32 = 6, ORC_I64 = 7, ORC_BOOL = 9 };

typedef struct {
  void *data;
  int32_t dtype;
  int32_t rank;
  int64_t shape[ORC_MAX_RANK];
  int64_t stride[ORC_MAX_RANK];
} orc_tensor;

static int64_t numel(const orc_tensor *t) {
  int64_t n = 1;
  for (int i = 0; i < t->rank; ++i) n *= t->shape[i];
  return n;
}

/* Unravel a row-major linear index over `shape` (rank r) into idx[]. */
static void unravel(int64_t lin, const int64_t *shape, int r, int64_t *idx) {
  for (int i = r - 1; i >= 0; --i) {
    idx[i] = lin % shape[i];
    lin /= shape[i];
  }
}

/* Offset of a logical index of the OUTPUT shape inside operand t, numpy broadcasting:
 * right-aligned, size-1 dims pinned to index 0
 * (src/structure/kernel/kernel/utils.cpp:15-51). */
static int64_t bcast_offset(const orc_tensor *t, const int64_t *idx, int out_rank) {
  int64_t off = 0;
  for (int i = 0; i < t->rank; ++i) {
    int oi = out_rank - t->rank + i;
    int64_t v = t->shape[i] == 1 ? 0 : idx[oi];
    off += v * t->stride[i];
  }
  return off;
}

static int64_t offset_of(const orc_tensor *t, const int64_t *idx) {
  int64_t off = 0;
  for (int i = 0; i < t->rank; ++i) off += idx[i] * t->stride[i];
  return off;
}

static size_t esize(int dtype) {
  switch (dtype) {
  case ORC_F32: case ORC_I32: return 4;
  case ORC_I64: return 8;
  default: return 1;
  }
}

/* ------------------------------------------------------------------ elementwise binary
 * add.cpp:83-124, mul.cpp:56-99, div.cpp:70-105, sub.cpp:71-99 (Common variants) and the
 * scalar-constant variants add.cpp:22-79, mul.cpp:19-54, div.cpp:18-66, sub.cpp:16-67:
 * a scalar constant is passed here as a rank-0 tensor.  Division is a true divide. */
enum { ORC_ADD = 0, ORC_MUL = 1, ORC_DIV = 2, ORC_SUB = 3, ORC_POW = 4, ORC_EQUAL = 5 };

int orc_binary(int op, const orc_tensor *a, const orc_tensor *b, orc_tensor *out) {
  int64_t n = numel(out), idx[ORC_MAX_RANK];
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int64_t oa = bcast_offset(a, idx, out->rank), ob = bcast_offset(b, idx, out->rank),
            oo = offset_of(out, idx);
    if (op == ORC_EQUAL) { /* equal.cpp:14-51, int64 == scalar -> bool */
      ((uint8_t *)out->data)[oo] = ((int64_t *)a->data)[oa] == ((int64_t *)b->data)[ob];
    } else if (out->dtype == ORC_F32) {
      float x = ((float *)a->data)[oa], y = ((float *)b->data)[ob], r;
      switch (op) {
      case ORC_ADD: r = x + y; break;
      case ORC_MUL: r = x * y; break;
      case ORC_DIV: r = x / y; break;
      case ORC_SUB: r = x - y; break;
      case ORC_POW: r = powf(x, y); break; /* pow.cpp:15-61 */
      default: return 1;
      }
      ((float *)out->data)[oo] = r;
    } else if (out->dtype == ORC_I64) {
      int64_t x = ((int64_t *)a->data)[oa], y = ((int64_t *)b->data)[ob], r;
      switch (op) {
      case ORC_ADD: r = x + y; break;
      case ORC_MUL: r = x * y; break;
      case ORC_SUB: r = x - y; break;
      default: return 1;
      }
      ((int64_t *)out->data)[oo] = r;
    } else {
      return 1;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ elementwise unary
 * erf.cpp:18-45, tanh.cpp:12-40, sqrt.cpp:13-36, neg.cpp:17-40, relu.cpp:12-46,
 * clip.cpp:13-48, not.cpp:11-41, dropout.cpp:13-33 (identity).  Sigmoid has no reference
 * kernel (the parser rejects the op, parser.cpp:320-326): ONNX semantics. */
enum { ORC_ERF = 0, ORC_TANH, ORC_SQRT, ORC_NEG, ORC_RELU, ORC_SIGMOID, ORC_CLIP,
       ORC_NOT, ORC_IDENTITY, ORC_EXP };

int orc_unary(int op, const orc_tensor *in, orc_tensor *out, float p0, float p1) {
  int64_t n = numel(out), idx[ORC_MAX_RANK];
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int64_t oi = offset_of(in, idx), oo = offset_of(out, idx);
    if (op == ORC_NOT) {
      ((uint8_t *)out->data)[oo] = !((uint8_t *)in->data)[oi];
      continue;
    }
    if (op == ORC_IDENTITY) {
      memcpy((char *)out->data + oo * esize(out->dtype),
             (char *)in->data + oi * esize(in->dtype), esize(in->dtype));
      continue;
    }
    float x = ((float *)in->data)[oi], r;
    switch (op) {
    case ORC_ERF: r = erff(x); break;
    case ORC_TANH: r = tanhf(x); break;
    case ORC_SQRT: r = sqrtf(x); break;
    case ORC_NEG: r = -x; break;
    case ORC_RELU: r = fmaxf(x, 0.0f); break;
    case ORC_SIGMOID: r = 1.0f / (1.0f + expf(-x)); break;
    case ORC_CLIP: r = fminf(fmaxf(x, p0), p1); break;
    case ORC_EXP: r = expf(x); break;
    default: return 1;
    }
    ((float *)out->data)[oo] = r;
  }
  return 0;
}

/* cast.cpp:12-62: integer/bool -> integer (zero-extend for bool); plus int -> f32 which
 * ONNX allows and the transformer exports use. */
int orc_cast(const orc_tensor *in, orc_tensor *out) {
  int64_t n = numel(out), idx[ORC_MAX_RANK];
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int64_t oi = offset_of(in, idx), oo = offset_of(out, idx);
    double v;
    switch (in->dtype) {
    case ORC_F32: v = ((float *)in->data)[oi]; break;
    case ORC_I32: v = ((int32_t *)in->data)[oi]; break;
    case ORC_I64: v = (double)((int64_t *)in->data)[oi]; break;
    default: v = ((uint8_t *)in->data)[oi]; break;
    }
    switch (out->dtype) {
    case ORC_F32: ((float *)out->data)[oo] = (float)v; break;
    case ORC_I32: ((int32_t *)out->data)[oo] = (int32_t)v; break;
    case ORC_I64: ((int64_t *)out->data)[oo] = (int64_t)v; break;
    default: ((uint8_t *)out->data)[oo] = v != 0; break;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ MatMul
 * matmul.cpp:28-59 + utils.cpp:62-146: zero-fill, then c += a*b over the last two dims,
 * leading dims broadcast.  `order` 0 = i-j-k (the reference default, matmul.cpp:19),
 * 1 = i-k-j (one of the orders its generator autotunes over,
 * generator/matmul.cpp:88-131).  Both accumulate every c[i][j] sequentially in k, so
 * they give the same bits; i-k-j is only faster.  `acc64` accumulates in double, giving a
 * summation-order-independent target. */
/* Rows of the product are independent, so they may be spread over host threads without
 * changing a single bit (each row keeps its k order); orc_set_threads(n) sets how many
 * (default 1: the reference executes single-threaded; the benchmark's CPU arm uses them all). */
static int orc_threads = 1;
void orc_set_threads(int n) { orc_threads = n < 1 ? 1 : n; }

int orc_matmul(const orc_tensor *a, const orc_tensor *b, orc_tensor *c, int order, int acc64) {
  int r = c->rank;
  int64_t M = c->shape[r - 2], N = c->shape[r - 1], K = a->shape[a->rank - 1];
  int64_t batch = 1, idx[ORC_MAX_RANK];
  for (int i = 0; i < r - 2; ++i) batch *= c->shape[i];
  int64_t sam = a->stride[a->rank - 2], sak = a->stride[a->rank - 1];
  int64_t sbk = b->stride[b->rank - 2], sbn = b->stride[b->rank - 1];
  int64_t scm = c->stride[r - 2], scn = c->stride[r - 1];
  for (int64_t bi = 0; bi < batch; ++bi) {
    unravel(bi, c->shape, r - 2, idx);
    int64_t oa = 0, ob = 0, oc = 0;
    for (int i = 0; i < r - 2; ++i) {
      int ia = i - (r - a->rank), ib = i - (r - b->rank);
      if (ia >= 0 && a->shape[ia] != 1) oa += idx[i] * a->stride[ia];
      if (ib >= 0 && b->shape[ib] != 1) ob += idx[i] * b->stride[ib];
      oc += idx[i] * c->stride[i];
    }
    const float *A = (const float *)a->data + oa, *B = (const float *)b->data + ob;
    float *C = (float *)c->data + oc;
#pragma omp parallel num_threads(orc_threads) if (orc_threads > 1)
    {
    double *acc = acc64 ? (double *)malloc(sizeof(double) * (size_t)N) : NULL;
#pragma omp for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
      if (acc64) {
        for (int64_t j = 0; j < N; ++j) acc[j] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
          double av = A[i * sam + k * sak];
          for (int64_t j = 0; j < N; ++j) acc[j] += av * (double)B[k * sbk + j * sbn];
        }
        for (int64_t j = 0; j < N; ++j) C[i * scm + j * scn] = (float)acc[j];
      } else if (order == 0) {
        for (int64_t j = 0; j < N; ++j) {
          float s = 0.0f;
          for (int64_t k = 0; k < K; ++k) s += A[i * sam + k * sak] * B[k * sbk + j * sbn];
          C[i * scm + j * scn] = s;
        }
      } else {
        for (int64_t j = 0; j < N; ++j) C[i * scm + j * scn] = 0.0f;
        for (int64_t k = 0; k < K; ++k) {
          float av = A[i * sam + k * sak];
          for (int64_t j = 0; j < N; ++j) C[i * scm + j * scn] += av * B[k * sbk + j * sbn];
        }
      }
    }
    free(acc);
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ Gemm
 * gemm.cpp:39-182: 2-D, transA/transB through the index maps, bias of rank 1 (per column)
 * or 2.  ONNX semantics Y = alpha*(A'B') + beta*C; the reference computes
 * alpha*C + beta*(A'B') (gemm.cpp:166-181), identical for alpha = beta = 1. */
int orc_gemm(const orc_tensor *a, const orc_tensor *b, const orc_tensor *bias, orc_tensor *y,
             float alpha, float beta, int transA, int transB, int acc64) {
  int64_t M = y->shape[0], N = y->shape[1];
  int64_t K = transA ? a->shape[0] : a->shape[1];
  int64_t sam = transA ? a->stride[1] : a->stride[0], sak = transA ? a->stride[0] : a->stride[1];
  int64_t sbk = transB ? b->stride[1] : b->stride[0], sbn = transB ? b->stride[0] : b->stride[1];
  const float *A = (const float *)a->data, *B = (const float *)b->data;
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float s;
      if (acc64) {
        double d = 0.0;
        for (int64_t k = 0; k < K; ++k) d += (double)A[i * sam + k * sak] * B[k * sbk + j * sbn];
        s = (float)d;
      } else {
        s = 0.0f;
        for (int64_t k = 0; k < K; ++k) s += A[i * sam + k * sak] * B[k * sbk + j * sbn];
      }
      float c = 0.0f;
      if (bias) {
        int64_t idx[2] = {i, j};
        c = ((const float *)bias->data)[bcast_offset(bias, idx, 2)];
      }
      ((float *)y->data)[i * y->stride[0] + j * y->stride[1]] = alpha * s + beta * c;
    }
  return 0;
}

/* ------------------------------------------------------------------ Softmax
 * softmax.cpp:22-139: per row along `axis`: max (init lowest), x-max, expf, sum, divide. */
int orc_softmax(const orc_tensor *in, orc_tensor *out, int axis) {
  if (axis < 0) axis += in->rank;
  int64_t L = in->shape[axis], rows = numel(in) / L, idx[ORC_MAX_RANK];
  int64_t rshape[ORC_MAX_RANK];
  memcpy(rshape, in->shape, sizeof(rshape));
  rshape[axis] = 1;
  for (int64_t r = 0; r < rows; ++r) {
    unravel(r, rshape, in->rank, idx);
    const float *x = (const float *)in->data + offset_of(in, idx);
    float *y = (float *)out->data + offset_of(out, idx);
    int64_t sx = in->stride[axis], sy = out->stride[axis];
    float mx = -3.402823466e+38f;
    for (int64_t i = 0; i < L; ++i) mx = fmaxf(mx, x[i * sx]);
    float sum = 0.0f;
    for (int64_t i = 0; i < L; ++i) {
      float e = expf(x[i * sx] - mx);
      y[i * sy] = e;
      sum += e;
    }
    for (int64_t i = 0; i < L; ++i) y[i * sy] = y[i * sy] / sum;
  }
  return 0;
}

/* ------------------------------------------------------------------ LayerNormalization
 * layer_normalization.cpp:33-220: along `axis`: mean = sum(x)/n ; d = x-mean ;
 * var = sum(d*d)/n ; y = d * (1/sqrtf(var+eps)) * scale + bias.  (The reference adds the
 * first sum into scratch it never cleared, :127-137; the sum here starts from zero.) */
int orc_layernorm(const orc_tensor *in, const orc_tensor *scale, const orc_tensor *bias,
                  orc_tensor *out, int axis, float eps, int acc64) {
  if (axis < 0) axis += in->rank;
  int64_t L = in->shape[axis], rows = numel(in) / L, idx[ORC_MAX_RANK];
  int64_t rshape[ORC_MAX_RANK];
  memcpy(rshape, in->shape, sizeof(rshape));
  rshape[axis] = 1;
  const float *g = (const float *)scale->data, *bt = (const float *)bias->data;
  int64_t sg = scale->stride[scale->rank - 1], sb = bias->stride[bias->rank - 1];
  for (int64_t r = 0; r < rows; ++r) {
    unravel(r, rshape, in->rank, idx);
    const float *x = (const float *)in->data + offset_of(in, idx);
    float *y = (float *)out->data + offset_of(out, idx);
    int64_t sx = in->stride[axis], sy = out->stride[axis];
    float mean, var;
    if (acc64) {
      double s = 0.0, v = 0.0;
      for (int64_t i = 0; i < L; ++i) s += x[i * sx];
      mean = (float)(s / (double)L);
      for (int64_t i = 0; i < L; ++i) {
        double d = x[i * sx] - mean;
        v += d * d;
      }
      var = (float)(v / (double)L);
    } else {
      float s = 0.0f, v = 0.0f;
      for (int64_t i = 0; i < L; ++i) s += x[i * sx];
      mean = s / (float)L;
      for (int64_t i = 0; i < L; ++i) {
        float d = x[i * sx] - mean;
        v += d * d;
      }
      var = v / (float)L;
    }
    float inv = 1.0f / sqrtf(var + eps);
    for (int64_t i = 0; i < L; ++i) y[i * sy] = (x[i * sx] - mean) * inv * g[i * sg] + bt[i * sb];
  }
  return 0;
}

/* ------------------------------------------------------------------ data movement
 * transpose.cpp:19-48: out[perm(i)] = in[i]. */
int orc_transpose(const orc_tensor *in, orc_tensor *out, const int64_t *perm) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], iidx[ORC_MAX_RANK];
  size_t es = esize(in->dtype);
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    for (int i = 0; i < out->rank; ++i) iidx[perm[i]] = idx[i];
    memcpy((char *)out->data + offset_of(out, idx) * es,
           (char *)in->data + offset_of(in, iidx) * es, es);
  }
  return 0;
}

/* reshape.cpp:18-64 (also unsqueeze.cpp:20-63, squeeze.cpp:17-54, flatten.cpp:15-63): the
 * e-th element in logical row-major order of the input is the e-th of the output,
 * whatever either layout is. */
int orc_reshape(const orc_tensor *in, orc_tensor *out) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], iidx[ORC_MAX_RANK];
  size_t es = esize(in->dtype);
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, in->shape, in->rank, iidx);
    unravel(e, out->shape, out->rank, idx);
    memcpy((char *)out->data + offset_of(out, idx) * es,
           (char *)in->data + offset_of(in, iidx) * es, es);
  }
  return 0;
}

/* gather.cpp:100-139 (constant scalar index), :149-186 (constant index tensor, any axis),
 * :195-272 (constant table, runtime indices, axis 0): out[.., i.., ..] = data[.., ind[i..], ..].
 * Indices are int64, non-negative, not range-checked by the reference. */
int orc_gather(const orc_tensor *data, const orc_tensor *ind, orc_tensor *out, int axis) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], didx[ORC_MAX_RANK];
  size_t es = esize(data->dtype);
  int q = ind->rank;
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int64_t iv = ((const int64_t *)ind->data)[q ? offset_of(ind, idx + axis) : 0];
    for (int i = 0; i < axis; ++i) didx[i] = idx[i];
    didx[axis] = iv;
    for (int i = axis + 1; i < data->rank; ++i) didx[i] = idx[i + q - 1];
    memcpy((char *)out->data + offset_of(out, idx) * es,
           (char *)data->data + offset_of(data, didx) * es, es);
  }
  return 0;
}

/* where.cpp:30-80, :90-150: cond ? x : y, all three broadcast to the output. */
int orc_where(const orc_tensor *cond, const orc_tensor *x, const orc_tensor *y, orc_tensor *out) {
  int64_t n = numel(out), idx[ORC_MAX_RANK];
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    uint8_t c = ((const uint8_t *)cond->data)[bcast_offset(cond, idx, out->rank)];
    float xv = ((const float *)x->data)[bcast_offset(x, idx, out->rank)];
    float yv = ((const float *)y->data)[bcast_offset(y, idx, out->rank)];
    ((float *)out->data)[offset_of(out, idx)] = c ? xv : yv;
  }
  return 0;
}

/* slice.cpp:17-55: out[i] = in[i + start] on the sliced axes (steps are 1). */
int orc_slice(const orc_tensor *in, orc_tensor *out, const int64_t *starts /* per dim */) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], iidx[ORC_MAX_RANK];
  size_t es = esize(in->dtype);
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    for (int i = 0; i < out->rank; ++i) iidx[i] = idx[i] + starts[i];
    memcpy((char *)out->data + offset_of(out, idx) * es,
           (char *)in->data + offset_of(in, iidx) * es, es);
  }
  return 0;
}

/* concat.cpp:18-68: two inputs along `axis`. */
int orc_concat2(const orc_tensor *a, const orc_tensor *b, orc_tensor *out, int axis) {
  int64_t n = numel(out), idx[ORC_MAX_RANK];
  size_t es = esize(a->dtype);
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int64_t oo = offset_of(out, idx);
    const orc_tensor *src = a;
    if (idx[axis] >= a->shape[axis]) {
      idx[axis] -= a->shape[axis];
      src = b;
    }
    memcpy((char *)out->data + oo * es, (char *)src->data + offset_of(src, idx) * es, es);
  }
  return 0;
}

/* pad.cpp:15-51 copies the input into the interior; the reference leaves the border as it
 * finds it (zero only because the arena starts zeroed).  ONNX constant mode, value 0. */
int orc_pad(const orc_tensor *in, orc_tensor *out, const int64_t *pads_begin) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], iidx[ORC_MAX_RANK];
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    int inside = 1;
    for (int i = 0; i < out->rank; ++i) {
      iidx[i] = idx[i] - pads_begin[i];
      if (iidx[i] < 0 || iidx[i] >= in->shape[i]) inside = 0;
    }
    ((float *)out->data)[offset_of(out, idx)] =
        inside ? ((const float *)in->data)[offset_of(in, iidx)] : 0.0f;
  }
  return 0;
}

/* reduce_mean.cpp:16-98, keepdims = 1: mean over the axes flagged in `reduce[]`. */
int orc_reduce_mean(const orc_tensor *in, orc_tensor *out, const int32_t *reduce) {
  int64_t n = numel(out), idx[ORC_MAX_RANK], iidx[ORC_MAX_RANK], rshape[ORC_MAX_RANK];
  int64_t cnt = 1;
  for (int i = 0; i < in->rank; ++i) {
    rshape[i] = reduce[i] ? in->shape[i] : 1;
    cnt *= rshape[i];
  }
  for (int64_t e = 0; e < n; ++e) {
    unravel(e, out->shape, out->rank, idx);
    float s = 0.0f;
    for (int64_t r = 0; r < cnt; ++r) {
      unravel(r, rshape, in->rank, iidx);
      for (int i = 0; i < in->rank; ++i) iidx[i] += reduce[i] ? 0 : idx[i];
      s += ((const float *)in->data)[offset_of(in, iidx)];
    }
    ((float *)out->data)[offset_of(out, idx)] = s / (float)cnt;
  }
  return 0;
}

/* cum_sum.cpp:53-87: int64, forward, inclusive, along `axis`. */
int orc_cumsum(const orc_tensor *in, orc_tensor *out, int axis) {
  int64_t L = in->shape[axis], rows = numel(in) / L, idx[ORC_MAX_RANK], rshape[ORC_MAX_RANK];
  memcpy(rshape, in->shape, sizeof(rshape));
  rshape[axis] = 1;
  for (int64_t r = 0; r < rows; ++r) {
    unravel(r, rshape, in->rank, idx);
    const int64_t *x = (const int64_t *)in->data + offset_of(in, idx);
    int64_t *y = (int64_t *)out->data + offset_of(out, idx), s = 0;
    for (int64_t i = 0; i < L; ++i) {
      s += x[i * in->stride[axis]];
      y[i * out->stride[axis]] = s;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ Conv
 * conv.cpp:27-201 (+ :214-280 padded variant): NCHW / OIHW direct convolution, 1-D or 2-D.
 * group == 1 or depthwise (group == C, multiplier 1), as in the reference (:103-149).
 * ONNX semantics for strides, dilations, zero padding and per-channel bias; the reference
 * ignores strides/dilations in its index maps (:68-76) and adds bias[1] to every channel
 * (:181-184), which agree with ONNX only for stride 1, dilation 1 and zero bias. */
int orc_conv(const orc_tensor *x, const orc_tensor *w, const orc_tensor *bias, orc_tensor *y,
             const int64_t *pads, const int64_t *strides, const int64_t *dil, int64_t group,
             int acc64) {
  int nd = x->rank - 2;
  int64_t N = y->shape[0], OC = y->shape[1], IC = x->shape[1];
  int64_t OH = nd == 2 ? y->shape[2] : 1, OW = y->shape[nd + 1];
  int64_t IH = nd == 2 ? x->shape[2] : 1, IW = x->shape[nd + 1];
  int64_t KH = nd == 2 ? w->shape[2] : 1, KW = w->shape[nd + 1];
  int64_t ph = nd == 2 ? pads[0] : 0, pw = nd == 2 ? pads[1] : pads[0];
  int64_t sh = nd == 2 ? strides[0] : 1, sw = nd == 2 ? strides[1] : strides[0];
  int64_t dh = nd == 2 ? dil[0] : 1, dw = nd == 2 ? dil[1] : dil[0];
  int64_t xsh = nd == 2 ? x->stride[2] : 0, xsw = x->stride[nd + 1];
  int64_t wsh = nd == 2 ? w->stride[2] : 0, wsw = w->stride[nd + 1];
  int64_t ysh = nd == 2 ? y->stride[2] : 0, ysw = y->stride[nd + 1];
  int64_t icg = IC / group, ocg = OC / group;
  const float *X = (const float *)x->data, *W = (const float *)w->data;
  /* (image, output channel) pairs are independent: with orc_set_threads(n > 1) they are spread
   * over n host threads; every output keeps its own summation order, so no bit changes. */
#pragma omp parallel for collapse(2) schedule(static) num_threads(orc_threads) if (orc_threads > 1)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t oc = 0; oc < OC; ++oc) {
      int64_t g = oc / ocg;
      for (int64_t oh = 0; oh < OH; ++oh)
        for (int64_t ow = 0; ow < OW; ++ow) {
          double sd = 0.0;
          float sf = 0.0f;
          for (int64_t ic = 0; ic < icg; ++ic)
            for (int64_t kh = 0; kh < KH; ++kh) {
              int64_t ih = oh * sh - ph + kh * dh;
              if (ih < 0 || ih >= IH) continue;
              for (int64_t kw = 0; kw < KW; ++kw) {
                int64_t iw = ow * sw - pw + kw * dw;
                if (iw < 0 || iw >= IW) continue;
                float xv = X[n * x->stride[0] + (g * icg + ic) * x->stride[1] + ih * xsh + iw * xsw];
                float wv = W[oc * w->stride[0] + ic * w->stride[1] + kh * wsh + kw * wsw];
                if (acc64) sd += (double)xv * wv; else sf += xv * wv;
              }
            }
          float r = acc64 ? (float)sd : sf;
          if (bias) r += ((const float *)bias->data)[oc * bias->stride[0]];
          ((float *)y->data)[n * y->stride[0] + oc * y->stride[1] + oh * ysh + ow * ysw] = r;
        }
    }
  return 0;
}

/* maxpool.cpp:17-82, averagepool.cpp:19-87: 2-D, no padding (converter.cpp:581-592,
 * :1569-1580).  mode 0 = max (maximumf fold), 1 = average (sum / k). */
int orc_pool2d(const orc_tensor *x, orc_tensor *y, int mode, const int64_t *kernel,
               const int64_t *strides) {
  for (int64_t n = 0; n < y->shape[0]; ++n)
    for (int64_t c = 0; c < y->shape[1]; ++c)
      for (int64_t oh = 0; oh < y->shape[2]; ++oh)
        for (int64_t ow = 0; ow < y->shape[3]; ++ow) {
          float r = mode ? 0.0f : -3.402823466e+38f;
          for (int64_t kh = 0; kh < kernel[0]; ++kh)
            for (int64_t kw = 0; kw < kernel[1]; ++kw) {
              float v = ((const float *)x->data)[n * x->stride[0] + c * x->stride[1] +
                                                 (oh * strides[0] + kh) * x->stride[2] +
                                                 (ow * strides[1] + kw) * x->stride[3]];
              r = mode ? r + v : fmaxf(r, v);
            }
          if (mode) r = r / (float)(kernel[0] * kernel[1]);
          ((float *)y->data)[n * y->stride[0] + c * y->stride[1] + oh * y->stride[2] +
                             ow * y->stride[3]] = r;
        }
  return 0;
}

/* ------------------------------------------------------------------ addressing helpers
 * src/utils/utils.cpp:26-41 (GenAllOrders), :64-102 (GenPhysicalShape / GenStrides),
 * src/structure/tensor/meta.cpp:59-137 (BroadcastShape / BroadcastMatMulShape). */
void orc_gen_strides(const int64_t *shape, const int64_t *layout, int rank, int64_t *strides) {
  int64_t phys[ORC_MAX_RANK], pstr[ORC_MAX_RANK];
  for (int i = 0; i < rank; ++i) phys[layout[i]] = shape[i];
  if (rank > 0) pstr[rank - 1] = 1;
  for (int i = rank - 1; i > 0; --i) pstr[i - 1] = pstr[i] * phys[i];
  for (int i = 0; i < rank; ++i) strides[i] = pstr[layout[i]];
}

/* Writes len! permutations of len entries each, in the reference's enumeration order:
 * take every permutation of len-1 and insert len-1 at positions 0..len-1. Returns count. */
int64_t orc_gen_all_orders(int len, int64_t *out) {
  if (len == 0) return 1;
  int64_t prev_n = 1;
  for (int i = 2; i < len; ++i) prev_n *= i;
  int64_t *prev = (int64_t *)malloc(sizeof(int64_t) * (size_t)(prev_n * (len > 1 ? len - 1 : 1)));
  orc_gen_all_orders(len - 1, prev);
  int64_t cnt = 0;
  for (int64_t p = 0; p < prev_n; ++p)
    for (int pos = 0; pos < len; ++pos) {
      int64_t *o = out + cnt * len;
      for (int i = 0, j = 0; i < len; ++i) o[i] = i == pos ? len - 1 : prev[p * (len - 1) + j++];
      ++cnt;
    }
  free(prev);
  return cnt;
}

/* Returns the output rank, or -1 when the shapes do not broadcast. */
int orc_broadcast_shape(const int64_t *a, int ra, const int64_t *b, int rb, int64_t *out) {
  int r = ra > rb ? ra : rb;
  for (int i = 0; i < r; ++i) {
    int ia = i - (r - ra), ib = i - (r - rb);
    int64_t da = ia >= 0 ? a[ia] : 1, db = ib >= 0 ? b[ib] : 1;
    if (da == db) out[i] = da;
    else if (da == 1) out[i] = db;
    else if (db == 1) out[i] = da;
    else return -1;
  }
  return r;
}

int orc_broadcast_matmul_shape(const int64_t *a, int ra, const int64_t *b, int rb, int64_t *out) {
  if (ra < 2 || rb < 2) return -1;
  if (a[ra - 1] != b[rb - 2]) return -1;
  int r = orc_broadcast_shape(a, ra - 2, b, rb - 2, out);
  if (r < 0) return -1;
  out[r] = a[ra - 2];
  out[r + 1] = b[rb - 1];
  return r + 2;
}
