// Bit-exact data movement: strided copy (Transpose / Slice / Concat / Pad interior),
// logical-order reshape copy, Gather, fused embedding lookup and Pad.
//
// All HBM-bound.  The strided copy picks one of three kernels after collapsing dims:
//   - vector path: both sides contiguous innermost -> 16-byte loads and stores;
//   - tile path: the input's contiguous dim differs from the output's -> 32x33 shared-memory
//     tile so that both the global read and the global write are coalesced;
//   - generic path: one element per thread.
#include "common.cuh"

namespace fml {
namespace {

template <typename T>
__global__ void copy_generic(Iter<2> it, T *out, const T *in) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < it.total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[2];
    offsets_of(it, i, off);
    out[off[0]] = in[off[1]];
  }
}

// Innermost dim contiguous on both sides, extent (in units of T) a multiple of V.
template <typename T, int V>
__global__ void copy_vec(Iter<2> it, T *out, const T *in) {
  pdl_prologue();
  struct alignas(sizeof(T) * V) Pack { T v[V]; };
  const int64_t innerv = it.shape[it.rank - 1] / V, totalv = it.total / V;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < totalv;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t row = i / innerv, c = (i - row * innerv) * V;
    int64_t oo = c, oi = c;
    for (int d = it.rank - 2; d >= 0; --d) {
      int64_t q = row / it.shape[d], r = row - q * it.shape[d];
      row = q;
      oo += r * it.stride[0][d];
      oi += r * it.stride[1][d];
    }
    *reinterpret_cast<Pack *>(out + oo) = *reinterpret_cast<const Pack *>(in + oi);
  }
}

// Tile transpose: dim `di` is contiguous in the input, dim `dout` in the output.  Each block
// moves a 32x32 tile of (di, do); the remaining dims are linearised over blockIdx.z/y.
template <typename T>
__global__ void copy_tile(Iter<2> it, int di, int dout, int64_t tiles_i, int64_t tiles_o,
                          T *out, const T *in) {
  pdl_prologue();
  __shared__ T tile[32][33];
  int64_t b = blockIdx.x;
  const int64_t ti = b % tiles_i; b /= tiles_i;
  const int64_t to = b % tiles_o; b /= tiles_o;
  int64_t base_o = 0, base_i = 0;
  for (int d = it.rank - 1; d >= 0; --d) {
    if (d == di || d == dout) continue;
    int64_t q = b / it.shape[d], r = b - q * it.shape[d];
    b = q;
    base_o += r * it.stride[0][d];
    base_i += r * it.stride[1][d];
  }
  const int64_t i0 = ti * 32, o0 = to * 32;
  // read: threadIdx.x walks the input-contiguous dim
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int64_t ci = i0 + threadIdx.x, co = o0 + r;
    if (ci < it.shape[di] && co < it.shape[dout])
      tile[r][threadIdx.x] = in[base_i + ci * it.stride[1][di] + co * it.stride[1][dout]];
  }
  __syncthreads();
  // write: threadIdx.x walks the output-contiguous dim
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int64_t ci = i0 + r, co = o0 + threadIdx.x;
    if (ci < it.shape[di] && co < it.shape[dout])
      out[base_o + ci * it.stride[0][di] + co * it.stride[0][dout]] = tile[threadIdx.x][r];
  }
}

// The same for 4-byte elements with 16-byte accesses on both sides: a 64x64 tile per block of
// 256 threads, read as float4 along the input-contiguous dim and written as float4 along the
// output-contiguous dim.  Both extents are multiples of 4 and every other stride keeps the
// 16-byte alignment, so a float4 is either wholly inside the tensor or wholly outside.
__global__ void copy_tile64(Iter<2> it, int di, int dout, int64_t tiles_i, int64_t tiles_o,
                            float *out, const float *in) {
  pdl_prologue();
  __shared__ float tile[64][65];
  int64_t b = blockIdx.x;
  const int64_t ti = b % tiles_i; b /= tiles_i;
  const int64_t to = b % tiles_o; b /= tiles_o;
  int64_t base_o = 0, base_i = 0;
  for (int d = it.rank - 1; d >= 0; --d) {
    if (d == di || d == dout) continue;
    int64_t q = b / it.shape[d], r = b - q * it.shape[d];
    b = q;
    base_o += r * it.stride[0][d];
    base_i += r * it.stride[1][d];
  }
  const int64_t i0 = ti * 64, o0 = to * 64;
  const int q = threadIdx.x & 15, r0 = threadIdx.x >> 4;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int r = r0 + 16 * p;
    const int64_t ci = i0 + q * 4, co = o0 + r;
    if (ci < it.shape[di] && co < it.shape[dout]) {
      const float4 v = *reinterpret_cast<const float4 *>(in + base_i + ci + co * it.stride[1][dout]);
      tile[r][q * 4 + 0] = v.x; tile[r][q * 4 + 1] = v.y; tile[r][q * 4 + 2] = v.z; tile[r][q * 4 + 3] = v.w;
    }
  }
  __syncthreads();
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int r = r0 + 16 * p;
    const int64_t ci = i0 + r, co = o0 + q * 4;
    if (ci < it.shape[di] && co < it.shape[dout])
      *reinterpret_cast<float4 *>(out + base_o + ci * it.stride[0][di] + co) =
          make_float4(tile[q * 4 + 0][r], tile[q * 4 + 1][r], tile[q * 4 + 2][r], tile[q * 4 + 3][r]);
  }
}

template <typename T>
int launch_copy(Iter<2> &it, void *out, const void *in, cudaStream_t s) {
  const int l = it.rank - 1;
  const bool out_contig = it.stride[0][l] == 1, in_contig = it.stride[1][l] == 1;
  if (out_contig && in_contig) {
    constexpr int V = 16 / sizeof(T);
    bool ok = it.shape[l] % V == 0 && aligned16(out) && aligned16(in);
    for (int d = 0; d < l && ok; ++d)
      ok = it.stride[0][d] % V == 0 && it.stride[1][d] % V == 0;
    if (ok) {
      FML_LAUNCH((copy_vec<T, V>), grid_for(it.total / V, 256), 256, 0, s, it, (T *)out, (const T *)in);
      FML_CUDA(cudaGetLastError());
      return FML_OK;
    }
  }
  // find a dim that is contiguous in the input while another is contiguous in the output
  int di = -1, dout = -1;
  for (int d = 0; d < it.rank; ++d) {
    if (it.stride[1][d] == 1 && di < 0) di = d;
    if (it.stride[0][d] == 1 && dout < 0) dout = d;
  }
  if (sizeof(T) == 4 && di >= 0 && dout >= 0 && di != dout && it.shape[di] >= 64 && it.shape[dout] >= 64 &&
      it.shape[di] % 4 == 0 && it.shape[dout] % 4 == 0 && aligned16(out) && aligned16(in)) {
    bool ok = true;
    for (int d = 0; d < it.rank; ++d) {
      if (d != dout && it.stride[0][d] % 4 != 0) ok = false;
      if (d != di && it.stride[1][d] % 4 != 0) ok = false;
    }
    int64_t tiles_i = (it.shape[di] + 63) / 64, tiles_o = (it.shape[dout] + 63) / 64;
    int64_t blocks = tiles_i * tiles_o;
    for (int d = 0; d < it.rank; ++d)
      if (d != di && d != dout) blocks *= it.shape[d];
    if (ok && blocks < (int64_t)1 << 31) {
      FML_LAUNCH((copy_tile64), (unsigned)blocks, 256, 0, s, it, di, dout, tiles_i, tiles_o,
                 (float *)out, (const float *)in);
      FML_CUDA(cudaGetLastError());
      return FML_OK;
    }
  }
  if (di >= 0 && dout >= 0 && di != dout && it.shape[di] >= 8 && it.shape[dout] >= 8) {
    int64_t tiles_i = (it.shape[di] + 31) / 32, tiles_o = (it.shape[dout] + 31) / 32;
    int64_t blocks = tiles_i * tiles_o;
    for (int d = 0; d < it.rank; ++d)
      if (d != di && d != dout) blocks *= it.shape[d];
    if (blocks < (int64_t)1 << 31) {
      FML_LAUNCH((copy_tile<T>), (unsigned)blocks, dim3(32, 8), 0, s, it, di, dout, tiles_i, tiles_o,
                                                            (T *)out, (const T *)in);
      FML_CUDA(cudaGetLastError());
      return FML_OK;
    }
  }
  FML_LAUNCH((copy_generic<T>), grid_for(it.total, 256), 256, 0, s, it, (T *)out, (const T *)in);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

// out: operand 0 strides over the OUTPUT's logical shape; input offsets are rebuilt by
// unravelling the same linear index over the INPUT's logical shape.
struct ReshapeArgs {
  int orank, irank;
  int64_t oshape[kMaxDims], ostride[kMaxDims], ishape[kMaxDims], istride[kMaxDims];
  int64_t total;
};

template <typename T>
__global__ void reshape_generic(ReshapeArgs a, T *out, const T *in) {
  pdl_prologue();
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < a.total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t oo = 0, oi = 0, l = e;
    for (int d = a.orank - 1; d >= 0; --d) {
      int64_t q = l / a.oshape[d];
      oo += (l - q * a.oshape[d]) * a.ostride[d];
      l = q;
    }
    l = e;
    for (int d = a.irank - 1; d >= 0; --d) {
      int64_t q = l / a.ishape[d];
      oi += (l - q * a.ishape[d]) * a.istride[d];
      l = q;
    }
    out[oo] = in[oi];
  }
}

bool is_row_major(const fml_tensor *t) {
  int64_t s = 1;
  for (int i = t->rank - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->stride[i] != s) return false;
    s *= t->shape[i];
  }
  return true;
}

// Gather: the output index splits into (pre.., q index dims.., post..).
struct GatherArgs {
  int orank, axis, qrank, drank;
  int64_t oshape[kMaxDims], ostride[kMaxDims];
  int64_t dstride[kMaxDims], istride[kMaxDims];
  int64_t axis_extent, total;
};

template <typename T>
__global__ void gather_generic(GatherArgs g, T *out, const T *data, const int64_t *ind,
                               int *status) {
  pdl_prologue();
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < g.total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t idx[kMaxDims], l = e, oo = 0;
    for (int d = g.orank - 1; d >= 0; --d) {
      int64_t q = l / g.oshape[d];
      idx[d] = l - q * g.oshape[d];
      oo += idx[d] * g.ostride[d];
      l = q;
    }
    int64_t io = 0;
    for (int d = 0; d < g.qrank; ++d) io += idx[g.axis + d] * g.istride[d];
    int64_t iv = ind[io];
    if (iv < 0 || iv >= g.axis_extent) {
      atomicOr(status, kStatusIndexRange);
      iv = iv < 0 ? 0 : g.axis_extent - 1;
    }
    int64_t off = iv * g.dstride[g.axis];
    for (int d = 0; d < g.axis; ++d) off += idx[d] * g.dstride[d];
    for (int d = g.axis + 1; d < g.drank; ++d) off += idx[d + g.qrank - 1] * g.dstride[d];
    out[oo] = data[off];
  }
}

// Embedding rows: one warp per output row, 16-byte lanes.  table rows contiguous.
__global__ void embedding_rows(int64_t rows, int64_t width, int64_t vocab, float *out,
                               const float *table, int64_t table_row_stride, const int64_t *ids,
                               const float *add0, int64_t add0_row_stride,
                               const float *add1, int64_t add1_row_stride, int64_t add_rows,
                               int *status) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (warp >= rows) return;
  int64_t id = ids[warp];
  if (id < 0 || id >= vocab) {
    if (lane == 0) atomicOr(status, kStatusIndexRange);
    id = id < 0 ? 0 : vocab - 1;
  }
  const float4 *src = reinterpret_cast<const float4 *>(table + id * table_row_stride);
  const float4 *a0 = add0 ? reinterpret_cast<const float4 *>(add0 + (warp % add_rows) * add0_row_stride) : nullptr;
  const float4 *a1 = add1 ? reinterpret_cast<const float4 *>(add1 + (warp % add_rows) * add1_row_stride) : nullptr;
  float4 *dst = reinterpret_cast<float4 *>(out + warp * width);
  for (int64_t c = lane; c < width / 4; c += 32) {
    float4 v = src[c];
    if (a0) { float4 t = a0[c]; v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
    if (a1) { float4 t = a1[c]; v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w; }
    dst[c] = v;
  }
}

// operand 0 = out, 1 = gathered row view (unused), 2 = add0, 3 = add1
__global__ void embedding_generic(GatherArgs g, Iter<3> add, float *out, const float *table,
                                  const int64_t *ind, const float *add0, const float *add1,
                                  int *status) {
  pdl_prologue();
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < g.total;
       e += (int64_t)gridDim.x * blockDim.x) {
    int64_t idx[kMaxDims], l = e, oo = 0, o0 = 0, o1 = 0;
    for (int d = g.orank - 1; d >= 0; --d) {
      int64_t q = l / g.oshape[d];
      idx[d] = l - q * g.oshape[d];
      oo += idx[d] * g.ostride[d];
      o0 += idx[d] * add.stride[1][d];
      o1 += idx[d] * add.stride[2][d];
      l = q;
    }
    int64_t io = 0;
    for (int d = 0; d < g.qrank; ++d) io += idx[d] * g.istride[d];
    int64_t iv = ind[io];
    if (iv < 0 || iv >= g.axis_extent) {
      atomicOr(status, kStatusIndexRange);
      iv = iv < 0 ? 0 : g.axis_extent - 1;
    }
    int64_t off = iv * g.dstride[0];
    for (int d = 1; d < g.drank; ++d) off += idx[d + g.qrank - 1] * g.dstride[d];
    float v = table[off];
    if (add0) v += add0[o0];
    if (add1) v += add1[o1];
    out[oo] = v;
  }
}

int fill_gather(GatherArgs &g, const fml_tensor *data, const fml_tensor *ind,
                const fml_tensor *out, int axis, const char *who) {
  FML_REQUIRE(valid_tensor(data) && valid_tensor(ind) && valid_tensor(out), FML_BAD_ARG,
              "%s: bad tensor", who);
  FML_REQUIRE(ind->dtype == FML_I64, FML_UNSUPPORTED, "%s: indices must be int64", who);
  FML_REQUIRE(axis >= 0 && axis < data->rank, FML_BAD_ARG, "%s: axis %d out of range", who, axis);
  FML_REQUIRE(out->rank == data->rank - 1 + ind->rank, FML_BAD_ARG, "%s: output rank", who);
  FML_REQUIRE(out->dtype == data->dtype, FML_BAD_ARG, "%s: dtype mismatch", who);
  g.orank = out->rank; g.axis = axis; g.qrank = ind->rank; g.drank = data->rank;
  for (int i = 0; i < out->rank; ++i) { g.oshape[i] = out->shape[i]; g.ostride[i] = out->stride[i]; }
  for (int i = 0; i < data->rank; ++i) g.dstride[i] = data->stride[i];
  for (int i = 0; i < ind->rank; ++i) {
    g.istride[i] = ind->stride[i];
    FML_REQUIRE(out->shape[axis + i] == ind->shape[i], FML_BAD_ARG, "%s: output shape", who);
  }
  for (int i = 0; i < axis; ++i)
    FML_REQUIRE(out->shape[i] == data->shape[i], FML_BAD_ARG, "%s: output shape", who);
  for (int i = axis + 1; i < data->rank; ++i)
    FML_REQUIRE(out->shape[i + ind->rank - 1] == data->shape[i], FML_BAD_ARG, "%s: output shape", who);
  g.axis_extent = data->shape[axis];
  g.total = numel(out);
  return FML_OK;
}

}  // namespace
}  // namespace fml

using namespace fml;

extern "C" int fml_copy_strided(const fml_tensor *in, const fml_tensor *out, void *stream) {
  FML_REQUIRE(valid_tensor(in) && valid_tensor(out), FML_BAD_ARG, "fml_copy_strided: bad tensor");
  FML_REQUIRE(in->dtype == out->dtype && in->rank == out->rank, FML_BAD_ARG,
              "fml_copy_strided: dtype or rank mismatch");
  Iter<2> it;
  it.rank = out->rank;
  for (int i = 0; i < out->rank; ++i) {
    FML_REQUIRE(in->shape[i] == out->shape[i], FML_BAD_ARG, "fml_copy_strided: shape mismatch");
    it.shape[i] = out->shape[i];
    it.stride[0][i] = out->stride[i];
    it.stride[1][i] = in->stride[i];
  }
  collapse(it);
  if (it.total == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  switch (dtype_size(in->dtype)) {
  case 4: return launch_copy<uint32_t>(it, out->data, in->data, s);
  case 8: return launch_copy<uint64_t>(it, out->data, in->data, s);
  default: return launch_copy<uint8_t>(it, out->data, in->data, s);
  }
}

extern "C" int fml_reshape_copy(const fml_tensor *in, const fml_tensor *out, void *stream) {
  FML_REQUIRE(valid_tensor(in) && valid_tensor(out), FML_BAD_ARG, "fml_reshape_copy: bad tensor");
  FML_REQUIRE(in->dtype == out->dtype && numel(in) == numel(out), FML_BAD_ARG,
              "fml_reshape_copy: dtype or element count mismatch");
  const int64_t n = numel(out);
  if (n == 0) return FML_OK;
  cudaStream_t s = as_stream(stream);
  const size_t es = dtype_size(in->dtype);
  if (is_row_major(in) && is_row_major(out)) {
    if (in->data != out->data)
      FML_CUDA(cudaMemcpyAsync(out->data, in->data, n * es, cudaMemcpyDeviceToDevice, s));
    return FML_OK;
  }
  // one side row-major: the copy is a plain strided copy over the other side's shape
  if (is_row_major(in) || is_row_major(out)) {
    const fml_tensor *shaped = is_row_major(in) ? out : in;
    fml_tensor flat = *shaped;
    int64_t st = 1;
    for (int i = flat.rank - 1; i >= 0; --i) { flat.stride[i] = st; st *= flat.shape[i]; }
    if (is_row_major(in)) { flat.data = in->data; return fml_copy_strided(&flat, out, stream); }
    flat.data = out->data;
    return fml_copy_strided(in, &flat, stream);
  }
  ReshapeArgs a;
  a.orank = out->rank; a.irank = in->rank; a.total = n;
  for (int i = 0; i < out->rank; ++i) { a.oshape[i] = out->shape[i]; a.ostride[i] = out->stride[i]; }
  for (int i = 0; i < in->rank; ++i) { a.ishape[i] = in->shape[i]; a.istride[i] = in->stride[i]; }
  const int grid = grid_for(n, 256);
  switch (es) {
  case 4: FML_LAUNCH((reshape_generic<uint32_t>), grid, 256, 0, s, a, (uint32_t *)out->data, (const uint32_t *)in->data); break;
  case 8: FML_LAUNCH((reshape_generic<uint64_t>), grid, 256, 0, s, a, (uint64_t *)out->data, (const uint64_t *)in->data); break;
  default: FML_LAUNCH((reshape_generic<uint8_t>), grid, 256, 0, s, a, (uint8_t *)out->data, (const uint8_t *)in->data); break;
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_gather(const fml_tensor *data, const fml_tensor *indices, const fml_tensor *out,
                          int axis, void *stream) {
  GatherArgs g;
  int st = fill_gather(g, data, indices, out, axis, "fml_gather");
  if (st != FML_OK) return st;
  if (g.total == 0) return FML_OK;
  int *status = device_status_word();
  FML_REQUIRE(status, FML_CUDA_ERROR, "fml_gather: no device status word");
  cudaStream_t s = as_stream(stream);
  // Row fast path: axis 0 of a row-major 2-D fp32 table into a row-major output.
  if (axis == 0 && data->rank == 2 && data->dtype == FML_F32 && data->stride[1] == 1 &&
      data->shape[1] % 4 == 0 && data->stride[0] % 4 == 0 && is_row_major(out) &&
      is_row_major(indices) && aligned16(data->data) && aligned16(out->data)) {
    int64_t rows = numel(indices);
    FML_LAUNCH((embedding_rows), (unsigned)((rows * 32 + 255) / 256), 256, 0, s, 
        rows, data->shape[1], data->shape[0], (float *)out->data, (const float *)data->data,
        data->stride[0], (const int64_t *)indices->data, nullptr, 0, nullptr, 0, 1, status);
    FML_CUDA(cudaGetLastError());
    return FML_OK;
  }
  const int grid = grid_for(g.total, 256);
  switch (dtype_size(data->dtype)) {
  case 4: FML_LAUNCH((gather_generic<uint32_t>), grid, 256, 0, s, g, (uint32_t *)out->data, (const uint32_t *)data->data, (const int64_t *)indices->data, status); break;
  case 8: FML_LAUNCH((gather_generic<uint64_t>), grid, 256, 0, s, g, (uint64_t *)out->data, (const uint64_t *)data->data, (const int64_t *)indices->data, status); break;
  default: FML_LAUNCH((gather_generic<uint8_t>), grid, 256, 0, s, g, (uint8_t *)out->data, (const uint8_t *)data->data, (const int64_t *)indices->data, status); break;
  }
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

extern "C" int fml_embedding(const fml_tensor *table, const fml_tensor *ids, const fml_tensor *add0,
                             const fml_tensor *add1, const fml_tensor *out, void *stream) {
  GatherArgs g;
  int st = fill_gather(g, table, ids, out, 0, "fml_embedding");
  if (st != FML_OK) return st;
  FML_REQUIRE(table->dtype == FML_F32, FML_UNSUPPORTED, "fml_embedding: fp32 table only");
  if (g.total == 0) return FML_OK;
  int *status = device_status_word();
  FML_REQUIRE(status, FML_CUDA_ERROR, "fml_embedding: no device status word");
  Iter<3> add;
  add.rank = out->rank;
  for (int i = 0; i < out->rank; ++i) { add.shape[i] = out->shape[i]; add.stride[0][i] = out->stride[i]; }
  const fml_tensor *adds[2] = {add0, add1};
  for (int o = 0; o < 2; ++o) {
    if (!adds[o]) { for (int i = 0; i < out->rank; ++i) add.stride[o + 1][i] = 0; continue; }
    FML_REQUIRE(valid_tensor(adds[o]) && adds[o]->dtype == FML_F32, FML_BAD_ARG, "fml_embedding: bad addend");
    FML_REQUIRE(broadcast_strides(adds[o], out, add.stride[o + 1]), FML_BAD_ARG,
                "fml_embedding: addend does not broadcast to the output");
  }
  FML_LAUNCH((embedding_generic), grid_for(g.total, 256), 256, 0, as_stream(stream), 
      g, add, (float *)out->data, (const float *)table->data, (const int64_t *)ids->data,
      add0 ? (const float *)add0->data : nullptr, add1 ? (const float *)add1->data : nullptr, status);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

namespace fml {
namespace {
struct PadArgs {
  int rank;
  int64_t oshape[kMaxDims], ostride[kMaxDims], istride[kMaxDims], begin[kMaxDims], ishape[kMaxDims];
  int64_t total;
};
// One pass over the output: an element inside the window of the input copies it, the rest is
// zero.  (A fill followed by a copy of the interior would be two launches and write the interior
// twice.)
__global__ void pad_kernel(PadArgs a, float *out, const float *in) {
  pdl_prologue();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < a.total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t lin = i, oo = 0, io = 0;
    bool inside = true;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t q = lin / a.oshape[d], c = lin - q * a.oshape[d];
      lin = q;
      oo += c * a.ostride[d];
      const int64_t ci = c - a.begin[d];
      inside = inside && ci >= 0 && ci < a.ishape[d];
      io += ci * a.istride[d];
    }
    out[oo] = inside ? in[io] : 0.0f;
  }
}
}  // namespace
}  // namespace fml

extern "C" int fml_pad(const fml_tensor *in, const fml_tensor *out, const int64_t *pads_begin,
                       void *stream) {
  FML_REQUIRE(valid_tensor(in) && valid_tensor(out) && pads_begin, FML_BAD_ARG, "fml_pad: bad argument");
  FML_REQUIRE(in->rank == out->rank && in->dtype == out->dtype && in->dtype == FML_F32, FML_BAD_ARG,
              "fml_pad: rank/dtype mismatch (fp32 only)");
  fml::PadArgs a;
  a.rank = out->rank;
  a.total = 1;
  for (int i = 0; i < out->rank; ++i) {
    FML_REQUIRE(pads_begin[i] >= 0 && pads_begin[i] + in->shape[i] <= out->shape[i], FML_BAD_ARG,
                "fml_pad: pads do not fit the output");
    a.oshape[i] = out->shape[i]; a.ostride[i] = out->stride[i];
    a.ishape[i] = in->shape[i]; a.istride[i] = in->stride[i];
    a.begin[i] = pads_begin[i];
    a.total *= out->shape[i];
  }
  if (a.total == 0) return FML_OK;
  FML_LAUNCH((fml::pad_kernel), fml::grid_for(a.total, 256), 256, 0, fml::as_stream(stream), a, (float *)out->data,
             (const float *)in->data);
  return FML_OK;
}

namespace fml {
namespace {
struct ConcatArgs {
  int rank, axis;
  uint32_t shape[kMaxDims];            // output shape, the innermost extent in units of V elements
  int64_t ostride[kMaxDims], astride[kMaxDims], bstride[kMaxDims];
  uint32_t split;                      // extent of the first operand along `axis` (in units of V if axis is innermost)
  uint32_t total;                      // output elements / V
};
// Both halves of a two-operand Concat in one launch: an output element (or group of V along a
// contiguous innermost dim) reads the first operand below the split and the second above it.
template <typename T, int V>
__global__ void concat2_kernel(const ConcatArgs a, T *out, const T *lhs, const T *rhs) {
  pdl_prologue();
  struct alignas(sizeof(T) * V) Vec { T v[V]; };
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += gridDim.x * blockDim.x) {
    uint32_t lin = i;
    int64_t oo = 0, ao = 0, bo = 0;
    bool first = true;
    for (int d = a.rank - 1; d >= 0; --d) {
      uint32_t c = lin;
      if (d > 0) { const uint32_t q = lin / a.shape[d]; c = lin - q * a.shape[d]; lin = q; }
      const int64_t unit = d == a.rank - 1 ? V : 1;
      oo += (int64_t)c * unit * a.ostride[d];
      if (d == a.axis) {
        first = c < a.split;
        ao += (int64_t)c * unit * a.astride[d];
        bo += (int64_t)(c - a.split) * unit * a.bstride[d];
      } else {
        ao += (int64_t)c * unit * a.astride[d];
        bo += (int64_t)c * unit * a.bstride[d];
      }
    }
    *reinterpret_cast<Vec *>(out + oo) = *reinterpret_cast<const Vec *>(first ? lhs + ao : rhs + bo);
  }
}
}  // namespace
}  // namespace fml

extern "C" int fml_concat2(const fml_tensor *lhs, const fml_tensor *rhs, const fml_tensor *out, int axis, void *stream) {
  FML_REQUIRE(valid_tensor(lhs) && valid_tensor(rhs) && valid_tensor(out), FML_BAD_ARG, "fml_concat2: bad argument");
  FML_REQUIRE(lhs->rank == out->rank && rhs->rank == out->rank && lhs->dtype == out->dtype && rhs->dtype == out->dtype,
              FML_BAD_ARG, "fml_concat2: rank / dtype mismatch");
  FML_REQUIRE(axis >= 0 && axis < out->rank, FML_BAD_ARG, "fml_concat2: axis %d out of range", axis);
  int64_t total = 1;
  for (int i = 0; i < out->rank; ++i) {
    const int64_t want = i == axis ? lhs->shape[i] + rhs->shape[i] : lhs->shape[i];
    FML_REQUIRE(out->shape[i] == want && (i == axis || rhs->shape[i] == lhs->shape[i]), FML_BAD_ARG,
                "fml_concat2: shapes do not concatenate along axis %d", axis);
    total *= out->shape[i];
  }
  if (total == 0) return FML_OK;
  const size_t es = dtype_size(out->dtype);
  if (total >= (1ll << 31) || (es != 4 && es != 8 && es != 1)) {  // beyond 32-bit indexing: the two strided copies
    fml_tensor o0 = *out, o1 = *out;
    o0.shape[axis] = lhs->shape[axis];
    o1.shape[axis] = rhs->shape[axis];
    o1.data = (char *)out->data + lhs->shape[axis] * out->stride[axis] * (int64_t)es;
    int st = fml_copy_strided(lhs, &o0, stream);
    return st != FML_OK ? st : fml_copy_strided(rhs, &o1, stream);
  }
  fml::ConcatArgs a;
  a.rank = out->rank; a.axis = axis;
  const int l = out->rank - 1;
  // 16-byte groups along a contiguous innermost dim when every piece keeps the alignment
  int V = es == 4 ? 4 : 1;
  if (V == 4) {
    bool ok = out->stride[l] == 1 && lhs->stride[l] == 1 && rhs->stride[l] == 1 && out->shape[l] % 4 == 0 &&
              fml::aligned16(out->data) && fml::aligned16(lhs->data) && fml::aligned16(rhs->data) &&
              (axis != l || (lhs->shape[l] % 4 == 0 && rhs->shape[l] % 4 == 0));
    for (int d = 0; d < l && ok; ++d)
      ok = out->stride[d] % 4 == 0 && lhs->stride[d] % 4 == 0 && rhs->stride[d] % 4 == 0;
    if (!ok) V = 1;
  }
  for (int d = 0; d < out->rank; ++d) {
    a.shape[d] = (uint32_t)(d == l ? out->shape[d] / V : out->shape[d]);
    a.ostride[d] = out->stride[d]; a.astride[d] = lhs->stride[d]; a.bstride[d] = rhs->stride[d];
  }
  a.split = (uint32_t)(axis == l ? lhs->shape[axis] / V : lhs->shape[axis]);
  a.total = (uint32_t)(total / V);
  cudaStream_t s = fml::as_stream(stream);
  const int grid = fml::grid_for(a.total, 256);
  if (V == 4) FML_LAUNCH((fml::concat2_kernel<uint32_t, 4>), grid, 256, 0, s, a, (uint32_t *)out->data, (const uint32_t *)lhs->data, (const uint32_t *)rhs->data);
  else if (es == 4) FML_LAUNCH((fml::concat2_kernel<uint32_t, 1>), grid, 256, 0, s, a, (uint32_t *)out->data, (const uint32_t *)lhs->data, (const uint32_t *)rhs->data);
  else if (es == 8) FML_LAUNCH((fml::concat2_kernel<uint64_t, 1>), grid, 256, 0, s, a, (uint64_t *)out->data, (const uint64_t *)lhs->data, (const uint64_t *)rhs->data);
  else FML_LAUNCH((fml::concat2_kernel<uint8_t, 1>), grid, 256, 0, s, a, (uint8_t *)out->data, (const uint8_t *)lhs->data, (const uint8_t *)rhs->data);
  return FML_OK;
}
