// Depthwise convolution over dense NCHW planes whose rows are a multiple of four floats: the
// pipelined variant of the tiled kernel in conv.cu (conv.cpp:27-280 in the reference is one
// loop nest per output element).
//
// A depthwise layer does KH*KW multiply-adds per element it moves: its roof is HBM.  The tiled
// kernel stages a patch with ordinary loads, so a CTA has a few dozen KB in flight and its
// load, compute and store phases run one after the other.  Here a persistent CTA walks a list
// of tiles with two patch buffers in shared memory: one thread issues ONE tensor-map copy
// (cp.async.bulk.tensor, 3-D box = patch columns x patch rows x planes) per tile, which also
// produces the zero padding (coordinates outside the tensor read as zero), and the copy of
// tile i + 1 runs under the arithmetic and the stores of tile i.  Every thread still computes a
// micro-tile of 4 x 4 outputs from 16-byte shared-memory loads with the window in registers.
//
// The box starts four columns left of the image (a tensor-map copy must start on a 16-byte
// boundary; the padding itself is one or two columns), so a thread's aligned 16-byte reads
// begin at patch column 4 * strip * stride and the window sits OFF = 4 - pad columns into them.
#include "tc_common.cuh"

namespace fml {
namespace {

constexpr int kDwThreads = 256;
constexpr int kDwMaxStages = 4;
constexpr size_t kDwStageBytes = 36 * 1024;  // measured best cap for a patch buffer (18 / 26 / 36 / 52 / 100 KB tried)

// A persistent grid is as large as the device can hold at once (registers count as much as shared
// memory: the occupancy calculator knows both) and no larger than the tile list.
template <typename Kernel>
int persistent_ctas(Kernel kernel, size_t smem, int items, int *ctas) {
  int per_sm = 0, sms = 0, dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  FML_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  FML_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kDwThreads, smem));
  *ctas = std::max(1, std::min(items, std::max(1, per_sm) * std::max(1, sms)));
  return FML_OK;
}

struct DwTmaArgs {
  int C, OH, OW, ph;
  int TR, PP, SW;          // thread rows (of 4 output rows) per tile, planes per tile, strips per output row
  int PH, PWt;             // patch rows, patch columns (= the box's inner extent)
  int row_tiles, planes, items;
  int stages;              // patch buffers of a CTA
  const float *w;
  int64_t ws0, ws2, ws3;
  const float *bias;
  int64_t bias_stride;
  float *y;
  int64_t ys[4];
  int act;
  int *status;
};

__device__ __forceinline__ float dwt_act(int act, float v) {
  switch (act) {
  case FML_ACT_RELU: return fmaxf(v, 0.0f);
  case FML_ACT_TANH: return tanhf(v);
  case FML_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
  case FML_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
  default: return v;
  }
}
template <int ACT>
__device__ __forceinline__ void dwt_store_row(float *yp, const float *v, float bias, bool vec, int valid, int64_t ys3) {
  if (vec) {
    *reinterpret_cast<float4 *>(yp) = make_float4(dwt_act(ACT, v[0] + bias), dwt_act(ACT, v[1] + bias),
                                                  dwt_act(ACT, v[2] + bias), dwt_act(ACT, v[3] + bias));
  } else {
#pragma unroll
    for (int o = 0; o < 4; ++o)
      if (o < valid) yp[o * ys3] = dwt_act(ACT, v[o] + bias);
  }
}
__device__ __forceinline__ void dwt_tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int KH, int KW, int S>
__global__ void __launch_bounds__(kDwThreads) conv_depthwise_tma_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                         const DwTmaArgs d) {
  constexpr int RT = 4;                              // output rows per thread
  constexpr int PADW = (KW - 1) / 2, OFF = 4 - PADW;  // window offset inside a thread's aligned reads
  constexpr int IN_V = (OFF + 3 * S + KW + 3) / 4;   // 16-byte loads per input row of the micro-tile
  constexpr int ROWS = (RT - 1) * S + KH;            // input rows of the micro-tile
  extern __shared__ __align__(128) uint8_t dwt_smem[];
  __shared__ __align__(8) uint64_t bars[kDwMaxStages];
  const int NS = d.stages;
  __shared__ int abort_flag;
  const uint32_t stage_floats = (uint32_t)(d.PP * d.PH * d.PWt);
  const uint32_t stage_bytes = stage_floats * 4u;
  const uint32_t stage_pitch = (stage_bytes + 127u) & ~127u;  // a tensor-map copy lands on a 128-byte boundary
  uint8_t *smem = dwt_smem + ((128u - (smem_u32(dwt_smem) & 127u)) & 127u);
  const int tid = threadIdx.x;

  pdl_launch_dependents();
  if (tid == 0) {
    tma_prefetch_map(&map_x);
    for (int s = 0; s < NS; ++s) mbar_init(smem_u32(&bars[s]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();

  // thread -> (plane of the tile, thread row, strip)
  const int per_plane = d.TR * d.SW;
  const int pl = d.PP == 1 ? 0 : tid / per_plane, rem = tid - pl * per_plane;
  const int tr = rem / d.SW, j = rem - tr * d.SW;
  const bool worker = pl < d.PP && tr < d.TR;
  const int drop = g_drop_loads;

  auto issue = [&](int item, int stage) {  // thread 0 only
    const int tile = item / d.row_tiles, band = item - tile * d.row_tiles;
    const uint32_t bar = smem_u32(&bars[stage]);
    mbar_expect_tx(bar, stage_bytes);
    if (!drop)
      dwt_tma_load_3d(smem_u32(smem) + (uint32_t)stage * stage_pitch, &map_x, bar, -4, band * d.TR * RT * S - d.ph,
                      tile * d.PP);
  };

  int issued = 0, consumed = 0;
  const int first = (int)blockIdx.x, stride = (int)gridDim.x;
  if (tid == 0)
    for (int q = 0; q < NS - 1 && first + q * stride < d.items; ++q) { issue(first + q * stride, q); ++issued; }
  bool ok = true;
  for (int item = first, k = 0; item < d.items; item += stride, ++k) {
    const int stage = k % NS;
    // the buffer of the tile before this one was released by the barrier that ended its iteration
    if (tid == 0 && item + (NS - 1) * stride < d.items) { issue(item + (NS - 1) * stride, (k + NS - 1) % NS); ++issued; }
    const int tile = item / d.row_tiles, band = item - tile * d.row_tiles;
    const int plane = tile * d.PP + pl;
    const int oh = (band * d.TR + tr) * RT, ow0 = j * 4;
    const bool active = worker && plane < d.planes && oh < d.OH;
    // the window and the bias of this thread's plane travel while the patch does
    float w[KH * KW], bias = 0.0f;
    int ch = 0, n = 0;
    if (active) {
      n = plane / d.C;
      ch = plane - n * d.C;
#pragma unroll
      for (int q = 0; q < KH * KW; ++q) w[q] = __ldg(d.w + ch * d.ws0 + (q / KW) * d.ws2 + (q % KW) * d.ws3);
      if (d.bias) bias = __ldg(d.bias + ch * d.bias_stride);
    }
    // (the outcome is made uniform: a thread that gave up must not leave the others at the barrier below)
    ok = __syncthreads_and(mbar_wait(smem_u32(&bars[stage]), ((uint32_t)(k / NS)) & 1u, &abort_flag) ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0) consumed = k + 1;
    if (active) {
      float acc[RT][4];
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int o = 0; o < 4; ++o) acc[i][o] = 0.0f;  // window first, bias last: the reference's order
      const float *prow = reinterpret_cast<const float *>(smem + (size_t)stage * stage_pitch) +
                          ((size_t)pl * d.PH + (size_t)tr * RT * S) * d.PWt + ow0 * S;
#pragma unroll
      for (int ir = 0; ir < ROWS; ++ir) {
        float in[IN_V * 4];
#pragma unroll
        for (int v = 0; v < IN_V; ++v) {
          const float4 t = *reinterpret_cast<const float4 *>(prow + ir * d.PWt + v * 4);
          in[4 * v] = t.x; in[4 * v + 1] = t.y; in[4 * v + 2] = t.z; in[4 * v + 3] = t.w;
        }
#pragma unroll
        for (int rr = 0; rr < RT; ++rr) {
          const int kh = ir - rr * S;  // compile-time after unrolling
          if (kh >= 0 && kh < KH) {
#pragma unroll
            for (int kw = 0; kw < KW; ++kw)
#pragma unroll
              for (int o = 0; o < 4; ++o) acc[rr][o] = fmaf(in[OFF + o * S + kw], w[kh * KW + kw], acc[rr][o]);
          }
        }
      }
      float *yp = d.y + n * d.ys[0] + ch * d.ys[1] + oh * d.ys[2] + ow0 * d.ys[3];
      const int valid = d.OW - ow0;
      const bool vec = d.ys[3] == 1 && valid >= 4 && ((reinterpret_cast<uintptr_t>(yp) & 15) == 0) && (d.ys[2] & 3) == 0;
      const int rows = min(RT, d.OH - oh);
      switch (d.act) {  // one dispatch per thread, outside the store loops
#define FML_DWT_ROWS(ACT)                                                                 \
  _Pragma("unroll") for (int rr = 0; rr < RT; ++rr)                                          \
    if (rr < rows) dwt_store_row<ACT>(yp + rr * d.ys[2], acc[rr], bias, vec, valid, d.ys[3]);
      case FML_ACT_RELU: FML_DWT_ROWS(FML_ACT_RELU) break;
      case FML_ACT_TANH: FML_DWT_ROWS(FML_ACT_TANH) break;
      case FML_ACT_SIGMOID: FML_DWT_ROWS(FML_ACT_SIGMOID) break;
      case FML_ACT_SILU: FML_DWT_ROWS(FML_ACT_SILU) break;
      default: FML_DWT_ROWS(FML_ACT_NONE) break;
#undef FML_DWT_ROWS
      }
    }
    __syncthreads();  // every thread has read this buffer: the copy after next may overwrite it
  }
  if (!ok) {
    // a bounded wait ran out: report it, and (thread 0) give the copies already issued a bounded
    // chance to land before the CTA's shared memory is released
    if (tid == 0) {
      atomicOr(d.status, kStatusTimeout);
      abort_flag = 1;
      volatile int never = 0;
      if (!drop)
        for (int k = consumed; k < issued; ++k) mbar_wait(smem_u32(&bars[k % NS]), ((uint32_t)(k / NS)) & 1u, &never);
    }
  }
}

// ---- narrow planes (rows that are not a multiple of four floats, or shorter than 16: the 14 x 14
// and 7 x 7 stages of an image network).  A tensor map cannot describe such rows (their pitch is
// not a multiple of 16 bytes), but a run of whole planes is one contiguous block: the persistent
// CTA fetches PP planes per tile with one bulk copy (cp.async.bulk) into a ring of two raw
// buffers, repacks them into a zero-padded patch (shared memory to shared memory), and computes
// 4 x 4 micro-tiles from the patch as above; the copy of tile i + 1 runs under all of that.
struct DwFlatArgs {
  int C, IH, IW, OH, OW, ph, pw;
  int TR, PP, SW;            // thread rows per plane, planes per tile, strips per output row
  int PH, PWn, pitch;        // patch rows, patch columns, patch row pitch (floats)
  int planes, items;
  int dense_y;               // y is dense NCHW on a 16-byte base: a tile's results are one contiguous block
  uint32_t m_plane, m_pwn;   // ceil(2^32 / d) for d = PH * PWn and PWn (dividends below 2^16)
  const float *x;
  const float *w;
  int64_t ws0, ws2, ws3;
  const float *bias;
  int64_t bias_stride;
  float *y;
  int64_t ys[4];
  int act;
  int *status;
};

__device__ __forceinline__ void dwt_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int KH, int KW, int S>
__global__ void __launch_bounds__(kDwThreads) conv_depthwise_planes_kernel(const DwFlatArgs d) {
  constexpr int RT = 4;
  constexpr int IN_V = (3 * S + KW + 3) / 4;
  constexpr int ROWS = (RT - 1) * S + KH;
  extern __shared__ __align__(128) uint8_t dwt_smem[];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  const int HW = d.IH * d.IW;
  const uint32_t raw_pitch = ((uint32_t)(d.PP * HW) * 4u + 127u) & ~127u;
  uint8_t *smem = dwt_smem + ((128u - (smem_u32(dwt_smem) & 127u)) & 127u);
  float *patch = reinterpret_cast<float *>(smem + 2 * (size_t)raw_pitch);  // [PP][PH][pitch]
  // results of a tile, dense [PP][OH * OW]: with y dense they leave as ONE bulk copy (rows of 7 or
  // 14 floats stored by the threads themselves are 4-byte writes scattered over partial sectors)
  const int OHW = d.OH * d.OW;
  float *out_s = patch + (((size_t)d.PP * d.PH * d.pitch + 31) & ~(size_t)31);
  const int tid = threadIdx.x;

  pdl_launch_dependents();
  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();

  const int per_plane = d.TR * d.SW;
  const int pl = tid / per_plane, rem = tid - pl * per_plane;
  const int tr = rem / d.SW, j = rem - tr * d.SW;
  const bool worker = pl < d.PP;
  const int drop = g_drop_loads;
  const int per_plane_elems = d.PH * d.PWn, patch_elems = d.PP * per_plane_elems;

  auto issue = [&](int item, int stage) {  // thread 0 only: the planes [item * PP, ...) of the tensor
    const int count = min(d.PP, d.planes - item * d.PP);
    const uint32_t bytes = (uint32_t)(count * HW) * 4u;
    const uint32_t bar = smem_u32(&bars[stage]);
    mbar_expect_tx(bar, bytes);
    if (!drop) dwt_bulk_load(smem_u32(smem) + (uint32_t)stage * raw_pitch, d.x + (size_t)item * d.PP * HW, bytes, bar);
  };

  int issued = 0, consumed = 0;
  const int first = (int)blockIdx.x, stride = (int)gridDim.x;
  if (tid == 0 && first < d.items) { issue(first, 0); issued = 1; }
  bool ok = true;
  for (int item = first, k = 0; item < d.items; item += stride, ++k) {
    const int stage = k & 1;
    if (tid == 0 && item + stride < d.items) { issue(item + stride, stage ^ 1); ++issued; }  // released after the repack of tile k - 1
    const int plane = item * d.PP + pl;
    const int oh = tr * RT, ow0 = j * 4;
    const bool active = worker && plane < d.planes && oh < d.OH;
    float w[KH * KW], bias = 0.0f;
    int ch = 0, n = 0;
    if (active) {  // the window and the bias of this thread's plane travel while the planes do
      n = plane / d.C;
      ch = plane - n * d.C;
#pragma unroll
      for (int q = 0; q < KH * KW; ++q) w[q] = __ldg(d.w + ch * d.ws0 + (q / KW) * d.ws2 + (q % KW) * d.ws3);
      if (d.bias) bias = __ldg(d.bias + ch * d.bias_stride);
    }
    ok = __syncthreads_and(mbar_wait(smem_u32(&bars[stage]), ((uint32_t)(k >> 1)) & 1u, &abort_flag) ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0) consumed = k + 1;
    // ---- repack: raw planes -> zero-padded patch (the previous tile's readers left it at the
    // barrier that ended their iteration)
    {
      const float *raw = reinterpret_cast<const float *>(smem + (size_t)stage * raw_pitch);
      for (int base = tid; base < patch_elems; base += 4 * kDwThreads) {
        float v[4];
        int at[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int e = base + kDwThreads * u;
          v[u] = 0.0f;
          at[u] = -1;
          if (e < patch_elems) {
            const int p = (int)__umulhi((uint32_t)e, d.m_plane), r2 = e - p * per_plane_elems;
            const int pr = (int)__umulhi((uint32_t)r2, d.m_pwn), pc = r2 - pr * d.PWn;
            const int ih = pr - d.ph, iw = pc - d.pw;
            at[u] = (p * d.PH + pr) * d.pitch + pc;
            if ((unsigned)ih < (unsigned)d.IH && (unsigned)iw < (unsigned)d.IW) v[u] = raw[p * HW + ih * d.IW + iw];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (at[u] >= 0) patch[at[u]] = v[u];
      }
    }
    // the previous tile's results have left shared memory before this tile's are written
    if (d.dense_y && tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncthreads();
    if (active) {
      float acc[RT][4];
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int o = 0; o < 4; ++o) acc[i][o] = 0.0f;  // window first, bias last: the reference's order
      const float *prow = patch + ((size_t)pl * d.PH + (size_t)tr * RT * S) * d.pitch + ow0 * S;
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
      const int valid = d.OW - ow0;
      const int rows = min(RT, d.OH - oh);
      if (d.dense_y) {
        float *op = out_s + (size_t)pl * OHW + oh * d.OW + ow0;
        switch (d.act) {  // one dispatch per thread, outside the store loops
#define FML_DWT_SROWS(ACT)                                                                \
  _Pragma("unroll") for (int rr = 0; rr < RT; ++rr)                                          \
    if (rr < rows) dwt_store_row<ACT>(op + rr * d.OW, acc[rr], bias, false, valid, 1);
        case FML_ACT_RELU: FML_DWT_SROWS(FML_ACT_RELU) break;
        case FML_ACT_TANH: FML_DWT_SROWS(FML_ACT_TANH) break;
        case FML_ACT_SIGMOID: FML_DWT_SROWS(FML_ACT_SIGMOID) break;
        case FML_ACT_SILU: FML_DWT_SROWS(FML_ACT_SILU) break;
        default: FML_DWT_SROWS(FML_ACT_NONE) break;
#undef FML_DWT_SROWS
        }
      } else {
        float *yp = d.y + n * d.ys[0] + ch * d.ys[1] + oh * d.ys[2] + ow0 * d.ys[3];
        const bool vec = d.ys[3] == 1 && valid >= 4 && ((reinterpret_cast<uintptr_t>(yp) & 15) == 0) && (d.ys[2] & 3) == 0;
        switch (d.act) {
#define FML_DWT_ROWS(ACT)                                                                 \
  _Pragma("unroll") for (int rr = 0; rr < RT; ++rr)                                          \
    if (rr < rows) dwt_store_row<ACT>(yp + rr * d.ys[2], acc[rr], bias, vec, valid, d.ys[3]);
        case FML_ACT_RELU: FML_DWT_ROWS(FML_ACT_RELU) break;
        case FML_ACT_TANH: FML_DWT_ROWS(FML_ACT_TANH) break;
        case FML_ACT_SIGMOID: FML_DWT_ROWS(FML_ACT_SIGMOID) break;
        case FML_ACT_SILU: FML_DWT_ROWS(FML_ACT_SILU) break;
        default: FML_DWT_ROWS(FML_ACT_NONE) break;
#undef FML_DWT_ROWS
        }
      }
    }
    __syncthreads();  // the patch may be rebuilt; the tile's results are complete
    if (d.dense_y && tid == 0) {
      const int count = min(d.PP, d.planes - item * d.PP);
      fence_async_smem();  // the threads' writes, before the copy engine reads them
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                   ::"l"(d.y + (size_t)item * d.PP * OHW), "r"(smem_u32(out_s)), "r"((uint32_t)(count * OHW) * 4u) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
  }
  if (d.dense_y && tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores complete before the CTA leaves
  if (!ok && tid == 0) {
    atomicOr(d.status, kStatusTimeout);
    abort_flag = 1;
    volatile int never = 0;
    if (!drop)
      for (int k = consumed; k < issued; ++k) mbar_wait(smem_u32(&bars[k & 1]), ((uint32_t)(k >> 1)) & 1u, &never);
  }
}

template <int KH, int KW, int S>
int launch_planes_variant(const DwFlatArgs &d, size_t smem, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    FML_CUDA(cudaFuncSetAttribute(conv_depthwise_planes_kernel<KH, KW, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[dev & 63] = true;
  }
  int ctas = 1;
  const int st = persistent_ctas(conv_depthwise_planes_kernel<KH, KW, S>, smem, d.items, &ctas);
  if (st != FML_OK) return st;
  FML_LAUNCH((conv_depthwise_planes_kernel<KH, KW, S>), dim3((unsigned)ctas), dim3(kDwThreads), smem, s, d);
  return FML_OK;
}

// The narrow-plane variant: dense NCHW x on a 16-byte base, planes of at most 1024 elements that
// fit one CTA's threads, a plane count that is a multiple of 4 (so that every copy is a multiple
// of 16 bytes).
bool launch_depthwise_planes(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias, const fml_tensor *y,
                             const fml_conv_params *p, cudaStream_t s, int *status) {
  const int64_t N = x->shape[0], C = x->shape[1], IH = x->shape[2], IW = x->shape[3];
  const int64_t OH = y->shape[2], OW = y->shape[3], KH = w->shape[2], KW = w->shape[3];
  const int64_t S = p->strides[0], HW = IH * IW;
  if (HW > 1024 || ((N * C) & 3) || N * C >= (1ll << 30)) return false;
  if (p->pads_begin[0] < 0 || p->pads_begin[0] > 8 || p->pads_begin[1] < 0 || p->pads_begin[1] > 8) return false;
  constexpr int RT = 4;
  DwFlatArgs d;
  memset(&d, 0, sizeof(d));
  d.C = (int)C; d.IH = (int)IH; d.IW = (int)IW; d.OH = (int)OH; d.OW = (int)OW;
  d.ph = (int)p->pads_begin[0]; d.pw = (int)p->pads_begin[1];
  d.SW = (int)((OW + 3) / 4);
  d.TR = (int)((OH + RT - 1) / RT);
  const int per_plane = d.TR * d.SW;
  if (per_plane > kDwThreads / 4) return false;  // at least four planes per tile
  const int in_v = (3 * (int)S + (int)KW + 3) / 4;
  d.PWn = (d.SW - 1) * 4 * (int)S + in_v * 4;
  d.pitch = d.PWn + 4;  // rows 16 bytes apart modulo the bank cycle
  d.PH = (d.TR * RT - 1) * (int)S + (int)KH;
  d.planes = (int)(N * C);
  d.PP = std::min(kDwThreads / per_plane / 4 * 4, d.planes);
  static const int bulk_store_env = [] { const char *e = getenv("FLUIDML_DEPTHWISE_BULK_STORE"); return e ? atoi(e) : -1; }();
  // (measured: the block store pays at stride 1, +10-20 %; at stride 2 the extra buffer costs more than it saves)
  d.dense_y = (bulk_store_env == 1 || (bulk_store_env < 0 && S == 1)) && aligned16(y->data) && y->stride[3] == 1 && y->stride[2] == OW && y->stride[1] == OH * OW &&
                      (N == 1 || y->stride[0] == C * OH * OW) ? 1 : 0;
  auto smem_of = [&]() {
    const size_t raw = ((size_t)d.PP * HW * 4 + 127) / 128 * 128;
    const size_t patch = ((size_t)d.PP * d.PH * d.pitch + 31) / 32 * 32 * 4;
    return 2 * raw + patch + (d.dense_y ? (size_t)d.PP * OH * OW * 4 : 0) + 128;
  };
  while (d.PP > 4 && smem_of() > 56 * 1024) d.PP -= 4;
  if (smem_of() > 100 * 1024 || (int64_t)d.PP * d.PH * d.PWn >= 65536) return false;
  d.items = (d.planes + d.PP - 1) / d.PP;
  auto magic = [](int64_t dv) { return (uint32_t)((0x100000000ull + (uint64_t)dv - 1) / (uint64_t)dv); };
  d.m_plane = magic((int64_t)d.PH * d.PWn); d.m_pwn = magic(d.PWn);
  d.x = (const float *)x->data;
  d.w = (const float *)w->data; d.ws0 = w->stride[0]; d.ws2 = w->stride[2]; d.ws3 = w->stride[3];
  if (bias) {
    d.bias = (const float *)bias->data;
    for (int i = 0; i < bias->rank; ++i) if (bias->shape[i] != 1) d.bias_stride = bias->stride[i];
  }
  d.y = (float *)y->data;
  for (int i = 0; i < 4; ++i) d.ys[i] = y->stride[i];
  d.act = p->act;
  d.status = device_status_word();
  if (!d.status) return false;
  const size_t smem = smem_of();
  const int key = (int)(KH * 10 + S);
  switch (key) {
  case 31: *status = launch_planes_variant<3, 3, 1>(d, smem, s); break;
  case 32: *status = launch_planes_variant<3, 3, 2>(d, smem, s); break;
  case 51: *status = launch_planes_variant<5, 5, 1>(d, smem, s); break;
  default: *status = launch_planes_variant<5, 5, 2>(d, smem, s); break;
  }
  return true;
}

using DwKernelFn = void (*)(const CUtensorMap, const DwTmaArgs);

template <int KH, int KW, int S>
int launch_variant(const CUtensorMap &map, const DwTmaArgs &d, size_t smem, cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    FML_CUDA(cudaFuncSetAttribute(conv_depthwise_tma_kernel<KH, KW, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[dev & 63] = true;
  }
  int ctas = 1;
  const int st = persistent_ctas(conv_depthwise_tma_kernel<KH, KW, S>, smem, d.items, &ctas);
  if (st != FML_OK) return st;
  FML_LAUNCH((conv_depthwise_tma_kernel<KH, KW, S>), dim3((unsigned)ctas), dim3(kDwThreads), smem, s, map, d);
  return FML_OK;
}

}  // namespace

// Takes the layer when it can: x dense NCHW with rows of a multiple of four floats on a 16-byte
// base, y with unit column stride, 3 x 3 or 5 x 5 window with "same" column padding, stride 1 or
// 2 in both directions, dilation 1.  Returns false (nothing launched, *status untouched) otherwise.
bool launch_depthwise_tma(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias, const fml_tensor *y,
                          const fml_conv_params *p, cudaStream_t s, int *status) {
  static const bool enabled = [] { const char *e = getenv("FLUIDML_DEPTHWISE_TMA"); return !(e && e[0] == '0'); }();
  if (!enabled || x->rank != 4 || y->rank != 4 || w->rank != 4) return false;
  const int64_t N = x->shape[0], C = x->shape[1], IH = x->shape[2], IW = x->shape[3];
  const int64_t OH = y->shape[2], OW = y->shape[3], KH = w->shape[2], KW = w->shape[3];
  const int64_t S = p->strides[0];
  if (p->strides[1] != S || (S != 1 && S != 2) || p->dilations[0] != 1 || p->dilations[1] != 1) return false;
  if (!((KH == 3 && KW == 3) || (KH == 5 && KW == 5))) return false;
  if (!aligned16(x->data) || x->stride[3] != 1 || x->stride[2] != IW || x->stride[1] != IH * IW ||
      (N > 1 && x->stride[0] != C * IH * IW))
    return false;
  if (N * C >= (1ll << 30) || IH >= (1 << 20) || y->stride[3] != 1) return false;
  for (int i = 0; i < 4; ++i) if (y->stride[i] < 0) return false;
  if ((IW & 3) || IW < 16) return launch_depthwise_planes(x, w, bias, y, p, s, status);
  if (p->pads_begin[1] != (KW - 1) / 2 || p->pads_begin[0] < 0 || p->pads_begin[0] > 8) return false;
  constexpr int RT = 4;
  DwTmaArgs d;
  memset(&d, 0, sizeof(d));
  d.C = (int)C; d.OH = (int)OH; d.OW = (int)OW; d.ph = (int)p->pads_begin[0];
  d.SW = (int)((OW + 3) / 4);
  const int RW = (int)((OH + RT - 1) / RT);
  if (d.SW > kDwThreads) return false;
  const int off = 4 - (int)(KW - 1) / 2, in_v = (off + 3 * (int)S + (int)KW + 3) / 4;
  d.PWt = (d.SW - 1) * 4 * (int)S + in_v * 4;
  if (d.PWt % 32 == 0) d.PWt += 4;  // consecutive patch rows start in different banks
  if (d.PWt > 256) return false;
  const int per_plane = RW * d.SW;
  d.row_tiles = 1;
  if (per_plane <= kDwThreads) {
    d.TR = RW; d.PP = kDwThreads / per_plane;
  } else {
    const int tr_max = kDwThreads / d.SW;
    d.row_tiles = (RW + tr_max - 1) / tr_max;
    d.TR = (RW + d.row_tiles - 1) / d.row_tiles;
    d.PP = 1;
  }
  d.planes = (int)(N * C);
  if (d.PP > d.planes) d.PP = d.planes;
  auto stage_bytes = [&]() {
    d.PH = (d.TR * RT - 1) * (int)S + (int)KH;
    return (size_t)d.PP * d.PH * d.PWt * sizeof(float);
  };
  static const size_t stage_cap = [] { const char *e = getenv("FLUIDML_DEPTHWISE_STAGE_KB"); return e ? (size_t)atoi(e) * 1024 : kDwStageBytes; }();
  while (stage_bytes() > stage_cap || d.PH > 256 || d.PP > 256) {  // fewer planes, then shorter bands
    if (d.PP > 1) { d.PP = (d.PP + 1) / 2; continue; }
    if (d.TR == 1) return false;
    d.row_tiles += 1;
    d.TR = (RW + d.row_tiles - 1) / d.row_tiles;
  }
  d.row_tiles = (RW + d.TR - 1) / d.TR;
  const size_t stage = stage_bytes();
  const int64_t items = (int64_t)((d.planes + d.PP - 1) / d.PP) * d.row_tiles;
  if (items > 0x7fffffff) return false;
  d.items = (int)items;
  d.w = (const float *)w->data; d.ws0 = w->stride[0]; d.ws2 = w->stride[2]; d.ws3 = w->stride[3];
  if (bias) {
    d.bias = (const float *)bias->data;
    for (int i = 0; i < bias->rank; ++i) if (bias->shape[i] != 1) d.bias_stride = bias->stride[i];
  }
  d.y = (float *)y->data;
  for (int i = 0; i < 4; ++i) d.ys[i] = y->stride[i];
  d.act = p->act;
  d.status = device_status_word();
  if (!d.status) return false;
  CUtensorMap map;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)IW, (cuuint64_t)IH, (cuuint64_t)(N * C)};
    const cuuint64_t str[2] = {(cuuint64_t)IW * 4, (cuuint64_t)IH * IW * 4};
    const cuuint32_t box[3] = {(cuuint32_t)d.PWt, (cuuint32_t)d.PH, (cuuint32_t)d.PP};
    if (make_f32_tensor_map(&map, (const float *)x->data, 3, dims, str, box) != FML_OK) return false;
  }
  static const int stages_env = [] { const char *e = getenv("FLUIDML_DEPTHWISE_STAGES"); return e ? atoi(e) : 0; }();
  d.stages = stages_env >= 2 && stages_env <= kDwMaxStages ? stages_env : 2;  // measured: more resident CTAs beat deeper rings
  const size_t smem = d.stages * ((stage + 127) / 128 * 128) + 128;
  const int key = (int)(KH * 10 + S);
  switch (key) {
  case 31: *status = launch_variant<3, 3, 1>(map, d, smem, s); break;
  case 32: *status = launch_variant<3, 3, 2>(map, d, smem, s); break;
  case 51: *status = launch_variant<5, 5, 1>(map, d, smem, s); break;
  default: *status = launch_variant<5, 5, 2>(map, d, smem, s); break;
  }
  return true;
}

}  // namespace fml
