// The gate of a squeeze-and-excite block in one launch:
//
//   gate[n, c] = act2(b2[c] + sum_j w2[c, j] * act1(b1[j] + sum_k w1[j, k] * mean_hw(x[n, k, :, :])))
//
// i.e. ReduceMean over the two spatial axes followed by two 1 x 1 convolutions over the single
// remaining pixel (reference kernels reduce_mean.cpp:16-98 and conv.cpp:27-280 run as three loop
// nests).  The three steps move a few kilobytes each and are pure dependency latency when
// launched separately; here one cluster of up to eight CTAs owns an image: every CTA averages
// its share of the channels into its own shared memory, the cluster synchronises once, every
// CTA pulls the other shares through distributed shared memory (at most a few KB), computes
// the whole hidden vector (redundantly: it is tiny) and then the gate of its own channels.
// No scratch memory, no atomics; the summation order is fixed, so results are bit-stable.
#include <algorithm>

#include "common.cuh"

namespace fml {
namespace {

constexpr int kSeThreads = 256;
constexpr int kSeWarps = kSeThreads / 32;
constexpr int kSeMaxCluster = 8;
constexpr int kSeMaxChannels = 4096;
constexpr int kSeMaxHidden = 512;
constexpr int kSeDepth = 24;                // loads a lane keeps in flight
constexpr int kSeMaxUnits = 2048;           // (plane, part) pairs of one CTA
constexpr size_t kSeStageBytes = 96 * 1024;  // weight rows a CTA keeps in shared memory

struct SeArgs {
  const float *x;
  int64_t xs[4];
  int N, C, H, W, Cr;
  const float *w1; int64_t w1s[2];  // [Cr, C]
  const float *b1; int64_t b1s;
  const float *w2; int64_t w2s[2];  // [C, Cr]
  const float *b2; int64_t b2s;
  float *gate; int64_t gs[2];
  int act1, act2;
  int per_rank;     // channels per CTA of the cluster
  int hid_per_rank; // hidden units per CTA
  int plane_dense;  // x[n, c, :, :] is H * W consecutive floats
  int vec;          // ... that can be read as float4
  int lanes;        // lanes that share one (plane, part) unit: 32, 16, 8, 4 or 2
  int parts;        // pieces a plane is cut into
  int part_len;     // elements (float4 when vec, else float) per piece
  int stage_w;      // the CTA's weight rows fit in shared memory
};

__device__ __forceinline__ float se_act(int act, float v) {
  switch (act) {
  case FML_ACT_RELU: return fmaxf(v, 0.0f);
  case FML_ACT_TANH: return tanhf(v);
  case FML_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
  case FML_ACT_SILU: return v * (1.0f / (1.0f + expf(-v)));
  default: return v;
  }
}
__device__ __forceinline__ float se_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ uint32_t se_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void se_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void se_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// value `index` of the float array at shared-memory address `base` (the same address in every CTA) of CTA `rank`
__device__ __forceinline__ float se_peer_load(uint32_t base, int index, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(base + 4u * (uint32_t)index), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
// Loads as volatile asm statements: the compiler keeps them in program order ahead of se_keep(),
// so a lane has all of a batch's loads in flight before it waits for the first.
__device__ __forceinline__ float4 se_ldg4(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float se_ldg1(const float *p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void se_keep(float4 &v) { asm volatile("" : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w)); }
// rows x cols block of a strided matrix into dense shared memory; 16-byte loads when the rows allow
__device__ __forceinline__ void se_stage(float *dst, const float *src, int rows, int cols, int64_t row_stride, int64_t col_stride) {
  const bool v4 = col_stride == 1 && (cols & 3) == 0 && (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  if (v4) {
    const int c4 = cols >> 2, total = rows * c4;
#pragma unroll 8
    for (int i = threadIdx.x; i < total; i += kSeThreads) {
      const int r = i / c4, c = i - r * c4;
      reinterpret_cast<float4 *>(dst)[i] = __ldg(reinterpret_cast<const float4 *>(src + (int64_t)r * row_stride) + c);
    }
  } else {
    const int total = rows * cols;
#pragma unroll 8
    for (int i = threadIdx.x; i < total; i += kSeThreads) {
      const int r = i / cols, c = i - r * cols;
      dst[i] = __ldg(src + (int64_t)r * row_stride + (int64_t)c * col_stride);
    }
  }
}

__global__ void __launch_bounds__(kSeThreads) squeeze_excite_gate_kernel(const SeArgs a) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) float se_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t rank = se_cluster_rank();
  const int n = blockIdx.y;
  const int c0 = min(a.C, (int)rank * a.per_rank), c1 = min(a.C, c0 + a.per_rank), planes = c1 - c0;
  const int j0 = min(a.Cr, (int)rank * a.hid_per_rank), j1 = min(a.Cr, j0 + a.hid_per_rank), hids = j1 - j0;
  const int HW = a.H * a.W;
  // shared-memory map (every CTA of the cluster uses the same offsets: peers address `own` and `hid_own`)
  float *w1_s = se_smem;                                                   // [hid_per_rank][C]     (stage_w)
  float *w2_s = w1_s + (a.stage_w ? (size_t)a.hid_per_rank * a.C : 0);     // [per_rank][Cr]        (stage_w)
  float *own = w2_s + (a.stage_w ? (size_t)a.per_rank * a.Cr : 0);         // [per_rank] means of this CTA's channels
  float *hid_own = own + a.per_rank;                                       // [hid_per_rank] this CTA's hidden units
  float *mean_s = hid_own + a.hid_per_rank;                                // [C]
  float *hid_s = mean_s + a.C;                                             // [Cr]
  float *b1_s = hid_s + a.Cr;                                              // [hid_per_rank]
  float *b2_s = b1_s + a.hid_per_rank;                                     // [per_rank]
  float *part_s = b2_s + a.per_rank;                                       // [planes * parts]

  // ---- 0. this CTA's weight rows and biases: constants, fetched before the dependency wait
  if (a.stage_w) {
    se_stage(w1_s, a.w1 + (int64_t)j0 * a.w1s[0], hids, a.C, a.w1s[0], a.w1s[1]);
    se_stage(w2_s, a.w2 + (int64_t)c0 * a.w2s[0], planes, a.Cr, a.w2s[0], a.w2s[1]);
  }
  for (int j = threadIdx.x; j < hids; j += kSeThreads) b1_s[j] = a.b1 ? __ldg(a.b1 + (int64_t)(j0 + j) * a.b1s) : 0.0f;
  for (int c = threadIdx.x; c < planes; c += kSeThreads) b2_s[c] = a.b2 ? __ldg(a.b2 + (int64_t)(c0 + c) * a.b2s) : 0.0f;
  pdl_wait();

  // ---- 1. means of the CTA's channels.  A unit is one piece of one plane, summed by `lanes`
  // lanes with all their loads in flight at once; the pieces of a plane are then added in order.
  {
    const float *xn = a.x + (int64_t)n * a.xs[0];
    const int L = a.lanes, groups = 32 / L, units = planes * a.parts;
    const int E = a.vec ? HW >> 2 : HW;
    const int g = lane / L, li = lane - g * L;
    for (int u0 = warp * groups; u0 < units; u0 += kSeWarps * groups) {
      const int u = u0 + g;
      float s = 0.0f;
      if (u < units) {
        const int pl = u / a.parts, pt = u - pl * a.parts;
        const int e0 = pt * a.part_len, e1 = min(E, e0 + a.part_len);
        const float *p = xn + (int64_t)(c0 + pl) * a.xs[1];
        if (a.vec) {
          // kSeDepth independent 16-byte loads per lane before the first add: the CTA lives on
          // memory-level parallelism (one cluster per image leaves most of the machine idle)
          const float4 *p4 = reinterpret_cast<const float4 *>(p);
          for (int b = e0 + li; b < e1; b += kSeDepth * L) {
            float4 v[kSeDepth];
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) {
              const int i = b + k * L;
              v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              if (i < e1) v[k] = se_ldg4(p4 + i);
            }
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) se_keep(v[k]);  // every load is issued before the first add
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
          }
        } else if (a.plane_dense) {
          for (int b = e0 + li; b < e1; b += kSeDepth * L) {
            float v[kSeDepth];
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) {
              const int i = b + k * L;
              v[k] = 0.0f;
              if (i < e1) v[k] = se_ldg1(p + i);
            }
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) asm volatile("" : "+f"(v[k]));  // every load is issued before the first add
#pragma unroll
            for (int k = 0; k < kSeDepth; ++k) s += v[k];
          }
        } else {
#pragma unroll 4
          for (int i = e0 + li; i < e1; i += L) {
            const int h = i / a.W, w = i - h * a.W;
            s += __ldg(p + (int64_t)h * a.xs[2] + (int64_t)w * a.xs[3]);
          }
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (li == 0 && u < units) part_s[u] = s;
    }
    __syncthreads();
    for (int pl = threadIdx.x; pl < planes; pl += kSeThreads) {
      float t = 0.0f;
      for (int pt = 0; pt < a.parts; ++pt) t += part_s[pl * a.parts + pt];
      own[pl] = t / (float)HW;
    }
  }

  // ---- 2. every CTA gathers all means of the image
  se_cluster_arrive();
  se_cluster_wait();
  {
    const uint32_t own_addr = (uint32_t)__cvta_generic_to_shared(own);
    for (int c = threadIdx.x; c < a.C; c += kSeThreads) {
      const int q = c / a.per_rank;
      mean_s[c] = se_peer_load(own_addr, c - q * a.per_rank, (uint32_t)q);
    }
  }
  __syncthreads();

  // ---- 3. this CTA's hidden units: one warp per unit, lanes along the channels
  for (int j = warp; j < hids; j += kSeWarps) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int k = lane;
    if (a.stage_w) {
      const float *wr = w1_s + (size_t)j * a.C;
      for (; k + 96 < a.C; k += 128) {
        s0 = fmaf(wr[k], mean_s[k], s0);
        s1 = fmaf(wr[k + 32], mean_s[k + 32], s1);
        s2 = fmaf(wr[k + 64], mean_s[k + 64], s2);
        s3 = fmaf(wr[k + 96], mean_s[k + 96], s3);
      }
      for (; k < a.C; k += 32) s0 = fmaf(wr[k], mean_s[k], s0);
    } else {
      const float *wr = a.w1 + (int64_t)(j0 + j) * a.w1s[0];
#pragma unroll 2
      for (; k + 96 < a.C; k += 128) {
        s0 = fmaf(__ldg(wr + (int64_t)k * a.w1s[1]), mean_s[k], s0);
        s1 = fmaf(__ldg(wr + (int64_t)(k + 32) * a.w1s[1]), mean_s[k + 32], s1);
        s2 = fmaf(__ldg(wr + (int64_t)(k + 64) * a.w1s[1]), mean_s[k + 64], s2);
        s3 = fmaf(__ldg(wr + (int64_t)(k + 96) * a.w1s[1]), mean_s[k + 96], s3);
      }
      for (; k < a.C; k += 32) s0 = fmaf(__ldg(wr + (int64_t)k * a.w1s[1]), mean_s[k], s0);
    }
    const float s = se_warp_sum((s0 + s1) + (s2 + s3));
    if (lane == 0) hid_own[j] = se_act(a.act1, s + b1_s[j]);
  }

  // ---- 4. every CTA gathers the hidden vector (the barrier also tells the peers that this CTA
  // has finished reading their means)
  se_cluster_arrive();
  se_cluster_wait();
  {
    const uint32_t hid_addr = (uint32_t)__cvta_generic_to_shared(hid_own);
    for (int j = threadIdx.x; j < a.Cr; j += kSeThreads) {
      const int q = j / a.hid_per_rank;
      hid_s[j] = se_peer_load(hid_addr, j - q * a.hid_per_rank, (uint32_t)q);
    }
  }
  // nobody leaves while a peer may still read its hidden units: arrive now, wait at the end
  se_cluster_arrive();
  __syncthreads();

  // ---- 5. gate of the CTA's channels: one thread per channel
  for (int c = threadIdx.x; c < planes; c += kSeThreads) {
    float s = 0.0f;
    if (a.stage_w) {
      const float *wr = w2_s + (size_t)c * a.Cr;
      for (int j = 0; j < a.Cr; ++j) s = fmaf(wr[j], hid_s[j], s);
    } else {
      const float *wr = a.w2 + (int64_t)(c0 + c) * a.w2s[0];
#pragma unroll 8
      for (int j = 0; j < a.Cr; ++j) s = fmaf(__ldg(wr + (int64_t)j * a.w2s[1]), hid_s[j], s);
    }
    a.gate[(int64_t)n * a.gs[0] + (int64_t)(c0 + c) * a.gs[1]] = se_act(a.act2, s + b2_s[c]);
  }
  se_cluster_wait();
}

}  // namespace
}  // namespace fml

using namespace fml;

extern "C" int fml_squeeze_excite_gate(const fml_tensor *x, const fml_tensor *w1, const fml_tensor *b1,
                                       const fml_tensor *w2, const fml_tensor *b2, int act1, int act2,
                                       const fml_tensor *gate, void *stream) {
  FML_REQUIRE(valid_tensor(x) && valid_tensor(w1) && valid_tensor(w2) && valid_tensor(gate), FML_BAD_ARG,
              "fml_squeeze_excite_gate: bad argument");
  FML_REQUIRE(x->dtype == FML_F32 && w1->dtype == FML_F32 && w2->dtype == FML_F32 && gate->dtype == FML_F32,
              FML_UNSUPPORTED, "fml_squeeze_excite_gate: fp32 only");
  FML_REQUIRE(x->rank == 4 && gate->rank == 4 && w1->rank >= 2 && w2->rank >= 2, FML_BAD_ARG,
              "fml_squeeze_excite_gate: x and gate are [N, C, H, W] / [N, C, 1, 1], weights [out, in(, 1, 1)]");
  for (int i = 2; i < w1->rank; ++i) FML_REQUIRE(w1->shape[i] == 1, FML_BAD_ARG, "fml_squeeze_excite_gate: w1 must be 1 x 1");
  for (int i = 2; i < w2->rank; ++i) FML_REQUIRE(w2->shape[i] == 1, FML_BAD_ARG, "fml_squeeze_excite_gate: w2 must be 1 x 1");
  SeArgs a;
  memset(&a, 0, sizeof(a));
  a.N = (int)x->shape[0]; a.C = (int)x->shape[1]; a.H = (int)x->shape[2]; a.W = (int)x->shape[3];
  a.Cr = (int)w1->shape[0];
  FML_REQUIRE(w1->shape[1] == a.C && w2->shape[0] == a.C && w2->shape[1] == a.Cr, FML_BAD_ARG,
              "fml_squeeze_excite_gate: weight shapes must be [Cr, C] and [C, Cr]");
  FML_REQUIRE(gate->shape[0] == a.N && gate->shape[1] == a.C && gate->shape[2] == 1 && gate->shape[3] == 1, FML_BAD_ARG,
              "fml_squeeze_excite_gate: gate shape must be [N, C, 1, 1]");
  FML_REQUIRE(act1 >= FML_ACT_NONE && act1 <= FML_ACT_SILU && act1 != FML_ACT_GELU_ERF && act2 >= FML_ACT_NONE &&
                  act2 <= FML_ACT_SILU && act2 != FML_ACT_GELU_ERF,
              FML_BAD_ARG, "fml_squeeze_excite_gate: activations are none, relu, tanh, sigmoid or silu");
  if (a.N == 0 || a.C == 0) return FML_OK;
  FML_REQUIRE(a.C <= kSeMaxChannels && a.Cr >= 1 && a.Cr <= kSeMaxHidden && a.N <= 65535 &&
                  (int64_t)a.H * a.W >= 1 && (int64_t)a.H * a.W < (1ll << 31),
              FML_UNSUPPORTED, "fml_squeeze_excite_gate: at most %d channels, %d hidden units, 65535 images",
              kSeMaxChannels, kSeMaxHidden);
  for (int i = 0; i < 4; ++i) a.xs[i] = x->stride[i];
  a.x = (const float *)x->data;
  a.w1 = (const float *)w1->data; a.w1s[0] = w1->stride[0]; a.w1s[1] = w1->stride[1];
  a.w2 = (const float *)w2->data; a.w2s[0] = w2->stride[0]; a.w2s[1] = w2->stride[1];
  if (b1) {
    FML_REQUIRE(valid_tensor(b1) && b1->dtype == FML_F32 && numel(b1) == a.Cr, FML_BAD_ARG, "fml_squeeze_excite_gate: b1 holds one value per hidden unit");
    a.b1 = (const float *)b1->data;
    for (int i = 0; i < b1->rank; ++i) if (b1->shape[i] != 1) a.b1s = b1->stride[i];
  }
  if (b2) {
    FML_REQUIRE(valid_tensor(b2) && b2->dtype == FML_F32 && numel(b2) == a.C, FML_BAD_ARG, "fml_squeeze_excite_gate: b2 holds one value per channel");
    a.b2 = (const float *)b2->data;
    for (int i = 0; i < b2->rank; ++i) if (b2->shape[i] != 1) a.b2s = b2->stride[i];
  }
  a.gate = (float *)gate->data; a.gs[0] = gate->stride[0]; a.gs[1] = gate->stride[1];
  a.act1 = act1; a.act2 = act2;
  a.plane_dense = (a.W == 1 || x->stride[3] == 1) && (a.H == 1 || x->stride[2] == a.W) ? 1 : 0;
  const int64_t HW = (int64_t)a.H * a.W;
  a.vec = a.plane_dense && (HW & 3) == 0 && aligned16(a.x) && (x->stride[0] & 3) == 0 && (x->stride[1] & 3) == 0 ? 1 : 0;
  // cluster size: eight CTAs per image unless the image has fewer than eight channels
  int ranks = kSeMaxCluster;
  while (ranks > 1 && a.C < ranks) ranks >>= 1;
  a.per_rank = (a.C + ranks - 1) / ranks;
  a.hid_per_rank = (a.Cr + ranks - 1) / ranks;
  // lanes per unit: up to 16 loads per lane for short planes; long planes are cut so that no lane has more than kSeDepth
  const int64_t E = a.vec ? HW >> 2 : HW;
  a.lanes = 2;
  while (a.lanes < 32 && (int64_t)a.lanes * 16 < E) a.lanes <<= 1;
  a.parts = 1;
  if (a.lanes == 32) {
    a.parts = (int)std::min<int64_t>((E + 32 * kSeDepth - 1) / (32 * kSeDepth), std::max(1, kSeMaxUnits / a.per_rank));
    if (a.parts < 1) a.parts = 1;
  }
  a.part_len = (int)((E + a.parts - 1) / a.parts);
  const size_t stage_bytes = ((size_t)a.hid_per_rank * a.C + (size_t)a.per_rank * a.Cr) * sizeof(float);
  a.stage_w = (((size_t)a.hid_per_rank * a.C) & 3) == 0 && stage_bytes <= kSeStageBytes ? 1 : 0;
  const size_t smem = (a.stage_w ? stage_bytes : 0) +
                      ((size_t)2 * a.per_rank + 2 * a.hid_per_rank + a.C + a.Cr + (size_t)a.per_rank * a.parts) * sizeof(float);
  {
    static bool attr_set[64] = {false};
    int dev = 0;
    FML_CUDA(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
      FML_CUDA(cudaFuncSetAttribute(squeeze_excite_gate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      attr_set[dev & 63] = true;
    }
  }

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)ranks, (unsigned)a.N, 1);
  cfg.blockDim = dim3(kSeThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;  // the CTAs of one image share a cluster
  attr[0].val.clusterDim.x = (unsigned)ranks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  FML_CUDA(cudaLaunchKernelEx(&cfg, squeeze_excite_gate_kernel, a));
  return FML_OK;
}
