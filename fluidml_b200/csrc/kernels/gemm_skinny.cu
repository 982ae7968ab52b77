// Skinny GEMM: C[M, N] = A[M, K] * B[K, N] for M <= 32 (the pooler, batch-1 classifier heads,
// VGG's fully connected layers at batch 1).  With so few rows the product is a stream over the
// weights: HBM-bound on B (K*N*4 bytes read once), CUDA-core FMAs in fp32, no tensor cores.
//
//   K-major B (b_sk == 1, e.g. Gemm with transB: weights stored [N, K]):
//       one warp per output column walks its K slice with 16-byte loads (lane-contiguous in
//       k), keeps M partial sums per lane and reduces them with shuffles;
//   N-major B (b_sn == 1, e.g. MatMul with weights stored [K, N]):
//       one thread per output column (lane-contiguous in n), A values broadcast from shared
//       memory.
//
// K is split over gridDim.y so that the grid covers the machine.  Each split writes its
// partial [M, tile] block to scratch memory; the split that arrives last on the tile's
// counter adds the partials in split order (results do not depend on arrival order), applies
// the epilogue and resets the counter.  The scratch (counters first, then partials) is global
// memory beyond the inputs and outputs, owned by the library per (device, stream).
#include "gemm_common.cuh"
#include <map>
#include <mutex>
#include <utility>

namespace fml {
namespace {

constexpr int kMaxM = 32;
constexpr int kColsPerCta = 32;  // output columns per CTA
constexpr int kThreads = 256;
constexpr size_t kCounterBytes = 64 << 10;  // 16384 tile counters

struct SkinnyArgs {
  GemmProblem p;
  GemmEpilogue e;
  int splits, tiles_n;
  int64_t k_per_split;
  unsigned *counters;  // one per (batch, n tile)
  float *partials;     // [batch * tiles_n][splits][M][kColsPerCta]
};

// FEW: the instantiation for at most four rows over 16-byte-aligned K-major operands (classifier
// heads and poolers at batch 1 to 4).  It holds only that path's registers (the general path's 32
// accumulators per lane made the shared kernel 176 registers = one CTA per SM = 12 % occupancy, and
// a 411 MB weight matrix streamed at 48 % of DRAM's cycles), so three CTAs share an SM.
template <bool KMAJOR, bool FEW>
__global__ void __launch_bounds__(kThreads, FEW ? 3 : 1) gemm_skinny_kernel(SkinnyArgs a) {
  pdl_launch_dependents();
  // B is what this kernel streams; while the preceding kernel drains, start it towards L2
  l2_prefetch_span(a.p.b, ((a.p.K - 1) * a.p.b_sk + (a.p.N - 1) * a.p.b_sn + 1) * (int64_t)sizeof(float), 4 << 20);
  pdl_wait();
  __shared__ float a_sh[KMAJOR ? 1 : kMaxM * 128];
  __shared__ float red[kMaxM][kColsPerCta];
  __shared__ int last_flag;
  const int M = (int)a.p.M;
  const int tile = blockIdx.x, split = blockIdx.y, z = blockIdx.z;
  const int64_t z0 = z % a.p.nb0, z1 = z / a.p.nb0;
  const float *A = a.p.a + z0 * a.p.a_b0 + z1 * a.p.a_b1;
  const float *B = a.p.b + z0 * a.p.b_b0 + z1 * a.p.b_b1;
  const int64_t n0 = (int64_t)tile * kColsPerCta;
  const int64_t k0 = (int64_t)split * a.k_per_split, k1 = min(a.p.K, k0 + a.k_per_split);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (KMAJOR) {
    // warp w owns columns n0 + w, n0 + w + 8, ... ; lanes stride over k in float4 steps
    const bool vec = a.p.a_sk == 1 && (a.p.a_sm & 3) == 0 && (a.p.b_sn & 3) == 0 && (k0 & 3) == 0 &&
                     ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0;
    // At most four rows (batch-1 classifier heads, the pooler): the warp takes its four columns
    // at once, so that eight weight loads are in flight per lane, the row chunks are loaded once
    // for all four columns, and the shuffle reductions are amortised.  Same per-lane summation
    // order as the general loop below.
    if (FEW) {  // the launcher checks `vec && M <= 4` before it picks this instantiation
      const int64_t kv = k0 + ((k1 - k0) & ~(int64_t)3);
      float acc4[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int m = 0; m < 4; ++m) acc4[j][m] = 0.0f;
      // columns past the edge of a ragged tile read the last column again (their sums are dropped below)
      const float *bcol[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) bcol[j] = B + min(n0 + warp * 4 + j, a.p.N - 1) * a.p.b_sn;
      auto dot4 = [](float4 x, float4 y, float t) { return fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, t)))); };
      int64_t k = k0 + lane * 4;
      for (; k + 128 < kv; k += 256) {
        float4 bw[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          bw[j][0] = __ldcs(reinterpret_cast<const float4 *>(bcol[j] + k));
          bw[j][1] = __ldcs(reinterpret_cast<const float4 *>(bcol[j] + k + 128));
        }
#pragma unroll
        for (int m = 0; m < 4; ++m)
          if (m < M) {
            const float4 a0 = *reinterpret_cast<const float4 *>(A + m * a.p.a_sm + k);
            const float4 a1 = *reinterpret_cast<const float4 *>(A + m * a.p.a_sm + k + 128);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc4[j][m] = dot4(a1, bw[j][1], dot4(a0, bw[j][0], acc4[j][m]));
          }
      }
      for (; k < kv; k += 128) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 bv = __ldcs(reinterpret_cast<const float4 *>(bcol[j] + k));
#pragma unroll
          for (int m = 0; m < 4; ++m)
            if (m < M) acc4[j][m] = dot4(*reinterpret_cast<const float4 *>(A + m * a.p.a_sm + k), bv, acc4[j][m]);
        }
      }
      for (int64_t kt = kv + lane; kt < k1; kt += 32)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float bv = bcol[j][kt];
#pragma unroll
          for (int m = 0; m < 4; ++m)
            if (m < M) acc4[j][m] = fmaf(A[m * a.p.a_sm + kt], bv, acc4[j][m]);
        }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int m = 0; m < 4; ++m)
          if (m < M) {
            float v = acc4[j][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[m][warp * 4 + j] = v;
          }
    }
    for (int c = FEW ? kColsPerCta : warp; c < kColsPerCta; c += kThreads / 32) {
      const int64_t n = n0 + c;
      float acc[kMaxM];
#pragma unroll
      for (int m = 0; m < kMaxM; ++m) acc[m] = 0.0f;
      if (n < a.p.N) {
        const float *brow = B + n * a.p.b_sn;
        if (vec) {
          const int64_t kv = k0 + ((k1 - k0) & ~(int64_t)3);
          int64_t k = k0 + lane * 4;
          // four independent 16-byte weight loads per lane and step: the kernel lives on memory-
          // level parallelism (weights are read once: streaming loads that do not pollute L1)
          for (; k + 384 < kv; k += 512) {
            const float4 b0 = __ldcs(reinterpret_cast<const float4 *>(brow + k));
            const float4 b1 = __ldcs(reinterpret_cast<const float4 *>(brow + k + 128));
            const float4 b2 = __ldcs(reinterpret_cast<const float4 *>(brow + k + 256));
            const float4 b3 = __ldcs(reinterpret_cast<const float4 *>(brow + k + 384));
#pragma unroll
            for (int m = 0; m < kMaxM; ++m)
              if (m < M) {
                const float *ap = A + m * a.p.a_sm + k;
                const float4 a0 = *reinterpret_cast<const float4 *>(ap), a1 = *reinterpret_cast<const float4 *>(ap + 128);
                const float4 a2 = *reinterpret_cast<const float4 *>(ap + 256), a3 = *reinterpret_cast<const float4 *>(ap + 384);
                float t = acc[m];
                t = fmaf(a0.x, b0.x, fmaf(a0.y, b0.y, fmaf(a0.z, b0.z, fmaf(a0.w, b0.w, t))));
                t = fmaf(a1.x, b1.x, fmaf(a1.y, b1.y, fmaf(a1.z, b1.z, fmaf(a1.w, b1.w, t))));
                t = fmaf(a2.x, b2.x, fmaf(a2.y, b2.y, fmaf(a2.z, b2.z, fmaf(a2.w, b2.w, t))));
                acc[m] = fmaf(a3.x, b3.x, fmaf(a3.y, b3.y, fmaf(a3.z, b3.z, fmaf(a3.w, b3.w, t))));
              }
          }
          for (; k < kv; k += 128) {
            const float4 bv = __ldcs(reinterpret_cast<const float4 *>(brow + k));
#pragma unroll
            for (int m = 0; m < kMaxM; ++m)
              if (m < M) {
                const float4 av = *reinterpret_cast<const float4 *>(A + m * a.p.a_sm + k);
                acc[m] = fmaf(av.x, bv.x, fmaf(av.y, bv.y, fmaf(av.z, bv.z, fmaf(av.w, bv.w, acc[m]))));
              }
          }
          for (int64_t k = kv + lane; k < k1; k += 32) {
            const float bv = brow[k];
#pragma unroll
            for (int m = 0; m < kMaxM; ++m)
              if (m < M) acc[m] = fmaf(A[m * a.p.a_sm + k], bv, acc[m]);
          }
        } else {
          for (int64_t k = k0 + lane; k < k1; k += 32) {
            const float bv = brow[k * a.p.b_sk];
#pragma unroll
            for (int m = 0; m < kMaxM; ++m)
              if (m < M) acc[m] = fmaf(A[m * a.p.a_sm + k * a.p.a_sk], bv, acc[m]);
          }
        }
      }
#pragma unroll
      for (int m = 0; m < kMaxM; ++m)
        if (m < M) {
          float v = acc[m];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) red[m][c] = v;
        }
    }
  } else {
    // thread (c, kq): column n0 + c, every 8th k of the slice; A staged in shared memory in
    // chunks of 128 k values
    const int c = threadIdx.x & 31, kq = threadIdx.x >> 5;
    const int64_t n = n0 + c;
    float acc[kMaxM];
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) acc[m] = 0.0f;
    for (int64_t kc = k0; kc < k1; kc += 128) {
      const int len = (int)min((int64_t)128, k1 - kc);
      __syncthreads();
      for (int i = threadIdx.x; i < M * 128; i += kThreads) {
        const int m = i >> 7, kk = i & 127;
        a_sh[i] = kk < len ? A[m * a.p.a_sm + (kc + kk) * a.p.a_sk] : 0.0f;
      }
      __syncthreads();
      if (n < a.p.N)
#pragma unroll 4
        for (int kk = kq; kk < len; kk += kThreads / 32) {
          const float bv = __ldcs(B + (kc + kk) * a.p.b_sk + n * a.p.b_sn);
#pragma unroll
          for (int m = 0; m < kMaxM; ++m)
            if (m < M) acc[m] = fmaf(a_sh[m * 128 + kk], bv, acc[m]);
        }
    }
    // reduce the 8 k-phases of each column through shared memory, in phase order
    for (int ph = 0; ph < kThreads / 32; ++ph) {
      __syncthreads();
      if (kq == ph)
#pragma unroll
        for (int m = 0; m < kMaxM; ++m)
          if (m < M) red[m][c] = (ph == 0 ? 0.0f : red[m][c]) + acc[m];
    }
  }
  __syncthreads();

  // red[m][c] = this split's partial sums.  Single split: finish directly.
  float *C = a.p.c + z0 * a.p.c_b0 + z1 * a.p.c_b1;
  const float *bias = a.p.bias ? a.p.bias + z0 * a.p.bias_b0 + z1 * a.p.bias_b1 : nullptr;
  const float *res = a.p.res ? a.p.res + z0 * a.p.res_b0 + z1 * a.p.res_b1 : nullptr;
  const int64_t tile_id = (int64_t)z * a.tiles_n + tile;
  if (a.splits > 1) {
    float *part = a.partials + ((tile_id * a.splits + split) * M) * kColsPerCta;
    for (int i = threadIdx.x; i < M * kColsPerCta; i += kThreads) part[i] = red[i / kColsPerCta][i % kColsPerCta];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_flag = atomicAdd(a.counters + tile_id, 1u) == (unsigned)a.splits - 1u;
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
  }
  for (int i = threadIdx.x; i < M * kColsPerCta; i += kThreads) {
    const int m = i / kColsPerCta, c = i % kColsPerCta;
    const int64_t n = n0 + c;
    if (n >= a.p.N) continue;
    float acc;
    if (a.splits > 1) {
      acc = 0.0f;
      const float *base = a.partials + (tile_id * a.splits * M) * kColsPerCta + i;
      for (int sp = 0; sp < a.splits; ++sp) acc += __ldcg(base + (int64_t)sp * M * kColsPerCta);
    } else {
      acc = red[m][c];
    }
    const float bv = bias ? bias[m * a.p.bias_sm + n * a.p.bias_sn] : 0.0f;
    const float rv = res ? res[m * a.p.res_sm + n * a.p.res_sn] : 0.0f;
    C[m * a.p.c_sm + n * a.p.c_sn] = gemm_epilogue(a.e, acc, bv, rv);
  }
  if (a.splits > 1 && threadIdx.x == 0) a.counters[tile_id] = 0u;  // ready for the next launch
}

struct SkinnyPlan {
  int splits, tiles_n;
  int64_t k_per_split;
  size_t counter_bytes, scratch_bytes;  // scratch = counters (256-byte aligned) + partials
};

SkinnyPlan plan_skinny(const GemmProblem &p) {
  SkinnyPlan pl;
  pl.tiles_n = (int)((p.N + kColsPerCta - 1) / kColsPerCta);
  const int64_t tiles = (int64_t)pl.tiles_n * p.nb0 * p.nb1;
  // enough CTAs for ~8 per SM, each split at least 256 k values long
  int64_t s = (148 * 8 + tiles - 1) / tiles;
  // (with at most four rows the kernel is a chain of load latencies, not arithmetic: slices of
  // 128 k values already pay there; more rows keep slices of at least 256)
  s = std::min<int64_t>(s, std::max<int64_t>(1, p.K / (p.M <= 4 ? 128 : 256)));
  s = std::max<int64_t>(1, std::min<int64_t>(s, 64));
  int64_t per = (p.K + s - 1) / s;
  per = (per + 127) / 128 * 128;  // keeps every slice start 16-byte aligned and chunked
  pl.k_per_split = per;
  pl.splits = (int)((p.K + per - 1) / per);
  // The counters live in a region of fixed size at the start of the scratch, so that partial
  // sums of one launch never land where a later launch of another shape keeps its counters
  // (they must read zero at launch).  Products with more tiles than counters run unsplit.
  if ((size_t)tiles * 4 > kCounterBytes) { pl.splits = 1; pl.k_per_split = p.K; }
  pl.counter_bytes = pl.splits > 1 ? kCounterBytes : 0;
  pl.scratch_bytes = pl.splits > 1 ? pl.counter_bytes + (size_t)tiles * pl.splits * p.M * kColsPerCta * 4 : 0;
  return pl;
}

int launch_skinny(const GemmProblem &p, const GemmEpilogue &e, const SkinnyPlan &pl, void *scratch, cudaStream_t s) {
  SkinnyArgs a;
  a.p = p; a.e = e;
  a.splits = pl.splits; a.k_per_split = pl.k_per_split; a.tiles_n = pl.tiles_n;
  a.counters = reinterpret_cast<unsigned *>(scratch);
  a.partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scratch) + pl.counter_bytes);
  const dim3 grid((unsigned)pl.tiles_n, (unsigned)pl.splits, (unsigned)(p.nb0 * p.nb1));
  if (p.b_sk == 1 && p.b_sn != 1) {
    // (k slices start at multiples of 128, so every slice keeps the 16-byte alignment of its row)
    const bool few = p.M <= 4 && p.a_sk == 1 && (p.a_sm & 3) == 0 && (p.b_sn & 3) == 0 && aligned16(p.a) && aligned16(p.b) &&
                     (p.a_b0 & 3) == 0 && (p.a_b1 & 3) == 0 && (p.b_b0 & 3) == 0 && (p.b_b1 & 3) == 0;
    if (few) FML_LAUNCH((gemm_skinny_kernel<true, true>), grid, kThreads, 0, s, a);
    else FML_LAUNCH((gemm_skinny_kernel<true, false>), grid, kThreads, 0, s, a);
  } else {
    FML_LAUNCH((gemm_skinny_kernel<false, false>), grid, kThreads, 0, s, a);
  }
  return FML_OK;
}

// Library-owned scratch, one buffer per (device, stream), grown on demand and cleared when it
// is (re)allocated.  Launches on one stream are ordered, so they can share it.
struct Scratch { void *ptr = nullptr; size_t bytes = 0; };
std::map<std::pair<int, cudaStream_t>, Scratch> g_scratch;
std::mutex g_scratch_mu;

int scratch_for(size_t bytes, cudaStream_t s, void **out) {
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  Scratch &sc = g_scratch[{dev, s}];
  if (sc.bytes < bytes) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cap);
    FML_REQUIRE(cap == cudaStreamCaptureStatusNone, FML_CUDA_ERROR,
                "fml_gemm: the skinny-GEMM scratch must grow (%zu bytes) but the stream is being captured; "
                "run the call once outside the capture first", bytes);
    FML_CUDA(cudaStreamSynchronize(s));
    if (sc.ptr) FML_CUDA(cudaFree(sc.ptr));
    sc.ptr = nullptr;
    sc.bytes = 0;
    const size_t want = std::max<size_t>(bytes, 1 << 20);
    FML_CUDA(cudaMalloc(&sc.ptr, want));
    FML_CUDA(cudaMemset(sc.ptr, 0, want));
    sc.bytes = want;
  }
  *out = sc.ptr;
  return FML_OK;
}

}  // namespace

bool skinny_eligible(const GemmProblem &p) {
  return p.M >= 1 && p.M <= kMaxM && p.K >= 1 && p.N >= 1 && p.nb0 * p.nb1 <= 65535 &&
         (p.N + kColsPerCta - 1) / kColsPerCta <= 0x7fffffff;
}

int launch_gemm_skinny(const GemmProblem &p, const GemmEpilogue &e, cudaStream_t s) {
  const SkinnyPlan pl = plan_skinny(p);
  void *scratch = nullptr;
  if (pl.scratch_bytes) {
    int st = scratch_for(pl.scratch_bytes, s, &scratch);
    if (st != FML_OK) return st;
  }
  return launch_skinny(p, e, pl, scratch, s);
}

size_t gemm_skinny_scratch_bytes(const GemmProblem &p) { return plan_skinny(p).scratch_bytes; }


// ---- the same product for callers that cannot let the library allocate ---------------------
//
// Some hosts may not have device memory allocated on their behalf while they call in: a
// serving loop that has handed all of HBM to its own pool, code that runs inside a section
// where cudaMalloc's implicit device synchronisation is not acceptable, or an embedding that
// audits every allocation.  fml_gemm's skinny path grows a cudaMalloc'ed scratch buffer on
// demand; the entry point below keeps its split-K counters and partial sums in an array that
// is part of the loaded module instead, so it never calls an allocating routine -- at the
// price of a fixed capacity.
constexpr size_t kStaticScratchBytes = 1 << 20;  // 64 KiB of tile counters + 960 KiB of partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void *g_static_scratch_addr[kMaxDevices] = {nullptr};  // per device: where the array lives
std::mutex g_static_mu;
}  // namespace

}  // namespace fml

using namespace fml;

// Declared in fluidml_cuda.h.  The first call on each device does the set-up: it asks the
// runtime where this device's copy of the array is (a host-side symbol is not a device
// address) and clears the counter region, which has to read zero when a launch starts
// (every launch leaves it zero again).  That first call enqueues a memset and waits for it,
// so make it before any stream capture.  All calls on one device share the one array: two
// calls whose kernels can overlap (different streams, no ordering between them) race on it.
extern "C" int fml_gemm_skinny_noalloc(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                                       const fml_tensor *bias, const fml_tensor *residual,
                                       const fml_gemm_params *gp, void *stream) {
  FML_REQUIRE(gp, FML_BAD_ARG, "fml_gemm_skinny_noalloc: null params");
  FML_REQUIRE(gp->precision == FML_GEMM_AUTO || gp->precision == FML_GEMM_FP32, FML_UNSUPPORTED,
              "fml_gemm_skinny_noalloc: computes in fp32 FMA only");
  GemmProblem p;
  int st = analyse_gemm(a, b, c, bias, residual, p);
  if (st != FML_OK) return st;
  if (p.M == 0 || p.N == 0 || p.nb0 * p.nb1 == 0) return FML_OK;
  FML_REQUIRE(skinny_eligible(p), FML_UNSUPPORTED,
              "fml_gemm_skinny_noalloc: needs 1 <= M <= %d rows and K >= 1 (M = %lld, K = %lld)", kMaxM,
              (long long)p.M, (long long)p.K);
  const SkinnyPlan pl = plan_skinny(p);
  FML_REQUIRE(pl.scratch_bytes <= kStaticScratchBytes, FML_OUT_OF_MEMORY,
              "fml_gemm_skinny_noalloc: this product needs %zu bytes of split-K scratch, the built-in "
              "buffer holds %zu; use fml_gemm", pl.scratch_bytes, kStaticScratchBytes);
  GemmEpilogue e;
  e.divisor = gp->divisor == 0.0f ? 1.0f : gp->divisor;
  e.alpha = gp->alpha; e.beta = gp->beta; e.act = gp->act;
  e.c0 = gp->act_param[0]; e.c1 = gp->act_param[1]; e.c2 = gp->act_param[2];
  e.has_bias = bias != nullptr; e.has_res = residual != nullptr;
  cudaStream_t s = as_stream(stream);
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  FML_REQUIRE(dev >= 0 && dev < kMaxDevices, FML_BAD_ARG, "fml_gemm_skinny_noalloc: device ordinal %d out of range", dev);
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_scratch_addr[dev]) {
      // The set-up below enqueues a memset and waits for it; inside a capture that would end up
      // in the caller's graph and the wait would invalidate the capture.  Refuse instead.
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      FML_CUDA(cudaStreamIsCapturing(s, &cap));
      FML_REQUIRE(cap == cudaStreamCaptureStatusNone, FML_CUDA_ERROR,
                  "fml_gemm_skinny_noalloc: the first call on a device sets up the scratch array and must be made "
                  "outside stream capture");
      void *addr = nullptr;
      FML_CUDA(cudaGetSymbolAddress(&addr, g_static_scratch));
      FML_REQUIRE(addr != nullptr, FML_CUDA_ERROR, "fml_gemm_skinny_noalloc: no device address for the scratch array");
      FML_CUDA(cudaMemsetAsync(addr, 0, kCounterBytes, s));
      FML_CUDA(cudaStreamSynchronize(s));  // set-up is complete when this call returns
      g_static_scratch_addr[dev] = addr;
    }
    scratch = g_static_scratch_addr[dev];
  }
  return launch_skinny(p, e, pl, scratch, s);
}
