// Persistent kernel of a resident stage program (see resident.cuh for the data model and
// resident_plan.cu for the planner): a chain of GEMM (+ bias / activation / residual /
// LayerNorm) and attention stages over one block of 128 activation rows runs inside one
// launch, one CTA per SM.  It replaces the reference's single compiled function per model
// (src/worker/builder.cpp:400-491 assembles it, src/worker/runner.cpp:101-112 calls it) for
// the operators MatMulKernel / GemmConstantBiasKernel (matmul.cpp:28-59, gemm.cpp:39-182),
// SoftmaxKernel (softmax.cpp:22-139) and LayerNormalizationConstantScaleBiasKernel
// (layer_normalization.cpp:33-220).
//
// Why one kernel.  At 128 rows a pass over an encoder layer is a chain of dependent operators
// of a few microseconds each; as separate launches each pays kernel exit, the next kernel's
// wake-up and a cold start of its weight stream, and HBM idles in between.  Here
//   * the weights of ALL stages are packed at creation into one stream per CTA, already in the
//     shared-memory image the tensor core reads (K-major rows of 128 bytes, 128-byte swizzle).
//     Warp 0 copies that stream into a ring of shared-memory slots with plain bulk copies
//     (cp.async.bulk, no tensor map, no multicast) and never waits for activations: weights
//     arrive while the CTA is still synchronising or reducing the previous stage;
//   * stages are ordered by counters in global memory: a step adds one to its counters when
//     its stores are visible (release), a consumer polls (acquire, bounded) just before it
//     needs the data, so only true dependencies wait, not whole grids;
//   * activations stay in a tiled order (resident.cuh) that every role reads and writes as
//     full cache lines straight from registers.
//
// Roles of a CTA (320 threads):
//   warp 0     weight producer (one lane);
//   warp 1     allocates TMEM, one lane issues tcgen05.mma kind::tf32 and the commits;
//   warps 2-5  converters: thread = activation row = TMEM lane.  Per k block they load the row's
//              32 A values from L2, split them into hi = x & 0xffffe000 and lo = x - hi (exact)
//              and write both to tensor memory; they write lo(B) next to the landed B tile (the
//              tensor core ignores the low 13 bits, so the landed tile is hi(B)).  The issuer
//              then adds lo*hi + hi*lo + hi*hi into one accumulator (3xTF32).  After the last
//              k block they move the accumulator to the partial buffer of their k split;
//   warps 2-9  together run the SIMT steps: the split-K reduction with its epilogue (bias,
//              activation, residual, LayerNorm over the row) and the attention core.
//
// Every wait is bounded.  When one gives up, the CTA records kStatusTimeout, raises the
// program-wide abort word, and from then on every wait of every CTA returns at once: the step
// lists are still walked to the end (so that barrier counts stay uniform), copies in flight are
// awaited, TMEM is freed and the kernel returns.
#include "resident.cuh"
#include "resident_host.h"
#include "tc_common.cuh"

namespace fml {
namespace res {
namespace {

constexpr uint32_t kPollLimit = 1u << 21;
constexpr uint32_t kAccCol = 0;      // accumulator tile: TMEM columns [0, 256)
constexpr uint32_t kACol = 256;      // A operand: 64 columns (32 hi, 32 lo) per converter stage

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned *p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async16(float *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Ctx {
  volatile int *abort_flag;  // shared memory: this CTA has given up (or learnt that another did)
  unsigned *abort_word;      // global memory: some CTA has given up
  int *status;
};
__device__ __forceinline__ void give_up(const Ctx &c) {
  atomicOr(c.status, kStatusTimeout);
  atomicExch(c.abort_word, 1u);
  *c.abort_flag = 1;
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const Ctx &c) {
  if (mbar_wait(bar, parity, c.abort_flag)) return true;
  give_up(c);
  return false;
}
// Waits until every counter the step names has reached its target.  One thread calls this.
__device__ bool poll_step(const Step &st, unsigned *counters, const Ctx &c) {
  for (int w = 0; w < st.nwait; ++w) {
    const unsigned *ctr = counters + st.wait_ctr[w];
    const unsigned target = st.wait_target[w];
    uint32_t it = 0;
    while (ld_acquire(ctr) < target) {
      if (*c.abort_flag) return false;
      if ((++it & 31u) == 0u) {
        if (ld_relaxed(c.abort_word)) { *c.abort_flag = 1; return false; }
        if (it > kPollLimit) { give_up(c); return false; }
      }
    }
  }
  return !*c.abort_flag;
}
__device__ __forceinline__ Step load_step(const Step *p) {
  Step s;
  const uint4 *src = reinterpret_cast<const uint4 *>(p);
  uint4 *dst = reinterpret_cast<uint4 *>(&s);
#pragma unroll
  for (int i = 0; i < (int)(sizeof(Step) / 16); ++i) dst[i] = __ldg(src + i);
  return s;
}

__device__ __forceinline__ float act_apply(int act, float c0, float c1, float c2, float v) {
  switch (act) {
  case FML_ACT_GELU_ERF: return v * (erff(v / c0) + c1) * c2;
  case FML_ACT_RELU: return fmaxf(v, 0.0f);
  case FML_ACT_TANH: return tanhf(v);
  case FML_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
  default: return v;
  }
}

// ---------------------------------------------------------------- finish step (256 threads)
// Sum of the S partial tiles at one (quad, row), in split order.
__device__ __forceinline__ float4 sum_partials(const float4 *p, size_t split_stride, int S) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  int s = 0;
  for (; s + 4 <= S; s += 4) {
    const float4 t0 = __ldcg(p), t1 = __ldcg(p + split_stride), t2 = __ldcg(p + 2 * split_stride),
                 t3 = __ldcg(p + 3 * split_stride);
    acc.x += t0.x; acc.y += t0.y; acc.z += t0.z; acc.w += t0.w;
    acc.x += t1.x; acc.y += t1.y; acc.z += t1.z; acc.w += t1.w;
    acc.x += t2.x; acc.y += t2.y; acc.z += t2.z; acc.w += t2.w;
    acc.x += t3.x; acc.y += t3.y; acc.z += t3.z; acc.w += t3.w;
    p += 4 * split_stride;
  }
  for (; s < S; ++s) {
    const float4 t = __ldcg(p);
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    p += split_stride;
  }
  return acc;
}

// value before LayerNorm at (row r, quad c): act(sum + bias) + residual
__device__ __forceinline__ float4 finish_value(const GemmStage &G, int r, int c) {
  const size_t split_stride = (size_t)(G.N >> 2) * kRows;
  float4 v = sum_partials(reinterpret_cast<const float4 *>(G.partial) + (size_t)c * kRows + r, split_stride, G.S);
  if (G.bias) {
    const float4 b = __ldg(reinterpret_cast<const float4 *>(G.bias) + c);
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  if (G.act != FML_ACT_NONE) {
    v.x = act_apply(G.act, G.c0, G.c1, G.c2, v.x); v.y = act_apply(G.act, G.c0, G.c1, G.c2, v.y);
    v.z = act_apply(G.act, G.c0, G.c1, G.c2, v.z); v.w = act_apply(G.act, G.c0, G.c1, G.c2, v.w);
  }
  if (G.res) {
    const float4 t = G.res_tiled ? __ldcg(reinterpret_cast<const float4 *>(G.res) + (size_t)c * kRows + r)
                                 : __ldcg(reinterpret_cast<const float4 *>(G.res + (size_t)r * G.res_ld) + c);
    v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
  }
  return v;
}
__device__ __forceinline__ void finish_store(const GemmStage &G, int r, int c, float4 v) {
  if (G.out_tiled) reinterpret_cast<float4 *>(G.out_tiled)[(size_t)c * kRows + r] = v;
  if (G.out_rm) reinterpret_cast<float4 *>(G.out_rm + (size_t)r * G.out_ld)[c] = v;
}

__device__ void finish_step(const GemmStage &G, const Step &st, int wt, float *red) {
  const int r0 = st.p0, r1 = st.p1, c0 = st.p2, c1 = st.p3;
  if (!G.ln) {
    const int nr = r1 - r0, items = nr * (c1 - c0);
    for (int i = wt; i < items; i += kWorkers) {  // consecutive threads on consecutive rows: 16-byte neighbours
      const int cc = i / nr, rr = i - cc * nr;
      finish_store(G, r0 + rr, c0 + cc, finish_value(G, r0 + rr, c0 + cc));
    }
    return;
  }
  // LayerNorm over whole rows (c0 = 0, c1 = N / 4 <= 1024): a thread keeps up to four quads of the row
  const int ww = wt >> 5, lane = wt & 31;
  const float inv_n = 1.0f / (float)G.N;
  for (int r = r0; r < r1; ++r) {
    float4 v[4];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = wt + kWorkers * i;
      if (c < c1) {
        v[i] = finish_value(G, r, c);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    s = warp_sum(s);
    if (lane == 0) red[ww] = s;
    bar_sync(2, kWorkers);
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float mean = tot * inv_n;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (wt + kWorkers * i < c1) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    q = warp_sum(q);
    if (lane == 0) red[8 + ww] = q;
    bar_sync(2, kWorkers);
    float qt = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) qt += red[8 + w];
    const float inv = 1.0f / sqrtf(qt * inv_n + G.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = wt + kWorkers * i;
      if (c < c1) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(G.gamma) + c), b = __ldg(reinterpret_cast<const float4 *>(G.beta) + c);
        finish_store(G, r, c, make_float4(v[i].x * inv * g.x + b.x, v[i].y * inv * g.y + b.y,
                                          v[i].z * inv * g.z + b.z, v[i].w * inv * g.w + b.w));
      }
    }
  }
}

// ---------------------------------------------------------------- attention step (256 threads)
// rows x cols block of a tiled matrix -> dst[r * pitch + c], asynchronous 16-byte copies
__device__ __forceinline__ void load_tiled(float *dst, int pitch, const float *mat, int col0, int row0, int rows,
                                           int cols, int wt) {
  const int c4 = cols >> 2;
  const float4 *src = reinterpret_cast<const float4 *>(mat) + (size_t)(col0 >> 2) * kRows + row0;
  for (int i = wt; i < rows * c4; i += kWorkers) {
    const int cc = i / rows, r = i - cc * rows;
    cp_async16(dst + r * pitch + 4 * cc, src + (size_t)cc * kRows + r);
  }
}

// softmax(Q K^T / divisor + mask) V for 16 query rows of one head; the arithmetic and the thread
// mapping are those of attention_kernel (attention.cu), the operands come from tiled matrices.
__device__ void attention_step(const AttnStage &A, int head, int row0, float *smem, int wt) {
  const int D = A.D, Dv = A.Dv, Sk = A.Sk;
  const int pk = D + 4, pp = Sk | 1;
  float *Qs = smem;
  float *Ks = Qs + kAttnRows * pk;
  float *Vs = Ks + (size_t)Sk * pk;
  float *Red = Vs + (size_t)Sk * Dv;
  float *Ps = Red + 8 * kAttnRows * Dv;
  float *Ms = Ps + kAttnRows * pp;
  const int warp = wt >> 5, lane = wt & 31;
  load_tiled(Qs, pk, A.q, A.q_col + head * A.q_hs, row0, kAttnRows, D, wt);
  load_tiled(Ks, pk, A.k, A.k_col + head * A.k_hs, 0, Sk, D, wt);
  cp_async_commit();
  load_tiled(Vs, Dv, A.v, A.v_col + head * A.v_hs, 0, Sk, Dv, wt);
  cp_async_commit();
  const int mrows = A.mask ? (A.m_sr == 0 ? 1 : kAttnRows) : 0;
  if (mrows) {
    const float *m = A.mask + head * A.m_sh + (A.m_sr ? row0 * A.m_sr : 0);
    for (int i = wt; i < mrows * Sk; i += kWorkers) {
      const int r = i / Sk, j = i - r * Sk;
      Ms[i] = __ldg(m + r * A.m_sr + j * A.m_sk);
    }
  }
  cp_async_wait<1>();
  bar_sync(2, kWorkers);
  // ---- scores
  {
    const int half = warp >> 2, rq = warp & 3, cq = lane;
    const int n4 = D >> 2, d_lo = half ? n4 >> 1 : 0, d_hi = half ? n4 : n4 >> 1;
    for (int jb = 0; jb < Sk; jb += 128) {
      float acc[4][4];
      const float4 *k4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[x][u] = 0.0f;
        k4[u] = reinterpret_cast<const float4 *>(Ks + (size_t)min(jb + cq + 32 * u, Sk - 1) * pk);
      }
      const float4 *q4 = reinterpret_cast<const float4 *>(Qs + rq * pk);
#pragma unroll 2
      for (int d = d_lo; d < d_hi; ++d) {
        float4 qv[4], kv[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) qv[x] = q4[x * pk + d];
#pragma unroll
        for (int u = 0; u < 4; ++u) kv[u] = k4[u][d];
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            acc[x][u] = fmaf(qv[x].x, kv[u].x, acc[x][u]);
            acc[x][u] = fmaf(qv[x].y, kv[u].y, acc[x][u]);
            acc[x][u] = fmaf(qv[x].z, kv[u].z, acc[x][u]);
            acc[x][u] = fmaf(qv[x].w, kv[u].w, acc[x][u]);
          }
      }
      for (int turn = 0; turn < 2; ++turn) {  // the first half stores, the second adds: a fixed order
        if (turn == half) {
#pragma unroll
          for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = jb + cq + 32 * u;
              if (j < Sk) {
                float *dst = Ps + (rq + 4 * x) * pp + j;
                *dst = turn ? *dst + acc[x][u] : acc[x][u];
              }
            }
        }
        bar_sync(2, kWorkers);
      }
    }
  }
  cp_async_wait<0>();
  bar_sync(2, kWorkers);
  // ---- softmax over each row; a row's 16 threads are half a warp
  {
    const int r = wt >> 4, cg = wt & 15;
    float *p = Ps + r * pp;
    const float *mr = Ms + (mrows > 1 ? r * Sk : 0);
    float mx = -3.402823466e+38f;
    for (int j = cg; j < Sk; j += 16) {
      float sc = p[j];
      if (A.divisor != 1.0f) sc = sc / A.divisor;
      if (mrows) sc += mr[j];
      p[j] = sc;
      mx = fmaxf(mx, sc);
    }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
    float sum = 0.0f;
    for (int j = cg; j < Sk; j += 16) {
      const float e = expf(p[j] - mx);
      p[j] = e;
      sum += e;
    }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
    for (int j = cg; j < Sk; j += 16) p[j] = p[j] / sum;
  }
  bar_sync(2, kWorkers);
  // ---- context
  {
    const int rg = lane >> 3, cgp = lane & 7;
    const int per = (Sk + 7) >> 3, j_lo = min(Sk, warp * per), j_hi = min(Sk, j_lo + per);
    const float *p0 = Ps + rg * pp;
    for (int dv0 = 0; dv0 < Dv; dv0 += 64) {
      const int ca = dv0 + cgp * 4, cb = ca + 32;
      const bool has_a = ca < Dv, has_b = cb < Dv;
      float4 acc[4][2];
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[x][0] = acc[x][1] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
      for (int j = j_lo; j < j_hi; ++j) {
        const float *vr = Vs + (size_t)j * Dv;
        const float4 va = has_a ? *reinterpret_cast<const float4 *>(vr + ca) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 vb = has_b ? *reinterpret_cast<const float4 *>(vr + cb) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float pj = p0[4 * x * pp + j];
          acc[x][0].x = fmaf(pj, va.x, acc[x][0].x); acc[x][0].y = fmaf(pj, va.y, acc[x][0].y);
          acc[x][0].z = fmaf(pj, va.z, acc[x][0].z); acc[x][0].w = fmaf(pj, va.w, acc[x][0].w);
          acc[x][1].x = fmaf(pj, vb.x, acc[x][1].x); acc[x][1].y = fmaf(pj, vb.y, acc[x][1].y);
          acc[x][1].z = fmaf(pj, vb.z, acc[x][1].z); acc[x][1].w = fmaf(pj, vb.w, acc[x][1].w);
        }
      }
      if (dv0) bar_sync(2, kWorkers);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        float *dst = Red + ((size_t)warp * kAttnRows + rg + 4 * x) * Dv;
        if (has_a) *reinterpret_cast<float4 *>(dst + ca) = acc[x][0];
        if (has_b) *reinterpret_cast<float4 *>(dst + cb) = acc[x][1];
      }
      bar_sync(2, kWorkers);
      const int w4 = min(64, Dv - dv0) >> 2;
      const int oc = A.o_col + head * A.o_hs;
      for (int i = wt; i < kAttnRows * w4; i += kWorkers) {  // rows fastest: 16-byte neighbours in the tiled order
        const int cc = i / kAttnRows, r = i - cc * kAttnRows, c = dv0 + (cc << 2);
        float4 t = *reinterpret_cast<const float4 *>(Red + (size_t)r * Dv + c);
#pragma unroll
        for (int w = 1; w < 8; ++w) {
          const float4 u = *reinterpret_cast<const float4 *>(Red + ((size_t)w * kAttnRows + r) * Dv + c);
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        if (A.out_tiled) reinterpret_cast<float4 *>(A.out_tiled)[(size_t)((oc + c) >> 2) * kRows + row0 + r] = t;
        if (A.out_rm) *reinterpret_cast<float4 *>(A.out_rm + (size_t)(row0 + r) * A.out_ld + oc + c) = t;
      }
    }
  }
}

// ---------------------------------------------------------------- the kernel
template <bool TRACE>
__global__ void __launch_bounds__(kThreads, 1) resident_kernel(const KernelArgs g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // [ weight ring: nslots x slot_bytes | overlay: lo(B) slots of the converter stages, or the
  //   attention step's tiles | mbarriers | TMEM slot, abort flag, reduction scratch ]
  const int nslots = g.nslots;
  const uint32_t slot_bytes = (uint32_t)g.slot_bytes;
  uint8_t *overlay = smem + (size_t)nslots * slot_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(overlay + g.overlay_bytes);
  const uint32_t ring_addr = smem_u32(smem), lo_addr = smem_u32(overlay);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8u * nslots;
  const uint32_t bar_conv = bar_empty + 8u * nslots;
  const uint32_t bar_cfree = bar_conv + 8u * kConvDepth;
  const uint32_t bar_accf = bar_cfree + 8u * kConvDepth;
  const uint32_t bar_acce = bar_accf + 8u;
  const uint32_t bar_final = bar_acce + 8u;
  // misc words: [0] TMEM base, [1] abort flag, [2] / [3] "go" verdict of the poller for the
  // converter group / all workers, [8..23] block-reduction scratch
  uint32_t *misc = reinterpret_cast<uint32_t *>(bars + 2 * nslots + 2 * kConvDepth + 3);
  uint32_t *tmem_slot = misc;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 1);
  volatile int *go_unit = reinterpret_cast<volatile int *>(misc + 2);
  volatile int *go_simt = reinterpret_cast<volatile int *>(misc + 3);
  float *red = reinterpret_cast<float *>(misc + 8);
  const Ctx ctx{abort_flag, g.abort_word, g.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const Step *steps = g.steps + g.step_begin[cta];

  if (threadIdx.x == 0) {
    for (int s = 0; s < nslots; ++s) {
      mbar_init(bar_full + 8u * s, 1);
      mbar_init(bar_empty + 8u * s, 1);
    }
    for (int s = 0; s < kConvDepth; ++s) {
      mbar_init(bar_conv + 8u * s, 4);  // one arrival per converter warp
      mbar_init(bar_cfree + 8u * s, 1);
    }
    mbar_init(bar_accf, 1);
    mbar_init(bar_acce, 4);
    mbar_init(bar_final, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ weight producer
    if (lane == 0) {
      const uint64_t policy = l2_policy_evict_first();  // streamed once per pass: do not displace the activations
      const uint8_t *src = g.weights + g.weight_begin[cta];
      uint32_t chunk = 0;
      bool ok = true;
      for (const Step *sp = steps; ok; ++sp) {
        const Step st = load_step(sp);
        if (st.kind == kEnd) break;
        if (st.kind != kUnit) continue;
        const uint32_t bytes = (uint32_t)g.gemm[st.stage].tile_n * 128u;
        for (int kb = 0; kb < st.p3; ++kb, ++chunk) {
          const uint32_t slot = chunk % (uint32_t)nslots, ph = (chunk / (uint32_t)nslots) & 1u;
          ok = wait_bar(bar_empty + 8u * slot, ph ^ 1u, ctx);  // passes at once the first time round
          if (!ok) break;
          mbar_expect_tx(bar_full + 8u * slot, bytes);
          bulk_g2s(ring_addr + slot * slot_bytes, src, bytes, bar_full + 8u * slot, policy);
          src += bytes;
        }
      }
      if (!ok) {  // bounded wait for the copies still in flight before the CTA may exit
        const uint32_t first = chunk > (uint32_t)nslots ? chunk - (uint32_t)nslots : 0u;
        for (uint32_t c = first; c < chunk; ++c) {
          volatile int never = 0;
          mbar_wait(bar_full + 8u * (c % (uint32_t)nslots), (c / (uint32_t)nslots) & 1u, &never);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t chunk = 0, cchunk = 0, unit = 0;
      bool ok = true;
      for (const Step *sp = steps;; ++sp) {
        const Step st = load_step(sp);
        if (st.kind == kEnd) break;
        if (st.kind != kUnit) continue;
        const int BN = g.gemm[st.stage].tile_n;
        const uint32_t idesc = instr_desc(BN, 0);
        // the converters have moved the previous unit's accumulator out of tensor memory
        if (ok) ok = wait_bar(bar_acce, (unit & 1u) ^ 1u, ctx);
        for (int kb = 0; kb < st.p3; ++kb, ++chunk, ++cchunk) {
          const uint32_t slot = chunk % (uint32_t)nslots;
          const uint32_t cs = cchunk % (uint32_t)kConvDepth, cph = (cchunk / (uint32_t)kConvDepth) & 1u;
          if (ok) ok = wait_bar(bar_conv + 8u * cs, cph, ctx);
          if (!ok) continue;
          tc_fence_after();
          const uint64_t d_hi = smem_desc(ring_addr + slot * slot_bytes, 16u, 1024u);
          const uint64_t d_lo = smem_desc(lo_addr + cs * slot_bytes, 16u, 1024u);
#pragma unroll
          for (int j = 0; j < kBK / 8; ++j) {
            const uint32_t a_hi = tmem_base + kACol + cs * 64u + (uint32_t)j * 8u, a_lo = a_hi + 32u;
            umma_tf32_ts(tmem_base + kAccCol, a_lo, d_hi + (uint64_t)(j * 2), idesc, (kb == 0 && j == 0) ? 0u : 1u);
            umma_tf32_ts(tmem_base + kAccCol, a_hi, d_lo + (uint64_t)(j * 2), idesc, 1u);
            umma_tf32_ts(tmem_base + kAccCol, a_hi, d_hi + (uint64_t)(j * 2), idesc, 1u);
          }
          umma_commit(bar_empty + 8u * slot);  // the ring slot may be refilled once these MMAs have read it
          umma_commit(bar_cfree + 8u * cs);    // and the converter stage reused
        }
        if (ok) umma_commit(bar_accf);
        ++unit;
      }
      // nothing may still be executing when tensor memory is freed
      umma_commit(bar_final);
      volatile int never = 0;
      mbar_wait(bar_final, 0u, &never);
    }
  } else {
    // ------------------------------------------------------------ converters (warps 2-5) and helpers (6-9)
    const int wt = threadIdx.x - 64;  // 0..255
    const bool converter = warp < 6;
    const int q = warp & 3, row = q * 32 + lane;  // converter: the TMEM lane quarter this warp may access
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t chunk = 0, cchunk = 0, unit = 0;
    bool ok = true;
    int step_index = 0;
    for (const Step *sp = steps;; ++sp, ++step_index) {
      const Step st = load_step(sp);
      if (st.kind == kEnd) break;
      if (st.kind == kUnit) {
        if (!converter) continue;
        // one thread polls; its verdict reaches the group through shared memory so that all 128
        // threads take the same path whatever the other roles do to the abort flag meanwhile
        if (wt == 0) *go_unit = poll_step(st, g.counters, ctx) ? 1 : 0;
        bar_sync(1, 128);
        ok = *go_unit != 0;
        if (TRACE && wt == 0) g.trace[((size_t)cta * g.max_steps + step_index) * 2] = gtime();
        const GemmStage &G = g.gemm[st.stage];
        const int BN = G.tile_n, kb0 = st.p2, nkb = st.p3;
        const int b_vec = BN * 8;  // 16-byte units in a B tile
        auto load_a = [&](int kb, float4(&x)[8]) {
          if (G.a_tiled) {
            const float4 *p = reinterpret_cast<const float4 *>(G.a) + (size_t)(kb * 8) * kRows + row;
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __ldcg(p + (size_t)j * kRows);
          } else {
            const float4 *p = reinterpret_cast<const float4 *>(G.a + (size_t)row * G.a_ld + (size_t)kb * kBK);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __ldcg(p + j);
          }
        };
        float4 nxt[8];
        if (ok && nkb > 0) load_a(kb0, nxt);
        for (int kb = 0; kb < nkb; ++kb, ++chunk, ++cchunk) {
          const uint32_t slot = chunk % (uint32_t)nslots, ph = (chunk / (uint32_t)nslots) & 1u;
          const uint32_t cs = cchunk % (uint32_t)kConvDepth, cph = (cchunk / (uint32_t)kConvDepth) & 1u;
          float4 cur[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
          if (ok && kb + 1 < nkb) load_a(kb0 + kb + 1, nxt);  // the next block's loads fly under this block's conversion
          if (ok) ok = wait_bar(bar_cfree + 8u * cs, cph ^ 1u, ctx);
          if (ok) ok = wait_bar(bar_full + 8u * slot, ph, ctx);
          ok = __all_sync(0xffffffffu, ok);  // the tensor-memory stores below need the whole warp
          if (!ok) continue;
          tc_fence_after();
          // lo(B) = B - hi(B), element by element in place order: the swizzle is the same on both sides
          const uint4 *hi_b = reinterpret_cast<const uint4 *>(smem + (size_t)slot * slot_bytes);
          uint4 *lo_b = reinterpret_cast<uint4 *>(overlay + (size_t)cs * slot_bytes);
          auto lo1 = [](uint32_t x) { return __float_as_uint(__uint_as_float(x) - __uint_as_float(x & 0xffffe000u)); };
          const int et = wt;  // 0..127
          for (int base = 0; base < b_vec; base += 512) {
            uint4 x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (base + et + 128 * j < b_vec) x[j] = hi_b[base + et + 128 * j];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (base + et + 128 * j < b_vec)
                lo_b[base + et + 128 * j] = make_uint4(lo1(x[j].x), lo1(x[j].y), lo1(x[j].z), lo1(x[j].w));
          }
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t x0 = __float_as_uint(cur[c].x), x1 = __float_as_uint(cur[c].y),
                           x2 = __float_as_uint(cur[c].z), x3 = __float_as_uint(cur[c].w);
            hi[4 * c + 0] = x0 & 0xffffe000u; hi[4 * c + 1] = x1 & 0xffffe000u;
            hi[4 * c + 2] = x2 & 0xffffe000u; hi[4 * c + 3] = x3 & 0xffffe000u;
            lo[4 * c + 0] = lo1(x0); lo[4 * c + 1] = lo1(x1); lo[4 * c + 2] = lo1(x2); lo[4 * c + 3] = lo1(x3);
          }
          const uint32_t t_hi = lane_addr + kACol + cs * 64u;
          tmem_st32(t_hi, hi);
          tmem_st32(t_hi + 32u, lo);
          tmem_wait_st();
          tc_fence_before();
          fence_async_smem();  // the lo(B) writes become visible to the tensor core
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_conv + 8u * cs);
        }
        // accumulator -> partial tile of this k split (tiled order, one float4 per quad and row)
        if (ok) ok = wait_bar(bar_accf, unit & 1u, ctx);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (ok) {
          float4 *P = reinterpret_cast<float4 *>(G.partial) +
                      ((size_t)st.p1 * (G.N >> 2) + (size_t)st.p0 * (BN >> 2)) * kRows + row;
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
            tmem_ld32(lane_addr + kAccCol + (uint32_t)c0, v);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (c0 + 4 * i < BN) P[(size_t)((c0 >> 2) + i) * kRows] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acce);
        ++unit;
        __threadfence();
        bar_sync(1, 128);
        if (wt == 0) {
          if (TRACE) g.trace[((size_t)cta * g.max_steps + step_index) * 2 + 1] = gtime();
          if (st.sig[0] >= 0) red_release_add(g.counters + st.sig[0], 1u);
          if (st.sig[1] >= 0) red_release_add(g.counters + st.sig[1], 1u);
        }
        continue;
      }
      // ---------------------------------------------------------- SIMT steps: all 256 workers
      if (wt == 0) *go_simt = poll_step(st, g.counters, ctx) ? 1 : 0;
      bar_sync(2, kWorkers);
      ok = *go_simt != 0;
      if (TRACE && wt == 0) g.trace[((size_t)cta * g.max_steps + step_index) * 2] = gtime();
      if (ok) {
        if (st.kind == kFinish) finish_step(g.gemm[st.stage], st, wt, red);
        else attention_step(g.attn[st.stage], st.p0, st.p1, reinterpret_cast<float *>(overlay), wt);
      }
      __threadfence();
      bar_sync(2, kWorkers);
      if (wt == 0) {
        if (TRACE) g.trace[((size_t)cta * g.max_steps + step_index) * 2 + 1] = gtime();
        if (st.sig[0] >= 0) red_release_add(g.counters + st.sig[0], 1u);
        if (st.sig[1] >= 0) red_release_add(g.counters + st.sig[1], 1u);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

// ---------------------------------------------------------------- launch (called by resident_host.cu)
size_t kernel_smem_bytes(int nslots, int slot_bytes, int overlay_bytes) {
  return (size_t)nslots * slot_bytes + overlay_bytes + (2 * nslots + 2 * kConvDepth + 3) * 8 + 32 * 4 + 1024;
}

int launch_resident_kernel(const KernelArgs &args, int ctas, size_t smem_bytes, bool trace, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    FML_CUDA(cudaFuncSetAttribute(resident_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    FML_CUDA(cudaFuncSetAttribute(resident_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  // cooperative: the runtime refuses the launch unless all CTAs can be resident together, which
  // the counters between them rely on
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (trace) FML_CUDA(cudaLaunchKernelEx(&cfg, resident_kernel<true>, args));
  else FML_CUDA(cudaLaunchKernelEx(&cfg, resident_kernel<false>, args));
  return FML_OK;
}

}  // namespace res
}  // namespace fml
