// Persistent kernel of a resident stage program (see resident.cuh for the data model and
// resident_host.cu for the planner): a chain of GEMM (+ bias / activation / residual /
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
//     (plain cp.async.bulk into this CTA only, no tensor map) and never waits for activations: weights
//     arrive while the CTA is still waiting for, or reducing, the previous stage;
//   * steps are ordered by the data itself: every word a step stores in the program's buffers
//     carries its buffer generation's parity (resident.cuh), a consumer fetches what it needs
//     into shared memory with all copies in flight and repeats the fetch for words that are not
//     there yet.  Writers never fence or signal, readers never poll a separate flag;
//   * activations stay in a tiled order (resident.cuh) that every role reads and writes as
//     full cache lines.
//
// Roles of a CTA (320 threads):
//   warp 0     weight producer (one lane);
//   warp 1     allocates TMEM, one lane issues tcgen05.mma kind::tf32 and the commits;
//   warps 2-9  workers, as two sets of four warps that alternate over the k blocks of a unit; in a
//              set, thread = activation row = TMEM lane.  For a GEMM unit they fetch the rows'
//              A values of up to four k blocks into shared memory, split each k block into
//              hi = x & 0xffffe000 and lo = x - hi (exact) and write both to tensor memory; they
//              write lo(B) next to the landed B tile (the tensor core ignores the low 13 bits,
//              so the landed tile is hi(B)).  The issuer then adds lo*hi + hi*lo + hi*hi into
//              one accumulator (3xTF32).  After the last k block they move the accumulator to the
//              partial buffer of their k split.  They also run the SIMT steps: the split-K
//              reduction with its epilogue (bias, activation, residual, LayerNorm over the row)
//              and the attention core.
//
// Every wait is bounded.  When one gives up, the CTA records kStatusTimeout, raises the
// program-wide abort word, and from then on every wait of every CTA returns at once: the step
// lists are still walked to the end (so that barrier counts stay uniform), copies in flight are
// awaited, TMEM is freed and the kernel returns.  The program's buffers then hold a mixture of
// generations: fml_resident_reset restores their initial state.
#include "resident.cuh"
#include "resident_host.h"
#include "tc_common.cuh"

namespace fml {
namespace res {
namespace {

constexpr uint32_t kFetchLimit = 1u << 20;  // re-fetch rounds (about a microsecond each) before a wait gives up
constexpr uint32_t kAccCol = 0;             // accumulator tile: TMEM columns [0, 256)
constexpr uint32_t kACol = 256;             // A operand: 64 columns (32 hi, 32 lo) per converter stage

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ld_relaxed(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed4(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------- generation tags
__device__ __forceinline__ float4 tag4(float4 v, uint32_t par) {
  return make_float4(__uint_as_float((__float_as_uint(v.x) & ~1u) | par), __uint_as_float((__float_as_uint(v.y) & ~1u) | par),
                     __uint_as_float((__float_as_uint(v.z) & ~1u) | par), __uint_as_float((__float_as_uint(v.w) & ~1u) | par));
}
__device__ __forceinline__ bool valid4(uint4 w, uint32_t par) {
  return ((((w.x ^ par) | (w.y ^ par)) | ((w.z ^ par) | (w.w ^ par))) & 1u) == 0u;
}
__device__ __forceinline__ float4 untag4(uint4 w) {
  return make_float4(__uint_as_float(w.x & ~1u), __uint_as_float(w.y & ~1u), __uint_as_float(w.z & ~1u), __uint_as_float(w.w & ~1u));
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

// One warp waits for a step's inputs on behalf of the CTA: it watches n sentinel words (the words
// the producers store last, as far as the consumer can tell) with plain loads, a few per lane and
// round, until all carry generation parity `par`.  Watching a handful of words with one warp keeps
// the traffic of waiting CTAs negligible; the fetch that follows still checks every word it
// copies, so a badly chosen sentinel costs time, never correctness.  Returns false when the wait
// was abandoned (the same on every lane).
template <typename AddrFn>
__device__ __forceinline__ bool await_sentinels(int n, AddrFn addr, uint32_t par, int lane, const Ctx &c) {
  for (uint32_t it = 0;; ++it) {
    bool all = true;
    for (int i0 = lane; i0 < n; i0 += 32 * 4) {
      uint4 w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + 32 * j < n) w[j] = ld_relaxed4(addr(i0 + 32 * j));
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + 32 * j < n) all = all && valid4(w[j], par);
    }
    if (__all_sync(0xffffffffu, all)) return true;
    int stop = *c.abort_flag;
    if ((it & 15u) == 15u && lane == 0) {
      if (ld_relaxed(c.abort_word)) { *c.abort_flag = 1; stop = 1; }
      else if (it > kFetchLimit) { give_up(c); stop = 1; }
    }
    if (__any_sync(0xffffffffu, stop != 0)) return false;
  }
}

// Fetches no x ni 16-byte words into this thread's shared-memory slots (dst(o, i) <- src(o, i))
// with all copies in flight at once.  When `tagged`, words whose generation bit is not `par` yet
// are fetched again: the thread first watches one of them with plain loads (a full re-fetch by
// every waiting thread would flood L2), then repeats the fetch for all that were missing.  Each
// thread reads back only what it copied itself, so no barrier is involved.  False when the wait
// was abandoned.
template <typename SrcFn, typename DstFn>
__device__ __forceinline__ bool fetch_words(int no, int ni, SrcFn src, DstFn dst, bool tagged, uint32_t par, const Ctx &c) {
  for (int o = 0; o < no; ++o)
    for (int i = 0; i < ni; ++i) cp_async16(dst(o, i), src(o, i));
  cp_async_commit();
  cp_async_wait_all();
  if (!tagged) return true;
  for (uint32_t round = 0;; ++round) {
    const void *watch = nullptr;
    for (int o = 0; o < no && !watch; ++o)
      for (int i = 0; i < ni; ++i)
        if (!valid4(*reinterpret_cast<const uint4 *>(dst(o, i)), par)) { watch = src(o, i); break; }
    if (!watch) return true;
    for (uint32_t it = 0; !valid4(ld_relaxed4(watch), par); ++it) {
      __nanosleep(64);
      if (*c.abort_flag) return false;
      if ((it & 15u) == 15u) {
        if (ld_relaxed(c.abort_word)) { *c.abort_flag = 1; return false; }
        if (it > kFetchLimit) { give_up(c); return false; }
      }
    }
    for (int o = 0; o < no; ++o)
      for (int i = 0; i < ni; ++i)
        if (!valid4(*reinterpret_cast<const uint4 *>(dst(o, i)), par)) cp_async16(dst(o, i), src(o, i));
    cp_async_commit();
    cp_async_wait_all();
    if (round > 4096u) { give_up(c); return false; }  // every round ends with at least one more word valid
  }
}

__device__ __forceinline__ Step load_step(const Step *p) {
  Step s;
  const uint4 *src = reinterpret_cast<const uint4 *>(p);
  uint4 *dst = reinterpret_cast<uint4 *>(&s);
  dst[0] = __ldg(src);
  dst[1] = __ldg(src + 1);
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

// ---------------------------------------------------------------- finish step (the 256 workers)
// act(sum + bias) + residual
__device__ __forceinline__ float4 finish_epilogue(const GemmStage &G, float4 v, float4 b, float4 t) {
  v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  if (G.act != FML_ACT_NONE) {
    v.x = act_apply(G.act, G.c0, G.c1, G.c2, v.x); v.y = act_apply(G.act, G.c0, G.c1, G.c2, v.y);
    v.z = act_apply(G.act, G.c0, G.c1, G.c2, v.z); v.w = act_apply(G.act, G.c0, G.c1, G.c2, v.w);
  }
  v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
  return v;
}
__device__ __forceinline__ float4 load_bias(const GemmStage &G, int c) {
  return G.bias ? __ldg(reinterpret_cast<const float4 *>(G.bias) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
}
__device__ __forceinline__ void finish_store(const GemmStage &G, int r, int c, float4 v, uint32_t out_par) {
  if (G.out_tiled) reinterpret_cast<float4 *>(G.out_tiled)[(size_t)c * kRows + r] = tag4(v, out_par);
  if (G.out_rm) reinterpret_cast<float4 *>(G.out_rm + (size_t)r * G.out_ld)[c] = v;
}

// Each thread owns a column of 16-byte slots in the staging area: slot k of thread t is at
// stage4[k * 256 + t], so that a warp's accesses to one slot index are one contiguous 512 bytes.
// Per item (one quad of one row) the slots hold the S partial sums and, when the residual is a
// tagged tensor of the program, the residual.
__device__ void finish_step(const GemmStage &G, const Step &st, int wt, float *red, float4 *stage4, int stage_slots,
                            uint32_t epoch, const Ctx &ctx, unsigned long long *tr) {
  const int r0 = st.p0, r1 = st.p1, c0 = st.p2, c1 = st.p3;
  const int S = G.S;
  const size_t split_stride = (size_t)(G.N >> 2) * kRows;
  const float4 *part = reinterpret_cast<const float4 *>(G.partial);
  const uint32_t part_par = tag_parity(G.part_tag, epoch), out_par = tag_parity(G.out_tag, epoch);
  const bool res_tagged = G.res != nullptr && G.res_tag >= 0;
  const uint32_t res_par = res_tagged ? tag_parity(G.res_tag, epoch) : 0u;
  const int per = S + (res_tagged ? 1 : 0);  // slots per item
  float4 *mine = stage4 + wt;
  // Wait for the partial tiles: the first warp watches, per split, the last quad of this step's
  // last row (one word per lane).
  if (wt < 32) {
    auto addr = [&](int i) -> const void * { return part + (size_t)i * split_stride + (size_t)(c1 - 1) * kRows + (r1 - 1); };
    await_sentinels(min(S, 32), addr, part_par, wt, ctx);
  }
  bar_sync(1, kWorkers);
  if (tr && wt == 0) tr[5] = gtime();
  // residual that is not tagged: an input from outside the program, valid since before the launch
  auto plain_residual = [&](int r, int c) {
    if (!G.res || res_tagged) return make_float4(0.f, 0.f, 0.f, 0.f);
    return G.res_tiled ? __ldcg(reinterpret_cast<const float4 *>(G.res) + (size_t)c * kRows + r)
                       : __ldcg(reinterpret_cast<const float4 *>(G.res + (size_t)r * G.res_ld) + c);
  };
  auto residual_src = [&](int r, int c) -> const void * {
    return G.res_tiled ? (const void *)(reinterpret_cast<const float4 *>(G.res) + (size_t)c * kRows + r)
                       : (const void *)(reinterpret_cast<const float4 *>(G.res + (size_t)r * G.res_ld) + c);
  };
  if (!G.ln) {
    // consecutive threads on consecutive rows: 16-byte neighbours in the tiled order
    const int nr = r1 - r0, items = nr * (c1 - c0);
    const int batch = max(1, min(8, stage_slots / per));  // items per thread and round
    for (int i0 = wt; i0 < items; i0 += batch * kWorkers) {
      const int mine_n = min(batch, (items - i0 + kWorkers - 1) / kWorkers);
      int ir[8], ic[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = min(i0 + u * kWorkers, items - 1), ci = i / nr;
        ic[u] = c0 + ci;
        ir[u] = r0 + (i - ci * nr);
      }
      // partial s of item u lives in slot u * per + s, the tagged residual in slot u * per + S
      auto src_p = [&](int u, int sp) -> const void * { return part + (size_t)sp * split_stride + (size_t)ic[u] * kRows + ir[u]; };
      auto dst_p = [&](int u, int sp) -> void * { return mine + (size_t)(u * per + sp) * kWorkers; };
      auto src_r = [&](int u, int) -> const void * { return residual_src(ir[u], ic[u]); };
      auto dst_r = [&](int u, int) -> void * { return mine + (size_t)(u * per + S) * kWorkers; };
      // bias and an untagged residual do not depend on this stage: their loads fly under the fetch
      float4 bv[8], tv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        bv[u] = load_bias(G, ic[u]);
        tv[u] = plain_residual(ir[u], ic[u]);
      }
      bool ok = fetch_words(mine_n, S, src_p, dst_p, true, part_par, ctx);
      if (res_tagged) ok = fetch_words(mine_n, 1, src_r, dst_r, true, res_par, ctx) && ok;
      if (tr && wt == 0) tr[2] = gtime();
      if (!ok) continue;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (u >= mine_n) break;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < S; ++sp) {
          const float4 x = untag4(*reinterpret_cast<const uint4 *>(mine + (size_t)(u * per + sp) * kWorkers));
          v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
        }
        const float4 t = res_tagged ? untag4(*reinterpret_cast<const uint4 *>(mine + (size_t)(u * per + S) * kWorkers)) : tv[u];
        finish_store(G, ir[u], ic[u], finish_epilogue(G, v, bv[u], t), out_par);
      }
    }
    return;
  }
  // LayerNorm over whole rows (c0 = 0, c1 = N / 4 <= 1024): a thread keeps up to four quads of the row
  const int ww = wt >> 5, lane = wt & 31;
  const float inv_n = 1.0f / (float)G.N;
  for (int r = r0; r < r1; ++r) {
    const int nq = c1 > wt ? (c1 - wt + kWorkers - 1) / kWorkers : 0;  // this thread's quads: wt, wt + 128, ..
    auto src_p = [&](int u, int sp) -> const void * { return part + (size_t)sp * split_stride + (size_t)(wt + u * kWorkers) * kRows + r; };
    auto dst_p = [&](int u, int sp) -> void * { return mine + (size_t)(u * per + sp) * kWorkers; };
    auto src_r = [&](int u, int) -> const void * { return residual_src(r, wt + u * kWorkers); };
    auto dst_r = [&](int u, int) -> void * { return mine + (size_t)(u * per + S) * kWorkers; };
    // after an abandoned wait the values are meaningless, but the barriers below still have to be met
    float4 bv[4], tv[4], gv[4], ev[4];  // loads that do not depend on this stage fly under the fetch
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = min(wt + kWorkers * i, c1 - 1);
      bv[i] = load_bias(G, c);
      tv[i] = plain_residual(r, c);
      gv[i] = __ldg(reinterpret_cast<const float4 *>(G.gamma) + c);
      ev[i] = __ldg(reinterpret_cast<const float4 *>(G.beta) + c);
    }
    fetch_words(nq, S, src_p, dst_p, true, part_par, ctx);
    if (res_tagged) fetch_words(nq, 1, src_r, dst_r, true, res_par, ctx);
    if (tr && wt == 0) tr[2] = gtime();
    float4 v[4];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < nq) {
        const int c = wt + kWorkers * i;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < S; ++sp) {
          const float4 x = untag4(*reinterpret_cast<const uint4 *>(mine + (size_t)(i * per + sp) * kWorkers));
          a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
        }
        const float4 t = res_tagged ? untag4(*reinterpret_cast<const uint4 *>(mine + (size_t)(i * per + S) * kWorkers)) : tv[i];
        v[i] = finish_epilogue(G, a, bv[i], t);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    s = warp_sum(s);
    if (lane == 0) red[ww] = s;
    bar_sync(1, kWorkers);
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float mean = tot * inv_n;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < nq) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    q = warp_sum(q);
    if (lane == 0) red[8 + ww] = q;
    bar_sync(1, kWorkers);
    float qt = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) qt += red[8 + w];
    const float inv = 1.0f / sqrtf(qt * inv_n + G.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < nq) {
        const int c = wt + kWorkers * i;
        const float4 g = gv[i], b = ev[i];
        finish_store(G, r, c, make_float4(v[i].x * inv * g.x + b.x, v[i].y * inv * g.y + b.y,
                                          v[i].z * inv * g.z + b.z, v[i].w * inv * g.w + b.w), out_par);
      }
    }
  }
}

// ---------------------------------------------------------------- attention step (the 256 workers)
// softmax(Q K^T / divisor + mask) V for 16 query rows of one head, fp32 FMA, 256 threads.  The
// operands come from tiled matrices (resident.cuh); the arithmetic per element is that of
// attention_kernel (attention.cu): dot products as two half sums over d added in order, maximum,
// exp, sum, divide, then the context as eight partial sums over 16 keys each, added in order.
//   scores   each half of the workers takes half of the head dimension; a thread holds a 4 x 4
//            tile (rows rq + 4x, keys cq + 32u); the second half adds its sums to the first's;
//   softmax  a row's 16 threads are half a warp, 8 keys each, all held in registers;
//   context  warp w takes keys [16w, 16w + 16); a thread holds 4 rows x 8 output columns.
__device__ void attention_step(const AttnStage &A, int head, int row0, float *smem, int wt, uint32_t epoch, const Ctx &ctx,
                               unsigned long long *tr) {
  const int D = A.D, Dv = A.Dv;
  constexpr int Sk = kRows;  // the planner admits 128 key rows only
  const int pk = D + 4, pp = Sk | 1;
  float *Qs = smem;                      // [16][pk]
  float *Ks = Qs + kAttnRows * pk;       // [Sk][pk]
  float *Vs = Ks + (size_t)Sk * pk;      // [Sk][Dv]
  float *Red = Vs + (size_t)Sk * Dv;     // [8][16][Dv]
  float *Ps = Red + 8 * kAttnRows * Dv;  // [16][pp]
  float *Ms = Ps + kAttnRows * pp;       // [16 or 1][Sk]
  const int warp = wt >> 5, lane = wt & 31;
  // Q rows [row0, row0 + 16), all of K and V of the head: quads in (quad, row) order over the
  // threads, rows fastest, so that a warp reads 16-byte neighbours of the tiled matrices
  {
    const int d4 = D >> 2, dv4 = Dv >> 2;
    const int nq = kAttnRows * d4, nk = Sk * d4, nv = Sk * dv4;
    const float4 *q4 = reinterpret_cast<const float4 *>(A.q) + (size_t)((A.q_col + head * A.q_hs) >> 2) * kRows;
    const float4 *k4 = reinterpret_cast<const float4 *>(A.k) + (size_t)((A.k_col + head * A.k_hs) >> 2) * kRows;
    const float4 *v4 = reinterpret_cast<const float4 *>(A.v) + (size_t)((A.v_col + head * A.v_hs) >> 2) * kRows;
    // the first warp watches the last quad of Q's first and last row and of every 16th row of K and V
    // (the rows the producing finish steps end on)
    if (wt < 32 && A.k_tag >= 0 && A.v_tag >= 0 && A.q_tag >= 0) {
      const uint32_t kp = tag_parity(A.k_tag, epoch), vp = tag_parity(A.v_tag, epoch), qp = tag_parity(A.q_tag, epoch);
      auto addr_k = [&](int i) -> const void * { return k4 + (size_t)(d4 - 1) * kRows + min(kRows - 1, 16 * i + 15); };
      auto addr_v = [&](int i) -> const void * { return v4 + (size_t)(dv4 - 1) * kRows + min(kRows - 1, 16 * i + 15); };
      auto addr_q = [&](int i) -> const void * { return q4 + (size_t)(d4 - 1) * kRows + row0 + (i ? kAttnRows - 1 : 0); };
      if (kp == vp && vp == qp) {
        auto addr_all = [&](int i) -> const void * { return i < 8 ? addr_k(i) : i < 16 ? addr_v(i - 8) : addr_q(i - 16); };
        await_sentinels(18, addr_all, kp, wt, ctx);
      } else {
        await_sentinels(kRows / 16, addr_k, kp, wt, ctx);
        await_sentinels(kRows / 16, addr_v, vp, wt, ctx);
        await_sentinels(2, addr_q, qp, wt, ctx);
      }
    }
    bar_sync(1, kWorkers);
    if (tr && wt == 0) tr[5] = gtime();
    auto count = [&](int total) { return total > wt ? (total - wt + kWorkers - 1) / kWorkers : 0; };
    const int cq = count(nq), ck = count(nk), cv = count(nv);
    auto src_q = [&](int k, int) -> const void * { const int i = wt + k * kWorkers, cc = i / kAttnRows, r = i - cc * kAttnRows; return q4 + (size_t)cc * kRows + row0 + r; };
    auto dst_q = [&](int k, int) -> void * { const int i = wt + k * kWorkers, cc = i / kAttnRows, r = i - cc * kAttnRows; return Qs + r * pk + 4 * cc; };
    auto src_k = [&](int k, int) -> const void * { const int i = wt + k * kWorkers, cc = i / kRows, r = i - cc * kRows; return k4 + (size_t)cc * kRows + r; };
    auto dst_k = [&](int k, int) -> void * { const int i = wt + k * kWorkers, cc = i / kRows, r = i - cc * kRows; return Ks + r * pk + 4 * cc; };
    auto src_v = [&](int k, int) -> const void * { const int i = wt + k * kWorkers, cc = i / kRows, r = i - cc * kRows; return v4 + (size_t)cc * kRows + r; };
    auto dst_v = [&](int k, int) -> void * { const int i = wt + k * kWorkers, cc = i / kRows, r = i - cc * kRows; return Vs + r * Dv + 4 * cc; };
    const uint32_t qp = tag_parity(A.q_tag, epoch), kp = tag_parity(A.k_tag, epoch), vp = tag_parity(A.v_tag, epoch);
    if (A.q_tag >= 0 && A.k_tag >= 0 && A.v_tag >= 0 && qp == kp && kp == vp) {
      // the usual case (one producer): every word of the three operands in flight at once
      auto src_all = [&](int k, int) -> const void * { return k < cq ? src_q(k, 0) : k < cq + ck ? src_k(k - cq, 0) : src_v(k - cq - ck, 0); };
      auto dst_all = [&](int k, int) -> void * { return k < cq ? dst_q(k, 0) : k < cq + ck ? dst_k(k - cq, 0) : dst_v(k - cq - ck, 0); };
      fetch_words(cq + ck + cv, 1, src_all, dst_all, true, qp, ctx);
    } else {
      fetch_words(cq, 1, src_q, dst_q, A.q_tag >= 0, qp, ctx);
      fetch_words(ck, 1, src_k, dst_k, A.k_tag >= 0, kp, ctx);
      fetch_words(cv, 1, src_v, dst_v, A.v_tag >= 0, vp, ctx);
    }
    if (tr && wt == 0) tr[6] = gtime();
    // the generation bit is not data: every thread clears it in the words it fetched
    auto clear = [&](int n, auto dstf) {
      for (int k = 0; k < n; ++k) {
        uint4 *p = reinterpret_cast<uint4 *>(dstf(k, 0));
        uint4 w = *p;
        w.x &= ~1u; w.y &= ~1u; w.z &= ~1u; w.w &= ~1u;
        *p = w;
      }
    };
    if (A.q_tag >= 0) clear(cq, dst_q);
    if (A.k_tag >= 0) clear(ck, dst_k);
    if (A.v_tag >= 0) clear(cv, dst_v);
  }
  const int mrows = A.mask ? (A.m_sr == 0 ? 1 : kAttnRows) : 0;
  if (mrows) {
    const float *m = A.mask + head * A.m_sh + (A.m_sr ? row0 * A.m_sr : 0);
    for (int i = wt; i < mrows * Sk; i += kWorkers) {
      const int r = i / Sk, j = i - r * Sk;
      Ms[i] = __ldg(m + r * A.m_sr + j * A.m_sk);
    }
  }
  bar_sync(1, kWorkers);
  if (tr && wt == 0) tr[2] = gtime();
  // ---- scores
  {
    const int half = warp >> 2, rq = warp & 3, cq = lane;
    const int n4 = D >> 2, d_lo = half ? n4 >> 1 : 0, d_hi = half ? n4 : n4 >> 1;
    float acc[4][4];
    const float4 *k4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[x][u] = 0.0f;
      k4[u] = reinterpret_cast<const float4 *>(Ks + (size_t)(cq + 32 * u) * pk);
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
            float *dst = Ps + (rq + 4 * x) * pp + cq + 32 * u;
            *dst = turn ? *dst + acc[x][u] : acc[x][u];
          }
      }
      bar_sync(1, kWorkers);
    }
  }
  if (tr && wt == 0) tr[3] = gtime();
  // ---- softmax over each row: 16 threads per row, 8 keys each, kept in registers
  {
    const int r = wt >> 4, cg = wt & 15;
    float *p = Ps + r * pp;
    const float *mr = Ms + (mrows > 1 ? r * Sk : 0);
    float sc[8];
    float mx = -3.402823466e+38f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sc[i] = p[cg + 16 * i];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (A.divisor != 1.0f) sc[i] = sc[i] / A.divisor;
      if (mrows) sc[i] += mr[cg + 16 * i];
      mx = fmaxf(mx, sc[i]);
    }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sc[i] = expf(sc[i] - mx);
      sum += sc[i];
    }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
#pragma unroll
    for (int i = 0; i < 8; ++i) p[cg + 16 * i] = sc[i] / sum;
  }
  bar_sync(1, kWorkers);
  if (tr && wt == 0) tr[4] = gtime();
  // ---- context
  {
    const uint32_t out_par = tag_parity(A.out_tag, epoch);
    const int rg = lane >> 3, cgp = lane & 7;
    const int per = Sk >> 3, j_lo = warp * per, j_hi = j_lo + per;
    const float *p0 = Ps + rg * pp;
    const int oc = A.o_col + head * A.o_hs;
    for (int dv0 = 0; dv0 < Dv; dv0 += 64) {
      const int ca = dv0 + cgp * 4, cb = ca + 32;
      const bool has_a = ca < Dv, has_b = cb < Dv;
      float4 acc[4][2];
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[x][0] = acc[x][1] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
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
      if (dv0) bar_sync(1, kWorkers);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        float *dst = Red + ((size_t)warp * kAttnRows + rg + 4 * x) * Dv;
        if (has_a) *reinterpret_cast<float4 *>(dst + ca) = acc[x][0];
        if (has_b) *reinterpret_cast<float4 *>(dst + cb) = acc[x][1];
      }
      bar_sync(1, kWorkers);
      const int w4 = min(64, Dv - dv0) >> 2;
      for (int i = wt; i < kAttnRows * w4; i += kWorkers) {  // rows fastest: 16-byte neighbours in the tiled order
        const int cc = i / kAttnRows, r = i - cc * kAttnRows, c = dv0 + (cc << 2);
        float4 t = *reinterpret_cast<const float4 *>(Red + (size_t)r * Dv + c);
#pragma unroll
        for (int w = 1; w < 8; ++w) {
          const float4 u = *reinterpret_cast<const float4 *>(Red + ((size_t)w * kAttnRows + r) * Dv + c);
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        if (A.out_tiled) reinterpret_cast<float4 *>(A.out_tiled)[(size_t)((oc + c) >> 2) * kRows + row0 + r] = tag4(t, out_par);
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
  // [ weight ring: nslots x slot_bytes | overlay: lo(B) slots of the converter stages followed by
  //   the staged A rows during a GEMM unit, the fetch slots of a finish step, or the attention
  //   step's tiles | mbarriers | TMEM slot, abort flag, reduction scratch ]
  const int nslots = g.nslots;
  const uint32_t slot_bytes = (uint32_t)g.slot_bytes;
  uint8_t *overlay = smem + (size_t)nslots * slot_bytes;
  float *a_stage = reinterpret_cast<float *>(overlay + (size_t)kConvDepth * slot_bytes);  // [kAStages][128][kAPitch]
  uint64_t *bars = reinterpret_cast<uint64_t *>(overlay + g.overlay_bytes);
  const uint32_t ring_addr = smem_u32(smem), lo_addr = smem_u32(overlay);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8u * nslots;
  const uint32_t bar_conv = bar_empty + 8u * nslots;
  const uint32_t bar_cfree = bar_conv + 8u * kConvDepth;
  const uint32_t bar_accf = bar_cfree + 8u * kConvDepth;
  const uint32_t bar_acce = bar_accf + 8u;
  const uint32_t bar_final = bar_acce + 8u;
  const uint32_t bar_afull = bar_final + 8u;
  // misc words: [0] TMEM base, [1] abort flag, [8..23] block-reduction scratch
  uint32_t *misc = reinterpret_cast<uint32_t *>(bars + 2 * nslots + 2 * kConvDepth + 4);
  uint32_t *tmem_slot = misc;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 1);
  float *red = reinterpret_cast<float *>(misc + 8);
  const Ctx ctx{abort_flag, g.abort_word, g.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const Step *steps = g.steps + g.step_begin[cta];
  const uint32_t epoch = ld_relaxed(g.epoch);
  trace_stamp();  // kernel-start stamp for fml_set_kernel_trace (one per launch, as every kernel of the library)

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
    mbar_init(bar_acce, 8);  // one arrival per worker warp
    mbar_init(bar_final, 1);
    mbar_init(bar_afull, 1);
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
    // ------------------------------------------------------------ workers (warps 2-9): converters and SIMT steps
    // Two converter sets (warps 2-5 and 6-9), each with one thread per activation row = TMEM lane:
    // set 0 takes the even k blocks of a unit, set 1 the odd ones, so that one set's shared-memory
    // and tensor-memory latencies hide behind the other's (a set alone has one warp per scheduler).
    const int wt = threadIdx.x - 64;  // 0..255
    const int set = wt >> 7, st_t = wt & 127;
    const int q = warp & 3, row = q * 32 + lane;  // the TMEM lane quarter this warp may access
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int stage_slots = g.overlay_bytes / (kWorkers * 16);
    uint32_t chunk = 0, cchunk = 0, unit = 0, agroup = 0;
    int step_index = 0;
    for (const Step *sp = steps;; ++sp, ++step_index) {
      const Step st = load_step(sp);
      if (st.kind == kEnd) break;
      unsigned long long *tr = TRACE ? g.trace + ((size_t)cta * g.max_steps + step_index) * kTraceSlots : nullptr;
      // The overlay is about to be reused (fetch slots, staged A rows, lo(B) slots, attention
      // tiles overlap): every worker must be past the previous step's reads of it.
      bar_sync(1, kWorkers);
      if (TRACE && wt == 0) tr[0] = gtime();
      if (st.kind == kUnit) {
        const GemmStage &G = g.gemm[st.stage];
        const int BN = G.tile_n, kb0 = st.p2, nkb = st.p3;
        const int b_vec = BN * 8;  // 16-byte units in a B tile
        const bool a_tagged = G.a_tag >= 0;
        const uint32_t a_par = a_tagged ? tag_parity(G.a_tag, epoch) : 0u;
        bool ok = true;
        if (a_tagged) {
          // the first warp watches the last quad of this unit's k range in every fourth row
          if (wt < 32) {
            const float4 *col = reinterpret_cast<const float4 *>(G.a) + (size_t)((kb0 + nkb) * 8 - 1) * kRows;
            auto addr = [&](int i) -> const void * { return col + min(kRows - 1, 4 * i + 3); };
            await_sentinels(kRows / 4, addr, a_par, wt, ctx);
          }
          bar_sync(1, kWorkers);
          if (TRACE && wt == 0) tr[5] = gtime();
        }
        for (int g0 = 0; g0 < nkb; g0 += kAStages) {
          const int gn = min(kAStages, nkb - g0);
          if (G.a_tiled) {
            // A k block of a tiled matrix is 16 KiB of consecutive bytes ([8 quads][128 rows] float4):
            // one bulk copy per k block, issued by one thread, lands it in the staging area in that
            // same order (thread = row reads one float4 per quad, conflict-free).  Every thread then
            // checks the generation bit of its own words; a word that was not there yet is re-read
            // from global memory until it is.
            bar_sync(1, kWorkers);  // everyone is done with the previous group's staging
            if (wt == 0) {
              mbar_expect_tx(bar_afull, (uint32_t)gn * 16384u);
              for (int kk = 0; kk < gn; ++kk)
                bulk_g2s_plain(smem_u32(a_stage) + (uint32_t)kk * 16384u,
                               reinterpret_cast<const float4 *>(G.a) + (size_t)(kb0 + g0 + kk) * 8 * kRows, 16384u, bar_afull);
              // the issuing thread waits whatever happens elsewhere: no copy may be in flight at exit
              volatile int never = 0;
              if (!mbar_wait(bar_afull, agroup & 1u, &never)) give_up(ctx);
            }
            if (ok) ok = wait_bar(bar_afull, agroup & 1u, ctx);
            ++agroup;
            if (ok && a_tagged) {
              for (int kk = set; kk < gn; kk += 2)
                for (int j = 0; j < 8; ++j) {
                  uint4 *w = reinterpret_cast<uint4 *>(a_stage) + ((size_t)kk * 8 + j) * kRows + row;
                  if (valid4(*w, a_par)) continue;
                  const float4 *src = reinterpret_cast<const float4 *>(G.a) + ((size_t)(kb0 + g0 + kk) * 8 + j) * kRows + row;
                  uint4 v = ld_relaxed4(src);
                  for (uint32_t it = 0; !valid4(v, a_par); ++it) {
                    __nanosleep(64);
                    if (*abort_flag) { ok = false; break; }
                    if ((it & 15u) == 15u) {
                      if (ld_relaxed(ctx.abort_word)) { *abort_flag = 1; ok = false; break; }
                      if (it > kFetchLimit) { give_up(ctx); ok = false; break; }
                    }
                    v = ld_relaxed4(src);
                  }
                  *w = v;
                }
            }
          } else {
            // a row-major input from outside the program: this thread's row, 16 bytes at a time
            const int mine_n = gn > set ? (gn - set + 1) >> 1 : 0;  // k blocks g0 + set, g0 + set + 2, ..
            auto src = [&](int m, int j) -> const void * {
              return reinterpret_cast<const float4 *>(G.a + (size_t)row * G.a_ld + (size_t)(kb0 + g0 + set + 2 * m) * kBK) + j;
            };
            auto dst = [&](int m, int j) -> void * { return reinterpret_cast<float4 *>(a_stage) + ((size_t)(set + 2 * m) * 8 + j) * kRows + row; };
            if (ok) ok = fetch_words(mine_n, 8, src, dst, false, 0u, ctx);
          }
          if (TRACE && wt == 0 && g0 == 0) tr[2] = gtime();
          for (int kk = 0; kk < gn; ++kk, ++chunk, ++cchunk) {
            if ((kk & 1) != set) continue;
            const uint32_t slot = chunk % (uint32_t)nslots, ph = (chunk / (uint32_t)nslots) & 1u;
            const uint32_t cs = cchunk % (uint32_t)kConvDepth, cph = (cchunk / (uint32_t)kConvDepth) & 1u;
            if (ok) ok = wait_bar(bar_cfree + 8u * cs, cph ^ 1u, ctx);
            if (ok) ok = wait_bar(bar_full + 8u * slot, ph, ctx);
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory stores below need the whole warp
            if (!ok) continue;
            tc_fence_after();
            // lo(B) = B - hi(B), element by element in place order: the swizzle is the same on both sides
            const uint4 *hi_b = reinterpret_cast<const uint4 *>(smem + (size_t)slot * slot_bytes);
            uint4 *lo_b = reinterpret_cast<uint4 *>(overlay + (size_t)cs * slot_bytes);
            auto lo1 = [](uint32_t x) { return __float_as_uint(__uint_as_float(x) - __uint_as_float(x & 0xffffe000u)); };
            for (int base = 0; base < b_vec; base += 512) {
              uint4 x[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (base + st_t + 128 * j < b_vec) x[j] = hi_b[base + st_t + 128 * j];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (base + st_t + 128 * j < b_vec)
                  lo_b[base + st_t + 128 * j] = make_uint4(lo1(x[j].x), lo1(x[j].y), lo1(x[j].z), lo1(x[j].w));
            }
            const uint4 *arow = reinterpret_cast<const uint4 *>(a_stage) + (size_t)kk * 8 * kRows + row;
            uint32_t hi[32], lo[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              uint4 w = arow[(size_t)c * kRows];
              if (a_tagged) { w.x &= ~1u; w.y &= ~1u; w.z &= ~1u; w.w &= ~1u; }  // the generation bit is not data
              hi[4 * c + 0] = w.x & 0xffffe000u; hi[4 * c + 1] = w.y & 0xffffe000u;
              hi[4 * c + 2] = w.z & 0xffffe000u; hi[4 * c + 3] = w.w & 0xffffe000u;
              lo[4 * c + 0] = lo1(w.x); lo[4 * c + 1] = lo1(w.y); lo[4 * c + 2] = lo1(w.z); lo[4 * c + 3] = lo1(w.w);
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
        }
        if (TRACE && wt == 0) tr[3] = gtime();
        // accumulator -> partial tile of this k split (tiled order, one float4 per quad and row);
        // the two sets take alternate groups of 32 columns
        if (ok) ok = wait_bar(bar_accf, unit & 1u, ctx);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (TRACE && wt == 0) tr[4] = gtime();
        if (ok) {
          const uint32_t part_par = tag_parity(G.part_tag, epoch);
          float4 *P = reinterpret_cast<float4 *>(G.partial) +
                      ((size_t)st.p1 * (G.N >> 2) + (size_t)st.p0 * (BN >> 2)) * kRows + row;
          for (int c0 = 32 * set; c0 < BN; c0 += 64) {
            float v[32];
            tmem_ld32(lane_addr + kAccCol + (uint32_t)c0, v);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (c0 + 4 * i < BN)
                P[(size_t)((c0 >> 2) + i) * kRows] = tag4(make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]), part_par);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acce);
        ++unit;
        if (TRACE && wt == 0) tr[1] = gtime();
        continue;
      }
      // ---------------------------------------------------------- SIMT steps
      if (st.kind == kFinish) finish_step(g.gemm[st.stage], st, wt, red, reinterpret_cast<float4 *>(overlay), stage_slots, epoch, ctx, tr);
      else attention_step(g.attn[st.stage], st.p0, st.p1, reinterpret_cast<float *>(overlay), wt, epoch, ctx, tr);
      if (TRACE && wt == 0) tr[1] = gtime();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

__global__ void bump_epoch_kernel(unsigned *epoch) { *epoch += 1u; }

}  // namespace

// ---------------------------------------------------------------- launch (called by resident_host.cu)
size_t kernel_smem_bytes(int nslots, int slot_bytes, int overlay_bytes) {
  return (size_t)nslots * slot_bytes + overlay_bytes + (2 * nslots + 2 * kConvDepth + 4) * 8 + 32 * 4 + 1024;
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
  // the waits between them rely on
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (trace) FML_CUDA(cudaLaunchKernelEx(&cfg, resident_kernel<true>, args));
  else FML_CUDA(cudaLaunchKernelEx(&cfg, resident_kernel<false>, args));
  // the next pass is one generation round further
  bump_epoch_kernel<<<1, 1, 0, stream>>>(args.epoch);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

}  // namespace res
}  // namespace fml
