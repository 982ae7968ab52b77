// tcgen05 GEMM for sm_100a: TMA-fed shared-memory ring, UMMA kind::tf32 with the fp32
// accumulator tile in tensor memory (TMEM), warp-specialised roles, split-K across a
// thread-block cluster with the partial sums reduced through distributed shared memory.
// Replaces the loop nests the reference generates for MatMulKernel
// (src/structure/kernel/kernel/matmul.cpp:28-59) and GemmConstantBiasKernel (gemm.cpp:39-182).
//
// Tile: 128 (M) x tile_n (N) per CTA, k consumed in blocks of 32 floats (one 128-byte
// swizzle span).  Roles, 192 threads:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B boxes into stage s,
//               completion counted on full[s];
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (4 k-steps of 8 per block, x3 in
//               the 3xTF32 mode) and tcgen05.commit to empty[s] / accum;
//   warps 2-5   3xTF32 only: split each landed stage into hi = x & 0xffffe000 and
//               lo = x - hi (exact) and publish it on conv[s]; afterwards the epilogue.
// 3xTF32 issues lo*hi, hi*lo, hi*hi into the same accumulator, so products carry ~2^-21
// relative error instead of TF32's 2^-11 while the weights still cross HBM once as fp32.
//
// Epilogue.  Each epilogue thread owns one TMEM lane = one output row; writing rows straight
// to global memory would scatter every store instruction over 32 cache lines.  Instead the
// accumulator tile is staged in shared memory (the pipeline stages are free by then) and read
// back with consecutive threads on consecutive columns, so bias / residual loads and the
// stores of C are full 128-byte lines.
//
// Split-K.  The S splits of one output tile form a cluster (1, S, 1): they are co-scheduled,
// each keeps its partial tile in its own shared memory, and after a cluster barrier CTA r
// sums rows [r*128/S, (r+1)*128/S) over all S partial tiles in rank order 0..S-1 (so the
// result does not depend on timing), applies the epilogue and stores them.  No global
// scratch, no atomics.
//
// Every mbarrier wait is bounded: when a wait gives up the kernel records kStatusTimeout in
// the device status word, stops issuing work, still takes part in the cluster barriers,
// frees its TMEM and returns.
//
// Each CTA loads its own tiles with plain TMA loads; nothing here is shared between CTAs
// at load time, and nothing reads another device's memory.
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include <cuda.h>
#include <algorithm>
#include <cstdlib>

namespace fml {
namespace {

constexpr int kBK = 32;                 // floats per k block = 128 bytes
constexpr int kABytes = kBM * kBK * 4;  // 16 KiB
constexpr int kThreads = 192;
constexpr size_t kSmemBudget = 200 * 1024;

struct TcArgs {
  GemmProblem p;
  GemmEpilogue e;
  int tile_n, split_k, stages, b_mn_major, three_pass, a_tmem;
  int tiles_m, tiles_n, kb_total, kb_per_split;
  int *status;
#ifdef FML_GEMM_PHASE_TRACE
  unsigned long long *trace;  // 16 stamps per CTA (fml_debug_set_gemm_trace)
#endif
};

#ifdef FML_GEMM_PHASE_TRACE
// Debug builds only (-DFML_GEMM_PHASE_TRACE): per-CTA stamps of the kernel's phases.
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define TRACE(slot)                                                                        \
  do {                                                                                     \
    if (a.trace)                                                                           \
      a.trace[((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (slot)] = ((slot) >= 8 ? (unsigned long long)clock64() : gtime()); \
  } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

// ---------------------------------------------------------------- epilogue helpers
// The activation is a template parameter of the kernel and bias / residual / scaling are
// cheap uniform predicates inside one short loop: every CTA runs each phase of this kernel
// once, so the cost of a phase is largely the instruction fetch of its (cold) code, and a
// compact, straight-line epilogue matters more than a branch-free one.
// erf by Abramowitz & Stegun 7.1.26 with the fast exponential and reciprocal: absolute error about
// 6e-7 in fp32 arithmetic (the formula's 1.5e-7 plus the cancellation in 1 - p t exp(-x^2) near 0;
// tests/test_erf_formula_cpu.py restates it on the host), below 1e-6 with ex2.approx's rounding,
// i.e. a GELU value off by at most 5e-7 |v| -- far below the 3xTF32 product it is applied to.
// The exact erff is ~45 dependent instructions per element; with one epilogue warp per scheduler
// that was 35 us of a 134 us FFN launch at 2048 rows (4096 columns each).
__device__ __forceinline__ float erf_fast(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  return copysignf(fmaf(-p * t, __expf(-ax * ax), 1.0f), x);
}

template <int ACT>
__device__ __forceinline__ float act_op(const GemmEpilogue &e, float v) {
  if (ACT == FML_ACT_GELU_ERF) return v * (erf_fast(v * __frcp_rn(e.c0)) + e.c1) * e.c2;  // (the reciprocal is loop-invariant)
  if (ACT == FML_ACT_RELU) return fmaxf(v, 0.0f);
  if (ACT == FML_ACT_TANH) return tanhf(v);
  if (ACT == FML_ACT_SIGMOID) return 1.0f / (1.0f + expf(-v));
  if (ACT == FML_ACT_SILU) return v / (1.0f + expf(-v));
  return v;
}

// ---------------------------------------------------------------- kernel
// THREE_PASS / B_MN are compile-time so that each variant carries only its own code: the kernel
// runs every phase once per CTA, and instruction fetch of cold code is a first-order cost.
template <bool THREE_PASS, bool B_MN, int ACT, bool A_TMEM>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  // (an offset added to the __shared__ array keeps the pointer in the shared state space, so the
  // converter and epilogue compile to ld/st.shared rather than slower generic accesses)
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int BN = a.tile_n;
  const int pitch = BN + 4;  // staging row pitch in floats: rows 16 bytes apart modulo 128, so the
                             // 16-byte row-wise writes of a quarter-warp hit distinct banks
  const uint32_t b_bytes = (uint32_t)BN * kBK * 4;
  // A_TMEM (3xTF32 only): the converter puts A's hi and lo parts into tensor memory instead of
  // writing a lo copy to shared memory, and the MMAs read A from there: shared-memory traffic
  // per k block drops from (TMA 24 + split 48 + MMA 72) KiB to (24 + 32 + 24) KiB at tile_n 64,
  // and a stage shrinks to A | B | B_lo, so more stages fit.
  const uint32_t stage_bytes = A_TMEM ? kABytes + 2 * b_bytes : (kABytes + b_bytes) * (THREE_PASS ? 2 : 1);
  // [ pipeline stages (reused as the epilogue staging tile) | barriers | flags ]
  const size_t ring_bytes = (size_t)a.stages * stage_bytes;
  const size_t staging_bytes = ((size_t)kBM * pitch * 4 + 1023) / 1024 * 1024;
  const size_t data_bytes = ring_bytes > staging_bytes ? ring_bytes : staging_bytes;
  const uint32_t tiles_base = smem_u32(smem);
  float *staging = reinterpret_cast<float *>(smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + data_bytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_conv = bar_full + 8u * a.stages;
  const uint32_t bar_empty = bar_conv + 8u * a.stages;
  const uint32_t bar_accum = bar_empty + 8u * a.stages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * a.stages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, tile_m = tile / a.tiles_n, tile_n = tile % a.tiles_n;
  const int split = blockIdx.y;  // == rank inside the (1, S, 1) cluster
  const int z = blockIdx.z, z0 = z % (int)a.p.nb0, z1 = z / (int)a.p.nb0;
  // Weights that one row of tiles reads cross L2 once per pass: mark them evict-first so that
  // the bytes streamed by a pass (more than L2 holds) do not displace what every launch
  // re-reads.  With several tile rows the weights are themselves re-read from L2 and keep the
  // default policy.
  const bool b_stream = a.p.b_constant != 0 && a.tiles_m == 1;
  const uint64_t b_policy = b_stream ? l2_policy_evict_first() : 0ull;
  auto load_b = [&](uint32_t dst, uint32_t bar, int c0, int c1, int c2, int c3) {
    if (b_stream) tma_load_4d_hint(dst, &map_b, bar, c0, c1, c2, c3, b_policy);
    else tma_load_4d(dst, &map_b, bar, c0, c1, c2, c3);
  };
  const int kb0 = min(a.kb_total, split * a.kb_per_split);
  const int kb1 = min(a.kb_total, kb0 + a.kb_per_split);
  const int nkb = kb1 - kb0;  // may be 0 for the last ranks of a cluster
  // TMEM columns: the accumulator tile, then (A_TMEM) 64 per stage: 32 of A hi, 32 of A lo
  const uint32_t a_col0 = ((uint32_t)BN + 31u) & ~31u;
  const uint32_t tmem_need = A_TMEM ? a_col0 + 64u * (uint32_t)a.stages : (uint32_t)BN;
  uint32_t tmem_cols = 32;
  while (tmem_cols < tmem_need) tmem_cols <<= 1;

  pdl_launch_dependents();  // the next kernel may start its own set-up while this one runs
  if (threadIdx.x == 0) {  // the first A load comes right after the dependency wait: have its descriptor ready
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_b);
  }
  if (a.p.prefetch_bytes && threadIdx.x == 64) {
    // Constant bytes a later launch will stream (the next weights): each CTA asks L2 to fetch
    // its share now, before this kernel even waits for its own inputs.  Fire and forget.
    const uint64_t pf_policy = l2_policy_evict_first();
    const unsigned long long ctas = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    const unsigned long long cta = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    const unsigned long long share = ((a.p.prefetch_bytes + ctas - 1) / ctas + 127ull) & ~127ull;
    const unsigned long long lo = cta * share, hi = min(a.p.prefetch_bytes & ~15ull, lo + share);
    for (unsigned long long off = lo; off < hi; off += 16384ull) {
      const unsigned n = (unsigned)min(16384ull, hi - off);
      asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;"
                   ::"l"(a.p.prefetch + off), "r"(n), "l"(pf_policy) : "memory");
    }
  }
  if (threadIdx.x == 0) {
    TRACE(0);
    TRACE(8);
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(bar_full + 8u * s, 1);
      mbar_init(bar_conv + 8u * s, 4);  // one arrival per converter warp
      mbar_init(bar_empty + 8u * s, 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers, TMEM and descriptors are ready.  Weights do not depend on the preceding kernel:
  // with a constant B the producer fills the B half of the first stages right away, so that
  // HBM latency overlaps the tail of that kernel; the A halves follow after the wait.
  int pre_b = 0;
  if (a.p.b_constant && warp == 0 && lane == 0 && !g_drop_loads) {
    const int cb2 = a.p.b_b0 ? z0 : 0, cb3 = a.p.b_b1 ? z1 : 0;
    pre_b = min(a.stages, nkb);
    for (int it = 0; it < pre_b; ++it) {
      const uint32_t sb = tiles_base + (uint32_t)it * stage_bytes + kABytes;
      const int k = (kb0 + it) * kBK;
      mbar_expect_tx(bar_full + 8u * it, kABytes + b_bytes);
      if (!B_MN) {
        load_b(sb, bar_full + 8u * it, k, tile_n * BN, cb2, cb3);
      } else {
        for (int g = 0; g < BN / 32; ++g)
          load_b(sb + (uint32_t)g * (kBK * 128), bar_full + 8u * it, tile_n * BN + g * 32, k, cb2, cb3);
      }
    }
  }
  // The per-column bias is a weight as well, cold in HBM when the epilogue asks for it: pull
  // this tile's slice into L2 now (a prefetch moves nothing into the SM, so it is safe
  // whoever produces the vector).
  if (warp == 2 && a.p.bias && a.p.bias_sm == 0 && a.p.bias_sn == 1) {
    const float *bp = a.p.bias + (int64_t)z0 * a.p.bias_b0 + (int64_t)z1 * a.p.bias_b1;
    for (int64_t n = (int64_t)tile_n * BN + lane * 8; n < min((int64_t)(tile_n + 1) * BN, a.p.N); n += 256)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(bp + n));
  }
  // From here on the preceding kernel's results are needed (and its inputs may be overwritten).
  pdl_wait();
  if (threadIdx.x == 0) TRACE(1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && !g_drop_loads) {  // (the wait test switches the loads off: every wait below then runs out)
      const int ca2 = a.p.a_b0 ? z0 : 0, ca3 = a.p.a_b1 ? z1 : 0;
      const int cb2 = a.p.b_b0 ? z0 : 0, cb3 = a.p.b_b1 ? z1 : 0;
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < nkb && ok; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        const uint32_t sa = tiles_base + (uint32_t)s * stage_bytes, sb = sa + kABytes;
        const int k = (kb0 + it) * kBK;
        if (it < pre_b) {  // B of this stage is already on its way, the byte count already posted
          tma_load_4d(sa, &map_a, bar_full + 8u * s, k, tile_m * kBM, ca2, ca3);
          ++issued;
          continue;
        }
        ok = mbar_wait(bar_empty + 8u * s, ph ^ 1u, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar_full + 8u * s, kABytes + b_bytes);
        tma_load_4d(sa, &map_a, bar_full + 8u * s, k, tile_m * kBM, ca2, ca3);
        if (!B_MN) {
          load_b(sb, bar_full + 8u * s, k, tile_n * BN, cb2, cb3);
        } else {
          for (int g = 0; g < BN / 32; ++g)  // one 32-wide column group per box
            load_b(sb + (uint32_t)g * (kBK * 128), bar_full + 8u * s, tile_n * BN + g * 32, k, cb2, cb3);
        }
        ++issued;
      }
      if (!ok) {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
        // bounded drain of the loads already in flight before the CTA may exit
        for (int it = max(0, issued - a.stages); it < issued; ++it) {
          volatile int never = 0;
          mbar_wait(bar_full + 8u * (it % a.stages), (uint32_t)(it / a.stages) & 1u, &never);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(BN, B_MN ? 1 : 0);
      const uint32_t ready = THREE_PASS ? bar_conv : bar_full;
      const uint32_t b_lbo = B_MN ? (uint32_t)(kBK * 128) : 16u;
      const uint32_t b_sbo = B_MN ? 512u : 1024u, b_type = B_MN ? 1u : 2u;
      // stage-0 descriptors: A | B | A_lo | B_lo (the address field cannot carry out: the whole
      // ring lies below 256 KiB of shared-memory address space)
      const uint64_t desc_a = smem_desc(tiles_base, 16u, 1024u);
      const uint64_t desc_b = smem_desc(tiles_base + kABytes, b_lbo, b_sbo, b_type);
      const uint64_t desc_al = smem_desc(tiles_base + kABytes + b_bytes, 16u, 1024u);
      const uint64_t desc_bl = smem_desc(tiles_base + (A_TMEM ? kABytes + b_bytes : 2 * kABytes + b_bytes), b_lbo, b_sbo, b_type);
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        ok = mbar_wait(ready + 8u * s, ph, abort_flag);
        if (!ok) break;
        if (it == 0) TRACE(2);
        tc_fence_after();
        // One thread issues everything, so its instruction count per MMA is on the critical
        // path: the four descriptors of stage 0 were built before the loop; a stage or k-step
        // is an add on the 14-bit (address >> 4) field in the low word.
        const uint32_t soff = ((uint32_t)s * stage_bytes) >> 4;
#pragma unroll
        for (int j = 0; j < kBK / 8; ++j) {
          // k-step j: 32 bytes further along a K-major row; 8 rows (1024 bytes) further
          // down an MN-major tile
          const uint32_t aj = soff + (uint32_t)j * 2u;
          const uint32_t bj = soff + (B_MN ? (uint32_t)j * 64u : (uint32_t)j * 2u);
          const uint64_t da = desc_a + aj, db = desc_b + bj;
          const uint32_t first = (it == 0 && j == 0) ? 0u : 1u;
          if (A_TMEM) {
            const uint32_t a_hi = tmem_base + a_col0 + (uint32_t)s * 64u + (uint32_t)j * 8u, a_lo = a_hi + 32u;
            const uint64_t dbl = desc_bl + bj;
            umma_tf32_ts(tmem_base, a_lo, db, idesc, first);
            umma_tf32_ts(tmem_base, a_hi, dbl, idesc, 1u);
            umma_tf32_ts(tmem_base, a_hi, db, idesc, 1u);
          } else if (THREE_PASS) {
            const uint64_t dal = desc_al + aj, dbl = desc_bl + bj;
            umma_tf32(tmem_base, dal, db, idesc, first);
            umma_tf32(tmem_base, da, dbl, idesc, 1u);
            umma_tf32(tmem_base, da, db, idesc, 1u);
          } else {
            umma_tf32(tmem_base, da, db, idesc, first);
          }
        }
        umma_commit(bar_empty + 8u * s);  // stage reusable once these MMAs have read it
      }
      if (ok) {
        TRACE(3);
        umma_commit(bar_accum);  // with no MMA outstanding (nkb == 0) this arrives at once
      } else {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ converter, then TMEM -> staging
    const int et = threadIdx.x - 64;  // 0..127
    bool ok = true;
    if (THREE_PASS) {
      const int b_vec = (int)b_bytes / 16;  // 16-byte units in the B tile: 8 per row of tile_n
      for (int it = 0; it < nkb && ok; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        ok = mbar_wait(bar_full + 8u * s, ph, abort_flag);
        if (!ok) break;
        uint8_t *st = smem + (size_t)s * stage_bytes;
        uint4 *hi_a = reinterpret_cast<uint4 *>(st);
        uint4 *hi_b = reinterpret_cast<uint4 *>(st + kABytes);
        uint4 *lo_a = reinterpret_cast<uint4 *>(st + kABytes + b_bytes);
        uint4 *lo_b = reinterpret_cast<uint4 *>(st + (A_TMEM ? kABytes + b_bytes : 2 * kABytes + b_bytes));
        // kind::tf32 reads the upper 19 bits of each fp32 operand and ignores the rest
        // (checked on the device: masking the low 13 bits beforehand changes no output bit), so
        // the tile TMA delivered already is the "hi" operand; only lo = x - hi is written.
        auto lo4 = [](uint4 x) {
          uint4 lo;
          lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(x.x & 0xffffe000u));
          lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(x.y & 0xffffe000u));
          lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(x.z & 0xffffe000u));
          lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(x.w & 0xffffe000u));
          return lo;
        };
        if (A_TMEM) {
          // This thread owns row (warp & 3) * 32 + lane of the A tile = the TMEM lane its warp may
          // write.  The row is 128 bytes whose 16-byte chunks TMA swizzled by (row & 7).
          const int q = warp & 3, row = q * 32 + lane, swz = row & 7;
          const uint4 *src = reinterpret_cast<const uint4 *>(st + row * 128);
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 x = src[c ^ swz];
            const uint4 l = lo4(x);
            hi[4 * c + 0] = x.x & 0xffffe000u; hi[4 * c + 1] = x.y & 0xffffe000u;
            hi[4 * c + 2] = x.z & 0xffffe000u; hi[4 * c + 3] = x.w & 0xffffe000u;
            lo[4 * c + 0] = l.x; lo[4 * c + 1] = l.y; lo[4 * c + 2] = l.z; lo[4 * c + 3] = l.w;
          }
          const uint32_t t_hi = tmem_base + ((uint32_t)(q * 32) << 16) + a_col0 + (uint32_t)s * 64u;
          tmem_st32(t_hi, hi);
          tmem_st32(t_hi + 32u, lo);
        } else {  // A: 1024 16-byte units over 128 threads = 8 each; loads first so latencies overlap
          uint4 x[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = hi_a[et + 128 * j];
#pragma unroll
          for (int j = 0; j < 8; ++j) lo_a[et + 128 * j] = lo4(x[j]);
        }
        for (int base = 0; base < b_vec; base += 512) {  // B: up to 4 units per thread per round
          uint4 x[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (base + et + 128 * j < b_vec) x[j] = hi_b[base + et + 128 * j];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (base + et + 128 * j < b_vec) lo_b[base + et + 128 * j] = lo4(x[j]);
        }
        if (A_TMEM) {
          tmem_wait_st();
          tc_fence_before();
        }
        fence_async_smem();  // make the generic-proxy writes visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_conv + 8u * s);  // 4 arrivals instead of 128 serialised ones
      }
    }
    if (ok) ok = mbar_wait(bar_accum, 0u, abort_flag);
    if (!ok) {
      atomicOr(a.status, kStatusTimeout);
      *abort_flag = 1;
    }
    if (et == 0) TRACE(4);
    // Accumulator row -> staging row.  The ring is free: bar_accum fires after every MMA has
    // finished reading it, and every load that was issued has been consumed by an MMA.
    tc_fence_after();
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    float *dst = staging + (size_t)row * pitch;
    for (int c0 = 0; c0 < BN; c0 += 32) {
      float v[32];
      if (ok && nkb > 0) {
        tmem_ld32(lane_addr + (uint32_t)c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        if (c0 + i < BN)  // BN is a multiple of 16
          *reinterpret_cast<float4 *>(dst + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    if (et == 0) TRACE(7);
  }

  // ---------------------------------------------------------------- reduce + epilogue
  tc_fence_before();
  __syncthreads();
  const int S = a.split_k;
  if (S > 1) cluster_sync_all();  // every rank's partial tile is in its shared memory
  if (warp >= 2) {
    const int et = threadIdx.x - 64;
    const int rows_per = (kBM + S - 1) / S;
    const int r0 = split * rows_per, r1 = min(kBM, r0 + rows_per);
    const int64_t zc = (int64_t)z0 * a.p.c_b0 + (int64_t)z1 * a.p.c_b1;
    const float *bias = a.p.bias ? a.p.bias + (int64_t)z0 * a.p.bias_b0 + (int64_t)z1 * a.p.bias_b1 : nullptr;
    const float *res = a.p.res ? a.p.res + (int64_t)z0 * a.p.res_b0 + (int64_t)z1 * a.p.res_b1 : nullptr;
    float *C = a.p.c + zc;
    const int64_t n_base = (int64_t)tile_n * BN, m_base = (int64_t)tile_m * kBM;
    // 16-byte path: unit column stride everywhere, every row start and the tile origin on a
    // 16-byte boundary, no ragged column edge inside this tile
    auto al4 = [](int64_t v) { return (v & 3) == 0; };
    bool vec = a.p.c_sn == 1 && al4(a.p.c_sm) && al4(n_base) && n_base + BN <= a.p.N &&
               ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    if (bias) vec = vec && (a.p.bias_sn == 1 || a.p.bias_sn == 0) && al4(a.p.bias_sm) &&
                    ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
    if (res) vec = vec && a.p.res_sn == 1 && al4(a.p.res_sm) && ((reinterpret_cast<uintptr_t>(res) & 15) == 0);
    const bool scale = a.e.divisor != 1.0f || a.e.alpha != 1.0f || (bias && a.e.beta != 1.0f);
    const float sc_div = a.e.divisor, sc_alpha = a.e.alpha, sc_beta = a.e.beta;
    const uint32_t staging_addr = smem_u32(staging);
    const int quads = BN >> 2;
    // Thread -> (column quad, row within a pass); rows advance by a constant, so every pointer
    // below is stepped with one add per iteration (no division, no 64-bit multiply in the loop:
    // with one warp per scheduler every dependent instruction costs its full latency).
    const int rows_pass = 128 / quads;          // quads 4..64 -> 32..2 rows per pass
    const int cq = et % quads, rsub = et / quads;
    const int r_end = (int)min((int64_t)r1, a.p.M - m_base);  // rows that exist
    if (vec) {
      if (rsub < rows_pass) {
        const int c = cq * 4;
        const int64_t n = n_base + c;
        int r = r0 + rsub;
        const float *sp = staging + (size_t)r * pitch + c;
        const int sp_step = rows_pass * pitch;
        uint32_t rank_addr[8];
        if (S > 1) {
#pragma unroll
          for (int rank = 0; rank < 8; ++rank)
            rank_addr[rank] = rank < S ? cluster_smem_addr(staging_addr + (uint32_t)(r * pitch + c) * 4u, (uint32_t)rank) : 0u;
        }
        float *cp = C + (m_base + r) * a.p.c_sm + n;
        const int64_t c_step = (int64_t)rows_pass * a.p.c_sm;
        const float *rp = res ? res + (m_base + r) * a.p.res_sm + n : nullptr;
        const int64_t r_step = (int64_t)rows_pass * a.p.res_sm;
        const float *bp = bias ? bias + (m_base + r) * a.p.bias_sm + (a.p.bias_sn ? n : 0) : nullptr;
        const int64_t b_step = (int64_t)rows_pass * a.p.bias_sm;
        float4 bvec = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool bias_per_col = bias && a.p.bias_sm == 0 && a.p.bias_sn == 1;  // the usual [N] bias: load once
        if (bias_per_col) bvec = *reinterpret_cast<const float4 *>(bp);
        for (; r < r_end; r += rows_pass) {
          float4 acc;
          if (S == 1) {
            acc = *reinterpret_cast<const float4 *>(sp);
          } else {
            float4 t[8];
#pragma unroll
            for (int rank = 0; rank < 8; ++rank)
              if (rank < S)
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(t[rank].x), "=f"(t[rank].y), "=f"(t[rank].z), "=f"(t[rank].w)
                             : "r"(rank_addr[rank]) : "memory");
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int rank = 0; rank < 8; ++rank)
              if (rank < S) {
                acc.x += t[rank].x; acc.y += t[rank].y; acc.z += t[rank].z; acc.w += t[rank].w;
                rank_addr[rank] += (uint32_t)sp_step * 4u;
              }
          }
          if (bias && !bias_per_col) {
            if (a.p.bias_sn == 1) bvec = *reinterpret_cast<const float4 *>(bp);
            else { const float t = *bp; bvec = make_float4(t, t, t, t); }
          }
          float4 rvec = make_float4(0.f, 0.f, 0.f, 0.f);
          if (res) rvec = *reinterpret_cast<const float4 *>(rp);
          float v[4] = {acc.x, acc.y, acc.z, acc.w};
          const float bv[4] = {bvec.x, bvec.y, bvec.z, bvec.w}, rv[4] = {rvec.x, rvec.y, rvec.z, rvec.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float y = v[j];
            if (scale) {
              if (sc_div != 1.0f) y = y / sc_div;
              y = bias ? sc_alpha * y + sc_beta * bv[j] : sc_alpha * y;
            } else {
              y += bv[j];
            }
            v[j] = act_op<ACT>(a.e, y) + rv[j];
          }
          *reinterpret_cast<float4 *>(cp) = make_float4(v[0], v[1], v[2], v[3]);
          sp += sp_step; cp += c_step; rp += r_step; bp += b_step;
        }
      }
    } else {
      // ragged column edge or non-unit strides: one element at a time, indices recomputed
      const int count = (r1 - r0) * quads;
      for (int i = et; i < count; i += 128) {
        const int rr = i / quads;
        const int r = r0 + rr, c = (i - rr * quads) * 4;
        const int64_t m = m_base + r;
        if (m >= a.p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int64_t n = n_base + c + j;
          if (n >= a.p.N) continue;
          float acc = 0.0f;
          const uint32_t off = staging_addr + (uint32_t)(r * pitch + c + j) * 4u;
          if (S == 1) acc = staging[(size_t)r * pitch + c + j];
          else
            for (int rank = 0; rank < S; ++rank) acc += ld_cluster_f32(cluster_smem_addr(off, (uint32_t)rank));
          const float bv = bias ? bias[m * a.p.bias_sm + n * a.p.bias_sn] : 0.0f;
          const float rv = res ? res[m * a.p.res_sm + n * a.p.res_sn] : 0.0f;
          float y = acc;
          if (scale) {
            if (sc_div != 1.0f) y = y / sc_div;
            y = bias ? sc_alpha * y + sc_beta * bv : sc_alpha * y;
          } else {
            y += bv;
          }
          C[m * a.p.c_sm + n * a.p.c_sn] = act_op<ACT>(a.e, y) + rv;
        }
      }
    }
    if (et == 0) TRACE(5);
  }
  if (S > 1) cluster_sync_all();  // nobody leaves while a peer may still read its tile
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0) { TRACE(6); TRACE(9); }
}

// ---------------------------------------------------------------- host side
// 4-D map: (inner contiguous dim, row dim, batch0, batch1), fp32.
int make_map(CUtensorMap *map, const float *base, int64_t inner, int64_t rows, int64_t row_stride,
             int64_t nb0, int64_t b0_stride, int64_t nb1, int64_t b1_stride, int box_inner,
             int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  FML_REQUIRE(fn, FML_CUDA_ERROR, "fml_gemm: cuTensorMapEncodeTiled is not available");
  // extent-1 dims take any valid stride
  const int64_t dummy = row_stride * rows;
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(b0_stride ? nb0 : 1),
                        (cuuint64_t)(b1_stride ? nb1 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)row_stride * 4, (cuuint64_t)(b0_stride ? b0_stride : dummy) * 4,
                           (cuuint64_t)(b1_stride ? b1_stride : dummy) * 4};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FML_REQUIRE(r == CUDA_SUCCESS, FML_CUDA_ERROR, "fml_gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return FML_OK;
}

bool stride_ok(int64_t s) { return s == 0 || (s > 0 && s % 4 == 0); }

size_t stage_bytes_for(int tile_n, int three_pass, int a_tmem) {
  const size_t b = (size_t)tile_n * kBK * 4;
  return a_tmem ? kABytes + 2 * b : (kABytes + b) * (three_pass ? 2 : 1);
}

// 3xTF32 keeps A's hi / lo parts in tensor memory unless FLUIDML_GEMM_A_TMEM=0.
bool a_tmem_default() {
  static const bool on = [] { const char *e = getenv("FLUIDML_GEMM_A_TMEM"); return !(e && e[0] == '0'); }();
  return on;
}

size_t smem_for(int tile_n, int stages, int three_pass, int a_tmem) {
  const size_t stage = stage_bytes_for(tile_n, three_pass, a_tmem);
  const size_t staging = ((size_t)kBM * (tile_n + 4) * 4 + 1023) / 1024 * 1024;
  const size_t data = std::max(stage * stages, staging);
  return data + (3 * stages + 1) * 8 + 16 + 1024;
}

#ifdef FML_GEMM_PHASE_TRACE
unsigned long long *g_trace = nullptr;
#endif

}  // namespace

bool plan_gemm_tc(const GemmProblem &p, const fml_gemm_params &gp, TcPlan &plan) {
  // A must be K-major; B either K-major or MN-major; bases and row strides 16-byte aligned.
  if (p.K < 1 || p.M < 1 || p.N < 1) return false;
  if (p.a_sk != 1) return false;
  const int mn = (p.b_sn == 1 && p.b_sk != 1) ? 1 : 0;
  if (!mn && p.b_sk != 1) return false;
  const int64_t b_row = mn ? p.b_sk : p.b_sn;
  if (!aligned16(p.a) || !aligned16(p.b)) return false;
  if (p.a_sm <= 0 || p.a_sm % 4 || b_row <= 0 || b_row % 4) return false;
  if (!stride_ok(p.a_b0) || !stride_ok(p.a_b1) || !stride_ok(p.b_b0) || !stride_ok(p.b_b1)) return false;
  if (p.M > (1ll << 30) || p.N > (1ll << 30) || p.K > (1ll << 30)) return false;
  const int64_t batch = p.nb0 * p.nb1;
  if (batch > 65535) return false;
  // Work too small to amortise a 128-row tile goes to the fp32 kernel in AUTO mode.
  if (gp.precision == FML_GEMM_AUTO && (p.M < 32 || p.N < 16 || p.K < 16)) return false;

  plan.b_mn_major = mn;
  plan.three_pass = gp.precision == FML_GEMM_TF32 ? 0 : 1;
  plan.a_tmem = plan.three_pass && a_tmem_default() ? 1 : 0;
  const int kb_total = (int)((p.K + kBK - 1) / kBK);
  const int64_t tiles_m = (p.M + kBM - 1) / kBM;

  // Candidate (tile_n, split) pairs are scored with a small time model: a CTA pulls its A and
  // B boxes through one SM's shared-memory fill path, all CTAs together cannot beat HBM on the
  // bytes that are read once, a cluster of S needs S free SMs in one GPC, and every CTA pays
  // a fixed set-up + epilogue cost.  Explicit tile_n / split_k requests bypass the search.
  const int tn_opts[] = {32, 48, 64, 96, 128, 192, 256};
  const int sk_opts[] = {1, 2, 4, 8};
  const int sk_cap[] = {148, 148, 144, 128};  // CTAs that can be resident for each cluster size
  double best = 1e30;
  int best_tn = 0, best_sk = 0;
  for (int tn : tn_opts) {
    if (gp.tile_n) tn = gp.tile_n;
    if (tn > p.N) tn = (int)((p.N + 15) / 16 * 16);
    if (mn) tn = (tn + 31) / 32 * 32;
    tn = std::max(16, std::min(256, tn / 16 * 16));
    for (int si = 0; si < 4; ++si) {
      int sk = gp.split_k ? gp.split_k : sk_opts[si];
      if (sk > kb_total) continue;
      if (smem_for(tn, 1, plan.three_pass, plan.a_tmem) > kSmemBudget + 8192) continue;
      const int64_t tiles = tiles_m * ((p.N + tn - 1) / tn) * batch;
      const int64_t ctas = tiles * sk;
      const int cap = sk <= 1 ? 148 : sk <= 2 ? sk_cap[1] : sk <= 4 ? sk_cap[2] : sk_cap[3];
      const double waves = (double)((ctas + cap - 1) / cap);
      const int per = (kb_total + sk - 1) / sk;
      const double kb_bytes = kABytes + tn * 128.0;
      const double per_sm_bw = 55e3;  // bytes per microsecond one SM sustains from L2
      const double t_kb = kb_bytes / per_sm_bw * (plan.three_pass ? 1.6 : 1.0);
      const double t_fixed = 3.0 + (double)kBM * tn / sk * 4.0 / 20e3 + (sk > 1 ? 0.6 : 0.0);
      const double t_cta = t_fixed + per * t_kb;
      const double unique = ((double)p.K * p.N + (double)p.M * p.K) * 4.0 * batch;
      const double l2_total = (double)ctas * per * kb_bytes;
      const double t = std::max(std::max(waves * t_cta, unique / 6.5e6), l2_total / 5.0e6);
      if (t < best) { best = t; best_tn = tn; best_sk = sk; }
      if (gp.split_k) break;
    }
    if (gp.tile_n) break;
  }
  if (!best_tn) return false;
  plan.tile_n = best_tn;
  plan.split_k = best_sk;
  if (plan.split_k > 8) return false;  // one cluster holds a tile's splits
  const int per = (kb_total + plan.split_k - 1) / plan.split_k;
  const size_t stage = stage_bytes_for(plan.tile_n, plan.three_pass, plan.a_tmem);
  // Half of the shared memory when that still gives three stages: two CTAs then fit on an SM, so
  // launches of independent streams overlap (+45 % aggregate throughput with four concurrent
  // BERT replicas on one GPU) at no cost to a single stream, whose main loop is paced by the
  // MMA issue rate rather than by the depth of the ring.  FLUIDML_GEMM_RING_KB overrides.
  static const size_t ring_budget = [] { const char *e = getenv("FLUIDML_GEMM_RING_KB"); return e ? (size_t)atoi(e) * 1024 : (size_t)100 * 1024; }();
  int stages = (int)(ring_budget / stage);
  if (stages < 3) stages = (int)(kSmemBudget / stage);
  stages = std::max(1, std::min(std::min(stages, 8), per));
  if (plan.a_tmem)  // 64 TMEM columns per stage beside the accumulator tile, 512 in all
    stages = std::max(1, std::min(stages, (512 - ((plan.tile_n + 31) / 32 * 32)) / 64));
  plan.stages = stages;
  plan.smem_bytes = smem_for(plan.tile_n, stages, plan.three_pass, plan.a_tmem);
  {
    // Never let more CTAs share an SM than its 512 TMEM columns can serve at once: a CTA that
    // had to wait inside tcgen05.alloc for a neighbour could hold up its whole cluster.  The
    // shared-memory request is what limits co-residency, so it is padded where needed.
    unsigned need = plan.a_tmem ? (unsigned)((plan.tile_n + 31) / 32 * 32 + 64 * stages) : (unsigned)plan.tile_n, cols = 32;
    while (cols < need) cols <<= 1;
    const size_t fit = 512 / cols;  // CTAs whose TMEM fits together
    const size_t floor_bytes = (size_t)(228 * 1024) / (fit + 1) + 1024;
    if (plan.smem_bytes < floor_bytes) plan.smem_bytes = floor_bytes;
  }
  if (plan.smem_bytes > 227 * 1024) return false;
  return true;
}

int launch_gemm_tc(const GemmProblem &p, const GemmEpilogue &e, const TcPlan &plan, cudaStream_t s) {
  TcArgs a;
  a.p = p; a.e = e;
  a.tile_n = plan.tile_n; a.split_k = plan.split_k; a.stages = plan.stages;
  a.b_mn_major = plan.b_mn_major; a.three_pass = plan.three_pass; a.a_tmem = plan.a_tmem;
  a.tiles_m = (int)((p.M + kBM - 1) / kBM);
  a.tiles_n = (int)((p.N + plan.tile_n - 1) / plan.tile_n);
  a.kb_total = (int)((p.K + kBK - 1) / kBK);
  a.kb_per_split = (a.kb_total + plan.split_k - 1) / plan.split_k;
  a.status = device_status_word();
#ifdef FML_GEMM_PHASE_TRACE
  a.trace = g_trace;
#endif
  FML_REQUIRE(a.status, FML_CUDA_ERROR, "fml_gemm: no device status word");
  CUtensorMap map_a, map_b;
  int st = make_map(&map_a, p.a, p.K, p.M, p.a_sm, p.nb0, p.a_b0, p.nb1, p.a_b1, kBK, kBM,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != FML_OK) return st;
  if (!plan.b_mn_major)
    st = make_map(&map_b, p.b, p.K, p.N, p.b_sn, p.nb0, p.b_b0, p.nb1, p.b_b1, kBK, plan.tile_n,
                  CU_TENSOR_MAP_SWIZZLE_128B);
  else
    st = make_map(&map_b, p.b, p.N, p.K, p.b_sk, p.nb0, p.b_b0, p.nb1, p.b_b1, 32, kBK,
                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (st != FML_OK) return st;
  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const TcArgs);
#define FML_TC_ROW(T, M, A)                                                               \
  gemm_tc_kernel<T, M, FML_ACT_NONE, A>, gemm_tc_kernel<T, M, FML_ACT_GELU_ERF, A>,       \
  gemm_tc_kernel<T, M, FML_ACT_RELU, A>, gemm_tc_kernel<T, M, FML_ACT_TANH, A>,           \
  gemm_tc_kernel<T, M, FML_ACT_SIGMOID, A>, gemm_tc_kernel<T, M, FML_ACT_SILU, A>
  static const KernelFn kernels[36] = {FML_TC_ROW(false, false, false), FML_TC_ROW(false, true, false),
                                       FML_TC_ROW(true, false, false),  FML_TC_ROW(true, true, false),
                                       FML_TC_ROW(true, false, true),   FML_TC_ROW(true, true, true)};
#undef FML_TC_ROW
  FML_REQUIRE(e.act >= 0 && e.act <= FML_ACT_SILU, FML_BAD_ARG, "fml_gemm: unknown activation %d", e.act);
  const int act = e.act;
  const int row = plan.a_tmem ? 4 + (plan.b_mn_major ? 1 : 0) : (plan.three_pass ? 2 : 0) + (plan.b_mn_major ? 1 : 0);
  const KernelFn kernel = kernels[row * 6 + act];
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    for (KernelFn k : kernels)
      FML_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)(a.tiles_m * a.tiles_n), (unsigned)plan.split_k, (unsigned)(p.nb0 * p.nb1));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = plan.smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)plan.split_k;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  FML_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, a));
  return FML_OK;
}

}  // namespace fml

#ifdef FML_GEMM_PHASE_TRACE
// Tracing hook: when set to a device buffer of 16 x (number of CTAs) u64, every tensor-core GEMM
// launch stamps %globaltimer at: 0 CTA start, 1 set-up done, 2 first stage landed, 3 last MMA
// issued, 4 accumulator ready, 5 epilogue done, 6 CTA end, 7 tile staged; 8 / 9 hold clock64()
// at CTA start / end (SM cycles, to read the SM clock against the timer).  NULL disables it.
extern "C" void fml_debug_set_gemm_trace(void *device_buffer) {
  fml::g_trace = static_cast<unsigned long long *>(device_buffer);
}
#endif
