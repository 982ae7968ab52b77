// Implicit-GEMM convolution on tcgen05 for sm_100a: M = output positions (a TH x TW patch of
// one image = 128 rows), N = output channels, K = (tap, input channel).  Replaces the loop
// nest the reference generates for ConvWithoutPaddingKernel / ConvWithPaddingKernel
// (src/structure/kernel/kernel/conv.cpp:27-280) for unit-stride, undilated, group-1 2-D
// convolutions in NCHW; everything else stays on the CUDA-core kernels of conv.cu.
//
// What makes it "implicit": the input is read once per input-channel block as a raw patch
// of (TH + KH - 1) x (TW + KW - 1, widened to 16-byte steps) pixels x ICB channels by ONE TMA
// box load -- out-of-range rows and columns come back as zeros, which is the padding -- and
// the KH*KW shifted A tiles are cut out of that patch on chip: each converter thread owns one
// output position (= one TMEM lane), gathers its ICB channel values for the tap from shared
// memory and writes them (split into TF32 hi / lo parts) into tensor memory, from where the
// MMAs read A.  A shifted window can not be loaded by TMA directly: the innermost coordinate
// of a tile load must be a multiple of 16 bytes and the taps shift by single pixels.
//
// When the image rows are not a multiple of 16 bytes long (14 x 14 feature maps) no box with
// the row as its second dimension can be described to TMA; if the tile spans the full width the
// patch is then loaded as one run of the flattened H*W plane ("flat mode": whole rows, start
// rounded down to a 16-byte step, rows above and below the image still zero-filled by TMA) and
// the missing left / right padding columns are masked in the gather.
//
// 1x1 convolutions over planes of at most 128 pixels whose size is not a multiple of 4 either
// (7 x 7) need no halo at all: 32 whole planes of one image are one contiguous run, fetched with
// a plain bulk copy ("linear mode"; the channel count must be a multiple of 32).
//
// Weights are expected tap-major with the output channel innermost ([KH][KW][IC][OC], i.e.
// the OIHW tensor stored with layout permutation (3, 2, 0, 1)): the B tile of a (tap, channel
// block) is then an MN-major box, loaded exactly like the GEMM's MN-major B.
//
// Roles and bounded waits follow the GEMM kernel (gemm_tc.cu), with one difference: cutting a tap
// out of the patch and splitting it is the longest stage of a k block here (the tensor pipe was
// 27 % busy with one set of converter warps), so two sets of four converter warps take the k
// blocks alternately, and share the epilogue's columns.
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include <algorithm>
#include <cstdlib>

namespace fml {
namespace {

constexpr int kThreads = 320;  // producer warp, MMA warp, two sets of four converter / epilogue warps
constexpr size_t kSmemBudget = 200 * 1024;

#ifdef FML_CONV_PHASE_TRACE
// Debug builds only (-DFML_CONV_PHASE_TRACE): per-CTA %globaltimer stamps of the kernel's phases.
#define CTRACE(slot)                                                                            \
  do {                                                                                          \
    if (a.trace) {                                                                              \
      unsigned long long t_;                                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                    \
      a.trace[(((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (slot)] = t_;                 \
    }                                                                                           \
  } while (0)
#else
#define CTRACE(slot) do { } while (0)
#endif

struct ConvTcArgs {
  int N, IC, OC, OH, OW, KH, KW, ph, pw;
  int TW, TH, PWD, PHT, xoff;  // tile geometry: patch PHT rows x PWD columns per channel
  int flat, IW, plane, raw_elems;  // flat: 1 = the patch is a run of whole image rows, 2 = whole planes
  const float *x;                  // input base (linear mode copies without a tensor map)
  int n_icb, taps, tile_n, stages, raw_stages;
  int split_k, icb_per_split;  // the channel blocks are split over blockIdx.z = the CTAs of a cluster (1, 1, split_k)
  int tiles_w, tiles_h;
  int64_t ys[4];
  float *y;
  const float *bias;
  int64_t bias_stride;
  int act;
  int *status;
  // optional scale of x per (image, input channel): the product is rounded to fp32 (as a separate
  // Mul kernel would) before the operand is split
  const float *scale;
  int64_t scale_sn, scale_sc;
#ifdef FML_CONV_PHASE_TRACE
  unsigned long long *trace;  // 16 stamps per CTA (fml_debug_set_conv_trace)
#endif
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t *r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ float conv_act(int act, float v) {
  switch (act) {
  case FML_ACT_RELU: return fmaxf(v, 0.0f);
  case FML_ACT_TANH: return tanhf(v);
  // exp2-based exponential and approximate reciprocal (about 2 ulp each): the exact forms are
  // ~40 dependent instructions per element, which a TMEM-lane-per-thread epilogue with two warps
  // per scheduler cannot hide (measured: 8.6 us of a 128x96 tile's epilogue against 1.x us)
  case FML_ACT_SIGMOID: return __fdividef(1.0f, 1.0f + __expf(-v));
  case FML_ACT_SILU: return __fdividef(v, 1.0f + __expf(-v));
  default: return v;
  }
}

// One 32-column group of the epilogue for one activation.  The activation is a template
// parameter and the dispatch sits outside the unrolled loop: with a switch inside it every one
// of the 32 unrolled stores carried the code of all five activations, and fetching those
// instructions (each CTA runs them once, cold) cost more than the stores themselves.
template <int ACT>
__device__ __forceinline__ void store_group(const float *v, const float *bias_s, float *yp, int64_t ys1, int oc_base,
                                            int OC) {
  float *p = yp + (int64_t)oc_base * ys1;
  if (oc_base + 32 <= OC) {  // the usual case: no channel tail inside the group
#pragma unroll
    for (int i = 0; i < 32; ++i, p += ys1) *p = conv_act(ACT, v[i] + bias_s[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i, p += ys1)
      if (oc_base + i < OC) *p = conv_act(ACT, v[i] + bias_s[i]);
  }
}

// ICB: input channels per k block (32, or 8 for the first layer's few channels).
// MODE: 0 = box patch, 1 = flat rows, 2 = linear (whole planes), see the header.
template <bool THREE_PASS, int ICB, int MODE>
__global__ void __launch_bounds__(kThreads, 2)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const ConvTcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int BN = a.tile_n, NS = a.stages, RS = a.raw_stages;
  const uint32_t b_bytes = (uint32_t)ICB * BN * 4;
  const uint32_t stage_bytes = b_bytes * (THREE_PASS ? 2 : 1);
  const uint32_t raw_bytes = (uint32_t)(a.raw_elems * ICB) * 4;
  const uint32_t raw_pitch = (raw_bytes + 127u) & ~127u;
  // [ B stages | raw patches | barriers | flags ]
  const uint32_t b_base = smem_u32(smem);
  uint8_t *raw_ptr = smem + (size_t)NS * stage_bytes;
  const uint32_t raw_base = smem_u32(raw_ptr);
  // split-K stages each CTA's partial tile over the (by then idle) rings: [128][BN + 4] floats
  const int pitch = BN + 4;
  const size_t ring_bytes = (size_t)NS * stage_bytes + (size_t)RS * raw_pitch;
  const size_t staging_bytes = a.split_k > 1 ? (((size_t)kBM * pitch * 4 + 127) & ~(size_t)127) : 0;
  float *staging = reinterpret_cast<float *>(smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (ring_bytes > staging_bytes ? ring_bytes : staging_bytes));
  const uint32_t bar_bfull = smem_u32(bars);
  const uint32_t bar_ready = bar_bfull + 8u * NS;
  const uint32_t bar_empty = bar_ready + 8u * NS;
  const uint32_t bar_rfull = bar_empty + 8u * NS;
  const uint32_t bar_rempty = bar_rfull + 8u * RS;
  const uint32_t bar_accum = bar_rempty + 8u * RS;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * NS + 2 * RS + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *bias_s = reinterpret_cast<float *>(tmem_slot + 4);  // this tile's slice of the bias, [BN]
  float *scale_s = bias_s + 256;                             // this image's input scale, [n_icb * ICB] (when a.scale)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int t = blockIdx.x;
  const int tw = t % a.tiles_w; t /= a.tiles_w;
  const int th = t % a.tiles_h; t /= a.tiles_h;
  const int n = t;
  const int oc0 = blockIdx.y * BN;
  const int oh0 = th * a.TH, ow0 = tw * a.TW;
  // split-K: this CTA reduces the channel blocks [icb_lo, icb_hi); ring positions count from icb_lo
  const int S = a.split_k, split = (int)blockIdx.z;
  const int icb_lo = min(a.n_icb, split * a.icb_per_split), icb_hi = min(a.n_icb, icb_lo + a.icb_per_split);
  const int total_kb = (icb_hi - icb_lo) * a.taps;
  const uint32_t a_col0 = ((uint32_t)BN + 31u) & ~31u;
  const uint32_t a_cols = THREE_PASS ? 2u * ICB : (uint32_t)ICB;  // per stage: hi [, lo]
  uint32_t tmem_cols = 32;
  while (tmem_cols < a_col0 + a_cols * (uint32_t)NS) tmem_cols <<= 1;

  pdl_launch_dependents();
  if (threadIdx.x == 0) CTRACE(0);
  if (threadIdx.x == 32) {  // descriptors ready for the first loads after the dependency wait
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
  }
  // this tile's slice of the bias (a weight, cold when the epilogue asks for it) into L2; a
  // prefetch moves nothing into the SM, so it is safe whoever produces the vector
  if (warp == 2 && a.bias && a.bias_stride == 1)
    for (int oc = oc0 + lane * 8; oc < min(oc0 + BN, a.OC); oc += 256)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a.bias + oc));
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_bfull + 8u * s, 1);
      mbar_init(bar_ready + 8u * s, 4);
      mbar_init(bar_empty + 8u * s, 1);
    }
    for (int s = 0; s < RS; ++s) {
      mbar_init(bar_rfull + 8u * s, 1);
      mbar_init(bar_rempty + 8u * s, 8);  // both converter sets must have left the patch
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
  pdl_wait();
  if (threadIdx.x == 0) CTRACE(1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && !g_drop_loads) {  // (the wait test switches the loads off)
      bool ok = true;
      int kb = 0, raw_issued = 0, b_issued = 0;
      for (int icb = icb_lo; icb < icb_hi && ok; ++icb) {
        const int li = icb - icb_lo, rs = li % RS;
        ok = mbar_wait(bar_rempty + 8u * rs, (((uint32_t)(li / RS)) & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar_rfull + 8u * rs, raw_bytes);
        ++raw_issued;
        // x = ow0 - pw - xoff is a multiple of 4 by construction; rows / columns / channels outside
        // the image are filled with zeros: the padding, and the channel tail of the last block
        if (MODE == 0)
          tma_load_4d(raw_base + (uint32_t)rs * raw_pitch, &map_x, bar_rfull + 8u * rs, ow0 - a.pw - a.xoff,
                      oh0 - a.ph, icb * ICB, n);
        else if (MODE == 1)  // whole rows from (oh0 - ph) on, as one run of the flattened H*W plane
          tma_load_3d(raw_base + (uint32_t)rs * raw_pitch, &map_x, bar_rfull + 8u * rs,
                      (oh0 - a.ph) * a.IW - a.pw - a.xoff, icb * ICB, n);
        else  // ICB whole planes of this image: one contiguous run, a plain bulk copy
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(raw_base + (uint32_t)rs * raw_pitch),
                         "l"(a.x + ((size_t)n * a.IC + (size_t)icb * ICB) * a.plane), "r"(raw_bytes),
                         "r"(bar_rfull + 8u * rs) : "memory");
        for (int tap = 0; tap < a.taps && ok; ++tap, ++kb) {
          const int s = kb % NS;
          ok = mbar_wait(bar_empty + 8u * s, (((uint32_t)(kb / NS)) & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          const uint32_t sb = b_base + (uint32_t)s * stage_bytes;
          mbar_expect_tx(bar_bfull + 8u * s, b_bytes);
          for (int g = 0; g < BN / 32; ++g)
            tma_load_3d(sb + (uint32_t)g * (ICB * 128), &map_w, bar_bfull + 8u * s, oc0 + g * 32, icb * ICB, tap);
          ++b_issued;
        }
      }
      if (!ok) {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
        // bounded drain: no copy may still be on its way into this CTA's shared memory when it exits
        volatile int never = 0;
        for (int it = max(0, raw_issued - RS); it < raw_issued; ++it)
          mbar_wait(bar_rfull + 8u * (it % RS), ((uint32_t)(it / RS)) & 1u, &never);
        for (int it = max(0, b_issued - NS); it < b_issued; ++it)
          mbar_wait(bar_bfull + 8u * (it % NS), ((uint32_t)(it / NS)) & 1u, &never);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc(BN, 1);
      const uint64_t desc_b = smem_desc(b_base, (uint32_t)(ICB * 128), 512u, 1u);
      const uint64_t desc_bl = smem_desc(b_base + b_bytes, (uint32_t)(ICB * 128), 512u, 1u);
      bool ok = true;
      for (int kb = 0; kb < total_kb; ++kb) {
        const int s = kb % NS;
        ok = mbar_wait(bar_ready + 8u * s, ((uint32_t)(kb / NS)) & 1u, abort_flag);
        if (!ok) break;
        if (kb == 0) CTRACE(6);
        tc_fence_after();
        const uint32_t soff = ((uint32_t)s * stage_bytes) >> 4;
#pragma unroll
        for (int j = 0; j < ICB / 8; ++j) {
          const uint32_t a_hi = tmem_base + a_col0 + (uint32_t)s * a_cols + (uint32_t)j * 8u;
          const uint64_t db = desc_b + soff + (uint32_t)j * 64u;  // 8 k rows = 1024 bytes further down
          const uint32_t first = (kb == 0 && j == 0) ? 0u : 1u;
          if (THREE_PASS) {
            const uint64_t dbl = desc_bl + soff + (uint32_t)j * 64u;
            umma_tf32_ts(tmem_base, a_hi + ICB, db, idesc, first);
            umma_tf32_ts(tmem_base, a_hi, dbl, idesc, 1u);
            umma_tf32_ts(tmem_base, a_hi, db, idesc, 1u);
          } else {
            umma_tf32_ts(tmem_base, a_hi, db, idesc, first);
          }
        }
        umma_commit(bar_empty + 8u * s);
      }
      CTRACE(11);
      if (ok) umma_commit(bar_accum);
      else {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ A gather + operand split, then epilogue
    const int set = (warp - 2) >> 2;          // converter set 0 takes the even k blocks, set 1 the odd ones
    const int et = (threadIdx.x - 64) & 127;  // thread within the set
    const int q = warp & 3, m = q * 32 + lane;  // output position = TMEM lane
    const int r = m / a.TW, c = m - r * a.TW;
    const int plane = a.plane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    bool ok = true;
    int kb = 0;
    auto lo1 = [](uint32_t x) { return __float_as_uint(__uint_as_float(x) - __uint_as_float(x & 0xffffe000u)); };
    // The bias slice goes to shared memory now.  Read from global memory inside the epilogue's
    // store loop it would serialise that loop: the compiler must assume that a store to y may
    // change the bias and orders every load behind the store before it (measured: 15 us of a
    // 128-channel tile's epilogue, against about 1 us with the slice on chip).
    {
      const int i = threadIdx.x - 64;
      if (i < BN) bias_s[i] = (a.bias && oc0 + i < a.OC) ? a.bias[(int64_t)(oc0 + i) * a.bias_stride] : 0.0f;
      if (a.scale)
        for (int k = i; k < a.n_icb * ICB; k += 256)
          scale_s[k] = k < a.IC ? a.scale[(int64_t)n * a.scale_sn + (int64_t)k * a.scale_sc] : 0.0f;
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight converter / epilogue warps
    }
    for (int icb = icb_lo; icb < icb_hi && ok; ++icb) {
      const int li = icb - icb_lo, rs = li % RS;
      ok = mbar_wait(bar_rfull + 8u * rs, ((uint32_t)(li / RS)) & 1u, abort_flag);
      if (!ok) break;
      if (li == 0 && threadIdx.x == 64) CTRACE(2);
      const uint32_t *rawp = reinterpret_cast<const uint32_t *>(raw_ptr + (size_t)rs * raw_pitch);
      for (int tap = 0; tap < a.taps && ok; ++tap, ++kb) {
        if ((kb & 1) != set) continue;
        const int kh = tap / a.KW, kw = tap - kh * a.KW;
        const int s = kb % NS;
        const uint32_t phs = ((uint32_t)(kb / NS)) & 1u;
        ok = mbar_wait(bar_empty + 8u * s, phs ^ 1u, abort_flag);  // the MMAs that read this A slot are done
        if (!ok) break;
        tc_fence_after();
        const uint32_t *src = rawp + (r + kh) * a.PWD + c + kw + a.xoff;
        // flat mode has no zero columns left and right of the image rows: mask them here
        const bool col_ok = MODE == 0 || (MODE == 1 ? ((unsigned)(c + kw - a.pw) < (unsigned)a.IW) : m < a.plane);
        uint32_t hi[ICB], lo[ICB];
        if (a.scale) {
          const float *sc = scale_s + icb * ICB;
#pragma unroll
          for (int ic = 0; ic < ICB; ++ic) {
            const uint32_t raw = (MODE == 0 || col_ok) ? src[ic * plane] : 0u;
            const uint32_t x = __float_as_uint(__fmul_rn(__uint_as_float(raw), sc[ic]));
            hi[ic] = x & 0xffffe000u;
            if (THREE_PASS) lo[ic] = lo1(x);
          }
        } else {
#pragma unroll
          for (int ic = 0; ic < ICB; ++ic) {
            const uint32_t x = (MODE == 0 || col_ok) ? src[ic * plane] : 0u;
            hi[ic] = x & 0xffffe000u;
            if (THREE_PASS) lo[ic] = lo1(x);
          }
        }
        const uint32_t t_hi = lane_addr + a_col0 + (uint32_t)s * a_cols;
        if (ICB == 32) {
          tmem_st32(t_hi, hi);
          if (THREE_PASS) tmem_st32(t_hi + 32u, lo);
        } else {
          tmem_st8(t_hi, hi);
          if (THREE_PASS) tmem_st8(t_hi + 8u, lo);
        }
        ok = mbar_wait(bar_bfull + 8u * s, phs, abort_flag);
        if (!ok) break;
        if (kb == 0 && threadIdx.x == 64) CTRACE(7);
        if (THREE_PASS) {
          uint4 *hi_b = reinterpret_cast<uint4 *>(smem + (size_t)s * stage_bytes);
          uint4 *lo_b = reinterpret_cast<uint4 *>(smem + (size_t)s * stage_bytes + b_bytes);
          const int b_vec = (int)b_bytes / 16;
          for (int base = 0; base < b_vec; base += 512) {
            uint4 x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (base + et + 128 * j < b_vec) x[j] = hi_b[base + et + 128 * j];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (base + et + 128 * j < b_vec) {
                uint4 l;
                l.x = lo1(x[j].x); l.y = lo1(x[j].y); l.z = lo1(x[j].z); l.w = lo1(x[j].w);
                lo_b[base + et + 128 * j] = l;
              }
          }
        }
        tmem_wait_st();
        tc_fence_before();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready + 8u * s);
        if (kb == 0 && threadIdx.x == 64) CTRACE(12);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_rempty + 8u * rs);  // the patch may be overwritten
    }
    if (threadIdx.x == 64) CTRACE(13);
    if (ok) ok = mbar_wait(bar_accum, 0u, abort_flag);
    if (!ok) {
      atomicOr(a.status, kStatusTimeout);
      *abort_flag = 1;
    }
    tc_fence_after();
    if (threadIdx.x == 64) CTRACE(3);
    // ---- epilogue: this thread's output position, all channels of the tile; for a fixed channel
    // the lanes of a warp write consecutive pixels of a row
    const int oh = oh0 + r, ow = ow0 + c;
    const bool inside = oh < a.OH && ow < a.OW;  // lanes outside the image still take part in the
                                                 // warp-wide TMEM loads
    float *yp = a.y + (int64_t)n * a.ys[0] + (int64_t)oh * a.ys[2] + (int64_t)ow * a.ys[3];
    // the two sets share the tile's columns: set 0 the first half of the 32-column groups
    const int groups = BN / 32, half = (groups + 1) / 2;
    const int c_lo = set == 0 ? 0 : half * 32, c_hi = set == 0 ? half * 32 : BN;
    if (S > 1) {
      // split-K: the partial tile goes to shared memory (zeros when this CTA had no channel block
      // or gave up); the cluster sums it below
      float *dst = staging + (size_t)m * pitch;
      for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        float v[32];
        if (ok && total_kb > 0) {
          tmem_ld32(lane_addr + (uint32_t)c0, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4 *>(dst + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      }
    } else if (ok) {
      for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
        float v[32];
        tmem_ld32(lane_addr + (uint32_t)c0, v);
        if (inside) {
          switch (a.act) {
          case FML_ACT_RELU: store_group<FML_ACT_RELU>(v, bias_s + c0, yp, a.ys[1], oc0 + c0, a.OC); break;
          case FML_ACT_TANH: store_group<FML_ACT_TANH>(v, bias_s + c0, yp, a.ys[1], oc0 + c0, a.OC); break;
          case FML_ACT_SIGMOID: store_group<FML_ACT_SIGMOID>(v, bias_s + c0, yp, a.ys[1], oc0 + c0, a.OC); break;
          case FML_ACT_SILU: store_group<FML_ACT_SILU>(v, bias_s + c0, yp, a.ys[1], oc0 + c0, a.OC); break;
          default: store_group<FML_ACT_NONE>(v, bias_s + c0, yp, a.ys[1], oc0 + c0, a.OC); break;
          }
        }
      }
    }
  }
  if (S > 1) {
    // ---- split-K reduction through distributed shared memory: rank r owns pixels
    // [r * 128 / S, (r + 1) * 128 / S) of the tile, sums them over the ranks in rank order (the
    // result does not depend on timing), adds the bias, applies the activation and stores
    __syncthreads();
    if (threadIdx.x == 64) CTRACE(8);
    cluster_sync_all();  // every rank's partial tile is in its shared memory
    if (threadIdx.x == 64) CTRACE(9);
    if (warp >= 2) {
      const int rows_per = kBM / S, r0 = split * rows_per;  // S is a power of two
      const int t = threadIdx.x - 64;
      // the ranks' staging tiles in this CTA's view of the cluster's shared memory (one mapa each)
      uint32_t rank_base[8];
#pragma unroll
      for (int rank = 0; rank < 8; ++rank) rank_base[rank] = rank < S ? cluster_smem_addr(smem_u32(staging), (uint32_t)rank) : 0u;
      // Lanes run along the channels: a warp reads 512 contiguous bytes of one pixel's row from each
      // rank (16-byte loads; scalar loads along the pixels moved 6.5 GB/s per SM through the
      // cluster network, a quarter of what 16-byte ones do), two quads per thread in flight.  The
      // stores that follow are strided by the channel plane; the tile is small.
      const int quads = BN >> 2;
      for (int base = t; base < rows_per * quads; base += 512) {
        float4 part[2][8];
        int pmv[2], oq[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int idx = base + 256 * u;
          pmv[u] = -1;
          if (idx < rows_per * quads) {
            pmv[u] = r0 + idx / quads;
            oq[u] = (idx % quads) * 4;
            const uint32_t off = (uint32_t)(pmv[u] * pitch + oq[u]) * 4u;
#pragma unroll
            for (int rank = 0; rank < 8; ++rank)
              if (rank < S)
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(part[u][rank].x), "=f"(part[u][rank].y), "=f"(part[u][rank].z), "=f"(part[u][rank].w)
                             : "r"(rank_base[rank] + off) : "memory");
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (pmv[u] < 0) continue;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int rank = 0; rank < 8; ++rank)
            if (rank < S) { acc.x += part[u][rank].x; acc.y += part[u][rank].y; acc.z += part[u][rank].z; acc.w += part[u][rank].w; }
          const int pr = pmv[u] / a.TW, pc = pmv[u] - pr * a.TW;
          const int oh = oh0 + pr, ow = ow0 + pc;
          if (oh >= a.OH || ow >= a.OW) continue;
          float *yp = a.y + (int64_t)n * a.ys[0] + (int64_t)oh * a.ys[2] + (int64_t)ow * a.ys[3];
          const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ocl = oq[u] + i;
            if (oc0 + ocl < a.OC) yp[(int64_t)(oc0 + ocl) * a.ys[1]] = conv_act(a.act, v[i] + bias_s[ocl]);
          }
        }
      }
    }
    if (threadIdx.x == 64) CTRACE(10);
    cluster_sync_all();  // nobody leaves while a peer may still read its tile
  }
  if (threadIdx.x == 64) CTRACE(4);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0) CTRACE(5);
}

#ifdef FML_CONV_PHASE_TRACE
unsigned long long *g_conv_trace = nullptr;
#endif

int make_map_nd(CUtensorMap *map, const float *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides_bytes,
                const cuuint32_t *box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  FML_REQUIRE(fn, FML_CUDA_ERROR, "fml_conv: cuTensorMapEncodeTiled is not available");
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<float *>(base), dims,
                  strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FML_REQUIRE(r == CUDA_SUCCESS, FML_CUDA_ERROR, "fml_conv: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return FML_OK;
}

}  // namespace

int make_f32_tensor_map(CUtensorMap *map, const float *base, int rank, const cuuint64_t *dims,
                        const cuuint64_t *strides_bytes, const cuuint32_t *box) {
  return make_map_nd(map, base, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Whether the tensor-core path takes this convolution (see the header of this file).
bool conv_tc_eligible(const fml_tensor *x, const fml_tensor *w, const fml_tensor *y, const fml_conv_params *p) {
  if (x->rank != 4 || p->precision == FML_GEMM_FP32) return false;
  if ((p->group > 1) || p->strides[0] != 1 || p->strides[1] != 1 || p->dilations[0] != 1 || p->dilations[1] != 1) return false;
  const int64_t N = x->shape[0], IC = x->shape[1], IH = x->shape[2], IW = x->shape[3];
  const int64_t OC = w->shape[0], KH = w->shape[2], KW = w->shape[3];
  if (N < 1 || IC < 1 || OC < 16 || (OC & 3) || KH * KW > 49 || KH > 7 || KW > 7) return false;
  if (IW & 3) {
    const int64_t OW = y->shape[3], TW = OW <= 8 ? 8 : OW <= 16 ? 16 : 32;
    const bool linear = KH == 1 && KW == 1 && p->pads_begin[0] == 0 && p->pads_begin[1] == 0 && IH * IW <= 128 &&
                        (IC & 31) == 0;
    // flat mode: the tile must span the width, planes must start on 16-byte steps
    const bool flat = OW <= TW && ((IH * IW) & 3) == 0 && (128 / TW + KH - 1) * IW + KW + 6 <= 256;
    if (!linear && !flat) return false;
  }
  if (p->pads_begin[0] < 0 || p->pads_begin[1] < 0 || p->pads_begin[0] > 8 || p->pads_begin[1] > 8) return false;
  // x: dense NCHW; w: [KH][KW][IC][OC] in memory
  if (x->stride[3] != 1 || x->stride[2] != IW || x->stride[1] != IH * IW || (N > 1 && x->stride[0] != IC * IH * IW)) return false;
  if (w->stride[0] != 1 || (IC > 1 && w->stride[1] != OC) || (KW > 1 && w->stride[3] != IC * OC) ||
      (KH > 1 && w->stride[2] != KW * IC * OC)) return false;
  if (!aligned16(x->data) || !aligned16(w->data)) return false;
  if (N * IC * IH * IW >= (1ll << 31) || y->shape[2] * y->shape[3] < 32) return false;
  return true;
}

int launch_conv_tc(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias, const fml_tensor *y,
                   const fml_conv_params *p, cudaStream_t s, const float *x_scale, int64_t x_scale_sn, int64_t x_scale_sc) {
  ConvTcArgs a;
  a.scale = x_scale; a.scale_sn = x_scale_sn; a.scale_sc = x_scale_sc;
  a.N = (int)x->shape[0]; a.IC = (int)x->shape[1]; a.OC = (int)w->shape[0];
  const int IH = (int)x->shape[2], IW = (int)x->shape[3];
  a.OH = (int)y->shape[2]; a.OW = (int)y->shape[3];
  a.KH = (int)w->shape[2]; a.KW = (int)w->shape[3];
  a.ph = (int)p->pads_begin[0]; a.pw = (int)p->pads_begin[1];
  a.flat = (IW & 3) ? 1 : 0;
  if (a.flat && a.KH == 1 && a.KW == 1 && a.ph == 0 && a.pw == 0 && IH * IW <= 128 && (a.IC & 31) == 0 && ((IH * IW) & 3))
    a.flat = 2;
  a.x = (const float *)x->data;
  a.TW = a.flat ? (a.OW <= 8 ? 8 : a.OW <= 16 ? 16 : 32) : (a.OW >= 32 ? 32 : a.OW >= 16 ? 16 : 8);
  if (a.flat == 2) a.TW = a.OW;  // position m = oh * OW + ow
  a.TH = a.flat == 2 ? a.OH : kBM / a.TW;
  a.PHT = a.TH + a.KH - 1;
  a.IW = IW;
  if (a.flat == 2) {
    a.xoff = 0;
    a.PWD = IW;
    a.plane = IH * IW;
  } else if (!a.flat) {
    a.xoff = (4 - a.pw % 4) % 4;
    a.PWD = (a.TW + a.KW - 1 + a.xoff + 3) / 4 * 4;
    a.plane = a.PHT * a.PWD;
  } else {
    // the run starts at flat index (oh0 - ph) * IW - pw; oh0 is a multiple of TH (even), so its
    // remainder modulo 4 is that of -(ph * IW + pw), the same for every tile
    const int start = -(a.ph * IW + a.pw);
    a.xoff = ((start % 4) + 4) % 4;
    a.PWD = IW;  // row pitch of the gather
    a.plane = (a.PHT * IW + a.KW + a.xoff + 3) / 4 * 4;
  }
  a.raw_elems = a.plane;
  const int icb = a.IC > 8 ? 32 : 8;
  a.n_icb = (a.IC + icb - 1) / icb;
  a.taps = a.KH * a.KW;
  const bool three = p->precision != FML_GEMM_TF32;
  a.tile_n = a.OC >= 128 ? 128 : (a.OC + 31) / 32 * 32;
  if (a.tile_n > 128) a.tile_n = 128;
  {
    // A tile of ONE k block is paid per tile, not per column: set-up, the first patch, the operand
    // split and the 12 MMAs cost the same for 16 columns as for 128 (a 144-channel layer cut
    // 128 + 16 ran two CTAs per pixel tile, each with the full fixed cost).  When such a layer has
    // more pixel tiles than SMs it takes the widest tile (a multiple of 32, at most 256) that
    // minimises tiles x (fixed cost + columns), the fixed cost counted as 128 columns; with one
    // operand stage two CTAs still share an SM up to 192 columns.  Measured on EfficientNet-B0:
    // batch 64 2.54 -> 2.47 ms; at batch 1, and for layers of two to eight k blocks, wide tiles
    // lose (FLUIDML_CONV_WIDE_TILES=1 takes those too, =0 none).
    static const int wide = [] { const char *e = getenv("FLUIDML_CONV_WIDE_TILES"); return e ? atoi(e) : 2; }();
    const int64_t px_tiles = (int64_t)((a.OW + a.TW - 1) / a.TW) * ((a.OH + a.TH - 1) / a.TH) * a.N;
    if (wide && a.OC > 128 && a.n_icb * a.taps <= (wide == 2 ? 1 : 8) && (wide == 1 || px_tiles > 148)) {
      int best = 128, best_cost = ((a.OC + 127) / 128) * (128 + 128);
      for (int tn = 160; tn <= 256; tn += 32) {
        const int cost = ((a.OC + tn - 1) / tn) * (128 + tn);
        if (cost < best_cost) { best = tn; best_cost = cost; }
      }
      a.tile_n = best;
    }
  }
  // a patch feeds `taps` k blocks: with a single tap every k block waits for its own patch, so the
  // patch ring must be as deep as the operand ring to cover the load latency
  a.raw_stages = a.taps == 1 ? 6 : a.taps <= 4 ? 3 : 2;
  // ... but never deeper than the work of one tile: a pointwise layer with few input channels is
  // one or two k blocks per tile, and rings sized for long reductions would only keep a second
  // CTA off the SM, whose loads and epilogue are what hides this one's latencies
  a.raw_stages = std::max(1, std::min(a.raw_stages, a.n_icb));
  const size_t raw_pitch = ((size_t)a.raw_elems * icb * 4 + 127) / 128 * 128;
  const size_t stage = (size_t)icb * a.tile_n * 4 * (three ? 2 : 1);
  const int min_stages = a.n_icb * a.taps == 1 ? 1 : 2;  // a tile of one k block needs one operand stage
  while (a.raw_stages > 1 && a.raw_stages * raw_pitch + min_stages * stage > kSmemBudget) --a.raw_stages;  // wide tiles: shorter patch ring
  FML_REQUIRE(a.raw_stages * raw_pitch + min_stages * stage <= kSmemBudget, FML_UNSUPPORTED, "fml_conv: patch does not fit in shared memory");
  int stages = (int)((kSmemBudget - a.raw_stages * raw_pitch) / stage);
  const int a_cols = (three ? 2 : 1) * icb;
  stages = std::min(stages, (512 - (a.tile_n + 31) / 32 * 32) / a_cols);
  stages = std::max(min_stages, std::min(std::min(stages, 8), a.n_icb * a.taps));
  {
    // A layer whose tiles are more than one wave of SMs runs two CTAs per SM with short rings
    // rather than one with deep ones: the second CTA's loads, conversions and epilogue fill the
    // gaps of the first (192 pointwise tiles of 7 x 7 maps took two rounds of 148 at one CTA per
    // SM: 128 -> 79 us; VGG's 64 -> 64 layer at 224 x 224, batch 32: 86 -> 141 TFLOP/s; 128 -> 128
    // at 112 x 112: 160 -> 203).  FLUIDML_CONV_RING=deep keeps the deep rings.
    static const bool deep = [] { const char *e = getenv("FLUIDML_CONV_RING"); return e && e[0] == 'd'; }();
    const int64_t ctas = (int64_t)((a.OW + a.TW - 1) / a.TW) * ((a.OH + a.TH - 1) / a.TH) * a.N * ((a.OC + a.tile_n - 1) / a.tile_n);
    if (!deep && ctas > 148 && a.tile_n <= 128) {
      stages = std::min(stages, 2);
      a.raw_stages = a.taps == 1 ? std::min(a.raw_stages, 3) : 1;
    }
  }
  a.stages = stages;
  a.tiles_w = (a.OW + a.TW - 1) / a.TW;
  a.tiles_h = (a.OH + a.TH - 1) / a.TH;
  {
    // Split-K over the channel blocks when the tiles alone leave most of the machine idle (small
    // maps at small batch: 512 -> 512 on 14 x 14, one image, is 8 tiles of 144 k blocks each):
    // the largest power of two <= 8 that keeps the grid within the SM count and gives every rank
    // at least one channel block.  FLUIDML_CONV_SPLIT_K forces a value (0 = never).
    static const int forced = [] { const char *e = getenv("FLUIDML_CONV_SPLIT_K"); return e ? atoi(e) : -1; }();
    const int64_t tiles = (int64_t)a.tiles_w * a.tiles_h * a.N * ((a.OC + a.tile_n - 1) / a.tile_n);
    int sk = 1;
    while (sk < 8 && tiles * (sk * 2) <= 148 && a.n_icb >= sk * 2 && a.n_icb * a.taps >= sk * 2 * 4) sk *= 2;
    if (forced == 0) sk = 1;
    else if (forced > 0) { sk = 1; while (sk < 8 && sk * 2 <= forced && a.n_icb >= sk * 2) sk *= 2; }
    a.split_k = sk;
    a.icb_per_split = (a.n_icb + sk - 1) / sk;
  }
  for (int i = 0; i < 4; ++i) a.ys[i] = y->stride[i];
  a.y = (float *)y->data;
  a.bias = nullptr; a.bias_stride = 0;
  if (bias) {
    a.bias = (const float *)bias->data;
    for (int i = 0; i < bias->rank; ++i) if (bias->shape[i] != 1) a.bias_stride = bias->stride[i];
  }
  a.act = p->act;
  a.status = device_status_word();
#ifdef FML_CONV_PHASE_TRACE
  a.trace = g_conv_trace;
#endif
  FML_REQUIRE(a.status, FML_CUDA_ERROR, "fml_conv: no device status word");
  const int64_t m_tiles = (int64_t)a.tiles_w * a.tiles_h * a.N;
  FML_REQUIRE(m_tiles <= 0x7fffffff && (a.OC + a.tile_n - 1) / a.tile_n <= 65535, FML_UNSUPPORTED, "fml_conv: grid too large");

  CUtensorMap map_x, map_w;
  if (a.flat == 2) {
    map_x = CUtensorMap{};  // unused
  } else if (a.flat) {
    const cuuint64_t dims[3] = {(cuuint64_t)IH * IW, (cuuint64_t)a.IC, (cuuint64_t)a.N};
    const cuuint64_t str[2] = {(cuuint64_t)IH * IW * 4, (cuuint64_t)a.IC * IH * IW * 4};
    const cuuint32_t box[3] = {(cuuint32_t)a.plane, (cuuint32_t)icb, 1};
    int st = make_map_nd(&map_x, (const float *)x->data, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != FML_OK) return st;
  } else {
    const cuuint64_t dims[4] = {(cuuint64_t)IW, (cuuint64_t)IH, (cuuint64_t)a.IC, (cuuint64_t)a.N};
    const cuuint64_t str[3] = {(cuuint64_t)IW * 4, (cuuint64_t)IH * IW * 4, (cuuint64_t)a.IC * IH * IW * 4};
    const cuuint32_t box[4] = {(cuuint32_t)a.PWD, (cuuint32_t)a.PHT, (cuuint32_t)icb, 1};
    int st = make_map_nd(&map_x, (const float *)x->data, 4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st != FML_OK) return st;
  }
  {
    const cuuint64_t dims[3] = {(cuuint64_t)a.OC, (cuuint64_t)a.IC, (cuuint64_t)a.taps};
    const cuuint64_t str[2] = {(cuuint64_t)a.OC * 4, (cuuint64_t)a.IC * a.OC * 4};
    const cuuint32_t box[3] = {32, (cuuint32_t)icb, 1};
    int st = make_map_nd(&map_w, (const float *)w->data, 3, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (st != FML_OK) return st;
  }
  const size_t ring = (size_t)stages * stage + a.raw_stages * raw_pitch;
  const size_t staging = a.split_k > 1 ? (((size_t)kBM * (a.tile_n + 4) * 4 + 127) & ~(size_t)127) : 0;
  size_t smem = std::max(ring, staging) + (3 * stages + 2 * a.raw_stages + 1) * 8 + 16 + 256 * 4 /* bias slice */ +
                (a.scale ? (size_t)a.n_icb * icb * 4 : 0) /* input scale */ + 1024;
  {  // co-residency capped by TMEM columns, as in the GEMM
    unsigned need = (unsigned)((a.tile_n + 31) / 32 * 32 + a_cols * stages), cols = 32;
    while (cols < need) cols <<= 1;
    const size_t fit = 512 / cols, floor_bytes = (size_t)(228 * 1024) / (fit + 1) + 1024;
    if (smem < floor_bytes) smem = floor_bytes;
  }
  FML_REQUIRE(smem <= 227 * 1024, FML_UNSUPPORTED, "fml_conv: shared memory");
  using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const ConvTcArgs);
  static const KernelFn kernels[12] = {conv_tc_kernel<false, 8, 0>, conv_tc_kernel<false, 32, 0>,
                                       conv_tc_kernel<true, 8, 0>,  conv_tc_kernel<true, 32, 0>,
                                       conv_tc_kernel<false, 8, 1>, conv_tc_kernel<false, 32, 1>,
                                       conv_tc_kernel<true, 8, 1>,  conv_tc_kernel<true, 32, 1>,
                                       conv_tc_kernel<false, 8, 2>, conv_tc_kernel<false, 32, 2>,
                                       conv_tc_kernel<true, 8, 2>,  conv_tc_kernel<true, 32, 2>};
  const KernelFn kernel = kernels[a.flat * 4 + (three ? 2 : 0) + (icb == 32 ? 1 : 0)];
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    for (KernelFn k : kernels) FML_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)m_tiles, (unsigned)((a.OC + a.tile_n - 1) / a.tile_n), (unsigned)a.split_k);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;  // the split-K ranks of a tile share a cluster
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)a.split_k;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  FML_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_x, map_w, a));
  return FML_OK;
}

}  // namespace fml

#ifdef FML_CONV_PHASE_TRACE
// Tracing hook of debug builds: a device buffer of 16 x (number of CTAs) u64 receives, per CTA,
// %globaltimer at 0 start, 1 dependency wait done, 2 first patch landed, 3 accumulator ready,
// 4 epilogue done, 5 end, 6 first k block ready for the MMAs, 7 first weight tile landed; with
// split-K 8 partial tile staged, 9 cluster barrier passed, 10 this rank's rows reduced and stored;
// 11 last MMA issued, 12 first k block converted, 13 converter loop left.
// NULL disables it.
extern "C" void fml_debug_set_conv_trace(void *device_buffer) {
  fml::g_conv_trace = static_cast<unsigned long long *>(device_buffer);
}
#endif
