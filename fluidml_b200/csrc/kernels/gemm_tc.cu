// tcgen05 GEMM for sm_100a: TMA-fed shared-memory ring, UMMA kind::tf32 with the fp32
// accumulator tile in tensor memory (TMEM), warp-specialised roles, split-K with a
// fixed-order reduction.  Replaces the loop nests the reference generates for
// MatMulKernel (src/structure/kernel/kernel/matmul.cpp:28-59) and GemmConstantBiasKernel
// (gemm.cpp:39-182).
//
// Tile: 128 (M) x tile_n (N) per CTA, k consumed in blocks of 32 floats (one 128-byte
// swizzle span).  Roles, 192 threads:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B boxes into stage s,
//               completion counted on full[s];
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (4 k-steps of 8 per block, x3 in
//               the 3xTF32 mode) and tcgen05.commit to empty[s] / accum;
//   warps 2-5   3xTF32 only: split each landed stage into hi = x & 0xffffe000 and
//               lo = x - hi (exact) and publish it on conv[s]; afterwards the epilogue:
//               tcgen05.ld the accumulator (one TMEM lane = one output row per thread),
//               apply divisor / bias / activation / residual and store.
// 3xTF32 issues lo*hi, hi*lo, hi*hi into the same accumulator, so products carry ~2^-21
// relative error instead of TF32's 2^-11 while the weights still cross HBM once as fp32.
//
// Split-K: every split writes its partial tile to the workspace; the split that arrives
// last on the tile's counter sums all partials in split order 0..S-1 (so the result does
// not depend on arrival order), applies the epilogue and resets the counter.
//
// Every mbarrier wait is bounded: when a wait gives up the kernel records
// kStatusTimeout in the device status word, stops issuing work, drains what it can with
// bounded waits, frees its TMEM and returns.
//
// Each CTA loads its own tiles; no load in this file is shared between CTAs or devices.
#include "gemm_common.cuh"
#include <cuda.h>

namespace fml {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 32;                 // floats per k block = 128 bytes
constexpr int kABytes = kBM * kBK * 4;  // 16 KiB
constexpr int kThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 22;

struct TcArgs {
  GemmProblem p;
  GemmEpilogue e;
  int tile_n, split_k, stages, b_mn_major, three_pass;
  int tiles_m, tiles_n, kb_total, kb_per_split;
  float *ws_partial;
  unsigned *ws_counter;
  int *status;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Bounded wait: false when the limit ran out or another role raised `abort`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255u) == 255u && *abort) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float *v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void epi_bar_sync() {  // the 128 epilogue threads only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, tile base 1024-byte aligned.
//   K-major tile (rows of 128 bytes = 32 k values): 8-row groups 1024 bytes apart (SBO);
//     the leading-dimension offset is unused for swizzled K-major operands.
//   MN-major tile (rows of 128 bytes = 32 n values, one row per k).  32-bit MN-major
//     operands exist only in the "128-byte swizzle, 32-byte atom" mode (layout type 1; TMA
//     writes it with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): the pattern repeats every 4 k
//     rows, so 4-k groups are 512 bytes apart (SBO) and 32-n column groups `lbo_bytes`
//     apart (LBO).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type = 2u) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for this architecture
  d |= (uint64_t)layout_type << 61;  // 2 = SWIZZLE_128B, 1 = SWIZZLE_128B with 32-byte atom
  return d;
}

// Instruction descriptor for kind::tf32: fp32 accumulate, TF32 A and B, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc(int n, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// ---------------------------------------------------------------- kernel
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~static_cast<uintptr_t>(1023));
  const int BN = a.tile_n;
  const uint32_t b_bytes = (uint32_t)BN * kBK * 4;
  const uint32_t stage_bytes = (kABytes + b_bytes) * (a.three_pass ? 2 : 1);
  // stage layout: A_hi | B_hi | (A_lo | B_lo)
  const uint32_t tiles_base = smem_u32(smem);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)a.stages * stage_bytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_conv = bar_full + 8u * a.stages;
  const uint32_t bar_empty = bar_conv + 8u * a.stages;
  const uint32_t bar_accum = bar_empty + 8u * a.stages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * a.stages + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *last_flag = reinterpret_cast<volatile int *>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, tile_m = tile / a.tiles_n, tile_n = tile % a.tiles_n;
  const int split = blockIdx.y;
  const int z = blockIdx.z, z0 = z % (int)a.p.nb0, z1 = z / (int)a.p.nb0;
  const int kb0 = split * a.kb_per_split;
  const int kb1 = min(a.kb_total, kb0 + a.kb_per_split);
  const int nkb = kb1 - kb0;  // >= 1 by construction of the plan
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < BN) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(bar_full + 8u * s, 1);
      mbar_init(bar_conv + 8u * s, 128);
      mbar_init(bar_empty + 8u * s, 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int ca2 = a.p.a_b0 ? z0 : 0, ca3 = a.p.a_b1 ? z1 : 0;
      const int cb2 = a.p.b_b0 ? z0 : 0, cb3 = a.p.b_b1 ? z1 : 0;
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < nkb && ok; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        ok = mbar_wait(bar_empty + 8u * s, ph ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t sa = tiles_base + (uint32_t)s * stage_bytes, sb = sa + kABytes;
        const int k = (kb0 + it) * kBK;
        mbar_expect_tx(bar_full + 8u * s, kABytes + b_bytes);
        tma_load_4d(sa, &map_a, bar_full + 8u * s, k, tile_m * kBM, ca2, ca3);
        if (!a.b_mn_major) {
          tma_load_4d(sb, &map_b, bar_full + 8u * s, k, tile_n * BN, cb2, cb3);
        } else {
          for (int g = 0; g < BN / 32; ++g)  // one 32-wide column group per box
            tma_load_4d(sb + (uint32_t)g * (kBK * 128), &map_b, bar_full + 8u * s,
                        tile_n * BN + g * 32, k, cb2, cb3);
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
      const uint32_t idesc = instr_desc(BN, a.b_mn_major);
      const uint32_t ready = a.three_pass ? bar_conv : bar_full;
      const uint32_t b_lbo = a.b_mn_major ? (uint32_t)(kBK * 128) : 16u;
      const uint32_t b_sbo = a.b_mn_major ? 512u : 1024u, b_type = a.b_mn_major ? 1u : 2u;
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        ok = mbar_wait(ready + 8u * s, ph, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = tiles_base + (uint32_t)s * stage_bytes, sb = sa + kABytes;
        const uint32_t sal = sb + b_bytes, sbl = sal + kABytes;
#pragma unroll
        for (int j = 0; j < kBK / 8; ++j) {
          // k-step j: 32 bytes further along a K-major row; 8 rows (1024 bytes) further
          // down an MN-major tile
          const uint32_t a_off = (uint32_t)j * 32u;
          const uint32_t b_off = a.b_mn_major ? (uint32_t)j * 1024u : (uint32_t)j * 32u;
          const uint64_t da = smem_desc(sa + a_off, 16u, 1024u);
          const uint64_t db = smem_desc(sb + b_off, b_lbo, b_sbo, b_type);
          const uint32_t first = (it == 0 && j == 0) ? 0u : 1u;
          if (a.three_pass) {
            const uint64_t dal = smem_desc(sal + a_off, 16u, 1024u);
            const uint64_t dbl = smem_desc(sbl + b_off, b_lbo, b_sbo, b_type);
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
        umma_commit(bar_accum);
      } else {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ converter + epilogue
    const int et = threadIdx.x - 64;  // 0..127
    bool ok = true;
    if (a.three_pass) {
      const int a_vec = kABytes / 16, b_vec = (int)b_bytes / 16;
      for (int it = 0; it < nkb && ok; ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (uint32_t)(it / a.stages) & 1u;
        ok = mbar_wait(bar_full + 8u * s, ph, abort_flag);
        if (!ok) break;
        uint8_t *st = smem + (size_t)s * stage_bytes;
        uint4 *hi_a = reinterpret_cast<uint4 *>(st);
        uint4 *hi_b = reinterpret_cast<uint4 *>(st + kABytes);
        uint4 *lo_a = reinterpret_cast<uint4 *>(st + kABytes + b_bytes);
        uint4 *lo_b = reinterpret_cast<uint4 *>(st + 2 * kABytes + b_bytes);
        auto split4 = [](uint4 x, uint4 &hi, uint4 &lo) {
          hi.x = x.x & 0xffffe000u; hi.y = x.y & 0xffffe000u;
          hi.z = x.z & 0xffffe000u; hi.w = x.w & 0xffffe000u;
          lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(hi.x));
          lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(hi.y));
          lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(hi.z));
          lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(hi.w));
        };
        for (int i = et; i < a_vec; i += 128) {
          uint4 hi, lo;
          split4(hi_a[i], hi, lo);
          hi_a[i] = hi;
          lo_a[i] = lo;
        }
        for (int i = et; i < b_vec; i += 128) {
          uint4 hi, lo;
          split4(hi_b[i], hi, lo);
          hi_b[i] = hi;
          lo_b[i] = lo;
        }
        fence_async_smem();  // make the generic-proxy writes visible to the tensor core
        mbar_arrive(bar_conv + 8u * s);
      }
    }
    if (ok) ok = mbar_wait(bar_accum, 0u, abort_flag);
    if (!ok) {
      atomicOr(a.status, kStatusTimeout);
      *abort_flag = 1;
    }
    // One decision for all 128 epilogue threads, so the named barriers below always see
    // every one of them: -1 = some role gave up, skip the epilogue.
    epi_bar_sync();
    if (et == 0) *last_flag = *abort_flag ? -1 : 0;
    epi_bar_sync();
    if (*last_flag == 0) {
      tc_fence_after();
      const int q = warp & 3;  // TMEM lane quarter this warp may read
      const int row = q * 32 + lane;
      const int64_t m = (int64_t)tile_m * kBM + row;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
      const int64_t zc = (int64_t)z0 * a.p.c_b0 + (int64_t)z1 * a.p.c_b1;
      const float *bias = a.p.bias ? a.p.bias + (int64_t)z0 * a.p.bias_b0 + (int64_t)z1 * a.p.bias_b1 : nullptr;
      const float *res = a.p.res ? a.p.res + (int64_t)z0 * a.p.res_b0 + (int64_t)z1 * a.p.res_b1 : nullptr;
      float *C = a.p.c + zc;
      const int64_t n_base = (int64_t)tile_n * BN;

      auto finish = [&](const float *v, int c0) {
        if (m >= a.p.M) return;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int64_t n = n_base + c0 + i;
          if (c0 + i < BN && n < a.p.N) {
            const float bv = bias ? bias[m * a.p.bias_sm + n * a.p.bias_sn] : 0.0f;
            const float rv = res ? res[m * a.p.res_sm + n * a.p.res_sn] : 0.0f;
            C[m * a.p.c_sm + n * a.p.c_sn] = gemm_epilogue(a.e, v[i], bv, rv);
          }
        }
      };

      if (a.split_k == 1) {
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          tmem_ld32(lane_addr + (uint32_t)c0, v);
          finish(v, c0);
        }
      } else {
        const int64_t tile_id = (int64_t)z * (a.tiles_m * a.tiles_n) + tile;
        float *part = a.ws_partial + ((tile_id * a.split_k + split) * kBM + row) * BN;
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          tmem_ld32(lane_addr + (uint32_t)c0, v);
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            if (c0 + i < BN)
              *reinterpret_cast<float4 *>(part + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        __threadfence();
        epi_bar_sync();
        if (et == 0) {
          const unsigned old = atomicAdd(a.ws_counter + tile_id, 1u);
          *last_flag = (old == (unsigned)a.split_k - 1u) ? 1 : 0;
        }
        epi_bar_sync();
        if (*last_flag) {
          __threadfence();
          const float *base = a.ws_partial + (tile_id * a.split_k * kBM + row) * BN;
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.0f;
            for (int sp = 0; sp < a.split_k; ++sp) {
              const float *src = base + (int64_t)sp * kBM * BN + c0;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                if (c0 + i < BN) {
                  const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + i));
                  v[i] += t.x; v[i + 1] += t.y; v[i + 2] += t.z; v[i + 3] += t.w;
                }
              }
            }
            finish(v, c0);
          }
          if (et == 0) a.ws_counter[tile_id] = 0u;  // ready for the next launch
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 4-D map: (inner contiguous dim, row dim, batch0, batch1), fp32, 128-byte swizzle.
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
  int tn = gp.tile_n;
  if (tn == 0) tn = p.N >= 1024 && p.M >= 1024 ? 128 : 64;
  if (tn > p.N) tn = (int)((p.N + 15) / 16 * 16);
  if (mn) tn = (tn + 31) / 32 * 32;  // MN-major B is loaded in 32-column boxes
  if (tn < 16) tn = 16;
  if (tn > 256) tn = 256;
  tn = tn / 16 * 16;
  plan.tile_n = tn;
  const int64_t tiles = ((p.M + kBM - 1) / kBM) * ((p.N + tn - 1) / tn) * batch;
  const int kb_total = (int)((p.K + kBK - 1) / kBK);
  int sk = gp.split_k;
  if (sk == 0) {
    // aim at one CTA per SM, keep at least two k blocks per split
    sk = (int)(148 / tiles);
    if (sk > kb_total / 2) sk = kb_total / 2;
    if (sk < 1) sk = 1;
  }
  if (sk > kb_total) sk = kb_total;
  if (sk > 65535) sk = 65535;
  // equalise: recompute from the per-split block count so no split is empty
  const int per = (kb_total + sk - 1) / sk;
  sk = (kb_total + per - 1) / per;
  plan.split_k = sk;
  const size_t stage = (size_t)(kABytes + tn * kBK * 4) * (plan.three_pass ? 2 : 1);
  int stages = (int)((200 * 1024) / stage);
  if (stages > 8) stages = 8;
  if (stages > per) stages = per;
  if (stages < 1) return false;
  plan.stages = stages;
  plan.smem_bytes = stages * stage + (3 * stages + 1) * 8 + 16 + 1024;
  plan.partial_bytes = sk > 1 ? (size_t)tiles * sk * kBM * tn * 4 : 0;
  plan.counter_bytes = sk > 1 ? (size_t)tiles * 4 : 0;
  return true;
}

int launch_gemm_tc(const GemmProblem &p, const GemmEpilogue &e, const TcPlan &plan, void *partials,
                   size_t partial_bytes, void *counters, size_t counter_bytes, cudaStream_t s) {
  TcArgs a;
  a.p = p; a.e = e;
  a.tile_n = plan.tile_n; a.split_k = plan.split_k; a.stages = plan.stages;
  a.b_mn_major = plan.b_mn_major; a.three_pass = plan.three_pass;
  a.tiles_m = (int)((p.M + kBM - 1) / kBM);
  a.tiles_n = (int)((p.N + plan.tile_n - 1) / plan.tile_n);
  a.kb_total = (int)((p.K + kBK - 1) / kBK);
  a.kb_per_split = (a.kb_total + plan.split_k - 1) / plan.split_k;
  a.status = device_status_word();
  FML_REQUIRE(a.status, FML_CUDA_ERROR, "fml_gemm: no device status word");
  a.ws_partial = nullptr; a.ws_counter = nullptr;
  if (plan.split_k > 1) {
    FML_REQUIRE(partials && partial_bytes >= plan.partial_bytes && counters &&
                    counter_bytes >= plan.counter_bytes, FML_BAD_ARG,
                "fml_gemm: split-K needs %zu partial and %zu counter bytes, got %zu and %zu",
                plan.partial_bytes, plan.counter_bytes, partial_bytes, counter_bytes);
    FML_REQUIRE(aligned16(partials) && ((uintptr_t)counters & 3) == 0, FML_MISALIGNED,
                "fml_gemm: partials must be 16-byte and counters 4-byte aligned");
    a.ws_counter = reinterpret_cast<unsigned *>(counters);
    a.ws_partial = reinterpret_cast<float *>(partials);
  }
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
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    FML_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev & 63] = true;
  }
  dim3 grid((unsigned)(a.tiles_m * a.tiles_n), (unsigned)plan.split_k, (unsigned)(p.nb0 * p.nb1));
  gemm_tc_kernel<<<grid, kThreads, plan.smem_bytes, s>>>(map_a, map_b, a);
  FML_CUDA(cudaGetLastError());
  return FML_OK;
}

}  // namespace fml
