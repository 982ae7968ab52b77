// Attention on tcgen05 for sm_100a: softmax(Q K^T / divisor + mask) V with both products on the
// tensor cores and the scores in tensor memory.  Replaces, for blocks too large for the CUDA-core
// kernel of attention.cu to pay off, the chain MatMul -> Div -> Add / Where -> Softmax -> MatMul
// the reference runs as five kernels (src/structure/kernel/kernel/matmul.cpp:28-59,
// softmax.cpp:22-139) with the [S_q, S_k] scores making two round trips through memory.
//
// One CTA per (batch x head, 128 query rows).  Keys are consumed in blocks of 128 with a running
// maximum (the streaming-softmax recurrence), so any number of keys works:
//   S   = Q K_blk^T        128 x 128 x D      tcgen05.mma kind::tf32, A = Q (shared memory,
//                                             K-major, 128-byte swizzle), B = K_blk (K-major),
//                                             accumulator in tensor memory
//   P   = exp(S / divisor + mask - m)         worker threads: one query row = one TMEM lane each
//   O_b = P V_blk          128 x D_v x 128    A = P from tensor memory (TS form), B = V_blk
//                                             (MN-major, 32-byte-atom swizzle)
//   O   = O * exp(m_old - m) + O_b            in registers, 64 floats per thread
// Both products are 3xTF32 (hi = x & 0xffffe000, lo = x - hi; lo*hi + hi*lo + hi*hi), so the
// result carries fp32-level error like the rest of the library: the workers write the lo parts of
// Q, K and V beside the tiles TMA delivered (the tensor core ignores the low 13 bits, so the
// delivered tile is the hi operand) and split P into hi / lo on its way into tensor memory.
//
// Roles (192 threads): warp 0 lane 0 issues the TMA loads (Q once, K / V per key block); warp 1
// allocates tensor memory and lane 0 issues the MMAs; warps 2-5 are the workers.  The phases of a
// key block run one after the other (no double buffering: Q, K, V and their lo parts fill the
// shared memory at D = 64); what the kernel saves is the memory traffic of the scores, not latency.
// Every wait is bounded: on expiry the kernel records kStatusTimeout, stops issuing work, frees its
// tensor memory and returns.
#include "common.cuh"
#include "tc_common.cuh"
#include <cuda.h>
#include <cstdlib>

namespace fml {
namespace {

constexpr int kKeys = 128;      // keys per block
constexpr int kThreads = 192;
constexpr float kNegBig = -3.0e38f;

struct AttnTcArgs {
  int Sq, Sk, D, Dv, nb0, nb1;  // nb0 = heads (inner batch), nb1 = batch
  int64_t m_s[4], o_s[4];
  const float *mask;
  float *out;
  float inv_divisor;
  int q_h, q_b, k_h, k_b, v_h, v_b;  // 0 where an operand is broadcast over heads / batch (the map's dim is 1 there)
  int *status;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const AttnTcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int dblk = a.D / 32, vgrp = a.Dv / 32;
  const uint32_t q_bytes = (uint32_t)dblk * 16384u;          // 128 rows x D floats
  const uint32_t k_bytes = q_bytes;                           // 128 keys x D floats
  const uint32_t v_kb_bytes = (uint32_t)vgrp * 4096u;         // 32 keys x D_v floats
  const uint32_t v_bytes = 4u * v_kb_bytes;                   // 128 keys x D_v floats
  // [ Q | Q_lo | K | K_lo | V | V_lo | barriers | flags ]
  uint8_t *q_hi = smem, *q_lo = q_hi + q_bytes, *k_hi = q_lo + q_bytes, *k_lo = k_hi + k_bytes;
  uint8_t *v_hi = k_lo + k_bytes, *v_lo = v_hi + v_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_lo + v_bytes);
  const uint32_t bar_q = smem_u32(bars), bar_kv = bar_q + 8, bar_conv = bar_q + 16, bar_s = bar_q + 24,
                 bar_p = bar_q + 32, bar_o = bar_q + 40;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 6);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // a 128-row x 32-key piece of a mask that differs between query rows (pitch 33: the piece is
  // written with lanes along the keys and read with lanes along the rows)
  float *mask_s = reinterpret_cast<float *>(tmem_slot + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = (int)blockIdx.x * kBM;
  const int z = (int)blockIdx.y, h = z % a.nb0, b = z / a.nb0;
  const int nkb = (a.Sk + kKeys - 1) / kKeys;
  // tensor memory: scores [0, 128), P hi / lo per 32 keys [128, 384), O_blk [384, 384 + D_v)
  constexpr uint32_t kColS = 0, kColP = 128, kColO = 384;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_conv, 4);  // one arrival per worker warp
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 4);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && !g_drop_loads) {  // (the wait test switches the loads off)
      bool ok = true;
      mbar_expect_tx(bar_q, q_bytes);
      for (int d = 0; d < dblk; ++d) tma_load_4d(smem_u32(q_hi) + (uint32_t)d * 16384u, &map_q, bar_q, d * 32, q0, h * a.q_h, b * a.q_b);
      int issued = 0;
      for (int it = 0; it < nkb && ok; ++it) {
        if (it > 0) {  // the MMAs of the previous block have read K and V
          ok = mbar_wait(bar_o, (uint32_t)(it - 1) & 1u, abort_flag);
          if (!ok) break;
        }
        const int key0 = it * kKeys;
        mbar_expect_tx(bar_kv, k_bytes + v_bytes);
        for (int d = 0; d < dblk; ++d) tma_load_4d(smem_u32(k_hi) + (uint32_t)d * 16384u, &map_k, bar_kv, d * 32, key0, h * a.k_h, b * a.k_b);
        for (int kb = 0; kb < 4; ++kb)
          for (int g = 0; g < vgrp; ++g)
            tma_load_4d(smem_u32(v_hi) + (uint32_t)kb * v_kb_bytes + (uint32_t)g * 4096u, &map_v, bar_kv, g * 32,
                        key0 + kb * 32, h * a.v_h, b * a.v_b);
        ++issued;
      }
      if (!ok) {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
        volatile int never = 0;  // bounded drain of the loads in flight before the CTA may exit
        mbar_wait(bar_q, 0u, &never);
        if (issued > 0) mbar_wait(bar_kv, (uint32_t)(issued - 1) & 1u, &never);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(kKeys, 0), idesc_o = instr_desc(a.Dv, 1);
      const uint64_t dq = smem_desc(smem_u32(q_hi), 16u, 1024u), dql = smem_desc(smem_u32(q_lo), 16u, 1024u);
      const uint64_t dk = smem_desc(smem_u32(k_hi), 16u, 1024u), dkl = smem_desc(smem_u32(k_lo), 16u, 1024u);
      const uint64_t dv = smem_desc(smem_u32(v_hi), 4096u, 512u, 1u), dvl = smem_desc(smem_u32(v_lo), 4096u, 512u, 1u);
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const uint32_t ph = (uint32_t)it & 1u;
        ok = mbar_wait(bar_conv, ph, abort_flag);  // lo parts written, previous O_blk read
        if (!ok) break;
        tc_fence_after();
        for (int d = 0; d < dblk; ++d) {
          const uint32_t toff = ((uint32_t)d * 16384u) >> 4;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t o = toff + (uint32_t)j * 2u;  // 32 bytes further along a K-major row
            umma_tf32(tmem_base + kColS, dql + o, dk + o, idesc_s, (d == 0 && j == 0) ? 0u : 1u);
            umma_tf32(tmem_base + kColS, dq + o, dkl + o, idesc_s, 1u);
            umma_tf32(tmem_base + kColS, dq + o, dk + o, idesc_s, 1u);
          }
        }
        umma_commit(bar_s);
        ok = mbar_wait(bar_p, ph, abort_flag);  // P is in tensor memory
        if (!ok) break;
        tc_fence_after();
        const int keys = min(kKeys, a.Sk - it * kKeys), kbs = (keys + 31) / 32;
        for (int kb = 0; kb < kbs; ++kb) {
          const uint32_t voff = ((uint32_t)kb * v_kb_bytes) >> 4;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t o = voff + (uint32_t)j * 64u;  // 8 k rows = 1024 bytes further down
            const uint32_t p_hi = tmem_base + kColP + (uint32_t)kb * 64u + (uint32_t)j * 8u, p_lo = p_hi + 32u;
            umma_tf32_ts(tmem_base + kColO, p_lo, dv + o, idesc_o, (kb == 0 && j == 0) ? 0u : 1u);
            umma_tf32_ts(tmem_base + kColO, p_hi, dvl + o, idesc_o, 1u);
            umma_tf32_ts(tmem_base + kColO, p_hi, dv + o, idesc_o, 1u);
          }
        }
        umma_commit(bar_o);
      }
      if (!ok) {
        atomicOr(a.status, kStatusTimeout);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ workers: one query row each
    const int et = threadIdx.x - 64;  // 0..127
    const int qw = warp & 3, row = qw * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(qw * 32) << 16);
    const int q = q0 + row;
    const bool q_ok = q < a.Sq;
    const float *mrow = a.mask ? a.mask + (int64_t)b * a.m_s[0] + (int64_t)h * a.m_s[1] + (int64_t)(q_ok ? q : a.Sq - 1) * a.m_s[2]
                               : nullptr;
    const int64_t m_sk = a.m_s[3];
    auto lo4 = [](uint4 x) {
      uint4 lo;
      lo.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(x.x & 0xffffe000u));
      lo.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(x.y & 0xffffe000u));
      lo.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(x.z & 0xffffe000u));
      lo.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(x.w & 0xffffe000u));
      return lo;
    };
    auto split_tile = [&](const uint8_t *hi, uint8_t *lo, uint32_t bytes) {  // layout-agnostic: element-wise
      const uint4 *src = reinterpret_cast<const uint4 *>(hi);
      uint4 *dst = reinterpret_cast<uint4 *>(lo);
      const int n = (int)(bytes >> 4);
      for (int i = et; i < n; i += 512) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) if (i + 128 * u < n) x[u] = src[i + 128 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u) if (i + 128 * u < n) dst[i + 128 * u] = lo4(x[u]);
      }
    };
    // The workers meet at named barriers below, so they must agree on whether to go on: a wait's
    // outcome is reduced over the 128 of them before anyone acts on it.
    auto all_ok = [](bool mine) -> bool {
      uint32_t r;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.b32 q, %1, 0;\n\t"
          "bar.red.and.pred p, 2, 128, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(r) : "r"((uint32_t)mine) : "memory");
      return r != 0;
    };
    float o_acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o_acc[i] = 0.0f;
    float m_run = kNegBig, l_run = 0.0f;
    const float log2e = 1.4426950408889634f;
    bool ok = true;
    for (int it = 0; it < nkb && ok; ++it) {
      const uint32_t ph = (uint32_t)it & 1u;
      if (it == 0) {
        ok = all_ok(mbar_wait(bar_q, 0u, abort_flag));
        if (!ok) break;
        split_tile(q_hi, q_lo, q_bytes);
      }
      ok = all_ok(mbar_wait(bar_kv, ph, abort_flag));
      if (!ok) break;
      split_tile(k_hi, k_lo, k_bytes);
      split_tile(v_hi, v_lo, v_bytes);
      tc_fence_before();   // this thread's reads of O_blk (previous block) are done
      fence_async_smem();  // the lo tiles are visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_conv);

      ok = all_ok(mbar_wait(bar_s, ph, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int key0 = it * kKeys;
      // pass 1: scaled and masked scores back into tensor memory, and the block's row maximum.
      // A mask that is the same for every query row is read directly (all lanes, one address); one
      // that differs between rows goes through shared memory in pieces of 32 keys, loaded with
      // lanes along the keys: read per thread along its own row it would touch 32 cache lines per
      // load instruction.
      const bool per_row_mask = mrow && a.m_s[2] != 0;
      float bmax = kNegBig;
      for (int c = 0; c < 4; ++c) {
        if (per_row_mask) {
          asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous piece has been consumed
          const float *mb = a.mask + (int64_t)b * a.m_s[0] + (int64_t)h * a.m_s[1];
          const int key = key0 + c * 32 + lane;
          for (int r = qw; r < kBM; r += 4) {
            const int qq = min(q0 + r, a.Sq - 1);
            mask_s[r * 33 + lane] = key < a.Sk ? __ldg(mb + (int64_t)qq * a.m_s[2] + (int64_t)key * m_sk) : 0.0f;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        float v[32];
        tmem_ld32(lane_addr + kColS + (uint32_t)c * 32u, v);
        uint32_t sv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + c * 32 + i;
          float s = kNegBig;
          if (key < a.Sk) {
            s = v[i] * a.inv_divisor;
            if (per_row_mask) s += mask_s[row * 33 + i];
            else if (mrow) s += __ldg(mrow + (int64_t)key * m_sk);
            s = fmaxf(s, kNegBig);
            bmax = fmaxf(bmax, s);
          }
          sv[i] = __float_as_uint(s);
        }
        tmem_st32(lane_addr + kColS + (uint32_t)c * 32u, sv);
      }
      tmem_wait_st();
      const float m_new = fmaxf(m_run, bmax);
      const float alpha = exp2f((m_run - m_new) * log2e);
      // pass 2: P = exp(s - m), split into hi / lo, into tensor memory; row sum
      float bsum = 0.0f;
      for (int c = 0; c < 4; ++c) {
        float v[32];
        tmem_ld32(lane_addr + kColS + (uint32_t)c * 32u, v);
        uint32_t hi[32], lo[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + c * 32 + i;
          const float p = key < a.Sk ? exp2f((v[i] - m_new) * log2e) : 0.0f;
          bsum += p;
          const uint32_t u = __float_as_uint(p), uh = u & 0xffffe000u;
          hi[i] = uh;
          lo[i] = __float_as_uint(p - __uint_as_float(uh));
        }
        tmem_st32(lane_addr + kColP + (uint32_t)c * 64u, hi);
        tmem_st32(lane_addr + kColP + (uint32_t)c * 64u + 32u, lo);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p);

      ok = all_ok(mbar_wait(bar_o, ph, abort_flag));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {  // compile-time bound: o_acc stays in registers
        if (c < vgrp) {
          float v[32];
          tmem_ld32(lane_addr + kColO + (uint32_t)c * 32u, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + v[i];
        }
      }
      l_run = l_run * alpha + bsum;
      m_run = m_new;
    }
    if (!ok) {
      atomicOr(a.status, kStatusTimeout);
      *abort_flag = 1;
    } else if (q_ok) {
      const float inv = 1.0f / l_run;
      float *op = a.out + (int64_t)b * a.o_s[0] + (int64_t)h * a.o_s[1] + (int64_t)q * a.o_s[2];
      if (a.o_s[3] == 1 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 64; i += 4)
          if (i < a.Dv)
            *reinterpret_cast<float4 *>(op + i) = make_float4(o_acc[i] * inv, o_acc[i + 1] * inv, o_acc[i + 2] * inv, o_acc[i + 3] * inv);
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < a.Dv) op[(int64_t)i * a.o_s[3]] = o_acc[i] * inv;
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

// 4-D map over a [batch, heads, rows, inner] view (inner contiguous), fp32.
int make_map4(CUtensorMap *map, const float *base, int64_t inner, int64_t rows, int64_t row_stride, int64_t nh,
              int64_t h_stride, int64_t nb, int64_t b_stride, int box_inner, int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  FML_REQUIRE(fn, FML_CUDA_ERROR, "fml_attention: cuTensorMapEncodeTiled is not available");
  const int64_t dummy = row_stride * rows;  // extent-1 dims take any valid stride
  cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(h_stride ? nh : 1), (cuuint64_t)(b_stride ? nb : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)row_stride * 4, (cuuint64_t)(h_stride ? h_stride : dummy) * 4,
                           (cuuint64_t)(b_stride ? b_stride : dummy) * 4};
  cuuint32_t box[4] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FML_REQUIRE(r == CUDA_SUCCESS, FML_CUDA_ERROR, "fml_attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return FML_OK;
}

bool stride_ok(int64_t s) { return s == 0 || (s > 0 && s % 4 == 0); }

}  // namespace

// Shapes the tensor-core kernel takes at all (operand strides are checked at launch).
bool attention_tc_shape_ok(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v) {
  return s_q >= 1 && s_k >= 1 && (d == 32 || d == 64) && (d_v == 32 || d_v == 64);
}

// Whether fml_attention sends this problem to the tensor-core kernel.  q: [nb1, nb0, Sq, D],
// kt: [nb1, nb0, D, Sk] (a view whose D stride is 1), v: [nb1, nb0, Sk, Dv]; strides in elements.
bool attention_tc_eligible(int64_t nb1, int64_t nb0, int64_t Sq, int64_t Sk, int64_t D, int64_t Dv, const int64_t *q_s,
                           const int64_t *k_s, const int64_t *v_s, const void *q, const void *k, const void *v) {
  static const int mode = [] { const char *e = getenv("FLUIDML_ATTENTION_TC"); return e ? atoi(e) : -1; }();
  if (mode == 0 || !attention_tc_shape_ok(Sq, Sk, D, Dv)) return false;
  if (q_s[3] != 1 || k_s[2] != 1 || v_s[3] != 1) return false;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v)) return false;
  if (q_s[2] <= 0 || q_s[2] % 4 || k_s[3] <= 0 || k_s[3] % 4 || v_s[2] <= 0 || v_s[2] % 4) return false;
  if (!stride_ok(q_s[0]) || !stride_ok(q_s[1]) || !stride_ok(k_s[0]) || !stride_ok(k_s[1]) || !stride_ok(v_s[0]) || !stride_ok(v_s[1]))
    return false;
  if (nb0 * nb1 > 65535 || nb0 * nb1 < 1) return false;
  if (mode == 1) return true;
  // below ~200 Mflop, or with fewer tiles than two thirds of the SMs, the CUDA-core kernel's many
  // small CTAs finish sooner than a few large tiles (8 x 6 heads x 128 rows: 25 us against 30)
  return 4.0 * (double)nb0 * (double)nb1 * (double)Sq * (double)Sk * (double)D >= 200e6 &&
         nb0 * nb1 * ((Sq + kBM - 1) / kBM) >= 96;
}

int launch_attention_tc(int64_t nb1, int64_t nb0, int64_t Sq, int64_t Sk, int64_t D, int64_t Dv, const float *q,
                        const int64_t *q_s, const float *k, const int64_t *k_s, const float *v, const int64_t *v_s,
                        const float *mask, const int64_t *m_s, float divisor, float *out, const int64_t *o_s,
                        cudaStream_t s) {
  AttnTcArgs a;
  a.Sq = (int)Sq; a.Sk = (int)Sk; a.D = (int)D; a.Dv = (int)Dv; a.nb0 = (int)nb0; a.nb1 = (int)nb1;
  for (int i = 0; i < 4; ++i) { a.m_s[i] = mask ? m_s[i] : 0; a.o_s[i] = o_s[i]; }
  a.mask = mask; a.out = out; a.inv_divisor = 1.0f / divisor;
  a.q_h = q_s[1] != 0; a.q_b = q_s[0] != 0; a.k_h = k_s[1] != 0; a.k_b = k_s[0] != 0; a.v_h = v_s[1] != 0; a.v_b = v_s[0] != 0;
  a.status = device_status_word();
  FML_REQUIRE(a.status, FML_CUDA_ERROR, "fml_attention: no device status word");
  CUtensorMap mq, mk, mv;
  int st = make_map4(&mq, q, D, Sq, q_s[2], nb0, q_s[1], nb1, q_s[0], 32, kBM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != FML_OK) return st;
  st = make_map4(&mk, k, D, Sk, k_s[3], nb0, k_s[1], nb1, k_s[0], 32, kKeys, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st != FML_OK) return st;
  st = make_map4(&mv, v, Dv, Sk, v_s[2], nb0, v_s[1], nb1, v_s[0], 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (st != FML_OK) return st;
  const size_t smem = (size_t)(D / 32) * 16384 * 4 + (size_t)(Dv / 32) * 4096 * 4 * 2 + 6 * 8 + 16 + 128 * 33 * 4 + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    FML_CUDA(cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev & 63] = true;
  }
  const dim3 grid((unsigned)((Sq + kBM - 1) / kBM), (unsigned)(nb0 * nb1));
  FML_CUDA(launch_kernel(attention_tc_kernel, grid, dim3(kThreads), smem, s, mq, mk, mv, a));
  return FML_OK;
}

}  // namespace fml
