// Fused attention core: out = softmax(Q K^T / divisor + mask) V for one block of query rows
// of one head per CTA, all in fp32 FMA.
//
// At batch-1 sequence lengths the three launches this replaces (scores GEMM, masked softmax,
// context GEMM) are each a few microseconds of launch, ramp and drain around well under a
// microsecond of arithmetic (12 heads x 128 x 128 x 64 x 2 products = 50 MFLOP), and the
// score matrix makes a round trip through L2 between them.  Here K and V of the head are
// staged once in shared memory (they fit: S_k * (D + D_v) floats), the 16 x S_k block of
// scores never leaves the SM, and the fp32 FMAs give the oracle's precision without the
// 3xTF32 split.  Operands are arbitrary strided views, so the head split / merge transposes
// of the graph stay views.
#include "common.cuh"

namespace fml {
namespace {

constexpr int kRows = 16;      // query rows per CTA
constexpr int kThreads = 256;  // 16 threads per query row
constexpr size_t kSmemLimit = 200 * 1024;

struct AttnArgs {
  int64_t Sq, Sk, D, Dv, nb0, nb1;
  // element strides: batch outer, batch inner, row, col
  int64_t q_s[4], k_s[4], v_s[4], o_s[4], m_s[4];  // k: [.., D, Sk] -> k_s[2] = stride of d, k_s[3] = stride of j
  const float *q, *k, *v, *mask;
  float *out;
  float divisor;
};

__device__ __forceinline__ void cp_async16(float *dst_smem, const float *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst_smem)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// dst[row * pitch + col] = src[row * s_row + col * s_col] for a rows x cols tile.  Rows that
// are contiguous and 16-byte aligned stream in with asynchronous 16-byte copies (no register
// staging, all of them in flight at once); other layouts go through registers, four loads
// at a time.  The caller commits / waits on the async group.
__device__ __forceinline__ void load_tile(float *dst, int pitch, const float *src, int rows, int cols,
                                          int64_t s_row, int64_t s_col) {
  const bool vec = s_col == 1 && (cols & 3) == 0 && (s_row & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  if (vec) {
    const int c4 = cols >> 2;
    for (int i = threadIdx.x; i < rows * c4; i += kThreads) {
      const int r = i / c4, c = (i - r * c4) << 2;
      cp_async16(dst + r * pitch + c, src + r * s_row + c);
    }
    return;
  }
  const bool by_rows = s_row == 1;  // rows are the contiguous direction: walk them fastest
  const int total = rows * cols;
  for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kThreads) {
    float v[4];
    int at[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * kThreads;
      int r = 0, c = 0;
      if (i < total) {
        if (by_rows) { c = i / rows; r = i - c * rows; }
        else { r = i / cols; c = i - r * cols; }
      }
      at[u] = i < total ? r * pitch + c : -1;
      v[u] = i < total ? src[r * s_row + c * s_col] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (at[u] >= 0) dst[at[u]] = v[u];
  }
}

// Shared-memory bandwidth (128 bytes per clock per SM, whatever the broadcast pattern of a
// 16-byte read) is what bounds the two products, so both use register tiles that do many
// FMAs per byte read:
//   scores   each half of the CTA takes half of the head dimension; a thread holds a 4 x 4
//            tile (rows rq + 4x, columns cq + 32u): per 4 values of d, 4 Q and 4 K 16-byte
//            reads feed 64 FMAs; the second half adds its partial scores to the first's.
//   context  warp w takes an eighth of the keys; a thread holds 4 rows x 8 output columns:
//            per key, 4 P values and two 16-byte V reads feed 32 FMAs; the eight partial
//            tiles are added in warp order through shared memory.
__global__ void __launch_bounds__(kThreads) attention_kernel(AttnArgs a) {
  const ExactDivisor div(a.divisor);  // 1 / sqrt(head size) is usually a power of two: a multiply, same bits
  pdl_prologue();
  extern __shared__ __align__(16) float smem[];
  const int D = (int)a.D, Dv = (int)a.Dv, Sk = (int)a.Sk;
  const int pk = D + 4;     // K / Q pitch: 16-byte aligned rows, conflict-free 16-byte reads
  const int pp = Sk | 1;    // score pitch, odd: rows rq, rq + 1, .. fall in different banks
  float *Qs = smem;                    // [kRows][pk]
  float *Ks = Qs + kRows * pk;         // [Sk][pk]
  float *Vs = Ks + (size_t)Sk * pk;    // [Sk][Dv]
  float *Red = Vs + (size_t)Sk * Dv;   // [8][kRows][Dv] partial context tiles
  float *Ps = Red + 8 * kRows * Dv;    // [kRows][pp]
  float *Ms = Ps + kRows * pp;         // [kRows or 1][Sk] mask values of this block
  const int64_t z0 = blockIdx.y % a.nb0, z1 = blockIdx.y / a.nb0;
  const int64_t row0 = (int64_t)blockIdx.x * kRows;
  const int rows = (int)min((int64_t)kRows, a.Sq - row0);
  const float *q = a.q + z1 * a.q_s[0] + z0 * a.q_s[1] + row0 * a.q_s[2];
  const float *k = a.k + z1 * a.k_s[0] + z0 * a.k_s[1];
  const float *v = a.v + z1 * a.v_s[0] + z0 * a.v_s[1];
  float *o = a.out + z1 * a.o_s[0] + z0 * a.o_s[1] + row0 * a.o_s[2];
  const float *m = a.mask ? a.mask + z1 * a.m_s[0] + z0 * a.m_s[1] + row0 * a.m_s[2] : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (rows < kRows)  // the tail block: unused query rows must not feed NaNs into the tiles
    for (int i = threadIdx.x; i < (kRows - rows) * pk; i += kThreads) Qs[rows * pk + i] = 0.0f;
  load_tile(Qs, pk, q, rows, D, a.q_s[2], a.q_s[3]);
  load_tile(Ks, pk, k, Sk, D, a.k_s[3], a.k_s[2]);  // Ks[j][d] = K^T[d][j]
  const int mrows = m ? (a.m_s[2] == 0 ? 1 : rows) : 0;  // a mask that broadcasts over query rows is staged once
  if (mrows) load_tile(Ms, Sk, m, mrows, Sk, a.m_s[2], a.m_s[3]);
  cp_async_commit();
  load_tile(Vs, Dv, v, Sk, Dv, a.v_s[2], a.v_s[3]);  // V keeps streaming under the score phase
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  // ---- scores: Ps[r][j] = q_r . k_j
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
      const int qstep = pk;  // rows rq, rq + 4, rq + 8, rq + 12 are 4 * pk floats = pk float4 apart
#pragma unroll 2
      for (int d = d_lo; d < d_hi; ++d) {
        float4 qv[4], kv[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) qv[x] = q4[x * qstep + d];
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
      // the first half stores, the second half adds: a fixed order
      for (int turn = 0; turn < 2; ++turn) {
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
        __syncthreads();
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // ---- softmax(s / divisor + mask) over each row; a row's 16 threads are half a warp
  {
    const int r = threadIdx.x >> 4, cg = threadIdx.x & 15;
    const bool live = r < rows;
    float *p = Ps + r * pp;
    const float *mr = Ms + (mrows > 1 ? r * Sk : 0);
    float mx = -3.402823466e+38f;
    if (live)
      for (int j = cg; j < Sk; j += 16) {
        float sc = p[j];
        if (a.divisor != 1.0f) sc = div(sc);
        if (m) sc += mr[j];
        p[j] = sc;
        mx = fmaxf(mx, sc);
      }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
    float sum = 0.0f;
    if (live)
      for (int j = cg; j < Sk; j += 16) {
        const float e = expf(p[j] - mx);
        p[j] = e;
        sum += e;
      }
#pragma unroll
    for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
    for (int j = cg; j < Sk; j += 16) p[j] = live ? p[j] / sum : 0.0f;
  }
  __syncthreads();
  // ---- context: out[r][dv] = sum_j P[r][j] V[j][dv]
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
      if (dv0) __syncthreads();  // the previous pass's partial tiles have been consumed
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        float *dst = Red + ((size_t)warp * kRows + rg + 4 * x) * Dv;
        if (has_a) *reinterpret_cast<float4 *>(dst + ca) = acc[x][0];
        if (has_b) *reinterpret_cast<float4 *>(dst + cb) = acc[x][1];
      }
      __syncthreads();
      // add the eight partial tiles in warp order and store 16 rows x up to 64 columns
      const int w4 = min(64, Dv - dv0) >> 2;
      for (int i = threadIdx.x; i < kRows * w4; i += kThreads) {
        const int r = i / w4, c = dv0 + ((i - r * w4) << 2);
        if (r >= rows) continue;
        float4 t = *reinterpret_cast<const float4 *>(Red + (size_t)r * Dv + c);
#pragma unroll
        for (int w = 1; w < 8; ++w) {
          const float4 u = *reinterpret_cast<const float4 *>(Red + ((size_t)w * kRows + r) * Dv + c);
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        float *dst = o + r * a.o_s[2] + c * a.o_s[3];
        const bool ovec = a.o_s[3] == 1 && (a.o_s[2] & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0;
        if (ovec) *reinterpret_cast<float4 *>(dst) = t;
        else { dst[0] = t.x; dst[a.o_s[3]] = t.y; dst[2 * a.o_s[3]] = t.z; dst[3 * a.o_s[3]] = t.w; }
      }
    }
  }
}

// Keys and values that do not fit in shared memory at once (long sequences) stream through it in
// chunks of 128 keys with the running-maximum ("online") softmax: per chunk the scores, their
// maximum m' = max(m, chunk max), the weights e = exp(s - m'), and the context accumulator and
// the normaliser l rescaled by exp(m - m') before the chunk's contribution is added; the output
// is accumulator / l.  The arithmetic is that of softmax followed by the product, in another
// order (within a few ulp per element).  Tiles, thread mappings and the warp-ordered reduction
// are those of attention_kernel.
constexpr int kChunk = 128;

__global__ void __launch_bounds__(kThreads) attention_flash_kernel(AttnArgs a) {
  const ExactDivisor div(a.divisor);  // 1 / sqrt(head size) is usually a power of two: a multiply, same bits
  pdl_prologue();
  extern __shared__ __align__(16) float smem[];
  const int D = (int)a.D, Dv = (int)a.Dv, Sk = (int)a.Sk;
  const int pk = D + 4, pp = kChunk | 1;
  float *Qs = smem;                        // [kRows][pk]
  float *Ks = Qs + kRows * pk;             // [kChunk][pk]
  float *Vs = Ks + (size_t)kChunk * pk;    // [kChunk][Dv]
  float *Red = Vs + (size_t)kChunk * Dv;   // [8][kRows][Dv]
  float *Ps = Red + 8 * kRows * Dv;        // [kRows][pp]
  float *Ms = Ps + kRows * pp;             // [kRows or 1][kChunk]
  float *row_m = Ms + kRows * kChunk;      // [kRows] running maximum
  float *row_l = row_m + kRows;            // [kRows] running normaliser
  float *row_scale = row_l + kRows;        // [kRows] exp(old maximum - new maximum) of the current chunk
  const int64_t z0 = blockIdx.y % a.nb0, z1 = blockIdx.y / a.nb0;
  const int64_t row0 = (int64_t)blockIdx.x * kRows;
  const int rows = (int)min((int64_t)kRows, a.Sq - row0);
  const float *q = a.q + z1 * a.q_s[0] + z0 * a.q_s[1] + row0 * a.q_s[2];
  const float *k = a.k + z1 * a.k_s[0] + z0 * a.k_s[1];
  const float *v = a.v + z1 * a.v_s[0] + z0 * a.v_s[1];
  float *o = a.out + z1 * a.o_s[0] + z0 * a.o_s[1] + row0 * a.o_s[2];
  const float *m = a.mask ? a.mask + z1 * a.m_s[0] + z0 * a.m_s[1] + row0 * a.m_s[2] : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mrows = m ? (a.m_s[2] == 0 ? 1 : rows) : 0;

  if (rows < kRows)
    for (int i = threadIdx.x; i < (kRows - rows) * pk; i += kThreads) Qs[rows * pk + i] = 0.0f;
  if (threadIdx.x < kRows) { row_m[threadIdx.x] = -3.402823466e+38f; row_l[threadIdx.x] = 0.0f; }
  load_tile(Qs, pk, q, rows, D, a.q_s[2], a.q_s[3]);
  // context accumulators of the threads that combine the partial tiles: 16 rows x Dv / 4 quads over
  // 256 threads = at most two per thread (Dv <= 128)
  float4 acc_out0 = make_float4(0.f, 0.f, 0.f, 0.f), acc_out1 = acc_out0;

  for (int j0 = 0; j0 < Sk; j0 += kChunk) {
    const int kc = min(kChunk, Sk - j0);
    __syncthreads();  // the previous chunk's K, V, P and partial tiles are no longer read
    load_tile(Ks, pk, k + (int64_t)j0 * a.k_s[3], kc, D, a.k_s[3], a.k_s[2]);
    if (mrows) load_tile(Ms, kChunk, m + (int64_t)j0 * a.m_s[3], mrows, kc, a.m_s[2], a.m_s[3]);
    cp_async_commit();
    load_tile(Vs, Dv, v + (int64_t)j0 * a.v_s[2], kc, Dv, a.v_s[2], a.v_s[3]);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    // ---- scores of the chunk
    {
      const int half = warp >> 2, rq = warp & 3, cq = lane;
      const int n4 = D >> 2, d_lo = half ? n4 >> 1 : 0, d_hi = half ? n4 : n4 >> 1;
      float acc[4][4];
      const float4 *k4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[x][u] = 0.0f;
        k4[u] = reinterpret_cast<const float4 *>(Ks + (size_t)min(cq + 32 * u, kc - 1) * pk);
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
      for (int turn = 0; turn < 2; ++turn) {
        if (turn == half) {
#pragma unroll
          for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int j = cq + 32 * u;
              if (j < kc) {
                float *dst = Ps + (rq + 4 * x) * pp + j;
                *dst = turn ? *dst + acc[x][u] : acc[x][u];
              }
            }
        }
        __syncthreads();
      }
    }
    cp_async_wait<0>();
    __syncthreads();
    // ---- running softmax of the chunk
    {
      const int r = threadIdx.x >> 4, cg = threadIdx.x & 15;
      const bool live = r < rows;
      float *p = Ps + r * pp;
      const float *mr = Ms + (mrows > 1 ? r * kChunk : 0);
      const float m_old = row_m[r], l_old = row_l[r];
      float mx = m_old;
      if (live)
        for (int j = cg; j < kc; j += 16) {
          float sc = p[j];
          if (a.divisor != 1.0f) sc = div(sc);
          if (m) sc += mr[j];
          p[j] = sc;
          mx = fmaxf(mx, sc);
        }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o2));
      float sum = 0.0f;
      for (int j = cg; j < kc; j += 16) {
        const float e = live ? expf(p[j] - mx) : 0.0f;
        p[j] = e;
        sum += e;
      }
#pragma unroll
      for (int o2 = 8; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
      __syncwarp();
      if (cg == 0) {
        const float sc = expf(m_old - mx);  // 0 for the first chunk (m_old is the float lowest)
        row_scale[r] = sc;
        row_m[r] = mx;
        row_l[r] = l_old * sc + sum;
      }
    }
    __syncthreads();
    // ---- context contribution of the chunk, added to the rescaled accumulators
    {
      const int rg = lane >> 3, cgp = lane & 7;
      const int per = (kc + 7) >> 3, j_lo = min(kc, warp * per), j_hi = min(kc, j_lo + per);
      const float *p0 = Ps + rg * pp;
      int pass = 0;
      for (int dv0 = 0; dv0 < Dv; dv0 += 64, ++pass) {
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
        if (dv0) __syncthreads();
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float *dst = Red + ((size_t)warp * kRows + rg + 4 * x) * Dv;
          if (has_a) *reinterpret_cast<float4 *>(dst + ca) = acc[x][0];
          if (has_b) *reinterpret_cast<float4 *>(dst + cb) = acc[x][1];
        }
        __syncthreads();
        const int w4 = min(64, Dv - dv0) >> 2;
        const int i = threadIdx.x;  // 16 rows x at most 16 quads: one (row, quad) per thread and pass
        if (i < kRows * w4) {
          const int r = i / w4, c = dv0 + ((i - r * w4) << 2);
          float4 t = *reinterpret_cast<const float4 *>(Red + (size_t)r * Dv + c);
#pragma unroll
          for (int w = 1; w < 8; ++w) {
            const float4 u = *reinterpret_cast<const float4 *>(Red + ((size_t)w * kRows + r) * Dv + c);
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
          }
          const float sc = row_scale[r];
          float4 &ao = pass == 0 ? acc_out0 : acc_out1;
          ao.x = ao.x * sc + t.x; ao.y = ao.y * sc + t.y; ao.z = ao.z * sc + t.z; ao.w = ao.w * sc + t.w;
        }
      }
    }
  }
  // ---- out = accumulator / normaliser
  int pass = 0;
  for (int dv0 = 0; dv0 < Dv; dv0 += 64, ++pass) {
    const int w4 = min(64, Dv - dv0) >> 2;
    const int i = threadIdx.x;
    if (i < kRows * w4) {
      const int r = i / w4, c = dv0 + ((i - r * w4) << 2);
      if (r < rows) {
        const float l = row_l[r];
        const float4 ao = pass == 0 ? acc_out0 : acc_out1;
        const float4 t = make_float4(ao.x / l, ao.y / l, ao.z / l, ao.w / l);
        float *dst = o + r * a.o_s[2] + c * a.o_s[3];
        const bool ovec = a.o_s[3] == 1 && (a.o_s[2] & 3) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0;
        if (ovec) *reinterpret_cast<float4 *>(dst) = t;
        else { dst[0] = t.x; dst[a.o_s[3]] = t.y; dst[2 * a.o_s[3]] = t.z; dst[3 * a.o_s[3]] = t.w; }
      }
    }
  }
}

size_t attn_flash_smem_bytes(int64_t D, int64_t Dv) {
  return (size_t)(kRows * (D + 4) + kChunk * (D + 4) + kChunk * Dv + 8 * kRows * Dv + kRows * (kChunk | 1) +
                  kRows * kChunk + 3 * kRows) * sizeof(float);
}

size_t attn_smem_bytes(int64_t Sk, int64_t D, int64_t Dv) {
  return (size_t)(kRows * (D + 4) + Sk * (D + 4) + Sk * Dv + 8 * kRows * Dv + kRows * (Sk | 1) + kRows * Sk) * sizeof(float);
}

// Pads the tensor's dims to [b1, b0, rows, cols] (leading 1s) and returns its strides.
bool as4(const fml_tensor *t, int64_t shape[4], int64_t stride[4]) {
  if (t->rank < 2 || t->rank > 4) return false;
  const int pad = 4 - t->rank;
  for (int i = 0; i < 4; ++i) {
    shape[i] = i < pad ? 1 : t->shape[i - pad];
    stride[i] = i < pad ? 0 : t->stride[i - pad];
  }
  return true;
}

}  // namespace
}  // namespace fml

using namespace fml;

namespace fml {  // attention_tc.cu
bool attention_tc_shape_ok(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v);
bool attention_tc_eligible(int64_t nb1, int64_t nb0, int64_t Sq, int64_t Sk, int64_t D, int64_t Dv, const int64_t *q_s,
                           const int64_t *k_s, const int64_t *v_s, const void *q, const void *k, const void *v);
int launch_attention_tc(int64_t nb1, int64_t nb0, int64_t Sq, int64_t Sk, int64_t D, int64_t Dv, const float *q,
                        const int64_t *q_s, const float *k, const int64_t *k_s, const float *v, const int64_t *v_s,
                        const float *mask, const int64_t *m_s, float divisor, float *out, const int64_t *o_s,
                        cudaStream_t s);
}  // namespace fml

// 1 when the tensor-core kernel (attention_tc.cu) takes blocks of these head sizes: such blocks are
// worth fusing whatever their size, the CUDA-core kernel only while the block is small.
extern "C" int fml_attention_on_tensor_cores(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v) {
  return attention_tc_shape_ok(s_q, s_k, d, d_v) ? 1 : 0;
}

extern "C" int fml_attention_supported(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v) {
  // any number of keys: those that do not fit in shared memory at once stream through it
  return s_q >= 1 && s_k >= 1 && d >= 4 && d_v >= 4 && d <= 128 && d_v <= 128 && (d & 3) == 0 && (d_v & 3) == 0 &&
                 (attn_smem_bytes(s_k, d, d_v) <= kSmemLimit || attn_flash_smem_bytes(d, d_v) <= kSmemLimit)
             ? 1 : 0;
}

extern "C" int fml_attention(const fml_tensor *q, const fml_tensor *kt, const fml_tensor *v,
                             const fml_tensor *mask, float divisor, const fml_tensor *out, void *stream) {
  FML_REQUIRE(q && kt && v && out, FML_BAD_ARG, "fml_attention: null tensor");
  FML_REQUIRE(q->dtype == FML_F32 && kt->dtype == FML_F32 && v->dtype == FML_F32 && out->dtype == FML_F32 &&
                  (!mask || mask->dtype == FML_F32), FML_UNSUPPORTED, "fml_attention: fp32 only");
  FML_REQUIRE(divisor != 0.0f, FML_BAD_ARG, "fml_attention: divisor is zero");
  AttnArgs a;
  int64_t qs[4], ks[4], vs[4], os[4], ms[4] = {1, 1, 1, 1};
  FML_REQUIRE(as4(q, qs, a.q_s) && as4(kt, ks, a.k_s) && as4(v, vs, a.v_s) && as4(out, os, a.o_s) &&
                  (!mask || as4(mask, ms, a.m_s)), FML_UNSUPPORTED, "fml_attention: ranks 2 to 4 only");
  a.nb1 = qs[0]; a.nb0 = qs[1]; a.Sq = qs[2]; a.D = qs[3]; a.Sk = ks[3]; a.Dv = vs[3];
  FML_REQUIRE(ks[2] == a.D && vs[2] == a.Sk && os[2] == a.Sq && os[3] == a.Dv, FML_BAD_ARG,
              "fml_attention: shapes do not chain (Q [..,%lld,%lld], K^T [..,%lld,%lld], V [..,%lld,%lld])",
              (long long)a.Sq, (long long)a.D, (long long)ks[2], (long long)ks[3], (long long)vs[2], (long long)vs[3]);
  for (int i = 0; i < 2; ++i)
    FML_REQUIRE(ks[i] == qs[i] && vs[i] == qs[i] && os[i] == qs[i], FML_BAD_ARG,
                "fml_attention: batch dims of Q, K^T, V and the output must agree");
  if (mask) {
    const int64_t want[4] = {a.nb1, a.nb0, a.Sq, a.Sk};
    for (int i = 0; i < 4; ++i) {
      FML_REQUIRE(ms[i] == want[i] || ms[i] == 1, FML_BAD_ARG, "fml_attention: mask does not broadcast to the scores");
      if (ms[i] == 1) a.m_s[i] = 0;
    }
  }
  if (a.Sq == 0 || a.Dv == 0 || a.nb0 * a.nb1 == 0) return FML_OK;
  FML_REQUIRE(fml_attention_supported(a.Sq, a.Sk, a.D, a.Dv), FML_UNSUPPORTED,
              "fml_attention: needs head sizes that are multiples of 4 up to 128 and K, V of one head within "
              "%zu bytes of shared memory (S_k = %lld, D = %lld, D_v = %lld)", kSmemLimit, (long long)a.Sk,
              (long long)a.D, (long long)a.Dv);
  FML_REQUIRE(a.nb0 * a.nb1 <= 65535, FML_UNSUPPORTED, "fml_attention: more than 65535 heads x batches");
  a.q = (const float *)q->data; a.k = (const float *)kt->data; a.v = (const float *)v->data;
  a.mask = mask ? (const float *)mask->data : nullptr;
  a.out = (float *)out->data;
  a.divisor = divisor;
  if (attention_tc_eligible(a.nb1, a.nb0, a.Sq, a.Sk, a.D, a.Dv, a.q_s, a.k_s, a.v_s, a.q, a.k, a.v))
    return launch_attention_tc(a.nb1, a.nb0, a.Sq, a.Sk, a.D, a.Dv, a.q, a.q_s, a.k, a.k_s, a.v, a.v_s, a.mask, a.m_s,
                               divisor, a.out, a.o_s, as_stream(stream));
  const bool whole = attn_smem_bytes(a.Sk, a.D, a.Dv) <= attn_flash_smem_bytes(a.D, a.Dv) ||
                     attn_flash_smem_bytes(a.D, a.Dv) > kSmemLimit;  // K and V of a head fit at once
  const size_t smem = whole ? attn_smem_bytes(a.Sk, a.D, a.Dv) : attn_flash_smem_bytes(a.D, a.Dv);
  static bool attr_set[64] = {false};
  int dev = 0;
  FML_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    FML_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit));
    FML_CUDA(cudaFuncSetAttribute(attention_flash_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemLimit));
    attr_set[dev] = true;
  }
  const dim3 grid((unsigned)((a.Sq + kRows - 1) / kRows), (unsigned)(a.nb0 * a.nb1));
  if (whole) FML_LAUNCH((attention_kernel), grid, kThreads, smem, as_stream(stream), a);
  else FML_LAUNCH((attention_flash_kernel), grid, kThreads, smem, as_stream(stream), a);
  return FML_OK;
}

// Whether fml_attention would run these operands on the tensor cores (tests and planners).
extern "C" int fml_attention_uses_tensor_cores(const fml_tensor *q, const fml_tensor *kt, const fml_tensor *v, int *uses) {
  FML_REQUIRE(q && kt && v && uses, FML_BAD_ARG, "fml_attention_uses_tensor_cores: null argument");
  AttnArgs a;
  int64_t qs[4], ks[4], vs[4];
  *uses = 0;
  if (q->dtype != FML_F32 || kt->dtype != FML_F32 || v->dtype != FML_F32) return FML_OK;
  if (!as4(q, qs, a.q_s) || !as4(kt, ks, a.k_s) || !as4(v, vs, a.v_s)) return FML_OK;
  *uses = attention_tc_eligible(qs[0], qs[1], qs[2], ks[3], qs[3], vs[3], a.q_s, a.k_s, a.v_s, q->data, kt->data, v->data) ? 1 : 0;
  return FML_OK;
}
