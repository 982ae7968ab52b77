// Data model shared by the planner (host) and the persistent kernel (device) of a resident
// stage program: the per-CTA step lists, the stage descriptors and the tiled activation order.
//
// Tiled order ("row-interleaved quads"): a [128 x N] fp32 matrix is stored as N/4 column quads,
// each a run of 128 float4 (one per row): element (r, c) lives at float index
// ((c >> 2) * 128 + r) * 4 + (c & 3).  A thread that owns row r (= a TMEM lane) reads or writes
// one float4 per quad, and the 32 lanes of a warp touch 512 consecutive bytes: GEMM operands,
// split-K partial tiles and finished outputs all move as full cache lines without a shared-
// memory transpose.  The matrix occupies exactly the bytes of its row-major form.
#pragma once
#include <cstdint>

namespace fml {
namespace res {

constexpr int kRows = 128;       // activation rows = TMEM lanes = batch x sequence
constexpr int kThreads = 320;    // warp 0 weight producer, warp 1 MMA issuer, warps 2-5 converters
                                 // (one TMEM lane each), warps 6-9 helpers of the SIMT steps
constexpr int kWorkers = 256;    // warps 2-9
constexpr int kMaxWait = 4;
constexpr int kBK = 32;          // k block: 32 floats = one 128-byte swizzle span
constexpr int kMaxTileN = 192;
constexpr int kConvDepth = 3;    // k blocks in flight between the converters and the MMA issuer
constexpr int kAttnRows = 16;    // query rows per attention step
constexpr int kTraceSlots = 2;

enum StepKind : int32_t { kEnd = 0, kUnit = 1, kFinish = 2, kAttention = 3 };

// One entry of a CTA's work list.  The meaning of p0..p3 depends on the kind:
//   kUnit       p0 = column slab, p1 = k split, p2 = first k block, p3 = k blocks: accumulates
//               A[:, k range] x W[k range, slab] in TMEM and stores the partial tile;
//   kFinish     p0..p1 = rows, p2..p3 = column quads: adds the split-K partials in split order,
//               applies bias / activation / residual / LayerNorm and stores the result;
//   kAttention  p0 = head, p1 = first query row.
// Before a step runs, counter wait_ctr[i] must have reached wait_target[i]; afterwards the step
// adds one to counters sig[0] and sig[1] (negative: none).
struct Step {
  int32_t kind, stage;
  int32_t p0, p1, p2, p3;
  int32_t nwait;
  int32_t wait_ctr[kMaxWait];
  uint32_t wait_target[kMaxWait];
  int32_t sig[2];
  int32_t pad[3];
};
static_assert(sizeof(Step) == 80, "Step is read as five 16-byte words");

struct GemmStage {
  const float *a;        // activations: tiled (a_tiled) or row-major with row stride a_ld
  long long a_ld;
  float *partial;        // [S][N / 4][128] float4: split-K partial tiles, tiled order per split
  const float *bias;
  const float *res;      // residual, tiled or row-major
  long long res_ld;
  const float *gamma, *beta;
  float *out_tiled;      // may be null
  float *out_rm;         // row-major copy for readers outside the program; may be null
  long long out_ld;
  int32_t N, K, S, tile_n;
  int32_t a_tiled, res_tiled, act, ln;
  float c0, c1, c2, eps;
};

struct AttnStage {
  const float *q, *k, *v;  // tiled matrices with 128 rows
  const float *mask;       // may be null
  float *out_tiled, *out_rm;
  long long out_ld;
  long long m_sh, m_sr, m_sk;  // mask element strides per head, query row and key (0 = broadcast)
  int32_t q_col, k_col, v_col, o_col;  // first column of head 0 inside its matrix
  int32_t q_hs, k_hs, v_hs, o_hs;      // column step from one head to the next
  int32_t heads, D, Dv, Sk;
  float divisor;
  int32_t pad;
};

}  // namespace res
}  // namespace fml
