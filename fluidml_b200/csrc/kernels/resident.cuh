// Data model shared by the planner (host) and the persistent kernel (device) of a resident
// stage program: the per-CTA step lists, the stage descriptors, the tiled activation order and
// the generation tags that order the steps.
//
// Tiled order ("row-interleaved quads"): a [128 x N] fp32 matrix is stored as N/4 column quads,
// each a run of 128 float4 (one per row): element (r, c) lives at float index
// ((c >> 2) * 128 + r) * 4 + (c & 3).  A thread that owns row r (= a TMEM lane) reads or writes
// one float4 per quad, and the 32 lanes of a warp touch 512 consecutive bytes: GEMM operands,
// split-K partial tiles and finished outputs all move as full cache lines without a shared-
// memory transpose.
//
// Generation tags.  A dependent step two kernels apart costs a launch; inside one kernel the
// usual flag protocol (store, fence, flag, poll, load) still costs three to four L2 round trips
// of about a microsecond each on this part, more than the arithmetic of a step.  Here the data
// validates itself instead: every fp32 word a step stores into one of the program's private
// buffers carries the parity of the buffer's write generation in the least significant bit of
// its mantissa.  Buffers are written once per generation, a reader knows which generation it
// wants, fetches the words it needs (cp.async into shared memory, all of them in flight) and
// repeats the fetch for those whose bit is still the old parity.  No fence, no flag, no poll of a
// separate location: one round trip after the data has landed.  Only 4-byte stores need to be
// atomic.  Readers clear the bit, so values are truncated to 23 mantissa bits (relative error
// <= 2^-23) and do not depend on the parity.  The parity of generation g of a buffer that is
// written u times per pass in pass e is (e * u + g) & 1; e is a device word bumped before each
// pass.  Buffers start out filled with words whose bit is 1, the opposite of generation 0 in
// pass 0, and a buffer is reused for another tensor only where the planner has proved, from the
// data dependences alone, that every reader of the previous generation is done.
#pragma once
#include <cstdint>

namespace fml {
namespace res {

constexpr int kRows = 128;       // activation rows = TMEM lanes = batch x sequence
constexpr int kThreads = 320;    // warp 0 weight producer, warp 1 MMA issuer, warps 2-9 workers
constexpr int kWorkers = 256;    // warps 2-9: two converter sets (one TMEM lane per thread each) and the SIMT steps
constexpr int kBK = 32;          // k block: 32 floats = one 128-byte swizzle span
constexpr int kMaxTileN = 192;
constexpr int kConvDepth = 3;    // k blocks in flight between the converters and the MMA issuer
constexpr int kAStages = 4;      // k blocks of the A operand staged in shared memory at once
constexpr int kAPitch = 36;      // floats per staged A row (32 + 4: conflict-free 16-byte row reads)
constexpr int kAttnRows = 16;    // query rows per attention step
constexpr int kTraceSlots = 8;   // time stamps per step in the traced kernel variant
constexpr uint32_t kFillWord = 1u;  // initial content of every tagged buffer

enum StepKind : int32_t { kEnd = 0, kUnit = 1, kFinish = 2, kAttention = 3 };

// One entry of a CTA's work list.  The meaning of p0..p3 depends on the kind:
//   kUnit       p0 = column slab, p1 = k split, p2 = first k block, p3 = k blocks: accumulates
//               A[:, k range] x W[k range, slab] in TMEM and stores the partial tile;
//   kFinish     p0..p1 = rows, p2..p3 = column quads: adds the split-K partials in split order,
//               applies bias / activation / residual / LayerNorm and stores the result;
//   kAttention  p0 = head, p1 = first query row.
struct Step {
  int32_t kind, stage;
  int32_t p0, p1, p2, p3;
  int32_t pad[2];
};
static_assert(sizeof(Step) == 32, "Step is read as two 16-byte words");

// A tag selector encodes how a buffer generation's parity follows from the pass number e:
// parity = (sel & 1) ^ ((sel >> 1) & e & 1).  Negative: the operand is not tagged (it comes from
// outside the program, or is a constant).
__host__ __device__ inline uint32_t tag_parity(int32_t sel, uint32_t epoch) {
  return ((uint32_t)sel & 1u) ^ (((uint32_t)sel >> 1) & epoch & 1u);
}

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
  int32_t a_tag, res_tag, part_tag, out_tag;  // tag selectors (see tag_parity)
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
  int32_t q_tag, k_tag, v_tag, out_tag;
  float divisor;
  int32_t pad;
};

}  // namespace res
}  // namespace fml
