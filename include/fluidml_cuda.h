/*
 * fluidml_cuda.h -- C ABI of the sm_100a kernel library that sits under Kernel::Run.
 *
 * In the reference every operator kernel emits a linalg.generic over strided memrefs that
 * LLVM compiles for the CPU (src/structure/kernel/kernel/<op>.cpp, lowered by
 * src/worker/lower.cpp:37-59).  Each entry point below replaces one family of those
 * emitters with a CUDA launch on device memory.  All tensors are described the way the
 * reference addresses them: a base pointer, a static shape and ELEMENT strides derived
 * from a layout permutation (src/utils/utils.cpp:64-102).
 *
 * Conventions
 *   - every pointer inside an fml_tensor is a DEVICE pointer; fml_tensor structs
 *     themselves live on the host and are read during the call;
 *   - dtype codes are the ONNX TensorProto codes the reference uses
 *     (src/utils/type.cpp:8-23);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream); calls only
 *     enqueue work, they never synchronise, and they may be stream-captured unless a
 *     function says otherwise;
 *   - the return value is an fml_status; nothing is launched when it is not FML_OK.
 *     The reference has no error path (asserts or __builtin_unreachable,
 *     e.g. src/worker/converter.cpp:268-274); bad arguments here are reported, never UB.
 */
#ifndef FLUIDML_CUDA_H_
#define FLUIDML_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FML_MAX_RANK 8

typedef enum fml_status {
  FML_OK = 0,
  FML_BAD_ARG = 1,        /* null pointer, rank/shape mismatch, axis out of range        */
  FML_UNSUPPORTED = 2,    /* dtype or variant no kernel exists for                        */
  FML_MISALIGNED = 3,     /* a fast path was forced on operands that cannot take it       */
  FML_CUDA_ERROR = 4,     /* a CUDA runtime/driver call failed; see fml_last_error()      */
  FML_DEVICE_TIMEOUT = 5, /* a bounded device-side wait gave up (read by fml_check_device)*/
  FML_OUT_OF_MEMORY = 6,
  FML_INDEX_OUT_OF_RANGE = 7 /* a gather index fell outside the table (it was clamped)    */
} fml_status;

typedef enum fml_dtype {
  FML_F32 = 1, FML_I32 = 6, FML_I64 = 7, FML_BOOL = 9
} fml_dtype;

typedef struct fml_tensor {
  void *data;
  int32_t dtype;
  int32_t rank;
  int64_t shape[FML_MAX_RANK];
  int64_t stride[FML_MAX_RANK]; /* in elements; 0 is allowed on inputs (broadcast)        */
} fml_tensor;

/* ---------------------------------------------------------------- runtime plumbing
 * What mlir::ExecutionEngine + malloc gave the reference runner
 * (src/worker/runner.cpp:56-120): device selection, buffers, copies, streams. */
const char *fml_last_error(void);
int fml_device_count(int *count);
int fml_set_device(int device);
int fml_mem_info(size_t *free_bytes, size_t *total_bytes); /* cudaMemGetInfo of the current device */
int fml_malloc(void **ptr, size_t bytes);
int fml_free(void *ptr);
int fml_memset(void *ptr, int value, size_t bytes, void *stream);
int fml_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
int fml_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
int fml_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
int fml_host_alloc_pinned(void **ptr, size_t bytes);
int fml_host_free_pinned(void *ptr);
int fml_stream_create(void **stream);
int fml_stream_destroy(void *stream);
int fml_stream_sync(void *stream);
/* Events and CUDA-graph capture, so a host that links only this library can time and replay
 * a recorded launch list (the reference timed a JIT'd function with std::chrono,
 * src/worker/runner.cpp:101-112). */
int fml_event_create(void **event);
int fml_event_destroy(void *event);
int fml_event_record(void *event, void *stream);
int fml_event_sync(void *event);
int fml_event_elapsed_ms(void *start, void *stop, float *ms);
int fml_graph_begin_capture(void *stream);
int fml_graph_end_capture(void *stream, void **graph_exec); /* instantiates; NULL exec on error */
int fml_graph_abort_capture(void *stream);
int fml_graph_launch(void *graph_exec, void *stream);
int fml_graph_destroy(void *graph_exec);
/* Allocates whatever the library creates lazily on first use (status word, attribute
 * settings) so that later calls can be stream-captured. */
int fml_warmup(void);

/* Timing aid.  With a trace buffer set, the first thread of every kernel of the library stores
 * the device's global nanosecond timer as the kernel's dependency wait returns: `buf` is a device
 * array of `cap` u64 entries, `cursor` a device u32 the caller zeroes (entry index of the next
 * stamp).  Consecutive stamps give each kernel's period inside a stream or a replayed graph.
 * buf == NULL switches the stamps off (the cost is then one predicated load per kernel).
 * Synchronises the device. */
int fml_set_kernel_trace(void *buf, void *cursor, unsigned cap);

/* Reads and clears the device status word kernels write when a bounded wait expires or a
 * gather index is clamped.  Synchronises `stream`.  Returns FML_OK, FML_DEVICE_TIMEOUT or
 * FML_INDEX_OUT_OF_RANGE. */
int fml_check_device(void *stream);
/* Test hook for the failure path: sets the iteration limit of every bounded wait in the
 * tensor-core kernels (0 = default) and, with drop_loads != 0, makes their producers issue no
 * loads, so that a launch's waits run out, the kernel reports the timeout through the status
 * word and returns.  Nothing faults or hangs.  Restore with (0, 0). */
int fml_debug_wait_test(unsigned limit, int drop_loads);

/* ---------------------------------------------------------------- elementwise
 * Binary ops broadcast numpy-style (right-aligned; size-1 dims pinned to index 0), as
 * GetBroadcastAffineMaps does (src/structure/kernel/kernel/utils.cpp:15-51).  A scalar
 * constant operand is a rank-0 tensor or, cheaper, FML_*_SCALAR ops taking it in p0. */
typedef enum fml_ew_op {
  /* binary: out = a (op) b                       reference kernel                        */
  FML_ADD = 0,     /* add.cpp:83-124   AddCommonKernel                                    */
  FML_MUL = 1,     /* mul.cpp:56-99    MulCommonKernel                                    */
  FML_DIV = 2,     /* div.cpp:70-105   DivCommonKernel (true division)                    */
  FML_SUB = 3,     /* sub.cpp:71-99    SubCommonKernel                                    */
  FML_POW = 4,     /* pow.cpp:15-61    PowKernel with a tensor exponent (ONNX)            */
  FML_EQUAL = 5,   /* equal.cpp:14-51  int64 == int64 -> bool                             */
  /* unary with scalar p0 (b == NULL)                                                    */
  FML_ADD_SCALAR = 16,  /* add.cpp:22-79   AddConstantKernel      out = a + p0            */
  FML_MUL_SCALAR = 17,  /* mul.cpp:19-54   MulConstantKernel      out = a * p0            */
  FML_DIV_SCALAR = 18,  /* div.cpp:18-66   DivConstantRhsKernel   out = a / p0            */
  FML_RSUB_SCALAR = 19, /* sub.cpp:16-67   SubConstantLhsKernel   out = p0 - a            */
  FML_POW_SCALAR = 20,  /* pow.cpp:15-61   PowKernel              out = powf(a, p0)       */
  FML_EQUAL_SCALAR = 21,/* equal.cpp:14-51 EqualKernel            out = (a == (int64)p0)  */
  FML_CLIP = 22,        /* clip.cpp:13-48  ClipKernel             out = min(max(a,p0),p1) */
  FML_RSUB_MUL_SCALAR = 23, /* unsqueeze_sub_mul.cpp:19-70        out = (p0 - a) * p1     */
  /* unary, no parameter                                                                 */
  FML_ERF = 32,     /* erf.cpp:18-45                                                      */
  FML_TANH = 33,    /* tanh.cpp:12-40                                                     */
  FML_SQRT = 34,    /* sqrt.cpp:13-36                                                     */
  FML_NEG = 35,     /* neg.cpp:17-40                                                      */
  FML_RELU = 36,    /* relu.cpp:12-46                                                     */
  FML_SIGMOID = 37, /* no reference kernel (parser.cpp:320-326 rejects it): ONNX          */
  FML_NOT = 38,     /* not.cpp:11-41                                                      */
  FML_COPY = 39,    /* dropout.cpp:13-33 (identity); same-dtype strided copy              */
  FML_CAST = 40,    /* cast.cpp:12-62; also int -> f32                                    */
  FML_EXP = 41,
  FML_SILU = 42     /* x * sigmoid(x): Sigmoid followed by Mul, fused                     */
} fml_ew_op;

int fml_elementwise(int op, const fml_tensor *a, const fml_tensor *b, const fml_tensor *out,
                    double p0, double p1, void *stream);

/* AddDivErfAddMulMulKernel (add_div_erf_add_mul_mul.cpp:29-132):
 * t = x + bias ; out = t * (erf(t / c0) + c1) * c2   (bias + exact GELU in one pass). */
int fml_bias_gelu(const fml_tensor *x, const fml_tensor *bias, const fml_tensor *out,
                  float c0, float c1, float c2, void *stream);

/* MulCommonKernel followed by AddCommonKernel (mul.cpp, add.cpp) in one pass: out = a * b + c, all
 * broadcast to out; two roundings, as the two kernels give (no fused multiply-add). */
int fml_mul_add(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c, const fml_tensor *out,
                void *stream);

/* Rotary position embedding over the first `rot` of D features, halves convention (GPT-NeoX):
 * the chain Slice, Slice, Neg (neg.cpp), Concat (concat.cpp), Mul, Mul (mul.cpp), Add (add.cpp),
 * Concat of the exported graph in one pass.  x, out [..., D]; cos, sin [..., rot] broadcast to x's
 * leading dims;  out[:rot] = x[:rot] * cos + rotate_half(x[:rot]) * sin,  out[rot:] = x[rot:],
 * with the chain's roundings (two rounded products, one rounded sum). */
int fml_rotary(const fml_tensor *x, const fml_tensor *cosv, const fml_tensor *sinv, int64_t rot,
               const fml_tensor *out, void *stream);

/* A chain of MulCommonKernel / AddCommonKernel launches (mul.cpp, add.cpp) that sums n products
 * (ConvBERT's span convolution: nine sliding windows times nine softmax columns) in one pass:
 *   acc = a[0] * b[0];  acc = a[i] * b[i] + acc  for i = 1 .. n-1,
 * every product and every sum rounded to fp32 as the separate kernels round them, all operands
 * broadcast to out.  1 <= n <= 12. */
int fml_sum_of_products(int n, const fml_tensor *const *a, const fml_tensor *const *b, const fml_tensor *out,
                        void *stream);

/* The gate of a squeeze-and-excite block: ReduceMeanKernel over the two spatial axes
 * (reduce_mean.cpp:16-98) followed by two 1 x 1 ConvWithoutPaddingKernel launches over the single
 * remaining pixel (conv.cpp:27-280), in one launch:
 *   gate[n, c, 0, 0] = act2(b2[c] + sum_j w2[c, j] * act1(b1[j] + sum_k w1[j, k] * mean(x[n, k, :, :])))
 * x [N, C, H, W] (any strides; dense planes are the fast case), w1 [Cr, C(, 1, 1)], w2 [C, Cr(, 1, 1)],
 * b1 / b2 may be NULL, act1 / act2 from fml_activation (none, relu, tanh, sigmoid, silu).  At most
 * 4096 channels and 512 hidden units (FML_UNSUPPORTED beyond). */
int fml_squeeze_excite_gate(const fml_tensor *x, const fml_tensor *w1, const fml_tensor *b1,
                            const fml_tensor *w2, const fml_tensor *b2, int act1, int act2,
                            const fml_tensor *gate, void *stream);

/* WhereConstantCond{ConstantScalarY,ConstantTensorY}Kernel (where.cpp:30-80, :90-150):
 * out = cond ? x : y, all broadcast to out.  y == NULL takes the scalar y_scalar. */
int fml_where(const fml_tensor *cond, const fml_tensor *x, const fml_tensor *y, float y_scalar,
              const fml_tensor *out, void *stream);

/* ---------------------------------------------------------------- data movement
 * fml_copy_strided: out[i] = in[i] for every logical index i of the common shape.  The
 * host expresses Transpose (transpose.cpp:19-48: a permuted-stride view of the input),
 * Slice (slice.cpp:17-55: an offset view), Concat2 (concat.cpp:18-68: two calls into
 * offset views of the output) and the interior of Pad (pad.cpp:15-51) through it.
 * Bit-exact for every dtype. */
int fml_copy_strided(const fml_tensor *in, const fml_tensor *out, void *stream);
/* Concat2Kernel (concat.cpp): out = lhs followed by rhs along `axis`, both halves in one launch. */
int fml_concat2(const fml_tensor *lhs, const fml_tensor *rhs, const fml_tensor *out, int axis, void *stream);

/* ReshapeKernel / UnsqueezeKernel / SqueezeKernel / FlattenKernel (reshape.cpp:18-64,
 * unsqueeze.cpp:20-63, squeeze.cpp:17-54, flatten.cpp:15-63): the e-th element in logical
 * row-major order of `in` becomes the e-th element of `out`, whatever the two layouts. */
int fml_reshape_copy(const fml_tensor *in, const fml_tensor *out, void *stream);

/* Gather (gather.cpp:100-139, :149-186, :195-272): out[pre.., i.., post..] =
 * data[pre.., indices[i..], post..], int64 indices (device memory).  Indices outside
 * [0, data.shape[axis]) are clamped and recorded in the device status word. */
int fml_gather(const fml_tensor *data, const fml_tensor *indices, const fml_tensor *out,
               int axis, void *stream);

/* GatherConstantDataTensorAddTensorLhsAddTensorLhsKernel (gather_add_add.cpp:25-163):
 * out = table[ids] + add0 + add1 (word + position + token-type embeddings), add0/add1
 * broadcast to out; either may be NULL. */
int fml_embedding(const fml_tensor *table, const fml_tensor *ids, const fml_tensor *add0,
                  const fml_tensor *add1, const fml_tensor *out, void *stream);

/* PadKernel (pad.cpp:15-51), constant mode with value 0 (the reference leaves the border
 * untouched and relies on a zeroed arena). */
int fml_pad(const fml_tensor *in, const fml_tensor *out, const int64_t *pads_begin, void *stream);

/* ---------------------------------------------------------------- reductions
 * SoftmaxKernel (softmax.cpp:22-139) in one pass.  With `mask` != NULL and/or
 * divisor != 1 it computes softmax(in / divisor + mask) (mask broadcast to in): the
 * Div + Add + Softmax chain of attention fused.  No scratch (the reference needs one
 * float per row, src/structure/flow/node.cpp:1355-1368). */
int fml_softmax(const fml_tensor *in, const fml_tensor *mask, float divisor,
                const fml_tensor *out, int axis, void *stream);

/* The attention core in one launch: out = softmax(Q K^T / divisor + mask) V, replacing the
 * reference's MatMulKernel -> (Div, Add) -> SoftmaxKernel -> MatMulKernel sequence
 * (matmul.cpp:5-44, softmax.cpp:22-139).  q [.., S_q, D], kt [.., D, S_k] (the transposed
 * keys, as the MatMul receives them), v [.., S_k, D_v], out [.., S_q, D_v], ranks 2 to 4 with
 * equal leading dims; mask (may be NULL) broadcasts to [.., S_q, S_k].  Any strides: the
 * head-split transposes can stay views.  fp32 FMA throughout; the scores never leave the SM.
 * K and V of a head are staged once when they fit in shared memory; longer key sequences stream
 * through it in chunks of 128 keys with a running-maximum softmax.  fml_attention_supported
 * tells whether a shape is taken (head sizes multiples of 4 up to 128); fml_attention returns
 * FML_UNSUPPORTED otherwise. */
int fml_attention_supported(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v);
/* 1 when blocks of these head sizes run on the tensor cores (tcgen05, scores in tensor memory,
 * 3xTF32) once they are large enough (about 200 Mflop) and their operands are 16-byte aligned
 * views with unit innermost stride; smaller or unaligned blocks take the CUDA-core kernel. */
int fml_attention_on_tensor_cores(int64_t s_q, int64_t s_k, int64_t d, int64_t d_v);
/* The same question for concrete operands (shapes, strides, alignment, size). */
int fml_attention_uses_tensor_cores(const fml_tensor *q, const fml_tensor *kt, const fml_tensor *v, int *uses);
int fml_attention(const fml_tensor *q, const fml_tensor *kt, const fml_tensor *v,
                  const fml_tensor *mask, float divisor, const fml_tensor *out, void *stream);

/* LayerNormalizationConstantScaleBiasKernel (layer_normalization.cpp:33-220) in one pass:
 * mean, biased variance about the mean, y = (x-mean) * (1/sqrtf(var+eps)) * scale + bias.
 * With `residual` != NULL the input is in + residual (Add + LayerNorm fused).  No scratch
 * (the reference needs one float per row, node.cpp:972-985). */
int fml_layernorm(const fml_tensor *in, const fml_tensor *residual, const fml_tensor *scale,
                  const fml_tensor *bias, const fml_tensor *out, int axis, float eps,
                  void *stream);

/* ReduceMeanKernel (reduce_mean.cpp:16-98), keepdims = 1; `reduce[i]` != 0 marks a reduced
 * axis. */
int fml_reduce_mean(const fml_tensor *in, const fml_tensor *out, const int32_t *reduce,
                    void *stream);

/* CumSumKernel (cum_sum.cpp:53-87): int64, forward, inclusive. */
int fml_cumsum(const fml_tensor *in, const fml_tensor *out, int axis, void *stream);

/* ---------------------------------------------------------------- GEMM
 * MatMulKernel (matmul.cpp:28-59 with the broadcast maps of utils.cpp:62-146) and
 * GemmConstantBiasKernel (gemm.cpp:39-182).  C[.., m, n] = sum_k A[.., m, k] * B[.., k, n]
 * over the last two dims, leading dims broadcast.  transA/transB of Gemm are expressed by
 * the caller through strides.  The epilogue is applied to the fp32 accumulator in this
 * order:   v = acc / divisor ; v = alpha * v + beta * bias ; v = act(v) ; v += residual.
 * `bias` and `residual` broadcast to C.
 */
typedef enum fml_gemm_act {
  FML_ACT_NONE = 0,
  FML_ACT_GELU_ERF = 1, /* v * (erf(v / c0) + c1) * c2, constants in act_param[3]         */
  FML_ACT_RELU = 2,
  FML_ACT_TANH = 3,
  FML_ACT_SIGMOID = 4,
  FML_ACT_SILU = 5 /* x * sigmoid(x) */
} fml_gemm_act;

typedef enum fml_gemm_precision {
  FML_GEMM_AUTO = 0,   /* 3xTF32 tensor-core path when operands allow it, else fp32 FMA   */
  FML_GEMM_FP32 = 1,   /* CUDA-core fp32 FMA, any strides                                 */
  FML_GEMM_3XTF32 = 2, /* tcgen05, hi/lo split: error ~2^-21 relative per product         */
  FML_GEMM_TF32 = 3    /* tcgen05, single pass: error ~2^-11 relative per product         */
} fml_gemm_precision;

typedef struct fml_gemm_params {
  int32_t precision;   /* fml_gemm_precision                                              */
  int32_t act;         /* fml_gemm_act                                                    */
  float divisor;       /* 1 = none                                                        */
  float alpha, beta;   /* Gemm attributes; MatMul uses 1, 1                               */
  float act_param[3];
  int32_t split_k;     /* 0 = let the library choose; at most 8 (one cluster per tile)    */
  int32_t tile_n;      /* 0 = let the library choose; a multiple of 16 up to 256          */
  int32_t b_constant;  /* non-zero: B holds weights that no earlier launch on the stream
                        * writes, so the kernel may load its first B tiles while the
                        * preceding kernel is still finishing                              */
  /* Optional hint: constant device bytes (16-byte aligned) that a LATER launch on this stream
   * will stream, typically the next layer's weights.  The tensor-core kernel asks L2 to fetch
   * them while it runs, so the later launch finds them on chip instead of waiting on HBM,
   * which is otherwise idle between the kernels of a batch-1 pass.  NULL / 0 = none.  The
   * bytes must stay valid and unchanged; they are only read. */
  const void *l2_prefetch;
  uint64_t l2_prefetch_bytes;
} fml_gemm_params;

void fml_gemm_default_params(fml_gemm_params *p);

/* Split-K partial sums never leave the chip (they are reduced across a thread-block cluster
 * through distributed shared memory), so the call needs no scratch buffer. */
int fml_gemm(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
             const fml_tensor *bias, const fml_tensor *residual, const fml_gemm_params *p,
             void *stream);

/* What the library chose for these operands (the counterpart of the loop-order autotuning in
 * the reference's MatMul / Gemm generators, src/structure/kernel/generator/matmul.cpp:88-131):
 * uses_tensor_cores 0 = fp32 FMA kernel, 1 = tcgen05; tile_n, split_k and stages are 0 for the
 * FMA kernel.  Pure host computation. */
typedef struct fml_gemm_plan_info {
  int32_t uses_tensor_cores, tile_n, split_k, stages, b_mn_major, three_pass;
  uint64_t shared_memory_bytes;
} fml_gemm_plan_info;
int fml_gemm_plan(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                  const fml_gemm_params *p, fml_gemm_plan_info *info);

/* On-device choice of tile_n and split_k for these operands: runs the candidate
 * configurations a few times each on `stream` (overwriting C with valid results), keeps the
 * fastest and remembers it per problem signature.  Synchronises; must not be stream-captured.
 * `tuned` receives a copy of `p` with tile_n / split_k filled in (unchanged when the fp32 FMA
 * kernel is used or the caller already fixed them).  The counterpart of the reference's
 * loop-order autotuning (src/structure/kernel/generator/matmul.cpp:88-131, gemm.cpp:107-151). */
int fml_gemm_autotune(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                      const fml_tensor *bias, const fml_tensor *residual, const fml_gemm_params *p,
                      void *stream, fml_gemm_params *tuned);

/* fml_gemm for products with 1 <= M <= 32 rows, for callers that cannot let the library
 * allocate device memory (no counterpart in the reference, which has no device side).  Same
 * arguments and results as fml_gemm with precision FP32 (AUTO is accepted and means FP32).
 * The split-K scratch is an array inside the loaded module: 1 MiB per device, of which
 * 960 KiB hold partial sums; a product that needs more (roughly splits * M * N * 4 bytes with
 * N rounded up to 32) fails with FML_OUT_OF_MEMORY and a message -- use fml_gemm then.  No
 * allocating CUDA routine is called.  The first call on each device looks up the array's
 * device address and clears its counters; make that call outside any stream capture.  Calls
 * on one device share the array: calls whose kernels may overlap (different streams without
 * ordering, several threads) race on it and must be serialised by the caller. */
int fml_gemm_skinny_noalloc(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                            const fml_tensor *bias, const fml_tensor *residual,
                            const fml_gemm_params *p, void *stream);

/* Reports which path fml_gemm would take for these operands: 0 = fp32 FMA, 1 = tcgen05. */
int fml_gemm_uses_tensor_cores(const fml_tensor *a, const fml_tensor *b, const fml_tensor *c,
                               const fml_gemm_params *p, int *uses);

/* ---------------------------------------------------------------- convolution, pooling
 * ConvWithoutPaddingKernel / ConvWithPaddingKernel (conv.cpp:27-280): NCHW x OIHW, 1-D or
 * 2-D, group == 1 or depthwise (group == C, multiplier 1) as in the reference (:103-149).
 * ONNX semantics for strides, dilations, zero padding and per-channel bias (the reference
 * ignores strides/dilations, :68-76, and adds bias[1] everywhere, :181-184).  Padding is
 * implicit: no padded copy, so the node needs no scratch (reference: node.cpp:500-519). */
typedef struct fml_conv_params {
  int64_t pads_begin[2], strides[2], dilations[2];
  int64_t group;
  int32_t act;       /* fml_gemm_act applied after bias (Relu fusion)                     */
  int32_t precision; /* fml_gemm_precision for the group == 1 implicit-GEMM path          */
} fml_conv_params;

int fml_conv(const fml_tensor *x, const fml_tensor *w, const fml_tensor *bias,
             const fml_tensor *y, const fml_conv_params *p, void *stream);

/* MulCommonKernel (mul.cpp) followed by a group-1 convolution (conv.cpp:27-280) without the
 * product ever reaching memory: y = conv(x * x_scale, w) + bias, x_scale broadcastable to
 * [N, IC, 1, 1] (the gate of a squeeze-and-excite block).  The product is rounded to fp32 before
 * it enters the convolution, as the separate kernel's output would be.  Same paths as fml_conv:
 * the tensor-core kernel when it is eligible, else the general implicit GEMM. */
int fml_conv_scaled(const fml_tensor *x, const fml_tensor *x_scale, const fml_tensor *w,
                    const fml_tensor *bias, const fml_tensor *y, const fml_conv_params *p, void *stream);

/* Reports which path fml_conv takes: 1 = the tcgen05 implicit GEMM (2-D, group 1, unit stride
 * and dilation, dense NCHW input whose row length is a multiple of 4, weights stored
 * [KH][KW][IC][OC] -- the OIHW tensor with layout permutation (3, 2, 0, 1) -- with OC a
 * multiple of 4, precision not FP32), 0 = the CUDA-core kernels. */
int fml_conv_uses_tensor_cores(const fml_tensor *x, const fml_tensor *w, const fml_tensor *y,
                               const fml_conv_params *p, int *uses);

/* MaxPoolWithoutPaddingKernel / AveragePoolWithoutPaddingKernel (maxpool.cpp:17-82,
 * averagepool.cpp:19-87): 2-D windows, no padding.  mode 0 = max, 1 = average. */
int fml_pool2d(const fml_tensor *x, const fml_tensor *y, int mode, const int64_t *kernel,
               const int64_t *strides, void *stream);

/* ---------------------------------------------------------------- resident stage program
 * The reference runs a whole model as ONE call into one compiled function
 * (src/worker/runner.cpp:101-112 invokes the single func that GeneralBuilder assembled,
 * src/worker/builder.cpp:400-491).  A resident program is the counterpart here for a chain of
 * operators over one block of 128 activation rows (batch x sequence = 128): every stage of the
 * chain runs inside ONE persistent kernel, one CTA per SM, so no kernel boundary separates
 * dependent operators.  The weights of all stages are packed once, at creation, into one
 * stream per CTA which a producer warp copies into a shared-memory ring without ever waiting
 * for activations.  Stages exchange data through buffers the program owns; every word stored
 * there carries a one-bit generation tag in the least significant bit of its mantissa, so a
 * consumer validates what it fetched instead of polling a flag, and a producer never fences
 * (values inside the program are therefore truncated to 23 mantissa bits).
 *
 * Stage kinds
 *   FML_RESIDENT_GEMM       out = [LayerNorm]( act(A W + bias) + residual ): MatMulKernel /
 *                           GemmConstantBiasKernel (matmul.cpp:28-59, gemm.cpp:39-182) with the
 *                           epilogue of fml_gemm, optionally followed by
 *                           LayerNormalizationConstantScaleBiasKernel
 *                           (layer_normalization.cpp:33-220) over the output row.  W is constant.
 *                           3xTF32 on tcgen05, split-K partial sums added in split order.
 *   FML_RESIDENT_ATTENTION  out = softmax(Q K^T / divisor + mask) V per head, as fml_attention.
 * Tensors are described as the launcher of the separate kernels would describe them (device
 * pointers, shapes, element strides).  An input that lies inside the `out` bytes of an earlier
 * stage is taken from that stage; such outputs live in the program's own buffers and `out` is
 * only their name, unless the stage sets `out_external`, which also stores them at `out` with the
 * strides given so that code outside the program can read them.  Inputs that no stage produces
 * are read as described and must be complete before the launch.
 * fml_resident_create returns FML_UNSUPPORTED (and creates nothing) when a stage does not fit:
 * the caller then launches the operators one by one.
 */
typedef enum fml_resident_kind { FML_RESIDENT_GEMM = 1, FML_RESIDENT_ATTENTION = 2 } fml_resident_kind;

typedef struct fml_resident_stage {
  int32_t kind;
  int32_t out_external;   /* non-zero: `out` is also read outside the program               */
  fml_tensor out;         /* GEMM [.., 128, N]; attention [.., H, 128, Dv]                   */
  /* GEMM */
  fml_tensor a;           /* [.., 128, K]                                                    */
  fml_tensor w;           /* [K, N] constant, any strides                                    */
  fml_tensor bias;        /* [N], data == NULL: none                                         */
  fml_tensor residual;    /* [.., 128, N], data == NULL: none                                */
  int32_t act;            /* fml_gemm_act: NONE, GELU_ERF, RELU, TANH, SIGMOID               */
  float act_param[3];
  int32_t layernorm;      /* non-zero: LayerNorm over N with ln_scale, ln_bias [N], ln_eps   */
  fml_tensor ln_scale, ln_bias;
  float ln_eps;
  int32_t tile_n, split_k; /* 0 = let the library choose                                     */
  /* attention */
  fml_tensor q, kt, v;    /* [.., H, 128, D], [.., H, D, 128], [.., H, 128, Dv]              */
  fml_tensor mask;        /* broadcasts to [.., H, 128, 128]; data == NULL: none             */
  float divisor;
} fml_resident_stage;

typedef struct fml_resident fml_resident;

typedef struct fml_resident_info {
  int32_t ctas, stages, steps, buffers;
  int32_t ring_slots, slot_bytes;
  uint64_t packed_weight_bytes, scratch_bytes, shared_memory_bytes;
} fml_resident_info;

/* Pure host computation: plans the program for `ctas` resident CTAs (0 = the SM count of the
 * current device), checks that every read is covered by writes of its generation and that a
 * buffer is only overwritten once the data dependences alone guarantee that all readers of its
 * previous content are done, and reports the plan.  Needs no device when `ctas` is given. */
int fml_resident_plan(const fml_resident_stage *stages, int32_t count, int32_t ctas,
                      fml_resident_info *info);
/* Plans, packs the weights (a device kernel on the default stream; synchronises) and allocates
 * the program's buffers.  Not capturable. */
int fml_resident_create(const fml_resident_stage *stages, int32_t count, fml_resident **out);
/* One pass: launches the persistent kernel (cooperatively, so that all CTAs are co-resident) and
 * a one-thread kernel that advances the pass number.  Capturable.  Passes of one program must
 * not overlap.  A bounded wait that expires sets the device status word (fml_check_device) and
 * ends the pass early on every CTA; call fml_resident_reset before the next pass then. */
int fml_resident_launch(fml_resident *program, void *stream);
/* Restores the initial state of the program's buffers and pass number (after a timeout). */
int fml_resident_reset(fml_resident *program, void *stream);
int fml_resident_info_of(const fml_resident *program, fml_resident_info *info);
int fml_resident_destroy(fml_resident *program);
/* Timing aid.  After fml_resident_set_trace(program, 1), fml_resident_launch runs a kernel
 * variant that records nanosecond stamps of the device's global timer per step: slot 0 start,
 * 1 end; GEMM units also 2 = A rows fetched, 3 = last k block converted, 4 = accumulator
 * complete; attention steps 2 = operands staged, 3 = scores, 4 = softmax done.
 * fml_resident_read_trace copies them to `host` as [cta][step][8] u64 (`capacity` counts u64
 * entries) and reports the two leading extents. */
int fml_resident_set_trace(fml_resident *program, int32_t on);
int fml_resident_read_trace(fml_resident *program, uint64_t *host, uint64_t capacity,
                            int32_t *ctas, int32_t *max_steps);

#ifdef __cplusplus
}
#endif
#endif /* FLUIDML_CUDA_H_ */
