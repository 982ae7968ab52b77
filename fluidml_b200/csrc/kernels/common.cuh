// Shared host/device helpers of the kernel library: status handling, operand checking,
// dimension collapsing and the device status word.
#pragma once
#include "fluidml_cuda.h"
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <utility>

namespace fml {

constexpr int kMaxDims = FML_MAX_RANK;

void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);
#define FML_CUDA(call)                                                                     \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) return ::fml::cuda_fail(e__, #call);                           \
  } while (0)
#define FML_REQUIRE(cond, status, ...)                                                     \
  do {                                                                                     \
    if (!(cond)) {                                                                         \
      ::fml::set_error(__VA_ARGS__);                                                       \
      return status;                                                                       \
    }                                                                                      \
  } while (0)

// Bits of the device status word (one int per device, written by kernels with atomicOr).
constexpr int kStatusTimeout = 1;
constexpr int kStatusIndexRange = 2;
int *device_status_word();  // device pointer for the current device (allocated on first use)

inline size_t dtype_size(int dtype) {
  switch (dtype) {
  case FML_F32: case FML_I32: return 4;
  case FML_I64: return 8;
  case FML_BOOL: return 1;
  default: return 0;
  }
}

inline int64_t numel(const fml_tensor *t) {
  int64_t n = 1;
  for (int i = 0; i < t->rank; ++i) n *= t->shape[i];
  return n;
}

inline bool valid_tensor(const fml_tensor *t) {
  if (!t || t->rank < 0 || t->rank > kMaxDims || dtype_size(t->dtype) == 0) return false;
  for (int i = 0; i < t->rank; ++i)
    if (t->shape[i] < 0) return false;
  return numel(t) == 0 || t->data != nullptr;
}

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// An iteration space over the output's logical shape with one stride vector per operand
// (operand 0 is the output).  After collapse(): size-1 dims removed, adjacent dims merged
// when every operand walks them contiguously, so most tensors become 1-3 dims.
template <int NOPS> struct Iter {
  int rank;
  int64_t shape[kMaxDims];
  int64_t stride[NOPS][kMaxDims];
  int64_t total;
};

// Strides of `t` expanded to the output's rank by numpy broadcasting (right-aligned,
// size-1 dims -> stride 0).  Returns false when the shapes do not broadcast.
inline bool broadcast_strides(const fml_tensor *t, const fml_tensor *out, int64_t *s) {
  if (t->rank > out->rank) return false;
  for (int i = 0; i < out->rank; ++i) {
    int ti = i - (out->rank - t->rank);
    if (ti < 0) { s[i] = 0; continue; }
    if (t->shape[ti] == out->shape[i]) s[i] = t->shape[ti] == 1 ? 0 : t->stride[ti];
    else if (t->shape[ti] == 1) s[i] = 0;
    else return false;
  }
  return true;
}

template <int NOPS> inline void collapse(Iter<NOPS> &it) {
  int r = 0;
  int64_t shape[kMaxDims], stride[NOPS][kMaxDims];
  for (int i = 0; i < it.rank; ++i) {
    if (it.shape[i] == 1) continue;
    bool merge = r > 0;
    if (merge)
      for (int o = 0; o < NOPS; ++o)
        if (stride[o][r - 1] != it.stride[o][i] * it.shape[i]) { merge = false; break; }
    if (merge) {
      shape[r - 1] *= it.shape[i];
      for (int o = 0; o < NOPS; ++o) stride[o][r - 1] = it.stride[o][i];
    } else {
      shape[r] = it.shape[i];
      for (int o = 0; o < NOPS; ++o) stride[o][r] = it.stride[o][i];
      ++r;
    }
  }
  if (r == 0) {
    shape[0] = 1;
    for (int o = 0; o < NOPS; ++o) stride[o][0] = 0;
    r = 1;
  }
  it.rank = r;
  it.total = 1;
  for (int i = 0; i < r; ++i) {
    it.shape[i] = shape[i];
    it.total *= shape[i];
    for (int o = 0; o < NOPS; ++o) it.stride[o][i] = stride[o][i];
  }
}

template <int NOPS>
__device__ __forceinline__ void offsets_of(const Iter<NOPS> &it, int64_t lin, int64_t *off) {
#pragma unroll
  for (int o = 0; o < NOPS; ++o) off[o] = 0;
  for (int d = it.rank - 1; d >= 0; --d) {
    int64_t q = lin / it.shape[d], c = lin - q * it.shape[d];
    lin = q;
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] += c * it.stride[o][d];
  }
}

// Programmatic dependent launch: every kernel of the library is launched with the
// "programmatic stream serialization" attribute and starts with pdl_prologue(), so inside a
// stream (or a captured graph) kernel N+1 may be scheduled, and run its own set-up, while
// kernel N drains; griddepcontrol.wait returns once kernel N has completed and its writes are
// visible, and no kernel reads or writes global data before it.  What a kernel may do before
// the wait: load operands the caller declared constant (the tensor-core GEMM's weights) and
// issue L2 prefetches (they move nothing into the SM, so they are safe whoever produces the
// bytes).  FLUIDML_PDL=0 turns the attribute off (the device instructions are then no-ops).
bool pdl_enabled();

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Kernel-start stamps, switched on at run time (fml_set_kernel_trace): when a trace buffer is set,
// the first thread of every kernel of the library writes %globaltimer as its dependency wait
// returns, so consecutive stamps give each kernel's period inside a stream or a replayed graph
// (its run time plus the gap to the next start) without event pairs between the launches.  With
// no buffer set the cost is one predicated load in one thread per kernel.  Each translation unit
// has its own copy of the pointers; fml_set_kernel_trace sets them all.
static __device__ unsigned long long *g_trace_buf;
static __device__ unsigned *g_trace_cursor;
static __device__ unsigned g_trace_cap;
void register_trace_setter(cudaError_t (*setter)(unsigned long long *, unsigned *, unsigned));
static cudaError_t set_trace_this_unit(unsigned long long *buf, unsigned *cursor, unsigned cap) {
  cudaError_t e = cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof(buf));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_cursor, &cursor, sizeof(cursor));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_trace_cap, &cap, sizeof(cap));
  return e;
}
static struct TraceRegistrar { TraceRegistrar() { register_trace_setter(&set_trace_this_unit); } } g_trace_registrar;
__device__ __forceinline__ void trace_stamp() {
  if ((threadIdx.x | threadIdx.y | threadIdx.z | blockIdx.x | blockIdx.y | blockIdx.z) == 0 && g_trace_buf) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    const unsigned i = atomicAdd(g_trace_cursor, 1u);
    if (i < g_trace_cap) g_trace_buf[i] = t;
  }
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  trace_stamp();
}
// For the stretch between launch_dependents and the wait: asks L2 for the first `bytes` (at
// most `cap`) of a weight tensor, one 128-byte line per thread of the grid's first row of
// blocks.  Weights are cold in a pass that streams more bytes than L2 holds; a prefetch moves
// nothing into the SM, so it is safe whoever produces the bytes.
__device__ __forceinline__ void l2_prefetch_span(const void *p, int64_t bytes, int64_t cap = 1 << 20) {
  if (!p || blockIdx.y != 0 || blockIdx.z != 0) return;
  if (bytes > cap) bytes = cap;
  const char *c = static_cast<const char *>(p);
  for (int64_t off = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 128; off < bytes;
       off += (int64_t)gridDim.x * blockDim.x * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}
__device__ __forceinline__ void pdl_prologue() {
  pdl_launch_dependents();
  pdl_wait();
}

template <typename... Exp, typename... Act>
inline cudaError_t launch_kernel(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Act &&...args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Act>(args)...);
}
#define FML_LAUNCH(kernel, grid, block, smem, stream, ...)                                 \
  FML_CUDA(::fml::launch_kernel(kernel, grid, block, smem, stream, __VA_ARGS__))

inline int grid_for(int64_t work, int block, int max_blocks = 148 * 16) {
  int64_t g = (work + block - 1) / block;
  if (g < 1) g = 1;
  if (g > max_blocks) g = max_blocks;
  return static_cast<int>(g);
}

// x / d.  When d is a power of two whose reciprocal is a normal number, 1 / d is exact and x * (1 / d)
// is the same correctly rounded value as x / d, bit for bit: the attention scale 1 / sqrt(64) = 1 / 8
// costs one multiply instead of a ~10-instruction IEEE division per score.
struct ExactDivisor {
  float d, inv;
  bool by_mul;
  __host__ __device__ explicit ExactDivisor(float divisor) : d(divisor), inv(1.0f / divisor) {
    uint32_t u;
    memcpy(&u, &divisor, sizeof(u));
    const uint32_t e = (u >> 23) & 0xffu;
    by_mul = (u & 0x007fffffu) == 0 && e >= 2 && e <= 252;
  }
  __device__ __forceinline__ float operator()(float x) const { return by_mul ? x * inv : x / d; }
};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace fml
