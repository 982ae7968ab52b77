/*
 * fluidml_executor.h -- C ABI over fluidml::worker::Executor for bindings that cannot
 * consume C++ (ctypes, cgo, JNI).  It is what the reference's pybind11 module binds
 * (src/python/pybind.cpp:66-87: Executor.make_plain_linear / make_plain_greedy /
 * make_dp_greedy, compile, invoke), expressed with plain pointers and sizes.
 * Every function returns 0 on success; on failure the message is available from
 * fml_executor_last_error() (per handle) and nothing has been left half-done.
 */
#ifndef FLUIDML_EXECUTOR_H_
#define FLUIDML_EXECUTOR_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fml_executor fml_executor;

enum { FML_EXECUTOR_PLAIN_LINEAR = 0, FML_EXECUTOR_PLAIN_GREEDY = 1, FML_EXECUTOR_DP_GREEDY = 2 };

/* pybind.cpp:68-76 (the three static factories). */
int fml_executor_create(const char *name, int mode, size_t epoch, fml_executor **out);
void fml_executor_destroy(fml_executor *e);
const char *fml_executor_last_error(const fml_executor *e);

/* See worker/executor.h for the option keys. */
int fml_executor_set_option(fml_executor *e, const char *key, const char *value);

/* pybind.cpp:77-82 (compile).  mlir / llvm / json may be NULL. */
int fml_executor_compile_file(fml_executor *e, const char *onnx_path, const char *mlir_path,
                              const char *llvm_path, const char *json_path);
int fml_executor_compile_buffer(fml_executor *e, const void *onnx_bytes, size_t size,
                                const char *mlir_path, const char *llvm_path,
                                const char *json_path);

/* pybind.cpp:83-87 (invoke): `names[i]` -> host pointer `buffers[i]`, for every graph input
 * and output.  Writes the average nanoseconds per forward pass. */
int fml_executor_invoke(fml_executor *e, const char *const *names, void *const *buffers,
                        size_t count, size_t *ns_per_epoch);

/* Planning only (parse, convert, fuse, order, layout search, memory plan): everything Compile
 * does before it touches the device, so it runs on a machine without a GPU.  Results are read
 * through fml_executor_stats_json and the optional dump files. */
int fml_executor_plan_buffer(fml_executor *e, const void *onnx_bytes, size_t size,
                             const char *llvm_path, const char *json_path);

/* Tracing (the reference's only tracing is the Runner's wall clock, src/worker/runner.cpp:
 * 101-119): replays the compiled launch list eagerly `passes` times with an event pair
 * around every launch and returns {"<KernelName>": {"us": total, "launches": n}, ...} as JSON
 * owned by the handle.  Only the inputs in `names` are read; outputs are not copied back. */
int fml_executor_profile(fml_executor *e, const char *const *names, void *const *buffers,
                         size_t count, size_t passes, const char **json_out);

/* The same breakdown without disturbing the pass: replays the captured graph `passes` + 2 times
 * with the library's kernel-start stamps switched on (fml_set_kernel_trace) and attributes to
 * every launch the time from its start to the next launch's start, median over the inner
 * passes.  Returns {"pass_us": .., "kernels": {"<KernelName>": {"us": per pass, "launches": n}},
 * "launch_list": [{"node", "kernel", "us"} in launch order]}.  The periods of a pass add up to
 * the pass. */
int fml_executor_trace(fml_executor *e, const char *const *names, void *const *buffers,
                       size_t count, size_t passes, const char **json_out);

/* JSON text owned by the handle, valid until the next call on it. */
const char *fml_executor_stats_json(fml_executor *e);

/* ---- host helpers exposed for bindings and unit tests -------------------------------
 * utils::GenStrides (src/utils/utils.cpp:64-102); `layout` may be NULL (default layout). */
int fml_host_gen_strides(const long long *shape, const long long *layout, int rank, long long *strides);
/* utils::GenAllOrders (src/utils/utils.cpp:26-41): writes len! rows of len entries in the
 * reference's enumeration order; returns the number of rows. */
long long fml_host_gen_all_orders(int len, long long *out);
/* BroadcastShape / BroadcastMatMulShape (src/structure/tensor/meta.cpp:59-137): returns the
 * output rank or -1. */
int fml_host_broadcast_shape(const long long *a, int ra, const long long *b, int rb, int matmul, long long *out);
/* LinearPlan / GreedyPlan (src/structure/memory/linear.cpp:5-15, greedy.cpp:239-270) over a
 * lifetime table; `alignment` 1 reproduces the reference. */
int fml_host_memory_plan(int greedy, int n, const char *const *names, const size_t *start,
                         const size_t *end, const size_t *size, size_t alignment, size_t *offset_out,
                         size_t *maximum_out);

/* What the layout search charges, in nanoseconds, for one node (the model that stands where the
 * reference measures: KernelEval::GetTimeCost, src/evaluation/eval.cpp:64-100, :261-302):
 * a MatMul [m,k] x constant [k,n] with the given layouts of A and of the output (NULL = default
 * layout), and a LayerNormalization over the last axis of [rows, cols].  `precision` is an
 * fml_gemm_precision.  Tests rank these against measured kernel times. */
int fml_host_model_gemm_cost(long long m, long long k, long long n, const long long *a_layout,
                             const long long *c_layout, int precision, double *ns);
int fml_host_model_layernorm_cost(long long rows, long long cols, const long long *in_layout,
                                  const long long *out_layout, double *ns);

#ifdef __cplusplus
}
#endif
#endif /* FLUIDML_EXECUTOR_H_ */
