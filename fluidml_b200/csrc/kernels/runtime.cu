// Runtime plumbing of the C ABI: error text, device selection, buffers, copies, streams and
// the per-device status word that kernels with bounded waits or clamped indices write.
#include "common.cuh"
#include <cstdarg>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace fml {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return e == cudaErrorMemoryAllocation ? FML_OUT_OF_MEMORY : FML_CUDA_ERROR;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char *v = getenv("FLUIDML_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

static int *g_status[64] = {nullptr};
static std::mutex g_status_mu;

int *device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mu);
  if (!g_status[dev]) {
    int *p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_status[dev] = p;
  }
  return g_status[dev];
}

}  // namespace fml

// Takes the device status word: *out = old value, word = 0.  `out` is pinned host memory.
static __global__ void status_take_kernel(int *word, int *out) { *out = atomicExch(word, 0); }

using namespace fml;

extern "C" {

const char *fml_last_error(void) { return g_error; }

int fml_device_count(int *count) {
  FML_REQUIRE(count, FML_BAD_ARG, "fml_device_count: null argument");
  FML_CUDA(cudaGetDeviceCount(count));
  return FML_OK;
}

int fml_mem_info(size_t *free_bytes, size_t *total_bytes) {
  FML_REQUIRE(free_bytes && total_bytes, FML_BAD_ARG, "fml_mem_info: null argument");
  FML_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return FML_OK;
}

int fml_set_device(int device) {
  FML_CUDA(cudaSetDevice(device));
  return FML_OK;
}

int fml_malloc(void **ptr, size_t bytes) {
  FML_REQUIRE(ptr, FML_BAD_ARG, "fml_malloc: null argument");
  FML_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
  return FML_OK;
}

int fml_free(void *ptr) {
  FML_CUDA(cudaFree(ptr));
  return FML_OK;
}

int fml_memset(void *ptr, int value, size_t bytes, void *stream) {
  FML_CUDA(cudaMemsetAsync(ptr, value, bytes, as_stream(stream)));
  return FML_OK;
}

int fml_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
  FML_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return FML_OK;
}

int fml_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
  FML_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return FML_OK;
}

int fml_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream) {
  FML_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return FML_OK;
}

int fml_host_alloc_pinned(void **ptr, size_t bytes) {
  FML_REQUIRE(ptr, FML_BAD_ARG, "fml_host_alloc_pinned: null argument");
  FML_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1));
  return FML_OK;
}

int fml_host_free_pinned(void *ptr) {
  FML_CUDA(cudaFreeHost(ptr));
  return FML_OK;
}

int fml_stream_create(void **stream) {
  FML_REQUIRE(stream, FML_BAD_ARG, "fml_stream_create: null argument");
  cudaStream_t s;
  FML_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return FML_OK;
}

int fml_stream_destroy(void *stream) {
  FML_CUDA(cudaStreamDestroy(as_stream(stream)));
  return FML_OK;
}

int fml_stream_sync(void *stream) {
  FML_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return FML_OK;
}

int fml_event_create(void **event) {
  FML_REQUIRE(event, FML_BAD_ARG, "fml_event_create: null argument");
  cudaEvent_t e;
  FML_CUDA(cudaEventCreate(&e));
  *event = e;
  return FML_OK;
}

int fml_event_destroy(void *event) {
  FML_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return FML_OK;
}

int fml_event_record(void *event, void *stream) {
  FML_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)));
  return FML_OK;
}

int fml_event_sync(void *event) {
  FML_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return FML_OK;
}

int fml_event_elapsed_ms(void *start, void *stop, float *ms) {
  FML_REQUIRE(ms, FML_BAD_ARG, "fml_event_elapsed_ms: null argument");
  FML_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return FML_OK;
}

int fml_graph_begin_capture(void *stream) {
  FML_CUDA(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal));
  return FML_OK;
}

int fml_graph_end_capture(void *stream, void **graph_exec) {
  FML_REQUIRE(graph_exec, FML_BAD_ARG, "fml_graph_end_capture: null argument");
  *graph_exec = nullptr;
  cudaGraph_t graph = nullptr;
  FML_CUDA(cudaStreamEndCapture(as_stream(stream), &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
  *graph_exec = exec;
  return FML_OK;
}

int fml_graph_abort_capture(void *stream) {
  cudaGraph_t graph = nullptr;
  cudaStreamEndCapture(as_stream(stream), &graph);
  if (graph) cudaGraphDestroy(graph);
  cudaGetLastError();
  return FML_OK;
}

int fml_graph_launch(void *graph_exec, void *stream) {
  FML_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), as_stream(stream)));
  return FML_OK;
}

int fml_graph_destroy(void *graph_exec) {
  FML_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)));
  return FML_OK;
}

int fml_warmup(void) {
  FML_REQUIRE(device_status_word(), FML_CUDA_ERROR, "fml_warmup: cannot allocate the device status word");
  return FML_OK;
}

int fml_check_device(void *stream) {
  int *w = device_status_word();
  FML_REQUIRE(w, FML_CUDA_ERROR, "fml_check_device: no status word");
  // One launch on the caller's stream takes the word (atomic exchange with 0, so a bit another
  // stream's kernel sets at the same moment is either taken now or left for the next check, never
  // lost) and writes it to a pinned host word; one synchronisation then serves both the caller's
  // work and the check.  One pinned word per calling thread.
  static thread_local int *pinned = nullptr;
  if (!pinned) FML_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&pinned), sizeof(int), cudaHostAllocDefault));
  status_take_kernel<<<1, 1, 0, as_stream(stream)>>>(w, pinned);
  FML_CUDA(cudaGetLastError());
  FML_CUDA(cudaStreamSynchronize(as_stream(stream)));
  const int v = *pinned;
  if (v & kStatusTimeout) {
    set_error("a bounded device-side wait expired");
    return FML_DEVICE_TIMEOUT;
  }
  if (v & kStatusIndexRange) {
    set_error("a gather index was outside the table and was clamped");
    return FML_INDEX_OUT_OF_RANGE;
  }
  return FML_OK;
}

}  // extern "C"

namespace fml {
namespace {
std::vector<cudaError_t (*)(unsigned long long *, unsigned *, unsigned)> &trace_setters() {
  static std::vector<cudaError_t (*)(unsigned long long *, unsigned *, unsigned)> v;
  return v;
}
}  // namespace
void register_trace_setter(cudaError_t (*setter)(unsigned long long *, unsigned *, unsigned)) {
  trace_setters().push_back(setter);
}
namespace {
std::vector<cudaError_t (*)(uint32_t, int)> &wait_test_setters() {
  static std::vector<cudaError_t (*)(uint32_t, int)> v;
  return v;
}
}  // namespace
void register_wait_test_setter(cudaError_t (*setter)(uint32_t, int)) { wait_test_setters().push_back(setter); }
}  // namespace fml
// Test hook: iteration limit of every bounded mbarrier wait of the tensor-core kernels (0 restores
// the default) and whether their producers skip their loads.  With (small limit, 1) a launch's
// waits all run out: the kernel sets the status bit fml_check_device reports as
// FML_DEVICE_TIMEOUT and returns; the context stays usable.  Synchronises the device.
extern "C" int fml_debug_wait_test(unsigned limit, int drop_loads) {
  FML_CUDA(cudaDeviceSynchronize());
  for (auto f : fml::wait_test_setters()) FML_CUDA(f(limit ? limit : (1u << 22), drop_loads));
  return FML_OK;
}
// buf = device array of `cap` 64-bit stamps, cursor = device counter (zeroed by the caller).
// NULL buf switches the stamps off.  Synchronises (the pointers are module variables).
extern "C" int fml_set_kernel_trace(void *buf, void *cursor, unsigned cap) {
  for (auto f : fml::trace_setters()) FML_CUDA(f((unsigned long long *)buf, (unsigned *)cursor, cap));
  return FML_OK;
}
