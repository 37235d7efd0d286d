// Library plumbing behind the C ABI: error strings, device checks, memory, streams, events and
// CUDA-graph capture.  No kernels here except the status word.
#include "common.cuh"
#include "sm100.cuh"

namespace qb {

__device__ unsigned int g_qb_status = 0;
unsigned long long g_launch_count = 0;
static int dependent_launch_default() {
  const char* e = getenv("QB_DEPENDENT_LAUNCH");
  return (e != nullptr && e[0] == '0') ? 0 : 1;
}
int g_dependent_launch = dependent_launch_default();

// Device address of the status word for the current device (one copy of the symbol per device).
unsigned int* status_word() {
  static unsigned int* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_qb_status) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<unsigned int*>(p);
  }
  return cache[dev];
}

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace qb

using namespace qb;

extern "C" {

int32_t qb_version(void) { return 100; }

const char* qb_last_error_string(void) { return error_buffer(); }

int32_t qb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int32_t qb_device_check(int32_t device) {
  int n = qb_device_count();
  QB_REQUIRE(device >= 0 && device < n, QB_ERR_DEVICE, "device %d not present (%d CUDA devices)", device, n);
  int major = 0, minor = 0;
  QB_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  QB_CUDA_OK(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  QB_REQUIRE(major == 10 && minor == 0, QB_ERR_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", device,
             major, minor);
  return QB_OK;
}

int32_t qb_set_device(int32_t device) {
  QB_CUDA_OK(cudaSetDevice(device));
  return QB_OK;
}

int32_t qb_device_status(uint32_t* status_host) {
  QB_REQUIRE(status_host != nullptr, QB_ERR_INVALID_ARG, "status_host is NULL");
  unsigned int v = 0, zero = 0;
  QB_CUDA_OK(cudaDeviceSynchronize());
  QB_CUDA_OK(cudaMemcpyFromSymbol(&v, g_qb_status, sizeof(v)));
  if (v != 0) QB_CUDA_OK(cudaMemcpyToSymbol(g_qb_status, &zero, sizeof(zero)));
  *status_host = v;
  return QB_OK;
}

uint64_t qb_kernel_launch_count(void) { return g_launch_count; }
int32_t qb_set_dependent_launch(int32_t enabled) {
  const int prev = g_dependent_launch;
  g_dependent_launch = enabled != 0;
  return prev;
}

int32_t qb_malloc(void** ptr_host, size_t bytes) {
  QB_REQUIRE(ptr_host != nullptr, QB_ERR_INVALID_ARG, "ptr_host is NULL");
  QB_CUDA_OK(cudaMalloc(ptr_host, bytes == 0 ? 16 : bytes));
  return QB_OK;
}
int32_t qb_free(void* ptr) {
  if (ptr) QB_CUDA_OK(cudaFree(ptr));
  return QB_OK;
}
int32_t qb_host_alloc(void** ptr_host, size_t bytes) {
  QB_REQUIRE(ptr_host != nullptr, QB_ERR_INVALID_ARG, "ptr_host is NULL");
  QB_CUDA_OK(cudaHostAlloc(ptr_host, bytes == 0 ? 16 : bytes, cudaHostAllocDefault));
  return QB_OK;
}
int32_t qb_host_free(void* ptr_hostmem) {
  if (ptr_hostmem) QB_CUDA_OK(cudaFreeHost(ptr_hostmem));
  return QB_OK;
}

int32_t qb_memcpy_async(void* dst, const void* src, size_t bytes, int32_t kind, void* stream) {
  QB_REQUIRE(kind >= 0 && kind <= 2, QB_ERR_INVALID_ARG, "memcpy kind %d", kind);
  if (bytes == 0) return QB_OK;
  QB_REQUIRE(dst && src, QB_ERR_INVALID_ARG, "memcpy with NULL pointer");
  const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  QB_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, k, static_cast<cudaStream_t>(stream)));
  return QB_OK;
}
int32_t qb_memset_async(void* dst, int32_t byte_value, size_t bytes, void* stream) {
  if (bytes == 0) return QB_OK;
  QB_REQUIRE(dst, QB_ERR_INVALID_ARG, "memset with NULL pointer");
  QB_CUDA_OK(cudaMemsetAsync(dst, byte_value, bytes, static_cast<cudaStream_t>(stream)));
  return QB_OK;
}

__global__ void fill32_kernel(uint32_t* p, uint32_t v, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) p[i] = v;
}
int32_t qb_memset32_async(void* dst, uint32_t value, size_t count, void* stream) {
  if (count == 0) return QB_OK;
  QB_REQUIRE(dst, QB_ERR_INVALID_ARG, "memset32 with NULL pointer");
  fill32_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint32_t*>(dst), value, count);
  return check_launch("memset32");
}

int32_t qb_stream_create(void** stream_host) {
  QB_REQUIRE(stream_host != nullptr, QB_ERR_INVALID_ARG, "stream_host is NULL");
  cudaStream_t s;
  QB_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream_host = s;
  return QB_OK;
}
int32_t qb_stream_destroy(void* stream) {
  if (stream) QB_CUDA_OK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return QB_OK;
}
int32_t qb_stream_sync(void* stream) {
  QB_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return QB_OK;
}
int32_t qb_device_sync(void) {
  QB_CUDA_OK(cudaDeviceSynchronize());
  return QB_OK;
}

int32_t qb_event_create(void** event_host) {
  QB_REQUIRE(event_host != nullptr, QB_ERR_INVALID_ARG, "event_host is NULL");
  cudaEvent_t e;
  QB_CUDA_OK(cudaEventCreate(&e));
  *event_host = e;
  return QB_OK;
}
int32_t qb_event_destroy(void* event) {
  if (event) QB_CUDA_OK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return QB_OK;
}
int32_t qb_event_record(void* event, void* stream) {
  QB_CUDA_OK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return QB_OK;
}
int32_t qb_event_sync(void* event) {
  QB_CUDA_OK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  return QB_OK;
}
int32_t qb_event_elapsed_ms(void* start, void* stop, float* ms_host) {
  QB_REQUIRE(ms_host != nullptr, QB_ERR_INVALID_ARG, "ms_host is NULL");
  QB_CUDA_OK(cudaEventElapsedTime(ms_host, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  return QB_OK;
}

int32_t qb_graph_begin(void* stream) {
  QB_REQUIRE(stream != nullptr, QB_ERR_INVALID_ARG, "graph capture needs a non-default stream");
  QB_CUDA_OK(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
  return QB_OK;
}
int32_t qb_graph_end(void* stream, void** graph_exec_host) {
  QB_REQUIRE(graph_exec_host != nullptr, QB_ERR_INVALID_ARG, "graph_exec_host is NULL");
  cudaGraph_t g = nullptr;
  QB_CUDA_OK(cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &g));
  cudaGraphExec_t ge = nullptr;
  cudaError_t e = cudaGraphInstantiate(&ge, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fail(QB_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  *graph_exec_host = ge;
  return QB_OK;
}
int32_t qb_graph_launch(void* graph_exec, void* stream) {
  QB_CUDA_OK(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), static_cast<cudaStream_t>(stream)));
  return QB_OK;
}
int32_t qb_graph_destroy(void* graph_exec) {
  if (graph_exec) QB_CUDA_OK(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)));
  return QB_OK;
}

}  // extern "C"
