// Runtime plumbing of the nvq C ABI: error text, device selection, memory, streams,
// events.  No compute here.
#include <stdarg.h>
#include <string.h>

#include "nvq_common.cuh"

std::atomic<uint64_t> g_nvq_launches{0};

static thread_local char t_err[512] = "";

void nvq_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

namespace {
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices];
int g_cc_major[kMaxDevices];
std::atomic<int> g_probed[kMaxDevices];
}  // namespace

nvq_status nvq_use_device(int device) {
    NVQ_REQUIRE(device >= 0 && device < kMaxDevices, "device %d out of range", device);
    NVQ_CUDA(cudaSetDevice(device));
    if (!g_probed[device].load(std::memory_order_acquire)) {
        cudaDeviceProp p;
        NVQ_CUDA(cudaGetDeviceProperties(&p, device));
        g_sm_count[device] = p.multiProcessorCount;
        g_cc_major[device] = p.major;
        g_probed[device].store(1, std::memory_order_release);
    }
    if (g_cc_major[device] != 10)
        NVQ_FAIL(NVQ_ERR_UNSUPPORTED, "device %d is compute capability %d.x; this library holds sm_100a code only",
                 device, g_cc_major[device]);
    return NVQ_OK;
}

// lazily allocated per-device state of other translation units (see nvq_shutdown)
nvq_status nvq_cast_release_staging();
nvq_status nvq_gemm_release_status_words();

int nvq_sm_count(int device) { return g_sm_count[device] > 0 ? g_sm_count[device] : 148; }

extern "C" {

const char* nvq_last_error(void) { return t_err; }
const char* nvq_version(void) { return "nvq 0.1 (sm_100a)"; }
uint64_t nvq_launch_count(void) { return g_nvq_launches.load(std::memory_order_relaxed); }

nvq_status nvq_device_count(int* count) {
    NVQ_REQUIRE(count, "null count");
    *count = 0;
    NVQ_CUDA(cudaGetDeviceCount(count));
    return NVQ_OK;
}

nvq_status nvq_device_info(int device, int* sm_count, size_t* total_bytes, int* cc_major,
                           int* cc_minor) {
    cudaDeviceProp p;
    NVQ_CUDA(cudaGetDeviceProperties(&p, device));
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (total_bytes) *total_bytes = p.totalGlobalMem;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    return NVQ_OK;
}

nvq_status nvq_shutdown(void) {
    nvq_status a = nvq_cast_release_staging();
    nvq_status b = nvq_gemm_release_status_words();
    return a != NVQ_OK ? a : b;
}

nvq_status nvq_malloc(int device, size_t bytes, void** d_ptr) {
    NVQ_REQUIRE(d_ptr, "null out pointer");
    *d_ptr = nullptr;
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    if (bytes == 0) return NVQ_OK;
    NVQ_CUDA(cudaMalloc(d_ptr, bytes));
    return NVQ_OK;
}

nvq_status nvq_free(int device, void* d_ptr) {
    if (!d_ptr) return NVQ_OK;
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaFree(d_ptr));
    return NVQ_OK;
}

nvq_status nvq_host_alloc(size_t bytes, void** h_ptr) {
    NVQ_REQUIRE(h_ptr, "null out pointer");
    *h_ptr = nullptr;
    if (bytes == 0) return NVQ_OK;
    NVQ_CUDA(cudaHostAlloc(h_ptr, bytes, cudaHostAllocPortable));
    return NVQ_OK;
}

nvq_status nvq_host_free(void* h_ptr) {
    if (!h_ptr) return NVQ_OK;
    NVQ_CUDA(cudaFreeHost(h_ptr));
    return NVQ_OK;
}

static nvq_status copy(void* dst, const void* src, size_t bytes, int device, void* stream,
                       cudaMemcpyKind kind) {
    if (bytes == 0) return NVQ_OK;
    NVQ_REQUIRE(dst && src, "null buffer in copy");
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream));
    return NVQ_OK;
}

nvq_status nvq_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, int device, void* stream) {
    return copy(d_dst, h_src, bytes, device, stream, cudaMemcpyHostToDevice);
}
nvq_status nvq_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, int device, void* stream) {
    return copy(h_dst, d_src, bytes, device, stream, cudaMemcpyDeviceToHost);
}
nvq_status nvq_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, int device, void* stream) {
    return copy(d_dst, d_src, bytes, device, stream, cudaMemcpyDeviceToDevice);
}
nvq_status nvq_memset(void* d_dst, int value, size_t bytes, int device, void* stream) {
    if (bytes == 0) return NVQ_OK;
    NVQ_REQUIRE(d_dst, "null buffer in memset");
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaMemsetAsync(d_dst, value, bytes, (cudaStream_t)stream));
    return NVQ_OK;
}

nvq_status nvq_stream_create(int device, void** stream) {
    NVQ_REQUIRE(stream, "null out pointer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st;
    NVQ_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    *stream = (void*)st;
    return NVQ_OK;
}
nvq_status nvq_stream_destroy(int device, void* stream) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaStreamDestroy((cudaStream_t)stream));
    return NVQ_OK;
}
nvq_status nvq_stream_sync(int device, void* stream) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return NVQ_OK;
}
nvq_status nvq_device_sync(int device) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaDeviceSynchronize());
    return NVQ_OK;
}
nvq_status nvq_event_create(int device, void** event) {
    NVQ_REQUIRE(event, "null out pointer");
    NVQ_CUDA(cudaSetDevice(device));
    cudaEvent_t e;
    NVQ_CUDA(cudaEventCreate(&e));
    *event = (void*)e;
    return NVQ_OK;
}
nvq_status nvq_event_destroy(int device, void* event) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return NVQ_OK;
}
nvq_status nvq_event_record(int device, void* event, void* stream) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return NVQ_OK;
}
nvq_status nvq_stream_wait_event(int device, void* stream, void* event) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
    return NVQ_OK;
}
nvq_status nvq_event_sync(int device, void* event) {
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaEventSynchronize((cudaEvent_t)event));
    return NVQ_OK;
}
nvq_status nvq_event_elapsed_ms(void* start, void* stop, float* ms) {
    NVQ_REQUIRE(ms, "null out pointer");
    NVQ_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return NVQ_OK;
}

// ---- CUDA graphs: capture a fixed launch sequence once, replay it with one launch -------
nvq_status nvq_graph_begin_capture(int device, void* stream) {
    NVQ_REQUIRE(stream, "graph capture needs an explicit (non-default) stream");
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
    return NVQ_OK;
}
nvq_status nvq_graph_end_capture(int device, void* stream, void** graph_exec) {
    NVQ_REQUIRE(stream && graph_exec, "null argument");
    NVQ_CUDA(cudaSetDevice(device));
    cudaGraph_t g = nullptr;
    NVQ_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &g));
    cudaGraphExec_t e = nullptr;
    cudaError_t err = cudaGraphInstantiate(&e, g, 0);
    cudaGraphDestroy(g);
    if (err != cudaSuccess) NVQ_FAIL(NVQ_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(err));
    *graph_exec = (void*)e;
    return NVQ_OK;
}
nvq_status nvq_graph_launch(int device, void* graph_exec, void* stream) {
    NVQ_REQUIRE(graph_exec, "null graph");
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
    return NVQ_OK;
}
nvq_status nvq_graph_destroy(int device, void* graph_exec) {
    if (!graph_exec) return NVQ_OK;
    NVQ_CUDA(cudaSetDevice(device));
    NVQ_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
    return NVQ_OK;
}

}  // extern "C"
