// hal.cu — device layer: the six HAL functions the reference names for its device layer
// (README.md:203) plus streams and pinned host memory, and the library's error plumbing.
// Semantics follow the reference's SYCL Device (code/device/sycl/device.h:143-148):
// upload/download block until the copy is done; a zero-byte alloc gives NULL.
#include <cstring>
#include <string>

#include "common.cuh"

namespace novab {
namespace {
thread_local std::string g_last_cuda;
std::atomic<uint64_t> g_launches{0};
}  // namespace

void set_cuda_error(cudaError_t e, const char* what) {
    g_last_cuda = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
}
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// Multiprocessors of the calling thread's current device (cudaDevAttrMultiProcessorCount), looked up once
// per device.  Concurrent first calls may both query and store the same value.  148 (a B200) when the
// query fails, so that grid sizing never sees zero.
int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}
}  // namespace novab

using namespace novab;

extern "C" {

const char* nova_status_string(int status) {
    switch (status) {
        case NOVA_OK: return "ok";
        case NOVA_ERR_INVALID: return "invalid argument";
        case NOVA_ERR_POOL_FULL: return "KV page pool is full";
        case NOVA_ERR_NO_SLICE: return "no free KV slice";
        case NOVA_ERR_NO_SESSION: return "no free session slot";
        case NOVA_ERR_CUDA: return "CUDA error";
        case NOVA_ERR_BAD_TABLE: return "block-table entry out of range";
        case NOVA_ERR_TIMEOUT: return "device-side wait timed out";
        case NOVA_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case NOVA_ERR_TOO_LARGE: return "size beyond the fixed maximum";
        case NOVA_ERR_BUSY: return "pages of the slice are still mapped by another session";
        default: return "unknown status";
    }
}

const char* nova_last_cuda_error(void) { return g_last_cuda.c_str(); }
uint64_t nova_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int dev_select(int device) {
    NOVA_CUDA_TRY(cudaSetDevice(device));
    return NOVA_OK;
}
int dev_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}
void* dev_alloc(size_t bytes) {
    if (bytes == 0) return nullptr;
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        set_cuda_error(e, "cudaMalloc");
        return nullptr;
    }
    return p;
}
void dev_free(void* p) {
    if (p) cudaFree(p);
}
int dev_upload(void* dst_dev, const void* src_host, size_t bytes) {
    if (bytes == 0) return NOVA_OK;
    if (!dst_dev || !src_host) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaMemcpy(dst_dev, src_host, bytes, cudaMemcpyHostToDevice));
    return NOVA_OK;
}
int dev_download(void* dst_host, const void* src_dev, size_t bytes) {
    if (bytes == 0) return NOVA_OK;
    if (!dst_host || !src_dev) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaMemcpy(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost));
    return NOVA_OK;
}
int dev_zero(void* dst_dev, size_t bytes) {
    if (bytes == 0) return NOVA_OK;
    if (!dst_dev) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaMemset(dst_dev, 0, bytes));
    return NOVA_OK;
}
int dev_sync(void) {
    NOVA_CUDA_TRY(cudaDeviceSynchronize());
    return NOVA_OK;
}
size_t dev_max_alloc(void) {
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return 0;
    return free_b;
}
void* dev_host_alloc(size_t bytes) {
    if (bytes == 0) return nullptr;
    void* p = nullptr;
    const cudaError_t e = cudaMallocHost(&p, bytes);
    if (e != cudaSuccess) {
        set_cuda_error(e, "cudaMallocHost");
        return nullptr;
    }
    return p;
}
void dev_host_free(void* p) {
    if (p) cudaFreeHost(p);
}
int dev_stream_create(nova_stream_t* out) {
    if (!out) return NOVA_ERR_INVALID;
    cudaStream_t s = nullptr;
    NOVA_CUDA_TRY(cudaStreamCreate(&s));   // blocking w.r.t. the legacy stream, as code/session.h:94
    *out = (nova_stream_t)s;
    return NOVA_OK;
}
int dev_stream_destroy(nova_stream_t s) {
    if (s) NOVA_CUDA_TRY(cudaStreamDestroy((cudaStream_t)s));
    return NOVA_OK;
}
int dev_event_create(nova_event_t* out) {
    if (!out) return NOVA_ERR_INVALID;
    cudaEvent_t e = nullptr;
    NOVA_CUDA_TRY(cudaEventCreate(&e));
    *out = (nova_event_t)e;
    return NOVA_OK;
}
int dev_event_destroy(nova_event_t e) {
    if (e) NOVA_CUDA_TRY(cudaEventDestroy((cudaEvent_t)e));
    return NOVA_OK;
}
int dev_event_record(nova_event_t e, nova_stream_t s) {
    NOVA_CUDA_TRY(cudaEventRecord((cudaEvent_t)e, (cudaStream_t)s));
    return NOVA_OK;
}
int dev_event_sync(nova_event_t e) {
    NOVA_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)e));
    return NOVA_OK;
}
int dev_event_elapsed_ms(nova_event_t start, nova_event_t stop, float* ms) {
    if (!ms) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return NOVA_OK;
}
int dev_stream_sync(nova_stream_t s) {
    NOVA_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)s));
    return NOVA_OK;
}

// Sharing one device allocation between the processes of a node (one process per GPU): the owner
// exports a 64-byte handle, a peer opens it and gets a pointer it can use in its own kernels (peer
// access over NVLink is enabled by the open).  Only whole dev_alloc allocations can be exported.
int dev_ipc_export(void* dev_ptr, void* handle64) {
    if (!dev_ptr || !handle64) return NOVA_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    NOVA_CUDA_TRY(cudaIpcGetMemHandle(&h, dev_ptr));
    std::memcpy(handle64, &h, sizeof(h));
    return NOVA_OK;
}
int dev_ipc_open(const void* handle64, void** dev_ptr) {
    if (!handle64 || !dev_ptr) return NOVA_ERR_INVALID;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    NOVA_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *dev_ptr = p;
    return NOVA_OK;
}
int dev_ipc_close(void* dev_ptr) {
    if (dev_ptr) NOVA_CUDA_TRY(cudaIpcCloseMemHandle(dev_ptr));
    return NOVA_OK;
}

}  // extern "C"
