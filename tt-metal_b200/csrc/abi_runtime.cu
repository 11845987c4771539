// C ABI: error reporting and the thin CUDA-runtime wrappers (device memory, copies, sync).
#include <cstring>

#include <nvtx3/nvToolsExt.h>   // header-only: ranges cost nothing unless a profiler injects its library

#include "common.cuh"

namespace ttb {
static thread_local char g_err[512] = "";

int32_t fail(int32_t code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace ttb

using ttb::fail;

extern "C" {

const char *ttb_last_error(void) { return ttb::g_err; }
int32_t ttb_version(void) { return 100; }

int32_t ttb_device_count(int32_t *count) {
    if (!count) return fail(TTB_E_INVALID, "ttb_device_count: null output pointer");
    int n = 0;
    TTB_CUDA_TRY(cudaGetDeviceCount(&n));
    *count = n;
    return TTB_OK;
}
int32_t ttb_set_device(int32_t device) {
    TTB_CUDA_TRY(cudaSetDevice(device));
    return TTB_OK;
}
int32_t ttb_get_device(int32_t *device) {
    if (!device) return fail(TTB_E_INVALID, "ttb_get_device: null output pointer");
    int d = 0;
    TTB_CUDA_TRY(cudaGetDevice(&d));
    *device = d;
    return TTB_OK;
}
int32_t ttb_malloc(void **dev_ptr, size_t bytes) {
    if (!dev_ptr) return fail(TTB_E_INVALID, "ttb_malloc: null output pointer");
    *dev_ptr = nullptr;
    if (bytes == 0) return TTB_OK;
    TTB_CUDA_TRY(cudaMalloc(dev_ptr, bytes));
    return TTB_OK;
}
int32_t ttb_mem_info(int64_t *free_bytes, int64_t *total_bytes) {
    size_t f = 0, t = 0;
    TTB_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = (int64_t)f;
    if (total_bytes) *total_bytes = (int64_t)t;
    return TTB_OK;
}
int32_t ttb_free(void *dev_ptr) {
    if (dev_ptr) TTB_CUDA_TRY(cudaFree(dev_ptr));
    return TTB_OK;
}
// ---- CUDA IPC: peer pointers for the gather epilogue ------------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) == TTB_IPC_HANDLE_BYTES, "IPC handle size");
int32_t ttb_ipc_export(void *ptr_dev, void *handle) {
    if (!ptr_dev || !handle) return fail(TTB_E_INVALID, "ttb_ipc_export: null pointer");
    cudaIpcMemHandle_t h;
    TTB_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr_dev));
    memcpy(handle, &h, sizeof(h));
    return TTB_OK;
}
int32_t ttb_ipc_open(const void *handle, void **ptr_dev) {
    if (!ptr_dev || !handle) return fail(TTB_E_INVALID, "ttb_ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    *ptr_dev = nullptr;
    TTB_CUDA_TRY(cudaIpcOpenMemHandle(ptr_dev, h, cudaIpcMemLazyEnablePeerAccess));
    return TTB_OK;
}
int32_t ttb_ipc_close(void *ptr_dev) {
    if (ptr_dev) TTB_CUDA_TRY(cudaIpcCloseMemHandle(ptr_dev));
    return TTB_OK;
}

int32_t ttb_host_alloc(void **host_ptr, size_t bytes) {
    if (!host_ptr) return fail(TTB_E_INVALID, "ttb_host_alloc: null output pointer");
    *host_ptr = nullptr;
    if (bytes == 0) return TTB_OK;
    TTB_CUDA_TRY(cudaMallocHost(host_ptr, bytes));
    return TTB_OK;
}
int32_t ttb_host_free(void *host_ptr) {
    if (host_ptr) TTB_CUDA_TRY(cudaFreeHost(host_ptr));
    return TTB_OK;
}
int32_t ttb_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return TTB_OK;
    if (!dst || !src) return fail(TTB_E_INVALID, "ttb_memcpy_h2d: null pointer");
    TTB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return TTB_OK;
}
int32_t ttb_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return TTB_OK;
    if (!dst || !src) return fail(TTB_E_INVALID, "ttb_memcpy_d2h: null pointer");
    TTB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return TTB_OK;
}
int32_t ttb_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return TTB_OK;
    if (!dst || !src) return fail(TTB_E_INVALID, "ttb_memcpy_d2d: null pointer");
    TTB_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return TTB_OK;
}
int32_t ttb_memset(void *dst, int32_t value, size_t bytes, void *stream) {
    if (bytes == 0) return TTB_OK;
    if (!dst) return fail(TTB_E_INVALID, "ttb_memset: null pointer");
    TTB_CUDA_TRY(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return TTB_OK;
}
int32_t ttb_stream_synchronize(void *stream) {
    TTB_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return TTB_OK;
}
int32_t ttb_device_synchronize(void) {
    TTB_CUDA_TRY(cudaDeviceSynchronize());
    return TTB_OK;
}

// ---- NVTX ranges (timeline tools show them around the calls they bracket) ---------------------------------------
int32_t ttb_nvtx_push(const char *name) {
    nvtxRangePushA(name ? name : "ttb");
    return TTB_OK;
}
int32_t ttb_nvtx_pop(void) {
    nvtxRangePop();
    return TTB_OK;
}

int64_t ttb_buffer_bytes(int32_t dtype, int64_t outer, int64_t Hp, int64_t Wp) {
    int64_t n = outer * Hp * Wp;
    switch (dtype) {
        case TTB_BFLOAT16:
        case TTB_UINT16: return n * 2;
        case TTB_FLOAT32:
        case TTB_UINT32: return n * 4;
        case TTB_BFLOAT8_B: return n / 1024 * ttb::kBfp8TileBytes;
        case TTB_BFLOAT4_B: return n / 1024 * ttb::kBfp4TileBytes;
        default: return -1;
    }
}

}  // extern "C"
