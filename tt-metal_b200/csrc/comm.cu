// Communicator behind the C ABI: NCCL over NVLink for the general form of ttnn.all_gather, with the failure handling a
// long-running server needs - non-blocking initialisation, asynchronous-error polling under a host-side time limit, and
// abort. Stands in for the ethernet ring set-up and the AllGather op of the reference
// (tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104, ttnn/ttnn/operations/ccl.py:26-39).
//
// NCCL is reached through a table of function pointers filled from libnccl.so.2 at first use (dlopen: the library loads
// and every other entry point works where NCCL is absent). Tests replace the table with a fake (ttb_comm_set_backend)
// to produce the failures - a peer that never joins, an asynchronous error - on the host, without any GPU.
#include <dlfcn.h>
#include <nccl.h>   // types and the configuration initialiser only: the library itself is loaded at run time

#include <chrono>
#include <cstring>
#include <thread>

#include "common.cuh"

namespace ttb {
namespace {

// Result codes of the backend (NCCL's numbering): 0 success, 7 in progress, anything else an error.
constexpr int kBackendOk = (int)ncclSuccess, kBackendInProgress = (int)ncclInProgress;

ttb_comm_backend g_backend = {};
bool g_backend_ready = false;
int g_nccl_version = 0;

int32_t load_backend() {
    if (g_backend_ready) return TTB_OK;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy the process already uses, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(TTB_E_UNSUPPORTED, "ttb_comm: libnccl.so.2 cannot be loaded (%s)", dlerror());
    ttb_comm_backend b = {};
    b.get_unique_id = (int (*)(void *))dlsym(h, "ncclGetUniqueId");
    b.init_rank_config = (int (*)(void **, int, const void *, int, void *))nullptr;
    b.get_async_error = (int (*)(void *, int *))dlsym(h, "ncclCommGetAsyncError");
    b.all_gather = (int (*)(const void *, void *, size_t, int, void *, void *))dlsym(h, "ncclAllGather");
    b.abort = (int (*)(void *))dlsym(h, "ncclCommAbort");
    b.destroy = (int (*)(void *))dlsym(h, "ncclCommDestroy");
    b.error_string = (const char *(*)(int))dlsym(h, "ncclGetErrorString");
    // ncclCommInitRankConfig takes the 128-byte id by value: reached through a small shim below
    void *init = dlsym(h, "ncclCommInitRankConfig");
    auto ver = (int (*)(int *))dlsym(h, "ncclGetVersion");
    if (!b.get_unique_id || !init || !b.get_async_error || !b.all_gather || !b.abort || !b.destroy)
        return fail(TTB_E_UNSUPPORTED, "ttb_comm: libnccl.so.2 lacks a required entry point");
    if (ver) ver(&g_nccl_version);
    b.user = init;
    g_backend = b;
    g_backend_ready = true;
    return TTB_OK;
}

int backend_init(const ttb_comm_backend &b, void **comm, int ranks, const void *id, int rank) {
    if (b.init_rank_config) return b.init_rank_config(comm, ranks, id, rank, b.user);
    // the real library, non-blocking: initialisation proceeds in the background and is polled by the caller
    using InitFn = ncclResult_t (*)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *);
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    ncclUniqueId uid;
    static_assert(sizeof(uid) == TTB_COMM_ID_BYTES, "unique id size");
    memcpy(&uid, id, sizeof(uid));
    return (int)reinterpret_cast<InitFn>(b.user)(reinterpret_cast<ncclComm_t *>(comm), ranks, uid, rank, &cfg);
}

const char *backend_error(const ttb_comm_backend &b, int code) {
    return b.error_string ? b.error_string(code) : "backend error";
}

struct Comm {
    void *handle = nullptr;
    int ranks = 0, rank = 0;
    bool aborted = false;
};

// Polls the communicator's asynchronous state until it leaves "in progress" or `timeout_ms` of host time have passed.
int32_t wait_ready(Comm *c, int64_t timeout_ms, const char *what) {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        int state = kBackendOk;
        const int rc = g_backend.get_async_error(c->handle, &state);
        if (rc != kBackendOk) return fail(TTB_E_CUDA, "%s: polling the communicator failed: %s", what, backend_error(g_backend, rc));
        if (state == kBackendOk) return TTB_OK;
        if (state != kBackendInProgress) return fail(TTB_E_CUDA, "%s: the communicator reported an asynchronous error: %s", what, backend_error(g_backend, state));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms >= 0 && ms > timeout_ms)
            return fail(TTB_E_TIMEOUT, "%s: not complete after %lld ms (rank %d of %d); abort the communicator", what, (long long)timeout_ms, c->rank, c->ranks);
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" {

int32_t ttb_comm_set_backend(const ttb_comm_backend *backend) {
    if (!backend) {   // back to the real library at next use
        g_backend = {};
        g_backend_ready = false;
        return TTB_OK;
    }
    if (!backend->get_unique_id || !backend->init_rank_config || !backend->get_async_error || !backend->all_gather || !backend->abort ||
        !backend->destroy)
        return fail(TTB_E_INVALID, "ttb_comm_set_backend: every entry except error_string and user must be set");
    g_backend = *backend;
    g_backend_ready = true;
    return TTB_OK;
}

int32_t ttb_comm_unique_id(void *id) {
    if (!id) return fail(TTB_E_INVALID, "ttb_comm_unique_id: null output pointer");
    if (int32_t rc = load_backend()) return rc;
    const int r = g_backend.get_unique_id(id);
    if (r != kBackendOk) return fail(TTB_E_CUDA, "ttb_comm_unique_id: %s", backend_error(g_backend, r));
    return TTB_OK;
}

int32_t ttb_comm_init(void **comm, int32_t ranks, int32_t rank, const void *unique_id, int64_t timeout_ms) {
    if (!comm || !unique_id) return fail(TTB_E_INVALID, "ttb_comm_init: null pointer");
    *comm = nullptr;
    if (ranks < 1 || ranks > TTB_MAX_RANKS) return fail(TTB_E_INVALID, "ttb_comm_init: ranks must be 1..%d, got %d", TTB_MAX_RANKS, ranks);
    if (rank < 0 || rank >= ranks) return fail(TTB_E_INVALID, "ttb_comm_init: rank %d is outside 0..%d", rank, ranks - 1);
    if (int32_t rc = load_backend()) return rc;
    Comm *c = new Comm();
    c->ranks = ranks;
    c->rank = rank;
    const int r = backend_init(g_backend, &c->handle, ranks, unique_id, rank);
    if (r != kBackendOk && r != kBackendInProgress) {
        delete c;
        return fail(TTB_E_CUDA, "ttb_comm_init: %s", backend_error(g_backend, r));
    }
    if (int32_t rc = wait_ready(c, timeout_ms, "ttb_comm_init")) {
        // a peer never joined, or the set-up failed: nothing of this communicator may be used, so it is aborted here
        if (c->handle) g_backend.abort(c->handle);
        delete c;
        return rc;
    }
    *comm = c;
    return TTB_OK;
}

int32_t ttb_comm_check(void *comm, int64_t timeout_ms) {
    Comm *c = static_cast<Comm *>(comm);
    if (!c || !c->handle) return fail(TTB_E_INVALID, "ttb_comm_check: null communicator");
    if (c->aborted) return fail(TTB_E_INVALID, "ttb_comm_check: the communicator was aborted");
    return wait_ready(c, timeout_ms, "ttb_comm_check");
}

int32_t ttb_all_gather(void *comm, const void *src_dev, void *dst_dev, int64_t bytes_per_rank, void *stream) {
    Comm *c = static_cast<Comm *>(comm);
    if (!c || !c->handle) return fail(TTB_E_INVALID, "ttb_all_gather: null communicator");
    if (c->aborted) return fail(TTB_E_INVALID, "ttb_all_gather: the communicator was aborted");
    if (!src_dev || !dst_dev || bytes_per_rank <= 0) return fail(TTB_E_INVALID, "ttb_all_gather: null buffer or empty shard");
    // element type ncclUint8: the gather moves bytes; tiled shards of one tile row and row-major shards both are whole
    // byte runs per rank (the [rows > 1] case is re-ordered afterwards by ttb_gather_interleave)
    const int r = g_backend.all_gather(src_dev, dst_dev, (size_t)bytes_per_rank, (int)ncclUint8, c->handle, stream);
    if (r == kBackendInProgress) return wait_ready(c, 10000, "ttb_all_gather");   // non-blocking communicator: enqueue still running
    if (r != kBackendOk) return fail(TTB_E_CUDA, "ttb_all_gather: %s", backend_error(g_backend, r));
    return TTB_OK;
}

int32_t ttb_comm_abort(void *comm) {
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return TTB_OK;
    int r = kBackendOk;
    if (c->handle && !c->aborted) r = g_backend.abort(c->handle);
    c->aborted = true;
    c->handle = nullptr;
    delete c;
    if (r != kBackendOk) return fail(TTB_E_CUDA, "ttb_comm_abort: %s", backend_error(g_backend, r));
    return TTB_OK;
}

int32_t ttb_comm_destroy(void *comm) {
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return TTB_OK;
    int r = kBackendOk;
    if (c->handle && !c->aborted) r = g_backend.destroy(c->handle);
    delete c;
    if (r != kBackendOk) return fail(TTB_E_CUDA, "ttb_comm_destroy: %s", backend_error(g_backend, r));
    return TTB_OK;
}

}  // extern "C"
