// Optional gather of the per-rank output slabs into one full tensor on every rank.
//
// The attention path shards over (batch * head) with no exchange in forward or backward; the only
// communication a caller may ask for is "give me the whole output on one rank". That is one
// ncclAllGather over equal slabs (NVLink / NVSwitch inside a box). The reference has no
// communication layer at all (its CMakeLists.txt:63,102 link only cuBLAS), so these entry points have
// no counterpart there.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy a host framework has already loaded
// if there is one), so the attention library itself carries no link-time dependency on it and
// single-GPU users never load it. No kernel of this library reads another GPU's memory.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <time.h>

#include "common.cuh"

using namespace ember;

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommFinalize)(ncclComm_t) = nullptr;  // optional (NCCL >= 2.14)
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi g_nccl;

template <typename F>
bool bind(F &fn, const char *name)
{
    fn = reinterpret_cast<F>(dlsym(g_nccl.handle, name));
    if (!fn) set_error("NCCL symbol %s not found: %s", name, dlerror());
    return fn != nullptr;
}

int load_nccl()
{
    if (g_nccl.ok) return EMBER_OK;
    if (!g_nccl.handle) {
        const char *env = getenv("EMBER_NCCL_LIB");
        const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (!n || !n[0]) continue;
            g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (g_nccl.handle) break;
        }
        if (!g_nccl.handle) {
            set_error("cannot load NCCL (libnccl.so.2): %s; set EMBER_NCCL_LIB to its path", dlerror());
            return EMBER_ERR_UNSUPPORTED;
        }
    }
    if (!bind(g_nccl.GetUniqueId, "ncclGetUniqueId") || !bind(g_nccl.CommInitRankConfig, "ncclCommInitRankConfig") ||
        !bind(g_nccl.CommGetAsyncError, "ncclCommGetAsyncError") || !bind(g_nccl.CommAbort, "ncclCommAbort") ||
        !bind(g_nccl.CommDestroy, "ncclCommDestroy") || !bind(g_nccl.AllGather, "ncclAllGather") ||
        !bind(g_nccl.GetErrorString, "ncclGetErrorString"))
        return EMBER_ERR_UNSUPPORTED;
    g_nccl.CommFinalize = reinterpret_cast<decltype(g_nccl.CommFinalize)>(dlsym(g_nccl.handle, "ncclCommFinalize"));
    g_nccl.ok = true;
    return EMBER_OK;
}

int nccl_fail(ncclResult_t r, const char *what)
{
    set_error("NCCL error %d (%s) in %s", (int)r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
    return EMBER_ERR_CUDA;
}

double now_ms()
{
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return t.tv_sec * 1e3 + t.tv_nsec * 1e-6;
}

}  // namespace

extern "C" {

int ember_comm_unique_id(void *id_out)
{
    EMBER_REQUIRE(id_out != nullptr, "ember_comm_unique_id: NULL argument");
    static_assert(sizeof(ncclUniqueId) == EMBER_COMM_ID_BYTES, "id size");
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id_out, &id, sizeof(id));
    return EMBER_OK;
}

int ember_comm_init(void **comm, const void *id, int rank, int world, int timeout_ms)
{
    EMBER_REQUIRE(comm && id, "ember_comm_init: NULL argument");
    EMBER_REQUIRE(world > 0 && rank >= 0 && rank < world, "ember_comm_init: bad rank %d of %d", rank, world);
    *comm = nullptr;
    int rc = load_nccl();
    if (rc) return rc;
    if (!device_state()) return EMBER_ERR_CUDA;
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    // Non-blocking initialisation, polled from the host: a rank that never arrives makes this call
    // return EMBER_ERR_TIMEOUT after timeout_ms (the half-built communicator is aborted) instead of
    // blocking forever. timeout_ms <= 0 waits without limit.
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    ncclComm_t c = nullptr;
    ncclResult_t r = g_nccl.CommInitRankConfig(&c, world, uid, rank, &cfg);
    const double t0 = now_ms();
    while (r == ncclInProgress) {
        if (timeout_ms > 0 && now_ms() - t0 > timeout_ms) {
            if (c) g_nccl.CommAbort(c);
            set_error("ember_comm_init: rank %d of %d gave up after %d ms waiting for the other ranks", rank, world, timeout_ms);
            return EMBER_ERR_TIMEOUT;
        }
        timespec nap = {0, 1000000};
        nanosleep(&nap, nullptr);
        ncclResult_t q = g_nccl.CommGetAsyncError(c, &r);
        if (q != ncclSuccess) return nccl_fail(q, "ncclCommGetAsyncError");
    }
    if (r != ncclSuccess) {
        if (c) g_nccl.CommAbort(c);
        return nccl_fail(r, "ncclCommInitRankConfig");
    }
    *comm = c;
    return EMBER_OK;
}

int ember_comm_destroy(void *comm)
{
    if (!comm) return EMBER_OK;
    int rc = load_nccl();
    if (rc) return rc;
    // The communicator is non-blocking: finish what is still queued on it first (polled), then destroy.
    ncclComm_t c = (ncclComm_t)comm;
    if (g_nccl.CommFinalize) {
        ncclResult_t f = g_nccl.CommFinalize(c);
        const double t0 = now_ms();
        while (f == ncclInProgress && now_ms() - t0 < 60000.0) {
            timespec nap = {0, 1000000};
            nanosleep(&nap, nullptr);
            if (g_nccl.CommGetAsyncError(c, &f) != ncclSuccess) break;
        }
    }
    ncclResult_t r = g_nccl.CommDestroy(c);
    return (r == ncclSuccess || r == ncclInProgress) ? EMBER_OK : nccl_fail(r, "ncclCommDestroy");
}

int ember_gather_outputs(void *out_full, const void *out_slab, size_t slab_bytes, void *comm, void *stream)
{
    EMBER_REQUIRE(out_full && out_slab && comm, "ember_gather_outputs: NULL argument");
    int rc = load_nccl();
    if (rc) return rc;
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    if (slab_bytes == 0) return EMBER_OK;
    ncclComm_t c = (ncclComm_t)comm;
    ncclResult_t r = g_nccl.AllGather(out_slab, out_full, slab_bytes, ncclInt8, c, pick_stream(stream, st));
    // the communicator is non-blocking: the enqueue may still be in progress when the call returns
    while (r == ncclInProgress) {
        ncclResult_t q = g_nccl.CommGetAsyncError(c, &r);
        if (q != ncclSuccess) return nccl_fail(q, "ncclCommGetAsyncError");
    }
    return r == ncclSuccess ? EMBER_OK : nccl_fail(r, "ncclAllGather");
}

}  // extern "C"
