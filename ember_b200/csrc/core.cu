// Device-buffer / stream plumbing of the attention library: the five memory entry points the
// reference declares in src/core/memory.h:10-14, re-implemented stream-ordered, plus device
// selection, bf16 conversion and status reporting.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"
#include "ptx.cuh"

namespace ember {

static thread_local char g_err[512] = "";
static const int kMaxDevices = 64;
static DeviceState g_dev[kMaxDevices];

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what)
{
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return e == cudaErrorMemoryAllocation ? EMBER_ERR_NOMEM : EMBER_ERR_CUDA;
}

DeviceState *device_state()
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDevice");
        return nullptr;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device index %d out of range", dev);
        return nullptr;
    }
    DeviceState *st = &g_dev[dev];
    if (st->ready) return st;
    if ((e = cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking)) != cudaSuccess) {
        cuda_fail(e, "cudaStreamCreateWithFlags");
        return nullptr;
    }
    if ((e = cudaMalloc(&st->status, sizeof(DeviceStatus))) != cudaSuccess ||
        (e = cudaMemset(st->status, 0, sizeof(DeviceStatus))) != cudaSuccess) {
        cuda_fail(e, "status word allocation");
        return nullptr;
    }
    cudaDeviceGetAttribute(&st->sm_count, cudaDevAttrMultiProcessorCount, dev);
    // Keep freed blocks in the pool instead of returning them to the driver at every sync.
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
        uint64_t thr = UINT64_MAX;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thr);
    }
    st->ready = true;
    return st;
}

template <typename In, typename Out>
__global__ void convert_kernel(const In *__restrict__ src, Out *__restrict__ dst, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        if constexpr (sizeof(In) == 4)
            dst[i] = __float2bfloat16_rn(src[i]);
        else
            dst[i] = __bfloat162float(src[i]);
    }
}

// One warp waits on an mbarrier that nothing ever arrives at, with a limit of about a millisecond:
// the bounded wait gives up, records EMBER_ERR_TIMEOUT with wait code 9001 in the status word and
// the kernel returns normally. Exercises the failure path of every kernel's waits without a fault.
__global__ void selftest_wait_timeout_kernel(DeviceStatus *status)
{
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ int abort_flag;
    const uint32_t bar = ptx::smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(bar, 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    ptx::mbar_wait(bar, 0, &abort_flag, status, 9001, 2LL * 1000 * 1000);
}

}  // namespace ember

using namespace ember;

extern "C" {

void *alloc_memory(size_t bytes)
{
    DeviceState *st = device_state();
    if (!st) return nullptr;
    void *p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, bytes ? bytes : 1, st->stream);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaMallocAsync");
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void free_memory(void *ptr)
{
    if (!ptr) return;
    DeviceState *st = device_state();
    if (!st) return;
    cudaFreeAsync(ptr, st->stream);
}

void copy_to_device(void *dst_device, const void *src_host, size_t bytes)
{
    DeviceState *st = device_state();
    if (!st) return;
    cudaError_t e = cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, st->stream);
    // The reference's copy is synchronous (src/core/memory_gpu.cu:32) and callers may reuse src as
    // soon as the call returns. A pageable source has been staged by then, so nothing more is
    // needed and uploads of several tensors queue up behind one another; a pinned (or managed)
    // source is read by the DMA engine later, so wait for it.
    if (e == cudaSuccess) {
        cudaPointerAttributes attr;
        const bool pageable = cudaPointerGetAttributes(&attr, src_host) == cudaSuccess && attr.type == cudaMemoryTypeUnregistered;
        cudaGetLastError();  // older runtimes report an error for plain host pointers
        if (!pageable) e = cudaStreamSynchronize(st->stream);
    }
    if (e != cudaSuccess) cuda_fail(e, "copy_to_device");
}

void *ember_alloc_async(size_t bytes, void *stream)
{
    DeviceState *st = device_state();
    if (!st) return nullptr;
    void *p = nullptr;
    cudaError_t e = cudaMallocAsync(&p, bytes ? bytes : 1, pick_stream(stream, st));
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaMallocAsync");
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

int ember_free_async(void *ptr, void *stream)
{
    if (!ptr) return EMBER_OK;
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    EMBER_CUDA_TRY(cudaFreeAsync(ptr, pick_stream(stream, st)));
    return EMBER_OK;
}

int ember_pool_stats(size_t *reserved_bytes, size_t *used_bytes)
{
    int dev = 0;
    EMBER_CUDA_TRY(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    EMBER_CUDA_TRY(cudaDeviceGetDefaultMemPool(&pool, dev));
    uint64_t r = 0, u = 0;
    EMBER_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &r));
    EMBER_CUDA_TRY(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &u));
    if (reserved_bytes) *reserved_bytes = (size_t)r;
    if (used_bytes) *used_bytes = (size_t)u;
    return EMBER_OK;
}

void copy_from_device(void *dst_host, const void *src_device, size_t bytes)
{
    DeviceState *st = device_state();
    if (!st) return;
    cudaError_t e = cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, st->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st->stream);
    if (e != cudaSuccess) cuda_fail(e, "copy_from_device");
}

void sync_device(void)
{
    DeviceState *st = device_state();
    if (!st) return;
    cudaError_t e = cudaStreamSynchronize(st->stream);
    if (e != cudaSuccess) cuda_fail(e, "sync_device");
}

int ember_work_order_item(int units, int blocks, int sm_count, size_t touched_bytes_per_unit, int causal, int index,
                          int *unit, int *rank)
{
    EMBER_REQUIRE(units > 0 && blocks > 0 && unit && rank, "ember_work_order_item: bad arguments");
    EMBER_REQUIRE(index >= 0 && (long long)index < (long long)units * blocks, "ember_work_order_item: index %d out of range", index);
    const WorkOrder w = make_work_order(units, blocks, sm_count, touched_bytes_per_unit, causal != 0);
    work_item(w, index, *unit, *rank);
    return EMBER_OK;
}

int ember_set_device(int device)
{
    EMBER_CUDA_TRY(cudaSetDevice(device));
    return device_state() ? EMBER_OK : EMBER_ERR_CUDA;
}

int ember_get_device(int *device)
{
    EMBER_REQUIRE(device != nullptr, "ember_get_device: NULL argument");
    EMBER_CUDA_TRY(cudaGetDevice(device));
    return EMBER_OK;
}

void *ember_stream(void)
{
    DeviceState *st = device_state();
    return st ? (void *)st->stream : nullptr;
}

int ember_f32_to_bf16(const float *src, void *dst, size_t n, void *stream)
{
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    EMBER_REQUIRE(src && dst, "ember_f32_to_bf16: NULL pointer");
    if (n == 0) return EMBER_OK;
    int blocks = (int)((n + 255) / 256 < (size_t)st->sm_count * 16 ? (n + 255) / 256 : (size_t)st->sm_count * 16);
    convert_kernel<float, __nv_bfloat16><<<blocks, 256, 0, pick_stream(stream, st)>>>(src, (__nv_bfloat16 *)dst, n);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

int ember_bf16_to_f32(const void *src, float *dst, size_t n, void *stream)
{
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    EMBER_REQUIRE(src && dst, "ember_bf16_to_f32: NULL pointer");
    if (n == 0) return EMBER_OK;
    int blocks = (int)((n + 255) / 256 < (size_t)st->sm_count * 16 ? (n + 255) / 256 : (size_t)st->sm_count * 16);
    convert_kernel<__nv_bfloat16, float><<<blocks, 256, 0, pick_stream(stream, st)>>>((const __nv_bfloat16 *)src, dst, n);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

const char *ember_status_string(int status)
{
    switch (status) {
        case EMBER_OK: return "ok";
        case EMBER_ERR_INVALID: return "invalid argument";
        case EMBER_ERR_UNSUPPORTED: return "unsupported configuration";
        case EMBER_ERR_CUDA: return "CUDA error";
        case EMBER_ERR_TIMEOUT: return "device-side wait timed out";
        case EMBER_ERR_NOMEM: return "out of device memory";
        case EMBER_ERR_WORKSPACE: return "workspace missing or too small";
        default: return "unknown status";
    }
}

const char *ember_last_error(void) { return g_err; }

int ember_selftest_wait_timeout(void *stream)
{
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    selftest_wait_timeout_kernel<<<1, 32, 0, pick_stream(stream, st)>>>(st->status);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

int ember_check_device_status(void *stream, int *where)
{
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    DeviceStatus h;
    EMBER_CUDA_TRY(cudaMemcpyAsync(&h, st->status, sizeof(h), cudaMemcpyDeviceToHost, s));
    EMBER_CUDA_TRY(cudaStreamSynchronize(s));
    if (where) *where = h.where;
    if (h.code != 0) {
        set_error("device-side wait gave up: where=%d block=%d extra=%d", h.where, h.block, h.extra);
        EMBER_CUDA_TRY(cudaMemsetAsync(st->status, 0, sizeof(DeviceStatus), s));
        EMBER_CUDA_TRY(cudaStreamSynchronize(s));
        return EMBER_ERR_TIMEOUT;
    }
    return EMBER_OK;
}

}  // extern "C"
