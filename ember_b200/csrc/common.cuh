// Shared host-side plumbing of the attention library: per-device state (stream,
// device status word), error reporting, argument checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/ember_b200.h"

namespace ember {

// Written by device code when a bounded wait gives up. code != 0 means a fault was recorded.
struct DeviceStatus {
    int code;   // ember_status (EMBER_ERR_TIMEOUT)
    int where;  // which wait (kernel-specific code)
    int block;  // linear block index of the first reporter
    int extra;
};

struct DeviceState {
    bool ready = false;
    cudaStream_t stream = nullptr;
    DeviceStatus *status = nullptr;  // device memory
    int sm_count = 0;
    // for the host-tensor entry point: copy streams and the events that chain them (made on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t in_done[2] = {}, compute_done[2] = {}, out_done[2] = {};
};

// State of the current device, created on first use. Returns nullptr and sets the error
// text when CUDA is unusable.
DeviceState *device_state();

void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

inline cudaStream_t pick_stream(void *stream, DeviceState *st)
{
    return stream ? reinterpret_cast<cudaStream_t>(stream) : st->stream;
}

#define EMBER_CUDA_TRY(expr)                                        \
    do {                                                            \
        cudaError_t _e = (expr);                                    \
        if (_e != cudaSuccess) return ::ember::cuda_fail(_e, #expr); \
    } while (0)

#define EMBER_REQUIRE(cond, ...)             \
    do {                                     \
        if (!(cond)) {                       \
            ::ember::set_error(__VA_ARGS__); \
            return EMBER_ERR_INVALID;        \
        }                                    \
    } while (0)

// Order in which the CTAs of the tensor-core kernels take their work. A work item is one block of
// rows (query rows, or key rows in the dK/dV pass) of one (batch*head) unit. Units are taken in
// groups; inside a group the heaviest blocks of every unit come first (rank 0 = heaviest under a
// causal mask), so a group behaves like a longest-job-first schedule. CTAs that run at the same
// time then belong to a few units whose tensors stay in L2 (126 MB) while all the blocks of the unit
// read them, instead of every resident CTA pulling a different unit's K and V from HBM.
// A group always has enough units to fill the SMs once. Without a mask all blocks weigh the same
// and that minimum is used. Under a causal mask larger groups balance better (the heavy blocks of
// the last group start that much earlier), so a group takes as many units as touch about 64 MB, and
// a short last group is merged into the one before it.
struct WorkOrder {
    int units;    // batch * heads
    int blocks;   // blocks per unit
    int group;    // units per group (the last group has units - (ngroups - 1) * group)
    int ngroups;
};

inline WorkOrder make_work_order(int units, int blocks, int sm_count, size_t touched_bytes_per_unit, bool causal)
{
    WorkOrder w;
    w.units = units;
    w.blocks = blocks;
    const int sms = sm_count > 0 ? sm_count : 148;
    long long g = (sms + blocks - 1) / blocks;
    if (causal) {
        const long long by_l2 = (long long)((64ull << 20) / (touched_bytes_per_unit ? touched_bytes_per_unit : 1));
        if (by_l2 > g) g = by_l2;
    }
    if (g < 1) g = 1;
    if (g > units) g = units;
    w.group = (int)g;
    // the last group holds the remainder: merged into the one before it under a causal mask
    w.ngroups = causal ? units / w.group : (units + w.group - 1) / w.group;
    return w;
}

#ifdef __CUDACC__
#define EMBER_HD __host__ __device__ __forceinline__
#else
#define EMBER_HD inline
#endif
EMBER_HD void work_item(const WorkOrder &w, int idx, int &unit, int &rank)
{
    const int per_group = w.group * w.blocks;
    int g = idx / per_group;
    if (g > w.ngroups - 1) g = w.ngroups - 1;
    const int rem = idx - g * per_group;
    const int units_here = (g == w.ngroups - 1) ? w.units - g * w.group : w.group;
    rank = rem / units_here;
    unit = g * w.group + (rem - rank * units_here);
}

// Bounds-checked debug build (-DEMBER_BOUNDS_CHECK, `python -m ember_b200.build --bounds`): every
// global store of the tensor-core attention kernels first checks that [ptr, ptr + len) lies inside the
// tensor it belongs to; a store that does not is skipped and reported through the device status word
// (EMBER_ERR_INVALID, wait code 9100, extra = the byte offset) instead of being made. It stands in for a
// memory checker where none can be run. In the normal build the check is a constant `true`.
#ifdef __CUDACC__
#ifdef EMBER_BOUNDS_CHECK
__device__ __forceinline__ bool store_in_bounds(const void *ptr, const void *base, size_t bytes, size_t len, DeviceStatus *status)
{
    const size_t off = (size_t)((const char *)ptr - (const char *)base);
    if ((const char *)ptr >= (const char *)base && off + len <= bytes) return true;
    if (atomicCAS(&status->code, 0, EMBER_ERR_INVALID) == 0) {
        status->where = 9100;
        status->block = blockIdx.x;
        status->extra = (int)(off > 0x7fffffffu ? 0x7fffffffu : off);
    }
    return false;
}
#define EMBER_STORE_OK(ptr, base, bytes, len, status) ::ember::store_in_bounds(ptr, base, bytes, len, status)
#else
#define EMBER_STORE_OK(ptr, base, bytes, len, status) true
#endif
#endif

inline size_t dtype_size(int dtype) { return dtype == EMBER_BF16 ? 2 : 4; }

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace ember
