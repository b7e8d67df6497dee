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
// groups that fill the SMs about once; inside a group the heaviest blocks of every unit come first
// (rank 0 = heaviest under a causal mask). CTAs that run at the same time then belong to a few
// units, whose K and V (a few MB) stay in L2 while all the blocks of the unit stream them, instead
// of every resident CTA streaming a different unit's tensors from HBM.
struct WorkOrder {
    int units;   // batch * heads
    int blocks;  // blocks per unit
    int group;   // units per group
};

inline WorkOrder make_work_order(int units, int blocks, int sm_count)
{
    WorkOrder w;
    w.units = units;
    w.blocks = blocks;
    const int sms = sm_count > 0 ? sm_count : 148;
    w.group = (sms + blocks - 1) / blocks;
    if (w.group < 1) w.group = 1;
    if (w.group > units) w.group = units;
    return w;
}

#ifdef __CUDACC__
__device__ __forceinline__ void work_item(const WorkOrder &w, int idx, int &unit, int &rank)
{
    const int per_group = w.group * w.blocks;
    const int g = idx / per_group, rem = idx - g * per_group;
    const int units_here = min(w.group, w.units - g * w.group);
    rank = rem / units_here;
    unit = g * w.group + (rem - rank * units_here);
}
#endif

inline size_t dtype_size(int dtype) { return dtype == EMBER_BF16 ? 2 : 4; }

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace ember
