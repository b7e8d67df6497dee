// Fused last-axis softmax, log-softmax and softmax cross-entropy (HBM-bound).
//
// The reference composes softmax from five operators (row max, broadcast subtract, exp, row sum,
// broadcast divide: ember/tensor/tensor.py:430-437), each a full pass over the tensor with its own
// allocation, and the cross-entropy loss from eight (ember/loss/losses.py:42-56). Here a row is read
// from HBM once, kept in shared memory as float32 while its maximum and sum are formed, and the
// result is written once: 2 (softmax) or 3 (cross-entropy: logits and targets in, probabilities
// out) element transfers per element instead of about 12 and 20.
//
// A row is owned by a group of W threads: W = 32 while a row is at most 8 KB (8 rows per
// 256-thread block, warp shuffles only, no block-wide barrier), W = 256 up to 64 KB and W = 1024
// beyond (one row per block; long rows need the threads to keep enough loads in flight). The cache
// holds the row in its storage type (a bf16 row needs half the shared memory of its float32 image,
// which decides how many blocks fit on an SM); rows longer than 192 KB are re-read from global memory.
// float32 arithmetic; exponentials are one FMA and one ex2.approx in the exp2 domain (with the accurate
// expf, twice per element, the kernels were bound by instruction issue at a third of the HBM rate). f32 or bf16
// storage; 16-byte vector accesses when the row length and the base addresses allow, element-wise
// accesses otherwise.
#include "common.cuh"
#include "kernels.cuh"

namespace ember {

namespace {

constexpr int BLOCK = 256;                // block size of the element-wise kernels
constexpr int WARP_ROW_MAX_BYTES = 8192;  // rows up to this size are owned by one warp
constexpr int BLOCK_ROW_MAX_BYTES = 65536;  // ... by 256 threads (measured: 64 KB rows run 6-13 % faster on 3 blocks
                                            // of 256 threads per SM than on 2 of 1024; 128 KB rows twice slower); longer rows by 1024
constexpr int CACHE_BYTES = 196608;       // shared memory for one long row

__device__ __forceinline__ float ldf(const float *p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float *p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16 bytes of T <-> NV floats
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
    static constexpr int NV = 4;
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&v)[4])
    {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[4])
    {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    }
};
template <>
struct Vec16<__nv_bfloat16> {
    static constexpr int NV = 8;
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&v)[8])
    {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&v)[8])
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// Reduction over the W threads that own a row. red: 32 floats of shared memory per block (W > 32).
template <int W, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float *red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = IS_MAX ? fmaxf(v, t) : v + t;
    }
    if (W == 32) return v;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    __syncthreads();  // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int i = 1; i < W / 32; i++) r = IS_MAX ? fmaxf(r, red[i]) : r + red[i];
    return r;
}

enum { MODE_SOFTMAX = 0, MODE_LOG_SOFTMAX = 1, MODE_CROSS_ENTROPY = 2 };

// x, y (and target): rows x cols. cache_elems: elements of T cached per row (0 = none: re-read x).
template <typename T, int W, int MODE, bool VEC>
__global__ void __launch_bounds__(W < 256 ? 256 : W) row_softmax_kernel(const T *__restrict__ x, const T *__restrict__ target,
                                                                         T *__restrict__ y, float *__restrict__ row_loss,
                                                                         long long rows, int cols, int cache_elems)
{
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    float *red = reinterpret_cast<float *>(smem_bytes);  // 32 floats
    constexpr int BS = W < 256 ? 256 : W, GROUPS = BS / W, NV = Vec16<T>::NV;
    const int group = threadIdx.x / W, t = threadIdx.x % W;
    T *buf = reinterpret_cast<T *>(smem_bytes + 128) + (size_t)group * cache_elems;
    uint4 *bufv = reinterpret_cast<uint4 *>(buf);
    const bool cached = cache_elems >= cols;
    const int nvec = cols / NV;  // VEC: cols is a multiple of NV

    for (long long row0 = (long long)blockIdx.x * GROUPS; row0 < rows; row0 += (long long)gridDim.x * GROUPS) {
        const long long row = row0 + group;
        const bool active = row < rows;  // W > 32: always true; W == 32: the whole warp agrees
        const T *xr = x + (size_t)(active ? row : 0) * cols;
        const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
        // ---- pass 1: maximum (and fill the cache)
        float m = -INFINITY;
        if (active) {
            if constexpr (VEC) {
#pragma unroll 4
                for (int j = t; j < nvec; j += W) {
                    const uint4 u = xv[j];
                    if (cached) bufv[j] = u;
                    float v[NV];
                    Vec16<T>::unpack(u, v);
#pragma unroll
                    for (int i = 0; i < NV; i++) m = fmaxf(m, v[i]);
                }
            } else {
                for (int j = t; j < cols; j += W) {
                    const T raw = xr[j];
                    if (cached) buf[j] = raw;
                    m = fmaxf(m, ldf(&raw));
                }
            }
        }
        m = group_reduce<W, true>(m, red);
        // exp(x - m) = exp2(x * log2(e) - m * log2(e)): one FMA and one ex2.approx per element
        constexpr float kLog2e = 1.4426950408889634f;
        const float m2 = m * kLog2e;
        // ---- pass 2: sum of exp(x - max)
        float s = 0.f;
        if (active) {
            if constexpr (VEC) {
#pragma unroll 4
                for (int j = t; j < nvec; j += W) {
                    float v[NV];
                    Vec16<T>::unpack(cached ? bufv[j] : xv[j], v);
#pragma unroll
                    for (int i = 0; i < NV; i++) s += fast_exp2(fmaf(v[i], kLog2e, -m2));
                }
            } else {
                for (int j = t; j < cols; j += W) s += fast_exp2(fmaf(ldf(cached ? buf + j : xr + j), kLog2e, -m2));
            }
        }
        s = group_reduce<W, false>(s, red);
        // ---- pass 3: results
        const float inv = 1.f / s, lg = logf(s);
        const float mlg2 = (m + lg) * kLog2e;  // exp(x - m - lg) = exp2(x * log2(e) - mlg2)
        float loss = 0.f;
        if (active) {
            T *yr = y + (size_t)row * cols;
            const T *tr = MODE == MODE_CROSS_ENTROPY ? target + (size_t)row * cols : nullptr;
            if constexpr (VEC) {
                uint4 *yv = reinterpret_cast<uint4 *>(yr);
                const uint4 *tv4 = reinterpret_cast<const uint4 *>(tr);
#pragma unroll 4
                for (int j = t; j < nvec; j += W) {
                    float v[NV], o[NV], tv[NV];
                    Vec16<T>::unpack(cached ? bufv[j] : xv[j], v);
                    if (MODE == MODE_CROSS_ENTROPY) Vec16<T>::unpack(tv4[j], tv);
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        if (MODE == MODE_SOFTMAX) {
                            o[i] = fast_exp2(fmaf(v[i], kLog2e, -m2)) * inv;
                        } else {
                            const float lp = (v[i] - m) - lg;
                            o[i] = MODE == MODE_LOG_SOFTMAX ? lp : fast_exp2(fmaf(v[i], kLog2e, -mlg2));
                            if (MODE == MODE_CROSS_ENTROPY) loss = fmaf(tv[i], lp, loss);
                        }
                    }
                    yv[j] = Vec16<T>::pack(o);
                }
            } else {
                for (int j = t; j < cols; j += W) {
                    const float v = ldf(cached ? buf + j : xr + j);
                    float o;
                    if (MODE == MODE_SOFTMAX) {
                        o = fast_exp2(fmaf(v, kLog2e, -m2)) * inv;
                    } else {
                        const float lp = (v - m) - lg;
                        o = MODE == MODE_LOG_SOFTMAX ? lp : fast_exp2(fmaf(v, kLog2e, -mlg2));
                        if (MODE == MODE_CROSS_ENTROPY) loss = fmaf(ldf(tr + j), lp, loss);
                    }
                    stf(yr + j, o);
                }
            }
        }
        if (MODE == MODE_CROSS_ENTROPY) {
            loss = group_reduce<W, false>(loss, red);
            if (active && t == 0) row_loss[row] = loss;
        }
        if (W > 32) __syncthreads();  // the cache is rewritten by the next row
    }
}

// The same three passes with the row held in REGISTERS: a thread loads its (at most 16) 16-byte pieces
// of the row up front, all of them in flight at once, and maximum, sum and results are computed from
// the registers. For rows of up to W x 256 bytes (W = 32: 8 KB, one warp per row and no block barrier;
// W = 256: 64 KB) this replaces the shared-memory cache of row_softmax_kernel: there a thread has four
// loads in flight during the first pass only, and nothing while it reduces and writes, which left the
// kernels latency-bound at 0.5-0.75 of the copy bandwidth. Two blocks per SM (128 registers per thread)
// so that one block's loads run under the other's arithmetic. 16-byte aligned rows only. MAXV: pieces
// per thread (a power of two up to 16, the smallest that covers the row: loops over pieces that do not
// exist would still cost their issue slots).
template <typename T, int W, int MODE, int MAXV>
__global__ void __launch_bounds__(256, 2) row_softmax_regs_kernel(const T *__restrict__ x, const T *__restrict__ target,
                                                                   T *__restrict__ y, float *__restrict__ row_loss,
                                                                   long long rows, int cols)
{
    __shared__ float red[32];
    constexpr int GROUPS = 256 / W, NV = Vec16<T>::NV;
    constexpr float kLog2e = 1.4426950408889634f;
    const int group = threadIdx.x / W, t = threadIdx.x % W;
    const int nvec = cols / NV;
    for (long long row0 = (long long)blockIdx.x * GROUPS; row0 < rows; row0 += (long long)gridDim.x * GROUPS) {
        const long long row = row0 + group;
        const bool active = row < rows;  // W == 256: always true; W == 32: the whole warp agrees
        const uint4 *xv = reinterpret_cast<const uint4 *>(x + (size_t)(active ? row : 0) * cols);
        uint4 raw[MAXV];
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            const int j = t + i * W;
            if (active && j < nvec) raw[i] = xv[j];
        }
        // ---- maximum
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            if (active && t + i * W < nvec) {
                float v[NV];
                Vec16<T>::unpack(raw[i], v);
#pragma unroll
                for (int k = 0; k < NV; k++) m = fmaxf(m, v[k]);
            }
        }
        m = group_reduce<W, true>(m, red);
        const float m2 = m * kLog2e;
        // ---- sum of exp(x - max)
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < MAXV; i++) {
            if (active && t + i * W < nvec) {
                float v[NV];
                Vec16<T>::unpack(raw[i], v);
#pragma unroll
                for (int k = 0; k < NV; k++) s += fast_exp2(fmaf(v[k], kLog2e, -m2));
            }
        }
        s = group_reduce<W, false>(s, red);
        // ---- results
        const float inv = 1.f / s, lg = logf(s);
        const float mlg2 = (m + lg) * kLog2e;  // exp(x - m - lg) = exp2(x * log2(e) - mlg2)
        float loss = 0.f;
        if (active) {
            uint4 *yv = reinterpret_cast<uint4 *>(y + (size_t)row * cols);
            const uint4 *tv4 = MODE == MODE_CROSS_ENTROPY ? reinterpret_cast<const uint4 *>(target + (size_t)row * cols) : nullptr;
            // cross-entropy: the targets are fetched four pieces at a time (the registers hold the row),
            // one group ahead of the group being computed
            constexpr int TB = MAXV < 4 ? MAXV : 4;
            uint4 tnext[TB];
            if (MODE == MODE_CROSS_ENTROPY) {
#pragma unroll
                for (int i = 0; i < TB; i++)
                    if (t + i * W < nvec) tnext[i] = tv4[t + i * W];
            }
#pragma unroll
            for (int i0 = 0; i0 < MAXV; i0 += TB) {
                uint4 traw[TB];
                if (MODE == MODE_CROSS_ENTROPY) {
#pragma unroll
                    for (int i = 0; i < TB; i++) traw[i] = tnext[i];
                    if (i0 + TB < MAXV) {
#pragma unroll
                        for (int i = 0; i < TB; i++)
                            if (t + (i0 + TB + i) * W < nvec) tnext[i] = tv4[t + (i0 + TB + i) * W];
                    }
                }
#pragma unroll
                for (int i = 0; i < TB; i++) {
                    const int j = t + (i0 + i) * W;
                    if (j < nvec) {
                        float v[NV], o[NV], tv[NV];
                        Vec16<T>::unpack(raw[i0 + i], v);
                        if (MODE == MODE_CROSS_ENTROPY) Vec16<T>::unpack(traw[i], tv);
#pragma unroll
                        for (int k = 0; k < NV; k++) {
                            if (MODE == MODE_SOFTMAX) {
                                o[k] = fast_exp2(fmaf(v[k], kLog2e, -m2)) * inv;
                            } else {
                                const float lp = (v[k] - m) - lg;
                                o[k] = MODE == MODE_LOG_SOFTMAX ? lp : fast_exp2(fmaf(v[k], kLog2e, -mlg2));
                                if (MODE == MODE_CROSS_ENTROPY) loss = fmaf(tv[k], lp, loss);
                            }
                        }
                        yv[j] = Vec16<T>::pack(o);
                    }
                }
            }
        }
        if (MODE == MODE_CROSS_ENTROPY) {
            loss = group_reduce<W, false>(loss, red);
            if (active && t == 0) row_loss[row] = loss;
        }
    }
}

// loss = -(sum of the row losses) / rows, added in a fixed order.
__global__ void __launch_bounds__(BLOCK) loss_finalize_kernel(const float *row_loss, long long rows, float *loss)
{
    __shared__ float red[BLOCK];
    float s = 0.f;
    for (long long r = threadIdx.x; r < rows; r += BLOCK) s += row_loss[r];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = BLOCK / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = -red[0] / (float)rows;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(BLOCK) ce_backward_kernel(const T *__restrict__ probs, const T *__restrict__ target,
                                                            T *__restrict__ grad, size_t total, float inv_n)
{
    constexpr int NV = Vec16<T>::NV;
    if constexpr (VEC) {
        const uint4 *pv = reinterpret_cast<const uint4 *>(probs), *tv = reinterpret_cast<const uint4 *>(target);
        uint4 *gv = reinterpret_cast<uint4 *>(grad);
        const size_t nvec = total / NV;
        for (size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x; i < nvec; i += (size_t)gridDim.x * BLOCK) {
            float p[NV], t[NV], g[NV];
            Vec16<T>::unpack(pv[i], p);
            Vec16<T>::unpack(tv[i], t);
#pragma unroll
            for (int k = 0; k < NV; k++) g[k] = (p[k] - t[k]) * inv_n;
            gv[i] = Vec16<T>::pack(g);
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x; i < total; i += (size_t)gridDim.x * BLOCK)
            stf(grad + i, (ldf(probs + i) - ldf(target + i)) * inv_n);
    }
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

template <typename T, int MODE>
int launch_rows(const T *x, const T *target, T *y, float *row_loss, long long rows, int cols, int sm_count,
                cudaStream_t s)
{
    constexpr int NV = Vec16<T>::NV;
    const bool vec = cols % NV == 0 && aligned16(x) && aligned16(y) && (MODE != MODE_CROSS_ENTROPY || aligned16(target));
    const size_t row_bytes = (size_t)cols * sizeof(T);
    const int width = row_bytes <= WARP_ROW_MAX_BYTES ? 32 : (row_bytes <= BLOCK_ROW_MAX_BYTES ? 256 : 1024);
    if (vec && width <= 256) {  // the row fits the registers of the threads that own it
        const int groups_r = 256 / width;
        const long long need_r = (rows + groups_r - 1) / groups_r;
        const long long cap_r = (long long)(sm_count > 0 ? sm_count : 148) * 16;
        const int grid_r = (int)(need_r < cap_r ? need_r : cap_r);
        const int pieces = (cols / NV + width - 1) / width;  // per thread, at most 16 here
#define EMBER_LAUNCH_REGS(W, NP) row_softmax_regs_kernel<T, W, MODE, NP><<<grid_r, 256, 0, s>>>(x, target, y, row_loss, rows, cols)
#define EMBER_LAUNCH_REGS_W(W)                    \
    do {                                          \
        if (pieces <= 1) EMBER_LAUNCH_REGS(W, 1); \
        else if (pieces <= 2) EMBER_LAUNCH_REGS(W, 2); \
        else if (pieces <= 4) EMBER_LAUNCH_REGS(W, 4); \
        else if (pieces <= 8) EMBER_LAUNCH_REGS(W, 8); \
        else EMBER_LAUNCH_REGS(W, 16);            \
    } while (0)
        if (width == 32) EMBER_LAUNCH_REGS_W(32); else EMBER_LAUNCH_REGS_W(256);
#undef EMBER_LAUNCH_REGS_W
#undef EMBER_LAUNCH_REGS
        EMBER_CUDA_TRY(cudaGetLastError());
        return EMBER_OK;
    }
    const int block = width < 256 ? 256 : width, groups = block / width;
    // per-row cache, rounded up to 16 bytes so that every group's cache stays vector-aligned
    const int cache_elems = row_bytes <= CACHE_BYTES ? (int)(align_up(row_bytes, 16) / sizeof(T)) : 0;
    const size_t smem = 128 + (size_t)groups * cache_elems * sizeof(T);
    const long long blocks_needed = (rows + groups - 1) / groups;
    const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 16;
    const int grid = (int)(blocks_needed < cap ? blocks_needed : cap);
#define EMBER_LAUNCH_ROWS(W, VEC)                                                                               \
    do {                                                                                                        \
        auto kern = row_softmax_kernel<T, W, MODE, VEC>;                                                        \
        EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));     \
        kern<<<grid, block, smem, s>>>(x, target, y, row_loss, rows, cols, cache_elems);                         \
    } while (0)
    if (width == 32) {
        if (vec) EMBER_LAUNCH_ROWS(32, true); else EMBER_LAUNCH_ROWS(32, false);
    } else if (width == 256) {
        if (vec) EMBER_LAUNCH_ROWS(256, true); else EMBER_LAUNCH_ROWS(256, false);
    } else {
        if (vec) EMBER_LAUNCH_ROWS(1024, true); else EMBER_LAUNCH_ROWS(1024, false);
    }
#undef EMBER_LAUNCH_ROWS
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

int check_rows(const char *fn, long long rows, int cols, int dtype)
{
    EMBER_REQUIRE(dtype == EMBER_F32 || dtype == EMBER_BF16, "%s: unknown dtype %d", fn, dtype);
    EMBER_REQUIRE(rows > 0 && cols > 0, "%s: extents must be positive, got rows=%lld cols=%d", fn, rows, cols);
    return EMBER_OK;
}

}  // namespace

}  // namespace ember

using namespace ember;

extern "C" {

int ember_softmax_fwd(const void *x, void *y, long long rows, int cols, int dtype, int log_softmax, void *stream)
{
    int rc = check_rows("ember_softmax_fwd", rows, cols, dtype);
    if (rc) return rc;
    EMBER_REQUIRE(x && y, "ember_softmax_fwd: NULL tensor pointer");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    if (dtype == EMBER_BF16) {
        auto xp = (const __nv_bfloat16 *)x;
        auto yp = (__nv_bfloat16 *)y;
        return log_softmax ? launch_rows<__nv_bfloat16, MODE_LOG_SOFTMAX>(xp, nullptr, yp, nullptr, rows, cols, st->sm_count, s)
                           : launch_rows<__nv_bfloat16, MODE_SOFTMAX>(xp, nullptr, yp, nullptr, rows, cols, st->sm_count, s);
    }
    auto xp = (const float *)x;
    auto yp = (float *)y;
    return log_softmax ? launch_rows<float, MODE_LOG_SOFTMAX>(xp, nullptr, yp, nullptr, rows, cols, st->sm_count, s)
                       : launch_rows<float, MODE_SOFTMAX>(xp, nullptr, yp, nullptr, rows, cols, st->sm_count, s);
}

size_t ember_cross_entropy_workspace_bytes(long long rows)
{
    return rows > 0 ? align_up((size_t)rows * sizeof(float), 256) : 0;
}

int ember_cross_entropy_fwd(const void *pred, const void *target, void *probs, float *loss, long long rows, int cols,
                            int dtype, void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_rows("ember_cross_entropy_fwd", rows, cols, dtype);
    if (rc) return rc;
    EMBER_REQUIRE(pred && target && probs && loss, "ember_cross_entropy_fwd: NULL tensor pointer");
    const size_t need = ember_cross_entropy_workspace_bytes(rows);
    if (!workspace || workspace_bytes < need) {
        set_error("ember_cross_entropy_fwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return EMBER_ERR_WORKSPACE;
    }
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    float *row_loss = (float *)workspace;
    if (dtype == EMBER_BF16)
        rc = launch_rows<__nv_bfloat16, MODE_CROSS_ENTROPY>((const __nv_bfloat16 *)pred, (const __nv_bfloat16 *)target,
                                                           (__nv_bfloat16 *)probs, row_loss, rows, cols, st->sm_count, s);
    else
        rc = launch_rows<float, MODE_CROSS_ENTROPY>((const float *)pred, (const float *)target, (float *)probs, row_loss,
                                                   rows, cols, st->sm_count, s);
    if (rc) return rc;
    loss_finalize_kernel<<<1, BLOCK, 0, s>>>(row_loss, rows, loss);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

int ember_cross_entropy_bwd(const void *probs, const void *target, void *grad, long long rows, int cols, int dtype,
                            void *stream)
{
    int rc = check_rows("ember_cross_entropy_bwd", rows, cols, dtype);
    if (rc) return rc;
    EMBER_REQUIRE(probs && target && grad, "ember_cross_entropy_bwd: NULL tensor pointer");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    const size_t total = (size_t)rows * cols;
    const size_t nv = dtype == EMBER_BF16 ? 8 : 4;
    const bool vec = total % nv == 0 && aligned16(probs) && aligned16(target) && aligned16(grad);
    const size_t per_block = (size_t)BLOCK * (vec ? nv : 1);
    const size_t want = (total + per_block - 1) / per_block;
    const size_t cap = (size_t)(st->sm_count > 0 ? st->sm_count : 148) * 32;
    const int grid = (int)(want < cap ? want : cap);
    const float inv_n = 1.f / (float)rows;
    if (dtype == EMBER_BF16) {
        if (vec) ce_backward_kernel<__nv_bfloat16, true><<<grid, BLOCK, 0, s>>>((const __nv_bfloat16 *)probs, (const __nv_bfloat16 *)target, (__nv_bfloat16 *)grad, total, inv_n);
        else ce_backward_kernel<__nv_bfloat16, false><<<grid, BLOCK, 0, s>>>((const __nv_bfloat16 *)probs, (const __nv_bfloat16 *)target, (__nv_bfloat16 *)grad, total, inv_n);
    } else {
        if (vec) ce_backward_kernel<float, true><<<grid, BLOCK, 0, s>>>((const float *)probs, (const float *)target, (float *)grad, total, inv_n);
        else ce_backward_kernel<float, false><<<grid, BLOCK, 0, s>>>((const float *)probs, (const float *)target, (float *)grad, total, inv_n);
    }
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // extern "C"
