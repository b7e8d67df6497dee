// Single-query decode against a long key/value cache: out = softmax(q K^T * scale) V with one
// query row per (batch*head). The work is one pass over K and V (arithmetic intensity about one
// flop per byte), so the kernel is shaped for HBM bandwidth, not for the tensor cores:
//
//   - the key axis of every (batch*head) is cut into `splits` contiguous chunks; one CTA streams
//     one chunk with 16-byte read-only, no-L1-allocate loads (nothing is read twice);
//   - a key row of d elements is spread over LPK lanes (16 bytes per lane), so one warp-wide load
//     covers 32/LPK consecutive keys = 512 contiguous bytes, and each warp keeps UNROLL such loads
//     of K and of V in flight;
//   - each lane group keeps its own running (max, sum, partial output) in registers in the exp2
//     domain; groups are merged by warp shuffles, warps through shared memory;
//   - with more than one split, per-split (max, sum, output) partials go to a float32 workspace
//     and a second kernel merges them by log-sum-exp.
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

namespace ember {

namespace {

constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int UNROLL = 4;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint4 ld_stream(const void *p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <typename T>
struct Vec;  // 16 bytes of T unpacked to floats
template <>
struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&f)[8])
    {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&f)[4])
    {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
};

// Merge (m2, l2, o2) into (m, l, o): both are partial softmax states in the exp2 domain.
template <int N>
__device__ __forceinline__ void merge_state(float &m, float &l, float (&o)[N], float m2, float l2,
                                            const float (&o2)[N])
{
    const float mn = fmaxf(m, m2);
    const float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    const float b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
    l = l * a + l2 * b;
#pragma unroll
    for (int i = 0; i < N; i++) o[i] = o[i] * a + o2[i] * b;
    m = mn;
}

// One-dimensional grid of bh * splits blocks (the splits of one row are neighbours). LPK lanes
// share one key row; lanes whose column offset is >= d idle.
template <typename T, int LPK>
__global__ void __launch_bounds__(DEC_THREADS)
    decode_split_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                        T *__restrict__ out, float *__restrict__ lse, float *__restrict__ ws_o,
                        float *__restrict__ ws_ml, int lk, int d, int chunk, int splits,
                        float scale_log2)
{
    constexpr int N = Vec<T>::N;
    constexpr int KPW = 32 / LPK;  // keys per warp-wide load
    const size_t bh = blockIdx.x / splits;
    const int split = blockIdx.x - (unsigned)bh * splits;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = lane / LPK;       // key slot inside the warp
    const int col = (lane % LPK) * N;  // first column this lane owns
    const bool col_ok = col < d;

    const int kbeg = split * chunk;
    const int kend = min(lk, kbeg + chunk);

    const T *kb = k + bh * (size_t)lk * d;
    const T *vb = v + bh * (size_t)lk * d;

    float qf[N];
    {
        uint4 qu = make_uint4(0, 0, 0, 0);
        if (col_ok) qu = *reinterpret_cast<const uint4 *>(q + bh * d + col);
        Vec<T>::unpack(qu, qf);
#pragma unroll
        for (int i = 0; i < N; i++) qf[i] *= scale_log2;
    }

    float m = -INFINITY, l = 0.f, o[N];
#pragma unroll
    for (int i = 0; i < N; i++) o[i] = 0.f;

    for (int base = kbeg + warp * (KPW * UNROLL); base < kend; base += DEC_WARPS * KPW * UNROLL) {
        uint4 ku[UNROLL], vu[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int key = base + u * KPW + g;
            ok[u] = key < kend;
            ku[u] = make_uint4(0, 0, 0, 0);
            vu[u] = make_uint4(0, 0, 0, 0);
            if (ok[u] && col_ok) {
                ku[u] = ld_stream(kb + (size_t)key * d + col);
                vu[u] = ld_stream(vb + (size_t)key * d + col);
            }
        }
        float s[UNROLL];
        float mx = m;
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            float kf[N];
            Vec<T>::unpack(ku[u], kf);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < N; i++) acc = fmaf(qf[i], kf[i], acc);
#pragma unroll
            for (int off = LPK / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            s[u] = ok[u] ? acc : -INFINITY;
            mx = fmaxf(mx, s[u]);
        }
        // A slot that has seen no key yet keeps m == -inf; use 0 as its reference so that no
        // inf - inf appears (every lane must reach the shuffles of the next iteration together,
        // so there is no early continue here).
        const float mref = (mx == -INFINITY) ? 0.f : mx;
        const float alpha = exp2f(m - mref);  // m == -inf gives 0
        m = mx;
        l *= alpha;
#pragma unroll
        for (int i = 0; i < N; i++) o[i] *= alpha;
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const float p = exp2f(s[u] - mref);  // -inf gives 0
            l += p;
            float vf[N];
            Vec<T>::unpack(vu[u], vf);
#pragma unroll
            for (int i = 0; i < N; i++) o[i] = fmaf(p, vf[i], o[i]);
        }
    }

    // merge the KPW key slots of this warp
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
        const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
        float o2[N];
#pragma unroll
        for (int i = 0; i < N; i++) o2[i] = __shfl_xor_sync(0xffffffffu, o[i], off);
        merge_state<N>(m, l, o, m2, l2, o2);
    }

    // merge the warps through shared memory
    __shared__ float sm_o[DEC_WARPS][LPK * N];
    __shared__ float sm_ml[DEC_WARPS][2];
    if (lane < LPK) {
#pragma unroll
        for (int i = 0; i < N; i++) sm_o[warp][col + i] = o[i];
        if (lane == 0) {
            sm_ml[warp][0] = m;
            sm_ml[warp][1] = l;
        }
    }
    __syncthreads();
    if (warp == 0 && lane < LPK) {
#pragma unroll
        for (int w = 1; w < DEC_WARPS; w++) {
            float o2[N];
#pragma unroll
            for (int i = 0; i < N; i++) o2[i] = sm_o[w][col + i];
            merge_state<N>(m, l, o, sm_ml[w][0], sm_ml[w][1], o2);
        }
        if (splits == 1) {
            const float inv = 1.f / l;
            if (col_ok) {
#pragma unroll
                for (int i = 0; i < N; i++) {
                    if constexpr (sizeof(T) == 4)
                        out[bh * d + col + i] = o[i] * inv;
                    else
                        out[bh * d + col + i] = __float2bfloat16_rn(o[i] * inv);
                }
            }
            if (lse && lane == 0) lse[bh] = (m + log2f(l)) * LN2;
        } else {
            float *po = ws_o + (bh * splits + split) * (size_t)d;
            if (col_ok) {
#pragma unroll
                for (int i = 0; i < N; i++) po[col + i] = o[i];
            }
            if (lane == 0) {
                ws_ml[(bh * splits + split) * 2] = m;
                ws_ml[(bh * splits + split) * 2 + 1] = l;
            }
        }
    }
}

// One block per (batch*head); thread c merges column c over the splits.
template <typename T>
__global__ void decode_combine_kernel(const float *__restrict__ ws_o, const float *__restrict__ ws_ml,
                                      T *__restrict__ out, float *__restrict__ lse, int d, int splits)
{
    const size_t bh = blockIdx.x;
    const float *ml = ws_ml + bh * splits * 2;
    float mx = -INFINITY;
    for (int s = 0; s < splits; s++) mx = fmaxf(mx, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < splits; s++) {
        const float ms = ml[2 * s];
        if (ms != -INFINITY) l += ml[2 * s + 1] * exp2f(ms - mx);
    }
    const float inv = 1.f / l;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) acc += ws_o[(bh * splits + s) * (size_t)d + c] * exp2f(ms - mx);
        }
        if constexpr (sizeof(T) == 4)
            out[bh * d + c] = acc * inv;
        else
            out[bh * d + c] = __float2bfloat16_rn(acc * inv);
    }
    if (lse && threadIdx.x == 0) lse[bh] = (mx + log2f(l)) * LN2;
}

template <typename T, int LPK>
int launch_decode(const AttnArgs &a, int splits, int chunk, float *ws_o, float *ws_ml, cudaStream_t s)
{
    const unsigned grid = (unsigned)((long long)splits * a.bh);
    decode_split_kernel<T, LPK><<<grid, DEC_THREADS, 0, s>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (T *)a.out, a.lse, ws_o, ws_ml, a.lk, a.d,
        chunk, splits, a.scale * LOG2E);
    EMBER_CUDA_TRY(cudaGetLastError());
    if (splits > 1) {
        decode_combine_kernel<T><<<a.bh, 128, 0, s>>>(ws_o, ws_ml, (T *)a.out, a.lse, a.d, splits);
        EMBER_CUDA_TRY(cudaGetLastError());
    }
    return EMBER_OK;
}

template <typename T>
int dispatch_lpk(const AttnArgs &a, int splits, int chunk, float *ws_o, float *ws_ml, cudaStream_t s)
{
    const int lanes = (a.d + Vec<T>::N - 1) / Vec<T>::N;
    if (lanes <= 2) return launch_decode<T, 2>(a, splits, chunk, ws_o, ws_ml, s);
    if (lanes <= 4) return launch_decode<T, 4>(a, splits, chunk, ws_o, ws_ml, s);
    if (lanes <= 8) return launch_decode<T, 8>(a, splits, chunk, ws_o, ws_ml, s);
    if (lanes <= 16) return launch_decode<T, 16>(a, splits, chunk, ws_o, ws_ml, s);
    return launch_decode<T, 32>(a, splits, chunk, ws_o, ws_ml, s);
}

}  // namespace

// Enough CTAs for ~32 waves at 8 resident CTAs per SM (so the last, partial wave costs a few
// per cent at most), but never chunks shorter than 512 keys.
int decode_pick_splits(int bh, int lk, int d, int dtype, int sm_count)
{
    (void)d;
    (void)dtype;
    if (sm_count <= 0) sm_count = 148;
    const long long want = 32LL * 8 * sm_count;
    long long splits = (want + bh - 1) / bh;
    const long long max_splits = (lk + 511) / 512;
    if (splits > max_splits) splits = max_splits;
    if (splits > 256) splits = 256;
    if (splits < 1) splits = 1;
    return (int)splits;
}

size_t decode_workspace_bytes(int bh, int d, int splits)
{
    if (splits <= 1) return 0;
    return align_up((size_t)bh * splits * d * sizeof(float), 256) +
           align_up((size_t)bh * splits * 2 * sizeof(float), 256);
}

int decode_attention(const AttnArgs &a, int splits, void *workspace, DeviceState *st, cudaStream_t s)
{
    (void)st;
    const int vec = a.dtype == EMBER_BF16 ? 8 : 4;
    if (a.d % vec != 0 || a.d > 32 * vec) {
        set_error("decode: head dimension %d must be a multiple of %d and at most %d", a.d, vec, 32 * vec);
        return EMBER_ERR_UNSUPPORTED;
    }
    int chunk = (a.lk + splits - 1) / splits;
    chunk = (chunk + 63) / 64 * 64;
    splits = (a.lk + chunk - 1) / chunk;  // drop empty trailing chunks; never exceeds the request
    if ((long long)a.bh * splits > 0x7fffffffLL) {
        set_error("decode: batch*heads %d times %d splits exceeds the grid limit", a.bh, splits);
        return EMBER_ERR_UNSUPPORTED;
    }
    float *ws_o = (float *)workspace;
    float *ws_ml = nullptr;
    if (splits > 1)
        ws_ml = (float *)((char *)workspace + align_up((size_t)a.bh * splits * a.d * sizeof(float), 256));
    if (a.dtype == EMBER_BF16) return dispatch_lpk<__nv_bfloat16>(a, splits, chunk, ws_o, ws_ml, s);
    return dispatch_lpk<float>(a, splits, chunk, ws_o, ws_ml, s);
}

}  // namespace ember

// ------------------------------------------------------------------------------------------------
// Decode without any allocation: the split partials live in a fixed array inside the library image.
// ------------------------------------------------------------------------------------------------
namespace {

// 4 MiB of float32 partials. Every GPU that loads this library carries the array until the process
// exits, so it is kept modest; it bounds batch_heads * splits * (d + 2) (see the entry point).
constexpr size_t kStaticScratchFloats = 1u << 20;
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

// Device address of g_decode_scratch, per device. In host code the array's name is only a handle
// for the runtime, not something a kernel can dereference, so the address is looked up once per
// device with cudaGetSymbolAddress while that device is current.
constexpr int kMaxScratchDevices = 64;
float *g_scratch_addr[kMaxScratchDevices] = {};

size_t static_partials_floats(int bh, int d, int splits)
{
    return ember::decode_workspace_bytes(bh, d, splits) / sizeof(float);
}

}  // namespace

extern "C" EMBER_API int ember_attention_decode_static(const void *q, const void *k, const void *v, void *out,
                                                       float *lse, int batch_heads, int lk, int d, float scale,
                                                       int dtype, int num_splits, void *stream)
{
    using namespace ember;
    EMBER_REQUIRE(dtype == EMBER_F32 || dtype == EMBER_BF16, "ember_attention_decode_static: unknown dtype %d", dtype);
    EMBER_REQUIRE(batch_heads > 0 && lk > 0 && d > 0,
                  "ember_attention_decode_static: extents must be positive, got batch_heads=%d lk=%d d=%d",
                  batch_heads, lk, d);
    EMBER_REQUIRE(isfinite(scale), "ember_attention_decode_static: scale must be finite");
    EMBER_REQUIRE(q && k && v && out, "ember_attention_decode_static: NULL tensor pointer");
    EMBER_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0,
                  "ember_attention_decode_static: q, k and v must be 16-byte aligned");

    int dev = 0;
    EMBER_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxScratchDevices) {
        set_error("ember_attention_decode_static: device index %d out of range", dev);
        return EMBER_ERR_UNSUPPORTED;
    }
    if (!g_scratch_addr[dev]) {  // first call on this device: resolve the array's device address
        float *ptr = nullptr;
        EMBER_CUDA_TRY(cudaGetSymbolAddress((void **)&ptr, g_decode_scratch));
        g_scratch_addr[dev] = ptr;
    }

    int splits = num_splits;
    if (splits <= 0) {
        int sms = 0;
        EMBER_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        splits = decode_pick_splits(batch_heads, lk, d, dtype, sms);
        // the library's own choice shrinks until the partials fit; one split needs no scratch at all
        while (splits > 1 && static_partials_floats(batch_heads, d, splits) > kStaticScratchFloats) splits--;
    }
    if (splits > lk) splits = lk;
    const size_t need = static_partials_floats(batch_heads, d, splits);
    if (need > kStaticScratchFloats) {
        set_error("ember_attention_decode_static: %d splits of %d (batch*head) rows with d=%d need %zu bytes of "
                  "partials, the built-in scratch holds %zu; pass fewer splits or use ember_attention_decode",
                  splits, batch_heads, d, need * sizeof(float), kStaticScratchFloats * sizeof(float));
        return EMBER_ERR_WORKSPACE;
    }
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    a.bh = batch_heads; a.lq = 1; a.lk = lk; a.d = d;
    a.scale = scale; a.causal = 0; a.dtype = dtype;
    return decode_attention(a, splits, g_scratch_addr[dev], nullptr, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" EMBER_API size_t ember_attention_decode_static_capacity(void)
{
    return kStaticScratchFloats * sizeof(float);
}

