// Generic attention kernels on the CUDA cores: float32 arithmetic throughout, float32 or bf16
// storage, any head dimension up to 128, any sequence lengths. They serve the float32 I/O mode
// (whose tolerance against the reference is 1e-3, too tight for bf16 tensor-core products) and
// every bf16 shape the tcgen05 kernels do not cover. Tiling: 64 query rows x 64 keys per step,
// 256 threads, each thread owning a 4x4 patch of the score tile and a 4 x (DPAD/16) patch of
// the output tile. Scores never leave shared memory.
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

namespace ember {

namespace {

constexpr int BM = 64;  // query rows per block / per step
constexpr int BN = 64;  // keys per step
constexpr int NT = 256;

template <typename T>
__device__ __forceinline__ float ld(const T *p)
{
    if constexpr (sizeof(T) == 4)
        return *p;
    else
        return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void st(T *p, float v)
{
    if constexpr (sizeof(T) == 4)
        *p = v;
    else
        *p = __float2bfloat16_rn(v);
}

// Loads rows [row0, row0+64) x cols [0, d) of a (nrows x d) matrix into a [64][DPAD+1] float
// tile; rows past nrows and columns past d are zero.
template <typename T, int DPAD>
__device__ __forceinline__ void load_tile(float *dst, const T *src, int row0, int nrows, int d)
{
    for (int idx = threadIdx.x; idx < 64 * DPAD; idx += NT) {
        int r = idx / DPAD, c = idx % DPAD;
        float v = 0.f;
        if (row0 + r < nrows && c < d) v = ld(src + (size_t)(row0 + r) * d + c);
        dst[r * (DPAD + 1) + c] = v;
    }
}

// acc[r][c] += sum_kk A[ty*4+r][kk] * B[tx+16c][kk], kk < d   (both tiles [64][DPAD+1])
template <int DPAD>
__device__ __forceinline__ void tile_abt(float (&acc)[4][4], const float *A, const float *B, int d,
                                         int ty, int tx)
{
    for (int kk = 0; kk < d; kk++) {
        float a[4], b[4];
#pragma unroll
        for (int r = 0; r < 4; r++) a[r] = A[(ty * 4 + r) * (DPAD + 1) + kk];
#pragma unroll
        for (int c = 0; c < 4; c++) b[c] = B[(tx + 16 * c) * (DPAD + 1) + kk];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[r][c] = fmaf(a[r], b[c], acc[r][c]);
    }
}

// acc[r][c] += sum_kk P[ty*4+r][kk] * V[kk][tx+16c], kk < 64   (P is [64][65], V is [64][DPAD+1])
template <int DPAD>
__device__ __forceinline__ void tile_pv(float (&acc)[4][DPAD / 16], const float *P, const float *V,
                                        int ty, int tx)
{
    for (int kk = 0; kk < 64; kk++) {
        float a[4];
#pragma unroll
        for (int r = 0; r < 4; r++) a[r] = P[(ty * 4 + r) * 65 + kk];
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) {
            float b = V[kk * (DPAD + 1) + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < 4; r++) acc[r][c] = fmaf(a[r], b, acc[r][c]);
        }
    }
}

// acc[r][c] += sum_kk P[kk][ty*4+r] * V[kk][tx+16c]   (transposed first operand)
template <int DPAD>
__device__ __forceinline__ void tile_ptv(float (&acc)[4][DPAD / 16], const float *P, const float *V,
                                         int ty, int tx)
{
    for (int kk = 0; kk < 64; kk++) {
        float a[4];
#pragma unroll
        for (int r = 0; r < 4; r++) a[r] = P[kk * 65 + ty * 4 + r];
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) {
            float b = V[kk * (DPAD + 1) + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < 4; r++) acc[r][c] = fmaf(a[r], b, acc[r][c]);
        }
    }
}

__device__ __forceinline__ float group16_max(float v)
{
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float group16_sum(float v)
{
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T, int DPAD>
__global__ void __launch_bounds__(NT) simt_fwd_kernel(const T *__restrict__ q, const T *__restrict__ k,
                                                      const T *__restrict__ v, T *__restrict__ out,
                                                      float *__restrict__ lse, int lq, int lk, int d,
                                                      float scale, int causal)
{
    extern __shared__ float smem[];
    float *Qs = smem;
    float *Ks = Qs + 64 * (DPAD + 1);
    float *Vs = Ks + 64 * (DPAD + 1);
    float *Ps = Vs + 64 * (DPAD + 1);

    const int bh = blockIdx.x;
    const int q0 = blockIdx.y * BM;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int off = lk - lq;
    q += (size_t)bh * lq * d;
    k += (size_t)bh * lk * d;
    v += (size_t)bh * lk * d;
    out += (size_t)bh * lq * d;

    load_tile<T, DPAD>(Qs, q, q0, lq, d);

    float m[4], l[4], o[4][DPAD / 16];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) o[r][c] = 0.f;
    }

    int kend = lk;
    if (causal) kend = min(lk, q0 + BM + off);  // keys visible to the last row of this block
    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();
        load_tile<T, DPAD>(Ks, k, k0, lk, d);
        load_tile<T, DPAD>(Vs, v, k0, lk, d);
        __syncthreads();

        float s[4][4] = {};
        tile_abt<DPAD>(s, Qs, Ks, d, ty, tx);

#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int row = q0 + ty * 4 + r;
            const int limit = causal ? min(lk - 1, row + off) : lk - 1;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int key = k0 + tx + 16 * c;
                s[r][c] = (key <= limit) ? s[r][c] * scale : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
            mx = group16_max(mx);
            const float m_new = fmaxf(m[r], mx);
            float alpha = 1.f, psum = 0.f;
            if (m_new != -INFINITY) {
                alpha = expf(m[r] - m_new);  // m[r] == -inf gives 0
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    s[r][c] = expf(s[r][c] - m_new);
                    psum += s[r][c];
                }
            } else {
#pragma unroll
                for (int c = 0; c < 4; c++) s[r][c] = 0.f;
            }
            psum = group16_sum(psum);
            l[r] = l[r] * alpha + psum;
            m[r] = m_new;
#pragma unroll
            for (int c = 0; c < DPAD / 16; c++) o[r][c] *= alpha;
#pragma unroll
            for (int c = 0; c < 4; c++) Ps[(ty * 4 + r) * 65 + tx + 16 * c] = s[r][c];
        }
        __syncthreads();
        tile_pv<DPAD>(o, Ps, Vs, ty, tx);
    }

#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = q0 + ty * 4 + r;
        if (row >= lq) continue;
        const float inv = 1.f / l[r];
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) {
            const int col = tx + 16 * c;
            if (col < d) st(out + (size_t)row * d + col, o[r][c] * inv);
        }
        if (lse && tx == 0) lse[(size_t)bh * lq + row] = m[r] + logf(l[r]);
    }
}

// delta[row] = sum_c dO[row][c] * O[row][c]; one warp per row.
template <typename T>
__global__ void delta_kernel(const T *__restrict__ out, const T *__restrict__ dout,
                             float *__restrict__ delta, size_t rows, int d)
{
    const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= rows) return;
    const int lane = threadIdx.x % 32;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) s += ld(out + row * d + c) * ld(dout + row * d + c);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) delta[row] = s;
}

// Recomputes the 64x64 tile of P and dS for (q-tile, k-tile) into shared memory.
// Ps[q][k] = exp(S*scale - lse[q]) (0 where masked), dSs[q][k] = P * (dP - delta[q]) * scale.
template <int DPAD>
__device__ __forceinline__ void recompute_p_ds(float *Ps, float *dSs, const float *Qs,
                                               const float *Ks, const float *Vs, const float *dOs,
                                               const float *lse_s, const float *delta_s, int q0,
                                               int k0, int lq, int lk, int d, float scale, int causal,
                                               int ty, int tx)
{
    float s[4][4] = {}, dp[4][4] = {};
    tile_abt<DPAD>(s, Qs, Ks, d, ty, tx);
    tile_abt<DPAD>(dp, dOs, Vs, d, ty, tx);
    const int off = lk - lq;
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = q0 + ty * 4 + r;
        const int limit = causal ? min(lk - 1, row + off) : lk - 1;
        const float L = lse_s[ty * 4 + r], dl = delta_s[ty * 4 + r];
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int key = k0 + tx + 16 * c;
            float p = 0.f;
            if (row < lq && key <= limit) p = expf(s[r][c] * scale - L);
            Ps[(ty * 4 + r) * 65 + tx + 16 * c] = p;
            if (dSs) dSs[(ty * 4 + r) * 65 + tx + 16 * c] = p * (dp[r][c] - dl) * scale;
        }
    }
}

template <typename T, int DPAD>
__global__ void __launch_bounds__(NT)
    simt_bwd_dkdv_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                         const T *__restrict__ dout, const float *__restrict__ lse,
                         const float *__restrict__ delta, T *__restrict__ dk, T *__restrict__ dv, int lq,
                         int lk, int d, float scale, int causal)
{
    extern __shared__ float smem[];
    float *Ks = smem;
    float *Vs = Ks + 64 * (DPAD + 1);
    float *Qs = Vs + 64 * (DPAD + 1);
    float *dOs = Qs + 64 * (DPAD + 1);
    float *Ps = dOs + 64 * (DPAD + 1);
    float *dSs = Ps + 64 * 65;
    float *lse_s = dSs + 64 * 65;
    float *delta_s = lse_s + 64;

    const int bh = blockIdx.x;
    const int k0 = blockIdx.y * BN;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int off = lk - lq;
    q += (size_t)bh * lq * d;
    dout += (size_t)bh * lq * d;
    k += (size_t)bh * lk * d;
    v += (size_t)bh * lk * d;
    dk += (size_t)bh * lk * d;
    dv += (size_t)bh * lk * d;
    lse += (size_t)bh * lq;
    delta += (size_t)bh * lq;

    load_tile<T, DPAD>(Ks, k, k0, lk, d);
    load_tile<T, DPAD>(Vs, v, k0, lk, d);

    float adk[4][DPAD / 16] = {}, adv[4][DPAD / 16] = {};
    int qstart = 0;
    if (causal) qstart = max(0, (k0 - off) / BM) * BM;  // first query row that sees key k0
    for (int q0 = qstart; q0 < lq; q0 += BM) {
        __syncthreads();
        load_tile<T, DPAD>(Qs, q, q0, lq, d);
        load_tile<T, DPAD>(dOs, dout, q0, lq, d);
        if (threadIdx.x < 64) {
            const int row = q0 + threadIdx.x;
            lse_s[threadIdx.x] = row < lq ? lse[row] : 0.f;
            delta_s[threadIdx.x] = row < lq ? delta[row] : 0.f;
        }
        __syncthreads();
        recompute_p_ds<DPAD>(Ps, dSs, Qs, Ks, Vs, dOs, lse_s, delta_s, q0, k0, lq, lk, d, scale,
                             causal, ty, tx);
        __syncthreads();
        tile_ptv<DPAD>(adv, Ps, dOs, ty, tx);
        tile_ptv<DPAD>(adk, dSs, Qs, ty, tx);
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int key = k0 + ty * 4 + r;
        if (key >= lk) continue;
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) {
            const int col = tx + 16 * c;
            if (col < d) {
                st(dk + (size_t)key * d + col, adk[r][c]);
                st(dv + (size_t)key * d + col, adv[r][c]);
            }
        }
    }
}

template <typename T, int DPAD>
__global__ void __launch_bounds__(NT)
    simt_bwd_dq_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ dout, const float *__restrict__ lse,
                       const float *__restrict__ delta, T *__restrict__ dq, int lq, int lk, int d,
                       float scale, int causal)
{
    extern __shared__ float smem[];
    float *Ks = smem;
    float *Vs = Ks + 64 * (DPAD + 1);
    float *Qs = Vs + 64 * (DPAD + 1);
    float *dOs = Qs + 64 * (DPAD + 1);
    float *Ps = dOs + 64 * (DPAD + 1);
    float *dSs = Ps + 64 * 65;
    float *lse_s = dSs + 64 * 65;
    float *delta_s = lse_s + 64;

    const int bh = blockIdx.x;
    const int q0 = blockIdx.y * BM;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
    const int off = lk - lq;
    q += (size_t)bh * lq * d;
    dout += (size_t)bh * lq * d;
    dq += (size_t)bh * lq * d;
    k += (size_t)bh * lk * d;
    v += (size_t)bh * lk * d;
    lse += (size_t)bh * lq;
    delta += (size_t)bh * lq;

    load_tile<T, DPAD>(Qs, q, q0, lq, d);
    load_tile<T, DPAD>(dOs, dout, q0, lq, d);
    if (threadIdx.x < 64) {
        const int row = q0 + threadIdx.x;
        lse_s[threadIdx.x] = row < lq ? lse[row] : 0.f;
        delta_s[threadIdx.x] = row < lq ? delta[row] : 0.f;
    }

    float adq[4][DPAD / 16] = {};
    int kend = lk;
    if (causal) kend = min(lk, q0 + BM + off);
    for (int k0 = 0; k0 < kend; k0 += BN) {
        __syncthreads();
        load_tile<T, DPAD>(Ks, k, k0, lk, d);
        load_tile<T, DPAD>(Vs, v, k0, lk, d);
        __syncthreads();
        recompute_p_ds<DPAD>(Ps, dSs, Qs, Ks, Vs, dOs, lse_s, delta_s, q0, k0, lq, lk, d, scale,
                             causal, ty, tx);
        __syncthreads();
        tile_pv<DPAD>(adq, dSs, Ks, ty, tx);
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int row = q0 + ty * 4 + r;
        if (row >= lq) continue;
#pragma unroll
        for (int c = 0; c < DPAD / 16; c++) {
            const int col = tx + 16 * c;
            if (col < d) st(dq + (size_t)row * d + col, adq[r][c]);
        }
    }
}

template <typename T, int DPAD>
int launch_fwd(const AttnArgs &a, cudaStream_t s)
{
    const size_t smem = (size_t)(3 * 64 * (DPAD + 1) + 64 * 65) * sizeof(float);
    auto kern = simt_fwd_kernel<T, DPAD>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(a.bh, (a.lq + BM - 1) / BM);
    kern<<<grid, NT, smem, s>>>((const T *)a.q, (const T *)a.k, (const T *)a.v, (T *)a.out, a.lse,
                                a.lq, a.lk, a.d, a.scale, a.causal);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

template <typename T, int DPAD>
int launch_bwd(const AttnArgs &a, float *delta, cudaStream_t s)
{
    const size_t rows = (size_t)a.bh * a.lq;
    delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const T *)a.out, (const T *)a.dout,
                                                               delta, rows, a.d);
    EMBER_CUDA_TRY(cudaGetLastError());
    const size_t smem = (size_t)(4 * 64 * (DPAD + 1) + 2 * 64 * 65 + 128) * sizeof(float);
    auto k1 = simt_bwd_dkdv_kernel<T, DPAD>;
    auto k2 = simt_bwd_dq_kernel<T, DPAD>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    EMBER_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k1<<<dim3(a.bh, (a.lk + BN - 1) / BN), NT, smem, s>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.dout, a.lse, delta, (T *)a.dk,
        (T *)a.dv, a.lq, a.lk, a.d, a.scale, a.causal);
    EMBER_CUDA_TRY(cudaGetLastError());
    k2<<<dim3(a.bh, (a.lq + BM - 1) / BM), NT, smem, s>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.dout, a.lse, delta, (T *)a.dq,
        a.lq, a.lk, a.d, a.scale, a.causal);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace

int simt_attention_fwd(const AttnArgs &a, cudaStream_t s)
{
    if (a.d > 128) {
        set_error("head dimension %d > 128 is not supported", a.d);
        return EMBER_ERR_UNSUPPORTED;
    }
    if (a.dtype == EMBER_F32)
        return a.d <= 64 ? launch_fwd<float, 64>(a, s) : launch_fwd<float, 128>(a, s);
    return a.d <= 64 ? launch_fwd<__nv_bfloat16, 64>(a, s) : launch_fwd<__nv_bfloat16, 128>(a, s);
}

int simt_attention_bwd(const AttnArgs &a, float *delta, cudaStream_t s)
{
    if (a.d > 128) {
        set_error("head dimension %d > 128 is not supported", a.d);
        return EMBER_ERR_UNSUPPORTED;
    }
    if (a.dtype == EMBER_F32)
        return a.d <= 64 ? launch_bwd<float, 64>(a, delta, s) : launch_bwd<float, 128>(a, delta, s);
    return a.d <= 64 ? launch_bwd<__nv_bfloat16, 64>(a, delta, s)
                     : launch_bwd<__nv_bfloat16, 128>(a, delta, s);
}

int launch_delta(const AttnArgs &a, float *delta, cudaStream_t s)
{
    const size_t rows = (size_t)a.bh * a.lq;
    if (a.dtype == EMBER_F32)
        delta_kernel<float><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const float *)a.out, (const float *)a.dout, delta, rows, a.d);
    else
        delta_kernel<__nv_bfloat16><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const __nv_bfloat16 *)a.out, (const __nv_bfloat16 *)a.dout, delta, rows, a.d);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace ember
