// CUDA-core matrix products for the Linear layers: float32 arithmetic, f32 or bf16 storage, any
// shape and any view (row-major or head-major operands). This is the float32 mode of the layers
// (bf16 tensor-core products would use up its 1e-3 tolerance) and the path for shapes the tcgen05
// kernel does not take. Also the column sums that give the bias gradient.
#include "common.cuh"
#include "kernels.cuh"

namespace ember {

namespace {

__device__ __forceinline__ float ld(const float *p, size_t i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16 *p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float *p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16 *p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int TS = 64, TK = 16;  // 64 x 64 output tile, K in steps of 16; 16 x 16 threads, 4 x 4 results each

template <typename T, int MODE>
__global__ void __launch_bounds__(256) simt_gemm_kernel(MatView a, MatView b, MatView c, const T *bias, long long m, int n,
                                                        int k)
{
    __shared__ float as[TK][TS + 1], bs[TK][TS + 1];
    const T *ap = (const T *)a.ptr, *bp = (const T *)b.ptr;
    const long long m0 = (long long)blockIdx.y * TS;
    const int n0 = blockIdx.x * TS;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += TK) {
        for (int e = threadIdx.x; e < TS * TK; e += 256) {
            const int kk = e % TK, ii = e / TK;
            const long long gi = m0 + ii;
            const int gk = k0 + kk, gj = n0 + ii;
            float av = 0.f, bv = 0.f;
            if (gi < m && gk < k) av = (MODE == GEMM_TN) ? ld(ap, view_offset(a, gk, (int)gi)) : ld(ap, view_offset(a, gi, gk));
            if (gj < n && gk < k) bv = (MODE == GEMM_NT) ? ld(bp, view_offset(b, gj, gk)) : ld(bp, view_offset(b, gk, gj));
            as[kk][ii] = av;
            bs[kk][ii] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float ar[4], br[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                ar[i] = as[kk][ty * 4 + i];
                br[i] = bs[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
    T *cp = (T *)c.ptr;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const long long gi = m0 + ty * 4 + i;
        if (gi >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gj = n0 + tx * 4 + j;
            if (gj < n) st(cp, view_offset(c, gi, gj), acc[i][j] + (bias ? ld(bias, (size_t)gj) : 0.f));
        }
    }
}

// out[j] = sum over the rows of a(:, j), rows added in order by 32 partial sums per column (one per
// lane of a warp; lane t takes rows t, t + 32, ...), then a warp reduction.
template <typename T>
__global__ void __launch_bounds__(256) column_sum_kernel(MatView a, T *out)
{
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int col = blockIdx.x * 8 + warp;
    if (col >= a.cols) return;
    const T *ap = (const T *)a.ptr;
    float s = 0.f;
    for (long long r = lane; r < a.rows; r += 32) s += ld(ap, view_offset(a, r, col));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) st(out, (size_t)col, s);
}

template <typename T>
int launch_gemm(const GemmArgs &g, cudaStream_t s)
{
    dim3 grid((g.n + TS - 1) / TS, (unsigned)((g.m + TS - 1) / TS));
    if (g.mode == GEMM_NN)
        simt_gemm_kernel<T, GEMM_NN><<<grid, 256, 0, s>>>(g.a, g.b, g.c, (const T *)g.bias, g.m, g.n, g.k);
    else if (g.mode == GEMM_NT)
        simt_gemm_kernel<T, GEMM_NT><<<grid, 256, 0, s>>>(g.a, g.b, g.c, (const T *)g.bias, g.m, g.n, g.k);
    else
        simt_gemm_kernel<T, GEMM_TN><<<grid, 256, 0, s>>>(g.a, g.b, g.c, (const T *)g.bias, g.m, g.n, g.k);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace

int simt_gemm(const GemmArgs &g, cudaStream_t s)
{
    if ((g.m + TS - 1) / TS > 65535) {
        set_error("linear: more than %d rows are not supported by the CUDA-core kernel", 65535 * TS);
        return EMBER_ERR_UNSUPPORTED;
    }
    return g.dtype == EMBER_BF16 ? launch_gemm<__nv_bfloat16>(g, s) : launch_gemm<float>(g, s);
}

int column_sums(const MatView &a, void *out, int dtype, cudaStream_t s)
{
    const int grid = (a.cols + 7) / 8;
    if (dtype == EMBER_BF16)
        column_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (__nv_bfloat16 *)out);
    else
        column_sum_kernel<float><<<grid, 256, 0, s>>>(a, (float *)out);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace ember
