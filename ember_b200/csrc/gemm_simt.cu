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

// out[j] = sum over the rows of a(:, j). One block owns 32 consecutive columns and all the rows:
// 4 threads read the 32 columns of a row as 8-element vectors (whole 64- or 128-byte segments), 64
// rows at a time; every thread keeps 8 float32 partial sums over the rows it visits (rows t, t + 64,
// ...), and shared memory adds the 64 partials of a column in a fixed order. Needs 8-element groups
// that do not straddle a head (cols, or the head dimension, a multiple of 8) and a 16-byte aligned
// base; other shapes take the element-wise kernel below.
template <typename T>
__global__ void __launch_bounds__(256) column_sum_vec_kernel(MatView a, T *out)
{
    __shared__ float part[64][33];
    const int part_col = (threadIdx.x % 4) * 8, rt = threadIdx.x / 4;
    const int col = blockIdx.x * 32 + part_col;
    const T *ap = (const T *)a.ptr;
    float s[8] = {};
    if (col < a.cols) {
        for (long long r = rt; r < a.rows; r += 64) {
            const T *src = ap + view_offset(a, r, col);
            if constexpr (sizeof(T) == 2) {
                const uint4 v = *reinterpret_cast<const uint4 *>(src);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    s[2 * i] += __uint_as_float(w[i] << 16);
                    s[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
                }
            } else {
                const float4 v0 = *reinterpret_cast<const float4 *>(src), v1 = *reinterpret_cast<const float4 *>(src + 4);
                s[0] += v0.x; s[1] += v0.y; s[2] += v0.z; s[3] += v0.w;
                s[4] += v1.x; s[5] += v1.y; s[6] += v1.z; s[7] += v1.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) part[rt][part_col + i] = s[i];
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = 0.f;
        for (int r = 0; r < 64; r++) t += part[r][threadIdx.x];
        const int c = blockIdx.x * 32 + threadIdx.x;
        if (c < a.cols) st(out, (size_t)c, t);
    }
}

// Element-wise variant for any shape: one warp per column, lane t takes rows t, t + 32, ...
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

// Column sums of a large bf16 matrix in two passes, both coalesced: the rows are cut into chunks; a block
// of 8 warps takes 256 columns of one chunk (a warp reads 512 contiguous bytes of a row, lane t its
// columns 8t..8t+7; the offset of a view element splits into a column part, computed once per lane,
// and a row part that is walked without divisions), adds its rows in float32 and writes one partial
// per column; a second kernel adds the partials of a column in a fixed order. The one-pass kernel
// above gives a block only 32 columns, i.e. 64-byte pieces of every row.
__global__ void __launch_bounds__(256) column_partial_kernel(MatView a, float *__restrict__ partial, int rows_per_chunk)
{
    __shared__ float red[8][256];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int col = blockIdx.x * 256 + lane * 8;
    const long long r0 = (long long)blockIdx.y * rows_per_chunk, r1 = min(a.rows, r0 + rows_per_chunk);
    float s[8] = {};
    if (col < a.cols) {
        const __nv_bfloat16 *ap = (const __nv_bfloat16 *)a.ptr;
        const size_t col_off = view_offset(a, 0, col);  // rows and columns of a view address independently
        // row part of the offset: row-major r * cols; head-major (b * heads * seq + l) * dim with r = b * seq + l
        long long r = r0 + warp;
        long long b = a.heads ? r / a.seq : 0;
        int l = a.heads ? (int)(r - b * a.seq) : 0;
#pragma unroll 4
        for (; r < r1; r += 8) {
            const size_t row_off = a.heads ? ((size_t)b * a.heads * a.seq + l) * a.dim : (size_t)r * a.cols;
            const uint4 v = *reinterpret_cast<const uint4 *>(ap + col_off + row_off);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s[2 * i] += __uint_as_float(w[i] << 16);
                s[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
            if (a.heads) {
                l += 8;
                if (l >= a.seq) { l -= a.seq; b++; }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) red[warp][lane * 8 + i] = s[i];
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < a.cols) {
        float t = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; w8++) t += red[w8][threadIdx.x];
        partial[(size_t)blockIdx.y * a.cols + c] = t;
    }
}

__global__ void __launch_bounds__(256) column_final_kernel(const float *__restrict__ partial, __nv_bfloat16 *__restrict__ out, int cols,
                                                           int chunks)
{
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= cols) return;
    float t = 0.f;
    for (int k = 0; k < chunks; k++) t += partial[(size_t)k * cols + c];
    out[c] = __float2bfloat16_rn(t);
}

int column_sums(const MatView &a, void *out, int dtype, cudaStream_t s)
{
    const bool vec = ((uintptr_t)a.ptr & 15) == 0 && (a.heads ? a.dim % 8 == 0 : a.cols % 8 == 0);
    if (vec && dtype == EMBER_BF16 && a.rows >= 4096 && (a.heads == 0 || a.seq % 8 == 0)) {
        const int chunks = 64;
        const int rows_per_chunk = (int)((a.rows + chunks - 1) / chunks + 7) / 8 * 8;
        float *partial = nullptr;
        EMBER_CUDA_TRY(cudaMallocAsync((void **)&partial, (size_t)chunks * a.cols * sizeof(float), s));
        column_partial_kernel<<<dim3((a.cols + 255) / 256, chunks), 256, 0, s>>>(a, partial, rows_per_chunk);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) {
            column_final_kernel<<<(a.cols + 255) / 256, 256, 0, s>>>(partial, (__nv_bfloat16 *)out, a.cols, chunks);
            e = cudaGetLastError();
        }
        cudaFreeAsync(partial, s);
        EMBER_CUDA_TRY(e);
        return EMBER_OK;
    }
    if (vec) {
        const int grid = (a.cols + 31) / 32;
        if (dtype == EMBER_BF16)
            column_sum_vec_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (__nv_bfloat16 *)out);
        else
            column_sum_vec_kernel<float><<<grid, 256, 0, s>>>(a, (float *)out);
    } else {
        const int grid = (a.cols + 7) / 8;
        if (dtype == EMBER_BF16)
            column_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (__nv_bfloat16 *)out);
        else
            column_sum_kernel<float><<<grid, 256, 0, s>>>(a, (float *)out);
    }
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace ember
