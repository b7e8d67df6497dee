// Internal interface between the C-ABI dispatcher and the kernel families.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace ember {

struct AttnArgs {
    const void *q = nullptr, *k = nullptr, *v = nullptr;
    void *out = nullptr;
    float *lse = nullptr;
    const void *dout = nullptr;
    void *dq = nullptr, *dk = nullptr, *dv = nullptr;
    int bh = 0, lq = 0, lk = 0, d = 0;
    float scale = 1.f;
    int causal = 0;
    int dtype = EMBER_F32;
};

// CUDA-core kernels (attn_simt.cu): float32 math, f32 or bf16 storage, d <= 128.
int simt_attention_fwd(const AttnArgs &a, cudaStream_t s);
int simt_attention_bwd(const AttnArgs &a, float *delta, cudaStream_t s);
int launch_delta(const AttnArgs &a, float *delta, cudaStream_t s);

// tcgen05 kernels (attn_fwd_sm100.cu / attn_bwd_sm100.cu): bf16 storage, d in {64, 128}.
bool sm100_fwd_supported(const AttnArgs &a);
int sm100_fwd_set_block_rows(int rows);  // 0 = choose per call, 128, 256; returns the previous setting
int sm100_attention_fwd(const AttnArgs &a, DeviceState *st, cudaStream_t s);
bool sm100_bwd_supported(const AttnArgs &a);
// deterministic: two kernels (dK/dV, then dQ), bit-reproducible; otherwise one pass that adds its dQ
// contributions into dq_acc (sm100_bwd_accumulator_bytes of float32 scratch after the delta vector).
size_t sm100_bwd_accumulator_bytes(int bh, int lq, int d);
int sm100_attention_bwd(const AttnArgs &a, float *delta, float *dq_acc, bool deterministic, DeviceState *st, cudaStream_t s);

// Decode over a contiguous key/value cache with grouped-query heads on the tensor cores
// (attn_fwd_sm100.cu: the forward kernel with the group's query heads as the rows of one tile and the
// key axis cut into splits). chunk: keys per split, a multiple of 128; workspace: partial outputs.
struct CacheDecodeArgs {
    const void *q = nullptr, *k_cache = nullptr, *v_cache = nullptr;
    void *out = nullptr;
    float *lse = nullptr;
    int batch = 0, q_heads = 0, kv_heads = 0, lk = 0, capacity = 0, d = 0, dtype = EMBER_BF16;
    float scale = 1.f;
    const int *seq_lens = nullptr;
    int splits = 1, chunk = 0;
    void *workspace = nullptr;
};
bool sm100_cache_decode_supported(const CacheDecodeArgs &a);
size_t sm100_cache_decode_workspace_bytes(int units, int rows, int d, int splits);
int sm100_cache_decode(const CacheDecodeArgs &a, DeviceState *st, cudaStream_t s);

// Split-KV decode (attn_decode.cu): lq == 1, bf16 or f32 storage, d <= 256 and d % 8 == 0.
int decode_pick_splits(int bh, int lk, int d, int dtype, int sm_count);
size_t decode_workspace_bytes(int bh, int d, int splits);
int decode_attention(const AttnArgs &a, int splits, void *workspace, DeviceState *st, cudaStream_t s);

// ---------------------------------------------------------------- projections either side of attention
// A logical (rows x cols) matrix and how it lies in memory.
//   heads == 0: row-major, leading dimension = cols.
//   heads  > 0: head-major (parts, batch, heads, seq, dim), the layout attention consumes:
//               row = b * seq + l, col = (part * heads + h) * dim + d, batch = rows / seq,
//               parts = cols / (heads * dim).
struct MatView {
    const void *ptr = nullptr;
    long long rows = 0;
    int cols = 0;
    int heads = 0, seq = 0, dim = 0;
};

__host__ __device__ inline size_t view_offset(const MatView &v, long long row, int col)
{
    if (v.heads == 0) return (size_t)row * v.cols + col;
    const long long b = row / v.seq, batch = v.rows / v.seq;
    const int l = (int)(row - b * v.seq), ph = col / v.dim, d = col - ph * v.dim;
    const int part = ph / v.heads, h = ph - part * v.heads;
    return ((((size_t)part * batch + b) * v.heads + h) * v.seq + l) * v.dim + d;
}

// C (m x n) = op(A) * op(B) [+ bias], bf16 or f32 storage, float32 accumulation.
enum GemmMode {
    GEMM_NN = 0,  // A view (m x k), B view (k x n)
    GEMM_NT = 1,  // A view (m x k), B view (n x k)
    GEMM_TN = 2   // A view (k x m), B view (k x n)
};
struct GemmArgs {
    int mode = GEMM_NN;
    MatView a, b, c;
    const void *bias = nullptr;  // n values of the storage dtype, or null
    long long m = 0;
    int n = 0, k = 0;
    int dtype = EMBER_F32;
};

// CUDA-core kernels (gemm_simt.cu): float32 math, any shape and view.
int simt_gemm(const GemmArgs &g, cudaStream_t s);
int column_sums(const MatView &a, void *out, int dtype, cudaStream_t s);  // out[j] = sum over rows of a(:, j)
// tcgen05 kernel (gemm_sm100.cu): bf16 storage; see sm100_gemm_supported for the shapes it takes.
bool sm100_gemm_supported(const GemmArgs &g);
int sm100_gemm(const GemmArgs &g, DeviceState *st, cudaStream_t s);
int make_tensor_map_bf16_view(CUtensorMap *map, const MatView &v, uint32_t box_cols, uint32_t box_rows);

}  // namespace ember
