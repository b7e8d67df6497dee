// The extern "C" entry points of the Linear layers either side of attention: argument checks,
// then dispatch of each matrix product to the tcgen05 kernel (bf16, aligned views) or the CUDA-core
// kernel (float32 mode and everything else).
#include "common.cuh"
#include "kernels.cuh"

using namespace ember;

namespace {

struct LinearShape {
    long long m;
    int n, k, dtype, x_heads, y_heads, seq, head_dim;
};

int check_linear(const char *fn, const LinearShape &s)
{
    EMBER_REQUIRE(s.dtype == EMBER_F32 || s.dtype == EMBER_BF16, "%s: unknown dtype %d", fn, s.dtype);
    EMBER_REQUIRE(s.m > 0 && s.n > 0 && s.k > 0, "%s: extents must be positive, got m=%lld n=%d k=%d", fn, s.m, s.n, s.k);
    EMBER_REQUIRE(s.x_heads >= 0 && s.y_heads >= 0, "%s: negative head count", fn);
    if (s.x_heads > 0 || s.y_heads > 0) {
        EMBER_REQUIRE(s.seq > 0 && s.head_dim > 0, "%s: head-major layout needs seq > 0 and head_dim > 0", fn);
        EMBER_REQUIRE(s.m % s.seq == 0, "%s: m=%lld is not a multiple of seq=%d", fn, s.m, s.seq);
    }
    if (s.x_heads > 0)
        EMBER_REQUIRE(s.k == s.x_heads * s.head_dim, "%s: k=%d must equal x_heads*head_dim=%d", fn, s.k,
                      s.x_heads * s.head_dim);
    if (s.y_heads > 0)
        EMBER_REQUIRE(s.n % (s.y_heads * s.head_dim) == 0, "%s: n=%d is not a multiple of y_heads*head_dim=%d", fn,
                      s.n, s.y_heads * s.head_dim);
    return EMBER_OK;
}

MatView view(const void *p, long long rows, int cols, int heads, const LinearShape &s)
{
    MatView v;
    v.ptr = p;
    v.rows = rows;
    v.cols = cols;
    v.heads = heads;
    v.seq = heads ? s.seq : 0;
    v.dim = heads ? s.head_dim : 0;
    return v;
}

int run(const GemmArgs &g, DeviceState *st, cudaStream_t s)
{
    if (sm100_gemm_supported(g)) return sm100_gemm(g, st, s);
    return simt_gemm(g, s);
}

}  // namespace

extern "C" {

int ember_linear_fwd(const void *x, const void *w, const void *bias, void *y, long long m, int n, int k, int dtype,
                     int x_heads, int y_heads, int seq, int head_dim, void *stream)
{
    const LinearShape sh = {m, n, k, dtype, x_heads, y_heads, seq, head_dim};
    int rc = check_linear("ember_linear_fwd", sh);
    if (rc) return rc;
    EMBER_REQUIRE(x && w && y, "ember_linear_fwd: NULL tensor pointer");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    GemmArgs g;
    g.mode = GEMM_NN;
    g.a = view(x, m, k, x_heads, sh);
    g.b = view(w, k, n, 0, sh);
    g.c = view(y, m, n, y_heads, sh);
    g.bias = bias;
    g.m = m; g.n = n; g.k = k; g.dtype = dtype;
    return run(g, st, pick_stream(stream, st));
}

int ember_linear_bwd(const void *x, const void *w, const void *dy, void *dx, void *dw, void *db, long long m, int n,
                     int k, int dtype, int x_heads, int y_heads, int seq, int head_dim, void *stream)
{
    const LinearShape sh = {m, n, k, dtype, x_heads, y_heads, seq, head_dim};
    int rc = check_linear("ember_linear_bwd", sh);
    if (rc) return rc;
    EMBER_REQUIRE(x && w && dy, "ember_linear_bwd: NULL tensor pointer");
    EMBER_REQUIRE(dx || dw || db, "ember_linear_bwd: no gradient requested");
    EMBER_REQUIRE(m <= 0x7fffffffLL, "ember_linear_bwd: m=%lld does not fit the weight-gradient product", m);
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    const MatView vx = view(x, m, k, x_heads, sh), vdy = view(dy, m, n, y_heads, sh);
    if (dw) {  // grad_w (k x n) = x^T dy
        GemmArgs g;
        g.mode = GEMM_TN;
        g.a = vx;
        g.b = vdy;
        g.c = view(dw, k, n, 0, sh);
        g.m = k; g.n = n; g.k = (int)m; g.dtype = dtype;
        if ((rc = run(g, st, s)) != EMBER_OK) return rc;
    }
    if (db && (rc = column_sums(vdy, db, dtype, s)) != EMBER_OK) return rc;  // grad_b = sum(dy, axis 0)
    if (dx) {  // grad_x (m x k) = dy w^T
        GemmArgs g;
        g.mode = GEMM_NT;
        g.a = vdy;
        g.b = view(w, k, n, 0, sh);
        g.c = view(dx, m, k, x_heads, sh);
        g.m = m; g.n = k; g.k = n; g.dtype = dtype;
        if ((rc = run(g, st, s)) != EMBER_OK) return rc;
    }
    return EMBER_OK;
}

const char *ember_linear_kernel_name(int product, long long m, int n, int k, int dtype, int x_heads, int y_heads,
                                     int seq, int head_dim)
{
    // Pointers do not matter for the answer except for their alignment; an aligned dummy stands in.
    static const uintptr_t dummy = 256;
    const LinearShape sh = {m, n, k, dtype, x_heads, y_heads, seq, head_dim};
    const void *p = (const void *)dummy;
    GemmArgs g;
    g.dtype = dtype;
    if (product == 1) {  // grad_w
        g.mode = GEMM_TN;
        g.a = view(p, m, k, x_heads, sh); g.b = view(p, m, n, y_heads, sh); g.c = view(p, k, n, 0, sh);
        g.m = k; g.n = n; g.k = (int)m;
    } else if (product == 2) {  // grad_x
        g.mode = GEMM_NT;
        g.a = view(p, m, n, y_heads, sh); g.b = view(p, k, n, 0, sh); g.c = view(p, m, k, x_heads, sh);
        g.m = m; g.n = k; g.k = n;
    } else {  // forward
        g.mode = GEMM_NN;
        g.a = view(p, m, k, x_heads, sh); g.b = view(p, k, n, 0, sh); g.c = view(p, m, n, y_heads, sh);
        g.m = m; g.n = n; g.k = k;
    }
    return sm100_gemm_supported(g) ? "sm100_tcgen05" : "simt_f32";
}

}  // extern "C"
