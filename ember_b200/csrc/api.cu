// The extern "C" entry points of the attention path: argument checks in the style of the
// reference's binding (shape mismatches are the caller's ValueError), then dispatch to the
// tcgen05 kernels (bf16, head dimension 64 or 128) or the CUDA-core kernels (everything else).
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

using namespace ember;

namespace {

int check_common(const char *fn, int bh, int lq, int lk, int d, int dtype, float scale)
{
    EMBER_REQUIRE(dtype == EMBER_F32 || dtype == EMBER_BF16, "%s: unknown dtype %d", fn, dtype);
    EMBER_REQUIRE(bh > 0 && lq > 0 && lk > 0 && d > 0,
                  "%s: extents must be positive, got batch_heads=%d lq=%d lk=%d d=%d", fn, bh, lq, lk, d);
    EMBER_REQUIRE(isfinite(scale), "%s: scale must be finite", fn);
    return EMBER_OK;
}

bool aligned(const void *p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

size_t bwd_workspace_bytes(int bh, int lq) { return align_up((size_t)bh * lq * sizeof(float), 256); }

}  // namespace

extern "C" {

int ember_attention_fwd(const void *q, const void *k, const void *v, void *out, float *lse, int batch_heads,
                        int lq, int lk, int d, float scale, int causal, int dtype, void *stream)
{
    int rc = check_common("ember_attention_fwd", batch_heads, lq, lk, d, dtype, scale);
    if (rc) return rc;
    EMBER_REQUIRE(q && k && v && out, "ember_attention_fwd: NULL tensor pointer");
    EMBER_REQUIRE(!causal || lq <= lk, "ember_attention_fwd: causal attention needs lq <= lk, got lq=%d lk=%d",
                  lq, lk);
    const size_t es = dtype_size(dtype);
    EMBER_REQUIRE(aligned(q, es) && aligned(k, es) && aligned(v, es) && aligned(out, es),
                  "ember_attention_fwd: misaligned tensor pointer");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    a.bh = batch_heads; a.lq = lq; a.lk = lk; a.d = d;
    a.scale = scale; a.causal = causal ? 1 : 0; a.dtype = dtype;
    cudaStream_t s = pick_stream(stream, st);
    if (sm100_fwd_supported(a)) return sm100_attention_fwd(a, st, s);
    return simt_attention_fwd(a, s);
}

int ember_attention_bwd(const void *q, const void *k, const void *v, const void *out, const float *lse,
                        const void *dout, void *dq, void *dk, void *dv, int batch_heads, int lq, int lk, int d,
                        float scale, int causal, int dtype, void *workspace, size_t workspace_bytes,
                        void *stream)
{
    int rc = check_common("ember_attention_bwd", batch_heads, lq, lk, d, dtype, scale);
    if (rc) return rc;
    EMBER_REQUIRE(q && k && v && out && lse && dout && dq && dk && dv, "ember_attention_bwd: NULL tensor pointer");
    EMBER_REQUIRE(!causal || lq <= lk, "ember_attention_bwd: causal attention needs lq <= lk, got lq=%d lk=%d",
                  lq, lk);
    const size_t need = bwd_workspace_bytes(batch_heads, lq);
    if (!workspace || workspace_bytes < need) {
        set_error("ember_attention_bwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return EMBER_ERR_WORKSPACE;
    }
    EMBER_REQUIRE(aligned(workspace, 256), "ember_attention_bwd: workspace must be 256-byte aligned");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.out = (void *)out; a.lse = (float *)lse; a.dout = dout;
    a.dq = dq; a.dk = dk; a.dv = dv;
    a.bh = batch_heads; a.lq = lq; a.lk = lk; a.d = d;
    a.scale = scale; a.causal = causal ? 1 : 0; a.dtype = dtype;
    cudaStream_t s = pick_stream(stream, st);
    if (sm100_bwd_supported(a)) return sm100_attention_bwd(a, (float *)workspace, st, s);
    return simt_attention_bwd(a, (float *)workspace, s);
}

int ember_attention_decode_splits(int batch_heads, int lk, int d, int dtype)
{
    DeviceState *st = device_state();
    return decode_pick_splits(batch_heads, lk, d, dtype, st ? st->sm_count : 148);
}

int ember_attention_decode(const void *q, const void *k, const void *v, void *out, float *lse, int batch_heads,
                           int lk, int d, float scale, int dtype, int num_splits, void *workspace,
                           size_t workspace_bytes, void *stream)
{
    int rc = check_common("ember_attention_decode", batch_heads, 1, lk, d, dtype, scale);
    if (rc) return rc;
    EMBER_REQUIRE(q && k && v && out, "ember_attention_decode: NULL tensor pointer");
    EMBER_REQUIRE(aligned(q, 16) && aligned(k, 16) && aligned(v, 16),
                  "ember_attention_decode: q, k and v must be 16-byte aligned");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    int splits = num_splits > 0 ? num_splits : decode_pick_splits(batch_heads, lk, d, dtype, st->sm_count);
    if (splits > lk) splits = lk;
    const size_t need = decode_workspace_bytes(batch_heads, d, splits);
    if (need > 0) {
        if (!workspace || workspace_bytes < need) {
            set_error("ember_attention_decode: workspace of %zu bytes needed for %d splits, %zu given", need,
                      splits, workspace_bytes);
            return EMBER_ERR_WORKSPACE;
        }
        EMBER_REQUIRE(aligned(workspace, 256), "ember_attention_decode: workspace must be 256-byte aligned");
    }
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.out = out; a.lse = lse;
    a.bh = batch_heads; a.lq = 1; a.lk = lk; a.d = d;
    a.scale = scale; a.causal = 0; a.dtype = dtype;
    return decode_attention(a, splits, workspace, st, pick_stream(stream, st));
}

size_t ember_attention_workspace_bytes(int op, int batch_heads, int lq, int lk, int d, int dtype, int num_splits)
{
    if (batch_heads <= 0 || d <= 0) return 0;
    switch (op) {
        case EMBER_OP_BWD: return lq > 0 ? bwd_workspace_bytes(batch_heads, lq) : 0;
        case EMBER_OP_DECODE: {
            if (lk <= 0) return 0;
            int splits = num_splits > 0 ? num_splits : ember_attention_decode_splits(batch_heads, lk, d, dtype);
            if (splits > lk) splits = lk;
            return decode_workspace_bytes(batch_heads, d, splits);
        }
        default: return 0;
    }
}

const char *ember_attention_kernel_name(int op, int lq, int lk, int d, int dtype)
{
    (void)lk;
    AttnArgs a;
    a.lq = lq; a.lk = lk; a.d = d; a.dtype = dtype; a.scale = 1.f;
    if (op == EMBER_OP_FWD) return sm100_fwd_supported(a) ? "sm100_tcgen05" : "simt_f32";
    if (op == EMBER_OP_BWD) return sm100_bwd_supported(a) ? "sm100_tcgen05" : "simt_f32";
    return "decode_split_kv";
}

}  // extern "C"
