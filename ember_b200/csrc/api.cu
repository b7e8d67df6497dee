// The extern "C" entry points of the attention path: argument checks in the style of the
// reference's binding (shape mismatches are the caller's ValueError), then dispatch to the
// tcgen05 kernels (bf16, head dimension 64 or 128) or the CUDA-core kernels (everything else).
#include <math.h>
#include <stdlib.h>

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

size_t delta_bytes(int bh, int lq) { return align_up((size_t)bh * lq * sizeof(float), 256); }

// -1: not read yet; the environment variable EMBER_DETERMINISTIC=1 sets the initial value
int g_deterministic = -1;
bool deterministic_mode()
{
    if (g_deterministic < 0) {
        const char *e = getenv("EMBER_DETERMINISTIC");
        g_deterministic = (e && e[0] && e[0] != '0') ? 1 : 0;
    }
    return g_deterministic != 0;
}

bool tensor_core_shape(int d, int dtype) { return dtype == EMBER_BF16 && d >= 8 && d <= 128 && d % 8 == 0; }

// delta vector, then (single-pass tensor-core backward only) the float32 dQ accumulator
size_t bwd_workspace_bytes(int bh, int lq, int d, int dtype)
{
    size_t n = delta_bytes(bh, lq);
    if (tensor_core_shape(d, dtype) && !deterministic_mode()) n += align_up(sm100_bwd_accumulator_bytes(bh, lq, d), 256);
    return n;
}

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
    const size_t need = bwd_workspace_bytes(batch_heads, lq, d, dtype);
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
    if (sm100_bwd_supported(a)) {
        const bool det = deterministic_mode();
        float *acc = det ? nullptr : (float *)((char *)workspace + delta_bytes(batch_heads, lq));
        return sm100_attention_bwd(a, (float *)workspace, acc, det, st, s);
    }
    return simt_attention_bwd(a, (float *)workspace, s);
}

int ember_set_deterministic(int on)
{
    const int before = deterministic_mode() ? 1 : 0;
    g_deterministic = on ? 1 : 0;
    return before;
}

int ember_get_deterministic(void) { return deterministic_mode() ? 1 : 0; }

int ember_set_forward_block_rows(int rows)
{
    if (rows != 0 && rows != 128 && rows != 256) {
        set_error("ember_set_forward_block_rows: %d is not 0, 128 or 256", rows);
        return -EMBER_ERR_INVALID;
    }
    return sm100_fwd_set_block_rows(rows);
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
        case EMBER_OP_BWD: return lq > 0 ? bwd_workspace_bytes(batch_heads, lq, d, dtype) : 0;
        case EMBER_OP_DECODE: {
            if (lk <= 0) return 0;
            int splits = num_splits > 0 ? num_splits : ember_attention_decode_splits(batch_heads, lk, d, dtype);
            if (splits > lk) splits = lk;
            return decode_workspace_bytes(batch_heads, d, splits);
        }
        default: return 0;
    }
}

// Forward over tensors that live in HOST memory (the reference's own calling pattern: NumPy in,
// NumPy out). The (batch*head) units are independent, so they are processed in chunks through two
// sets of device staging buffers: while chunk c computes, chunk c+1 is copied in and chunk c-1 is
// copied out, on three streams chained by events. With pinned host memory the copies run at the
// PCIe rate in both directions at once and the kernel time disappears behind them.
int ember_attention_fwd_host(const void *q_host, const void *k_host, const void *v_host, void *out_host, float *lse_host,
                             int batch_heads, int lq, int lk, int d, float scale, int causal, int dtype)
{
    int rc = check_common("ember_attention_fwd_host", batch_heads, lq, lk, d, dtype, scale);
    if (rc) return rc;
    EMBER_REQUIRE(q_host && k_host && v_host && out_host, "ember_attention_fwd_host: NULL tensor pointer");
    EMBER_REQUIRE(!causal || lq <= lk, "ember_attention_fwd_host: causal attention needs lq <= lk, got lq=%d lk=%d", lq, lk);
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    if (!st->copy_in) {
        EMBER_CUDA_TRY(cudaStreamCreateWithFlags(&st->copy_in, cudaStreamNonBlocking));
        EMBER_CUDA_TRY(cudaStreamCreateWithFlags(&st->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; i++) {
            EMBER_CUDA_TRY(cudaEventCreateWithFlags(&st->in_done[i], cudaEventDisableTiming));
            EMBER_CUDA_TRY(cudaEventCreateWithFlags(&st->compute_done[i], cudaEventDisableTiming));
            EMBER_CUDA_TRY(cudaEventCreateWithFlags(&st->out_done[i], cudaEventDisableTiming));
        }
    }
    const size_t es = dtype_size(dtype);
    const size_t q_unit = (size_t)lq * d * es, k_unit = (size_t)lk * d * es, l_unit = (size_t)lq * sizeof(float);
    // Chunks of about 64 MB of inputs (fewer, larger copies measured faster than many small ones: 8.24 ms
    // against 8.42 at 32 MB and 8.92 at 16 MB for 403 MB in / 134 MB out), tapering towards the end: what
    // is left after the last copy-in is that chunk's kernel and copy-out, so the last chunks halve down
    // to a single unit.
    const size_t unit_in = q_unit + 2 * k_unit;
    const size_t chunk_target = (size_t)64 << 20;
    int per = (int)(chunk_target / (unit_in ? unit_in : 1));
    if (per < 1) per = 1;
    if (per > (batch_heads + 1) / 2) per = (batch_heads + 1) / 2;  // at least two chunks, so that copies and compute overlap
    if (per < 1) per = 1;
    // two sets of staging buffers: q, k, v, out, lse for `per` units each
    const size_t set_bytes = align_up(per * q_unit, 256) * 2 + align_up(per * k_unit, 256) * 2 + align_up(per * l_unit, 256);
    char *stage = (char *)alloc_memory(2 * set_bytes);
    if (!stage) return EMBER_ERR_NOMEM;
    // Any failure below goes through one exit that drains the three streams before the staging
    // block is released, so that no queued copy or kernel still refers to it.
    cudaError_t e = cudaSuccess;
    const char *what = "";
    rc = EMBER_OK;
#define HOST_TRY(expr)                      \
    do {                                    \
        if ((e = (expr)) != cudaSuccess) {  \
            what = #expr;                   \
            goto done;                      \
        }                                   \
    } while (0)
    // the staging memory was allocated in the order of the compute stream: the copy stream waits for it
    HOST_TRY(cudaEventRecord(st->compute_done[0], st->stream));
    HOST_TRY(cudaEventRecord(st->compute_done[1], st->stream));
    HOST_TRY(cudaEventRecord(st->out_done[0], st->copy_out));
    HOST_TRY(cudaEventRecord(st->out_done[1], st->copy_out));
    for (int c = 0, u0 = 0, n = 0; u0 < batch_heads; c++, u0 += n) {
        const int b = c & 1, left = batch_heads - u0;
        n = left > 2 * per ? per : (left + 1) / 2;  // full chunks, then halves of what is left
        if (n > per) n = per;
        char *dq = stage + b * set_bytes, *dk = dq + align_up(per * q_unit, 256), *dv = dk + align_up(per * k_unit, 256);
        char *dout = dv + align_up(per * k_unit, 256), *dl = dout + align_up(per * q_unit, 256);
        // inputs of this set may be overwritten once the kernel that last read them is done
        HOST_TRY(cudaStreamWaitEvent(st->copy_in, st->compute_done[b], 0));
        HOST_TRY(cudaMemcpyAsync(dq, (const char *)q_host + u0 * q_unit, n * q_unit, cudaMemcpyHostToDevice, st->copy_in));
        HOST_TRY(cudaMemcpyAsync(dk, (const char *)k_host + u0 * k_unit, n * k_unit, cudaMemcpyHostToDevice, st->copy_in));
        HOST_TRY(cudaMemcpyAsync(dv, (const char *)v_host + u0 * k_unit, n * k_unit, cudaMemcpyHostToDevice, st->copy_in));
        HOST_TRY(cudaEventRecord(st->in_done[b], st->copy_in));
        // the kernel needs its inputs, and its output buffer must have been copied out
        HOST_TRY(cudaStreamWaitEvent(st->stream, st->in_done[b], 0));
        HOST_TRY(cudaStreamWaitEvent(st->stream, st->out_done[b], 0));
        if ((rc = ember_attention_fwd(dq, dk, dv, dout, (float *)dl, n, lq, lk, d, scale, causal, dtype, st->stream)) != EMBER_OK)
            goto done;
        HOST_TRY(cudaEventRecord(st->compute_done[b], st->stream));
        HOST_TRY(cudaStreamWaitEvent(st->copy_out, st->compute_done[b], 0));
        HOST_TRY(cudaMemcpyAsync((char *)out_host + u0 * q_unit, dout, n * q_unit, cudaMemcpyDeviceToHost, st->copy_out));
        if (lse_host)
            HOST_TRY(cudaMemcpyAsync((char *)lse_host + u0 * l_unit, dl, n * l_unit, cudaMemcpyDeviceToHost, st->copy_out));
        HOST_TRY(cudaEventRecord(st->out_done[b], st->copy_out));
    }
done:
#undef HOST_TRY
    {
        // every user of the staging memory must have finished before it goes back to the pool (in
        // the compute stream's order); the first failure, if any, is the one reported
        const cudaError_t s1 = cudaStreamSynchronize(st->copy_out), s2 = cudaStreamSynchronize(st->copy_in),
                          s3 = cudaStreamSynchronize(st->stream);
        free_memory(stage);
        if (e != cudaSuccess) return cuda_fail(e, what);
        if (rc != EMBER_OK) return rc;
        if (s1 != cudaSuccess) return cuda_fail(s1, "cudaStreamSynchronize(copy_out)");
        if (s2 != cudaSuccess) return cuda_fail(s2, "cudaStreamSynchronize(copy_in)");
        if (s3 != cudaSuccess) return cuda_fail(s3, "cudaStreamSynchronize(stream)");
    }
    return EMBER_OK;
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
