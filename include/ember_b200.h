/* ember_b200.h -- C ABI of the B200 (sm_100a) attention library.
 *
 * This header is the drop-in boundary: the declarations a binding for the
 * reference project (its CPython extension module built from
 * src/tensor/tensor_api.c) would call, in the style of the reference's own
 * operator header (src/tensor/operators.h:21-27: raw device pointers, integer
 * extents, caller-allocated outputs) and memory header (src/core/memory.h:10-14).
 *
 * Conventions
 *   - All tensor pointers are DEVICE pointers to contiguous row-major buffers,
 *     the only layout the reference has (ember/tensor/tensor_utils.py:85-94).
 *     q: (batch_heads, lq, d)   k, v: (batch_heads, lk, d)   out: like q
 *     lse: (batch_heads, lq) float32, natural-log log-sum-exp of the scaled,
 *     masked scores of each query row.
 *   - dtype selects the storage type of q/k/v/out/dout/dq/dk/dv: EMBER_F32 or
 *     EMBER_BF16. Softmax and all accumulation are float32 in both modes.
 *   - causal != 0 masks key j for query i when j > i + (lk - lq) (lower
 *     triangle aligned to the bottom-right corner; requires lq <= lk). This is
 *     the additive {0,-inf} mask the reference would need a broadcast add for
 *     (src/tensor/operators.def:65).
 *   - stream is a cudaStream_t passed as void*; NULL means the library's own
 *     non-blocking stream of the current device (see ember_stream()).
 *     Calls enqueue work and return; nothing synchronises except where stated.
 *   - Every function returning int returns an ember_status. The library never
 *     calls exit() (the reference's GPU_ERR_CHK does: src/core/utils_gpu.cuh:9-19).
 *   - Not thread-safe, like the reference (its cuBLAS handle is a bare static:
 *     src/tensor/operators_gpu.cu:24-31).
 */
#ifndef EMBER_B200_H
#define EMBER_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define EMBER_API __attribute__((visibility("default")))
#else
#define EMBER_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    EMBER_OK = 0,
    EMBER_ERR_INVALID = 1,     /* bad shape, NULL pointer, misaligned pointer */
    EMBER_ERR_UNSUPPORTED = 2, /* valid request this build has no kernel for  */
    EMBER_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed           */
    EMBER_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up          */
    EMBER_ERR_NOMEM = 5,       /* device allocation failed                    */
    EMBER_ERR_WORKSPACE = 6    /* workspace missing or too small              */
} ember_status;

enum { EMBER_F32 = 0, EMBER_BF16 = 1 };

/* Which operation a workspace is sized for. */
enum { EMBER_OP_FWD = 0, EMBER_OP_BWD = 1, EMBER_OP_DECODE = 2 };

/* ---- device memory: same five entry points, same meaning, as the reference's
 *      src/core/memory.h:10-14 (GPU implementation: src/core/memory_gpu.cu:10-43).
 *      alloc_memory returns NULL on failure (memory_gpu.cu:15-19). Allocation is
 *      stream-ordered on the library stream instead of one cudaMalloc/cudaFree
 *      per tensor; copies are ordered on that stream and copy_from_device
 *      waits for it, as the reference's synchronous cudaMemcpy does. ---- */
EMBER_API void *alloc_memory(size_t bytes);
EMBER_API void free_memory(void *ptr);
EMBER_API void copy_to_device(void *dst_device, const void *src_host, size_t bytes);
EMBER_API void copy_from_device(void *dst_host, const void *src_device, size_t bytes);
EMBER_API void sync_device(void);

/* ---- the same allocator in the order of a stream of the caller's choice (no counterpart in the
 *      reference, whose cudaMalloc/cudaFree per tensor synchronise the device:
 *      src/core/memory_gpu.cu:10-28, TODO.md:12). free_memory releases a block in the order of
 *      the LIBRARY stream: a block that a kernel on another stream may still be using must either
 *      be released with ember_free_async on that stream, or only after that stream has been
 *      synchronised; otherwise the pool may hand the block to the next allocation while the kernel
 *      still runs. stream NULL = the library stream. ember_alloc_async returns NULL on failure
 *      (text in ember_last_error()). Freed blocks stay in the device's pool (release threshold
 *      unlimited) and are reused without a new driver allocation; ember_pool_stats reports what the
 *      pool currently holds from the driver (reserved) and has handed out (used). ---- */
EMBER_API void *ember_alloc_async(size_t bytes, void *stream);
EMBER_API int ember_free_async(void *ptr, void *stream);
EMBER_API int ember_pool_stats(size_t *reserved_bytes, size_t *used_bytes);

/* ---- additions the attention path needs from src/core (no counterpart in the
 *      reference, which is single-device, default-stream, float32-only) ---- */
EMBER_API int ember_set_device(int device);
EMBER_API int ember_get_device(int *device);
EMBER_API void *ember_stream(void); /* the library's stream of the current device, as cudaStream_t */
EMBER_API int ember_f32_to_bf16(const float *src, void *dst, size_t n, void *stream);
EMBER_API int ember_bf16_to_f32(const void *src, float *dst, size_t n, void *stream);
EMBER_API const char *ember_status_string(int status);
/* Text of the most recent failure on this thread's last call ("" if none). */
EMBER_API const char *ember_last_error(void);
/* Reads and clears the device-side status word written by bounded waits.
 * Synchronises the stream. Returns EMBER_OK or EMBER_ERR_TIMEOUT; *where gets
 * the code of the wait that gave up (0 if none). */
EMBER_API int ember_check_device_status(void *stream, int *where);

/* Self-test of the failure path (no counterpart in the reference): launches one warp that waits on
 * a barrier nobody arrives at; its bounded wait gives up after about a millisecond and reports
 * through the status word, so the next ember_check_device_status returns EMBER_ERR_TIMEOUT with
 * *where == 9001. Nothing faults or hangs and the context stays usable. */
EMBER_API int ember_selftest_wait_timeout(void *stream);

/* ---- attention forward (prefill, optionally causal). Replaces the composed
 *      reference path  softmax((q @ kT) * scale [+ mask]) @ v :
 *      ember/tensor/tensor.py:163-197 (__matmul__) -> src/tensor/tensor_api.c:330-354
 *      -> src/tensor/operators_gpu.cu:126-136 (cublasSgemmStridedBatched), scalar
 *      multiply src/tensor/operators.def:54, softmax ember/tensor/tensor.py:430-437
 *      (max_axis src/tensor/operators_gpu.cu:198-219, sum_axis :175-196).
 *      k is taken in its natural (batch_heads, lk, d) layout; no host transpose.
 *      lse may be NULL when the caller does not need it. ---- */
EMBER_API int ember_attention_fwd(const void *q, const void *k, const void *v, void *out, float *lse,
                        int batch_heads, int lq, int lk, int d, float scale, int causal, int dtype,
                        void *stream);

/* ---- attention backward. Replaces the manual-backward composition the
 *      reference's layers use (ember/nn/layers.py:50-56; softmax gradient as in
 *      ember/loss/losses.py:53-56): dV = P^T dO, dP = dO V^T, dS = P*(dP - delta)*scale,
 *      dQ = dS K, dK = dS^T Q, with P recomputed from the saved lse.
 *      workspace: ember_attention_workspace_bytes(EMBER_OP_BWD, ...) bytes of
 *      device memory, 256-byte aligned, contents undefined on entry (the row sums of dO*O,
 *      and for the single-pass bf16 kernel a float32 dQ accumulator of lq rounded up to 128 rows
 *      per batch_head, which the call clears itself). ---- */
EMBER_API int ember_attention_bwd(const void *q, const void *k, const void *v, const void *out,
                        const float *lse, const void *dout, void *dq, void *dk, void *dv,
                        int batch_heads, int lq, int lk, int d, float scale, int causal, int dtype,
                        void *workspace, size_t workspace_bytes, void *stream);

/* ---- run-to-run reproducibility of the backward (no counterpart in the reference, whose CPU
 *      loops are sequential). By default the bf16 tensor-core backward makes ONE pass over the
 *      (key tile, query tile) pairs and adds each key tile's contribution to dQ into a float32
 *      accumulator in the workspace; those additions arrive in no fixed order, so dQ is
 *      reproducible to float32 rounding only (dK, dV and everything else are bit-reproducible).
 *      ember_set_deterministic(1) selects the two-kernel form (dK/dV, then a separate dQ pass that
 *      recomputes the scores): bit-identical results from run to run at about 1.4x the tile
 *      products. The setting is process-wide; its initial value is 1 when the environment variable
 *      EMBER_DETERMINISTIC is set to something other than 0. Returns the previous setting.
 *      Change it only between calls; workspace sizes depend on it (query them after changing). ---- */
EMBER_API int ember_set_deterministic(int on);
EMBER_API int ember_get_deterministic(void);

/* ---- query rows per CTA of the bf16 tensor-core forward (a tuning and test switch; no counterpart
 *      in the reference). 0 (the default) lets the library choose per call: 256 rows (two 128-row
 *      tiles sharing the key/value stream), or 128 rows for launches too small to keep every SM
 *      busy. 128 or 256 forces one form for every later call; both give the same bits. The initial
 *      value comes from the environment variable EMBER_FWD_ROWS when it is 128 or 256.
 *      Returns the previous setting; other values are EMBER_ERR_INVALID (negative). ---- */
EMBER_API int ember_set_forward_block_rows(int rows);

/* ---- single-query decode against a long key/value cache (lq == 1, no mask),
 *      split over the key axis with a log-sum-exp combine. Same reference path as
 *      the forward with n = 1 rows per batch (src/tensor/operators_gpu.cu:126-136).
 *      num_splits <= 0 lets the library choose. workspace as above with
 *      EMBER_OP_DECODE (may be NULL/0 when the chosen split count is 1). ---- */
EMBER_API int ember_attention_decode(const void *q, const void *k, const void *v, void *out, float *lse,
                           int batch_heads, int lk, int d, float scale, int dtype, int num_splits,
                           void *workspace, size_t workspace_bytes, void *stream);

/* ---- decode for callers that cannot allocate. No counterpart in the reference.
 *      Some hosts of this library may not call cudaMalloc on the path that runs decode: a
 *      serving loop that has handed the whole device to its own arena, code running where an
 *      allocation would synchronise the device or is forbidden outright. This variant takes no
 *      workspace and allocates nothing (no cudaMalloc/cudaFree, no pool, no stream creation): the
 *      per-split partials go to a fixed 4 MiB array that is part of the library image, so every
 *      GPU that loads the library holds those 4 MiB until the process exits.
 *      Limits: batch_heads * splits * d * 4 bytes plus batch_heads * splits * 8 bytes (each
 *      rounded up to 256) must fit in ember_attention_decode_static_capacity() bytes; a request
 *      beyond that returns EMBER_ERR_WORKSPACE with the sizes in ember_last_error(). With
 *      num_splits <= 0 the library lowers its own split choice until it fits (one split needs no
 *      scratch), so that form never fails for size.
 *      stream: a cudaStream_t as void*; NULL here means the CUDA default stream (the library's
 *      own stream is not created by this call).
 *      The first call on each device looks up the array's device address
 *      (cudaGetSymbolAddress) with that device current; make that first call outside any
 *      stream capture. All calls share the one array and it keeps the previous call's contents:
 *      nothing in it needs clearing (each call overwrites what it later reads), but two calls
 *      that overlap on the GPU (different streams, no ordering between them) race on it. ---- */
EMBER_API int ember_attention_decode_static(const void *q, const void *k, const void *v, void *out,
                                            float *lse, int batch_heads, int lk, int d, float scale,
                                            int dtype, int num_splits, void *stream);
/* Forward over tensors in HOST memory, the reference's own calling pattern (NumPy array in,
 * Tensor, operators, to_np() out: ember/tensor/tensor.py:78-117,224-226). q, k, v, out (and lse,
 * which may be NULL) are host pointers with the layouts of ember_attention_fwd; pinned (page-locked)
 * memory lets the copies overlap. The (batch*head) units are streamed through device staging
 * buffers in chunks, copy-in, compute and copy-out on three streams, so the call costs about the
 * larger of the two PCIe directions instead of their sum plus the kernel. Returns when out_host is
 * complete. */
EMBER_API int ember_attention_fwd_host(const void *q_host, const void *k_host, const void *v_host, void *out_host,
                                       float *lse_host, int batch_heads, int lq, int lk, int d, float scale, int causal,
                                       int dtype);

/* Size in bytes of the built-in scratch array of ember_attention_decode_static. */
EMBER_API size_t ember_attention_decode_static_capacity(void);

/* Bytes of workspace the call with these arguments needs (0 if none). For
 * EMBER_OP_DECODE lq is ignored; num_splits <= 0 means "the library's choice". */
EMBER_API size_t ember_attention_workspace_bytes(int op, int batch_heads, int lq, int lk, int d, int dtype,
                                       int num_splits);
/* The split count ember_attention_decode uses for num_splits <= 0. */
EMBER_API int ember_attention_decode_splits(int batch_heads, int lk, int d, int dtype);

/* The order in which the CTAs of the tensor-core attention kernels take their work, for tests and
 * tools (pure host arithmetic, no device needed): CTA `index` of a launch over `units` (batch*head)
 * units of `blocks` row blocks each works on block rank *rank (0 = heaviest under a causal mask) of
 * unit *unit. Units are taken in groups sized from sm_count and, under a causal mask, from the bytes
 * one unit touches, so that concurrently running CTAs share their K/V through L2. */
EMBER_API int ember_work_order_item(int units, int blocks, int sm_count, size_t touched_bytes_per_unit, int causal,
                                    int index, int *unit, int *rank);

/* Name of the kernel family the forward/backward dispatcher picks for these
 * arguments: "sm100_tcgen05" or "simt_f32". For tests and the benchmark. */
EMBER_API const char *ember_attention_kernel_name(int op, int lq, int lk, int d, int dtype);

/* ---- Optional gather of the per-rank output slabs (no counterpart in the reference, which has no
 *      communication layer: its CMakeLists.txt:63,102 link only cuBLAS).
 *
 * The path shards over (batch * head) with no exchange in forward or backward. When a caller wants
 * the whole result on every rank, rank r of `world` passes its slab (equal sizes on all ranks)
 * and receives the concatenation in rank order: one ncclAllGather over NVLink inside a box,
 * enqueued on `stream` (NULL = the library stream). NCCL is loaded at run time (libnccl.so.2, or the
 * path in the environment variable EMBER_NCCL_LIB); without it these calls return
 * EMBER_ERR_UNSUPPORTED and everything else works.
 *
 * Set-up: one rank calls ember_comm_unique_id and hands the EMBER_COMM_ID_BYTES bytes to the others
 * by any host-side means (a file, a socket, the launcher's key/value store); every rank then calls
 * ember_comm_init with its device current. A rank that never arrives makes the others return
 * EMBER_ERR_TIMEOUT after timeout_ms (<= 0: wait without limit) with nothing left running on the
 * GPU. out_full may alias the slab (in place: out_slab == out_full + rank * slab_bytes). ---- */
#define EMBER_COMM_ID_BYTES 128
EMBER_API int ember_comm_unique_id(void *id_out);
EMBER_API int ember_comm_init(void **comm, const void *id, int rank, int world, int timeout_ms);
EMBER_API int ember_comm_destroy(void *comm);
EMBER_API int ember_gather_outputs(void *out_full, const void *out_slab, size_t slab_bytes, void *comm, void *stream);

/* ---- The Linear layers either side of attention -----------------------------
 *
 * Replaces the reference's Linear layer (ember/nn/layers.py:9-56), which composes
 *     forward   y      = b + x @ w            (tensor.py:163-197 -> tensor_api.c:330-354, operators.def:65)
 *     backward  grad_w = T(x) @ grad_y ; grad_b = sum(grad_y, axis=0) ; grad_x = grad_y @ T(w)
 * from its matmul, transpose, broadcast-add and sum operators, one allocation per step.
 *
 * x is a logical (m, k) matrix, w is (k, n) row-major as the reference stores it (in_features,
 * out_features), bias has n elements (or NULL), y is (m, n). dtype selects storage as for attention
 * (float32 arithmetic on CUDA cores for EMBER_F32; bf16 tensor-core products with float32
 * accumulation for EMBER_BF16 when the shapes allow, else float32 arithmetic on bf16 storage).
 *
 * Head-major operands, so that no transpose runs between a projection and attention:
 *   x_heads > 0: x (and grad_x) lie as (batch, x_heads, seq, head_dim), the layout attention
 *                writes; k == x_heads * head_dim, m == batch * seq.
 *   y_heads > 0: y (and grad_y) lie as (parts, batch, y_heads, seq, head_dim) with
 *                n == parts * y_heads * head_dim: a fused q/k/v projection (parts == 3) writes the
 *                three (batch, heads, seq, head_dim) tensors attention reads, back to back.
 *   0 means row-major. seq and head_dim are ignored when both head counts are 0.
 *
 * ember_linear_bwd: any of grad_x, grad_w, grad_b may be NULL and is then skipped. */
EMBER_API int ember_linear_fwd(const void *x, const void *w, const void *bias, void *y, long long m, int n, int k,
                               int dtype, int x_heads, int y_heads, int seq, int head_dim, void *stream);
EMBER_API int ember_linear_bwd(const void *x, const void *w, const void *grad_y, void *grad_x, void *grad_w,
                               void *grad_b, long long m, int n, int k, int dtype, int x_heads, int y_heads,
                               int seq, int head_dim, void *stream);
/* Kernel family the dispatcher picks for one of the three products (0 forward, 1 grad_w,
 * 2 grad_x) with 16-byte aligned pointers: "sm100_tcgen05" or "simt_f32". */
EMBER_API const char *ember_linear_kernel_name(int product, long long m, int n, int k, int dtype, int x_heads,
                                               int y_heads, int seq, int head_dim);

/* ---- Fused softmax and softmax cross-entropy --------------------------------
 *
 * ember_softmax_fwd replaces the reference's softmax over the last axis
 * (ember/tensor/tensor.py:430-437: amax, broadcast subtract, exp, sum, broadcast divide, i.e. five
 * passes and five allocations) with one read and one write per element; log_softmax != 0 gives
 * x - max - log(sum(exp(x - max))) instead. x and y are (rows, cols) row-major of `dtype`.
 *
 * ember_cross_entropy_fwd / _bwd replace CrossEntropyLoss.forward / .backward
 * (ember/loss/losses.py:42-56): pred are logits and target probabilities (one-hot in the
 * reference's use), both (rows, cols); probs receives softmax(pred) (the reference caches it for the
 * backward), *loss (one float32 in device memory) receives -sum(target * log_softmax(pred)) / rows.
 * workspace: ember_cross_entropy_workspace_bytes(rows) bytes of device memory (one partial per row,
 * added in a fixed order). backward: grad = (probs - target) / rows. */
EMBER_API int ember_softmax_fwd(const void *x, void *y, long long rows, int cols, int dtype, int log_softmax,
                                void *stream);
EMBER_API size_t ember_cross_entropy_workspace_bytes(long long rows);
EMBER_API int ember_cross_entropy_fwd(const void *pred, const void *target, void *probs, float *loss, long long rows,
                                      int cols, int dtype, void *workspace, size_t workspace_bytes, void *stream);
EMBER_API int ember_cross_entropy_bwd(const void *probs, const void *target, void *grad, long long rows, int cols,
                                      int dtype, void *stream);

/* ---- Key/value cache for decode ---------------------------------------------
 *
 * The reference has no cache concept: a decode step would re-run the composed attention over
 * freshly built (B, H, Lk, D) tensors, whose element count is a C int (src/core/tensor_types.h:8).
 * These entry points keep K and V in a preallocated cache, append new rows in place and decode
 * over the filled part, with grouped-query heads and an optional page table.
 *
 * Contiguous cache: K and V are (batch, kv_heads, capacity, d). Paged cache (block_table != NULL):
 * K and V are (num_pages, kv_heads, page_size, d), page_size a power of two, and key j of sequence
 * b lives in page block_table[b * max_blocks + j / page_size], row j % page_size; `capacity` is
 * ignored. seq_lens (device int32[batch], or NULL) gives each sequence's filled length.
 *
 * ember_kv_cache_append: k_new, v_new are (batch, kv_heads, n_new, d); they are written at rows
 * [p, p + n_new) with p = seq_lens[b], or `pos` when seq_lens is NULL. Rows that do not fit are
 * skipped and reported through ember_check_device_status (EMBER_ERR_INVALID). The caller advances
 * its lengths.
 *
 * ember_attention_decode_cache: q and out are (batch, q_heads, d), q_heads a multiple of kv_heads
 * (1, 2, 4 or 8 times on the CUDA-core kernel, any multiple up to 128 on the tensor-core path); query head h reads K/V head h / (q_heads / kv_heads), and the K/V rows of a group
 * are loaded once for all its query heads. Sequence b attends to its first seq_lens[b] keys (each
 * >= 1), or to `lk` keys when seq_lens is NULL; with seq_lens, `lk` is an upper bound of the lengths
 * (it sizes the split of the key axis). lse (batch, q_heads) may be NULL. Workspace as for
 * ember_attention_decode, sized by ember_attention_decode_cache_workspace_bytes.
 * Kernels: bf16, d in {64, 128}, a contiguous cache and more than one query head per K/V head run
 * on the tensor cores (the group's query heads are the rows of one tile); everything else (one
 * query head per K/V head, float32, a page table, other head dimensions) on the CUDA-core kernel. */
EMBER_API int ember_kv_cache_append(void *k_cache, void *v_cache, const void *k_new, const void *v_new, int batch,
                                    int kv_heads, int capacity, int d, int n_new, int pos, const int *seq_lens,
                                    const int *block_table, int page_size, int max_blocks, int dtype, void *stream);
EMBER_API int ember_attention_decode_cache(const void *q, const void *k_cache, const void *v_cache, void *out, float *lse,
                                           int batch, int q_heads, int kv_heads, int lk, int capacity, int d, float scale,
                                           int dtype, const int *seq_lens, const int *block_table, int page_size,
                                           int max_blocks, int num_splits, void *workspace, size_t workspace_bytes,
                                           void *stream);
EMBER_API size_t ember_attention_decode_cache_workspace_bytes(int batch, int q_heads, int kv_heads, int lk, int d,
                                                              int num_splits);
EMBER_API int ember_attention_decode_cache_splits(int batch, int kv_heads, int lk);

#ifdef __cplusplus
}
#endif

#endif /* EMBER_B200_H */
