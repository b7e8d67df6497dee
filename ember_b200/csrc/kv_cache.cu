// Key/value cache for decode: append in place, decode over a cache that is longer than what is
// filled, per-sequence lengths, grouped-query heads (several query heads share one K/V head) and an
// optional page table.
//
// Layouts (row-major, element type f32 or bf16):
//   contiguous cache   K, V: (batch, kv_heads, capacity, d); sequence b has seq_lens[b] (or `lk`)
//                      valid keys at the front of its rows
//   paged cache        K, V: (num_pages, kv_heads, page_size, d); key j of sequence b lives in page
//                      block_table[b * max_blocks + j / page_size] at row j % page_size
//   queries / outputs  (batch, q_heads, d), q_heads = group * kv_heads; query head h reads K/V head
//                      h / group
//
// Two decode paths. With bf16 storage, head dimension 64 or 128, a contiguous cache and several
// query heads per K/V head, the step runs on the tensor cores: the forward kernel of
// attn_fwd_sm100.cu takes the group's query heads as the rows of one (zero-padded) 128-row tile, one
// CTA per (batch, kv_head, split) streams its keys by TMA, and a small kernel merges the splits'
// normalised partial outputs by their log-sum-exps. On CUDA cores the same step is bound by
// arithmetic as soon as four query heads share a key row (1.85 TB/s of cache traffic measured for
// groups of 4, no faster than reading the cache once per query head).
// Everything else (one query head per K/V head, float32, a page table, other head dimensions)
// runs the CUDA-core kernel below,
// the split-KV kernel of attn_decode.cu with one change that matters for
// bandwidth: a CTA owns one (batch, kv_head, split) and ALL `group` query heads that share it, so a
// K or V row is loaded from HBM once and used by every query head of the group (the cache is the
// only large stream of a decode step; with group = 4 the step moves a quarter of the bytes a
// per-query-head kernel would). Everything else is as there: 16-byte streaming loads, a key row
// spread over LPK lanes, per-lane-group online softmax in the exp2 domain, float32 partials and a
// log-sum-exp combine when the key axis is split.
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"

namespace ember {

namespace {

constexpr int KV_WARPS = 8;
constexpr int KV_THREADS = KV_WARPS * 32;
constexpr float LOG2E_KV = 1.4426950408889634f;
constexpr float LN2_KV = 0.6931471805599453f;

struct CacheGeom {
    int kv_heads, capacity, d;
    int page_shift, page_mask, max_blocks;  // paged cache: page_size = 1 << page_shift
    const int *block_table;                 // null: contiguous cache
    const int *seq_lens;                    // null: every sequence has `lk` keys
    int lk;
};

__device__ __forceinline__ size_t row_offset(const CacheGeom &g, int b, int hkv, int key)
{
    if (!g.block_table) return (((size_t)b * g.kv_heads + hkv) * g.capacity + key) * g.d;
    const int page = g.block_table[(size_t)b * g.max_blocks + (key >> g.page_shift)];
    return ((((size_t)page * g.kv_heads + hkv) << g.page_shift) + (key & g.page_mask)) * (size_t)g.d;
}

__device__ __forceinline__ uint4 ld_stream16(const void *p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <typename T>
struct V16;  // 16 bytes of T as floats
template <>
struct V16<__nv_bfloat16> {
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
struct V16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4 &u, float (&f)[4])
    {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
};

template <int N>
__device__ __forceinline__ void merge(float &m, float &l, float (&o)[N], float m2, float l2, const float (&o2)[N])
{
    const float mn = fmaxf(m, m2);
    const float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    const float b = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
    l = l * a + l2 * b;
#pragma unroll
    for (int i = 0; i < N; i++) o[i] = o[i] * a + o2[i] * b;
    m = mn;
}

// One-dimensional grid of splits * batch * kv_heads blocks (the splits of one K/V head are
// neighbours). G query heads per K/V head; LPK lanes share one key row.
template <typename T, int LPK, int G>
__global__ void __launch_bounds__(KV_THREADS)
    decode_gqa_kernel(const T *__restrict__ q, const T *__restrict__ kc, const T *__restrict__ vc, T *__restrict__ out,
                      float *__restrict__ lse, float *__restrict__ ws_o, float *__restrict__ ws_ml, const CacheGeom g,
                      int chunk, int splits, float scale_log2)
{
    constexpr int N = V16<T>::N;
    constexpr int KPW = 32 / LPK;              // keys per warp-wide load
    constexpr int UNROLL = G <= 2 ? 4 : 2;     // loads of K and of V in flight per warp
    const int unit = blockIdx.x / splits, split = blockIdx.x - unit * splits;
    const int b = unit / g.kv_heads, hkv = unit - b * g.kv_heads;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int slot = lane / LPK;               // key slot inside the warp
    const int col = (lane % LPK) * N;          // first column this lane owns
    const bool col_ok = col < g.d;
    const int q_heads = g.kv_heads * G;

    int len = g.seq_lens ? g.seq_lens[b] : g.lk;
    len = max(0, min(len, g.block_table ? (g.max_blocks << g.page_shift) : g.capacity));
    const int kbeg = split * chunk;
    const int kend = min(len, kbeg + chunk);

    float qf[G][N];
#pragma unroll
    for (int h = 0; h < G; h++) {
        uint4 qu = make_uint4(0, 0, 0, 0);
        if (col_ok) qu = *reinterpret_cast<const uint4 *>(q + ((size_t)b * q_heads + hkv * G + h) * g.d + col);
        V16<T>::unpack(qu, qf[h]);
#pragma unroll
        for (int i = 0; i < N; i++) qf[h][i] *= scale_log2;
    }
    float m[G], l[G], o[G][N];
#pragma unroll
    for (int h = 0; h < G; h++) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < N; i++) o[h][i] = 0.f;
    }

    for (int base = kbeg + warp * (KPW * UNROLL); base < kend; base += KV_WARPS * KPW * UNROLL) {
        uint4 ku[UNROLL], vu[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int key = base + u * KPW + slot;
            ok[u] = key < kend;
            ku[u] = make_uint4(0, 0, 0, 0);
            vu[u] = make_uint4(0, 0, 0, 0);
            if (ok[u] && col_ok) {
                const size_t off = row_offset(g, b, hkv, key) + col;
                ku[u] = ld_stream16(kc + off);
                vu[u] = ld_stream16(vc + off);
            }
        }
        float kf[UNROLL][N], vf[UNROLL][N];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            V16<T>::unpack(ku[u], kf[u]);
            V16<T>::unpack(vu[u], vf[u]);
        }
#pragma unroll
        for (int h = 0; h < G; h++) {
            float s[UNROLL];
            float mx = m[h];
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < N; i++) acc = fmaf(qf[h][i], kf[u][i], acc);
#pragma unroll
                for (int off = LPK / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                s[u] = ok[u] ? acc : -INFINITY;
                mx = fmaxf(mx, s[u]);
            }
            // a slot that has seen no key yet keeps m == -inf; 0 as its reference avoids inf - inf
            const float mref = (mx == -INFINITY) ? 0.f : mx;
            const float alpha = exp2f(m[h] - mref);
            m[h] = mx;
            l[h] *= alpha;
#pragma unroll
            for (int i = 0; i < N; i++) o[h][i] *= alpha;
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const float p = exp2f(s[u] - mref);
                l[h] += p;
#pragma unroll
                for (int i = 0; i < N; i++) o[h][i] = fmaf(p, vf[u][i], o[h][i]);
            }
        }
    }

    __shared__ float sm_o[KV_WARPS][LPK * N];
    __shared__ float sm_ml[KV_WARPS][2];
#pragma unroll
    for (int h = 0; h < G; h++) {
        // merge the key slots of this warp, then the warps through shared memory (one head at a time)
#pragma unroll
        for (int off = LPK; off < 32; off <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m[h], off);
            const float l2 = __shfl_xor_sync(0xffffffffu, l[h], off);
            float o2[N];
#pragma unroll
            for (int i = 0; i < N; i++) o2[i] = __shfl_xor_sync(0xffffffffu, o[h][i], off);
            merge<N>(m[h], l[h], o[h], m2, l2, o2);
        }
        __syncthreads();  // the previous head's partials have been read
        if (lane < LPK) {
#pragma unroll
            for (int i = 0; i < N; i++) sm_o[warp][col + i] = o[h][i];
            if (lane == 0) {
                sm_ml[warp][0] = m[h];
                sm_ml[warp][1] = l[h];
            }
        }
        __syncthreads();
        if (warp == 0 && lane < LPK) {
            float mm = m[h], ll = l[h], oo[N];
#pragma unroll
            for (int i = 0; i < N; i++) oo[i] = o[h][i];
#pragma unroll
            for (int w = 1; w < KV_WARPS; w++) {
                float o2[N];
#pragma unroll
                for (int i = 0; i < N; i++) o2[i] = sm_o[w][col + i];
                merge<N>(mm, ll, oo, sm_ml[w][0], sm_ml[w][1], o2);
            }
            const size_t row = (size_t)b * q_heads + hkv * G + h;  // which (batch, query head)
            if (splits == 1) {
                const float inv = ll > 0.f ? 1.f / ll : 0.f;  // an empty sequence gives zeros and lse = -inf
                if (col_ok) {
#pragma unroll
                    for (int i = 0; i < N; i++) {
                        if constexpr (sizeof(T) == 4)
                            out[row * g.d + col + i] = oo[i] * inv;
                        else
                            out[row * g.d + col + i] = __float2bfloat16_rn(oo[i] * inv);
                    }
                }
                if (lse && lane == 0) lse[row] = ll > 0.f ? (mm + log2f(ll)) * LN2_KV : -INFINITY;
            } else {
                float *po = ws_o + (row * splits + split) * (size_t)g.d;
                if (col_ok) {
#pragma unroll
                    for (int i = 0; i < N; i++) po[col + i] = oo[i];
                }
                if (lane == 0) {
                    ws_ml[(row * splits + split) * 2] = mm;
                    ws_ml[(row * splits + split) * 2 + 1] = ll;
                }
            }
        }
    }
}

// One block per (batch, query head); thread c merges column c over the splits.
template <typename T>
__global__ void gqa_combine_kernel(const float *__restrict__ ws_o, const float *__restrict__ ws_ml, T *__restrict__ out,
                                   float *__restrict__ lse, int d, int splits)
{
    const size_t row = blockIdx.x;
    const float *ml = ws_ml + row * splits * 2;
    float mx = -INFINITY;
    for (int s = 0; s < splits; s++) mx = fmaxf(mx, ml[2 * s]);
    float l = 0.f;
    for (int s = 0; s < splits; s++) {
        const float ms = ml[2 * s];
        if (ms != -INFINITY) l += ml[2 * s + 1] * exp2f(ms - mx);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;  // no split saw a key: zeros and lse = -inf
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) acc += ws_o[(row * splits + s) * (size_t)d + c] * exp2f(ms - mx);
        }
        if constexpr (sizeof(T) == 4)
            out[row * d + c] = acc * inv;
        else
            out[row * d + c] = __float2bfloat16_rn(acc * inv);
    }
    if (lse && threadIdx.x == 0) lse[row] = l > 0.f ? (mx + log2f(l)) * LN2_KV : -INFINITY;
}

// Copies n_new rows per (batch, kv_head) from (batch, kv_heads, n_new, d) into the cache at
// positions [pos_b, pos_b + n_new), pos_b = seq_lens[b] or `pos`. 16 bytes per thread.
__global__ void __launch_bounds__(256) kv_append_kernel(uint4 *__restrict__ kc, uint4 *__restrict__ vc,
                                                        const uint4 *__restrict__ kn, const uint4 *__restrict__ vn,
                                                        const CacheGeom g, int batch, int n_new, int pos, int vec_per_row,
                                                        int elems_per_vec, DeviceStatus *status)
{
    const size_t total = (size_t)batch * g.kv_heads * n_new * vec_per_row;
    const int limit = g.block_table ? (g.max_blocks << g.page_shift) : g.capacity;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int vcol = (int)(i % vec_per_row);
        size_t r = i / vec_per_row;
        const int j = (int)(r % n_new);
        r /= n_new;
        const int hkv = (int)(r % g.kv_heads), b = (int)(r / g.kv_heads);
        const int key = (g.seq_lens ? g.seq_lens[b] : pos) + j;
        if (key < 0 || key >= limit) {  // no room: skip the row and report it
            if (atomicCAS(&status->code, 0, EMBER_ERR_INVALID) == 0) {
                status->where = 301;
                status->block = b;
                status->extra = key;
            }
            continue;
        }
        const size_t dst = row_offset(g, b, hkv, key) / elems_per_vec + vcol;
        kc[dst] = kn[i];
        vc[dst] = vn[i];
    }
}

struct GqaArgs {
    const void *q, *kc, *vc;
    void *out;
    float *lse;
    int batch, q_heads, kv_heads, lk, capacity, d, dtype;
    float scale;
    const int *seq_lens, *block_table;
    int page_size, max_blocks;
};

CacheGeom make_geom(const GqaArgs &a)
{
    CacheGeom g;
    g.kv_heads = a.kv_heads;
    g.capacity = a.capacity;
    g.d = a.d;
    g.block_table = a.block_table;
    g.seq_lens = a.seq_lens;
    g.lk = a.lk;
    g.max_blocks = a.max_blocks;
    g.page_shift = 0;
    while (a.block_table && (1 << g.page_shift) < a.page_size) g.page_shift++;
    g.page_mask = (1 << g.page_shift) - 1;
    return g;
}

template <typename T, int LPK, int G>
int launch_gqa(const GqaArgs &a, int splits, int chunk, float *ws_o, float *ws_ml, cudaStream_t s)
{
    const unsigned grid = (unsigned)((long long)splits * a.batch * a.kv_heads);
    decode_gqa_kernel<T, LPK, G><<<grid, KV_THREADS, 0, s>>>((const T *)a.q, (const T *)a.kc, (const T *)a.vc, (T *)a.out,
                                                            a.lse, ws_o, ws_ml, make_geom(a), chunk, splits,
                                                            a.scale * LOG2E_KV);
    EMBER_CUDA_TRY(cudaGetLastError());
    if (splits > 1) {
        gqa_combine_kernel<T><<<a.batch * a.q_heads, 128, 0, s>>>(ws_o, ws_ml, (T *)a.out, a.lse, a.d, splits);
        EMBER_CUDA_TRY(cudaGetLastError());
    }
    return EMBER_OK;
}

template <typename T, int LPK>
int dispatch_group(const GqaArgs &a, int splits, int chunk, float *ws_o, float *ws_ml, cudaStream_t s)
{
    switch (a.q_heads / a.kv_heads) {
    case 1: return launch_gqa<T, LPK, 1>(a, splits, chunk, ws_o, ws_ml, s);
    case 2: return launch_gqa<T, LPK, 2>(a, splits, chunk, ws_o, ws_ml, s);
    case 4: return launch_gqa<T, LPK, 4>(a, splits, chunk, ws_o, ws_ml, s);
    case 8: return launch_gqa<T, LPK, 8>(a, splits, chunk, ws_o, ws_ml, s);
    default:
        set_error("decode: %d query heads per key/value head is not supported (1, 2, 4 or 8)", a.q_heads / a.kv_heads);
        return EMBER_ERR_UNSUPPORTED;
    }
}

template <typename T>
int dispatch_lanes(const GqaArgs &a, int splits, int chunk, float *ws_o, float *ws_ml, cudaStream_t s)
{
    const int lanes = (a.d + V16<T>::N - 1) / V16<T>::N;
    if (lanes <= 4) return dispatch_group<T, 4>(a, splits, chunk, ws_o, ws_ml, s);
    if (lanes <= 8) return dispatch_group<T, 8>(a, splits, chunk, ws_o, ws_ml, s);
    if (lanes <= 16) return dispatch_group<T, 16>(a, splits, chunk, ws_o, ws_ml, s);
    return dispatch_group<T, 32>(a, splits, chunk, ws_o, ws_ml, s);
}

size_t gqa_workspace_bytes(int rows, int d, int splits)
{
    if (splits <= 1) return 0;
    return align_up((size_t)rows * splits * d * sizeof(float), 256) + align_up((size_t)rows * splits * 2 * sizeof(float), 256);
}

int pick_splits(int batch, int kv_heads, int lk, int sm_count)
{
    return decode_pick_splits(batch * kv_heads, lk, 0, 0, sm_count);
}

// Tensor-core path: one CTA per (batch, kv_head, split) streams its keys through a 128-key pipeline,
// so a few CTAs per SM in total are enough; splits of at least 512 keys, in multiples of 128.
void tensor_core_split(int units, int lk, int sm_count, int requested, int &splits, int &chunk)
{
    if (sm_count <= 0) sm_count = 148;
    long long want = requested > 0 ? requested : (3LL * sm_count + units - 1) / units;
    const long long most = requested > 0 ? (lk + 127) / 128 : (lk + 511) / 512;
    if (want > most) want = most;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    chunk = (int)((lk + want - 1) / want);
    chunk = (chunk + 127) / 128 * 128;
    splits = (lk + chunk - 1) / chunk;
}

int check_cache(const char *fn, int batch, int q_heads, int kv_heads, int lk, int capacity, int d, int dtype,
                const int *block_table, int page_size, int max_blocks)
{
    EMBER_REQUIRE(dtype == EMBER_F32 || dtype == EMBER_BF16, "%s: unknown dtype %d", fn, dtype);
    EMBER_REQUIRE(batch > 0 && q_heads > 0 && kv_heads > 0 && d > 0, "%s: extents must be positive", fn);
    EMBER_REQUIRE(q_heads % kv_heads == 0, "%s: q_heads=%d is not a multiple of kv_heads=%d", fn, q_heads, kv_heads);
    const int vec = dtype == EMBER_BF16 ? 8 : 4;
    if (d % vec != 0 || d > 32 * vec) {
        set_error("%s: head dimension %d must be a multiple of %d and at most %d", fn, d, vec, 32 * vec);
        return EMBER_ERR_UNSUPPORTED;
    }
    if (block_table) {
        EMBER_REQUIRE(page_size >= 1 && (page_size & (page_size - 1)) == 0 && max_blocks > 0,
                      "%s: page_size=%d must be a power of two and max_blocks=%d positive", fn, page_size, max_blocks);
        EMBER_REQUIRE(lk <= (long long)page_size * max_blocks, "%s: lk=%d exceeds page_size*max_blocks", fn, lk);
    } else {
        EMBER_REQUIRE(capacity > 0 && lk <= capacity, "%s: lk=%d exceeds the cache capacity %d", fn, lk, capacity);
    }
    // the decode grid is one-dimensional: splits (at most 256 by the library's choice, at most lk
    // by request) times batch * kv_heads blocks
    if ((long long)batch * kv_heads > (0x7fffffffLL >> 8)) {
        set_error("%s: batch*kv_heads=%lld exceeds %lld", fn, (long long)batch * kv_heads, 0x7fffffffLL >> 8);
        return EMBER_ERR_UNSUPPORTED;
    }
    return EMBER_OK;
}

}  // namespace

}  // namespace ember

using namespace ember;

extern "C" {

int ember_kv_cache_append(void *k_cache, void *v_cache, const void *k_new, const void *v_new, int batch, int kv_heads,
                          int capacity, int d, int n_new, int pos, const int *seq_lens, const int *block_table,
                          int page_size, int max_blocks, int dtype, void *stream)
{
    int rc = check_cache("ember_kv_cache_append", batch, kv_heads, kv_heads, 0, capacity, d, dtype, block_table, page_size,
                         max_blocks);
    if (rc) return rc;
    EMBER_REQUIRE(k_cache && v_cache && k_new && v_new, "ember_kv_cache_append: NULL tensor pointer");
    EMBER_REQUIRE(n_new > 0, "ember_kv_cache_append: n_new must be positive, got %d", n_new);
    EMBER_REQUIRE((((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)k_new | (uintptr_t)v_new) & 15) == 0,
                  "ember_kv_cache_append: tensors must be 16-byte aligned");
    if (!seq_lens) {
        const long long limit = block_table ? (long long)page_size * max_blocks : capacity;
        EMBER_REQUIRE(pos >= 0 && (long long)pos + n_new <= limit,
                      "ember_kv_cache_append: rows [%d, %d) do not fit a cache of %lld rows", pos, pos + n_new, limit);
    }
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    GqaArgs a = {};
    a.kv_heads = kv_heads; a.capacity = capacity; a.d = d; a.seq_lens = seq_lens; a.block_table = block_table;
    a.page_size = page_size; a.max_blocks = max_blocks;
    const int elems_per_vec = dtype == EMBER_BF16 ? 8 : 4;
    const int vec_per_row = d / elems_per_vec;
    const size_t total = (size_t)batch * kv_heads * n_new * vec_per_row;
    const size_t want = (total + 255) / 256, cap = (size_t)(st->sm_count > 0 ? st->sm_count : 148) * 16;
    kv_append_kernel<<<(int)(want < cap ? want : cap), 256, 0, pick_stream(stream, st)>>>(
        (uint4 *)k_cache, (uint4 *)v_cache, (const uint4 *)k_new, (const uint4 *)v_new, make_geom(a), batch, n_new, pos,
        vec_per_row, elems_per_vec, st->status);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

int ember_attention_decode_cache_splits(int batch, int kv_heads, int lk)
{
    DeviceState *st = device_state();
    return pick_splits(batch, kv_heads, lk, st ? st->sm_count : 148);
}

size_t ember_attention_decode_cache_workspace_bytes(int batch, int q_heads, int kv_heads, int lk, int d, int num_splits)
{
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || lk <= 0 || d <= 0) return 0;
    int splits = num_splits > 0 ? num_splits : ember_attention_decode_cache_splits(batch, kv_heads, lk);
    if (splits > lk) splits = lk;
    size_t need = gqa_workspace_bytes(batch * q_heads, d, splits);
    // the tensor-core path (bf16, contiguous cache) makes its own split choice; cover both
    DeviceState *st = device_state();
    int tsplits, tchunk;
    tensor_core_split(batch * kv_heads, lk, st ? st->sm_count : 148, num_splits, tsplits, tchunk);
    const size_t tneed = sm100_cache_decode_workspace_bytes(batch * kv_heads, q_heads / kv_heads, d, tsplits);
    return tneed > need ? tneed : need;
}

int ember_attention_decode_cache(const void *q, const void *k_cache, const void *v_cache, void *out, float *lse, int batch,
                                 int q_heads, int kv_heads, int lk, int capacity, int d, float scale, int dtype,
                                 const int *seq_lens, const int *block_table, int page_size, int max_blocks,
                                 int num_splits, void *workspace, size_t workspace_bytes, void *stream)
{
    int rc = check_cache("ember_attention_decode_cache", batch, q_heads, kv_heads, lk, capacity, d, dtype, block_table,
                         page_size, max_blocks);
    if (rc) return rc;
    EMBER_REQUIRE(lk > 0, "ember_attention_decode_cache: lk must be positive, got %d", lk);
    EMBER_REQUIRE(isfinite(scale), "ember_attention_decode_cache: scale must be finite");
    EMBER_REQUIRE(q && k_cache && v_cache && out, "ember_attention_decode_cache: NULL tensor pointer");
    EMBER_REQUIRE((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0,
                  "ember_attention_decode_cache: q and the caches must be 16-byte aligned");
    DeviceState *st = device_state();
    if (!st) return EMBER_ERR_CUDA;
    cudaStream_t s = pick_stream(stream, st);
    if (!block_table && q_heads / kv_heads > 1) {
        // Grouped-query heads over a contiguous bf16 cache: tensor cores (the CUDA-core kernel below
        // is arithmetic-bound once several query heads share a key row).
        CacheDecodeArgs t;
        t.q = q; t.k_cache = k_cache; t.v_cache = v_cache; t.out = out; t.lse = lse;
        t.batch = batch; t.q_heads = q_heads; t.kv_heads = kv_heads; t.lk = lk; t.capacity = capacity; t.d = d;
        t.dtype = dtype; t.scale = scale; t.seq_lens = seq_lens;
        if (sm100_cache_decode_supported(t)) {
            tensor_core_split(batch * kv_heads, lk, st->sm_count, num_splits, t.splits, t.chunk);
            const size_t tneed = sm100_cache_decode_workspace_bytes(batch * kv_heads, q_heads / kv_heads, d, t.splits);
            if (tneed > 0) {
                if (!workspace || workspace_bytes < tneed) {
                    set_error("ember_attention_decode_cache: workspace of %zu bytes needed for %d splits, %zu given", tneed,
                              t.splits, workspace_bytes);
                    return EMBER_ERR_WORKSPACE;
                }
                EMBER_REQUIRE(((uintptr_t)workspace & 255) == 0, "ember_attention_decode_cache: workspace must be 256-byte aligned");
            }
            t.workspace = workspace;
            return sm100_cache_decode(t, st, s);
        }
    }
    int splits = num_splits > 0 ? num_splits : pick_splits(batch, kv_heads, lk, st->sm_count);
    if (splits > lk) splits = lk;
    const size_t need = gqa_workspace_bytes(batch * q_heads, d, splits);
    if (need > 0) {
        if (!workspace || workspace_bytes < need) {
            set_error("ember_attention_decode_cache: workspace of %zu bytes needed for %d splits, %zu given", need, splits,
                      workspace_bytes);
            return EMBER_ERR_WORKSPACE;
        }
        EMBER_REQUIRE(((uintptr_t)workspace & 255) == 0, "ember_attention_decode_cache: workspace must be 256-byte aligned");
    }
    int chunk = (lk + splits - 1) / splits;
    chunk = (chunk + 63) / 64 * 64;
    const int used = (lk + chunk - 1) / chunk;  // drop empty trailing chunks
    if ((long long)used * batch * kv_heads > 0x7fffffffLL) {
        set_error("ember_attention_decode_cache: %d splits of %d (batch, K/V head) pairs exceed the grid limit", used,
                  batch * kv_heads);
        return EMBER_ERR_UNSUPPORTED;
    }
    // The partial layout follows the split count the workspace was sized for only when it is used
    // as is; recompute the second block's offset from the splits actually launched.
    float *ws_o = (float *)workspace;
    float *ws_ml = used > 1 ? (float *)((char *)workspace + align_up((size_t)batch * q_heads * used * d * sizeof(float), 256))
                            : nullptr;
    GqaArgs a;
    a.q = q; a.kc = k_cache; a.vc = v_cache; a.out = out; a.lse = lse;
    a.batch = batch; a.q_heads = q_heads; a.kv_heads = kv_heads; a.lk = lk; a.capacity = capacity; a.d = d;
    a.dtype = dtype; a.scale = scale; a.seq_lens = seq_lens; a.block_table = block_table; a.page_size = page_size;
    a.max_blocks = max_blocks;
    if (dtype == EMBER_BF16) return dispatch_lanes<__nv_bfloat16>(a, used, chunk, ws_o, ws_ml, s);
    return dispatch_lanes<float>(a, used, chunk, ws_o, ws_ml, s);
}

}  // extern "C"
