// Projection GEMM for sm_100a: C (m x n) = op(A) * op(B) [+ bias], bf16 in and out, float32
// accumulation in tensor memory. It serves the Linear layers either side of attention:
//   forward          y  = x * w + b          (NN; y may be written head-major: the layout attention reads)
//   input gradient   dx = dy * w^T           (NT)
//   weight gradient  dw = x^T * dy           (TN)
// where x, dy and y may lie head-major (parts, batch, heads, seq, dim) instead of row-major, so that
// no transpose kernel runs between a projection and attention.
//
// Persistent kernel, one CTA per SM, CTAs in PAIRS (clusters of two, cta_group::2): a pair computes
// 256 x 256 output tiles, K in steps of 64. Each CTA of a pair
//   * loads its own 128 rows of A and its own 128 of the tile's 256 columns of B (its own TMA copies;
//     the completion bytes of both CTAs are counted by rank 0's barrier),
//   * receives its 128 rows x 256 columns of the result in its own tensor memory and writes them out.
// Rank 0 issues tcgen05.mma M=256 N=256 K=16 for both. A single CTA working alone on 128 x 256
// tiles reads 12 KB of operands per MMA and receives 48 KB per K step through the same 128 bytes
// per clock of shared-memory bandwidth, about 190 bytes per clock of demand: that form measured
// 0.70-0.76 of the library GEMM. In a pair each SM reads 8 KB per MMA and receives 32 KB per step.
//   warps 0-3  epilogue: accumulator (TMEM) + bias -> bf16 -> shared memory -> coalesced rows
//   warp  4    TMEM allocation (both CTAs), then MMA issue (rank 0; warp-collective, one elected lane)
//   warp  5    TMA producer (one lane): a ring of 6 stages of A (16 KB) and B (16 KB) tiles
// Two accumulators of 256 columns (all 512 TMEM columns): the MMAs of the next tile run while the
// epilogue drains the previous one.
// Operand tiles in shared memory use the 128-byte swizzle. An operand whose contraction index runs
// along its memory rows (K-major: A of NN/NT, B of NT) is one TMA box of 64 k x 128 rows;
// one whose contraction index runs across rows (MN-major: A of TN, B of NN/TN) is stored as
// sub-tiles of 64 k-rows x 64 columns, 8 KB apart.
#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace ember {

namespace {

using namespace ptx;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 6;  // BM: rows per CTA; a pair covers 2 * BM
constexpr int BNH = BN / 2;                             // B columns held by one CTA of a pair
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SUB_BYTES = 64 * 128;                   // 64 rows x 128 bytes
constexpr int OFF_OUT = STAGES * STAGE_BYTES;         // 128 rows x 128 columns of bf16 for the epilogue
constexpr int OFF_BIAS = OFF_OUT + BM * 128 * 2;      // 256 floats
constexpr int OFF_BAR = OFF_BIAS + BN * 4;
constexpr int USED_BYTES = OFF_BAR + 128;
constexpr int SMEM_BYTES = 232448;                    // the whole opt-in limit; the base is checked in the kernel
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;                           // tiles that share B columns run together

enum { B_FULL = 0, B_EMPTY = B_FULL + STAGES, B_ACCFULL = B_EMPTY + STAGES, B_ACCEMPTY = B_ACCFULL + 2, NUM_BARS = B_ACCEMPTY + 2 };
enum { WG_EMPTY = 201, WG_FULL, WG_ACCEMPTY, WG_ACCFULL, WG_SMEM };

struct ViewGeom {
    int heads, seq, dim;
};

struct GemmParams {
    long long m;
    int n, k;
    int tiles_m, tiles_n;
    ViewGeom a, b;
    MatView c;
    const __nv_bfloat16 *bias;
    DeviceStatus *status;
};

// TMA coordinates of a 64-column box of a view, walked along the contraction index. The producer
// computes coordinates on the critical path of every stage, so the divisions that split a row into
// (batch, position) and a column into (part, head, element) are done once per tile and the walk
// itself only adds and carries (all steps are 64; seq and dim are multiples of 64 for head-major
// views the kernel accepts).
struct BoxWalker {
    int c0, c1, c2, c3, c4;  // column | element, row | position, head, batch, part
    int heads, seq, dim;

    __device__ __forceinline__ void init(const ViewGeom &g, int row0, int col0)
    {
        heads = g.heads;
        seq = g.seq;
        dim = g.dim;
        if (heads == 0) {
            c0 = col0; c1 = row0; c2 = c3 = c4 = 0;
        } else {
            c3 = row0 / seq; c1 = row0 - c3 * seq;
            const int ph = col0 / dim;
            c0 = col0 - ph * dim;
            c4 = ph / heads; c2 = ph - c4 * heads;
        }
    }
    __device__ __forceinline__ void step_rows()  // 64 rows further
    {
        c1 += 64;
        if (heads != 0 && c1 >= seq) { c1 -= seq; c3++; }
    }
    __device__ __forceinline__ void step_cols()  // 64 columns further
    {
        c0 += 64;
        if (heads != 0 && c0 >= dim) {
            c0 = 0;
            if (++c2 >= heads) { c2 = 0; c4++; }
        }
    }
    __device__ __forceinline__ void load(uint32_t dst, const CUtensorMap *map, uint32_t bar) const
    {
        tma_load_5d_pair(dst, map, bar, c0, c1, c2, c3, c4);
    }
};

__device__ __forceinline__ void tile_coords(const GemmParams &p, int tile, int &tm, int &tn)
{
    const int per_group = GROUP_M * p.tiles_n;
    const int g = tile / per_group, rem = tile - g * per_group;
    const int rows_here = min(GROUP_M, p.tiles_m - g * GROUP_M);
    tn = rem / rows_here;
    tm = g * GROUP_M + (rem - tn * rows_here);
}

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    sm100_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    {   // every thread takes the same decision, before any barrier exists
        uint32_t dyn;
        asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        if (smem_base + USED_BYTES > smem_u32(smem_raw) + dyn) {
            if (threadIdx.x == 0 && atomicCAS(&p.status->code, 0, EMBER_ERR_UNSUPPORTED) == 0) {
                p.status->where = WG_SMEM;
                p.status->block = blockIdx.x;
                p.status->extra = (int)(smem_base - smem_u32(smem_raw));
            }
            return;
        }
    }
    const uint32_t bar0 = smem_base + OFF_BAR;
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + OFF_BAR + 8 * NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *bias_s = reinterpret_cast<float *>(smem_gen + OFF_BIAS);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles of 2*BM x BN, one per CTA pair at a time
    const int kblocks = (p.k + BK - 1) / BK;
    const uint32_t rank = cluster_ctarank();      // 0 issues the MMAs
    const int pair = blockIdx.x / 2, npairs = gridDim.x / 2;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(BAR(B_FULL + s), 1);   // rank 0: its producer's arrive + the bytes of both CTAs
            mbar_init(BAR(B_EMPTY + s), 1);  // one commit (delivered to both CTAs)
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(BAR(B_ACCFULL + b), 1);
            mbar_init(BAR(B_ACCEMPTY + b), 8);  // rank 0: one arrival per epilogue warp of both CTAs
        }
        fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);
        tmem_relinquish_pair();
    }
    if (warp == 5 && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 5) {
        if (lane == 0) {
            // ------------------------------------------------------------ TMA producer (both CTAs)
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                int tm, tn;
                tile_coords(p, tile, tm, tn);
                const int m0 = tm * 2 * BM + (int)rank * BM, n0 = tn * BN + (int)rank * BNH;  // this CTA's A rows and B columns
                constexpr int NA = MODE == GEMM_TN ? BM / 64 : 1, NB = MODE == GEMM_NT ? 1 : BNH / 64;
                BoxWalker wa[NA], wb[NB];
#pragma unroll
                for (int sub = 0; sub < NA; sub++)  // TN: A view is (k x m), boxes of 64 k-rows x 64 m-columns
                    wa[sub].init(p.a, MODE == GEMM_TN ? 0 : m0, MODE == GEMM_TN ? m0 + sub * 64 : 0);
#pragma unroll
                for (int sub = 0; sub < NB; sub++)  // NN, TN: B view is (k x n), boxes of 64 k-rows x 64 n-columns
                    wb[sub].init(p.b, MODE == GEMM_NT ? n0 : 0, MODE == GEMM_NT ? 0 : n0 + sub * 64);
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (!(ok = mbar_wait(BAR(B_EMPTY + s), ((it / STAGES) & 1) ^ 1, abort_flag, p.status, WG_EMPTY))) break;
                    const uint32_t a_dst = smem_base + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    if (rank == 0) mbar_arrive_expect_tx(BAR(B_FULL + s), 2 * STAGE_BYTES);
#pragma unroll
                    for (int sub = 0; sub < NA; sub++) {
                        wa[sub].load(a_dst + sub * SUB_BYTES, &tm_a, BAR(B_FULL + s));
                        if (MODE == GEMM_TN) wa[sub].step_rows(); else wa[sub].step_cols();
                    }
#pragma unroll
                    for (int sub = 0; sub < NB; sub++) {
                        wb[sub].load(b_dst + sub * SUB_BYTES, &tm_b, BAR(B_FULL + s));
                        if (MODE == GEMM_NT) wb[sub].step_cols(); else wb[sub].step_rows();
                    }
                }
            }
            // Do not leave while a copy of this pair is still landing in shared memory: rank 0's
            // barriers count the bytes of both CTAs, and the cluster barrier below keeps rank 1 here
            // until rank 0 has seen them.
            if (rank == 0) {
                const long long t0 = clock64();
                for (int j = max(0, it - STAGES); j < it; j++)
                    while (!mbar_try_wait(BAR(B_FULL + j % STAGES), (j / STAGES) & 1) && clock64() - t0 < kWaitLimitCycles) {}
            }
        }
    } else if (warp == 4) {
        // ---------------------------------------------------------------- MMA issue (rank 0 for the pair)
        if (rank == 0) {
            constexpr uint32_t IDESC = idesc_bf16_f32(2 * BM, BN, MODE == GEMM_TN ? 1 : 0, MODE == GEMM_NT ? 0 : 1);
            constexpr uint32_t A_LBO = MODE == GEMM_TN ? SUB_BYTES : 16, A_STEP = (MODE == GEMM_TN ? 2048 : 32) >> 4;
            constexpr uint32_t B_LBO = MODE == GEMM_NT ? 16 : SUB_BYTES, B_STEP = (MODE == GEMM_NT ? 32 : 2048) >> 4;
            int it = 0, tcount = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles; tile += npairs, tcount++) {
                const int buf = tcount & 1;
                ok = ok && mbar_wait(BAR(B_ACCEMPTY + buf), ((tcount >> 1) & 1) ^ 1, abort_flag, p.status, WG_ACCEMPTY);
                tc_fence_after();
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    ok = ok && mbar_wait(BAR(B_FULL + s), (it / STAGES) & 1, abort_flag, p.status, WG_FULL);
                    tc_fence_after();
                    const uint32_t a_lo = desc_lo(smem_base + s * STAGE_BYTES, A_LBO);
                    const uint32_t b_lo = desc_lo(smem_base + s * STAGE_BYTES + A_BYTES, B_LBO);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; k16++)
                        mma_ss_lo_pair(tmem + buf * BN, a_lo + k16 * A_STEP, b_lo + k16 * B_STEP, IDESC, (kb > 0 || k16 > 0) ? 1u : 0u);
                    tc_commit_pair(BAR(B_EMPTY + s), 3);  // the stage is free in both CTAs
                }
                tc_commit_pair(BAR(B_ACCFULL + buf), 3);
            }
        }
    } else {
        // -------------------------------------------------------------------- epilogue (warps 0-3, both CTAs)
        const int r = threadIdx.x;  // row inside this CTA's half of the tile == TMEM lane
        const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
        uint8_t *stage = smem_gen + OFF_OUT;
        __nv_bfloat16 *cptr = (__nv_bfloat16 *)p.c.ptr;
        const uint32_t accempty0 = map_to_cta(BAR(B_ACCEMPTY), 0);  // rank 0's barriers, as cluster addresses
        int tcount = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles; tile += npairs, tcount++) {
            int tm, tn;
            tile_coords(p, tile, tm, tn);
            const int buf = tcount & 1;
            const long long m0 = (long long)tm * 2 * BM + (long long)rank * BM;
            const int n0 = tn * BN;
            named_bar_sync(1, 128);  // the previous tile's bias has been read by every thread
            for (int j = r; j < BN; j += 128)
                bias_s[j] = (p.bias && n0 + j < p.n) ? __bfloat162float(p.bias[n0 + j]) : 0.f;
            named_bar_sync(1, 128);
            ok = ok && mbar_wait(BAR(B_ACCFULL + buf), (tcount >> 1) & 1, abort_flag, p.status, WG_ACCFULL);
            tc_fence_after();
            const uint32_t tacc = tmem + lane_sel + buf * BN;
#pragma unroll 1
            for (int half = 0; half < 2; half++) {
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t u[32];
                    tmem_ld_32x32b_x32(tacc + half * 128 + ch * 32, u);
                    tmem_wait_ld();
                    if (half == 1 && ch == 3) {  // the accumulator is in registers: the next tile may use it
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(accempty0 + 8u * (uint32_t)buf);
                    }
                    const float *bs = bias_s + half * 128 + ch * 32;
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {  // 8 columns = one 16-byte chunk
                        uint4 wv;
                        wv.x = pack_bf16(__uint_as_float(u[q4 * 8 + 0]) + bs[q4 * 8 + 0], __uint_as_float(u[q4 * 8 + 1]) + bs[q4 * 8 + 1]);
                        wv.y = pack_bf16(__uint_as_float(u[q4 * 8 + 2]) + bs[q4 * 8 + 2], __uint_as_float(u[q4 * 8 + 3]) + bs[q4 * 8 + 3]);
                        wv.z = pack_bf16(__uint_as_float(u[q4 * 8 + 4]) + bs[q4 * 8 + 4], __uint_as_float(u[q4 * 8 + 5]) + bs[q4 * 8 + 5]);
                        wv.w = pack_bf16(__uint_as_float(u[q4 * 8 + 6]) + bs[q4 * 8 + 6], __uint_as_float(u[q4 * 8 + 7]) + bs[q4 * 8 + 7]);
                        const int chunk = ch * 4 + q4;
                        const int sw = (chunk & ~7) | ((chunk ^ r) & 7);
                        *reinterpret_cast<uint4 *>(stage + r * 256 + sw * 16) = wv;
                    }
                }
                __syncwarp();
                // Each warp copies its own 32 rows: two rows of 16 chunks per instruction. The destination
                // of a chunk is found without divisions in the loop: this thread's column is fixed, and
                // the 128 rows of a CTA's tile are consecutive in memory rows (row-major: `cols` apart;
                // head-major: the tile lies inside one batch entry because seq is a multiple of 128, so
                // consecutive rows are `dim` apart).
                const int chunk = lane % 16;
                const int col = n0 + half * 128 + chunk * 8;
                const size_t row_stride = p.c.heads == 0 ? (size_t)p.c.cols : (size_t)p.c.dim;
                const size_t base = (m0 < p.m && col < p.n) ? view_offset(p.c, m0, col) : 0;
#pragma unroll 4
                for (int it2 = 0; it2 < 16; it2++) {
                    const int rr = warp * 32 + it2 * 2 + lane / 16;
                    const int sw = (chunk & ~7) | ((chunk ^ rr) & 7);
                    const uint4 wv = *reinterpret_cast<const uint4 *>(stage + rr * 256 + sw * 16);
                    const long long grow = m0 + rr;
                    if (ok && grow < p.m && col < p.n) *reinterpret_cast<uint4 *>(cptr + base + (size_t)rr * row_stride) = wv;
                }
                __syncwarp();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers or use the shared allocation
    if (warp == 4) tmem_dealloc_pair(tmem, 512);
}

bool view_ok(const MatView &v, int row_box)
{
    if (((uintptr_t)v.ptr & 15) != 0) return false;
    if (v.heads == 0) return v.cols % 8 == 0;
    // head-major: a box of 64 columns must stay inside one head and a box of rows inside one batch entry
    return v.dim % 64 == 0 && v.seq % row_box == 0 && v.rows % v.seq == 0 && v.cols % (v.heads * v.dim) == 0;
}

template <int MODE>
int launch(const GemmArgs &g, DeviceState *st, cudaStream_t s)
{
    CUtensorMap ta, tb;
    int rc;
    if ((rc = make_tensor_map_bf16_view(&ta, g.a, 64, MODE == GEMM_TN ? 64 : BM)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_view(&tb, g.b, 64, MODE == GEMM_NT ? BNH : 64)) != EMBER_OK) return rc;
    GemmParams p;
    p.m = g.m;
    p.n = g.n;
    p.k = g.k;
    p.tiles_m = (int)((g.m + 2 * BM - 1) / (2 * BM));
    p.tiles_n = (g.n + BN - 1) / BN;
    p.a = {g.a.heads, g.a.seq, g.a.dim};
    p.b = {g.b.heads, g.b.seq, g.b.dim};
    p.c = g.c;
    p.bias = (const __nv_bfloat16 *)g.bias;
    p.status = st->status;
    auto kern = sm100_gemm_kernel<MODE>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const int sms = st->sm_count > 0 ? st->sm_count : 148;
    const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;  // consecutive CTAs 2i, 2i+1 form a pair
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
    return EMBER_OK;
}

}  // namespace

bool sm100_gemm_supported(const GemmArgs &g)
{
    if (g.dtype != EMBER_BF16 || g.m <= 0 || g.n <= 0 || g.k <= 0) return false;
    if (g.m > 0x7fffff00LL || g.a.rows > 0x7fffff00LL || g.b.rows > 0x7fffff00LL) return false;  // 32-bit box coordinates
    if ((g.m + 2 * BM - 1) / (2 * BM) * (long long)((g.n + BN - 1) / BN) > 0x7fffffffLL) return false;
    if (g.n % 8 != 0 || ((uintptr_t)g.c.ptr & 15) != 0) return false;       // 16-byte output chunks
    if (g.c.heads > 0 && (g.c.dim % 8 != 0 || g.c.seq % BM != 0)) return false;  // a CTA's 128 result rows lie in one batch entry
    const int a_rows = g.mode == GEMM_TN ? 64 : BM, b_rows = g.mode == GEMM_NT ? BNH : 64;
    return view_ok(g.a, a_rows) && view_ok(g.b, b_rows);
}

int sm100_gemm(const GemmArgs &g, DeviceState *st, cudaStream_t s)
{
    switch (g.mode) {
    case GEMM_NN: return launch<GEMM_NN>(g, st, s);
    case GEMM_NT: return launch<GEMM_NT>(g, st, s);
    default: return launch<GEMM_TN>(g, st, s);
    }
}

}  // namespace ember
