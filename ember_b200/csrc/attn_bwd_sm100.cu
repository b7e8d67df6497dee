// Attention backward for sm_100a: bf16 in/out, float32 recompute of P from the saved log-sum-exp,
// float32 accumulation in tensor memory. Two kernels plus the delta preprocess:
//
//   delta[row] = sum_c dO[row][c] * O[row][c]                      (CUDA cores, attn_simt.cu)
//
//   dK/dV kernel: one CTA per (batch*head, 128-key tile), looping over the 128-row query tiles that
//     can see those keys. Scores are formed TRANSPOSED so that keys sit on the TMEM lanes:
//       S^T  = K Q^T          dP^T = V dO^T                       (smem x smem -> TMEM)
//       P^T  = exp2(S^T*c - lse*log2e)     dS^T = P^T * (dP^T - delta)   (registers, bf16 -> TMEM)
//       dV  += P^T dO         dK  += dS^T Q                       (TMEM x smem -> TMEM)
//     TMEM: S^T 128 + dP^T 128 + dV HD + dK HD columns -- full at HD = 128, so no dQ accumulator
//     fits next to them; dQ gets its own pass:
//
//   dQ kernel: one CTA per (batch*head, 128-row query tile), looping over the key tiles it sees:
//       S = Q K^T   dP = dO V^T   dS = P * (dP - delta)   dQ += dS K
//
// Both results are deterministic (no atomics). The scale factor of dS is applied once, to the
// accumulated dK / dQ, in the epilogue.
//
// Each kernel is software-pipelined over its tiles in two phases so that the tensor core works
// while the compute warps do: in the dK/dV kernel the exponentials of tile i+1 run while
// dK(i) and dP^T(i+1) are multiplied, and dS^T(i+1) is formed while dV(i+1) and S^T(i+2) are; the
// dQ kernel issues S(j+1) as soon as S(j) has been read into registers. Half of the
// exponentials are evaluated as a polynomial on the FMA pipe to keep the MUFU off the critical path.
//
//   warps 0-7   compute: thread (row r, slice h) owns TMEM lane r and 64 of the 128 score columns
//   warp  8     MMA issue, score chain:    S^T(i+1) and dV(i)   (dQ kernel: S(j+1))
//   warp  9     MMA issue, gradient chain: dP^T(i+1) and dK(i)  (dQ kernel: dQ(j) and dP(j+1))
//               Two issuing warps on different schedulers: each chain only orders MMAs that share
//               TMEM columns, and one warp's barrier waits no longer delay the other chain.
//   warp  10    TMA producer (one lane)       warp 11  TMEM allocation
#include <math.h>

#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace ember {

namespace {

using namespace ptx;

// Compute warps: every TMEM lane quarter is served by NCW/4 warps, each thread owning CPT of the 128
// score columns of its lane. Eight warps (two per scheduler, 64 columns per thread) and sixteen
// (four per scheduler, 32 columns) measured the same; eight is the default.
#ifndef BWD_COMPUTE_WARPS
#define BWD_COMPUTE_WARPS 8
#endif
constexpr int NCW = BWD_COMPUTE_WARPS;
constexpr int CPT = 128 / (NCW / 4);   // score columns per thread: 64 or 32
constexpr int NCT = NCW * 32;          // compute threads
constexpr int BWD_THREADS = (NCW + 4) * 32;
constexpr int W_MMA_A = NCW, W_MMA_B = NCW + 1, W_TMA = NCW + 2, W_ALLOC = NCW + 3;
constexpr float LOG2E_B = 1.4426950408889634f;

template <int HD>
struct BwdCfg {
    static constexpr int NSUB = HD / 64;
    static constexpr int SUB_BYTES = 128 * 128;
    static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
    // Two rings of streamed tiles. Ring A holds the operand that stays in use until the END of an
    // iteration (Q in the dK/dV kernel: last read by dK; K in the dQ kernel: last read by dQ), so its
    // next-but-one tile can only start loading late; three buffers keep that TMA latency off the
    // critical path. Ring B (dO, resp. V) is released in the first half of an iteration; two suffice.
    static constexpr int NA = 3, NB = 2;
    static constexpr int OFF_RES0 = 0;                  // resident tile 0 (K, or Q)
    static constexpr int OFF_RES1 = TILE_BYTES;         // resident tile 1 (V, or dO)
    static constexpr int OFF_A = 2 * TILE_BYTES;
    static constexpr int OFF_B = OFF_A + NA * TILE_BYTES;
    static constexpr int OFF_BAR = OFF_B + NB * TILE_BYTES;
    static constexpr int OFF_ROWVEC = OFF_BAR + 160;    // [2 buffers][2 vectors][128] floats
    static constexpr int USED_BYTES = OFF_ROWVEC + 2048;
    // 7 tiles of 32 KB leave 864 bytes below the 227 KB limit at HD = 128: that is the room for
    // rounding the dynamic shared memory base up to 1024 bytes (the kernel checks that it fits).
    static constexpr int SMEM_BYTES = HD == 128 ? 232448 : USED_BYTES + 1024;
    static constexpr int T_S = 0, T_DP = 128, T_ACC0 = 256, T_ACC1 = 256 + HD;
    // barrier indices
    static constexpr int B_RES = 0, B_FULLA = 1, B_EMPTYA = B_FULLA + NA, B_FULLB = B_EMPTYA + NA,
                         B_EMPTYB = B_FULLB + NB,
                         B_S = B_EMPTYB + NB,      // S (or S^T) of the current tile is in TMEM
                         B_DP = B_S + 1,           // dP (or dP^T) is in TMEM
                         B_P = B_DP + 1,           // dK/dV: P^T written; dQ: S has been read (8 warp arrivals)
                         B_DS = B_P + 1,           // dS (or dS^T) written (8 warp arrivals)
                         B_ACC = B_DS + 1,
                         B_DP1 = B_ACC + 1,        // dQ kernel: second dP / dS buffer (odd key tiles)
                         B_DS1 = B_DP1 + 1, NUM_BARS = B_DS1 + 1;
};

enum { WB_RES = 101, WB_FULL, WB_EMPTY, WB_S, WB_DP, WB_P, WB_DS, WB_ACC, WB_SMEM };

struct BwdParams {
    __nv_bfloat16 *dq, *dk, *dv;
    const float *lse, *delta;
    int lq, lk, causal;
    int d;  // elements per row in memory (a multiple of 8, <= HD): the TMA copies read the columns past d
            // as zero, so the accumulators' columns past d are zero too and the epilogues skip them
    float scale, scale_log2;
    DeviceStatus *status;
    WorkOrder order;  // set per launch
};

// Common prologue: barriers, TMEM allocation, tensor-map prefetch. Returns the TMEM base.
template <typename C>
__device__ __forceinline__ uint32_t bwd_setup(uint32_t smem_base, uint8_t *smem_gen, int warp, int lane,
                                              const CUtensorMap *m0, const CUtensorMap *m1,
                                              const CUtensorMap *m2, const CUtensorMap *m3, int empty_b_count)
{
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar0 + 8 * C::B_RES, 1);
        for (int s = 0; s < C::NA; s++) {
            mbar_init(bar0 + 8 * (C::B_FULLA + s), 1);
            mbar_init(bar0 + 8 * (C::B_EMPTYA + s), 2);  // released by both MMA warps
        }
        for (int s = 0; s < C::NB; s++) {
            mbar_init(bar0 + 8 * (C::B_FULLB + s), 1);
            mbar_init(bar0 + 8 * (C::B_EMPTYB + s), empty_b_count);
        }
        mbar_init(bar0 + 8 * C::B_S, 1);
        mbar_init(bar0 + 8 * C::B_DP, 1);
        mbar_init(bar0 + 8 * C::B_P, NCW);   // one arrival per compute warp
        mbar_init(bar0 + 8 * C::B_DS, NCW);
        mbar_init(bar0 + 8 * C::B_ACC, 2);  // one commit from each MMA warp
        mbar_init(bar0 + 8 * C::B_DP1, 1);
        mbar_init(bar0 + 8 * C::B_DS1, NCW);
        fence_mbar_init();
    }
    if (warp == W_ALLOC) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    if (warp == W_TMA && lane == 0) {
        prefetch_tensormap(m0);
        prefetch_tensormap(m1);
        prefetch_tensormap(m2);
        prefetch_tensormap(m3);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return *tmem_slot;
}

// Bounded drain of the producer's outstanding copies before the CTA may exit.
template <typename C>
__device__ __forceinline__ void drain_copies(uint32_t bar0, int issued_a, int issued_b)
{
    const long long t0 = clock64();
    for (int j = max(0, issued_a - C::NA); j < issued_a; j++)
        while (!mbar_try_wait(bar0 + 8 * (C::B_FULLA + j % C::NA), (j / C::NA) & 1) &&
               clock64() - t0 < kWaitLimitCycles) {}
    for (int j = max(0, issued_b - C::NB); j < issued_b; j++)
        while (!mbar_try_wait(bar0 + 8 * (C::B_FULLB + j % C::NB), (j / C::NB) & 1) &&
               clock64() - t0 < kWaitLimitCycles) {}
    while (!mbar_try_wait(bar0 + 8 * C::B_RES, 0) && clock64() - t0 < kWaitLimitCycles) {}
}

// The kernels round the dynamic shared memory base up to 1024 bytes; true when the rounded layout
// still fits in what was allocated. Otherwise the CTA records the fact and returns at once (every
// thread takes the same decision, before any barrier exists).
template <typename C>
__device__ __forceinline__ bool smem_layout_fits(uint32_t raw_base, uint32_t aligned_base, DeviceStatus *status)
{
    uint32_t dyn;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (aligned_base + C::USED_BYTES <= raw_base + dyn) return true;
    if (threadIdx.x == 0 && atomicCAS(&status->code, 0, EMBER_ERR_UNSUPPORTED) == 0) {
        status->where = WB_SMEM;
        status->block = blockIdx.x;
        status->extra = (int)(aligned_base - raw_base);
    }
    return false;
}

__device__ __forceinline__ void compute_reg_alloc()
{
    if constexpr (NCW == 8)
        reg_alloc_232();
    else
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");  // 16 x 32 x 104 + 4 x 32 x 40 <= 65536
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Loads N (16, 32 or 64) consecutive float32 columns of this thread's TMEM lane.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float (&v)[N])
{
    if constexpr (N == 16) {
        uint32_t u[16];
        tmem_ld_32x32b_x16(taddr, u);
#pragma unroll
        for (int x = 0; x < 16; x++) v[x] = __uint_as_float(u[x]);
    } else {
#pragma unroll
        for (int ch = 0; ch < N / 32; ch++) {
            uint32_t u[32];
            tmem_ld_32x32b_x32(taddr + ch * 32, u);
#pragma unroll
            for (int x = 0; x < 32; x++) v[ch * 32 + x] = __uint_as_float(u[x]);
        }
    }
    tmem_wait_ld();
}

// Epilogue helpers. A thread owns a whole accumulator row, and storing rows straight to global
// memory makes every store instruction touch 32 different lines; the results therefore go through
// shared memory (a resident operand tile that is no longer needed) and leave as coalesced rows.
// 16-byte chunks are XOR-swizzled by the row so that neither phase has bank conflicts.
//
// stage_acc: accumulator (TMEM, fp32, 128 x HD) times `mul` -> bf16 rows of a 128 x (HD*2 bytes)
// shared tile; thread (r, h) writes columns [h*HD/2, (h+1)*HD/2) of row r.
template <int HD>
__device__ __forceinline__ void stage_acc(uint32_t tacc, uint8_t *stage, int r, int h, float mul)
{
    constexpr int ROWB = HD * 2, COLS = HD / (NCW / 4);  // columns of this thread: 64, 32 or 16
    float o[COLS];
    tmem_ld_cols<COLS>(tacc + h * COLS, o);
#pragma unroll
    for (int q4 = 0; q4 < COLS / 8; q4++) {  // 8 columns = one 16-byte chunk
        uint4 wv;
        wv.x = pack_bf16(o[q4 * 8 + 0] * mul, o[q4 * 8 + 1] * mul);
        wv.y = pack_bf16(o[q4 * 8 + 2] * mul, o[q4 * 8 + 3] * mul);
        wv.z = pack_bf16(o[q4 * 8 + 4] * mul, o[q4 * 8 + 5] * mul);
        wv.w = pack_bf16(o[q4 * 8 + 6] * mul, o[q4 * 8 + 7] * mul);
        const int chunk = h * (COLS / 8) + q4;
        const int sw = (chunk & ~7) | ((chunk ^ r) & 7);
        *reinterpret_cast<uint4 *>(stage + r * ROWB + sw * 16) = wv;
    }
}

// store_staged: after all compute threads have staged (caller synchronises), compute warp w8 copies
// its 128/NCW rows of the tile to global memory, whole rows per instruction.
// gtile points at row 0 of the tile in the (rows x d) global matrix, d <= HD elements per row; rows >=
// rows_valid and the 16-byte chunks past column d are skipped.
// (tensor, tensor_bytes, status: the whole destination tensor, for the bounds-checked debug build)
template <int HD>
__device__ __forceinline__ void store_staged(const uint8_t *stage, __nv_bfloat16 *gtile, int d, int rows_valid, int w8,
                                             int lane, const void *tensor, size_t tensor_bytes, DeviceStatus *status)
{
    constexpr int ROWB = HD * 2, CHUNKS = ROWB / 16, ROWS_PER_ST = 32 / CHUNKS, ROWS_PER_WARP = 128 / NCW;
    const int chunk = lane % CHUNKS;
#pragma unroll
    for (int it = 0; it < ROWS_PER_WARP / ROWS_PER_ST; it++) {
        const int rr = w8 * ROWS_PER_WARP + it * ROWS_PER_ST + lane / CHUNKS;
        const int sw = (chunk & ~7) | ((chunk ^ rr) & 7);
        const uint4 wv = *reinterpret_cast<const uint4 *>(stage + rr * ROWB + sw * 16);
        __nv_bfloat16 *dst = gtile + (size_t)rr * d + chunk * 8;
        if (rr < rows_valid && chunk * 8 < d && EMBER_STORE_OK(dst, tensor, tensor_bytes, 16, status))
            *reinterpret_cast<uint4 *>(dst) = wv;
    }
}

#ifndef BWD_EMU_PAIRS_OF_4
#define BWD_EMU_PAIRS_OF_4 2  // pairs per group of 4 whose exponentials avoid the MUFU (128 columns)
#endif
// At 64 columns every exponential goes through the MUFU: a tile pair has half the tensor and
// shared-memory work there, the compute warps' instruction issue is the limit, and the polynomial costs
// more instructions than it frees MUFU slots (measured at 128 units x L4096: 1.57 against 1.70 ms without
// a mask, 0.906 against 0.913 ms causal).
template <int HD>
struct BwdEmu {
    static constexpr int PAIRS_OF_4 = HD >= 128 ? BWD_EMU_PAIRS_OF_4 : 0;
};

// p = 2^x for a pair, through the MUFU or the FMA-pipe polynomial depending on the pair's position
template <int EMU_OF_4>
__device__ __forceinline__ void exp2_pair(f32x2 x2, int pair_index, float &p0, float &p1)
{
    if (pair_index % 4 < EMU_OF_4) {
        exp2_poly2(x2, p0, p1);
    } else {
        float x0, x1;
        unpack2(x2, x0, x1);
        p0 = ex2(x0);
        p1 = ex2(x1);
    }
}

__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// After this warp's TMEM stores (or loads) are complete: one arrival per warp on `bar`.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane)
{
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// ------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    sm100_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                          const BwdParams p)
{
    using C = BwdCfg<HD>;
    constexpr int EMPTY_B = 2;  // dO is read by both MMA chains (dP^T and dV)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    if (!smem_layout_fits<C>(smem_u32(smem_raw), smem_base, p.status)) return;
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile int *abort_flag =
        reinterpret_cast<volatile int *>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS + 4);
    float *rowvec = reinterpret_cast<float *>(smem_gen + C::OFF_ROWVEC);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    int bh, rank;
    work_item(p.order, blockIdx.x, bh, rank);
    const int k0 = rank * 128;  // under a causal mask the first key blocks are seen by the most queries
    const int off = p.lk - p.lq;
    const int i_begin = p.causal ? max(0, k0 - off) / 128 : 0;  // first query tile that sees key k0
    const int n = (p.lq + 127) / 128 - i_begin;

    const uint32_t tmem = bwd_setup<C>(smem_base, smem_gen, warp, lane, &tm_q, &tm_k, &tm_v, &tm_do, EMPTY_B);

    if (warp >= NCW) {
        reg_dealloc_40();
        if (warp == W_TMA && lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            mbar_arrive_expect_tx(BAR(C::B_RES), 2 * C::TILE_BYTES);
            for (int s = 0; s < C::NSUB; s++) {
                tma_load_3d(smem_base + C::OFF_RES0 + s * C::SUB_BYTES, &tm_k, BAR(C::B_RES), s * 64, k0, bh);
                tma_load_3d(smem_base + C::OFF_RES1 + s * C::SUB_BYTES, &tm_v, BAR(C::B_RES), s * 64, k0, bh);
            }
            int issued_a = 0, issued_b = 0;
            for (int i = 0; i < n; i++) {
                const int sa = i % C::NA, sb = i % C::NB;
                const int q0 = (i_begin + i) * 128;
                if (!mbar_wait(BAR(C::B_EMPTYA + sa), ((i / C::NA) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLA + sa), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_A + sa * C::TILE_BYTES + s * C::SUB_BYTES, &tm_q,
                                BAR(C::B_FULLA + sa), s * 64, q0, bh);
                issued_a = i + 1;
                if (!mbar_wait(BAR(C::B_EMPTYB + sb), ((i / C::NB) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLB + sb), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_B + sb * C::TILE_BYTES + s * C::SUB_BYTES, &tm_do,
                                BAR(C::B_FULLB + sb), s * 64, q0, bh);
                issued_b = i + 1;
            }
            drain_copies<C>(bar0, issued_a, issued_b);
        } else if (warp == W_MMA_A || warp == W_MMA_B) {  // all 32 lanes, converged; one elected lane issues
            // ---------------------------------------------------------------- MMA issue
            constexpr uint32_t IDESC_SS = idesc_bf16_f32(128, 128, 0, 0);
            constexpr uint32_t IDESC_TS = idesc_bf16_f32(128, HD, 0, 1);
            const uint32_t ka = smem_base + C::OFF_RES0, va = smem_base + C::OFF_RES1;
            const uint32_t k_lo = desc_lo(ka, 16), v_lo = desc_lo(va, 16);
            auto q_addr = [&](int i) { return smem_base + C::OFF_A + (i % C::NA) * C::TILE_BYTES; };
            auto do_addr = [&](int i) { return smem_base + C::OFF_B + (i % C::NB) * C::TILE_BYTES; };
            auto issue_st = [&](int i) {  // S^T = K Q^T
                const uint32_t q_lo = desc_lo(q_addr(i), 16);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                    mma_ss_lo(tmem + C::T_S, k_lo + o16, q_lo + o16, IDESC_SS, ks > 0);
                }
                tc_commit_elect(BAR(C::B_S));
            };
            auto issue_dpt = [&](int i) {  // dP^T = V dO^T
                const uint32_t do_lo = desc_lo(do_addr(i), 16);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                    mma_ss_lo(tmem + C::T_DP, v_lo + o16, do_lo + o16, IDESC_SS, ks > 0);
                }
                tc_commit_elect(BAR(C::B_DP));
            };
            bool ok = mbar_wait(BAR(C::B_RES), 0, abort_flag, p.status, WB_RES);
            if (warp == W_MMA_A) {
                // score chain: S^T(0); then per tile dV(i) (reads P^T, dO) and S^T(i+1) (overwrites P^T)
                ok = ok && mbar_wait(BAR(C::B_FULLA + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_st(0);
                for (int i = 0; i < n && ok; i++) {
                    const uint32_t domn_lo = desc_lo(do_addr(i), C::SUB_BYTES);
                    ok = ok && mbar_wait(BAR(C::B_FULLB + i % C::NB), (i / C::NB) & 1, abort_flag, p.status, WB_FULL);
                    ok = ok && mbar_wait(BAR(C::B_P), i & 1, abort_flag, p.status, WB_P);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)  // dV += P^T dO
                        mma_ts_lo(tmem + C::T_ACC0, tmem + C::T_S + ks * 8, domn_lo + ks * (2048 >> 4), IDESC_TS,
                                  (i > 0 || ks > 0) ? 1u : 0u);
                    tc_commit_elect(BAR(C::B_EMPTYB + i % C::NB));  // this chain's last read of dO(i)
                    if (i + 1 < n) {
                        ok = ok && mbar_wait(BAR(C::B_FULLA + (i + 1) % C::NA), ((i + 1) / C::NA) & 1, abort_flag,
                                             p.status, WB_FULL);
                        tc_fence_after();
                        issue_st(i + 1);  // overwrites P^T(i): ordered after dV(i) by issue order
                    }
                    tc_commit_elect(BAR(C::B_EMPTYA + i % C::NA));  // this chain's last read of Q(i) was S^T(i)
                }
                tc_commit_elect(BAR(C::B_ACC));
            } else {
                // gradient chain: dP^T(0); then per tile dK(i) (reads dS^T, Q) and dP^T(i+1) (overwrites dS^T)
                ok = ok && mbar_wait(BAR(C::B_FULLB + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_dpt(0);
                for (int i = 0; i < n && ok; i++) {
                    const uint32_t qmn_lo = desc_lo(q_addr(i), C::SUB_BYTES);
                    ok = ok && mbar_wait(BAR(C::B_FULLA + i % C::NA), (i / C::NA) & 1, abort_flag, p.status, WB_FULL);
                    ok = ok && mbar_wait(BAR(C::B_DS), i & 1, abort_flag, p.status, WB_DS);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)  // dK += dS^T Q
                        mma_ts_lo(tmem + C::T_ACC1, tmem + C::T_DP + ks * 8, qmn_lo + ks * (2048 >> 4), IDESC_TS,
                                  (i > 0 || ks > 0) ? 1u : 0u);
                    tc_commit_elect(BAR(C::B_EMPTYA + i % C::NA));  // this chain's last read of Q(i)
                    if (i + 1 < n) {
                        ok = ok && mbar_wait(BAR(C::B_FULLB + (i + 1) % C::NB), ((i + 1) / C::NB) & 1, abort_flag,
                                             p.status, WB_FULL);
                        tc_fence_after();
                        issue_dpt(i + 1);  // overwrites dS^T(i): ordered after dK(i)
                    }
                    tc_commit_elect(BAR(C::B_EMPTYB + i % C::NB));  // this chain's last read of dO(i) was dP^T(i)
                }
                tc_commit_elect(BAR(C::B_ACC));
            }
        }
    } else {
        // -------------------------------------------------------------------- compute
        compute_reg_alloc();
        const int h = warp / 4;                // which CPT-column slice of the 128 score columns
        const int r = threadIdx.x % 128;       // TMEM lane == key row inside the tile
        const int key = k0 + r;
        const uint32_t lane_sel = (uint32_t)((warp % 4) * 32) << 16;
        const uint32_t t_s = tmem + lane_sel + C::T_S, t_dp = tmem + lane_sel + C::T_DP;
        const float c = p.scale_log2;
        const float *lse_g = p.lse + (size_t)bh * p.lq;
        const float *delta_g = p.delta + (size_t)bh * p.lq;
        bool ok = true;
        // This thread's element of the next tile's row vectors (threads 0-127: lse, threads 128-255:
        // delta) is fetched from global memory one tile ahead so that its latency is hidden. The load
        // is a volatile asm (the compiler must not sink it next to its use) and its value is not
        // touched until the next iteration (any arithmetic on it here would wait for the load).
        const float *rowvec_src = (threadIdx.x < 128 ? lse_g : delta_g);
        auto fetch_raw = [&](int i) -> float {
            const int qrow = (i_begin + i) * 128 + (threadIdx.x & 127);
            float v = 0.f;
            if (threadIdx.x < 256 && i < n && qrow < p.lq) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(rowvec_src + qrow));
            return v;
        };
        float raw_next = fetch_raw(0);
        for (int i = 0; i < n; i++) {
            const int q0 = (i_begin + i) * 128;
            float *rv = rowvec + (i & 1) * 256;
            {
                const bool in_range = q0 + (threadIdx.x & 127) < p.lq;
                if (threadIdx.x < 256)
                    rv[threadIdx.x] = threadIdx.x < 128 ? (in_range ? -raw_next * LOG2E_B : -INFINITY) : (in_range ? raw_next : 0.f);
            }
            raw_next = fetch_raw(i + 1);
            // ---- phase 1: P^T = exp2(S^T * c - lse2), bf16 into TMEM for dV += P^T dO
            ok = ok && mbar_wait(BAR(C::B_S), i & 1, abort_flag, p.status, WB_S);
            tc_fence_after();
            float pv[CPT];
            tmem_ld_cols<CPT>(t_s + h * CPT, pv);
            // Every thread has read its scores (the bf16 P^T overwrites columns another thread of the
            // same lane still needs) and the lse/delta vectors are visible.
            named_bar_sync(1, NCT);
            if (p.causal && (k0 + 127 > q0 + off)) {  // tile crossed by the diagonal: mask before the exp
                const float masked = c > 0.f ? -INFINITY : INFINITY;
#pragma unroll
                for (int cc = 0; cc < CPT; cc++)
                    if (key > q0 + h * CPT + cc + off) pv[cc] = masked;
            }
            const f32x2 c2 = pack2(c, c);
#pragma unroll
            for (int ch = 0; ch < CPT / 16; ch++) {
                uint32_t pk[8];
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int cc = ch * 16 + 2 * x;
                    const int qq = h * CPT + cc;
                    const f32x2 x2 = fma2(pack2(pv[cc], pv[cc + 1]), c2, *reinterpret_cast<const f32x2 *>(&rv[qq]));
                    float p0, p1;
                    exp2_pair<BwdEmu<HD>::PAIRS_OF_4>(x2, x, p0, p1);
                    pv[cc] = p0;
                    pv[cc + 1] = p1;
                    pk[x] = pack_bf16(p0, p1);
                }
                tmem_st_x8(t_s + h * (CPT / 2) + ch * 8, pk);  // 16 score columns -> 8 packed columns
            }
            tmem_wait_st();
            warp_arrive(BAR(C::B_P), lane);

            // ---- phase 2: dS^T = P^T * (dP^T - delta), bf16 into TMEM for dK += dS^T Q
            ok = ok && mbar_wait(BAR(C::B_DP), i & 1, abort_flag, p.status, WB_DP);
            tc_fence_after();
            float dp[CPT];
            tmem_ld_cols<CPT>(t_dp + h * CPT, dp);
            named_bar_sync(2, NCT);  // all of dP^T is read before any thread overwrites it with dS^T
#pragma unroll
            for (int ch = 0; ch < CPT / 16; ch++) {
                uint32_t pk[8];
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int cc = ch * 16 + 2 * x;
                    const f32x2 ds2 = mul2(pack2(pv[cc], pv[cc + 1]),
                                           sub2(pack2(dp[cc], dp[cc + 1]), *reinterpret_cast<const f32x2 *>(&rv[128 + h * CPT + cc])));
                    float d0, d1;
                    unpack2(ds2, d0, d1);
                    pk[x] = pack_bf16(d0, d1);
                }
                tmem_st_x8(t_dp + h * (CPT / 2) + ch * 8, pk);
            }
            tmem_wait_st();
            warp_arrive(BAR(C::B_DS), lane);
        }
        ok = ok && mbar_wait(BAR(C::B_ACC), 0, abort_flag, p.status, WB_ACC);
        tc_fence_after();
        // dV through the V tile's buffer, dK (times the softmax scale) through the K tile's: both
        // resident tiles are dead once the last MMAs have completed.
        stage_acc<HD>(tmem + lane_sel + C::T_ACC0, smem_gen + C::OFF_RES1, r, h, 1.f);
        stage_acc<HD>(tmem + lane_sel + C::T_ACC1, smem_gen + C::OFF_RES0, r, h, p.scale);
        named_bar_sync(3, NCT);
        const int rows_valid = ok ? min(128, p.lk - k0) : 0;
        const size_t gtile = ((size_t)bh * p.lk + k0) * p.d;
        store_staged<HD>(smem_gen + C::OFF_RES1, p.dv + gtile, p.d, rows_valid, warp, lane, p.dv, (size_t)p.order.units * p.lk * p.d * 2, p.status);
        store_staged<HD>(smem_gen + C::OFF_RES0, p.dk + gtile, p.d, rows_valid, warp, lane, p.dk, (size_t)p.order.units * p.lk * p.d * 2, p.status);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_ALLOC) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
    sm100_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                        const BwdParams p)
{
    using C = BwdCfg<HD>;
    constexpr int EMPTY_B = 1;  // V is read by the gradient chain only (dP)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    if (!smem_layout_fits<C>(smem_u32(smem_raw), smem_base, p.status)) return;
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    volatile int *abort_flag =
        reinterpret_cast<volatile int *>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    int bh, rank;
    work_item(p.order, blockIdx.x, bh, rank);
    const int qtile = p.order.blocks - 1 - rank;  // heaviest causal tiles first
    const int q0 = qtile * 128;
    const int off = p.lk - p.lq;
    const int visible = p.causal ? min(p.lk, q0 + 128 + off) : p.lk;
    const int n = (visible + 127) / 128;

    const uint32_t tmem = bwd_setup<C>(smem_base, smem_gen, warp, lane, &tm_q, &tm_k, &tm_v, &tm_do, EMPTY_B);

    if (warp >= NCW) {
        reg_dealloc_40();
        if (warp == W_TMA && lane == 0) {
            mbar_arrive_expect_tx(BAR(C::B_RES), 2 * C::TILE_BYTES);
            for (int s = 0; s < C::NSUB; s++) {
                tma_load_3d(smem_base + C::OFF_RES0 + s * C::SUB_BYTES, &tm_q, BAR(C::B_RES), s * 64, q0, bh);
                tma_load_3d(smem_base + C::OFF_RES1 + s * C::SUB_BYTES, &tm_do, BAR(C::B_RES), s * 64, q0, bh);
            }
            int issued_a = 0, issued_b = 0;
            for (int j = 0; j < n; j++) {
                const int sa = j % C::NA, sb = j % C::NB;
                if (!mbar_wait(BAR(C::B_EMPTYA + sa), ((j / C::NA) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLA + sa), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_A + sa * C::TILE_BYTES + s * C::SUB_BYTES, &tm_k,
                                BAR(C::B_FULLA + sa), s * 64, j * 128, bh);
                issued_a = j + 1;
                if (!mbar_wait(BAR(C::B_EMPTYB + sb), ((j / C::NB) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLB + sb), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_B + sb * C::TILE_BYTES + s * C::SUB_BYTES, &tm_v,
                                BAR(C::B_FULLB + sb), s * 64, j * 128, bh);
                issued_b = j + 1;
            }
            drain_copies<C>(bar0, issued_a, issued_b);
        } else if (warp == W_MMA_A || warp == W_MMA_B) {  // all 32 lanes, converged; one elected lane issues
            constexpr uint32_t IDESC_SS = idesc_bf16_f32(128, 128, 0, 0);
            constexpr uint32_t IDESC_TS = idesc_bf16_f32(128, HD, 0, 1);
            const uint32_t qa = smem_base + C::OFF_RES0, doa = smem_base + C::OFF_RES1;
            const uint32_t q_lo = desc_lo(qa, 16), do_lo = desc_lo(doa, 16);
            auto k_addr = [&](int j) { return smem_base + C::OFF_A + (j % C::NA) * C::TILE_BYTES; };
            auto v_addr = [&](int j) { return smem_base + C::OFF_B + (j % C::NB) * C::TILE_BYTES; };
            auto issue_s = [&](int j) {  // S = Q K^T
                const uint32_t k_lo = desc_lo(k_addr(j), 16);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                    mma_ss_lo(tmem + C::T_S, q_lo + o16, k_lo + o16, IDESC_SS, ks > 0);
                }
                tc_commit_elect(BAR(C::B_S));
            };
            // dP and dS live in two TMEM buffers, by the parity of the key tile (the dQ accumulator
            // leaves 128 columns free in this kernel): dP(j+2) is computed while dQ(j+1) still reads
            // dS(j+1) from the other buffer, so the gradient chain never waits for its own MMA.
            auto issue_dp = [&](int j) {  // dP = dO V^T
                const uint32_t v_lo = desc_lo(v_addr(j), 16);
                const uint32_t t_dp = tmem + ((j & 1) ? C::T_ACC1 : C::T_DP);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                    mma_ss_lo(t_dp, do_lo + o16, v_lo + o16, IDESC_SS, ks > 0);
                }
                tc_commit_elect(BAR((j & 1) ? C::B_DP1 : C::B_DP));
                tc_commit_elect(BAR(C::B_EMPTYB + j % C::NB));  // V(j) is only read by dP(j)
            };
            bool ok = mbar_wait(BAR(C::B_RES), 0, abort_flag, p.status, WB_RES);
            if (warp == W_MMA_A) {
                // score chain: S(j+1) as soon as the compute warps have copied S(j) out
                ok = ok && mbar_wait(BAR(C::B_FULLA + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_s(0);
                for (int j = 0; j < n && ok; j++) {
                    if (j + 1 < n) {
                        ok = ok && mbar_wait(BAR(C::B_FULLA + (j + 1) % C::NA), ((j + 1) / C::NA) & 1, abort_flag,
                                             p.status, WB_FULL);
                        ok = ok && mbar_wait(BAR(C::B_P), j & 1, abort_flag, p.status, WB_P);  // S(j) has been read
                        tc_fence_after();
                        issue_s(j + 1);
                    }
                    tc_commit_elect(BAR(C::B_EMPTYA + j % C::NA));  // this chain's last read of K(j) was S(j)
                }
                tc_commit_elect(BAR(C::B_ACC));
            } else {
                // gradient chain: dP(0), dP(1); then per tile dQ(j) (reads dS(j) and K(j)) and dP(j+2)
                // (overwrites dS(j): issued after dQ(j), and the tensor core keeps that order)
                ok = ok && mbar_wait(BAR(C::B_FULLB + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_dp(0);
                if (n > 1) {
                    ok = ok && mbar_wait(BAR(C::B_FULLB + 1 % C::NB), (1 / C::NB) & 1, abort_flag, p.status, WB_FULL);
                    tc_fence_after();
                    issue_dp(1);
                }
                for (int j = 0; j < n && ok; j++) {
                    const uint32_t kmn_lo = desc_lo(k_addr(j), C::SUB_BYTES);
                    const uint32_t t_ds = tmem + ((j & 1) ? C::T_ACC1 : C::T_DP);
                    ok = ok && mbar_wait(BAR(C::B_FULLA + j % C::NA), (j / C::NA) & 1, abort_flag, p.status, WB_FULL);
                    ok = ok && mbar_wait(BAR((j & 1) ? C::B_DS1 : C::B_DS), (j >> 1) & 1, abort_flag, p.status, WB_DS);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)  // dQ += dS K
                        mma_ts_lo(tmem + C::T_ACC0, t_ds + ks * 8, kmn_lo + ks * (2048 >> 4), IDESC_TS,
                                  (j > 0 || ks > 0) ? 1u : 0u);
                    tc_commit_elect(BAR(C::B_EMPTYA + j % C::NA));  // this chain's last read of K(j)
                    if (j + 2 < n) {
                        ok = ok && mbar_wait(BAR(C::B_FULLB + (j + 2) % C::NB), ((j + 2) / C::NB) & 1, abort_flag,
                                             p.status, WB_FULL);
                        tc_fence_after();
                        issue_dp(j + 2);  // also releases V(j+2)
                    }
                }
                tc_commit_elect(BAR(C::B_ACC));
            }
        }
    } else {
        compute_reg_alloc();
        const int h = warp / 4;
        const int r = threadIdx.x % 128;
        const int row = q0 + r;
        const uint32_t lane_sel = (uint32_t)((warp % 4) * 32) << 16;
        const uint32_t t_s = tmem + lane_sel + C::T_S;
        const float c = p.scale_log2;
        const bool row_ok = row < p.lq;
        const float lse2 = row_ok ? p.lse[(size_t)bh * p.lq + row] * LOG2E_B : INFINITY;
        const float dl = row_ok ? p.delta[(size_t)bh * p.lq + row] : 0.f;
        const int limit_row = p.causal ? min(p.lk - 1, row + off) : p.lk - 1;
        const int limit_tile = p.causal ? min(p.lk - 1, q0 + off) : p.lk - 1;
        bool ok = true;
        for (int j = 0; j < n; j++) {
            // ---- phase 1: P = exp2(S * c - lse2) in registers; S is released as soon as it is read
            ok = ok && mbar_wait(BAR(C::B_S), j & 1, abort_flag, p.status, WB_S);
            tc_fence_after();
            float pv[CPT];
            tmem_ld_cols<CPT>(t_s + h * CPT, pv);
            warp_arrive(BAR(C::B_P), lane);
            if (j * 128 + 127 > limit_tile) {  // tile crossed by the diagonal or the end of the keys
                const float masked = c > 0.f ? -INFINITY : INFINITY;
                const int kbase = j * 128 + h * CPT;
#pragma unroll
                for (int cc = 0; cc < CPT; cc++)
                    if (kbase + cc > limit_row) pv[cc] = masked;
            }
            const f32x2 c2 = pack2(c, c), nl2 = pack2(-lse2, -lse2);
#pragma unroll
            for (int x = 0; x < CPT / 2; x++) {
                const f32x2 x2 = fma2(pack2(pv[2 * x], pv[2 * x + 1]), c2, nl2);
                float p0, p1;
                exp2_pair<BwdEmu<HD>::PAIRS_OF_4>(x2, x, p0, p1);
                pv[2 * x] = p0;
                pv[2 * x + 1] = p1;
            }
            // ---- phase 2: dS = P * (dP - delta), bf16 into TMEM for dQ += dS K
            const uint32_t t_dp = tmem + lane_sel + ((j & 1) ? C::T_ACC1 : C::T_DP);  // this tile's dP / dS buffer
            ok = ok && mbar_wait(BAR((j & 1) ? C::B_DP1 : C::B_DP), (j >> 1) & 1, abort_flag, p.status, WB_DP);
            tc_fence_after();
            float dp[CPT];
            tmem_ld_cols<CPT>(t_dp + h * CPT, dp);
            named_bar_sync(1, NCT);  // all of dP is read before any thread overwrites it with dS
            const f32x2 dl2 = pack2(dl, dl);
#pragma unroll
            for (int ch = 0; ch < CPT / 16; ch++) {
                uint32_t pk[8];
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int cc = ch * 16 + 2 * x;
                    const f32x2 ds2 = mul2(pack2(pv[cc], pv[cc + 1]), sub2(pack2(dp[cc], dp[cc + 1]), dl2));
                    float d0, d1;
                    unpack2(ds2, d0, d1);
                    pk[x] = pack_bf16(d0, d1);
                }
                tmem_st_x8(t_dp + h * (CPT / 2) + ch * 8, pk);
            }
            tmem_wait_st();
            warp_arrive(BAR((j & 1) ? C::B_DS1 : C::B_DS), lane);
        }
        ok = ok && mbar_wait(BAR(C::B_ACC), 0, abort_flag, p.status, WB_ACC);
        tc_fence_after();
        // dQ (times the softmax scale) through the Q tile's buffer, which is dead by now.
        stage_acc<HD>(tmem + lane_sel + C::T_ACC0, smem_gen + C::OFF_RES0, r, h, p.scale);
        named_bar_sync(3, NCT);
        store_staged<HD>(smem_gen + C::OFF_RES0, p.dq + ((size_t)bh * p.lq + q0) * p.d, p.d, ok ? min(128, p.lq - q0) : 0, warp,
                         lane, p.dq, (size_t)p.order.units * p.lq * p.d * 2, p.status);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_ALLOC) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------
// Single pass: dK, dV and dQ from one sweep over the (key tile, query tile) pairs
// ------------------------------------------------------------------------------------------------
// The two-kernel form above multiplies seven 128x128 tile products for the five the gradients need
// (the dQ pass forms S and dP a second time). Here the CTA that owns a key tile also forms
//     dQ(i) = dS(i) K        (this key tile's contribution to the gradient of query tile i)
// and adds it into a float32 accumulator in global memory with a bulk reduce-add; a small kernel
// afterwards scales and converts that accumulator to bf16. Changes against the dK/dV kernel:
//   * dS^T goes to SHARED memory (bf16, the 128-byte-swizzled layout a TMA tile has) instead of
//     tensor memory: the same 32 KB buffer is the K-major A operand of dK += dS^T Q (keys = M along
//     rows, queries = K along the row) and the MN-major A operand of dQ = dS K (queries = M along the
//     row, keys = K across rows); K itself, resident in shared memory, is the MN-major B operand.
//   * the dP^T columns of tensor memory are dead once the compute warps have read them, so dQ(i)
//     is accumulated there (tensor memory is full otherwise at HD = 128); four drain warps copy a
//     whole row of it into registers at once while dK(i) is multiplied (dP^T(i+1) waits for that),
//     then pass it through shared staging buffers to cp.reduce.async.bulk add.f32. (Adding straight
//     from registers with red.global measured slower: the additions back up in the load/store path
//     that the compute warps' shared-memory and barrier traffic also uses.)
//   * with all operands of S^T, dP^T, dK and dQ read from shared memory (128 bytes per clock, which
//     one 128x128x16 product per 64 clocks uses up by itself), the kernel is bound by shared-memory
//     bandwidth: about 512 KB per tile pair (288 KB of operands, 96 KB written by TMA and the dS^T
//     stores, 128 KB through the staging buffers) = 4000 clocks, against 3750 for the two kernels
//     above together, which in practice take 5800.
//   * the accumulator's layout is private to the two kernels: per (unit, query tile, lane quarter,
//     32-column chunk) one contiguous 4 KB block holding [4-column group][row][4 floats], which makes
//     the staging writes conflict-free and every bulk operation one contiguous block.
// The float32 additions into the accumulator arrive in no fixed order, so dQ is reproducible only
// to rounding (dK and dV stay bit-reproducible); the two-kernel form remains available for callers
// who need run-to-run identical bits.
//
//   warps 0-7   compute (as above)            warp 8 / 9   MMA issue: score chain / gradient chain
//   warp 10     TMA producer                   warp 11      tensor-memory allocation
//   warps 12-15 drain dQ(i) from tensor memory into the global accumulator
constexpr int SP_THREADS = (NCW + 8) * 32;
constexpr int W_DRAIN0 = NCW + 4;

template <int HD>
struct SpCfg {
    static constexpr int NSUB = HD / 64;
    static constexpr int SUB_BYTES = 128 * 128;
    static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
    // Shared memory at HD = 128 holds seven 32 KB tiles: K, V, dS^T and the drain staging leave three
    // for the streamed operands, two for Q (in use from S^T(i) until dK(i)) and one for dO.
    static constexpr int NA = HD == 128 ? 2 : 3, NB = HD == 128 ? 1 : 2;
    static constexpr int DS_BYTES = 2 * SUB_BYTES;       // 128 keys x 128 queries, bf16
    static constexpr int STAGE_WARP_BYTES = 2 * 4096;    // two 4 KB chunk buffers per drain warp
    static constexpr int OFF_RES0 = 0;                   // K
    static constexpr int OFF_RES1 = TILE_BYTES;          // V
    static constexpr int OFF_A = 2 * TILE_BYTES;         // Q ring
    static constexpr int OFF_B = OFF_A + NA * TILE_BYTES;  // dO ring
    static constexpr int OFF_DS = OFF_B + NB * TILE_BYTES;
    static constexpr int OFF_STAGE = OFF_DS + DS_BYTES;
    static constexpr int OFF_BAR = OFF_STAGE + 4 * STAGE_WARP_BYTES;
    static constexpr int OFF_ROWVEC = OFF_BAR + 192;
    static constexpr int USED_BYTES = OFF_ROWVEC + 2048;
    static constexpr int SMEM_BYTES = HD == 128 ? 232448 : USED_BYTES + 1024;
    static constexpr int T_S = 0, T_DP = 128, T_ACC0 = 256, T_ACC1 = 256 + HD;
    static constexpr int B_RES = 0, B_FULLA = 1, B_EMPTYA = B_FULLA + NA, B_FULLB = B_EMPTYA + NA,
                         B_EMPTYB = B_FULLB + NB,
                         B_S = B_EMPTYB + NB,   // S^T of the current tile is in tensor memory
                         B_DP = B_S + 1,        // dP^T is in tensor memory
                         B_P = B_DP + 1,        // P^T written (one arrival per compute warp)
                         B_DS = B_P + 1,        // dS^T written to shared memory (one arrival per compute warp)
                         B_DSFREE = B_DS + 1,   // dQ(i) and dK(i) have read dS^T(i)
                         B_DQ = B_DSFREE + 1,   // dQ(i) is in tensor memory
                         B_DQFREE = B_DQ + 1,   // the drain warps have copied dQ(i) out (4 arrivals)
                         B_ACC = B_DQFREE + 1, NUM_BARS = B_ACC + 1;
    static_assert(8 * NUM_BARS + 8 <= 192, "barrier block");
    static_assert(HD != 128 || USED_BYTES + 800 <= SMEM_BYTES, "shared memory layout");
};

struct SpParams {
    __nv_bfloat16 *dk, *dv;
    float *dq_acc;  // [unit][query tile][lane quarter][HD/32 chunks][1024] float32, zero on entry
    const float *lse, *delta;
    int lq, lk, causal;
    int d;  // elements per row in memory (a multiple of 8, <= HD), as in BwdParams
    float scale, scale_log2;
    DeviceStatus *status;
    WorkOrder order;
};

__device__ __forceinline__ void bulk_reduce_add_f32(float *gdst, uint32_t smem_src, uint32_t bytes)
{
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

#ifdef EMBER_BWD_TRACE
// Development aid (not compiled into the library): one CTA records clock64() at the hand-over points
// of its first iterations.
__device__ long long g_bwd_trace[64 * 32];
#define TR(slot, it)                                                                          \
    do {                                                                                      \
        if (blockIdx.x == gridDim.x / 2 && (it) < 64) g_bwd_trace[(it) * 32 + (slot)] = clock64(); \
    } while (0)
#else
#define TR(slot, it) \
    do {             \
    } while (0)
#endif

template <int HD>
__global__ void __launch_bounds__(SP_THREADS, 1)
    sm100_bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                           const SpParams p)
{
    using C = SpCfg<HD>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    if (!smem_layout_fits<C>(smem_u32(smem_raw), smem_base, p.status)) return;
    const uint32_t bar0 = smem_base + C::OFF_BAR;
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *rowvec = reinterpret_cast<float *>(smem_gen + C::OFF_ROWVEC);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    int bh, rank;
    work_item(p.order, blockIdx.x, bh, rank);
    const int k0 = rank * 128;  // under a causal mask the first key blocks are seen by the most queries
    const int off = p.lk - p.lq;
    const int i_begin = p.causal ? max(0, k0 - off) / 128 : 0;  // first query tile that sees key k0
    const int nqt = (p.lq + 127) / 128;
    const int n = nqt - i_begin;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(BAR(C::B_RES), 1);
        for (int s = 0; s < C::NA; s++) {
            mbar_init(BAR(C::B_FULLA + s), 1);
            mbar_init(BAR(C::B_EMPTYA + s), 2);  // released by both MMA warps
        }
        for (int s = 0; s < C::NB; s++) {
            mbar_init(BAR(C::B_FULLB + s), 1);
            mbar_init(BAR(C::B_EMPTYB + s), 2);  // dO is read by both chains (dP^T and dV)
        }
        mbar_init(BAR(C::B_S), 1);
        mbar_init(BAR(C::B_DP), 1);
        mbar_init(BAR(C::B_P), NCW);
        mbar_init(BAR(C::B_DS), NCW);
        mbar_init(BAR(C::B_DSFREE), 1);
        mbar_init(BAR(C::B_DQ), 1);
        mbar_init(BAR(C::B_DQFREE), 4);
        mbar_init(BAR(C::B_ACC), 2);
        fence_mbar_init();
    }
    if (warp == W_ALLOC) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    if (warp == W_TMA && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_do);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    pdl_launch_dependents();  // the dQ finish kernel may be placed on SMs as they fall idle; it waits for this grid's end
    if (warp >= W_DRAIN0) {
        // -------------------------------------------------------------------- drain dQ(i)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");  // holds half a row (64 columns) of dQ(i) at a time
        pdl_wait();  // the accumulator is cleared by the delta launch before this one
        const int w = warp - W_DRAIN0;  // == warp % 4: the tensor-memory lane quarter this warp may read
        const uint32_t t_dq = tmem + ((uint32_t)(w * 32) << 16) + C::T_DP;
        uint8_t *stage = smem_gen + C::OFF_STAGE + w * C::STAGE_WARP_BYTES;
        const uint32_t stage_u32 = smem_base + C::OFF_STAGE + w * C::STAGE_WARP_BYTES;
        bool ok = true;
        int cnt = 0;
        for (int i = 0; i < n; i++) {
            ok = ok && mbar_wait(BAR(C::B_DQ), i & 1, abort_flag, p.status, WB_ACC);
            tc_fence_after();
            if (w == 0 && lane == 0) TR(16, i);
            float *gdst = p.dq_acc + ((((size_t)bh * nqt + (i_begin + i)) * 4 + w) * (HD / 32)) * 1024;
            // The row leaves tensor memory in two halves of 64 columns (the registers of these warps are
            // what the compute warps do not get); dP^T(i+1) may overwrite it once the second half is read.
#pragma unroll
            for (int hf = 0; hf < HD / 64; hf++) {
                uint32_t u[2][32];
                tmem_ld_32x32b_x32(t_dq + hf * 64, u[0]);
                tmem_ld_32x32b_x32(t_dq + hf * 64 + 32, u[1]);
                tmem_wait_ld();
                if (hf == HD / 64 - 1) {
                    warp_arrive(BAR(C::B_DQFREE), lane);
                    if (w == 0 && lane == 0) TR(17, i);
                }
#pragma unroll
                for (int c2 = 0; c2 < 2; c2++) {
                    const int c = hf * 2 + c2;
                    // the bulk operation that read this buffer two chunks ago must be done with it
                    if (lane == 0) bulk_wait_read_1();
                    __syncwarp();
                    uint8_t *buf = stage + (cnt & 1) * 4096;
#pragma unroll
                    for (int cg = 0; cg < 8; cg++)
                        *reinterpret_cast<uint4 *>(buf + (cg * 32 + lane) * 16) =
                            make_uint4(u[c2][4 * cg], u[c2][4 * cg + 1], u[c2][4 * cg + 2], u[c2][4 * cg + 3]);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (ok) bulk_reduce_add_f32(gdst + c * 1024, stage_u32 + (cnt & 1) * 4096, 4096);
                        bulk_commit();
                    }
                    cnt++;
                }
            }
        }
        if (lane == 0) bulk_wait_all();
    } else if (warp >= NCW) {
        reg_dealloc_40();
        if (warp == W_TMA && lane == 0) {
            // ---------------------------------------------------------------- TMA producer
            mbar_arrive_expect_tx(BAR(C::B_RES), 2 * C::TILE_BYTES);
            for (int s = 0; s < C::NSUB; s++) {
                tma_load_3d(smem_base + C::OFF_RES0 + s * C::SUB_BYTES, &tm_k, BAR(C::B_RES), s * 64, k0, bh);
                tma_load_3d(smem_base + C::OFF_RES1 + s * C::SUB_BYTES, &tm_v, BAR(C::B_RES), s * 64, k0, bh);
            }
            int issued_a = 0, issued_b = 0;
            for (int i = 0; i < n; i++) {
                const int sa = i % C::NA, sb = i % C::NB;
                const int q0 = (i_begin + i) * 128;
                if (!mbar_wait(BAR(C::B_EMPTYA + sa), ((i / C::NA) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLA + sa), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_A + sa * C::TILE_BYTES + s * C::SUB_BYTES, &tm_q,
                                BAR(C::B_FULLA + sa), s * 64, q0, bh);
                issued_a = i + 1;
                if (!mbar_wait(BAR(C::B_EMPTYB + sb), ((i / C::NB) & 1) ^ 1, abort_flag, p.status, WB_EMPTY)) break;
                mbar_arrive_expect_tx(BAR(C::B_FULLB + sb), C::TILE_BYTES);
                for (int s = 0; s < C::NSUB; s++)
                    tma_load_3d(smem_base + C::OFF_B + sb * C::TILE_BYTES + s * C::SUB_BYTES, &tm_do,
                                BAR(C::B_FULLB + sb), s * 64, q0, bh);
                issued_b = i + 1;
            }
            drain_copies<C>(bar0, issued_a, issued_b);
        } else if (warp == W_MMA_A || warp == W_MMA_B) {  // all 32 lanes, converged; one elected lane issues
            // ---------------------------------------------------------------- MMA issue
            constexpr uint32_t IDESC_SS = idesc_bf16_f32(128, 128, 0, 0);
            constexpr uint32_t IDESC_TS = idesc_bf16_f32(128, HD, 0, 1);   // dV: A from tensor memory; dK: A K-major
            constexpr uint32_t IDESC_DQ = idesc_bf16_f32(128, HD, 1, 1);   // A = dS^T read MN-major, B = K MN-major
            const uint32_t ka = smem_base + C::OFF_RES0, va = smem_base + C::OFF_RES1, dsa = smem_base + C::OFF_DS;
            const uint32_t k_lo = desc_lo(ka, 16), v_lo = desc_lo(va, 16);
            auto q_addr = [&](int i) { return smem_base + C::OFF_A + (i % C::NA) * C::TILE_BYTES; };
            auto do_addr = [&](int i) { return smem_base + C::OFF_B + (i % C::NB) * C::TILE_BYTES; };
            bool ok = mbar_wait(BAR(C::B_RES), 0, abort_flag, p.status, WB_RES);
            if (warp == W_MMA_A) {
                // score chain: S^T(0); then per tile dV(i) (reads P^T, dO) and S^T(i+1) (overwrites P^T)
                auto issue_st = [&](int i) {  // S^T = K Q^T
                    const uint32_t q_lo = desc_lo(q_addr(i), 16);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                        mma_ss_lo(tmem + C::T_S, k_lo + o16, q_lo + o16, IDESC_SS, ks > 0);
                    }
                    tc_commit_elect(BAR(C::B_S));
                };
                ok = ok && mbar_wait(BAR(C::B_FULLA + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_st(0);
                for (int i = 0; i < n && ok; i++) {
                    const uint32_t domn_lo = desc_lo(do_addr(i), C::SUB_BYTES);
                    ok = ok && mbar_wait(BAR(C::B_FULLB + i % C::NB), (i / C::NB) & 1, abort_flag, p.status, WB_FULL);
                    ok = ok && mbar_wait(BAR(C::B_P), i & 1, abort_flag, p.status, WB_P);
                    tc_fence_after();
                    if (lane == 0) TR(8, i);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)  // dV += P^T dO
                        mma_ts_lo(tmem + C::T_ACC0, tmem + C::T_S + ks * 8, domn_lo + ks * (2048 >> 4), IDESC_TS,
                                  (i > 0 || ks > 0) ? 1u : 0u);
                    tc_commit_elect(BAR(C::B_EMPTYB + i % C::NB));  // this chain's last read of dO(i)
                    if (i + 1 < n) {
                        ok = ok && mbar_wait(BAR(C::B_FULLA + (i + 1) % C::NA), ((i + 1) / C::NA) & 1, abort_flag,
                                             p.status, WB_FULL);
                        tc_fence_after();
                        issue_st(i + 1);  // overwrites P^T(i): ordered after dV(i) by issue order
                    }
                    if (lane == 0) TR(9, i);
                    tc_commit_elect(BAR(C::B_EMPTYA + i % C::NA));  // this chain's last read of Q(i) was S^T(i)
                }
                tc_commit_elect(BAR(C::B_ACC));
            } else {
                // gradient chain: dP^T(0); then per tile dQ(i), dK(i) (both read dS^T from shared memory)
                // and dP^T(i+1), which overwrites dQ(i) and therefore waits for the drain warps
                auto issue_dpt = [&](int i) {  // dP^T = V dO^T
                    const uint32_t do_lo = desc_lo(do_addr(i), 16);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                        mma_ss_lo(tmem + C::T_DP, v_lo + o16, do_lo + o16, IDESC_SS, ks > 0);
                    }
                    tc_commit_elect(BAR(C::B_DP));
                    tc_commit_elect(BAR(C::B_EMPTYB + i % C::NB));  // this chain's only read of dO(i)
                };
                const uint32_t ds_lo = desc_lo(dsa, 16), dsmn_lo = desc_lo(dsa, C::SUB_BYTES);
                const uint32_t kmn_lo = desc_lo(ka, C::SUB_BYTES);
                ok = ok && mbar_wait(BAR(C::B_FULLB + 0), 0, abort_flag, p.status, WB_FULL);
                tc_fence_after();
                issue_dpt(0);
                for (int i = 0; i < n && ok; i++) {
                    const uint32_t qmn_lo = desc_lo(q_addr(i), C::SUB_BYTES);
                    ok = ok && mbar_wait(BAR(C::B_FULLA + i % C::NA), (i / C::NA) & 1, abort_flag, p.status, WB_FULL);
                    ok = ok && mbar_wait(BAR(C::B_DS), i & 1, abort_flag, p.status, WB_DS);
                    tc_fence_after();
                    if (lane == 0) TR(12, i);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)  // dQ(i) = dS K: 16 keys per step
                        mma_ss_lo(tmem + C::T_DP, dsmn_lo + ks * (2048 >> 4), kmn_lo + ks * (2048 >> 4), IDESC_DQ, ks > 0);
                    tc_commit_elect(BAR(C::B_DQ));  // the drain warps copy dQ(i) out while dK(i) is multiplied
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {  // dK += dS^T Q: 16 queries per step
                        const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                        mma_ss_lo(tmem + C::T_ACC1, ds_lo + o16, qmn_lo + ks * (2048 >> 4), IDESC_TS, (i > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit_elect(BAR(C::B_DSFREE));
                    tc_commit_elect(BAR(C::B_EMPTYA + i % C::NA));  // this chain's last read of Q(i)
                    if (lane == 0) TR(13, i);
                    if (i + 1 < n) {
                        ok = ok && mbar_wait(BAR(C::B_DQFREE), i & 1, abort_flag, p.status, WB_ACC);
                        if (lane == 0) TR(14, i);
                        ok = ok && mbar_wait(BAR(C::B_FULLB + (i + 1) % C::NB), ((i + 1) / C::NB) & 1, abort_flag,
                                             p.status, WB_FULL);
                        tc_fence_after();
                        issue_dpt(i + 1);
                        if (lane == 0) TR(15, i);
                    }
                }
                tc_commit_elect(BAR(C::B_ACC));
            }
        }
    } else {
        // -------------------------------------------------------------------- compute
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");  // 8 x 32 x 192 + 4 x 32 x 40 + 4 x 32 x 88 == 65536
        const int h = warp / 4;                // which 64-column half of the 128 score columns (queries)
        const int r = threadIdx.x % 128;       // TMEM lane == key row inside the tile
        const int key = k0 + r;
        const uint32_t lane_sel = (uint32_t)((warp % 4) * 32) << 16;
        const uint32_t t_s = tmem + lane_sel + C::T_S, t_dp = tmem + lane_sel + C::T_DP;
        const float c = p.scale_log2;
        const float *lse_g = p.lse + (size_t)bh * p.lq;
        const float *delta_g = p.delta + (size_t)bh * p.lq;
        // this thread's 128 bytes of dS^T: row r of the sub-tile of its 64 queries; 16-byte chunk j of
        // the row lies at chunk position j ^ (r % 8) (the 128-byte swizzle of the MMA descriptors)
        uint8_t *ds_row = smem_gen + C::OFF_DS + h * C::SUB_BYTES + r * 128;
        bool ok = true;
        const float *rowvec_src = (threadIdx.x < 128 ? lse_g : delta_g);
        auto fetch_raw = [&](int i) -> float {
            const int qrow = (i_begin + i) * 128 + (threadIdx.x & 127);
            float v = 0.f;
            if (i < n && qrow < p.lq) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(rowvec_src + qrow));
            return v;
        };
        // Everything up to here (and the producer's copies and the first two products) needs nothing
        // from the delta launch before this one; the delta vector does.
        pdl_wait();
        float raw_next = fetch_raw(0);
        for (int i = 0; i < n; i++) {
            const int q0 = (i_begin + i) * 128;
            float *rv = rowvec + (i & 1) * 256;
            {
                const bool in_range = q0 + (threadIdx.x & 127) < p.lq;
                rv[threadIdx.x] = threadIdx.x < 128 ? (in_range ? -raw_next * LOG2E_B : -INFINITY) : (in_range ? raw_next : 0.f);
            }
            raw_next = fetch_raw(i + 1);
            // ---- phase 1: P^T = exp2(S^T * c - lse2), bf16 into tensor memory for dV += P^T dO
            ok = ok && mbar_wait(BAR(C::B_S), i & 1, abort_flag, p.status, WB_S);
            tc_fence_after();
            if (threadIdx.x == 0) TR(0, i);
            float pv[64];
            tmem_ld_cols<64>(t_s + h * 64, pv);
            // every thread has read its scores (the bf16 P^T overwrites columns another thread of the
            // same lane still needs) and the lse/delta vectors are visible
            named_bar_sync(1, NCT);
            if (threadIdx.x == 0) TR(1, i);
            if (p.causal && (k0 + 127 > q0 + off)) {  // tile crossed by the diagonal: mask before the exp
                const float masked = c > 0.f ? -INFINITY : INFINITY;
#pragma unroll
                for (int cc = 0; cc < 64; cc++)
                    if (key > q0 + h * 64 + cc + off) pv[cc] = masked;
            }
            const f32x2 c2 = pack2(c, c);
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                uint32_t pk[8];
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int cc = ch * 16 + 2 * x;
                    const f32x2 x2 = fma2(pack2(pv[cc], pv[cc + 1]), c2, *reinterpret_cast<const f32x2 *>(&rv[h * 64 + cc]));
                    float p0, p1;
                    exp2_pair<BwdEmu<HD>::PAIRS_OF_4>(x2, x, p0, p1);
                    pv[cc] = p0;
                    pv[cc + 1] = p1;
                    pk[x] = pack_bf16(p0, p1);
                }
                tmem_st_x8(t_s + h * 32 + ch * 8, pk);  // 16 score columns -> 8 packed columns
            }
            tmem_wait_st();
            warp_arrive(BAR(C::B_P), lane);
            if (threadIdx.x == 0) TR(2, i);

            // ---- phase 2: dS^T = P^T * (dP^T - delta), bf16 into shared memory for dQ = dS K and dK += dS^T Q
            ok = ok && mbar_wait(BAR(C::B_DP), i & 1, abort_flag, p.status, WB_DP);
            if (i > 0) ok = ok && mbar_wait(BAR(C::B_DSFREE), (i - 1) & 1, abort_flag, p.status, WB_DS);
            tc_fence_after();
            if (threadIdx.x == 0) TR(3, i);
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float dp[32];
                tmem_ld_cols<32>(t_dp + h * 64 + half * 32, dp);
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {  // 8 queries = one 16-byte chunk
                    uint32_t w4[4];
#pragma unroll
                    for (int x = 0; x < 4; x++) {
                        const int cd = q4 * 8 + 2 * x, cc = half * 32 + cd;
                        const f32x2 ds2 = mul2(pack2(pv[cc], pv[cc + 1]),
                                               sub2(pack2(dp[cd], dp[cd + 1]), *reinterpret_cast<const f32x2 *>(&rv[128 + h * 64 + cc])));
                        float d0, d1;
                        unpack2(ds2, d0, d1);
                        w4[x] = pack_bf16(d0, d1);
                    }
                    const int chunk = half * 4 + q4;
                    *reinterpret_cast<uint4 *>(ds_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
            }
            fence_proxy_async();  // the MMAs read dS^T through the async proxy
            warp_arrive(BAR(C::B_DS), lane);
            if (threadIdx.x == 0) TR(4, i);
        }
        ok = ok && mbar_wait(BAR(C::B_ACC), 0, abort_flag, p.status, WB_ACC);
        tc_fence_after();
        // dV through the V tile's buffer, dK (times the softmax scale) through the K tile's: both
        // resident tiles are dead once the last MMAs have completed.
        stage_acc<HD>(tmem + lane_sel + C::T_ACC0, smem_gen + C::OFF_RES1, r, h, 1.f);
        stage_acc<HD>(tmem + lane_sel + C::T_ACC1, smem_gen + C::OFF_RES0, r, h, p.scale);
        named_bar_sync(3, NCT);
        const int rows_valid = ok ? min(128, p.lk - k0) : 0;
        const size_t gtile = ((size_t)bh * p.lk + k0) * p.d;
        store_staged<HD>(smem_gen + C::OFF_RES1, p.dv + gtile, p.d, rows_valid, warp, lane, p.dv, (size_t)p.order.units * p.lk * p.d * 2, p.status);
        store_staged<HD>(smem_gen + C::OFF_RES0, p.dk + gtile, p.d, rows_valid, warp, lane, p.dk, (size_t)p.order.units * p.lk * p.d * 2, p.status);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_ALLOC) tmem_dealloc(tmem, 512);
}

// dq = bf16(scale * accumulator): one block per (unit, query tile, 32-column chunk), warp w takes lane
// quarter w of the accumulator's block layout ([4-column group][row][4 floats], 4 KB). A lane owns one
// 16-byte piece of dq (8 columns = two column groups) of one row per pass, four lanes side by side on a
// row: a warp-wide load reads four whole 128-byte runs of the block, a warp-wide store writes 64
// contiguous bytes (two full sectors) of each of 8 rows. (One row per lane, as the accumulator is laid
// out, made every store touch 32 lines with 16 bytes each and ran at half the memory bandwidth.)
template <int HD>
__global__ void __launch_bounds__(128) dq_finish_kernel(const float *__restrict__ acc, __nv_bfloat16 *__restrict__ dq, int lq,
                                                        int nqt, float scale, int d)
{
    const size_t tile = blockIdx.x;  // unit * nqt + query tile
    const int c = blockIdx.y;        // 32-column chunk
    const int qt = (int)(tile % nqt);
    const size_t unit = tile / nqt;
    const int w = threadIdx.x / 32, lane = threadIdx.x % 32;
    pdl_wait();                      // the accumulator is complete when the single-pass kernel has ended
    const int q = lane % 4;          // which 8 columns of the chunk
    const int col = c * 32 + q * 8;
    if (col >= d) return;            // d: elements per dq row in memory (<= HD, a multiple of 8)
    const int row0 = qt * 128 + w * 32 + lane / 4;
    const float4 *src = reinterpret_cast<const float4 *>(acc + ((tile * 4 + w) * (HD / 32) + c) * 1024);
    float4 v[4][2];
#pragma unroll
    for (int it = 0; it < 4; it++) {  // all eight loads in flight
        v[it][0] = src[(2 * q) * 32 + it * 8 + lane / 4];
        v[it][1] = src[(2 * q + 1) * 32 + it * 8 + lane / 4];
    }
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int row = row0 + it * 8;
        if (row >= lq) continue;
        uint4 o;
        o.x = pack_bf16(v[it][0].x * scale, v[it][0].y * scale);
        o.y = pack_bf16(v[it][0].z * scale, v[it][0].w * scale);
        o.z = pack_bf16(v[it][1].x * scale, v[it][1].y * scale);
        o.w = pack_bf16(v[it][1].z * scale, v[it][1].w * scale);
        *reinterpret_cast<uint4 *>(dq + (unit * lq + row) * d + col) = o;
    }
}

// delta[row] = sum_c dO[row][c] * O[row][c] for bf16 rows of HD elements: HD / 16 lanes per row, two
// 16-byte loads per tensor and lane, 32 / (HD / 16) rows per warp.
// The same launch clears the float32 dQ accumulator of the single-pass kernel (zero_vecs 16-byte
// vectors at `zero`, an equal slice per block): one launch less than a memset of its own. zero_vecs == 0: nothing to clear.
__device__ __forceinline__ void zero_slice(uint4 *__restrict__ zero, size_t zero_vecs)
{
    const size_t per = (zero_vecs + gridDim.x - 1) / gridDim.x;
    const size_t begin = (size_t)blockIdx.x * per;
    const size_t end = begin + per < zero_vecs ? begin + per : zero_vecs;
    for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) zero[i] = make_uint4(0u, 0u, 0u, 0u);
}

template <int HD>
__global__ void __launch_bounds__(256) delta_bf16_kernel(const uint4 *__restrict__ out, const uint4 *__restrict__ dout,
                                                         float *__restrict__ delta, size_t rows, uint4 *__restrict__ zero,
                                                         size_t zero_vecs)
{
    constexpr int LPR = HD / 16, RPW = 32 / LPR;
    const int lane = threadIdx.x % 32;
    const size_t row = ((size_t)blockIdx.x * 8 + threadIdx.x / 32) * RPW + lane / LPR;
    pdl_wait();                   // O comes from the kernel before (the forward, when it directly precedes)
    pdl_launch_dependents();      // the single-pass kernel may start its loads and first products under this kernel's tail
    zero_slice(zero, zero_vecs);  // every thread of every block, also those past the last row
    float s = 0.f;
    if (row < rows) {
        const size_t base = row * (HD / 8) + (lane % LPR) * 2;
        const uint4 a[2] = {out[base], out[base + 1]}, b[2] = {dout[base], dout[base + 1]};
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t x[4] = {a[h].x, a[h].y, a[h].z, a[h].w}, y[4] = {b[h].x, b[h].y, b[h].z, b[h].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s = fmaf(__uint_as_float(x[i] << 16), __uint_as_float(y[i] << 16), s);
                s = fmaf(__uint_as_float(x[i] & 0xffff0000u), __uint_as_float(y[i] & 0xffff0000u), s);
            }
        }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (row < rows && lane % LPR == 0) delta[row] = s;
}

// The same for rows of any multiple of 8 elements up to 128: 16 lanes per row, one 16-byte load per
// tensor and lane where the row has that chunk.
__global__ void __launch_bounds__(256) delta_bf16_rows_kernel(const uint4 *__restrict__ out, const uint4 *__restrict__ dout,
                                                              float *__restrict__ delta, size_t rows, int chunks,
                                                              uint4 *__restrict__ zero, size_t zero_vecs)
{
    const int lane = threadIdx.x % 32, c = lane % 16;
    const size_t row = ((size_t)blockIdx.x * 8 + threadIdx.x / 32) * 2 + lane / 16;
    pdl_wait();
    pdl_launch_dependents();
    zero_slice(zero, zero_vecs);
    float s = 0.f;
    if (row < rows && c < chunks) {
        const uint4 a = out[row * chunks + c], b = dout[row * chunks + c];
        const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s = fmaf(__uint_as_float(x[i] << 16), __uint_as_float(y[i] << 16), s);
            s = fmaf(__uint_as_float(x[i] & 0xffff0000u), __uint_as_float(y[i] & 0xffff0000u), s);
        }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (row < rows && c == 0) delta[row] = s;
}

// EMBER_PDL=0 (read once) launches the backward's kernels without programmatic stream serialization:
// plain stream order, for comparison or for a tool that cannot follow programmatic edges.
static int pdl_attr_count()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("EMBER_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v;
}

// zero / zero_bytes: the accumulator to clear in the same launch (16-byte aligned, a multiple of 16 bytes), or NULL / 0
template <int HD>
int launch_delta_bf16(const AttnArgs &a, float *delta, cudaStream_t s, void *zero = nullptr, size_t zero_bytes = 0)
{
    const size_t rows = (size_t)a.bh * a.lq;
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = pdl;
    cfg.numAttrs = pdl_attr_count();
    if (a.d != HD) {
        cfg.gridDim = dim3((unsigned)((rows + 15) / 16));
        EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, delta_bf16_rows_kernel, (const uint4 *)a.out, (const uint4 *)a.dout, delta, rows,
                                          a.d / 8, (uint4 *)zero, zero_bytes / 16));
        return EMBER_OK;
    }
    constexpr int ROWS_PER_BLOCK = 8 * (32 / (HD / 16));
    cfg.gridDim = dim3((unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK));
    EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, delta_bf16_kernel<HD>, (const uint4 *)a.out, (const uint4 *)a.dout, delta, rows,
                                      (uint4 *)zero, zero_bytes / 16));
    return EMBER_OK;
}

template <int HD>
int launch_fused(const AttnArgs &a, float *delta, float *dq_acc, DeviceState *st, cudaStream_t s)
{
    using C = SpCfg<HD>;
    static_assert(NCW == 8, "the single-pass kernel is written for eight compute warps");
    const int nqt = (a.lq + 127) / 128;
    // delta, and the accumulator cleared by the same launch
    int rc = launch_delta_bf16<HD>(a, delta, s, dq_acc, (size_t)a.bh * nqt * 128 * HD * sizeof(float));
    if (rc) return rc;
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_tensor_map_bf16_3d(&tq, a.q, a.d, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tk, a.k, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tv, a.v, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tdo, a.dout, a.d, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    SpParams p;
    p.dk = (__nv_bfloat16 *)a.dk;
    p.dv = (__nv_bfloat16 *)a.dv;
    p.dq_acc = dq_acc;
    p.lse = a.lse;
    p.delta = delta;
    p.lq = a.lq;
    p.lk = a.lk;
    p.d = a.d;
    p.causal = a.causal;
    p.scale = a.scale;
    p.scale_log2 = a.scale * LOG2E_B;
    p.status = st->status;
    auto k1 = sm100_bwd_fused_kernel<HD>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    const size_t touched = ((size_t)a.lq + a.lk) * HD * 2 * 4 + (size_t)a.lq * HD * 4;  // + the float32 dQ accumulator
    p.order = make_work_order(a.bh, (a.lk + 127) / 128, st->sm_count, touched, a.causal != 0);
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.order.units * p.order.blocks));
    cfg.blockDim = dim3(SP_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cfg.attrs = pdl;
    cfg.numAttrs = pdl_attr_count();
    EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, k1, tq, tk, tv, tdo, p));
    cfg.gridDim = dim3((unsigned)((size_t)a.bh * nqt), HD / 32);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, dq_finish_kernel<HD>, (const float *)dq_acc, (__nv_bfloat16 *)a.dq, a.lq, nqt, a.scale, a.d));
    return EMBER_OK;
}

template <int HD>
int launch(const AttnArgs &a, float *delta, DeviceState *st, cudaStream_t s)
{
    using C = BwdCfg<HD>;
    int rc = launch_delta_bf16<HD>(a, delta, s);
    if (rc) return rc;
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_tensor_map_bf16_3d(&tq, a.q, a.d, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tk, a.k, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tv, a.v, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tdo, a.dout, a.d, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    BwdParams p;
    p.dq = (__nv_bfloat16 *)a.dq;
    p.dk = (__nv_bfloat16 *)a.dk;
    p.dv = (__nv_bfloat16 *)a.dv;
    p.lse = a.lse;
    p.delta = delta;
    p.lq = a.lq;
    p.lk = a.lk;
    p.d = a.d;
    p.causal = a.causal;
    p.scale = a.scale;
    p.scale_log2 = a.scale * LOG2E_B;
    p.status = st->status;
    auto k1 = sm100_bwd_dkdv_kernel<HD>;
    auto k2 = sm100_bwd_dq_kernel<HD>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    EMBER_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    const size_t touched = ((size_t)a.lq + a.lk) * HD * 2 * 4;  // Q, dO, dQ, K, V, dK, dV and the row vectors
    p.order = make_work_order(a.bh, (a.lk + 127) / 128, st->sm_count, touched, a.causal != 0);
    k1<<<dim3((unsigned)(p.order.units * p.order.blocks)), BWD_THREADS, C::SMEM_BYTES, s>>>(tq, tk, tv, tdo, p);
    EMBER_CUDA_TRY(cudaGetLastError());
    p.order = make_work_order(a.bh, (a.lq + 127) / 128, st->sm_count, touched, a.causal != 0);
    k2<<<dim3((unsigned)(p.order.units * p.order.blocks)), BWD_THREADS, C::SMEM_BYTES, s>>>(tq, tk, tv, tdo, p);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

}  // namespace

bool sm100_bwd_supported(const AttnArgs &a)
{
    if (a.dtype != EMBER_BF16) return false;
    if (a.d < 8 || a.d > 128 || a.d % 8 != 0) return false;  // zero-padded to 64 or 128 columns by the TMA copies
    if (!isfinite(a.scale)) return false;
    if ((long long)a.bh * ((a.lq + 127) / 128) > 0x7fffffffLL || (long long)a.bh * ((a.lk + 127) / 128) > 0x7fffffffLL)
        return false;
    // TMA needs 16-byte aligned bases; the epilogues store 16-byte vectors.
    const uintptr_t bits = (uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.dout | (uintptr_t)a.out |
                           (uintptr_t)a.dq | (uintptr_t)a.dk | (uintptr_t)a.dv;
    return (bits & 15) == 0;
}

#ifdef EMBER_BWD_TRACE
extern "C" EMBER_API int ember_debug_bwd_trace(long long *host)
{
    return (int)cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(long long) * 64 * 32);
}
#endif

// Bytes of float32 dQ accumulator the single-pass kernel needs after the delta vector.
size_t sm100_bwd_accumulator_bytes(int bh, int lq, int d)
{
    const int hd = d <= 64 ? 64 : 128;  // the kernel's column count
    return (size_t)bh * ((lq + 127) / 128) * 128 * hd * sizeof(float);
}

int sm100_attention_bwd(const AttnArgs &a, float *delta, float *dq_acc, bool deterministic, DeviceState *st, cudaStream_t s)
{
    if (deterministic || !dq_acc) return a.d > 64 ? launch<128>(a, delta, st, s) : launch<64>(a, delta, st, s);
    return a.d > 64 ? launch_fused<128>(a, delta, dq_acc, st, s) : launch_fused<64>(a, delta, dq_acc, st, s);
}

}  // namespace ember
