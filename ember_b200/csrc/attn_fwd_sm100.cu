// Prefill attention forward for sm_100a: bf16 in/out, float32 softmax and accumulation.
//
// One CTA owns 256 consecutive query rows of one (batch*head) as two 128-row tiles whose softmax
// warpgroups run half a period apart, so that the tensor core always has the other tile's MMAs.
//
//   warps 0-3   softmax + epilogue of tile 0 (one thread per query row, row state in registers)
//   warps 4-7   softmax + epilogue of tile 1
//   warp  8/9   MMA issue for tile 0 / tile 1 (warp-collective, one elected lane each): S = Q K^T and
//               O += P V with tcgen05.mma, accumulators in TMEM. One issuing warp per tile, on
//               different schedulers: an issuing warp shares its scheduler with two busy softmax
//               warps and a single one could not keep up with both tiles.
//   warp 10     TMA producer (one lane): Q once, then K (2-stage ring) and V (3-stage ring)
//   warp 11     TMEM allocation / release
//
// Tensor memory (512 columns x 128 lanes of 32 bit):
//   P0 [0,64)  P1 [64,128)  S [128,256)  O0 [256,256+HD)  O1 [256+HD,256+2HD)
// There is ONE score buffer S, used by the two tiles in turn: a softmax warpgroup copies its 128
// scores per row into registers as soon as it is free (about 100 cycles), signals "S read", and the
// MMA warp immediately computes the other tile's next scores into the same columns. The bf16
// probabilities go to the tile's own P columns and are consumed from there as the A operand of the
// PV MMA, so P never touches shared memory and the score MMAs never wait for a PV MMA: the next
// scores of a tile are already waiting when its softmax finishes the current ones.
// Softmax runs in the exp2 domain (scale*log2(e) folded into one FMA per score); the running
// reference maximum is only moved, and O rescaled, when the row maximum grew by more than 2^8,
// which after the first tiles is rare. Causal tiles above the diagonal are never loaded or
// multiplied; only tiles crossed by the diagonal (or by the end of the key axis) pay for a mask.
// CTAs take their work in the order of WorkOrder (common.cuh): a few (batch*head) units at a time,
// heaviest query blocks first, so that the K and V of the units in flight stay in L2.
// The same kernel serves decode over a key/value cache with grouped-query heads (split-key mode):
// the query heads that share a K/V head are the rows of one zero-padded tile, a CTA covers one split
// of the key axis and writes a normalised partial output with its log-sum-exp, and
// split_merge_kernel combines the splits.
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

namespace ember {

namespace {

using namespace ptx;

constexpr int FWD_THREADS = 384;
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float LN2_F = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

// PAIR: two CTAs of a cluster work as one (cta_group::2). Each 256-row MMA covers one 128-row query
// tile of each CTA; a CTA holds only HALF of every K tile (64 of its 128 keys) and half of every V
// tile (64 of its HD columns) in shared memory and loads that half with its own TMA copies, so per
// key tile an SM receives 32 KB instead of 64 KB and the score MMAs read 48 KB of operands per
// 128x128x128 product instead of 64 KB. Shared memory moves 128 bytes per clock; the single-CTA
// form needs about 125 of them at the full MMA rate, which is what held it near 2850 clocks per key
// tile where the tensor core needs 2048.
template <int HD, bool PAIR = false>
struct FwdCfg {
    static constexpr int NSUB = HD / 64;                 // 64-column (128-byte) sub-tiles per tile
    static constexpr int SUB_BYTES = 128 * 128;          // 128 rows x 128 bytes
    static constexpr int TILE_BYTES = NSUB * SUB_BYTES;  // one 128 x HD bf16 tile
    // what one CTA holds of a K tile (PAIR: 64 keys x HD as NSUB sub-tiles of 64 rows) and of a V
    // tile (PAIR: 128 keys x 64 columns, one sub-tile)
    static constexpr int K_SUB_BYTES = PAIR ? 64 * 128 : SUB_BYTES;
    static constexpr int K_BYTES = NSUB * K_SUB_BYTES;
    static constexpr int V_BYTES = PAIR ? SUB_BYTES : TILE_BYTES;
    // K(j) is released as soon as both score MMAs of step j are issued; V(j) stays in use until the
    // second tile's PV MMA one step later, so V gets the deeper ring.
    static constexpr int KSTAGES = PAIR ? 3 : 2, VSTAGES = PAIR ? 4 : 3;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
    static constexpr int OFF_V = OFF_K + KSTAGES * K_BYTES;
    static constexpr int OFF_BAR = OFF_V + VSTAGES * V_BYTES;
    static constexpr int USED_BYTES = OFF_BAR + 320;     // barriers + TMEM slot + abort flag
    static constexpr int SMEM_BYTES = USED_BYTES + 1024; // + room to round the base up to 1024
    static constexpr int TMEM_P = 0, TMEM_S = 128, TMEM_O = 256;
    // barrier indices
    static constexpr int B_Q = 0, B_KFULL = 1, B_KEMPTY = B_KFULL + KSTAGES, B_VFULL = B_KEMPTY + KSTAGES,
                         B_VEMPTY = B_VFULL + VSTAGES,
                         B_S = B_VEMPTY + VSTAGES,  // [2] scores of tile t are in TMEM
                         B_R = B_S + 2,             // [2] tile t has copied its scores out (4 warp arrivals)
                         B_P = B_R + 2,             // [2][2] P of tile t, keys [0,64) / [64,128) written
                         B_O = B_P + 4,             // [2] PV MMA of tile t finished
                         NUM_BARS = B_O + 2;
};

// Wait codes reported in the device status word.
enum {
    W_MMA_Q = 1, W_MMA_K, W_MMA_V, W_MMA_P, W_MMA_R, W_SM_S, W_SM_O, W_SM_OFINAL, W_TMA_KEMPTY, W_TMA_VEMPTY
};

struct FwdParams {
    __nv_bfloat16 *out;
    float *lse;
    int lq, lk;
    int d;  // elements per row of q, k, v and out in memory (a multiple of 8, <= HD): the kernel works on
            // HD columns, the TMA copies read the columns past d as zero and the epilogue skips them
    int causal;
    int block_rows;  // query rows per CTA: 256 (two tiles) or 128 (tile 0 alone; tile 1's warps idle)
    float scale_log2;  // scale * log2(e)
    DeviceStatus *status;
    WorkOrder order;
    // Split-key use (decode over a key/value cache with a few query rows per unit): a work unit is
    // (sequence unit, split); the split covers keys [split * chunk, split * chunk + chunk) of the
    // unit's first seq_lens[unit / lens_div] (or lk) keys and writes a normalised partial output
    // plus its log-sum-exp, which a second kernel merges. splits == 1 is the plain forward.
    int splits, chunk, lens_div;
    const int *seq_lens;
};

// EMU: of every 4 pairs of exponentials, how many are evaluated as a polynomial on the FMA pipe
// instead of the MUFU (0..4).
// MMA, commit, allocation and arrival forms of a single CTA or of a CTA pair.
template <bool PAIR>
__device__ __forceinline__ void f_mma_ss(uint32_t d, uint32_t a, uint32_t b, uint32_t idesc, uint32_t acc)
{
    if constexpr (PAIR) mma_ss_lo_pair(d, a, b, idesc, acc); else mma_ss_lo(d, a, b, idesc, acc);
}
__device__ __forceinline__ void mma_ts_lo_pair(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 db;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "mov.b64 db, {%2, %5};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void f_mma_ts(uint32_t d, uint32_t a, uint32_t b, uint32_t idesc, uint32_t acc)
{
    if constexpr (PAIR) mma_ts_lo_pair(d, a, b, idesc, acc); else mma_ts_lo(d, a, b, idesc, acc);
}
template <bool PAIR>
__device__ __forceinline__ void f_commit(uint32_t bar)  // PAIR: the barrier of BOTH CTAs gets the arrival
{
    if constexpr (PAIR) tc_commit_pair(bar, 3); else tc_commit_elect(bar);
}
// 3-D tile load of one CTA of a pair into its own shared memory, bytes reported to rank 0's barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst_smem, const CUtensorMap *m, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void f_tma_3d(uint32_t dst, const CUtensorMap *m, uint32_t bar, int c0, int c1, int c2)
{
    if constexpr (PAIR) tma_load_3d_pair(dst, m, bar, c0, c1, c2); else tma_load_3d(dst, m, bar, c0, c1, c2);
}

template <int HD, int EMU, bool PAIR>
__global__ void __launch_bounds__(FWD_THREADS, 1)
    sm100_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const FwdParams p)
{
    using C = FwdCfg<HD, PAIR>;
    static_assert(!PAIR || HD == 128, "the pair form halves V along its 128 columns");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bar0 = smem_base + C::OFF_BAR;
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    constexpr int B_Q = C::B_Q, B_KFULL = C::B_KFULL, B_KEMPTY = C::B_KEMPTY, B_VFULL = C::B_VFULL,
                  B_VEMPTY = C::B_VEMPTY, B_S = C::B_S, B_R = C::B_R, B_P = C::B_P, B_O = C::B_O;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + C::OFF_BAR + 8 * C::NUM_BARS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    // A kernel launched behind this one with programmatic stream serialization (the backward's delta
    // kernel) may have its CTAs placed on SMs as they fall idle; it waits for this grid's end itself.
    pdl_launch_dependents();
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;  // rank 0 of a pair issues the MMAs
    int bh, rank;
    work_item(p.order, PAIR ? blockIdx.x / 2 : blockIdx.x, bh, rank);
    const int qblock = p.order.blocks - 1 - rank;  // heaviest (latest) causal rows first
    // A CTA has two 128-row query tiles. Alone they are consecutive rows. In a pair the four tiles of
    // a 512-row block alternate between the CTAs (rank r has tiles r and 2 + r), so that the two tiles
    // multiplied by one 256-row MMA are neighbours and see the same key tiles but one under a mask.
    const int q_base = PAIR ? qblock * 512 + (int)crank * 128 : qblock * p.block_rows;
    constexpr int TSTEP = PAIR ? 256 : 128;        // rows from this CTA's tile 0 to its tile 1
    // which tensor slab the unit reads, where its keys start and how many it sees
    const int unit = p.splits > 1 ? bh / p.splits : bh;
    const int k_row0 = p.splits > 1 ? (bh - unit * p.splits) * p.chunk : 0;
    int lk = p.seq_lens ? min(p.lk, p.seq_lens[unit / p.lens_div]) : p.lk;
    lk = p.splits > 1 ? min(p.chunk, lk - k_row0) : lk;
    if (!PAIR && lk <= 0) {
        // An empty split (a sequence shorter than the others): its partial is "no weight". Every
        // thread leaves here, before any barrier or tensor-memory allocation exists. Without splits
        // the (empty) sequence's result is defined as zeros with lse = -inf.
        if (p.lse && (int)threadIdx.x < p.block_rows && q_base + (int)threadIdx.x < p.lq)
            p.lse[(size_t)bh * p.lq + q_base + threadIdx.x] = -INFINITY;
        if (p.splits == 1)
            for (int i = threadIdx.x; i < p.block_rows * p.d; i += FWD_THREADS)
                if (q_base + i / p.d < p.lq) p.out[((size_t)bh * p.lq + q_base) * p.d + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int off = lk - p.lq;

    // number of key tiles each query tile visits
    int n_t[2];
#pragma unroll
    for (int t = 0; t < 2; t++) {
        // PAIR: both CTAs walk the key tiles of the later of the two paired tiles (the earlier one sees
        // its last key tile fully masked), and a pair of tiles exists if its first tile does
        const int qs_first = PAIR ? qblock * 512 + t * 256 : q_base + t * 128;
        const int qs_last = PAIR ? qs_first + 128 : qs_first;
        if (qs_first >= p.lq || (!PAIR && t == 1 && p.block_rows == 128)) {
            n_t[t] = 0;
        } else {
            const int visible = p.causal ? min(lk, qs_last + 128 + off) : lk;
            n_t[t] = (visible + 127) / 128;
        }
    }
    const int n = max(n_t[0], n_t[1]);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(BAR(B_Q), 1);
        for (int s = 0; s < C::KSTAGES; s++) {
            mbar_init(BAR(B_KFULL + s), 1);
            mbar_init(BAR(B_KEMPTY + s), 2);  // one commit from each MMA warp
        }
        for (int s = 0; s < C::VSTAGES; s++) {
            mbar_init(BAR(B_VFULL + s), 1);
            mbar_init(BAR(B_VEMPTY + s), 2);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(BAR(B_S + t), 1);
            mbar_init(BAR(B_R + t), PAIR ? 8 : 4);          // one arrival per softmax warp (of both CTAs of a pair)
            mbar_init(BAR(B_P + 2 * t), PAIR ? 8 : 4);      // first 64 keys of P written (one arrival per warp)
            mbar_init(BAR(B_P + 2 * t + 1), PAIR ? 8 : 4);  // last 64 keys of P written
            mbar_init(BAR(B_O + t), 1);
        }
        fence_mbar_init();
    }
    if (warp == 11) {
        if constexpr (PAIR) {
            tmem_alloc_pair(smem_u32(tmem_slot), 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), 512);
            tmem_relinquish();
        }
    }
    if (warp == 10 && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp >= 8) {
        reg_dealloc_40();
        if (warp == 10 && lane == 0) {
            // ------------------------------------------------------------ TMA producer
            // In a pair every CTA loads its own tiles; the bytes of both are counted by rank 0's
            // barriers, whose expected total rank 0 announces.
            constexpr int NCTA = PAIR ? 2 : 1;
            const int ntiles_q = (n_t[1] > 0) ? 2 : 1;
            if (crank == 0) mbar_arrive_expect_tx(BAR(B_Q), NCTA * ntiles_q * C::TILE_BYTES);
            for (int t = 0; t < ntiles_q; t++)
                for (int s = 0; s < C::NSUB; s++)
                    f_tma_3d<PAIR>(smem_base + C::OFF_Q + t * C::TILE_BYTES + s * C::SUB_BYTES, &tm_q,
                                   BAR(B_Q), s * 64, q_base + t * TSTEP, p.splits > 1 ? unit : bh);
            int k_issued = 0, v_issued = 0;
            for (int j = 0; j < n; j++) {
                const int ks = j % C::KSTAGES, vs = j % C::VSTAGES;
                if (!mbar_wait(BAR(B_KEMPTY + ks), ((j / C::KSTAGES) & 1) ^ 1, abort_flag, p.status, W_TMA_KEMPTY)) break;
                if (crank == 0) mbar_arrive_expect_tx(BAR(B_KFULL + ks), NCTA * C::K_BYTES);
                for (int s = 0; s < C::NSUB; s++)  // PAIR: this CTA's 64 of the tile's 128 keys
                    f_tma_3d<PAIR>(smem_base + C::OFF_K + ks * C::K_BYTES + s * C::K_SUB_BYTES, &tm_k,
                                   BAR(B_KFULL + ks), s * 64, k_row0 + j * 128 + (PAIR ? (int)crank * 64 : 0), unit);
                k_issued = j + 1;
                if (!mbar_wait(BAR(B_VEMPTY + vs), ((j / C::VSTAGES) & 1) ^ 1, abort_flag, p.status, W_TMA_VEMPTY)) break;
                if (crank == 0) mbar_arrive_expect_tx(BAR(B_VFULL + vs), NCTA * C::V_BYTES);
                if constexpr (PAIR) {              // this CTA's 64 of the tile's 128 columns
                    f_tma_3d<PAIR>(smem_base + C::OFF_V + vs * C::V_BYTES, &tm_v, BAR(B_VFULL + vs), (int)crank * 64,
                                   k_row0 + j * 128, unit);
                } else {
                    for (int s = 0; s < C::NSUB; s++)
                        tma_load_3d(smem_base + C::OFF_V + vs * C::V_BYTES + s * C::SUB_BYTES, &tm_v,
                                    BAR(B_VFULL + vs), s * 64, k_row0 + j * 128, unit);
                }
                v_issued = j + 1;
            }
            // Do not leave the CTA while one of its own copies is still landing in shared memory:
            // a bounded poll (ignoring the abort flag; a copy that was issued always completes) on
            // the full-barrier of every stage still in flight.
            // (In a pair rank 0's barriers count the copies of both CTAs, and the cluster barrier at the
            // end keeps rank 1 resident until rank 0 has passed this point.)
            if (crank == 0) {
                const long long t0 = clock64();
                for (int j = max(0, k_issued - C::KSTAGES); j < k_issued; j++)
                    while (!mbar_try_wait(BAR(B_KFULL + j % C::KSTAGES), (j / C::KSTAGES) & 1) &&
                           clock64() - t0 < kWaitLimitCycles) {}
                for (int j = max(0, v_issued - C::VSTAGES); j < v_issued; j++)
                    while (!mbar_try_wait(BAR(B_VFULL + j % C::VSTAGES), (j / C::VSTAGES) & 1) &&
                           clock64() - t0 < kWaitLimitCycles) {}
                while (!mbar_try_wait(BAR(B_Q), 0) && clock64() - t0 < kWaitLimitCycles) {}
            }
        } else if ((warp == 8 || warp == 9) && crank == 0) {  // all 32 lanes, converged; one elected lane issues
            // ------------------------------------------------------------ MMA issue for tile t (of both CTAs of a pair)
            const int t = warp - 8;
            constexpr uint32_t IDESC_S = idesc_bf16_f32(PAIR ? 256 : 128, 128, 0, 0);
            constexpr uint32_t IDESC_O = idesc_bf16_f32(PAIR ? 256 : 128, HD, 0, 1);
            const int nt = n_t[t], no = n_t[1 - t];  // key tiles of this tile / of the other tile
            const uint32_t q_lo = desc_lo(smem_base + C::OFF_Q + t * C::TILE_BYTES, 16);
            bool ok = mbar_wait(BAR(B_Q), 0, abort_flag, p.status, W_MMA_Q);
            // The score buffer is used in the order S0(0) S1(0) S0(1) S1(1) ...; each user waits until
            // the softmax warps of the previous user have copied their scores out.
            auto issue_s = [&](int j) {
                if (t == 0) {
                    if (j >= 1) {  // previous user: S1(j-1) if the other tile has it, else our own S0(j-1)
                        const int pt = (j - 1 < no) ? 1 : 0;
                        ok = ok && mbar_wait(BAR(B_R + pt), (j - 1) & 1, abort_flag, p.status, W_MMA_R);
                    }
                } else {           // previous user: S0(j) if the other tile has it, else our own S1(j-1)
                    if (j < no)
                        ok = ok && mbar_wait(BAR(B_R + 0), j & 1, abort_flag, p.status, W_MMA_R);
                    else if (j >= 1)
                        ok = ok && mbar_wait(BAR(B_R + 1), (j - 1) & 1, abort_flag, p.status, W_MMA_R);
                }
                tc_fence_after();
                const uint32_t k_lo = desc_lo(smem_base + C::OFF_K + (j % C::KSTAGES) * C::K_BYTES, 16);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t o16 = ((ks / 4) * C::SUB_BYTES + (ks % 4) * 32) >> 4;
                    const uint32_t k16 = ((ks / 4) * C::K_SUB_BYTES + (ks % 4) * 32) >> 4;
                    f_mma_ss<PAIR>(tmem + C::TMEM_S, q_lo + o16, k_lo + k16, IDESC_S, ks > 0);
                }
                f_commit<PAIR>(BAR(B_S + t));
            };
            // O_t += P_t(j) V_j for keys [64*half, 64*half + 64) of the tile
            auto issue_pv_half = [&](int j, int half) {
                ok = ok && mbar_wait(BAR(B_P + 2 * t + half), j & 1, abort_flag, p.status, W_MMA_P);
                tc_fence_after();
                const uint32_t v_lo = desc_lo(smem_base + C::OFF_V + (j % C::VSTAGES) * C::V_BYTES, C::SUB_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++) {
                    const int ks = half * 4 + k4;
                    f_mma_ts<PAIR>(tmem + C::TMEM_O + t * HD, tmem + C::TMEM_P + t * 64 + ks * 8, v_lo + ks * (2048 >> 4),
                                   IDESC_O, (j > 0 || ks > 0) ? 1u : 0u);
                }
                if (half == 1) f_commit<PAIR>(BAR(B_O + t));
            };
            // Both MMA warps release every K and V stage (the "empty" barriers count two commits), also
            // for key tiles this query tile does not visit; a warp waits for the stage to be full
            // before it commits, so that its arrival can never land in an earlier phase of the barrier.
            ok = ok && mbar_wait(BAR(B_KFULL + 0), 0, abort_flag, p.status, W_MMA_K);
            if (nt > 0) issue_s(0);
            f_commit<PAIR>(BAR(B_KEMPTY + 0));
            // Step j of this tile: S_t(j+1), then the two halves of PV_t(j). The score MMA comes
            // first: its buffer is free (the other tile copied out) about half a period before this
            // tile's probabilities are ready.
            for (int j = 0; j < n && ok; j++) {
                if (j + 1 < n) {
                    ok = ok && mbar_wait(BAR(B_KFULL + (j + 1) % C::KSTAGES), ((j + 1) / C::KSTAGES) & 1, abort_flag,
                                         p.status, W_MMA_K);
                    if (j + 1 < nt) issue_s(j + 1);
                    f_commit<PAIR>(BAR(B_KEMPTY + (j + 1) % C::KSTAGES));  // our reads of K(j+1) are issued
                }
                ok = ok && mbar_wait(BAR(B_VFULL + j % C::VSTAGES), (j / C::VSTAGES) & 1, abort_flag, p.status, W_MMA_V);
                if (!PAIR && p.seq_lens && j < nt && j * 128 + 128 > lk) {
                    // Cache decode with a per-sequence length below the tensor map's extent: TMA only
                    // zero-fills rows past the MAP's end, so V rows [lk, ...) of this tile hold whatever
                    // the cache holds there, and 0 * Inf (or NaN) would poison the product although
                    // their probabilities are exactly zero. Zero those rows in shared memory (a row is
                    // 128 bytes of each 64-column sub-tile; the swizzle only permutes inside a row).
                    uint8_t *vt = smem_gen + C::OFF_V + (j % C::VSTAGES) * C::V_BYTES;
                    const int r0 = lk - j * 128;
                    for (int i = lane; i < (128 - r0) * C::NSUB * 8; i += 32) {
                        const int rr = r0 + i / (C::NSUB * 8), sub = (i / 8) % C::NSUB, ch = i % 8;
                        *reinterpret_cast<uint4 *>(vt + sub * C::SUB_BYTES + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
                if (j < nt) {
                    issue_pv_half(j, 0);
                    issue_pv_half(j, 1);
                }
                f_commit<PAIR>(BAR(B_VEMPTY + j % C::VSTAGES));  // our reads of V(j) are issued
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax + epilogue
        reg_alloc_232();
        const int t = warp / 4;                   // which query tile
        const int r = threadIdx.x % 128;          // row inside the tile == TMEM lane
        const int row = q_base + t * TSTEP + r;   // query row
        const uint32_t lane_sel = (uint32_t)((warp % 4) * 32) << 16;
        const uint32_t ts = tmem + lane_sel + C::TMEM_S;           // the shared score buffer
        const uint32_t tp = tmem + lane_sel + C::TMEM_P + t * 64;  // this tile's probabilities
        const uint32_t to = tmem + lane_sel + C::TMEM_O + t * HD;
        const int nk = n_t[t];
        const float c = p.scale_log2;
        const int limit_row = p.causal ? min(lk - 1, row + off) : lk - 1;
        const int limit_tile = p.causal ? min(lk - 1, q_base + t * TSTEP + off) : lk - 1;
        // where this warp reports "scores read" and "P written": the issuing CTA's barriers
        const uint32_t bar_r = PAIR ? map_to_cta(BAR(B_R + t), 0) : BAR(B_R + t);
        const uint32_t bar_p = PAIR ? map_to_cta(BAR(B_P + 2 * t), 0) : BAR(B_P + 2 * t);
        auto arrive = [&](uint32_t bar) {
            if constexpr (PAIR) mbar_arrive_cluster(bar); else mbar_arrive(bar);
        };

        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nk; j++) {
            ok = ok && mbar_wait(BAR(B_S + t), j & 1, abort_flag, p.status, W_SM_S);
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                uint32_t u[32];
                tmem_ld_32x32b_x32(ts + ch * 32, u);
#pragma unroll
                for (int i = 0; i < 32; i++) s[ch * 32 + i] = __uint_as_float(u[i]);
            }
            tmem_wait_ld();
            // The scores are in registers: hand the buffer to the other tile.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive(bar_r);

            if (j * 128 + 127 > limit_tile) {
#pragma unroll
                for (int i = 0; i < 128; i++)
                    if (j * 128 + i > limit_row) s[i] = (c > 0.f) ? -INFINITY : INFINITY;
            }
            // row maximum (minimum for a negative scale): 8 independent chains of 3-input max
            float mx8[8];
#pragma unroll
            for (int i = 0; i < 8; i++) mx8[i] = s[i];
            if (c > 0.f) {
#pragma unroll
                for (int i = 8; i + 16 <= 128; i += 16)
#pragma unroll
                    for (int k8 = 0; k8 < 8; k8++) mx8[k8] = max3(mx8[k8], s[i + k8], s[i + 8 + k8]);
#pragma unroll
                for (int k8 = 0; k8 < 8; k8++) mx8[k8] = fmaxf(mx8[k8], s[120 + k8]);
                mx8[0] = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
            } else {
#pragma unroll
                for (int i = 8; i + 16 <= 128; i += 16)
#pragma unroll
                    for (int k8 = 0; k8 < 8; k8++) mx8[k8] = min3(mx8[k8], s[i + k8], s[i + 8 + k8]);
#pragma unroll
                for (int k8 = 0; k8 < 8; k8++) mx8[k8] = fminf(mx8[k8], s[120 + k8]);
                mx8[0] = min3(min3(mx8[0], mx8[1], mx8[2]), min3(mx8[3], mx8[4], mx8[5]), fminf(mx8[6], mx8[7]));
            }
            const float mx = mx8[0];
            const float m_new = fmaxf(m_ref, mx * c);
            bool o_done = (j == 0);  // P(j-1) consumed by the PV MMA, so the P columns may be overwritten
            if (j == 0) {
                m_ref = m_new;  // finite: key 0 is visible to every row
            } else {
                const bool need = (m_new - m_ref) > RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffu, need)) {
                    const float alpha = ex2(m_ref - m_new);
                    m_ref = m_new;
                    l *= alpha;
                    ok = ok && mbar_wait(BAR(B_O + t), (j - 1) & 1, abort_flag, p.status, W_SM_O);
                    o_done = true;
                    tc_fence_after();
#pragma unroll
                    for (int ch = 0; ch < HD / 32; ch++) {
                        uint32_t o[32];
                        tmem_ld_32x32b_x32(to + ch * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32b_x32(to + ch * 32, o);
                    }
                }
            }
            const f32x2 negm2 = pack2(-m_ref, -m_ref);
            const f32x2 c2 = pack2(c, c);
            f32x2 sum2[4] = {0, 0, 0, 0};  // bit pattern of (0.f, 0.f)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t pk[2][16];
#pragma unroll
                for (int c2i = 0; c2i < 2; c2i++) {
                    const int ch = 2 * half + c2i;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const f32x2 x2 = fma2(pack2(s[ch * 32 + 2 * i], s[ch * 32 + 2 * i + 1]), c2, negm2);
                        float p0, p1;
                        if (i % 4 < EMU) {  // polynomial on the FMA pipe
                            exp2_poly2(x2, p0, p1);
                        } else {            // MUFU
                            float x0, x1;
                            unpack2(x2, x0, x1);
                            p0 = ex2(x0);
                            p1 = ex2(x1);
                        }
                        sum2[i & 3] = add2(sum2[i & 3], pack2(p0, p1));
                        pk[c2i][i] = pack_bf16(p0, p1);
                    }
                }
                if (!o_done) {  // before the first store: PV(j-1) must have read the old P (waited for as
                                // late as possible: the 64 probabilities of this half are already computed)
                    ok = ok && mbar_wait(BAR(B_O + t), (j - 1) & 1, abort_flag, p.status, W_SM_O);
                    tc_fence_after();
                    o_done = true;
                }
                tmem_st_32x32b_x16(tp + (2 * half) * 16, pk[0]);
                tmem_st_32x32b_x16(tp + (2 * half + 1) * 16, pk[1]);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) arrive(bar_p + 8u * (uint32_t)half);
            }
            {
                float a0, a1;
                unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), a0, a1);
                l += a0 + a1;
            }
        }

        if (nk > 0) {
            ok = ok && mbar_wait(BAR(B_O + t), (nk - 1) & 1, abort_flag, p.status, W_SM_OFINAL);
            tc_fence_after();
            const float inv = 1.f / l;
            const bool store = ok && row < p.lq;
            // O / l as bf16 goes through shared memory so that the global stores are coalesced (a
            // thread owns a whole row; storing rows directly makes every store instruction touch 32
            // different lines, which clogs the load/store pipe also for the MMA warps' barrier
            // traffic). The tile's Q buffer is free by now (its last score MMA has completed) and each
            // warp stages only its own 32 rows, so a __syncwarp is all the synchronisation needed.
            // 16-byte chunks are XOR-swizzled by the row to keep both phases free of bank conflicts.
            constexpr int ROWB = HD * 2, CHUNKS = ROWB / 16;
            uint8_t *stage = smem_gen + C::OFF_Q + t * C::TILE_BYTES;
#pragma unroll
            for (int ch = 0; ch < HD / 32; ch++) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(to + ch * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {  // 8 columns = one 16-byte chunk
                    uint4 wv;
                    wv.x = pack_bf16(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv);
                    wv.y = pack_bf16(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv);
                    wv.z = pack_bf16(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv);
                    wv.w = pack_bf16(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv);
                    const int chunk = ch * 4 + q4;
                    const int sw = (chunk & ~7) | ((chunk ^ r) & 7);
                    *reinterpret_cast<uint4 *>(stage + r * ROWB + sw * 16) = wv;
                }
            }
            __syncwarp();
            {
                constexpr int ROWS_PER_ST = 32 / CHUNKS;  // rows covered by one warp-wide 16-byte store
                const int wrow0 = (warp % 4) * 32;        // first row of this warp inside the tile
                const int chunk = lane % CHUNKS;
#pragma unroll
                for (int it = 0; it < 32 / ROWS_PER_ST; it++) {
                    const int rr = wrow0 + it * ROWS_PER_ST + lane / CHUNKS;
                    const int sw = (chunk & ~7) | ((chunk ^ rr) & 7);
                    const uint4 wv = *reinterpret_cast<const uint4 *>(stage + rr * ROWB + sw * 16);
                    const int grow = q_base + t * TSTEP + rr;
                    __nv_bfloat16 *dst = p.out + ((size_t)bh * p.lq + grow) * p.d + chunk * 8;
                    if (ok && grow < p.lq && chunk * 8 < p.d &&
                        EMBER_STORE_OK(dst, p.out, (size_t)p.order.units * p.lq * p.d * 2, 16, p.status))
                        *reinterpret_cast<uint4 *>(dst) = wv;
                }
            }
            if (store && p.lse && EMBER_STORE_OK(p.lse + (size_t)bh * p.lq + row, p.lse, (size_t)p.order.units * p.lq * 4, 4, p.status))
                p.lse[(size_t)bh * p.lq + row] = (m_ref + log2f(l)) * LN2_F;
        }
    }

    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) {
        cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers
        if (warp == 11) tmem_dealloc_pair(tmem, 512);
    } else {
        if (warp == 11) tmem_dealloc(tmem, 512);
    }
}

template <int HD, int EMU>
int launch_pair(const AttnArgs &a, DeviceState *st, cudaStream_t s)
{
    using C = FwdCfg<HD, true>;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tensor_map_bf16_3d(&tq, a.q, HD, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tk, a.k, HD, a.lk, a.bh, 64, 64)) != EMBER_OK) return rc;   // half a key tile per CTA
    if ((rc = make_tensor_map_bf16_3d(&tv, a.v, HD, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;  // half the columns per CTA
    FwdParams p;
    p.out = (__nv_bfloat16 *)a.out;
    p.lse = a.lse;
    p.lq = a.lq;
    p.lk = a.lk;
    p.d = HD;
    p.block_rows = 256;
    p.causal = a.causal;
    p.scale_log2 = a.scale * LOG2E_F;
    p.status = st->status;
    p.splits = 1;
    p.chunk = a.lk;
    p.lens_div = 1;
    p.seq_lens = nullptr;
    auto kern = sm100_fwd_kernel<HD, EMU, true>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    // a work item is a 512-row block of one unit, taken by one pair of CTAs
    p.order = make_work_order(a.bh, (a.lq + 511) / 512, st->sm_count / 2, ((size_t)a.lq + a.lk) * HD * 2 * 2, a.causal != 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)(p.order.units * p.order.blocks));
    cfg.blockDim = dim3(FWD_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;  // consecutive CTAs 2i, 2i+1 form a pair
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    EMBER_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, p));
    return EMBER_OK;
}

// Query rows per CTA. Two tiles (256 rows) share the key/value stream and interleave their softmax
// with each other's MMAs: 1.3x the throughput per SM of a CTA that works on tile 0 alone. One tile per
// CTA (128 rows) makes twice as many CTAs of half the length, which wins while the SMs are not all
// busy: measured at D = 128 on 148 SMs, a launch of up to one 128-row CTA per SM is 12-30 % faster that
// way (8 units x L 2048: 32.8 -> 26.8 us causal, 39.6 -> 28.7 us without a mask), and under a causal
// mask, whose last blocks are the longest, up to two per SM from L = 2048 (16 x 2048: 34.3 -> 30.8 us;
// 8 x 4096: 59.5 -> 46.5 us); beyond that the two-tile form is faster (16 x 4096: 61.7 against 89.1 us).
// A row's arithmetic does not depend on the choice: both forms give the same bits.
// ember_set_forward_block_rows (initially EMBER_FWD_ROWS=128|256) forces one form, for tests and tuning.
static int g_fwd_rows = -1;  // -1: not read from the environment yet; 0: choose per call

static int fwd_rows_setting()
{
    if (g_fwd_rows < 0) {
        const char *e = getenv("EMBER_FWD_ROWS");
        const int v = e ? atoi(e) : 0;
        g_fwd_rows = (v == 128 || v == 256) ? v : 0;
    }
    return g_fwd_rows;
}

static int fwd_block_rows(const AttnArgs &a, DeviceState *st)
{
    const int forced = fwd_rows_setting();
    if (forced == 128 || forced == 256) return forced;
    const long long ctas128 = (long long)a.bh * ((a.lq + 127) / 128);
    const int sms = st->sm_count > 0 ? st->sm_count : 148;
    if (a.lq <= 128) return 256;  // a single tile either way
    if (ctas128 <= sms) return 128;
    if (a.causal && a.lq >= 2048 && ctas128 <= 2LL * sms) return 128;
    return 256;
}

template <int HD, int EMU>
int launch(const AttnArgs &a, DeviceState *st, cudaStream_t s)
{
    using C = FwdCfg<HD>;
    CUtensorMap tq, tk, tv;
    int rc;
    // a.d < HD: the maps describe rows of a.d elements; a box reaches to column HD and reads zeros there
    if ((rc = make_tensor_map_bf16_3d(&tq, a.q, a.d, a.lq, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tk, a.k, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tv, a.v, a.d, a.lk, a.bh, 64, 128)) != EMBER_OK) return rc;
    FwdParams p;
    p.out = (__nv_bfloat16 *)a.out;
    p.lse = a.lse;
    p.lq = a.lq;
    p.lk = a.lk;
    p.d = a.d;
    p.block_rows = fwd_block_rows(a, st);
    p.causal = a.causal;
    p.scale_log2 = a.scale * LOG2E_F;
    p.status = st->status;
    p.splits = 1;
    p.chunk = a.lk;
    p.lens_div = 1;
    p.seq_lens = nullptr;
    auto kern = sm100_fwd_kernel<HD, EMU, false>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    p.order = make_work_order(a.bh, (a.lq + p.block_rows - 1) / p.block_rows, st->sm_count, ((size_t)a.lq + a.lk) * HD * 2 * 2,  // Q, O, K, V
                              a.causal != 0);
    dim3 grid((unsigned)(p.order.units * p.order.blocks));
    kern<<<grid, FWD_THREADS, C::SMEM_BYTES, s>>>(tq, tk, tv, p);
    EMBER_CUDA_TRY(cudaGetLastError());
    return EMBER_OK;
}

// Merges the normalised partial outputs of the splits of one (unit, query row):
// out = sum_s w_s O_s / sum_s w_s with w_s = exp(lse_s - max lse). One block per (unit, row).
__global__ void split_merge_kernel(const __nv_bfloat16 *__restrict__ o_part, const float *__restrict__ lse_part,
                                   __nv_bfloat16 *__restrict__ out, float *__restrict__ lse, int rows_per_unit, int splits,
                                   int d)
{
    const size_t unit = blockIdx.x / rows_per_unit;
    const int row = blockIdx.x - (int)unit * rows_per_unit;
    float mx = -INFINITY;
    for (int s = 0; s < splits; s++) mx = fmaxf(mx, lse_part[(unit * splits + s) * rows_per_unit + row]);
    float wsum = 0.f;
    for (int s = 0; s < splits; s++) {
        const float ls = lse_part[(unit * splits + s) * rows_per_unit + row];
        if (ls != -INFINITY) wsum += expf(ls - mx);
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;  // every split empty: zeros and lse = -inf
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; s++) {
            const float ls = lse_part[(unit * splits + s) * rows_per_unit + row];
            if (ls != -INFINITY)
                acc += expf(ls - mx) * __bfloat162float(o_part[((unit * splits + s) * rows_per_unit + row) * (size_t)d + c]);
        }
        out[((size_t)unit * rows_per_unit + row) * d + c] = __float2bfloat16_rn(acc * inv);
    }
    if (lse && threadIdx.x == 0) lse[unit * rows_per_unit + row] = wsum > 0.f ? mx + logf(wsum) : -INFINITY;
}

template <int HD>
int launch_cache_decode(const CacheDecodeArgs &a, DeviceState *st, cudaStream_t s)
{
    using C = FwdCfg<HD>;
    const int units = a.batch * a.kv_heads, rows = a.q_heads / a.kv_heads;
    CUtensorMap tq, tk, tv;
    int rc;
    if ((rc = make_tensor_map_bf16_3d(&tq, a.q, HD, rows, units, 64, 128)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tk, a.k_cache, HD, a.lk, units, 64, 128, a.capacity)) != EMBER_OK) return rc;
    if ((rc = make_tensor_map_bf16_3d(&tv, a.v_cache, HD, a.lk, units, 64, 128, a.capacity)) != EMBER_OK) return rc;
    FwdParams p;
    const bool split = a.splits > 1;
    __nv_bfloat16 *o_part = (__nv_bfloat16 *)a.workspace;
    float *lse_part = (float *)((char *)a.workspace + align_up((size_t)units * a.splits * rows * HD * 2, 256));
    p.out = split ? o_part : (__nv_bfloat16 *)a.out;
    p.lse = split ? lse_part : a.lse;
    p.lq = rows;
    p.lk = a.lk;
    p.d = HD;
    p.block_rows = 256;
    p.causal = 0;
    p.scale_log2 = a.scale * LOG2E_F;
    p.status = st->status;
    p.splits = a.splits;
    p.chunk = a.chunk;
    p.lens_div = a.kv_heads;
    p.seq_lens = a.seq_lens;
    p.order = make_work_order(units * a.splits, 1, st->sm_count, 1, false);
    auto kern = sm100_fwd_kernel<HD, 1, false>;
    EMBER_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    kern<<<(unsigned)(units * a.splits), FWD_THREADS, C::SMEM_BYTES, s>>>(tq, tk, tv, p);
    EMBER_CUDA_TRY(cudaGetLastError());
    if (split) {
        split_merge_kernel<<<units * rows, 128, 0, s>>>(o_part, lse_part, (__nv_bfloat16 *)a.out, a.lse, rows, a.splits, HD);
        EMBER_CUDA_TRY(cudaGetLastError());
    }
    return EMBER_OK;
}

}  // namespace

bool sm100_fwd_supported(const AttnArgs &a)
{
    if (a.dtype != EMBER_BF16) return false;
    // Rows of any multiple of 8 elements up to 128 (16-byte rows for the TMA copies and the epilogue's
    // stores): the kernel runs at 64 or 128 columns and the copies pad with zeros, which changes neither
    // the scores (zero products) nor the valid output columns.
    if (a.d < 8 || a.d > 128 || a.d % 8 != 0) return false;
    if (!(a.scale != 0.f) || !isfinite(a.scale)) return false;
    if ((long long)a.bh * ((a.lq + 255) / 256) > 0x7fffffffLL) return false;
    // TMA needs 16-byte aligned bases; the epilogue stores 16-byte vectors.
    const uintptr_t bits = (uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v;
    return (bits & 15) == 0 && ((uintptr_t)a.out & 15) == 0;
}

// EMBER_FWD_EMU=0..2 sets the share of polynomial exponentials (read once). Default at 128 columns 0:
// with the softmax warps no longer bound by the MUFU, every exponential there measured 1.3 % faster at
// B4 H32 L4096 than a quarter of them on the FMA pipe (0.487 against 0.494 ms), and half of them 5 %
// slower. Default at 64 columns 1: a key tile then needs half the tensor time for the same 16384
// exponentials, the MUFU is the limit, and a quarter on the FMA pipe measured 2.7 % faster (0.421 against
// 0.432 ms at 128 units x L4096 causal; half of them 2 % slower).
static int fwd_emu_setting(int hd)
{
    static int v = -2;
    if (v == -2) {
        const char *e = getenv("EMBER_FWD_EMU");
        v = e ? atoi(e) : -1;
        if (v < 0 || v > 2) v = -1;
    }
    return v >= 0 ? v : (hd <= 64 ? 1 : 0);
}

// EMBER_FWD_PAIR=1 sends D = 128 shapes with more than 256 query rows to the CTA-pair form of the
// kernel (read once). It is off by default: the pair form halves the shared-memory traffic per SM, but
// one thread issues the MMAs of both CTAs, so every hand-over between the second CTA's softmax warps
// and the issuing warp (scores read, P written, scores ready, PV done) crosses SMs, and with ONE score
// buffer ping-ponged between the tiles those latencies sit on the critical path: it measured 0.75x
// (no mask) and 0.67x (causal) of the single-CTA kernel at B4 H32 L4096 D128.
static bool fwd_pair_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("EMBER_FWD_PAIR");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v != 0;
}

int sm100_fwd_set_block_rows(int rows)
{
    const int before = fwd_rows_setting();
    g_fwd_rows = rows;
    return before;
}

int sm100_attention_fwd(const AttnArgs &a, DeviceState *st, cudaStream_t s)
{
    const int emu = fwd_emu_setting(a.d > 64 ? 128 : 64);
    if (a.d > 64) {
        // CTA pairs take 512-row blocks; below three query tiles a pair would mostly idle
        if (a.d == 128 && a.lq > 256 && fwd_pair_enabled()) {
            if (emu == 0) return launch_pair<128, 0>(a, st, s);
            if (emu == 2) return launch_pair<128, 2>(a, st, s);
            return launch_pair<128, 1>(a, st, s);
        }
        if (emu == 0) return launch<128, 0>(a, st, s);
        if (emu == 2) return launch<128, 2>(a, st, s);
        return launch<128, 1>(a, st, s);
    }
    if (emu == 0) return launch<64, 0>(a, st, s);
    if (emu == 2) return launch<64, 2>(a, st, s);
    return launch<64, 1>(a, st, s);
}

// Decode over a contiguous key/value cache on the tensor cores: the query heads that share a K/V
// head are the rows of one 128-row tile (zero-padded), the key axis is cut into splits.
bool sm100_cache_decode_supported(const CacheDecodeArgs &a)
{
    if (a.dtype != EMBER_BF16 || (a.d != 64 && a.d != 128)) return false;
    if (a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > 128) return false;
    if (!(a.scale != 0.f) || !isfinite(a.scale)) return false;
    const uintptr_t bits = (uintptr_t)a.q | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache | (uintptr_t)a.out;
    return (bits & 15) == 0;
}

size_t sm100_cache_decode_workspace_bytes(int units, int rows, int d, int splits)
{
    if (splits <= 1) return 0;
    return align_up((size_t)units * splits * rows * d * 2, 256) + align_up((size_t)units * splits * rows * sizeof(float), 256);
}

int sm100_cache_decode(const CacheDecodeArgs &a, DeviceState *st, cudaStream_t s)
{
    return a.d == 128 ? launch_cache_decode<128>(a, st, s) : launch_cache_decode<64>(a, st, s);
}

}  // namespace ember
