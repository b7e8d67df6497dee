// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention kernels use:
// mbarrier, TMA tensor loads (never multicast), tcgen05 tensor-memory allocation, MMA, loads and
// stores, and the descriptors the MMA reads. Every wait is bounded: after a time limit it
// records where it gave up in a device status word and returns false instead of spinning.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace ember {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Upper bound of one wait, in SM clock cycles (about a quarter of a second). A healthy kernel
// never comes near it: the longest legitimate wait is one CTA's whole work, a few milliseconds.
constexpr long long kWaitLimitCycles = 400LL * 1000 * 1000;

// Waits for the phase with the given parity. On timeout (or when another thread of this CTA
// already gave up, signalled through *abort_flag in shared memory) records the failure and
// returns false; the caller carries on so that the CTA still reaches its common exit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          DeviceStatus *status, int where,
                                          long long limit_cycles = kWaitLimitCycles)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            if (atomicCAS(&status->code, 0, EMBER_ERR_TIMEOUT) == 0) {
                status->where = where;
                status->block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
                status->extra = (int)parity;
            }
            return false;
        }
    }
}

// ---------------------------------------------------------------- TMA (tensor loads, no multicast)
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tile load: coordinates (c0 = innermost element, c1 = row, c2 = batch*head).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap *m, uint32_t bar,
                                            int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// 5-D tile load (matrix views: column, row, head, batch, part).
__device__ __forceinline__ void tma_load_5d(uint32_t dst_smem, const CUtensorMap *m, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// ---------------------------------------------------------------- tcgen05: tensor memory
// Allocates ncols (power of two, 32..512) TMEM columns; the base address lands in *dst_smem.
// Must be executed by one full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Warp-collective commit: the elected lane (the same one the *_lo MMA forms elect) makes the
// mbarrier receive one arrival when every tcgen05.mma it issued before has finished.
__device__ __forceinline__ void tc_commit_elect(uint32_t bar)
{
    asm volatile(
        "{\n"
        ".reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n" ::"r"(bar)
        : "memory");
}

// The mbarrier gets one arrival when every tcgen05.mma this thread issued before has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 bit, 32 consecutive columns: thread t of the warp gets lane (base lane + t),
// register i gets column (base column + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---------------------------------------------------------------- tcgen05: descriptors and MMA
// Shared-memory matrix descriptor for a bf16 operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (the layout a TMA box of 64 bf16 x R rows with SWIZZLE_128B produces; the tile
// base must be 1024-byte aligned). Fields (bit positions): start address >> 4 [0,14), leading
// byte offset >> 4 [16,30), stride byte offset >> 4 [32,46), descriptor version 1 [46,48),
// layout type [61,64) with 2 = 128-byte swizzle.
//   K-major use   (the operand's K runs along the 128-byte row): 8-row groups are SBO = 1024
//                 bytes apart; LBO is unused. Advance K by 16 elements = +32 bytes of address.
//   MN-major use  (the operand's M/N runs along the 128-byte row): 8-row (K) groups are SBO =
//                 1024 bytes apart; the next 64 M/N elements are LBO bytes away (the next
//                 64-column sub-tile). Advance K by 16 rows = +2048 bytes of address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and float32 accumulation.
// Bits: D format [4,6) = 1 (f32); A format [7,10) = 1 (bf16); B format [10,13) = 1 (bf16);
// A major [15], B major [16] (0 = K-major, 1 = MN-major); N >> 3 at [17,23); M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n, int a_mn_major, int b_mn_major)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Lean, WARP-COLLECTIVE forms for issue loops: all 32 lanes of the issuing warp call them
// converged and one elected lane issues the MMA. The MMA warp shares its scheduler with compute
// warps, so every instruction spent per MMA shows up as tensor-pipe idle time; keeping the warp
// converged lets the compiler hold descriptors and loop state on the uniform datapath. The
// descriptor is a 32-bit low word (start address >> 4 | LBO field) advanced by an integer add, and
// a constant high word (SBO = 1024 bytes, version 1, 128-byte swizzle) shared by every operand.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes)
{
    return ((smem_addr & 0x3FFFF) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 da, db;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "mov.b64 da, {%1, %5};\n"
        "mov.b64 db, {%2, %5};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 db;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "mov.b64 db, {%2, %5};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 0 and 1, on the two SMs of one TPC) act as one 256-row MMA: rank 0
// issues, each CTA supplies its own 128 rows of A and its own half of B's N columns from its own
// shared memory, and each CTA's tensor memory receives its 128 rows of the result. Every CTA loads
// its own operands with its own TMA copies (no multicast); the completion bytes of both CTAs are
// counted by rank 0's barrier.
// Programmatic dependent launch. A kernel launched with programmatic stream serialization may have its
// CTAs placed (and run whatever does not depend on the kernel before it on the stream) as soon as every
// CTA of that kernel has passed pdl_launch_dependents(); pdl_wait() then blocks until that kernel has
// completed and its writes are visible. Launched without the attribute, or after something that is
// not a kernel, both are no-ops. Used along forward -> delta -> single-pass backward -> dQ finish.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the CTA of the given rank of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// In the shared::cluster window the rank of the owning CTA is bit 24 of an address; clearing it
// turns the address of a barrier in this CTA into the address of the same barrier in rank 0.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
// 5-D tile load of one CTA of a pair into its OWN shared memory; the bytes are reported to rank 0's
// barrier at the same offset.
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst_smem, const CUtensorMap *m, uint32_t bar, int c0, int c1,
                                                 int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
// Tensor-memory allocation of a CTA pair: one warp of EACH CTA (the same warp index) executes it,
// with the same destination offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Warp-collective (rank 0 only): D[tmem of both CTAs] (+)= A[smem of both] * B[smem of both].
__device__ __forceinline__ void mma_ss_lo_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 da, db;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "mov.b64 da, {%1, %5};\n"
        "mov.b64 db, {%2, %5};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "@q tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}
// Warp-collective (rank 0 only): when every MMA issued before has finished, the barrier at this
// offset receives one arrival in each CTA named in cta_mask (bit r = rank r).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "{\n"
        ".reg .pred q;\n"
        "elect.sync _|q, 0xffffffff;\n"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
        "}\n" ::"r"(bar), "h"(cta_mask)
        : "memory");
}

// Named barrier (ids 1..15; 0 is __syncthreads) over `count` threads, a multiple of 32.
__device__ __forceinline__ void named_bar_sync(int id, int count)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ void reg_alloc_232() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }
__device__ __forceinline__ void reg_alloc_208() { asm volatile("setmaxnreg.inc.sync.aligned.u32 208;"); }
__device__ __forceinline__ void reg_dealloc_40() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }
__device__ __forceinline__ void reg_dealloc_64() { asm volatile("setmaxnreg.dec.sync.aligned.u32 64;"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---------------------------------------------------------------- packed float32 pairs (sm_100)
// Two float32 values in one 64-bit register; one instruction operates on both.
typedef uint64_t f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi)
{
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b)
{
    f32x2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float min3(float a, float b, float c)
{
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}


__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for a pair of x <= ~8 on the FMA/ALU pipes (packed float32 pairs): round-to-nearest split
// x = n + f, f in [-0.5, 0.5], a cubic for 2^f (relative error 7.5e-5, far below bf16 resolution) and
// an exponent-field add for 2^n. Inputs below -125 (masked scores are -inf) are clamped and come out
// as ~2^-125, i.e. zero in bf16.
__device__ __forceinline__ void exp2_poly2(f32x2 x2, float &p0, float &p1)
{
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
    const f32x2 magic = pack2(12582912.f, 12582912.f);  // 1.5 * 2^23: integer part -> low mantissa bits
    const f32x2 xr = add2(x2, magic);
    const f32x2 f = sub2(x2, sub2(xr, magic));
    f32x2 pl = fma2(pack2(0.05517167f, 0.05517167f), f, pack2(0.24261112f, 0.24261112f));
    pl = fma2(pl, f, pack2(0.69326099f, 0.69326099f));
    pl = fma2(pl, f, pack2(0.99992807f, 0.99992807f));
    float r0, r1, q0, q1;
    unpack2(xr, r0, r1);
    unpack2(pl, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

}  // namespace ptx

// Host side: building TMA tensor maps through the driver entry point (no link against libcuda).
int make_tensor_map_bf16_3d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows,
                            uint64_t batch, uint32_t box_inner, uint32_t box_rows, uint64_t batch_stride_rows = 0);

}  // namespace ember
