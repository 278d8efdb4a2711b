// Thin inline-PTX layer for sm_100a: mbarriers with bounded waits, TMA gather4,
// tensor-memory management and tcgen05 block-scaled MMA.  Everything the attention kernels need
// from the hardware goes through this file; nothing here is specific to attention.
//
// Conventions
//  * shared-memory operands are passed as 32-bit shared-window addresses (smem_u32()).
//  * a tensor-memory address is (lane << 16) | column.
//  * every wait is bounded: it gives up after about 0.6 s (or as soon as another thread of the
//    CTA pair has raised the abort word) and reports failure to the caller, who leaves through
//    the kernel's normal tear-down.  No trap, no endless spin.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace sm100 {

#define SM100_DEVICE __device__ __forceinline__


SM100_DEVICE uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
SM100_DEVICE uint32_t cluster_cta_rank() {
    uint32_t v;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(v));
    return v;
}
// true in exactly one lane of a converged warp
SM100_DEVICE bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}
// address of the same shared-memory offset in CTA `rank` of the cluster
SM100_DEVICE uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
SM100_DEVICE void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
SM100_DEVICE void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
SM100_DEVICE void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrival on a barrier of another CTA of the cluster (address from map_to_cta()).  Default
// semantics (release at CTA scope): what the peer's consumers read is either tensor memory, ordered
// by tcgen05 fences, or this CTA's own shared memory through the async proxy, ordered by
// fence.proxy.async -- a cluster-scope release fence per arrival would only cost time.
SM100_DEVICE void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
SM100_DEVICE void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// expect_tx + one arrival on a barrier of any CTA of the cluster (address from map_to_cta())
SM100_DEVICE void mbar_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr), "r"(bytes)
                 : "memory");
}
SM100_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Blocking flavour: the hardware may suspend the thread for up to `ns` nanoseconds while the phase
// is pending, so a waiting warp does not compete for issue slots with the warps doing the work.
SM100_DEVICE bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns, bool cluster_scope) {
    uint32_t ok;
    if (cluster_scope)
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(ns)
            : "memory");
    else
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(ns)
            : "memory");
    return ok != 0;
}

// Bounds of the kernels' waits (the loops themselves are written out at the wait sites, see
// attn_sm100.cuh): a suspending wait sleeps in slices of kWaitSliceNs and gives up after kWaitSlices
// of them (about 0.6 s); a polling wait gives up after 2^24 tries.
static constexpr uint32_t kWaitSliceNs = 100000;
static constexpr int kWaitSlices = 6000;
SM100_DEVICE void named_bar_arrive(uint32_t id, uint32_t threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

SM100_DEVICE void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
SM100_DEVICE void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
SM100_DEVICE void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
SM100_DEVICE void cluster_sync() {
    cluster_arrive();
    cluster_wait();
}
SM100_DEVICE void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ----------------------------------------------------------------------------------------------
// TMA
// ----------------------------------------------------------------------------------------------
// Ask for the 128-byte line that holds `p` to be brought into L2; nothing is written back to the thread.
SM100_DEVICE void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
SM100_DEVICE void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Tiled store shared -> global of one 2-D box; the issuing thread groups its stores with tma_store_commit and
// learns that their shared-memory source has been read (tma_store_wait_read) or that they are complete.
SM100_DEVICE void tma_store_2d(const void* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(map), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
SM100_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> SM100_DEVICE void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
SM100_DEVICE void st_shared_16B(uint32_t dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
static constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
static constexpr uint64_t kEvictLast = 0x14F0000000000000ull;
static constexpr uint64_t kEvictNormal = 0x1000000000000000ull;

// gather4: four rows (r0..r3 of a 2-D tensor map whose box is {box_cols, 1}) starting at column `col` land as four
// consecutive box rows at `dst`.  The completion bytes may be routed to a barrier of either CTA of the pair:
// `bar` is a shared::cluster address (own window address, or the peer's from map_to_cta()).
SM100_DEVICE void tma_gather4_pair(uint32_t dst, const void* map, int col, int r0, int r1, int r2,
                                   int r3, uint32_t bar, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes"
        ".cta_group::2.L2::cache_hint [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
        :
        : "r"(dst), "l"(map), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar), "l"(hint)
        : "memory");
}

// ----------------------------------------------------------------------------------------------
// tensor memory
// ----------------------------------------------------------------------------------------------
template <int CG> SM100_DEVICE void tmem_alloc(uint32_t result_smem, uint32_t cols) {
    static_assert(CG == 2, "only CTA-pair (cta_group::2) operations are used");
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem),
                     "r"(cols)
                     : "memory");
}
template <int CG> SM100_DEVICE void tmem_relinquish() {
    static_assert(CG == 2, "only CTA-pair (cta_group::2) operations are used");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG> SM100_DEVICE void tmem_dealloc(uint32_t addr, uint32_t cols) {
    static_assert(CG == 2, "only CTA-pair (cta_group::2) operations are used");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
SM100_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
SM100_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
SM100_DEVICE void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
SM100_DEVICE void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tcgen05.ld/st .32x32b: thread t of the warp accesses lane (warp%4)*32+t, N consecutive columns.
SM100_DEVICE void tmem_st8(uint32_t addr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(addr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]));
}
SM100_DEVICE void tmem_ld32(uint32_t addr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(addr));
}
SM100_DEVICE void tmem_st32(uint32_t addr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]),
        "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
        "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]));
}

// shared -> tensor memory copy of scale-factor rows (16 bytes per row).
// 64 rows; rows 0-31 go to lane quadrants 0 and 1, rows 32-63 to quadrants 2 and 3, in both CTAs of the pair.
SM100_DEVICE void tmem_cp_sf_pair(uint32_t tmem_addr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.64x128b.warpx2::01_23 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc)
                 : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05 block-scaled MMA (E4M3 x E4M3, UE8M0 scale per 32 K-elements, fp32 accumulate)
// ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets in
// 16-byte units, descriptor version 1, swizzle mode in bits 61-63 (2 = 128 B, 4 = 64 B, 0 = none).
SM100_DEVICE constexpr uint64_t smem_desc_base(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    return (uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16) | (uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32) |
           (uint64_t(1) << 46) | (uint64_t(swizzle) << 61);
}
SM100_DEVICE uint64_t smem_desc(uint64_t base, uint32_t smem_addr) {
    return base | uint64_t((smem_addr >> 4) & 0x3FFF);
}
// Instruction descriptor: M, N, UE8M0 scales, E4M3 operands; `b_mn_major` when B's N dimension is
// the contiguous one in shared memory; scale-factor byte selectors for A and B.
SM100_DEVICE constexpr uint32_t mx_idesc(uint32_t m, uint32_t n, bool b_mn_major, uint32_t a_sf, uint32_t b_sf) {
    return ((m >> 4) << 24) | (1u << 23) | ((n >> 3) << 17) | (uint32_t(b_mn_major) << 16) |
           ((a_sf & 3u) << 29) | ((b_sf & 3u) << 4);
}
template <int CG>
SM100_DEVICE void mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                           uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate) {
    static_assert(CG == 2, "only CTA-pair (cta_group::2) operations are used");
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
}
// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread has finished.
// `bar` is a shared::cluster address, so the peer's barrier can be targeted through map_to_cta().
template <int CG> SM100_DEVICE void mma_commit(uint32_t bar) {
    static_assert(CG == 2, "only CTA-pair (cta_group::2) operations are used");
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
}

// ----------------------------------------------------------------------------------------------
// small math helpers with fixed instruction selection (results must not depend on -use_fast_math)
// ----------------------------------------------------------------------------------------------
SM100_DEVICE float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
SM100_DEVICE float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two floats -> two E4M3 bytes (round to nearest even, saturate to +-448); `lo` lands in bits 0-7
SM100_DEVICE uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// smallest UE8M0 byte whose value is >= x (x > 0)
SM100_DEVICE uint32_t cvt_ue8m0_roundup(float x) {
    uint16_t r;
    asm("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xFFu;
}

// 128-byte swizzle: byte offset inside a tile whose rows are 128 bytes and whose base is aligned
// to 1024 bytes (16-byte chunk index XOR row-in-group-of-8).
SM100_DEVICE constexpr uint32_t swz128(uint32_t row, uint32_t byte_in_row) {
    return row * 128u + ((((byte_in_row >> 4) ^ (row & 7u)) << 4) | (byte_in_row & 15u));
}

}  // namespace sm100
