// Thin inline-PTX layer for sm_100a: mbarrier, TMA (non-multicast), tcgen05/TMEM,
// system-scope flag operations and bounded waits.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace cb {

// Status words written by a kernel that gave up on a wait (all waits are bounded).
enum StatusWord : int {
    ST_CODE = 0,      // 0 = ok, otherwise one of the ERR_* codes
    ST_WHERE = 1,     // which wait site
    ST_RANK = 2,
    ST_INDEX = 3,     // flag index / tile index
    ST_EXPECTED = 4,
    ST_SEEN = 5,
    ST_WORDS = 8
};
enum ErrCode : int {
    ERR_NONE = 0, ERR_FLAG_TIMEOUT = 1, ERR_MBAR_TIMEOUT = 2, ERR_ABORTED = 3,
    ERR_MOE_CAPACITY = 4,      // MoE: the routing needs more receive rows than the buffer holds
    ERR_PARTIAL_RANGE = 5      // reduce family: a partial product does not fit the fp16 exchange format
};
enum WaitSite : int {
    W_ENTERED = 1, W_AG_CHUNK = 2, W_RS_PARTIAL = 3, W_AR_FINAL = 4, W_MBAR_FULL = 5, W_MBAR_EMPTY = 6,
    W_TMEM_FULL = 7, W_TMEM_EMPTY = 8, W_DRAIN = 9, W_TEST = 10, W_MOE_COUNTS = 11, W_MOE_ROWS = 12,
    W_MOE_ACT = 13, W_MOE_COMBINE = 14, W_MXAG = 15, W_TILE_QUEUE = 16
};

struct WaitCtl {
    volatile int *abort_smem;   // CTA-wide abort flag in shared memory
    int *status;                // device status words (global)
    uint64_t deadline_ns;       // %globaltimer value after which waits give up
    int rank;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n .reg .pred P;\n elect.sync _|P, 0xffffffff;\n selp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- failure ----
__device__ __forceinline__ void report_failure(const WaitCtl &c, int code, int where, int index, int expected,
                                               int seen) {
    if (atomicCAS(c.status + ST_CODE, 0, code) == 0) {
        c.status[ST_WHERE] = where;
        c.status[ST_RANK] = c.rank;
        c.status[ST_INDEX] = index;
        c.status[ST_EXPECTED] = expected;
        c.status[ST_SEEN] = seen;
    }
    *c.abort_smem = 1;
}

// --------------------------------------------------------------- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred P;\n mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n selp.u32 %0, 1, 0, P;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (someone timed out) or the
// deadline passed; the caller then leaves its loop and joins the common teardown.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, const WaitCtl &c, int where) {
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*c.abort_smem) return false;
            if (globaltimer_ns() > c.deadline_ns) {
                report_failure(c, ERR_MBAR_TIMEOUT, where, 0, static_cast<int>(parity), 0);
                return false;
            }
        }
    }
    return true;
}

// ------------------------------------------------------------------- TMA ----
__device__ __forceinline__ void prefetch_tensormap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// 2-D tiled load global -> shared, completion on an mbarrier.  No multicast.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const void *tmap, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, uint64_t *bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Untiled bulk copies (16-byte aligned addresses and size).  global -> shared completes on an
// mbarrier; shared -> global (possibly a peer's memory) is tracked by the thread's bulk group.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void *gmem_dst, const void *smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
// 2-D tiled store shared -> global (this GPU's or a peer's memory) as part of the thread's current
// bulk group; rows and columns past the tensor's extent are not written.
__device__ __forceinline__ void tma_store_2d(const void *tmap, const void *smem_src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N committed groups may still be reading their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// at most N committed groups may still be incomplete (their global writes not yet performed)
template <int N>
__device__ __forceinline__ void bulk_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders earlier generic-proxy accesses (including acquired remote writes) before
// later async-proxy (TMA) accesses of the same memory.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// the same, restricted to one state space: shared-memory writes of this thread before a bulk copy
// reads them, or global memory seen through flags before TMA reads it
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// --------------------------------------------------------------- tcgen05 ----
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], dense f16/bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Block-scaled MXFP8 (e4m3/e5m2 data, UE8M0 scale per 32 along K) with scale factors in TMEM.
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
// Block-scaled FP4 (e2m1 data, two per byte, K = 64 per instruction).  VEC4 = true: NVFP4, one UE4M3
// scale per 16 along K (four per instruction, scale_vec::4X); false: MXFP4, one UE8M0 scale per 32
// (two per instruction, scale_vec::2X; the descriptor's sf_id picks the byte pair).
template <bool VEC4>
__device__ __forceinline__ void umma_fp4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa_tmem,
                                         uint32_t sfb_tmem, uint32_t accumulate) {
    if (VEC4) {
        asm volatile(
            "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
            " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(
                d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
            " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(
                d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
            : "memory");
    }
}
// All previously issued tcgen05.mma of this thread arrive on `bar` when they complete.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 16-byte store to a multicast address: the NVSwitch writes the value at the same offset of every bound heap.
// Only for addresses inside a multicast mapping (Team::mc_base); such addresses are never loaded from.
__device__ __forceinline__ void multimem_st_v4(void *mc_addr, const uint4 &v) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ----------------------------------------------------- CTA pairs (cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `smem_addr` (a shared::cta address) in CTA `cta` of this cluster
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive (+ expected transaction bytes) on a barrier given by its shared::cluster address
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion is signalled on a barrier that may
// live in the other CTA of the pair (no multicast: each CTA fetches its own half).
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const void *tmap, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
// the same for a 3-D tensor (used for per-expert weight matrices: the third coordinate picks the expert, so a
// tile that runs past an expert's rows is zero-filled instead of reading its neighbour)
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const void *tmap, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one MMA over both CTAs of the pair: M = 256 (128 rows per CTA), each CTA supplies half of B's columns
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// completion of the pair's MMAs -> one barrier, addressed in shared::cluster space (either CTA)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// block-scaled MXFP8 MMA and scale-factor copy over a CTA pair
__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
// MXFP4 (e2m1, UE8M0 scale per 32, K = 64 per instruction) on a CTA pair
__device__ __forceinline__ void umma_mxfp4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
// NVFP4 (e2m1, UE4M3 scale per 16, K = 64 per instruction, four scales per row and instruction) on a CTA pair
__device__ __forceinline__ void umma_nvfp4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred P;\n setp.ne.b32 P, %6, 0;\n"
        " tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], P;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
// each CTA of the pair copies 32 rows x 128 bit from its own shared memory (same offset) into its own TMEM
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// shared memory -> TMEM copy of scale factors: 32 rows x 128 bit, replicated to the 4 lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// TMEM -> registers: this warp's 32 lanes x 32 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// registers -> TMEM: this warp's 32 lanes x 4 consecutive 32-bit columns (one 16-byte row of a scale atom per lane)
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, const uint4 &v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format: version 1 at bit 46, 3-bit layout type at 61).
// Offsets are in bytes; the hardware fields drop the 4 LSBs.
constexpr uint64_t kSwizzle128B = 2;
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (kSwizzle128B << 61);
}
constexpr uint64_t kNoSwizzle = 0;
__host__ __device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes,
                                                                      uint32_t sbo_bytes) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46);
}

// Instruction descriptor, kind::f16: fp32 accumulate, A K-major, B K- or MN-major.
// fmt: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc_f16(uint32_t fmt, uint32_t m, uint32_t n, uint32_t a_mn_major,
                                                      uint32_t b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}
// Instruction descriptor, kind::mxf8f6f4 block-scaled: e4m3 x e4m3, UE8M0 scales, K-major A and B.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(uint32_t m, uint32_t n, uint32_t a_sf_id, uint32_t b_sf_id) {
    return (b_sf_id << 4) | (0u << 7) | (0u << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) |
           (a_sf_id << 29);
}

// Instruction descriptor, kind::mxf4nvf4 block-scaled: e2m1 x e2m1 (format code 1), K-major A and B;
// ue8m0 = 1: UE8M0 scales (MXFP4), 0: UE4M3 scales (NVFP4).
__host__ __device__ constexpr uint32_t make_idesc_fp4(uint32_t m, uint32_t n, uint32_t a_sf_id, uint32_t b_sf_id,
                                                      uint32_t ue8m0) {
    return (b_sf_id << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (ue8m0 << 23) | ((m >> 4) << 24) | (a_sf_id << 29);
}

// ------------------------------------------------- system-scope flag ops ----
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Bounded spin until *flag >= expected (flags are epochs: monotonic, single writer).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t *flag, uint32_t expected, const WaitCtl &c, int where,
                                             int index) {
    uint32_t spins = 0;
    uint32_t seen;
    while (static_cast<int32_t>((seen = ld_acquire_sys(flag)) - expected) < 0) {
        if ((++spins & 255u) == 0) {
            if (*c.abort_smem) return false;
            if (globaltimer_ns() > c.deadline_ns) {
                report_failure(c, ERR_FLAG_TIMEOUT, where, index, static_cast<int>(expected), static_cast<int>(seen));
                return false;
            }
        }
    }
    return true;
}

// Bounded spin until a counter in shared memory, advanced by another warp of the CTA, exceeds idx.
__device__ __forceinline__ bool wait_smem_counter_gt(const uint32_t *ctr, uint32_t idx, const WaitCtl &c, int where) {
    uint32_t spins = 0, seen;
    for (;;) {
        asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(seen) : "r"(smem_u32(ctr)) : "memory");
        if (seen > idx) return true;
        if ((++spins & 255u) == 0) {
            if (*c.abort_smem) return false;
            if (globaltimer_ns() > c.deadline_ns) {
                report_failure(c, ERR_FLAG_TIMEOUT, where, static_cast<int>(idx), static_cast<int>(idx) + 1,
                               static_cast<int>(seen));
                return false;
            }
        }
    }
}
__device__ __forceinline__ void st_release_cta_smem(uint32_t *ctr, uint32_t v) {
    asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(ctr)), "r"(v) : "memory");
}

// Words in the shared memory of a CTA of this cluster, given by their shared::cluster address (mapa_cluster):
// plain store, release store at cluster scope, and the matching acquire load / bounded wait on this
// CTA's own copy (the writer may be the other CTA of the pair).
__device__ __forceinline__ void st_cluster_smem(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_cluster_smem(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.release.cluster.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_cluster_smem(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.cluster.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ bool wait_cluster_counter_gt(const uint32_t *ctr, uint32_t idx, const WaitCtl &c, int where) {
    uint32_t spins = 0, seen;
    for (;;) {
        seen = ld_acquire_cluster_smem(ctr);
        if (seen > idx) return true;
        if ((++spins & 255u) == 0) {
            if (*c.abort_smem) return false;
            if (globaltimer_ns() > c.deadline_ns) {
                report_failure(c, ERR_FLAG_TIMEOUT, where, static_cast<int>(idx), static_cast<int>(idx) + 1,
                               static_cast<int>(seen));
                return false;
            }
        }
    }
}

// Whole warp: lane q waits for flags[q], q + 32, ... (< count); every lane gets true when all are up.
__device__ __forceinline__ bool wait_flags_warp(const uint32_t *flags, int count, uint32_t expected, const WaitCtl &c,
                                                int where, int index0) {
    bool mine = true;
    for (int q = threadIdx.x & 31; q < count && mine; q += 32)
        mine = wait_flag_ge(flags + q, expected, c, where, index0 + q);
    const bool all = __all_sync(0xffffffffu, mine);
    __syncwarp();
    return all;
}

// ---------------------------------------------------------------- helpers ----
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    __device__ static __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
    }
};
template <> struct Pack2<__half> {
    __device__ static __forceinline__ uint32_t pack(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2 *>(&u));
    }
};

// Reduce family: a partial tile travels as fp16 (when `fp16` is set) or in the output type T.
template <typename T>
__device__ __forceinline__ uint32_t pack_partial(float a, float b, bool fp16) {
    return fp16 ? Pack2<__half>::pack(a, b) : Pack2<T>::pack(a, b);
}
template <typename T>
__device__ __forceinline__ float2 unpack_partial(uint32_t u, bool fp16) {
    return fp16 ? Pack2<__half>::unpack(u) : Pack2<T>::unpack(u);
}
// a value beyond the fp16 range was sent as a partial: recorded (first error wins), nothing is aborted
__device__ __forceinline__ void report_partial_range(int *status, int rank, int tile) {
    if (atomicCAS(status + ST_CODE, 0, ERR_PARTIAL_RANGE) == 0) {
        status[ST_WHERE] = W_RS_PARTIAL;
        status[ST_RANK] = rank;
        status[ST_INDEX] = tile;
    }
}

}  // namespace cb
