// MX quantisation + AllGather (the reference's MxQuantAllGather,
// include/catccos/comm/kernel/mx_quant_allgather.hpp:57-288): every rank quantises its bf16 rows
// (e4m3 codes + E8M0 scale per 32) and all ranks end up with all ranks' codes and scales.
//
// The caller's outputs are ordinary device memory, so the exchange goes through the symmetric
// region: quantise into the own slot of the outputs, push that slot (codes then scales, as one
// byte range) into every peer's staging slot with bulk copies in 32 KiB units, one epoch flag per
// unit (flag-driven, no world barrier, like the reference), and copy the peers' units from staging
// into the outputs as their flags arrive.
#include "mxq_allgather.h"

#include <string.h>

#include "mx_quant.h"
#include "ptx.cuh"

namespace cb {

namespace {

constexpr int kQagLanes = 4;
constexpr int kQagUnitBytes = 32 * 1024;
constexpr int kQagThreads = 256;

struct QagRank {
    uint8_t *codes;      // [R*m, n] output
    uint8_t *scales;     // [R*m, sld] output
};
struct QagParams {
    QagRank ranks[kMaxRanks];
    uint8_t *heap_base[kMaxRanks];
    uint64_t symm_off;
    size_t codes_bytes, scale_bytes, slot_bytes;   // per rank; slot = codes (padded to 1 KiB) + scales (padded)
    int world, rank_base, n_local, ctas_per_rank;
    uint32_t epoch;
    uint64_t timeout_ns;
    int *status;
};

struct QagSmem {
    uint64_t bar[kQagLanes];
    uint64_t group;
    int abort_flag;
    int ok;
};

__global__ void __launch_bounds__(kQagThreads) mxq_allgather_kernel(const QagParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ QagSmem sh;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const QagRank &ra = p.ranks[lrank];
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int l = 0; l < kQagLanes; ++l) mbar_init(&sh.bar[l], 1);
        mbar_init(&sh.group, kQagThreads);
        sh.abort_flag = 0;
        sh.ok = 1;
        mbar_init_fence();
    }
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &sh.abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    auto flagp = [&](int pe, uint32_t w) { return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + w; };
    const size_t codes_pad = p.slot_bytes - ((p.scale_bytes + 1023) / 1024 * 1024);
    const int units = static_cast<int>((p.slot_bytes + kQagUnitBytes - 1) / kQagUnitBytes);

    if (cta == 0 && tid < R && tid != rank) {
        fence_sys();
        st_release_sys(flagp(tid, kFlagEntered + rank), p.epoch);
    }
    // byte `off` of my slot lives in the codes output or (after the padded codes) in the scales output
    auto src_ptr = [&](const QagRank &q, int slot_rank, size_t off, size_t *run) -> uint8_t * {
        if (off < codes_pad) {
            *run = (off < p.codes_bytes) ? p.codes_bytes - off : 0;
            return q.codes + static_cast<size_t>(slot_rank) * p.codes_bytes + off;
        }
        const size_t so = off - codes_pad;
        *run = (so < p.scale_bytes) ? p.scale_bytes - so : 0;
        return q.scales + static_cast<size_t>(slot_rank) * p.scale_bytes + so;
    };

    // ---- push my slot to every peer (destination rank-1 first), kQagLanes threads drive bulk copies ----
    if (tid < kQagLanes) {
        uint8_t *buf = smem + tid * kPushPieceBytes;
        uint64_t *bar = &sh.bar[tid];
        const int lane_id = cta * kQagLanes + tid;
        const int n_lanes = p.ctas_per_rank * kQagLanes;
        const int total = (R - 1) * units;
        uint32_t piece = 0, entered_ok = 0;
        bool ok = true;
        for (int u = lane_id; u < total && ok; u += n_lanes) {
            const int jj = u / units, un = u - jj * units;
            const int d = (rank + R - 1 - jj) % R;
            if (!((entered_ok >> d) & 1)) {
                if (!(ok = wait_flag_ge(flagp(rank, kFlagEntered + d), p.epoch, ctl, W_ENTERED, d))) break;
                entered_ok |= 1u << d;
            }
            const size_t u0 = static_cast<size_t>(un) * kQagUnitBytes;
            const size_t u1 = min(p.slot_bytes, u0 + kQagUnitBytes);
            uint8_t *dst_slot = p.heap_base[d] + p.symm_off + static_cast<size_t>(rank) * p.slot_bytes;
            for (size_t off = u0; off < u1 && ok;) {
                size_t run;
                const uint8_t *src = src_ptr(ra, rank, off, &run);
                size_t len = min(min(run, static_cast<size_t>(kPushPieceBytes)), u1 - off);
                if (len == 0) {            // padding between the two parts of the slot
                    off = (off < codes_pad) ? min(codes_pad, u1) : u1;
                    continue;
                }
                len = (len + 15) & ~static_cast<size_t>(15);      // parts are multiples of 16 bytes (checked on the host)
                bulk_wait_read<0>();
                mbar_expect_tx(bar, static_cast<uint32_t>(len));
                bulk_load(buf, src, static_cast<uint32_t>(len), bar);
                if (!(ok = mbar_wait(bar, piece & 1, ctl, W_DRAIN))) break;
                bulk_store(dst_slot + off, buf, static_cast<uint32_t>(len));
                bulk_commit();
                ++piece;
                off += len;
            }
            if (!ok) break;
            bulk_wait<0>();
            fence_proxy_async_global();
            fence_sys();
            st_release_sys(flagp(d, kFlagOpBase + rank * units + un), p.epoch);
        }
        bulk_wait<0>();
    }

    // ---- copy the peers' units from my staging into the outputs as they arrive ----
    uint32_t gphase = 0;
    const int total_in = (R - 1) * units;
    for (int u = cta; u < total_in; u += p.ctas_per_rank) {
        const int jj = u / units, un = u - jj * units;
        const int s = (rank + 1 + jj) % R;
        if (tid == 0 && !wait_flag_ge(flagp(rank, kFlagOpBase + s * units + un), p.epoch, ctl, W_MXAG, s * units + un))
            *reinterpret_cast<volatile int *>(&sh.ok) = 0;
        mbar_arrive(&sh.group);
        const bool okw = mbar_wait(&sh.group, gphase, ctl, W_DRAIN);
        gphase ^= 1;
        if (!okw || !*reinterpret_cast<volatile int *>(&sh.ok)) break;
        const size_t u0 = static_cast<size_t>(un) * kQagUnitBytes;
        const size_t u1 = min(p.slot_bytes, u0 + kQagUnitBytes);
        const uint8_t *stage = p.heap_base[rank] + p.symm_off + static_cast<size_t>(s) * p.slot_bytes;
        for (size_t off = u0 + static_cast<size_t>(tid) * 16; off < u1; off += kQagThreads * 16) {
            size_t run;
            uint8_t *dst = src_ptr(ra, s, off, &run);
            if (run >= 16) *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(stage + off);
        }
    }
}

}  // namespace

size_t mxq_allgather_symmetric_bytes(int world, int m, int n) {
    if (world <= 1) return 0;
    const size_t sld = (static_cast<size_t>(n) / 32 + 1) / 2 * 2;
    const size_t slot = (static_cast<size_t>(m) * n + 1023) / 1024 * 1024 + (static_cast<size_t>(m) * sld + 1023) / 1024 * 1024;
    return static_cast<size_t>(world) * slot;
}

int launch_mx_quant_allgather(cudaStream_t stream, uint32_t block_num, const MxqAgArgs *args, void *symmetric, int m,
                              int n) {
    Team *t = team();
    if (!t) {
        set_error("symmetric heap not initialised (call catccos_shmem_init first)");
        return CATCCOS_ERR_NOT_INIT;
    }
    if (m <= 0 || n <= 0 || (n % 32) != 0) {
        set_error("MX quant + AllGather needs n a positive multiple of 32 (m=%d n=%d)", m, n);
        return CATCCOS_ERR_INVALID;
    }
    const int R = t->n_pes;
    const int n_local = t->emulated ? R : 1;
    const size_t sld = (static_cast<size_t>(n) / 32 + 1) / 2 * 2;
    const size_t codes_bytes = static_cast<size_t>(m) * n, scale_bytes = static_cast<size_t>(m) * sld;
    if (R > 1 && ((codes_bytes | scale_bytes) & 15)) {
        set_error("MX quant + AllGather over several ranks needs m*n and m*(n/32) to be multiples of 16");
        return CATCCOS_ERR_INVALID;
    }
    QagParams p;
    memset(&p, 0, sizeof(p));
    for (int l = 0; l < n_local; ++l) {
        const MxqAgArgs &a = args[l];
        if (!a.input || !a.codes || !a.scales || (reinterpret_cast<uintptr_t>(a.codes) & 15) ||
            (reinterpret_cast<uintptr_t>(a.scales) & 15)) {
            set_error("input, output and scale buffers must be non-null and 16-byte aligned");
            return CATCCOS_ERR_INVALID;
        }
        const int rank = t->emulated ? l : t->my_pe;
        int rc = mx_quant_launch(stream, a.input, m, n, a.codes + static_cast<size_t>(rank) * codes_bytes, n,
                                 a.scales + static_cast<size_t>(rank) * scale_bytes, static_cast<int>(sld), nullptr);
        if (rc) return rc;
        p.ranks[l].codes = a.codes;
        p.ranks[l].scales = a.scales;
    }
    if (R == 1) return CATCCOS_OK;
    const size_t need = mxq_allgather_symmetric_bytes(R, m, n);
    uint8_t *sp = static_cast<uint8_t *>(symmetric);
    uint8_t *hb = t->base[t->my_pe];
    if (sp == nullptr || sp < hb + kFlagBytes || sp + need > hb + t->heap_bytes || ((sp - hb) % 1024) != 0) {
        set_error("symmetric buffer %p (+%zu bytes) is not a 1024-aligned range of the symmetric heap", symmetric, need);
        return CATCCOS_ERR_INVALID;
    }
    p.symm_off = static_cast<uint64_t>(sp - hb);
    p.codes_bytes = codes_bytes;
    p.scale_bytes = scale_bytes;
    p.slot_bytes = need / R;
    const size_t units = (p.slot_bytes + kQagUnitBytes - 1) / kQagUnitBytes;
    if (kFlagOpBase + static_cast<size_t>(R) * units > kFlagWords) {
        set_error("shape needs more flags than the flag region holds");
        return CATCCOS_ERR_INVALID;
    }
    for (int pe = 0; pe < R; ++pe) p.heap_base[pe] = t->base[pe];
    p.world = R;
    p.rank_base = t->emulated ? 0 : t->my_pe;
    p.n_local = n_local;
    int per_rank = t->num_sms / n_local;
    if (block_num > 0 && static_cast<int>(block_num) < per_rank) per_rank = static_cast<int>(block_num);
    if (per_rank < 1) per_rank = 1;
    p.ctas_per_rank = per_rank;
    p.epoch = ++t->epoch;
    p.timeout_ns = t->timeout_ns;
    p.status = t->status_dev;
    const size_t smem = static_cast<size_t>(kQagLanes) * kPushPieceBytes;
    cudaError_t e = cudaFuncSetAttribute(mxq_allgather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) {
        if (n_local > 1) {
            void *kargs[] = {&p};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(mxq_allgather_kernel), dim3(per_rank * n_local),
                                            dim3(kQagThreads), kargs, smem, stream);
        } else {
            mxq_allgather_kernel<<<per_rank, kQagThreads, smem, stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("mxq_allgather_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

}  // namespace cb
