// Block-scaled MXFP8 GEMM (e4m3 data, UE8M0 scale per 32 along K) fused with the all-gather of
// the activation rows and their scale factors (sm_100a).
//
// Same organisation as the f16/bf16 kernel: warp 0 = TMA producer, warp 1 = tcgen05 issuer,
// warps 2-5 = epilogue, warp 6 = all-gather push.  Differences:
//   * tcgen05.mma.kind::mxf8f6f4.block_scale: K = 32 per instruction, BK = 128 per stage;
//   * scale factors travel as 512-byte "atoms" (128 rows x 4 k-blocks, the layout tcgen05.cp
//     expects), are bulk-copied next to the operand tiles and copied smem -> TMEM by the MMA
//     thread right before the four instructions that use them (tcgen05.cp and tcgen05.mma of one
//     thread execute in issue order, so one TMEM scale buffer is enough);
//   * TMEM holds ONE 128 x 256 fp32 accumulator plus 12 scale columns; the epilogue drains it into
//     registers as packed 16-bit values first and releases it before writing to memory.
#pragma once
#include <type_traits>

#include "common.h"
#include "ptx.cuh"

namespace cb {

constexpr int MX_BK = 128;                      // fp8 elements (= bytes) per stage along K
constexpr int kMxAStage = BM * MX_BK;           // 16 KiB
constexpr int kMxBStage = BN * MX_BK;           // 32 KiB
constexpr int kMxSfStage = 2048;                // A atom (512 B) + two B atoms (1024 B), padded
constexpr int kMxStageBytes = kMxAStage + kMxBStage + kMxSfStage;
constexpr int kMxStages = 4;
constexpr int kMxSideBytes = 24 * 1024;         // all-gather push staging: 3 lanes x 8 KiB
constexpr int kMxPushLanes = kMxSideBytes / kPushPieceBytes;
constexpr int kMxSmemBytes = kMxStages * kMxStageBytes + kMxSideBytes + 1024 + 512;
constexpr int kMxFlagsPerChunk = kAgSubChunks + 1;   // data units + one scale-factor unit

// Operand format of the one-CTA kernel.  MXFP4 (e2m1, two codes per byte, K-major operands only): a stage holds
// 128 bytes = 256 elements of K per row, i.e. two scale atoms per operand tile instead of one, and is consumed by
// four tcgen05.mma.kind::mxf4nvf4 (scale_vec::2X) of K = 64.
enum MxFormat : int { MX_FP8 = 0, MX_FP4 = 1 };
template <int FMT>
struct MxCfg {
    static constexpr int kAtoms = FMT == MX_FP4 ? 2 : 1;                 // scale atoms per operand tile and stage
    static constexpr int kSfStage = FMT == MX_FP4 ? 3072 : 2048;         // A atoms + 2 x B atoms
    static constexpr int kStageBytes = kMxAStage + kMxBStage + kSfStage;
    static constexpr int kSideBytes = FMT == MX_FP4 ? 16 * 1024 : kMxSideBytes;
    static constexpr int kPushLanes = kSideBytes / kPushPieceBytes;
    static constexpr int kSmemBytes = kMxStages * kStageBytes + kSideBytes + 1024 + 512;
    static constexpr int kSfCols = 12 * kAtoms;                          // TMEM columns of one stage's scales
    static_assert(kSmemBytes <= 232448, "shared memory budget");
    static_assert(kPushLanes <= kMxPushLanes, "push barriers");
};

struct alignas(64) MxRankArgs {
    CUtensorMap tmA;        // local activations  [m, K] bytes, box {128, BM}
    CUtensorMap tmAg;       // gathered activations [R*m, K] bytes in this PE's symmetric region
    CUtensorMap tmB;        // transB=1: [N, K] box {128, BN} (pair kernel: {128, 128});  transB=0: [K, N] box {128 (n), 128 (k)}
    CUtensorMap tmSfa;      // pair kernel: scale atoms as rows of 128 u32, box {128, 1}: local activations,
    CUtensorMap tmSfag;     //              gathered activations (symmetric region),
    CUtensorMap tmSfb;      //              weights
    const uint8_t *A;       // raw local activations (push source)
    const uint8_t *sfa;     // local scale atoms [ceil(m/128)][ceil(K/128)][512]
    const uint8_t *sfb;     // weight scale atoms [ceil(N/128)][ceil(K/128)][512]
    void *C;                // output [R*m, N] 16-bit
};

struct MxParams {
    MxRankArgs ranks[kMaxRanks];
    uint8_t *heap_base[kMaxRanks];
    uint64_t symm_off;        // gathered data region; the gathered scale atoms follow at sf_off
    uint64_t sf_off;          // byte offset (inside the heap) of the gathered scale atoms
    int world, rank_base, n_local, ctas_per_rank;
    int M, N, K;              // M = rows held by one rank
    int fp4;                  // pair kernel: 1 = MXFP4 operands (the one-CTA kernel takes the format as a template argument)
    uint32_t epoch;
    uint32_t entered_need;     // a peer's data region may be written once it has entered this epoch
    int compute_only;
    uint64_t timeout_ns;
    int *status;
    unsigned long long *trace;
};

struct MxSmem {
    uint64_t full[kMxStages];
    uint64_t empty[kMxStages];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint64_t drain;
    uint64_t push_bar[kMxPushLanes];
    uint32_t tmem_base;
    int abort_flag;
};

#define CB_MX_TRACE(slot, value)                                                             \
    do {                                                                                     \
        if (p.trace) p.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + (slot)] = (value); \
    } while (0)

template <typename TOut, bool B_MN, int FMT = MX_FP8>
__global__ void __launch_bounds__(kGemmThreads, 1) mx_allgather_gemm_kernel(const __grid_constant__ MxParams p) {
    using Cfg = MxCfg<FMT>;
    static_assert(!(FMT == MX_FP4 && B_MN), "4-bit operands are K-major");
    constexpr int kMxStageBytes = Cfg::kStageBytes;       // shadows the MXFP8 constants of the same names
    constexpr int kMxPushLanes = Cfg::kPushLanes;
    constexpr int kAtoms = Cfg::kAtoms;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_push = smem + kMxStages * kMxStageBytes;
    MxSmem *sh = reinterpret_cast<MxSmem *>(smem_push + Cfg::kSideBytes);
    static_assert(sizeof(MxSmem) <= 512, "barrier block outgrew its budget");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MxRankArgs &ra = p.ranks[lrank];
    const int mt = (p.M + BM - 1) / BM;            // row tiles (= all-gather chunks) per rank
    const int nt = (p.N + BN - 1) / BN;
    const int per_src = mt * nt;
    const int num_tiles = R * per_src;
    const int Kb = FMT == MX_FP4 ? p.K / 2 : p.K;  // bytes of one operand row
    const int kblocks = (Kb + MX_BK - 1) / MX_BK;   // pipeline stages per tile
    const int kb4 = (p.K + 127) / 128;              // scale atoms per row tile (one per 128 elements of K)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMxStages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 4);
        mbar_init(&sh->drain, 1);
        for (int l = 0; l < kMxPushLanes; ++l) mbar_init(&sh->push_bar[l], 1);
        sh->abort_flag = 0;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
        prefetch_tensormap(&ra.tmAg);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    // scale factors: 4 (A) + 8 (B) columns per K-step, four sets used in turn so that the copy for
    // one K-step does not have to wait for the MMAs of the step before it
    const uint32_t tmem_sf0 = tmem_base + BN;

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x == 0) CB_MX_TRACE(TR_START, globaltimer_ns());

    auto flagp = [&](int pe, uint32_t word) { return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + word; };

    // tile t -> (source rank s, row tile mi, column tile ni); own rows first, then rank+1, rank+2, ...
    auto decode = [&](int t, int &s, int &mi, int &ni, bool &gathered) {
        const int j = t / per_src;
        const int u = t - j * per_src;
        s = (rank + j) % R;
        mi = u / nt;
        ni = u - mi * nt;
        gathered = (j != 0);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = cta; t < num_tiles && ok; t += p.ctas_per_rank) {
                int s, mi, ni;
                bool gathered;
                decode(t, s, mi, ni, gathered);
                if (gathered && !p.compute_only) {
                    const uint32_t w = kFlagOpBase + (s * mt + mi) * kMxFlagsPerChunk;
                    for (int q = 0; q < kMxFlagsPerChunk && ok; ++q)
                        ok = wait_flag_ge(flagp(rank, w + q), p.epoch, ctl, W_MXAG, w + q);
                    if (!ok) break;
                    fence_proxy_async();
                }
                const CUtensorMap *tma = gathered ? &ra.tmAg : &ra.tmA;
                const int a_row = gathered ? s * p.M + mi * BM : mi * BM;
                const uint8_t *sfa = gathered ? p.heap_base[rank] + p.sf_off + (static_cast<size_t>(s) * mt + mi) * kb4 * 512
                                              : ra.sfa + static_cast<size_t>(mi) * kb4 * 512;
                const uint8_t *sfb = ra.sfb + static_cast<size_t>(ni) * 2 * kb4 * 512;   // two 128-column atom rows
                const bool second_b_atom = (ni * BN + 128) < p.N;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxStages;
                    const uint32_t ph = (it / kMxStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    uint8_t *sa = smem + st * kMxStageBytes;
                    uint8_t *sb = sa + kMxAStage;
                    uint8_t *ssf = sb + kMxBStage;
                    // scale atoms of this stage (the last stage of an MXFP4 tile may hold one instead of two)
                    const int atoms = min(kAtoms, kb4 - kb * kAtoms);
                    const uint32_t sfb_bytes = static_cast<uint32_t>(atoms) * 512;
                    mbar_expect_tx(&sh->full[st], kMxAStage + kMxBStage + sfb_bytes * (second_b_atom ? 3 : 2));
                    tma_load_2d(sa, tma, &sh->full[st], kb * MX_BK, a_row);
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(sb + j * (128 * MX_BK), &ra.tmB, &sh->full[st], ni * BN + j * 128, kb * MX_BK);
                    } else {
                        tma_load_2d(sb, &ra.tmB, &sh->full[st], kb * MX_BK, ni * BN);
                    }
                    bulk_load(ssf, sfa + static_cast<size_t>(kb) * kAtoms * 512, sfb_bytes, &sh->full[st]);
                    bulk_load(ssf + kAtoms * 512, sfb + static_cast<size_t>(kb) * kAtoms * 512, sfb_bytes, &sh->full[st]);
                    if (second_b_atom)
                        bulk_load(ssf + 2 * kAtoms * 512, sfb + (static_cast<size_t>(kb4) + kb * kAtoms) * 512, sfb_bytes,
                                  &sh->full[st]);
                }
            }
            if (!ok) {
                for (uint32_t back = 1; back <= kMxStages && back <= it; ++back) {
                    const uint32_t i2 = it - back;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(&sh->full[i2 % kMxStages], (i2 / kMxStages) & 1)) {
                        if (globaltimer_ns() - t0 > 2000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer ----
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int t = cta; t < num_tiles && ok; t += p.ctas_per_rank) {
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxStages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kMxStages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + st * kMxStageBytes);
                    const uint32_t b_addr = a_addr + kMxAStage;
                    const uint32_t sf_addr = b_addr + kMxBStage;
                    // scale atoms: 32 rows x 16 B, 8-row groups 128 B apart, no swizzle
                    const uint32_t tmem_sfa = tmem_sf0 + (it & 3u) * (FMT == MX_FP4 ? 24u : 16u);
                    if constexpr (FMT == MX_FP4) {
                        const uint32_t tmem_sfb = tmem_sfa + 4 * kAtoms;     // per atom: 4 columns (n 0-127) + 4 (n 128-255)
                        const int mmas = min(4, p.K / 64 - kb * 4);
                        const int atoms = (mmas + 1) / 2;
                        for (int a = 0; a < atoms; ++a) {
                            tmem_cp_32x128b_warpx4(tmem_sfa + a * 4, make_smem_desc_noswizzle(sf_addr + a * 512, 16, 128));
                            tmem_cp_32x128b_warpx4(tmem_sfb + a * 8,
                                                   make_smem_desc_noswizzle(sf_addr + kAtoms * 512 + a * 512, 16, 128));
                            tmem_cp_32x128b_warpx4(tmem_sfb + a * 8 + 4,
                                                   make_smem_desc_noswizzle(sf_addr + 2 * kAtoms * 512 + a * 512, 16, 128));
                        }
                        for (int k = 0; k < mmas; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);   // 64 e2m1 = 32 bytes of a row
                            const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t sf_id = static_cast<uint32_t>(k & 1) * 2u;
                            umma_fp4<false>(tmem_base, ad, bd, make_idesc_fp4(BM, BN, sf_id, sf_id, 1u), tmem_sfa + (k >> 1) * 4,
                                            tmem_sfb + (k >> 1) * 8, (kb | k) != 0);
                        }
                    } else {
                        const uint32_t tmem_sfb = tmem_sfa + 4;
                        tmem_cp_32x128b_warpx4(tmem_sfa, make_smem_desc_noswizzle(sf_addr, 16, 128));
                        tmem_cp_32x128b_warpx4(tmem_sfb, make_smem_desc_noswizzle(sf_addr + 512, 16, 128));
                        tmem_cp_32x128b_warpx4(tmem_sfb + 4, make_smem_desc_noswizzle(sf_addr + 1024, 16, 128));
#pragma unroll
                        for (int k = 0; k < MX_BK / 32; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                            // B MN-major (8-bit): 128-column chunks 128*MX_BK B apart, 8-row (K) groups 1024 B
                            // apart, 32 K-rows = 4096 B
                            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 4096, 128 * MX_BK, 1024)
                                                     : make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t idesc = make_idesc_mxf8(BM, BN, k, k) | (B_MN ? (1u << 16) : 0u);
                            umma_mxf8(tmem_base, ad, bd, idesc, tmem_sfa, tmem_sfb, (kb | k) != 0);
                        }
                    }
                    umma_commit(&sh->empty[st]);
                }
                if (!ok) break;
                umma_commit(&sh->tmem_full);
                ++tcount;
            }
            CB_MX_TRACE(TR_TILES, tcount);
            if (!ok) {
                umma_commit(&sh->drain);
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(&sh->drain, 0)) {
                    if (globaltimer_ns() - t0 > 2000000ull) break;
                }
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue ----
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        bool ok = true;
        TOut *const C = reinterpret_cast<TOut *>(ra.C);
        for (int t = cta; t < num_tiles && ok; t += p.ctas_per_rank) {
            int s, mi, ni;
            bool gathered;
            decode(t, s, mi, ni, gathered);
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            // drain the whole accumulator row into registers as packed 16-bit pairs, then free TMEM
            uint32_t pk[BN / 2];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[c * 16 + i] = Pack2<TOut>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty);
            const int row = s * p.M + mi * BM + row_in_tile;
            if (row < (s + 1) * p.M) {
                TOut *dst = C + static_cast<size_t>(row) * p.N + ni * BN;
#pragma unroll
                for (int g = 0; g < BN / 8; ++g)
                    if (ni * BN + g * 8 < p.N)
                        *reinterpret_cast<uint4 *>(dst + g * 8) =
                            make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
            }
            ++tcount;
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------------ push ----
        const int ctid = lane;
        if (R > 1 && !p.compute_only) {
            if (cta == 0 && ctid < R && ctid != rank) {
                fence_sys();
                st_release_sys(flagp(ctid, kFlagEntered + rank), p.epoch);
            }
            if (ctid < kMxPushLanes) {
                // units per destination: for every chunk (128 rows) kAgSubChunks data units of BM/kAgSubChunks rows and
                // one unit with the chunk's scale atoms; destination rank-1 first
                const int units_per_dest = mt * kMxFlagsPerChunk;
                const int total = (R - 1) * units_per_dest;
                const size_t row_bytes = static_cast<size_t>(Kb);
                const int lane_id = cta * kMxPushLanes + ctid;
                const int n_lanes = p.ctas_per_rank * kMxPushLanes;
                uint8_t *buf = smem_push + ctid * kPushPieceBytes;
                uint64_t *bar = &sh->push_bar[ctid];
                bool ok = true;
                uint32_t entered_ok = 0;
                uint32_t piece = 0;
                for (int u = lane_id; u < total && ok; u += n_lanes) {
                    const int jj = u / units_per_dest;
                    const int d = (rank + R - 1 - jj) % R;
                    const int cu = u - jj * units_per_dest;
                    const int chunk = cu / kMxFlagsPerChunk, sub = cu % kMxFlagsPerChunk;
                    const uint8_t *src;
                    uint8_t *dst;
                    size_t bytes;
                    if (sub < kAgSubChunks) {
                        const int r0 = chunk * BM + sub * (BM / kAgSubChunks);
                        const int r1 = min(p.M, r0 + BM / kAgSubChunks);
                        bytes = r1 > r0 ? (r1 - r0) * row_bytes : 0;
                        src = ra.A + r0 * row_bytes;
                        dst = p.heap_base[d] + p.symm_off + (static_cast<size_t>(rank) * p.M + r0) * row_bytes;
                    } else {
                        bytes = static_cast<size_t>(kb4) * 512;
                        src = ra.sfa + static_cast<size_t>(chunk) * kb4 * 512;
                        dst = p.heap_base[d] + p.sf_off + (static_cast<size_t>(rank) * mt + chunk) * kb4 * 512;
                    }
                    if (!((entered_ok >> d) & 1)) {
                        if (!(ok = wait_flag_ge(flagp(rank, kFlagEntered + d), p.entered_need, ctl, W_ENTERED, d))) break;
                        entered_ok |= 1u << d;
                    }
                    for (size_t off = 0; off < bytes && ok; off += kPushPieceBytes, ++piece) {
                        const uint32_t len = static_cast<uint32_t>(min(static_cast<size_t>(kPushPieceBytes), bytes - off));
                        bulk_wait_read<0>();
                        mbar_expect_tx(bar, len);
                        bulk_load(buf, src + off, len, bar);
                        if (!(ok = mbar_wait(bar, piece & 1, ctl, W_DRAIN))) break;
                        bulk_store(dst + off, buf, len);
                        bulk_commit();
                    }
                    if (!ok) break;
                    bulk_wait<0>();
                    fence_proxy_async();
                    fence_sys();
                    st_release_sys(flagp(d, kFlagOpBase + (rank * mt + chunk) * kMxFlagsPerChunk + sub), p.epoch);
                }
                bulk_wait<0>();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0) CB_MX_TRACE(TR_END, globaltimer_ns());
}

}  // namespace cb
