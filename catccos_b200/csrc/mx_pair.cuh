// MXFP8 AllGather-Matmul on CTA pairs (tcgen05 cta_group::2 block-scaled MMA), sm_100a.
//
// A pair computes a 256 x 256 tile.  Each CTA loads its 128 rows of A with their scale atom, its
// 128 columns of B, and BOTH scale atoms of the 256 B columns (each CTA's accumulator spans all
// 256 columns, so it needs all of B's scales in its own TMEM).  Scale atoms are fetched with TMA
// through a [atoms][128 x u32] tensor map so that, like the operand tiles, they can complete on
// the leader CTA's barrier.  The leader issues tcgen05.cp.cta_group::2 (each CTA copies from its
// own shared memory to its own TMEM) and one M=256 MMA per 32 K-elements.  34.5 KiB per K-step
// per SM instead of 49.5 KiB, six stages instead of four.
#pragma once
#include "mx_gemm.cuh"
#include "sched.h"

namespace cb {

constexpr int kMxPStages = 6;
constexpr int kMxPA = BM * MX_BK;               // 16 KiB
constexpr int kMxPB = 128 * MX_BK;              // 16 KiB
constexpr int kMxPairThreads = 480;             // warps 0-10 as the f16/bf16 pair kernel, warps 11-14 feed the scale factors
constexpr int kMxPSf = 1536;                    // kernels that still stage scale atoms in shared memory: A atom + two B atoms
constexpr int kMxSfCols = 24;                   // TMEM columns of one stage's scales: MXFP8 4 (A) + 8 (B); MXFP4 twice that
constexpr int kMxPairSmemBytes = kMxPStages * (kMxPA + kMxPB) + kMxSideBytes + 1024 + 512;
static_assert(kMxPairSmemBytes <= 232448, "shared memory budget");

struct MxPairSmem {
    uint64_t full[kMxPStages];      // in the leader: both CTAs' loads landed (2 arrivals + bytes)
    uint64_t empty[kMxPStages];     // per CTA
    uint64_t tmem_full;             // per CTA
    uint64_t tmem_empty;            // in the leader: 8 epilogue warps of the pair
    uint64_t drain;
    uint64_t push_bar[kMxPushLanes];
    uint32_t tmem_base;
    int abort_flag;
    uint32_t tiles_ready;           // tiles of this CTA (in its own order) whose gathered rows and scales are in
};

template <typename TOut, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMxPairThreads, 1)
    mx_pair_agmm_kernel(const __grid_constant__ MxParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kMxPStages * kMxPA;
    uint8_t *smem_push = smem_b + kMxPStages * kMxPB;
    MxPairSmem *sh = reinterpret_cast<MxPairSmem *>(smem_push + kMxSideBytes);
    static_assert(sizeof(MxPairSmem) <= 512, "barrier block outgrew its budget");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int pair = cta >> 1, pairs = p.ctas_per_rank >> 1;
    const uint32_t cr = cluster_ctarank();
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MxRankArgs &ra = p.ranks[lrank];
    const int mt = (p.M + BM - 1) / BM;             // 128-row chunks (push units, scale atom rows) per rank
    const int mt2 = (p.M + 2 * BM - 1) / (2 * BM);  // 256-row tiles per rank
    const int nt = (p.N + BN - 1) / BN;
    const int per_src = mt2 * nt;
    const int num_tiles = R * per_src;
    const bool fp4 = !B_MN && p.fp4 != 0;          // MXFP4: two codes per byte, K-major operands only
    const int Kb = fp4 ? p.K / 2 : p.K;           // bytes of one operand row
    const int kblocks = (Kb + MX_BK - 1) / MX_BK;  // pipeline stages per tile
    const int kb4 = (p.K + 127) / 128;             // scale atoms per row tile (one per 128 elements of K)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMxPStages; ++s) {
            mbar_init(&sh->full[s], 2 + 8);      // two producers (with their bytes) + the pair's eight scale-factor warps
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 8);
        mbar_init(&sh->drain, 1);
        for (int l = 0; l < kMxPushLanes; ++l) mbar_init(&sh->push_bar[l], 1);
        sh->abort_flag = 0;
        sh->tiles_ready = 0;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
        prefetch_tensormap(&ra.tmAg);
    }
    if (warp == 1) {
        tmem_alloc_pair(&sh->tmem_base, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    // scale factors: 4 (A) + 8 (B) TMEM columns per pipeline stage, written by warps 11-14 straight from
    // global memory (tcgen05.st), so that nothing but MMAs sits in the tensor pipe's queue
    const uint32_t tmem_sf0 = tmem_base + BN;

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x == 0) CB_MX_TRACE(TR_START, globaltimer_ns());
    auto flagp = [&](int pe, uint32_t word) { return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + word; };
    auto decode = [&](int t, int &s, int &mi2, int &ni, bool &gathered) {
        ag_order_decode(R, per_src, nt, rank, t, s, mi2, ni);
        gathered = (s != rank);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        // lane 0 issues the loads; the arrival flags of gathered rows are polled ahead of it by warp 10
        uint32_t it = 0, seq = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += pairs, ++seq) {
            int s, mi2, ni;
            bool gathered;
            decode(t, s, mi2, ni, gathered);
            const int chunk = mi2 * 2 + static_cast<int>(cr);       // this CTA's 128-row chunk of the source rank
            const bool have_rows = chunk < mt;
            if (gathered && !p.compute_only && have_rows && lane == 0) {
                ok = wait_smem_counter_gt(&sh->tiles_ready, seq, ctl, W_MXAG);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0) {
                const CUtensorMap *tma = gathered ? &ra.tmAg : &ra.tmA;
                const int a_row = (gathered ? s * p.M : 0) + chunk * BM;
                const int n_half = ni * BN + static_cast<int>(cr) * 128;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxPStages;
                    const uint32_t ph = (it / kMxPStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    mbar_expect_tx_cluster(full_leader, kMxPA + kMxPB);
                    tma_load_2d_pair(smem_a + st * kMxPA, tma, full_leader, kb * MX_BK, a_row);
                    if (B_MN)
                        tma_load_2d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, n_half, kb * MX_BK);
                    else
                        tma_load_2d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, kb * MX_BK, n_half);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
        }
        if (!ok && lane == 0) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 20000ull) {
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------- MMA issuer (leader CTA only) ----
        if (lane == 0 && cr == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            uint64_t wait_tmem = 0, wait_smem = 0;
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                const uint64_t tm0 = p.trace ? globaltimer_ns() : 0;
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                if (p.trace) wait_tmem += globaltimer_ns() - tm0;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxPStages;
                    const uint64_t ts0 = p.trace ? globaltimer_ns() : 0;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kMxPStages) & 1, ctl, W_MBAR_FULL))) break;
                    if (p.trace) wait_smem += globaltimer_ns() - ts0;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + st * kMxPA);
                    const uint32_t b_addr = smem_u32(smem_b + st * kMxPB);
                    const uint32_t tmem_sfa = tmem_sf0 + static_cast<uint32_t>(st) * kMxSfCols;   // written by warps 11-14
                    if (fp4) {
                        // four MMAs of K = 64 (fewer in a ragged last stage); atom a = k / 2: A at +4a, B at +8 + 8a
                        const int mmas = min(4, p.K / 64 - kb * 4);
                        for (int k = 0; k < mmas; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                            const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t sf_id = static_cast<uint32_t>(k & 1) * 2u;
                            umma_mxfp4_pair(tmem_base, ad, bd, make_idesc_fp4(2 * BM, BN, sf_id, sf_id, 1u), tmem_sfa + (k >> 1) * 4,
                                            tmem_sfa + 8 + (k >> 1) * 8, (kb | k) != 0);
                        }
                    } else {
                        const uint32_t tmem_sfb = tmem_sfa + 4;
#pragma unroll
                        for (int k = 0; k < MX_BK / 32; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 4096, 128 * MX_BK, 1024)
                                                     : make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t idesc = make_idesc_mxf8(2 * BM, BN, k, k) | (B_MN ? (1u << 16) : 0u);
                            umma_mxf8_pair(tmem_base, ad, bd, idesc, tmem_sfa, tmem_sfb, (kb | k) != 0);
                        }
                    }
                    umma_commit_pair(mapa_cluster(smem_u32(&sh->empty[st]), 0));
                    umma_commit_pair(mapa_cluster(smem_u32(&sh->empty[st]), 1));
                }
                if (!ok) break;
                umma_commit_pair(mapa_cluster(smem_u32(&sh->tmem_full), 0));
                umma_commit_pair(mapa_cluster(smem_u32(&sh->tmem_full), 1));
                ++tcount;
            }
            CB_MX_TRACE(TR_MMA_WAIT_TMEM_NS, wait_tmem);
            CB_MX_TRACE(TR_MMA_WAIT_SMEM_NS, wait_smem);
            CB_MX_TRACE(TR_TILES, tcount);
            if (!ok) {
                umma_commit_pair(mapa_cluster(smem_u32(&sh->drain), 0));
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
        for (int t = pair; t < num_tiles && ok; t += pairs) {
            int s, mi2, ni;
            bool gathered;
            decode(t, s, mi2, ni, gathered);
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            // two halves of 128 columns: the first half's stores are issued before the second half is read, and
            // the accumulator goes back to the MMA thread right after the last TMEM read
            const int row = s * p.M + mi2 * 2 * BM + static_cast<int>(cr) * BM + row_in_tile;
            const bool row_ok = row < (s + 1) * p.M;
            TOut *dst = C + static_cast<size_t>(row) * p.N + ni * BN;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t pk[BN / 4];
#pragma unroll
                for (int c = 0; c < BN / 64; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + (h * 4 + c) * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[c * 16 + i] = Pack2<TOut>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                }
                if (h == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty), 0));
                }
                if (row_ok) {
#pragma unroll
                    for (int g = 0; g < BN / 16; ++g)
                        if (ni * BN + h * 128 + g * 8 < p.N)
                            *reinterpret_cast<uint4 *>(dst + h * 128 + g * 8) =
                                make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                }
            }
            ++tcount;
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------ flag scout ----
        // walks this CTA's tiles ahead of the producer and waits (whole warp, one lane per unit) for
        // the rows and scales of every gathered chunk; the count of cleared tiles goes to shared memory
        if (R > 1 && !p.compute_only) {
            uint32_t seq = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += pairs, ++seq) {
                int s, mi2, ni;
                bool gathered;
                decode(t, s, mi2, ni, gathered);
                const int chunk = mi2 * 2 + static_cast<int>(cr);
                if (gathered && chunk < mt) {
                    const uint32_t w = kFlagOpBase + (s * mt + chunk) * kMxFlagsPerChunk;
                    if (!(ok = wait_flags_warp(flagp(rank, w), kMxFlagsPerChunk, p.epoch, ctl, W_MXAG, w))) break;
                    fence_proxy_async_global();     // rows seen through the flags -> the producer's TMA loads
                }
                if (lane == 0) st_release_cta_smem(&sh->tiles_ready, seq + 1);
            }
        }
    } else if (warp >= 11) {
        // ---------------------------------------------------------- scale factors ----
        // Warp 11 + j owns TMEM lane quarter (11 + j) % 4.  Per pipeline stage every lane reads its 16-byte
        // row of the A atom and of the two B atoms from global memory (the atoms are 512 contiguous bytes:
        // one coalesced request per warp, the other three warps hit L1) and stores them into the stage's
        // scale columns; the stage's "full" barrier in the leader counts these eight warps next to the loads.
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        uint32_t it = 0, seq = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += pairs, ++seq) {
            int s, mi2, ni;
            bool gathered;
            decode(t, s, mi2, ni, gathered);
            const int chunk = mi2 * 2 + static_cast<int>(cr);
            const bool have_rows = chunk < mt;
            if (gathered && !p.compute_only && have_rows) {
                if (lane == 0) ok = wait_smem_counter_gt(&sh->tiles_ready, seq, ctl, W_MXAG);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            // a chunk past the rank's rows has no scale atoms of its own: reuse the last chunk's (rows are masked)
            const uint8_t *sfa_base = gathered ? p.heap_base[rank] + p.sf_off : ra.sfa;
            const uint8_t *sfa = sfa_base + (static_cast<size_t>((gathered ? s * mt : 0) + (have_rows ? chunk : mt - 1)) * kb4) * 512 + lane * 16;
            const uint8_t *sfb0 = ra.sfb + static_cast<size_t>(ni * 2) * kb4 * 512 + lane * 16;
            const bool second_b_atom = (ni * BN + 128) < p.N;
            const uint8_t *sfb1 = second_b_atom ? sfb0 + static_cast<size_t>(kb4) * 512 : sfb0;
            if (fp4) {
                // MXFP4: two atoms per operand tile and stage (one in a ragged last stage: the second index is clamped)
                uint4 cur[6], nxt[6];
                auto load6 = [&](uint4 (&v)[6], int kb) {
                    const size_t o0 = static_cast<size_t>(min(2 * kb, kb4 - 1)) * 512, o1 = static_cast<size_t>(min(2 * kb + 1, kb4 - 1)) * 512;
                    v[0] = *reinterpret_cast<const uint4 *>(sfa + o0);
                    v[1] = *reinterpret_cast<const uint4 *>(sfa + o1);
                    v[2] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + o0));
                    v[3] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + o0));
                    v[4] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + o1));
                    v[5] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + o1));
                };
                load6(nxt, 0);
                for (int kb = 0; kb < kblocks && ok; ++kb) {
#pragma unroll
                    for (int j = 0; j < 6; ++j) cur[j] = nxt[j];
                    load6(nxt, kb + 1 < kblocks ? kb + 1 : kb);
                    const int st = it % kMxPStages;
                    const uint32_t ph = (it / kMxPStages) & 1;
                    ++it;
                    if (lane == 0) ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t col = tmem_sf0 + static_cast<uint32_t>(st) * kMxSfCols + lane_field;
                    tmem_st_32x4(col, cur[0]);
                    tmem_st_32x4(col + 4, cur[1]);
                    tmem_st_32x4(col + 8, cur[2]);
                    tmem_st_32x4(col + 12, cur[3]);
                    tmem_st_32x4(col + 16, cur[4]);
                    tmem_st_32x4(col + 20, cur[5]);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->full[st]), 0));
                }
                continue;
            }
            // the atoms of the next kSfAhead K-steps are kept in flight (an L2 round trip is longer than a K-step)
            constexpr int kSfAhead = 4;
            uint4 va[kSfAhead], vb0[kSfAhead], vb1[kSfAhead];
#pragma unroll
            for (int d = 0; d < kSfAhead; ++d) {
                const int kk = d < kblocks ? d : kblocks - 1;
                va[d] = __ldg(reinterpret_cast<const uint4 *>(sfa + static_cast<size_t>(kk) * 512));
                vb0[d] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + static_cast<size_t>(kk) * 512));
                vb1[d] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + static_cast<size_t>(kk) * 512));
            }
            for (int kb0 = 0; kb0 < kblocks && ok; kb0 += kSfAhead) {
#pragma unroll
                for (int d = 0; d < kSfAhead; ++d) {
                    const int kb = kb0 + d;
                    if (kb >= kblocks) break;
                    const int st = it % kMxPStages;
                    const uint32_t ph = (it / kMxPStages) & 1;
                    ++it;
                    const uint4 a = va[d], b0 = vb0[d], b1 = vb1[d];
                    {
                        const int kk = kb + kSfAhead < kblocks ? kb + kSfAhead : kblocks - 1;
                        va[d] = __ldg(reinterpret_cast<const uint4 *>(sfa + static_cast<size_t>(kk) * 512));
                        vb0[d] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + static_cast<size_t>(kk) * 512));
                        vb1[d] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + static_cast<size_t>(kk) * 512));
                    }
                    // the MMAs that read this stage's scale columns one round ago have finished
                    if (lane == 0) ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t col = tmem_sf0 + static_cast<uint32_t>(st) * kMxSfCols + lane_field;
                    tmem_st_32x4(col, a);
                    tmem_st_32x4(col + 4, b0);
                    tmem_st_32x4(col + 8, b1);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->full[st]), 0));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ push ----
        // warps 6..9: one push lane per warp
        const int ctid = warp - 6;
        if (R > 1 && !p.compute_only) {
            if (warp == 6 && cta == 0 && lane < R && lane != rank) {
                fence_sys();
                st_release_sys(flagp(lane, kFlagEntered + rank), p.epoch);
            }
            __syncwarp();
            if (lane == 0 && ctid < kMxPushLanes) {
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
                    int d, cu;
                    ag_push_decode(R, units_per_dest, rank, u, d, cu);
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
                    fence_proxy_async_global();
                    fence_sys();
                    st_release_sys(flagp(d, kFlagOpBase + (rank * mt + chunk) * kMxFlagsPerChunk + sub), p.epoch);
                }
                bulk_wait<0>();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0) CB_MX_TRACE(TR_END, globaltimer_ns());
}

}  // namespace cb
