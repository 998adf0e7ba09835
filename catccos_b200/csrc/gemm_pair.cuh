// AllGather-Matmul f16/bf16 with CTA pairs (tcgen05 cta_group::2), sm_100a.
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile: each CTA loads its own
// 128 rows of A and its own 128 columns of B (no multicast) and holds the accumulator of its 128
// rows in its own TMEM; the leader CTA issues one M=256 MMA per 16 K-elements that reads both
// CTAs' shared memory.  Per SM and K-step this moves 32 KiB from L2 instead of the 48 KiB of the
// one-CTA 128 x 256 tile, which is what limits that kernel, and leaves room for 6 pipeline stages.
// The all-gather push lanes, flags and bounded waits are the one-CTA kernel's.  Tiles are handed out
// dynamically: every pair starts on tile `pair` and then takes the next unclaimed tile of its rank from
// a global counter, so a pair that had to wait for a peer's rows simply ends up with fewer tiles
// instead of finishing late; the tile sequence itself is the L2-grouped order of sched.h.
#pragma once
#include <type_traits>

#include "common.h"
#include "gemm_fused.cuh"
#include "ptx.cuh"
#include "sched.h"
#include "tile_queue.cuh"

namespace cb {

constexpr int kPStages = 6;
constexpr int kPStagesSolo = 7;     // AllGather-Matmul of a single rank: no copy lanes, their staging is a seventh stage
constexpr int kPAStage = BM * BK * 2;          // 128 rows of A      : 16 KiB
constexpr int kPBStage = 128 * BK * 2;         // 128 columns of B   : 16 KiB
constexpr int kPairSmemBytes = kPStages * (kPAStage + kPBStage) + kSideSmemBytes + 1024 + 512;
constexpr int kPairSoloSmemBytes = kPStagesSolo * (kPAStage + kPBStage) + 1024 + 512;
static_assert(kPairSoloSmemBytes <= 232448, "shared memory budget");
constexpr int BM2 = 2 * BM;                    // rows of a pair's tile

struct PairSmem {
    uint64_t full[kPStagesSolo];    // used in the leader: both CTAs' loads of a stage have landed
    uint64_t empty[kPStagesSolo];   // per CTA: the pair's MMAs have finished reading this stage
    uint64_t tmem_full[2];          // per CTA: accumulator complete
    uint64_t tmem_empty[2];         // used in the leader: both CTAs' epilogues have drained the accumulator
    uint64_t drain;
    uint64_t push_bar[kPushLanesShared];
    uint32_t tmem_base;
    int abort_flag;
    uint32_t tiles_ready;           // tiles of this CTA (in claim order) whose gathered rows are known to be in
    TileQueue tq;                   // claimed tiles (written by the leader's warp 10)
};

template <typename T, bool B_MN, int STAGES = kPStages>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairAgThreads, 1)
    pair_agmm_kernel(const __grid_constant__ FusedParams p) {
    static_assert(STAGES == kPStages || STAGES == kPStagesSolo, "pipeline depth");
    constexpr int kPStages = STAGES;                 // shadows the default depth inside this kernel
    constexpr bool kHasSide = STAGES == cb::kPStages;   // the seven-stage form has no copy lanes (world size 1, no gather result)
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + kPStages * kPAStage;
    uint8_t *smem_push = smem + kPStages * (kPAStage + kPBStage);
    PairSmem *sh = reinterpret_cast<PairSmem *>(smem_push + (kHasSide ? kSideSmemBytes : 0));
    static_assert(sizeof(PairSmem) <= 512, "barrier block outgrew its budget");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;      // ctas_per_rank is even
    const int pair = cta >> 1;
    const int pairs = p.ctas_per_rank >> 1;
    const uint32_t cr = cluster_ctarank();                      // 0 = leader
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const RankArgs &ra = p.ranks[lrank];
    const int mt2 = ceil_div(p.M, BM2);
    const int nt = ceil_div(p.N, BN);
    const int per_src = mt2 * nt;
    const int num_tiles = R * per_src;
    const int kblocks = ceil_div(p.K, BK);
    const int mt_ag = ceil_div(p.M, BM);                        // 128-row push chunks per source rank

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(&sh->full[s], 2);
            mbar_init(&sh->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh->tmem_full[a], 1);
            mbar_init(&sh->tmem_empty[a], 8);
        }
        mbar_init(&sh->drain, 1);
        for (int l = 0; l < kPushLanesShared; ++l) mbar_init(&sh->push_bar[l], 1);
        sh->abort_flag = 0;
        sh->tiles_ready = 0;
        tq_init(&sh->tq);
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
    cluster_sync();                 // the peer's barriers are initialised before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x == 0) CB_TRACE(TR_START, globaltimer_ns());

    // tile t -> (source rank s, 256-row tile mi2, column tile ni): own rows first, then rank+1, ..., in L2 groups
    auto decode = [&](int t, int &s, int &mi2, int &ni, bool &gathered) {
        ag_order_grouped(R, mt2, nt, p.ag_group, rank, t, s, mi2, ni);
        gathered = (s != rank);
    };
    // claim number seq -> tile index, once the leader's warp 10 has published it (kTileEnd: no more tiles)
    auto claimed_tile = [&](uint32_t seq, uint32_t &t) -> bool { return tq_get(&sh->tq, seq, t, ctl); };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        // lane 0 issues the loads; the arrival flags of gathered rows are polled ahead of it by warp 10
        uint32_t it = 0;
        bool ok = true;
        uint64_t prod_wait_ns = 0;
        if (lane == 0) {
            for (uint32_t seq = 0; ok; ++seq) {
                uint32_t tq;
                if (!(ok = claimed_tile(seq, tq)) || tq == kTileEnd) break;
                int s, mi2, ni;
                bool gathered;
                decode(static_cast<int>(tq), s, mi2, ni, gathered);
                const int row_in_src = mi2 * BM2 + static_cast<int>(cr) * BM;    // this CTA's 128 rows
                if (gathered && !p.compute_only && row_in_src < p.M) {
                    const uint64_t tw0 = p.trace ? globaltimer_ns() : 0;
                    if (!(ok = wait_smem_counter_gt(&sh->tiles_ready, seq, ctl, W_AG_CHUNK))) break;
                    if (p.trace) {
                        if (prod_wait_ns == 0) CB_TRACE(TR_PROD_WAIT_FIRST, tw0);
                        prod_wait_ns += globaltimer_ns() - tw0 + 1;
                    }
                }
                const CUtensorMap *tma = gathered ? &ra.tmAg : &ra.tmA;
                const int a_row = (gathered ? s * p.M : (p.ag_a2a ? rank * p.M : 0)) + row_in_src;
                const int n_half = ni * BN + static_cast<int>(cr) * 128;         // this CTA's 128 columns of B
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kPStages;
                    const uint32_t ph = (it / kPStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    mbar_expect_tx_cluster(full_leader, kPAStage + kPBStage);
                    tma_load_2d_pair(smem_a + st * kPAStage, tma, full_leader, kb * BK, a_row);
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            tma_load_2d_pair(smem_b + st * kPBStage + j * (64 * BK * 2), &ra.tmB, full_leader,
                                             n_half + j * 64, kb * BK);
                    } else {
                        tma_load_2d_pair(smem_b + st * kPBStage, &ra.tmB, full_leader, kb * BK, n_half);
                    }
                }
            }
        }
        if (lane == 0) CB_TRACE(TR_PROD_WAIT_NS, prod_wait_ns);
        if (!ok && lane == 0) {
            // loads already issued still land in shared memory; give them time (bounded)
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 20000ull) {
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------- MMA issuer (leader CTA only) ----
        if (lane == 0 && cr == 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc = make_idesc_f16(fmt, BM2, BN, 0, B_MN ? 1 : 0);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            uint64_t wait_tmem = 0, wait_smem = 0;
            for (;;) {
                uint32_t tq;
                if (!(ok = claimed_tile(tcount, tq)) || tq == kTileEnd) break;
                const uint32_t acc = tcount & 1;
                const uint64_t tm0 = p.trace ? globaltimer_ns() : 0;
                if (!(ok = mbar_wait(&sh->tmem_empty[acc], ((tcount >> 1) & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                if (p.trace) wait_tmem += globaltimer_ns() - tm0;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kPStages;
                    const uint64_t ts0 = p.trace ? globaltimer_ns() : 0;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kPStages) & 1, ctl, W_MBAR_FULL))) break;
                    if (p.trace) wait_smem += globaltimer_ns() - ts0;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + st * kPAStage);
                    const uint32_t b_addr = smem_u32(smem_b + st * kPBStage);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 2048, 64 * BK * 2, 1024)
                                                 : make_smem_desc(b_addr + k * 32, 16, 1024);
                        umma_f16_pair(d_tmem, ad, bd, idesc, (kb | k) != 0);
                    }
                    // the stage is free in both CTAs once these MMAs have read it
                    umma_commit_pair(mapa_cluster(smem_u32(&sh->empty[st]), 0));
                    umma_commit_pair(mapa_cluster(smem_u32(&sh->empty[st]), 1));
                }
                if (!ok) break;
                umma_commit_pair(mapa_cluster(smem_u32(&sh->tmem_full[acc]), 0));
                umma_commit_pair(mapa_cluster(smem_u32(&sh->tmem_full[acc]), 1));
                ++tcount;
            }
            CB_TRACE(TR_MMA_WAIT_TMEM_NS, wait_tmem);
            CB_TRACE(TR_MMA_WAIT_SMEM_NS, wait_smem);
            CB_TRACE(TR_TILES, tcount);
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
        T *const C = reinterpret_cast<T *>(ra.C);
        for (;;) {
            uint32_t tq;
            if (!(ok = claimed_tile(tcount, tq)) || tq == kTileEnd) break;
            int s, mi2, ni;
            bool gathered;
            decode(static_cast<int>(tq), s, mi2, ni, gathered);
            const uint32_t acc = tcount & 1;
            if (!(ok = mbar_wait(&sh->tmem_full[acc], (tcount >> 1) & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const int row = s * p.M + mi2 * BM2 + static_cast<int>(cr) * BM + row_in_tile;
            const bool row_ok = row < (s + 1) * p.M;
            T *dst_row = C + static_cast<size_t>(row) * p.N;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                tmem_ld_wait();
                const int col = ni * BN + c * 32;
                if (!row_ok || col >= p.N) continue;
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[i] = Pack2<T>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    if (col + g * 8 < p.N)
                        *reinterpret_cast<uint4 *>(dst_row + col + g * 8) =
                            make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
            }
            // accumulator drained: tell the leader's MMA thread (8 warps of the pair arrive)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty[acc]), 0));
            ++tcount;
            // progress of this CTA's epilogue, which paces the claiming of further tiles
            if (warp == 2 && lane == 0) tq_done(&sh->tq, cr, tcount);
        }
    } else if (warp == 10) {
        // ------------------------------------------------- tile queue and flag scout ----
        // Leader: claims the pair's next tile (the first one is tile `pair`, the others come from the
        // rank's counter), publishes it to both CTAs, at most kTileAhead tiles beyond the epilogues.
        // Both CTAs: wait (whole warp, one lane per unit) for the rows of a gathered tile's chunk and
        // publish the count of cleared tiles to the producer.
        bool ok = true;
        int *const next_tile = p.sched + 2 * lrank;
        for (uint32_t seq = 0; ok; ++seq) {
            uint32_t tq = 0;
            if (cr == 0) {
                if (lane == 0) ok = tq_claim(&sh->tq, seq, pair, pairs, num_tiles, next_tile, ctl, tq);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                tq = __shfl_sync(0xffffffffu, tq, 0);
                if (!ok) break;
            } else {
                if (lane == 0) ok = claimed_tile(seq, tq);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                tq = __shfl_sync(0xffffffffu, tq, 0);
                if (!ok) break;
            }
            if (tq == kTileEnd) break;
            if (R > 1 && !p.compute_only) {
                int s, mi2, ni;
                bool gathered;
                decode(static_cast<int>(tq), s, mi2, ni, gathered);
                const int row_in_src = mi2 * BM2 + static_cast<int>(cr) * BM;
                if (gathered && row_in_src < p.M) {
                    const uint32_t w = kFlagOpBase + (s * mt_ag + (row_in_src / BM)) * kAgSubChunks;
                    if (!(ok = wait_flags_warp(flag_ptr(p, rank, w), kAgSubChunks, p.epoch, ctl, W_AG_CHUNK, w))) break;
                    fence_proxy_async_global();     // rows seen through the flags -> the producer's TMA loads
                }
                if (lane == 0) st_release_cta_smem(&sh->tiles_ready, seq + 1);
            }
        }
        // the last pair of the rank to run out of tiles leaves the counters at zero for the next launch
        if (cr == 0 && lane == 0) {
            if (!ok) tq_publish_end(&sh->tq);      // this pair gave up: nobody waits for claims that will not come
            tq_retire(next_tile, pairs);
        }
    } else {
        // ------------------------------------------------- all-gather data movement ----
        // warps 6..9: one copy lane per warp.  Default: this rank's rows are pushed into every peer's gathered
        // region.  Remote read (p.ag_pull): this rank stages its rows in its own region, tells the peers, and
        // fetches the peers' staged rows into its own region.  Either way a unit's arrival flag in this rank's
        // flag region tells the scout that the rows are in local memory.  With a gather-result output the lanes
        // finally copy every unit (own rows from A, the others from the gathered region) to the caller's buffer.
        const int ctid = warp - 6;
        const bool moves = R > 1 && !p.compute_only;
        if (moves) {
            if (warp == 6 && cta == 0 && lane < R && lane != rank) {
                fence_sys();
                st_release_sys(flag_ptr(p, lane, kFlagEntered + rank), p.epoch);
            }
            __syncwarp();
        }
        if (kHasSide && moves && !p.ag_pull && p.mc_base != nullptr) {
            // push through the multicast view: every unit is read once and stored once, the switch delivers it to
            // all ranks (this one included).  The whole warp moves a unit, 16 bytes per lane and step; the flags
            // stay unicast, one release store per peer by lanes 1..R-1 after their own system fence.
            if (ctid < kPushLanesShared) {
                const int units = mt_ag * kAgSubChunks;
                const size_t row_bytes = static_cast<size_t>(p.K) * sizeof(T);
                const int lane_id = cta * kPushLanesShared + ctid;
                const int n_lanes = p.ctas_per_rank * kPushLanesShared;
                if (ctid == 0 && lane == 0) CB_TRACE(TR_PUSH_BEGIN, globaltimer_ns());
                // nobody's region may be written before its owner has entered
                bool ok = true;
                if (lane < R && lane != rank)
                    ok = wait_flag_ge(flag_ptr(p, rank, kFlagEntered + lane), p.entered_need, ctl, W_ENTERED, lane);
                ok = __all_sync(0xffffffffu, ok);
                uint8_t *mc_slot = p.mc_base + p.symm_off + static_cast<size_t>(rank) * p.M * row_bytes;
                for (int cu = lane_id; cu < units && ok; cu += n_lanes) {
                    const int chunk = cu / kAgSubChunks, sub = cu % kAgSubChunks;
                    const int r0 = chunk * BM + sub * (BM / kAgSubChunks);
                    const int r1 = min(p.M, r0 + BM / kAgSubChunks);
                    if (r1 > r0) {
                        const size_t bytes = (r1 - r0) * row_bytes;            // a multiple of 16
                        const uint8_t *src = static_cast<const uint8_t *>(ra.A) + r0 * row_bytes;
                        uint8_t *dst = mc_slot + r0 * row_bytes;
                        constexpr int kInFlight = 8;
                        for (size_t off = static_cast<size_t>(lane) * 16; off < bytes; off += 32 * 16 * kInFlight) {
                            uint4 v[kInFlight];
#pragma unroll
                            for (int j = 0; j < kInFlight; ++j)
                                if (off + j * 512 < bytes) v[j] = ld_nc_v4(src + off + j * 512);
#pragma unroll
                            for (int j = 0; j < kInFlight; ++j)
                                if (off + j * 512 < bytes) multimem_st_v4(dst + off + j * 512, v[j]);
                        }
                    }
                    __syncwarp();
                    if (lane >= 1 && lane < R) {
                        fence_sys();
                        st_release_sys(flag_ptr(p, (rank + lane) % R, kFlagOpBase + rank * units + cu), p.epoch);
                    }
                    __syncwarp();
                }
                if (ctid == 0 && lane == 0) CB_TRACE(TR_PUSH_END, globaltimer_ns());
            }
        } else if (kHasSide && lane == 0 && ctid < kPushLanesShared && (moves || (ra.gather_out && !p.compute_only))) {
            // units of BM/kAgSubChunks rows, one flag per unit, every lane owns whole units
            const int units_per_dest = mt_ag * kAgSubChunks;
            const size_t row_bytes = static_cast<size_t>(p.K) * sizeof(T);
            const int lane_id = cta * kPushLanesShared + ctid;
            const int n_lanes = p.ctas_per_rank * kPushLanesShared;
            uint8_t *buf = smem_push + ctid * kPushPieceBytes;
            uint64_t *bar = &sh->push_bar[ctid];
            bool ok = true;
            uint32_t entered_ok = 0;
            uint32_t piece = 0;
            uint64_t entered_wait_ns = 0;
            const uint32_t staged_base = kFlagOpBase + static_cast<uint32_t>(R * mt_ag * kAgSubChunks);
            auto unit_rows = [&](int cu, int &r0, int &r1) {
                const int chunk = cu / kAgSubChunks, sub = cu % kAgSubChunks;
                r0 = chunk * BM + sub * (BM / kAgSubChunks);
                r1 = min(p.M, r0 + BM / kAgSubChunks);
            };
            auto unit_flag = [&](int src, int cu) { return kFlagOpBase + static_cast<uint32_t>(src * units_per_dest + cu); };
            // bytes from src to dst through this lane's 8 KiB staging piece (async proxy both ways)
            auto copy_rows = [&](const uint8_t *src, uint8_t *dst, size_t bytes) {
                for (size_t off = 0; off < bytes && ok; off += kPushPieceBytes, ++piece) {
                    const uint32_t len = static_cast<uint32_t>(min(static_cast<size_t>(kPushPieceBytes), bytes - off));
                    bulk_wait_read<0>();
                    mbar_expect_tx(bar, len);
                    bulk_load(buf, src + off, len, bar);
                    if (!(ok = mbar_wait(bar, piece & 1, ctl, W_DRAIN))) break;
                    bulk_store(dst + off, buf, len);
                    bulk_commit();
                }
            };
            auto wait_entered = [&](int d) {
                if ((entered_ok >> d) & 1) return;
                const uint64_t te0 = p.trace ? globaltimer_ns() : 0;
                ok = wait_flag_ge(flag_ptr(p, rank, kFlagEntered + d), p.entered_need, ctl, W_ENTERED, d);
                if (p.trace) entered_wait_ns += globaltimer_ns() - te0;
                entered_ok |= 1u << d;
            };
            if (ctid == 0) CB_TRACE(TR_PUSH_BEGIN, globaltimer_ns());
            if (moves && !p.ag_pull) {
                // push: same units, order and flags as the one-CTA kernel, destination rank-1 first
                const int total = (R - 1) * units_per_dest;
                for (int u = lane_id; u < total && ok; u += n_lanes) {
                    int d, cu, r0, r1;
                    ag_push_decode(R, units_per_dest, rank, u, d, cu);
                    unit_rows(cu, r0, r1);
                    wait_entered(d);
                    if (!ok) break;
                    if (r1 > r0)      // AllToAll-Matmul sends block d of A, AllGather-Matmul the whole A
                        copy_rows(static_cast<const uint8_t *>(ra.A) + (static_cast<size_t>(p.ag_a2a ? d * p.M : 0) + r0) * row_bytes,
                                  p.heap_base[d] + p.symm_off + (static_cast<size_t>(rank) * p.M + r0) * row_bytes,
                                  (r1 - r0) * row_bytes);
                    if (!ok) break;
                    bulk_wait<0>();
                    fence_proxy_async_global();
                    fence_sys();
                    st_release_sys(flag_ptr(p, d, unit_flag(rank, cu)), p.epoch);
                }
            } else if (moves) {
                // remote read, stage: my rows into my own region once no peer reads what an earlier launch left
                // there, then one "staged" flag per unit in every peer's flag region
                uint8_t *mine = p.heap_base[rank] + p.symm_off;
                for (int cu = lane_id; cu < units_per_dest && ok; cu += n_lanes) {
                    int r0, r1;
                    unit_rows(cu, r0, r1);
                    for (int j = 1; j < R && ok; ++j) wait_entered((rank + j) % R);
                    if (!ok) break;
                    if (r1 > r0)
                        copy_rows(static_cast<const uint8_t *>(ra.A) + r0 * row_bytes,
                                  mine + (static_cast<size_t>(rank) * p.M + r0) * row_bytes, (r1 - r0) * row_bytes);
                    if (!ok) break;
                    bulk_wait<0>();
                    fence_proxy_async_global();
                    fence_sys();
                    for (int j = 1; j < R; ++j)
                        st_release_sys(flag_ptr(p, (rank + R - j) % R, staged_base + rank * units_per_dest + cu), p.epoch);
                }
                // fetch: source rank+1 first (the order the tiles need them), unit by unit
                const int total = (R - 1) * units_per_dest;
                for (int u = lane_id; u < total && ok; u += n_lanes) {
                    const int s = (rank + 1 + u / units_per_dest) % R;
                    const int cu = u % units_per_dest;
                    int r0, r1;
                    unit_rows(cu, r0, r1);
                    if (!(ok = wait_flag_ge(flag_ptr(p, rank, staged_base + s * units_per_dest + cu), p.epoch, ctl, W_AG_CHUNK, s)))
                        break;
                    fence_proxy_async_global();
                    const size_t off = (static_cast<size_t>(s) * p.M + r0) * row_bytes;
                    if (r1 > r0) copy_rows(p.heap_base[s] + p.symm_off + off, mine + off, (r1 - r0) * row_bytes);
                    if (!ok) break;
                    bulk_wait<0>();
                    fence_proxy_async_global();
                    fence_sys();
                    st_release_sys(flag_ptr(p, rank, unit_flag(s, cu)), p.epoch);
                }
            }
            if (ra.gather_out && ok) {
                // gather result: own rows first, then the sources in the order their rows arrive
                const int total = R * units_per_dest;
                for (int u = lane_id; u < total && ok; u += n_lanes) {
                    const int s = (rank + u / units_per_dest) % R;
                    const int cu = u % units_per_dest;
                    int r0, r1;
                    unit_rows(cu, r0, r1);
                    if (r1 <= r0) continue;
                    const size_t off = (static_cast<size_t>(s) * p.M + r0) * row_bytes;
                    const uint8_t *src = static_cast<const uint8_t *>(ra.A) + r0 * row_bytes;
                    if (s != rank) {
                        if (!(ok = wait_flag_ge(flag_ptr(p, rank, unit_flag(s, cu)), p.epoch, ctl, W_AG_CHUNK, s))) break;
                        fence_proxy_async_global();
                        src = p.heap_base[rank] + p.symm_off + off;
                    }
                    copy_rows(src, static_cast<uint8_t *>(ra.gather_out) + off, (r1 - r0) * row_bytes);
                }
            }
            bulk_wait<0>();
            if (ctid == 0) {
                CB_TRACE(TR_PUSH_END, globaltimer_ns());
                CB_TRACE(TR_EPI_WAIT_NS, entered_wait_ns);     // time this lane waited for peers to enter
            }
        }
    }

    // ------------------------------------------------------------------ teardown ----
    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0) CB_TRACE(TR_END, globaltimer_ns());
}

}  // namespace cb
