// Matmul-ReduceScatter / Matmul-AllReduce f16/bf16 with CTA pairs (tcgen05 cta_group::2), sm_100a.
//
// Main loop of the pair AllGather-Matmul kernel (256 x 256 tile per pair, every CTA loads its own
// 128 rows of A and 128 columns of B, accumulator of its 128 rows in its own TMEM); each CTA's
// epilogue then treats its 128 x 256 half as the one-CTA kernel treats a tile: a partial
// half-tile goes to the owner's staging rows (tiled TMA stores, 32 rows x 64 columns each)
// followed by one flag, the own rows are reduced in fixed rank order (own fp32 accumulator
// first) once every peer's flag for that half-tile is up.  Flag words and symmetric layout are the one-CTA kernel's, so
// both kernels serve the same buffers.
#pragma once
#include <type_traits>

#include "common.h"
#include "gemm_fused.cuh"
#include "gemm_pair.cuh"
#include "ptx.cuh"
#include "sched.h"

namespace cb {

struct PairRsSmem {
    uint64_t full[kPStages];
    uint64_t empty[kPStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t drain;
    uint64_t epi_bar;               // the CTA's 128 epilogue threads
    uint32_t tmem_base;
    int abort_flag;
    int epi_ok[2];                  // verdicts of the epilogue's peer checks, used in turn
};

template <int OP, typename T, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    pair_rs_kernel(const __grid_constant__ FusedParams p, const __grid_constant__ RsMapsAll maps) {
    static_assert(OP == OP_MMRS || OP == OP_MMAR || OP == OP_MMA2A, "reduce-scatter family only");
    // OP_MMA2A (Matmul-AllToAll): the same movement of row blocks to their owners, without the sum -- a block is
    // stored in the output type into the owner's staging slot, the owner copies the R - 1 slots it received into
    // its output behind its own block (examples/ascend950_matmul_alltoall/scripts/gen_data.py:19-89).
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + kPStages * kPAStage;
    uint8_t *smem_side = smem + kPStages * (kPAStage + kPBStage);
    PairRsSmem *sh = reinterpret_cast<PairRsSmem *>(smem_side + kSideSmemBytes);
    static_assert(sizeof(PairRsSmem) <= 512, "barrier block outgrew its budget");
    static_assert(4 * 2 * 32 * 128 <= kSideSmemBytes, "epilogue staging: 4 warps x 2 buffers x 32 rows x 128 B");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;      // ctas_per_rank is even
    const int pair = cta >> 1;
    const int pairs = p.ctas_per_rank >> 1;
    const uint32_t cr = cluster_ctarank();
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const RankArgs &ra = p.ranks[lrank];
    const RsMaps &mp = maps.r[lrank];
    const int mr = rows_per_rank<OP>(p);                        // rows owned by one rank
    const int nt = ceil_div(p.N, BN);
    const int mt2 = ceil_div(mr, BM2);                          // pair tiles per owner along M
    const int per2 = mt2 * nt;
    const int per = ceil_div(mr, BM) * nt;                      // 128-row tiles per owner: the flag index space
    const int num_tiles = R * per2;
    const int kblocks = ceil_div(p.K, BK);

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
        mbar_init(&sh->epi_bar, 128);
        sh->abort_flag = 0;
        sh->epi_ok[0] = sh->epi_ok[1] = 1;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
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

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x == 0) CB_TRACE(TR_START, globaltimer_ns());

    // tile order: super-rounds of peer stripes followed by a lagging own stripe (sched.h)
    const RsOrder order = rs_order_make(R, nt, mt2, pairs);
    auto decode = [&](int t, int &d, int &mi2, int &ni, bool &lead_ok) {
        rs_order_decode(order, rank, t, d, mi2, ni);
        lead_ok = d * mr + mi2 * BM2 < min(p.M, (d + 1) * mr);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                int d, mi2, ni;
                bool lead_ok;
                decode(t, d, mi2, ni, lead_ok);
                if (!lead_ok) continue;
                const int a_row = d * mr + mi2 * BM2 + static_cast<int>(cr) * BM;   // rows past M read as zero
                const int n_half = ni * BN + static_cast<int>(cr) * 128;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kPStages;
                    const uint32_t ph = (it / kPStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    mbar_expect_tx_cluster(full_leader, kPAStage + kPBStage);
                    tma_load_2d_pair(smem_a + st * kPAStage, &ra.tmA, full_leader, kb * BK, a_row);
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
            if (!ok) {
                const uint64_t t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 20000ull) {
                }
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
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                int d, mi2, ni;
                bool lead_ok;
                decode(t, d, mi2, ni, lead_ok);
                if (!lead_ok) continue;
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
        // Every epilogue warp owns 32 rows of the CTA's half-tile.  It drains them 64 columns at a
        // time into its own swizzled staging buffer (32 rows x 128 B, two buffers) and lane 0 sends
        // each buffer with ONE tiled TMA store: to the owner's staging rows over NVLink, to this
        // rank's output, or (Matmul-AllReduce, own rows) to the output and every peer's final rows.
        // 16 stores per half-tile; the tensor maps end at the last valid row, so ragged tiles are
        // clipped by the copy engine.
        const int q = warp & 3;
        const int etid = (warp - 2) * 32 + lane;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        uint32_t entered_ok = 0;
        uint32_t check_no = 0;
        bool ok = true;
        GroupSync epi{&sh->epi_bar, 0};
        uint64_t epi_wait_ns = 0, epi_store_ns = 0, flush_ns = 0;
        T *const C = reinterpret_cast<T *>(ra.C);
        const T *const my_stage = reinterpret_cast<const T *>(p.heap_base[rank] + p.symm_off);
        uint8_t *const wbuf = smem_side + q * 8192;          // this warp's two 4 KiB staging buffers
        constexpr int kSlabs = BN / 64;                       // stores (bulk groups) per half-tile and warp
        // A half-tile's flag is raised one tile late: its stores then complete (a round trip to the
        // peer) while the next accumulator is drained, instead of holding this one up.  The pending
        // flag is always raised before this CTA waits for a peer, so no rank can wait for a flag
        // whose writer waits for it.
        bool pend = false, pend_remote = false;
        int pend_d = 0, pend_tip = 0;
        const bool fp16x = p.rs_fp16 != 0;       // exchange format of the partial tiles
        float amax_sent = 0.0f;                  // largest magnitude this thread sent as fp16
        auto publish = [&](bool everything) -> bool {
            if (!pend) return true;
            if (lane == 0) {
                if (everything) bulk_wait<0>(); else bulk_wait<kSlabs>();
                fence_proxy_async_global();
            }
            if (!epi.sync(ctl)) return false;
            if (etid == 0) {
                fence_sys();
                if (pend_remote) {
                    st_release_sys(flag_ptr(p, pend_d, kFlagOpBase + rank * per + pend_tip), p.epoch);
                } else {
                    for (int jj = 1; jj < R; ++jj) {
                        const int dd = (rank + jj) % R;
                        st_release_sys(flag_ptr(p, dd, kFlagOpBase + (R + rank) * per + pend_tip), p.epoch);
                    }
                }
            }
            pend = false;
            return true;
        };
        for (int t = pair; t < num_tiles && ok; t += pairs) {
            int d, mi2, ni;
            bool lead_ok;
            decode(t, d, mi2, ni, lead_ok);
            if (!lead_ok) continue;
            const uint32_t acc = tcount & 1;
            if (!(ok = mbar_wait(&sh->tmem_full[acc], (tcount >> 1) & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const int row_end = min(p.M, (d + 1) * mr);
            const int out_row0 = d * mr + mi2 * BM2 + static_cast<int>(cr) * BM;
            const bool half_ok = out_row0 < row_end;            // this CTA's half holds rows of the owner
            const int row = out_row0 + row_in_tile;
            const bool row_ok = row < row_end;
            const bool warp_ok = out_row0 + q * 32 < row_end;   // this warp has at least one row
            const int n0 = ni * BN;
            const int tile_in_peer = (mi2 * 2 + static_cast<int>(cr)) * nt + ni;
            const bool remote = d != rank;
            const bool comm = R > 1 && !p.compute_only && half_ok;

            if (comm && (remote ? !((entered_ok >> d) & 1) : OP != OP_MMA2A)) {
                // This half-tile depends on peers: the owner must have entered (remote rows), or every
                // peer's partial must be in (own rows).  Warp 2 looks once without blocking, lane s for
                // rank s; only if something is missing is the pending flag raised first (which costs a
                // round trip to a peer) and the wait made blocking.
                const uint64_t tp0 = p.trace ? globaltimer_ns() : 0;
                volatile int *verdict = &sh->epi_ok[check_no & 1];
                ++check_no;
                const uint32_t *my_flag = nullptr;      // the flag this lane looks at
                uint32_t my_need = 0;
                if (warp == 2) {
                    if (remote) {
                        if (lane == 0) {
                            my_flag = flag_ptr(p, rank, kFlagEntered + d);
                            my_need = p.entered_need;
                        }
                    } else if (lane < R && lane != rank) {
                        my_flag = flag_ptr(p, rank, kFlagOpBase + lane * per + tile_in_peer);
                        my_need = p.epoch;
                    }
                    const bool up = !my_flag || static_cast<int32_t>(ld_acquire_sys(my_flag) - my_need) >= 0;
                    if (__all_sync(0xffffffffu, up)) {
                        if (lane == 0) *verdict = 1;
                    } else if (lane == 0) {
                        *verdict = 2;
                    }
                }
                if (!(ok = epi.sync(ctl))) break;
                if (*verdict == 2) {
                    // every thread has to have read the first verdict before warp 2 overwrites it
                    if (!(ok = epi.sync(ctl))) break;
                    if (!(ok = publish(true))) break;
                    if (p.trace) flush_ns += globaltimer_ns() - tp0;
                    if (warp == 2) {
                        const bool w = !my_flag || wait_flag_ge(my_flag, my_need, ctl, remote ? W_ENTERED : W_RS_PARTIAL,
                                                                 remote ? d : static_cast<int>(my_flag - flag_ptr(p, rank, 0)));
                        const bool all_up = __all_sync(0xffffffffu, w);
                        if (lane == 0) *verdict = all_up ? 1 : 0;
                    }
                    if (!(ok = epi.sync(ctl))) break;
                }
                if (!(ok = (*verdict == 1))) break;
                if (remote) entered_ok |= 1u << d;
                if (p.trace) epi_wait_ns += globaltimer_ns() - tp0;
            }

            const int y_map = out_row0 - d * mr + q * 32;        // first row of this warp inside the maps of owner d
            const uint64_t te0 = p.trace ? globaltimer_ns() : 0;
            if (half_ok) {
#pragma unroll 1
                for (int sl = 0; sl < kSlabs; ++sl) {
                    uint8_t *buf = wbuf + (sl & 1) * 4096;
                    if (lane == 0) bulk_wait_read<1>();         // the store two slabs ago has read this buffer
                    __syncwarp();
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = sl * 2 + cc;
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                        const int col = n0 + c * 32;
                        const bool reduce = OP != OP_MMA2A && !remote && R > 1 && row_ok && col < p.N;
                        uint4 part[kMaxRanks][4];
                        if (reduce) {
#pragma unroll
                            for (int s = 0; s < kMaxRanks; ++s) {
                                if (s < R && s != rank) {
                                    const T *src = my_stage + (static_cast<size_t>(s) * mr + (row - rank * mr)) * p.N + col;
#pragma unroll
                                    for (int g = 0; g < 4; ++g)
                                        part[s][g] = (col + g * 8 < p.N) ? *reinterpret_cast<const uint4 *>(src + g * 8)
                                                                         : make_uint4(0, 0, 0, 0);
                                }
                            }
                        }
                        tmem_ld_wait();
                        float f[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
                        if (reduce) {
                            // fixed order: own fp32 accumulator, then the peers' partials by rank
#pragma unroll
                            for (int s = 0; s < kMaxRanks; ++s) {
                                if (s < R && s != rank) {
#pragma unroll
                                    for (int g = 0; g < 4; ++g) {
                                        const uint32_t w4[4] = {part[s][g].x, part[s][g].y, part[s][g].z, part[s][g].w};
#pragma unroll
                                        for (int h = 0; h < 4; ++h) {
                                            const float2 x = unpack_partial<T>(w4[h], fp16x);
                                            f[g * 8 + h * 2] += x.x;
                                            f[g * 8 + h * 2 + 1] += x.y;
                                        }
                                    }
                                }
                            }
                        }
                        uint32_t pk[16];
                        if (remote && fp16x) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) amax_sent = fmaxf(amax_sent, fabsf(f[i]));
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            pk[i] = remote ? pack_partial<T>(f[2 * i], f[2 * i + 1], fp16x) : Pack2<T>::pack(f[2 * i], f[2 * i + 1]);
                        // row `lane` of the buffer; 16-byte chunk j sits at j ^ (row & 7) (128-byte swizzle)
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int j = (cc * 4 + g) ^ (lane & 7);
                            *reinterpret_cast<uint4 *>(buf + lane * 128 + j * 16) =
                                make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int x = n0 + sl * 64;
                        if (warp_ok && x < p.N) {
                            tma_store_2d(&mp.out[d], buf, x, y_map);
                            if (OP == OP_MMAR && !remote && R > 1 && !p.compute_only) {
                                for (int jj = 1; jj < R; ++jj) tma_store_2d(&mp.fin[(rank + jj) % R], buf, x, y_map);
                            }
                        }
                        bulk_commit();          // one group per slab, stored or not: the count is uniform
                    }
                }
            }
            if (p.trace) epi_store_ns += globaltimer_ns() - te0;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty[acc]), 0));

            if (!(ok = publish(!half_ok))) break;       // the tile before this one
            if (comm && (remote || OP == OP_MMAR)) {
                pend = true;
                pend_remote = remote;
                pend_d = d;
                pend_tip = tile_in_peer;
            }
            ++tcount;
        }
        if (ok) ok = publish(true);
        if (lane == 0) bulk_wait<0>();
        if (!(amax_sent <= 65504.0f)) report_partial_range(p.status, rank, static_cast<int>(tcount));
        if (etid == 0) {
            CB_TRACE(TR_EPI_WAIT_NS, epi_wait_ns);
            CB_TRACE(TR_EPI_STORE_NS, epi_store_ns);
            CB_TRACE(TR_PROD_WAIT_NS, flush_ns);            // of the wait time: slow path (flag raised first)
        }
        if (OP == OP_MMAR && R > 1 && ok && !p.compute_only) {
            // second phase: copy the peers' reduced tiles from my "final" rows into D
            const size_t final_off = static_cast<size_t>(R) * mr * p.N;
            const T *fin = reinterpret_cast<const T *>(p.heap_base[rank] + p.symm_off) + final_off;
            const int total = (R - 1) * per;
            for (int u = cta; u < total && ok; u += p.ctas_per_rank) {
                const int o = (rank + 1 + u / per) % R;
                const int tip = u % per;
                const int mi = tip / nt, ni = tip % nt;
                const int r0 = o * mr + mi * BM;
                const int r1 = min(min(p.M, (o + 1) * mr), r0 + BM);
                if (r0 >= r1) continue;
                const uint32_t w = kFlagOpBase + (R + o) * per + tip;
                if (!(ok = wait_flag_ge(flag_ptr(p, rank, w), p.epoch, ctl, W_AR_FINAL, w))) break;
                const int c0 = ni * BN;
                const int c1 = min(p.N, c0 + BN);
                const int vec_per_row = (c1 - c0) / 8;
                for (int i = etid; i < (r1 - r0) * vec_per_row; i += 128) {
                    const int rr = r0 + i / vec_per_row;
                    const int cc = c0 + (i % vec_per_row) * 8;
                    const size_t off = static_cast<size_t>(rr) * p.N + cc;
                    *reinterpret_cast<uint4 *>(C + off) = *reinterpret_cast<const uint4 *>(fin + off);
                }
            }
        }
        if (OP == OP_MMA2A && R > 1 && ok && !p.compute_only) {
            // second phase: the blocks the peers stored into my staging slots go into D behind my own block
            const int total = (R - 1) * per;
            for (int u = cta; u < total && ok; u += p.ctas_per_rank) {
                const int s = (rank + 1 + u / per) % R;
                const int tip = u % per;
                const int mi = tip / nt, ni = tip % nt;
                const int r0 = mi * BM;                                   // row inside the block
                const int r1 = min(mr, r0 + BM);
                if (r0 >= r1) continue;
                const uint32_t w = kFlagOpBase + s * per + tip;
                if (!(ok = wait_flag_ge(flag_ptr(p, rank, w), p.epoch, ctl, W_RS_PARTIAL, w))) break;
                const int c0 = ni * BN;
                const int c1 = min(p.N, c0 + BN);
                const int vec_per_row = (c1 - c0) / 8;
                const T *src = my_stage + static_cast<size_t>(s) * mr * p.N;
                T *dst = C + static_cast<size_t>(s) * mr * p.N;
                for (int i = etid; i < (r1 - r0) * vec_per_row; i += 128) {
                    const size_t off = static_cast<size_t>(r0 + i / vec_per_row) * p.N + c0 + (i % vec_per_row) * 8;
                    *reinterpret_cast<uint4 *>(dst + off) = *reinterpret_cast<const uint4 *>(src + off);
                }
            }
        }
    } else if (warp == 6) {
        // tell every peer that this rank has entered the epoch: its staging rows may be overwritten
        if (R > 1 && !p.compute_only && cta == 0 && lane < R && lane != rank) {
            fence_sys();
            st_release_sys(flag_ptr(p, lane, kFlagEntered + rank), p.epoch);
        }
    }

    // ------------------------------------------------------------------ teardown ----
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
