// MXFP8 Matmul-ReduceScatter on CTA pairs (sm_100a): the block-scaled main loop of the MXFP8
// AllGather-Matmul pair kernel (256 x 256 tile per pair, e4m3 or e5m2 codes with UE8M0 scales per
// 32 along K, scale atoms by TMA, one accumulator + scale columns in TMEM) under the epilogue of
// the f16/bf16 pair reduce-scatter kernel (per-warp tiled TMA stores into the owner's staging
// rows, flags raised one tile late, non-blocking peer checks, own rows reduced in fixed rank
// order).  Symmetric layout and flag words are those of the f16/bf16 Matmul-ReduceScatter.
// Reference: include/catccos/dgemm/kernel/matmul_reduce_scatter_mx_tla.hpp:39,
// examples/ascend950_mxfp8_matmul_reduce_scatter/main.cpp:32-141.
#pragma once
#include "gemm_pair_rs.cuh"
#include "mx_pair.cuh"
#include "sched.h"

namespace cb {

constexpr int kMxRsStages = 5;                  // 5 x 33.5 KiB + 32 KiB of epilogue staging
constexpr int kMxRsSmemBytes = kMxRsStages * (kMxPA + kMxPB + kMxPSf) + kSideSmemBytes + 1024 + 512;
static_assert(kMxRsSmemBytes <= 232448, "shared memory budget");
// MXFP4 operands (e2m1, K-major only): a stage of 128 bytes per row holds 256 elements = two scale atoms per operand tile
constexpr int kMxRsSfFp4 = 3072;
constexpr int kMxRsSmemBytesFp4 = kMxRsStages * (kMxPA + kMxPB + kMxRsSfFp4) + kSideSmemBytes + 1024 + 512;
static_assert(kMxRsSmemBytesFp4 <= 232448, "shared memory budget");

struct MxRsParams {
    MxRankArgs ranks[kMaxRanks];     // tmA [M, K], tmB, tmSfa / tmSfb scale atoms, C; the gathered maps are unused
    uint8_t *heap_base[kMaxRanks];
    uint64_t symm_off;               // this launch's half of the staging region
    int world, rank_base, n_local, ctas_per_rank;
    int M, N, K;                     // M = rows of the full product, K = this rank's share of the contraction
    uint32_t fmt_bits;               // a/b format fields of the instruction descriptor (0: e4m3, e5m2: bits 7 and 10)
    uint32_t epoch;
    uint32_t entered_need;
    int compute_only;
    int rs_fp16;                     // partial tiles cross the link as fp16 (0: in the output type)
    int a2a;                         // Matmul-AllToAll: row blocks go to their owners without the sum; C is [M, N]
    uint64_t timeout_ns;
    int *status;
    unsigned long long *trace;
};

struct MxRsSmem {
    uint64_t full[kMxRsStages];
    uint64_t empty[kMxRsStages];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint64_t drain;
    uint64_t epi_bar;
    uint32_t tmem_base;
    int abort_flag;
    int epi_ok[2];
};

template <typename TOut, bool B_MN, int FMT = MX_FP8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    mx_pair_rs_kernel(const __grid_constant__ MxRsParams p, const __grid_constant__ RsMapsAll maps) {
    static_assert(!(FMT == MX_FP4 && B_MN), "4-bit operands are K-major");
    constexpr int kMxPSf = FMT == MX_FP4 ? kMxRsSfFp4 : cb::kMxPSf;     // shadows the MXFP8 constant
    constexpr int kAtoms = FMT == MX_FP4 ? 2 : 1;                        // scale atoms per operand tile and stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kMxRsStages * kMxPA;
    uint8_t *smem_side = smem_b + kMxRsStages * kMxPB;          // epilogue staging (1024-byte aligned for the swizzle)
    uint8_t *smem_sf = smem_side + kSideSmemBytes;
    MxRsSmem *sh = reinterpret_cast<MxRsSmem *>(smem_sf + kMxRsStages * kMxPSf);
    static_assert(sizeof(MxRsSmem) <= 512, "barrier block outgrew its budget");
    static_assert((kMxRsStages * (kMxPA + kMxPB)) % 1024 == 0, "epilogue staging must stay 1024-byte aligned");
    static_assert((kMxRsStages * kMxPSf) % 8 == 0 && kMxPSf % 512 == 0, "scale stages: 512-byte atoms, barriers 8-byte aligned");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int pair = cta >> 1, pairs = p.ctas_per_rank >> 1;
    const uint32_t cr = cluster_ctarank();
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MxRankArgs &ra = p.ranks[lrank];
    const RsMaps &mp = maps.r[lrank];
    const int mr = p.M / R;                                     // rows owned by one rank
    const int nt = (p.N + BN - 1) / BN;
    const int mt2 = (mr + BM2 - 1) / BM2;
    const int per = ((mr + BM - 1) / BM) * nt;                  // flag index space: 128-row tiles per owner
    const int num_tiles = R * mt2 * nt;
    const int Kb = FMT == MX_FP4 ? p.K / 2 : p.K;               // bytes of one operand row
    const int kblocks = (Kb + MX_BK - 1) / MX_BK;               // pipeline stages per tile
    const int kb4 = (p.K + 127) / 128;                          // scale atoms per row tile
    const int a_atoms_rows = (p.M + BM - 1) / BM;               // atom rows of A's scales

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMxRsStages; ++s) {
            mbar_init(&sh->full[s], 2);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 8);
        mbar_init(&sh->drain, 1);
        mbar_init(&sh->epi_bar, 128);
        sh->abort_flag = 0;
        sh->epi_ok[0] = sh->epi_ok[1] = 1;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
        prefetch_tensormap(&ra.tmSfa);
        prefetch_tensormap(&ra.tmSfb);
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
    const uint32_t tmem_sf0 = tmem_base + BN;                   // 4 sets of 4 (A) + 8 (B) scale columns

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x == 0) CB_MX_TRACE(TR_START, globaltimer_ns());
    auto flagp = [&](int pe, uint32_t word) { return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + word; };

    // tile order: super-rounds of peer stripes followed by a lagging own stripe (sched.h)
    const RsOrder order = rs_order_make(R, nt, mt2, pairs);
    auto decode = [&](int t, int &d, int &mi2, int &ni, bool &lead_ok) {
        rs_order_decode(order, rank, t, d, mi2, ni);
        lead_ok = d * mr + mi2 * BM2 < (d + 1) * mr;
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
                const int a_row = d * mr + mi2 * BM2 + static_cast<int>(cr) * BM;    // rows past M read as zero
                // a chunk past the matrix has no scale atoms: reuse the last row of atoms (its rows are never stored)
                const int sfa_atom0 = min(a_row >> 7, a_atoms_rows - 1) * kb4;
                const int n_half = ni * BN + static_cast<int>(cr) * 128;
                const int sfb_atom0 = (ni * 2) * kb4;
                const bool second_b_atom = (ni * BN + 128) < p.N;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxRsStages;
                    const uint32_t ph = (it / kMxRsStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    uint8_t *ssf = smem_sf + st * kMxPSf;
                    const int atoms = min(kAtoms, kb4 - kb * kAtoms);      // the last MXFP4 stage may hold one atom
                    mbar_expect_tx_cluster(full_leader, kMxPA + kMxPB + atoms * 512 * (second_b_atom ? 3 : 2));
                    tma_load_2d_pair(smem_a + st * kMxPA, &ra.tmA, full_leader, kb * MX_BK, a_row);
                    if (B_MN)
                        tma_load_2d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, n_half, kb * MX_BK);
                    else
                        tma_load_2d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, kb * MX_BK, n_half);
                    for (int a = 0; a < atoms; ++a) {
                        const int ka = kb * kAtoms + a;
                        tma_load_2d_pair(ssf + a * 512, &ra.tmSfa, full_leader, 0, sfa_atom0 + ka);
                        tma_load_2d_pair(ssf + (kAtoms + a) * 512, &ra.tmSfb, full_leader, 0, sfb_atom0 + ka);
                        if (second_b_atom)
                            tma_load_2d_pair(ssf + (2 * kAtoms + a) * 512, &ra.tmSfb, full_leader, 0, sfb_atom0 + kb4 + ka);
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
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                int d, mi2, ni;
                bool lead_ok;
                decode(t, d, mi2, ni, lead_ok);
                if (!lead_ok) continue;
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMxRsStages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kMxRsStages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + st * kMxPA);
                    const uint32_t b_addr = smem_u32(smem_b + st * kMxPB);
                    const uint32_t sf_addr = smem_u32(smem_sf + st * kMxPSf);
                    const uint32_t tmem_sfa = tmem_sf0 + (it & 3u) * (FMT == MX_FP4 ? 24u : 16u);
                    if constexpr (FMT == MX_FP4) {
                        const uint32_t tmem_sfb = tmem_sfa + 4 * kAtoms;     // per atom: 4 columns (n 0-127) + 4 (n 128-255)
                        const int mmas = min(4, p.K / 64 - kb * 4);
                        const int atoms = (mmas + 1) / 2;
                        for (int a = 0; a < atoms; ++a) {
                            tmem_cp_32x128b_warpx4_pair(tmem_sfa + a * 4, make_smem_desc_noswizzle(sf_addr + a * 512, 16, 128));
                            tmem_cp_32x128b_warpx4_pair(tmem_sfb + a * 8,
                                                        make_smem_desc_noswizzle(sf_addr + (kAtoms + a) * 512, 16, 128));
                            tmem_cp_32x128b_warpx4_pair(tmem_sfb + a * 8 + 4,
                                                        make_smem_desc_noswizzle(sf_addr + (2 * kAtoms + a) * 512, 16, 128));
                        }
                        for (int k = 0; k < mmas; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);   // 64 e2m1 = 32 bytes of a row
                            const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t sf_id = static_cast<uint32_t>(k & 1) * 2u;
                            umma_mxfp4_pair(tmem_base, ad, bd, make_idesc_fp4(2 * BM, BN, sf_id, sf_id, 1u), tmem_sfa + (k >> 1) * 4,
                                            tmem_sfb + (k >> 1) * 8, (kb | k) != 0);
                        }
                    } else {
                        const uint32_t tmem_sfb = tmem_sfa + 4;
                        tmem_cp_32x128b_warpx4_pair(tmem_sfa, make_smem_desc_noswizzle(sf_addr, 16, 128));
                        tmem_cp_32x128b_warpx4_pair(tmem_sfb, make_smem_desc_noswizzle(sf_addr + 512, 16, 128));
                        tmem_cp_32x128b_warpx4_pair(tmem_sfb + 4, make_smem_desc_noswizzle(sf_addr + 1024, 16, 128));
#pragma unroll
                        for (int k = 0; k < MX_BK / 32; ++k) {
                            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 4096, 128 * MX_BK, 1024)
                                                     : make_smem_desc(b_addr + k * 32, 16, 1024);
                            const uint32_t idesc = make_idesc_mxf8(2 * BM, BN, k, k) | p.fmt_bits | (B_MN ? (1u << 16) : 0u);
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
        // as in the f16/bf16 pair reduce-scatter kernel: every warp drains its 32 rows 64 columns at a
        // time into a swizzled staging buffer, lane 0 sends each buffer with one tiled TMA store
        const int q = warp & 3;
        const int etid = (warp - 2) * 32 + lane;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        uint32_t entered_ok = 0;
        uint32_t check_no = 0;
        bool ok = true;
        GroupSync epi{&sh->epi_bar, 0};
        const TOut *const my_stage = reinterpret_cast<const TOut *>(p.heap_base[rank] + p.symm_off);
        uint8_t *const wbuf = smem_side + q * 8192;
        constexpr int kSlabs = BN / 64;
        bool pend = false;
        const bool fp16x = p.rs_fp16 != 0;       // exchange format of the partial tiles
        float amax_sent = 0.0f;                  // largest magnitude this thread sent as fp16
        int pend_d = 0, pend_tip = 0;
        auto publish = [&](bool everything) -> bool {
            if (!pend) return true;
            if (lane == 0) {
                if (everything) bulk_wait<0>(); else bulk_wait<kSlabs>();
                fence_proxy_async_global();
            }
            if (!epi.sync(ctl)) return false;
            if (etid == 0) {
                fence_sys();
                st_release_sys(flagp(pend_d, kFlagOpBase + rank * per + pend_tip), p.epoch);
            }
            pend = false;
            return true;
        };
        for (int t = pair; t < num_tiles && ok; t += pairs) {
            int d, mi2, ni;
            bool lead_ok;
            decode(t, d, mi2, ni, lead_ok);
            if (!lead_ok) continue;
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const int row_end = (d + 1) * mr;
            const int out_row0 = d * mr + mi2 * BM2 + static_cast<int>(cr) * BM;
            const bool half_ok = out_row0 < row_end;
            const int row = out_row0 + row_in_tile;
            const bool row_ok = row < row_end;
            const bool warp_ok = out_row0 + q * 32 < row_end;
            const int n0 = ni * BN;
            const int tile_in_peer = (mi2 * 2 + static_cast<int>(cr)) * nt + ni;
            const bool remote = d != rank;
            const bool comm = R > 1 && !p.compute_only && half_ok;

            if (comm && (remote ? !((entered_ok >> d) & 1) : !p.a2a)) {
                // look once without blocking (lane s for rank s); only if something is missing raise the
                // pending flag first and wait
                volatile int *verdict = &sh->epi_ok[check_no & 1];
                ++check_no;
                const uint32_t *my_flag = nullptr;
                uint32_t my_need = 0;
                if (warp == 2) {
                    if (remote) {
                        if (lane == 0) {
                            my_flag = flagp(rank, kFlagEntered + d);
                            my_need = p.entered_need;
                        }
                    } else if (lane < R && lane != rank) {
                        my_flag = flagp(rank, kFlagOpBase + lane * per + tile_in_peer);
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
                    if (warp == 2) {
                        const bool w = !my_flag || wait_flag_ge(my_flag, my_need, ctl, remote ? W_ENTERED : W_RS_PARTIAL,
                                                                 remote ? d : static_cast<int>(my_flag - flagp(rank, 0)));
                        const bool all_up = __all_sync(0xffffffffu, w);
                        if (lane == 0) *verdict = all_up ? 1 : 0;
                    }
                    if (!(ok = epi.sync(ctl))) break;
                }
                if (!(ok = (*verdict == 1))) break;
                if (remote) entered_ok |= 1u << d;
            }

            const int y_map = out_row0 - d * mr + q * 32;
            if (half_ok) {
#pragma unroll 1
                for (int sl = 0; sl < kSlabs; ++sl) {
                    uint8_t *buf = wbuf + (sl & 1) * 4096;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = sl * 2 + cc;
                        uint32_t v[32];
                        tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                        const int col = n0 + c * 32;
                        const bool reduce = !p.a2a && !remote && R > 1 && row_ok && col < p.N;
                        uint4 part[kMaxRanks][4];
                        if (reduce) {
#pragma unroll
                            for (int s = 0; s < kMaxRanks; ++s) {
                                if (s < R && s != rank) {
                                    const TOut *src = my_stage + (static_cast<size_t>(s) * mr + (row - rank * mr)) * p.N + col;
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
                                            const float2 x = unpack_partial<TOut>(w4[h], fp16x);
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
                            pk[i] = remote ? pack_partial<TOut>(f[2 * i], f[2 * i + 1], fp16x) : Pack2<TOut>::pack(f[2 * i], f[2 * i + 1]);
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
                        if (warp_ok && x < p.N) tma_store_2d(&mp.out[d], buf, x, y_map);
                        bulk_commit();
                    }
                }
            }
            // accumulator drained (there is only one): the next tile's MMAs may start
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty), 0));

            if (!(ok = publish(!half_ok))) break;
            if (comm && remote) {
                pend = true;
                pend_d = d;
                pend_tip = tile_in_peer;
            }
            ++tcount;
        }
        if (ok) ok = publish(true);
        if (!(amax_sent <= 65504.0f)) report_partial_range(p.status, rank, static_cast<int>(tcount));
        if (lane == 0) bulk_wait<0>();
        if (p.a2a && R > 1 && ok && !p.compute_only) {
            // Matmul-AllToAll, second phase: the blocks the peers stored into my staging slots go into C behind my own
            TOut *const C = reinterpret_cast<TOut *>(ra.C);
            const int total = (R - 1) * per;
            for (int u = cta; u < total && ok; u += p.ctas_per_rank) {
                const int s = (rank + 1 + u / per) % R;
                const int tip = u % per;
                const int mi = tip / nt, ni = tip % nt;
                const int r0 = mi * BM;
                const int r1 = min(mr, r0 + BM);
                if (r0 >= r1) continue;
                const uint32_t w = kFlagOpBase + s * per + tip;
                if (!(ok = wait_flag_ge(flagp(rank, w), p.epoch, ctl, W_RS_PARTIAL, w))) break;
                const int c0 = ni * BN;
                const int c1 = min(p.N, c0 + BN);
                const int vec_per_row = (c1 - c0) / 8;
                const TOut *src = my_stage + static_cast<size_t>(s) * mr * p.N;
                TOut *dst = C + static_cast<size_t>(s) * mr * p.N;
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
            st_release_sys(flagp(lane, kFlagEntered + rank), p.epoch);
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
    if (threadIdx.x == 0) CB_MX_TRACE(TR_END, globaltimer_ns());
}

}  // namespace cb
