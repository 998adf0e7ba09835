// Fused GEMM + collective kernel for f16/bf16 (sm_100a).
//
// One persistent CTA per SM.  Warp 0 feeds shared memory with TMA (no multicast),
// warp 1 issues tcgen05.mma into two TMEM accumulators (128 lanes x 256 fp32 columns each),
// warps 2-5 drain an accumulator while the next tile is being multiplied, warps 6-7 move
// all-gather traffic to the peers.  The collective is done tile by tile over peer-mapped
// memory: every remote tile is either pushed into the consumer's own symmetric region before
// the consumer's TMA reads it (AllGather-Matmul) or written by the producing epilogue straight
// into the owner's staging rows (Matmul-ReduceScatter / Matmul-AllReduce); readiness travels as
// single-writer epoch flags with release/acquire at system scope.  Every wait is bounded.
//
// This is the one-CTA (128 x 256 tile) form: the fallback of the CTA-pair kernels in gemm_pair.cuh and
// gemm_pair_rs.cuh (CATCCOS_TWO_CTA=0) and the kernel behind catccos_gemm_no_alloc.
#pragma once
#include <type_traits>

#include "common.h"
#include "ptx.cuh"

namespace cb {

struct GemmSmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t drain;
    uint64_t epi_bar;    // 128 epilogue threads
    uint64_t push_bar[kPushLanes];   // pusher CTA: one per lane (bulk load landed)
    uint32_t tmem_base;
    int abort_flag;
    int epi_ok;
};

// Bounded barrier among a fixed group of threads (an mbarrier instead of bar.sync so that a
// group member that gave up cannot strand the others).
struct GroupSync {
    uint64_t *bar;
    uint32_t phase;
    __device__ __forceinline__ bool sync(const WaitCtl &c) {
        mbar_arrive(bar);
        const bool ok = mbar_wait(bar, phase, c, W_DRAIN);
        phase ^= 1;
        return ok;
    }
};

struct Tile {
    bool valid;
    bool a_gathered;   // AG-MM: rows come from the gathered region (another rank pushed them)
    int a_row;         // first row in the A tensor map used
    int n0;            // first output column
    int out_row;       // first output row (operator's output coordinates)
    int row_end;       // rows >= row_end are not written
    int peer;          // AG-MM: source rank of the rows;  MM-RS/AR: destination (owner) rank
    int mi, ni;        // tile coordinates inside the peer's block
};

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Rows owned by one rank in the reduce-scatter family.
template <int OP>
__device__ __forceinline__ int rows_per_rank(const FusedParams &p) {
    return OP == OP_MMAR ? ceil_div(p.M, p.world) : p.M / p.world;
}

template <int OP>
__device__ __forceinline__ int tiles_per_peer(const FusedParams &p) {
    const int rows = (OP == OP_AGMM) ? p.M : rows_per_rank<OP>(p);
    return ceil_div(rows, BM) * ceil_div(p.N, BN);
}

// Tile order.  AG-MM: own rows first, then source ranks rank+1, rank+2, ... (the order in which
// the peers push to us).  MM-RS / MM-AR: destination ranks rank+1, rank+2, ..., own rows last, so
// that partial tiles leave early and the own-row reduction runs when the peers' tiles are in.
template <int OP>
__device__ __forceinline__ Tile decode_tile(const FusedParams &p, int rank, int t) {
    Tile tl;
    const int nt = ceil_div(p.N, BN);
    const int per = tiles_per_peer<OP>(p);
    const int j = t / per;
    const int u = t - j * per;
    tl.mi = u / nt;
    tl.ni = u - tl.mi * nt;
    tl.n0 = tl.ni * BN;
    if (OP == OP_AGMM) {
        const int s = (rank + j) % p.world;
        tl.peer = s;
        tl.a_gathered = (j != 0);
        tl.a_row = tl.a_gathered ? s * p.M + tl.mi * BM : tl.mi * BM;
        tl.out_row = s * p.M + tl.mi * BM;
        tl.row_end = (s + 1) * p.M;
        tl.valid = true;
    } else {
        const int mr = rows_per_rank<OP>(p);
        const int d = (rank + 1 + j) % p.world;
        tl.peer = d;
        tl.a_gathered = false;
        tl.a_row = d * mr + tl.mi * BM;
        tl.out_row = tl.a_row;
        tl.row_end = min(p.M, (d + 1) * mr);
        tl.valid = tl.out_row < tl.row_end;
    }
    return tl;
}

#define CB_TRACE(slot, value)                                                     \
    do {                                                                          \
        if (p.trace) p.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + (slot)] = (value); \
    } while (0)

__device__ __forceinline__ uint32_t *flag_ptr(const FusedParams &p, int pe, uint32_t word) {
    return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + word;
}

template <int OP, typename T, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1) fused_gemm_kernel(const __grid_constant__ FusedParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + kStages * kAStageBytes;
    uint8_t *smem_push = smem + kStages * (kAStageBytes + kBStageBytes);
    GemmSmem *sh = reinterpret_cast<GemmSmem *>(smem_push + kSideSmemBytes);
    static_assert(sizeof(GemmSmem) <= 512, "barrier block outgrew its budget");
    static_assert(kPushLanes * kPushPieceBytes <= kStages * (kAStageBytes + kBStageBytes), "pusher staging");
    static_assert(BM * 256 <= kSideSmemBytes, "epilogue row staging");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const RankArgs &ra = p.ranks[lrank];
    const int num_tiles = R * tiles_per_peer<OP>(p);
    // AG-MM with peers: the last push_ctas CTAs do no GEMM; the others share the tiles
    const int gemm_ctas = p.ctas_per_rank - ((OP == OP_AGMM && R > 1 && !p.compute_only) ? p.push_ctas : 0);
    const bool is_pusher = cta >= gemm_ctas;
    const int kblocks = ceil_div(p.K, BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh->tmem_full[a], 1);
            mbar_init(&sh->tmem_empty[a], 4);
        }
        mbar_init(&sh->drain, 1);
        mbar_init(&sh->epi_bar, 128);
        for (int l = 0; l < kPushLanes; ++l) mbar_init(&sh->push_bar[l], 1);
        sh->abort_flag = 0;
        sh->epi_ok = 1;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
        if (OP == OP_AGMM) prefetch_tensormap(&ra.tmAg);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;

    const int mt_ag = ceil_div(p.M, BM);   // AG-MM: chunks per source rank
    if (threadIdx.x == 0) CB_TRACE(TR_START, globaltimer_ns());

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            uint64_t prod_wait_ns = 0;
            for (int t = cta; t < num_tiles && ok && !is_pusher; t += gemm_ctas) {
                const Tile tl = decode_tile<OP>(p, rank, t);
                if (!tl.valid) continue;
                if (OP == OP_AGMM && tl.a_gathered && !p.compute_only) {
                    // rows of this tile were pushed by rank tl.peer as kAgSubChunks units
                    const uint32_t w = kFlagOpBase + (tl.peer * mt_ag + tl.mi) * kAgSubChunks;
                    const uint64_t tw0 = p.trace ? globaltimer_ns() : 0;
                    for (int q = 0; q < kAgSubChunks && ok; ++q)
                        ok = wait_flag_ge(flag_ptr(p, rank, w + q), p.epoch, ctl, W_AG_CHUNK, w + q);
                    if (!ok) break;
                    fence_proxy_async();
                    if (p.trace) {
                        if (prod_wait_ns == 0) CB_TRACE(TR_PROD_WAIT_FIRST, tw0);
                        prod_wait_ns += globaltimer_ns() - tw0 + 1;
                    }
                }
                const CUtensorMap *tma = (OP == OP_AGMM && tl.a_gathered) ? &ra.tmAg : &ra.tmA;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[s], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    mbar_expect_tx(&sh->full[s], kAStageBytes + kBStageBytes);
                    tma_load_2d(smem_a + s * kAStageBytes, tma, &sh->full[s], kb * BK, tl.a_row);
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(smem_b + s * kBStageBytes + j * (64 * BK * 2), &ra.tmB, &sh->full[s],
                                        tl.n0 + j * 64, kb * BK);
                    } else {
                        tma_load_2d(smem_b + s * kBStageBytes, &ra.tmB, &sh->full[s], kb * BK, tl.n0);
                    }
                }
            }
            CB_TRACE(TR_PROD_WAIT_NS, prod_wait_ns);
            if (!ok) {
                // Aborting: loads already issued still land in shared memory; wait for them (bounded).
                for (uint32_t back = 1; back <= kStages && back <= it; ++back) {
                    const uint32_t i2 = it - back;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(&sh->full[i2 % kStages], (i2 / kStages) & 1)) {
                        if (globaltimer_ns() - t0 > 2000000ull) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t idesc = make_idesc_f16(fmt, BM, BN, 0, B_MN ? 1 : 0);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            uint64_t mma_wait_tmem = 0, mma_wait_smem = 0;
            for (int t = cta; t < num_tiles && ok && !is_pusher; t += gemm_ctas) {
                const Tile tl = decode_tile<OP>(p, rank, t);
                if (!tl.valid) continue;
                const uint32_t acc = tcount & 1;
                const uint64_t tm0 = p.trace ? globaltimer_ns() : 0;
                if (!(ok = mbar_wait(&sh->tmem_empty[acc], ((tcount >> 1) & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                if (p.trace) mma_wait_tmem += globaltimer_ns() - tm0;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint64_t ts0 = p.trace ? globaltimer_ns() : 0;
                    if (!(ok = mbar_wait(&sh->full[s], (it / kStages) & 1, ctl, W_MBAR_FULL))) break;
                    if (p.trace) mma_wait_smem += globaltimer_ns() - ts0;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + s * kAStageBytes);
                    const uint32_t b_addr = smem_u32(smem_b + s * kBStageBytes);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // A: K-major, 128B swizzle: 8-row groups 1024 B apart, 16 K-elements = 32 B.
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                        // B K-major: same shape.  B MN-major: 64-column chunks 64*BK*2 B apart,
                        // 8-row (K) groups 1024 B apart, 16 K-rows = 2048 B.
                        const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 2048, 64 * BK * 2, 1024)
                                                 : make_smem_desc(b_addr + k * 32, 16, 1024);
                        umma_f16(d_tmem, ad, bd, idesc, (kb | k) != 0);
                    }
                    umma_commit(&sh->empty[s]);
                }
                if (!ok) break;
                umma_commit(&sh->tmem_full[acc]);
                ++tcount;
            }
            CB_TRACE(TR_MMA_WAIT_TMEM_NS, mma_wait_tmem);
            CB_TRACE(TR_MMA_WAIT_SMEM_NS, mma_wait_smem);
            CB_TRACE(TR_TILES, tcount);
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
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int etid = (warp - 2) * 32 + lane;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        uint32_t entered_ok = 0;                // bitmap of peers known to have entered this epoch
        bool ok = true;
        GroupSync epi{&sh->epi_bar, 0};
        uint64_t epi_wait_ns = 0, epi_store_ns = 0;
        const int mr = (OP == OP_AGMM) ? 0 : rows_per_rank<OP>(p);
        const int per = tiles_per_peer<OP>(p);
        T *const C = reinterpret_cast<T *>(ra.C);
        for (int t = cta; t < num_tiles && ok && !is_pusher; t += gemm_ctas) {
            const Tile tl = decode_tile<OP>(p, rank, t);
            if (!tl.valid) continue;
            const uint32_t acc = tcount & 1;
            if (!(ok = mbar_wait(&sh->tmem_full[acc], (tcount >> 1) & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const int row = tl.out_row + row_in_tile;
            const bool row_ok = row < tl.row_end;
            const int tile_in_peer = tl.mi * ceil_div(p.N, BN) + tl.ni;
            const bool remote = (OP != OP_AGMM) && (tl.peer != rank);

            // Waits on peers are done by one thread; the group then meets on a bounded barrier.
            const bool need_pre =
                (OP != OP_AGMM) && R > 1 && !p.compute_only && (remote ? !((entered_ok >> tl.peer) & 1) : true);
            if (need_pre) {
                const uint64_t tp0 = p.trace ? globaltimer_ns() : 0;
                if (etid == 0) {
                    bool w = true;
                    if (remote) {
                        // the owner must have entered this epoch before its staging rows are overwritten
                        w = wait_flag_ge(flag_ptr(p, rank, kFlagEntered + tl.peer), p.entered_need, ctl, W_ENTERED, tl.peer);
                    } else {
                        // own rows: every peer's partial of this tile must have landed in my staging rows
                        for (int s = 0; s < R && w; ++s) {
                            if (s == rank) continue;
                            const uint32_t wd = kFlagOpBase + s * per + tile_in_peer;
                            w = wait_flag_ge(flag_ptr(p, rank, wd), p.epoch, ctl, W_RS_PARTIAL, wd);
                        }
                    }
                    if (!w) *reinterpret_cast<volatile int *>(&sh->epi_ok) = 0;
                }
                if (!(ok = epi.sync(ctl))) break;
                if (!(ok = (*reinterpret_cast<volatile int *>(&sh->epi_ok) != 0))) break;
                if (remote) entered_ok |= 1u << tl.peer;
                if (p.trace) epi_wait_ns += globaltimer_ns() - tp0;
            }

            T *dst_row = nullptr;        // where this thread's row of the tile goes
            if (OP == OP_AGMM) {
                dst_row = C + static_cast<size_t>(row) * p.N;
            } else if (remote) {
                // partial tile -> owner's staging rows [src = rank][row inside the owner's block]
                // (compute-only measurement: same stores, but into this rank's own staging rows)
                T *stage = reinterpret_cast<T *>(p.heap_base[p.compute_only ? rank : tl.peer] + p.symm_off);
                dst_row = stage + (static_cast<size_t>(rank) * mr + (row - tl.peer * mr)) * p.N;
            } else {
                dst_row = (OP == OP_MMRS) ? C + static_cast<size_t>(row - rank * mr) * p.N
                                          : C + static_cast<size_t>(row) * p.N;
            }
            const T *my_stage = (OP != OP_AGMM) ? reinterpret_cast<const T *>(p.heap_base[rank] + p.symm_off) : nullptr;

            // MM-RS / MM-AR: every output row segment (128 columns = 256 B) is staged in this thread's
            // private shared-memory row and leaves as one bulk copy, so that a peer receives full
            // 128-byte lines instead of 16-byte fragments.  AG-MM writes its (local) rows directly.
            constexpr bool kStaged = (OP != OP_AGMM);
            uint8_t *my_row_smem = smem_push + row_in_tile * 256;
            const uint64_t te0 = p.trace ? globaltimer_ns() : 0;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                if (kStaged && (c & 3) == 0) bulk_wait_read<0>();   // my staging row is free again
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                const int col = tl.n0 + c * 32;
                const bool live = row_ok && col < p.N;
                const bool reduce = (OP != OP_AGMM) && !remote && R > 1 && live;
                // own rows: fetch every peer's partial of this chunk while the accumulator is on its way
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
                if (!kStaged && !live) continue;
                float f[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
                if (reduce) {
                    // fixed summation order (own fp32 accumulator, then the peers' partials by rank):
                    // every output element has one owner, so results are reproducible run to run
#pragma unroll
                    for (int s = 0; s < kMaxRanks; ++s) {
                        if (s < R && s != rank) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                const uint32_t w4[4] = {part[s][g].x, part[s][g].y, part[s][g].z, part[s][g].w};
#pragma unroll
                                for (int h = 0; h < 4; ++h) {
                                    const float2 x = Pack2<T>::unpack(w4[h]);
                                    f[g * 8 + h * 2] += x.x;
                                    f[g * 8 + h * 2 + 1] += x.y;
                                }
                            }
                        }
                    }
                }
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[i] = Pack2<T>::pack(f[2 * i], f[2 * i + 1]);
                if (!kStaged) {
#pragma unroll
                    for (int g = 0; g < 4; ++g)
                        if (col + g * 8 < p.N)
                            *reinterpret_cast<uint4 *>(dst_row + col + g * 8) =
                                make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                } else {
#pragma unroll
                    for (int g = 0; g < 4; ++g)
                        *reinterpret_cast<uint4 *>(my_row_smem + (c & 3) * 64 + g * 16) =
                            make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                    if ((c & 3) == 3) {
                        fence_proxy_async();    // my shared-memory writes -> visible to the copy engine
                        const int colh = tl.n0 + (c >> 2) * 128;
                        if (row_ok && colh < p.N) {
                            const uint32_t len = static_cast<uint32_t>(min(128, p.N - colh)) * sizeof(T);
                            bulk_store(dst_row + colh, my_row_smem, len);
                            if (OP == OP_MMAR && !remote && R > 1 && !p.compute_only) {
                                // reduced rows -> every peer's "final" rows (second half of the symmetric region)
                                const size_t final_off = static_cast<size_t>(R) * mr * p.N;
                                for (int jj = 1; jj < R; ++jj) {
                                    const int d = (rank + jj) % R;
                                    T *fin = reinterpret_cast<T *>(p.heap_base[d] + p.symm_off) + final_off +
                                             static_cast<size_t>(row) * p.N + colh;
                                    bulk_store(fin, my_row_smem, len);
                                }
                            }
                            bulk_commit();
                        }
                    }
                }
            }
            if (p.trace) epi_store_ns += globaltimer_ns() - te0;
            // accumulator drained: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);

            if (OP != OP_AGMM && R > 1 && !p.compute_only && (remote || OP == OP_MMAR)) {
                // every thread's rows have been written to the peer(s) -> one thread publishes the tile
                bulk_wait<0>();
                fence_proxy_async();
                if (!(ok = epi.sync(ctl))) break;
                if (etid == 0) {
                    fence_sys();
                    if (remote) {
                        st_release_sys(flag_ptr(p, tl.peer, kFlagOpBase + rank * per + tile_in_peer), p.epoch);
                    } else {
                        // reduced tile now sits in every peer's final rows (each peer has entered the
                        // epoch: its partial of this tile was waited for above)
                        for (int jj = 1; jj < R; ++jj) {
                            const int d = (rank + jj) % R;
                            st_release_sys(flag_ptr(p, d, kFlagOpBase + (R + rank) * per + tile_in_peer), p.epoch);
                        }
                    }
                }
            }
            ++tcount;
        }

        if (OP != OP_AGMM) bulk_wait<0>();     // my staging row must outlive the copies that read it
        if (etid == 0) {
            CB_TRACE(TR_EPI_WAIT_NS, epi_wait_ns);
            CB_TRACE(TR_EPI_STORE_NS, epi_store_ns);
        }
        if (OP == OP_MMAR && R > 1 && ok && !p.compute_only) {
            // second phase: copy the peers' reduced tiles from my "final" rows into D
            const int mrr = rows_per_rank<OP>(p);
            const int nt = ceil_div(p.N, BN);
            const size_t final_off = static_cast<size_t>(R) * mrr * p.N;
            const T *fin = reinterpret_cast<const T *>(p.heap_base[rank] + p.symm_off) + final_off;
            const int total = (R - 1) * per;
            for (int u = cta; u < total && ok; u += p.ctas_per_rank) {
                const int o = (rank + 1 + u / per) % R;       // owner whose tile this is
                const int tip = u % per;
                const int mi = tip / nt, ni = tip % nt;
                const int r0 = o * mrr + mi * BM;
                const int r1 = min(min(p.M, (o + 1) * mrr), r0 + BM);
                if (r0 >= r1) continue;
                const uint32_t w = kFlagOpBase + (R + o) * per + tip;
                if (!(ok = wait_flag_ge(flag_ptr(p, rank, w), p.epoch, ctl, W_AR_FINAL, w))) break;
                const int c0 = ni * BN;
                const int c1 = min(p.N, c0 + BN);
                const int vec_per_row = (c1 - c0) / 8;        // N % 8 == 0 is required by the host checks
                for (int i = etid; i < (r1 - r0) * vec_per_row; i += 128) {
                    const int rr = r0 + i / vec_per_row;
                    const int cc = c0 + (i % vec_per_row) * 8;
                    const size_t off = static_cast<size_t>(rr) * p.N + cc;
                    *reinterpret_cast<uint4 *>(C + off) = *reinterpret_cast<const uint4 *>(fin + off);
                }
            }
        }
    } else {
        // ------------------------------------------------------------- comm warps ----
        const int ctid = (warp - 6) * 32 + lane;     // 0..63
        if (R > 1 && !p.compute_only) {
            if (cta == 0 && ctid < R && ctid != rank) {
                // tell every peer that this rank has entered the epoch: its symmetric data region
                // may now be overwritten
                fence_sys();
                st_release_sys(flag_ptr(p, ctid, kFlagEntered + rank), p.epoch);
            }
            const bool dedicated = p.push_ctas > 0;
            const int my_lanes = dedicated ? kPushLanes : kPushLanesShared;
            if (OP == OP_AGMM && (is_pusher || !dedicated) && ctid < my_lanes) {
                // All-gather push: my rows go into every peer's gathered region with bulk copies
                // (global -> shared -> peer global), destination rank-1 first (it consumes my rows
                // first), in units of BM/kAgSubChunks rows with one flag per unit.  Every pushing
                // thread ("lane") owns a kPushPieceBytes staging piece and whole units, so a unit's flag
                // has a single writer.  Default: each GEMM CTA pushes with kPushLanesShared lanes of its
                // comm warp (staging next to the GEMM stages); optionally a few CTAs are dedicated to
                // pushing with kPushLanes lanes each (the GEMM stage area is free there).  (This one-CTA
                // kernel is the fallback; the pair kernel gives every lane a warp of its own.)
                const int units_per_dest = mt_ag * kAgSubChunks;
                const int total = (R - 1) * units_per_dest;
                const size_t row_bytes = static_cast<size_t>(p.K) * sizeof(T);
                const int lane_id = (dedicated ? (cta - gemm_ctas) : cta) * my_lanes + ctid;
                const int n_lanes = (dedicated ? p.push_ctas : p.ctas_per_rank) * my_lanes;
                uint8_t *buf = (dedicated ? smem : smem_push) + ctid * kPushPieceBytes;
                uint64_t *bar = &sh->push_bar[ctid];
                bool ok = true;
                uint32_t entered_ok = 0;
                uint32_t piece = 0;
                if (ctid == 0) CB_TRACE(TR_PUSH_BEGIN, globaltimer_ns());
                for (int u = lane_id; u < total && ok; u += n_lanes) {
                    const int jj = u / units_per_dest;              // 0 -> rank-1, 1 -> rank-2, ...
                    const int d = (rank + R - 1 - jj) % R;
                    const int cu = u - jj * units_per_dest;
                    const int chunk = cu / kAgSubChunks, sub = cu % kAgSubChunks;
                    const int r0 = chunk * BM + sub * (BM / kAgSubChunks);
                    const int r1 = min(p.M, r0 + BM / kAgSubChunks);
                    if (!((entered_ok >> d) & 1)) {
                        if (!(ok = wait_flag_ge(flag_ptr(p, rank, kFlagEntered + d), p.entered_need, ctl, W_ENTERED, d)))
                            break;
                        entered_ok |= 1u << d;
                    }
                    if (r1 > r0) {
                        const uint8_t *src = static_cast<const uint8_t *>(ra.A) + r0 * row_bytes;
                        uint8_t *dst = p.heap_base[d] + p.symm_off + (static_cast<size_t>(rank) * p.M + r0) * row_bytes;
                        const size_t bytes = (r1 - r0) * row_bytes;
                        for (size_t off = 0; off < bytes && ok; off += kPushPieceBytes, ++piece) {
                            const uint32_t len = static_cast<uint32_t>(min(static_cast<size_t>(kPushPieceBytes), bytes - off));
                            bulk_wait_read<0>();     // my previous store has read the piece
                            mbar_expect_tx(bar, len);
                            bulk_load(buf, src + off, len, bar);
                            if (!(ok = mbar_wait(bar, piece & 1, ctl, W_DRAIN))) break;
                            bulk_store(dst + off, buf, len);
                            bulk_commit();
                        }
                    }
                    if (!ok) break;
                    bulk_wait<0>();          // every piece of the unit has been written to the peer
                    fence_proxy_async();
                    fence_sys();
                    st_release_sys(flag_ptr(p, d, kFlagOpBase + (rank * mt_ag + chunk) * kAgSubChunks + sub), p.epoch);
                }
                bulk_wait<0>();
                if (ctid == 0) CB_TRACE(TR_PUSH_END, globaltimer_ns());
            }
        }
    }

    // ------------------------------------------------------------------ teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0) CB_TRACE(TR_END, globaltimer_ns());
}

}  // namespace cb
