// Grouped (ragged-M) block-scaled MXFP8 GEMM for the MoE expert FFN on CTA pairs (tcgen05 cta_group::2).
//
// A pair computes a 256-row x 256-column tile of ONE local expert: CTA c of the pair takes the
// expert's 128-row tile 2 * j + c (an expert's rows start on a multiple of 128 in the receive
// buffer; the second half of an expert's last pair tile may be empty and is then masked), its half
// of the expert's weight tile; four helper warps read the scale atoms of both operands from global
// memory and write them into TMEM with tcgen05.st, so they never enter shared memory or the MMA
// queue.  Per K-step an SM pulls 32 KiB from L2 instead of the 49.5 KiB of the one-CTA kernel
// (moe_gemm.cuh), and there is room for six pipeline stages.  Tiles are handed out dynamically (tile_queue.cuh)
// in expert order, so an expert with many rows is shared by all pairs and the pairs that finish
// early take what is left.
//   MODE 1 (up projection): the pair's B tile is 128 "act" rows (CTA 0) + 128 "gate" rows (CTA 1) of
//     the expert's [N, K] weight; every CTA's accumulator holds act | gate for its 128 rows, and the
//     epilogue applies y = bf16(act * sigmoid(act) * gate) and MX-quantises y (moe_gemm.cuh, MODE 1).
//   MODE 2 (down projection, and GroupedMatmul-AllToAllV): plain 256-wide tile; rows go back to their source
//     rank's combine buffer, at the row's position in that rank's expert-sorted order.
//   MODE 3 (AllToAllV-GroupedMatmul): plain 256-wide tile; rows are written to this rank's output in receive
//     order (local expert major, source rank minor) without the 128-row padding of the receive buffer.
// B_MN: the weights are [E_local, K, N] (K x N row-major per expert, the standalone operators' transB = 0)
// instead of [E_local * N, K]; they are read through a 3-D tensor map whose third coordinate is the expert.
// Reference: include/catccos/dgemm/kernel/ascend950_alltoall_gmm.hpp:57-506,
// include/catccos/dgemm/kernel/ascend950_gmm_alltoall.hpp:104-486; golden examples/utils/gen_data_moe.py:546-588.
#pragma once
#include <cuda_fp8.h>

#include "moe_common.h"
#include "moe_gemm.cuh"
#include "mx_pair.cuh"
#include "tile_queue.cuh"

namespace cb {

constexpr int kMoePStages = 6;
constexpr int kMoePStageBytes = kMxPA + kMxPB;                           // 32 KiB (scale factors go to TMEM directly)
constexpr int kMoePairThreads = 448;      // warp 0: producer (lane 0) and tile queue (lane 1), 1: MMA, 2-9: epilogue, 10-13: scale factors
constexpr int kMoePairSideBytes = 32 * 1024;   // MODE 2: 2 column halves x 128 rows x 128 B of row staging
constexpr int kMoePairSmemBytes = kMoePStages * kMoePStageBytes + kMoePairSideBytes + 1024 + 1024;   // + alignment + barrier block
static_assert(kMoePairSmemBytes <= 232448, "shared memory budget");

struct alignas(64) MoePairRankArgs {
    CUtensorMap tmA;          // activations [rows_cap, Kin] bytes, box {128, 128}
    CUtensorMap tmB;          // weights [E_local * Nw, Kin] bytes, box {128, 128};  B_MN: [E_local][Kin][Nw], box {128, 128, 1}
    const uint8_t *sfa;       // activation scale atoms [rows_cap/128][Kin/128][512]
    const uint8_t *sfb;       // weight scale atoms [E_local * ceil(Nw/128)][Kin/128][512]
    uint8_t *act_codes;       // MODE 1 out: [rows_cap, Nw/2]
    uint8_t *act_sf;          // MODE 1 out: atoms [rows_cap/128][(Nw/2)/128][512]
    void *out;                // MODE 3 out: 16-bit [rows, Nw]
    MoeMeta *meta;
};

struct MoePairParams {
    MoePairRankArgs ranks[kMaxRanks];
    uint8_t *heap_base[kMaxRanks];
    uint64_t combine_off;      // MODE 2: bf16 [m*topK, Nw] combine buffer inside every heap
    int world, rank_base, n_local, ctas_per_rank;      // ctas_per_rank is even
    int Kin, Nw;               // Kin: BYTES of one activation / weight row along the contraction
    int fp4;                   // 1: MXFP4 operands (two e2m1 codes per byte, K-major weights, two scale atoms per stage)
    int rows_cap;              // rows of the activation buffer (a multiple of 128)
    int experts, experts_per_rank;
    int counter_slot;          // MoeMeta::done_counter / tile_queue slot of this launch
    uint32_t epoch;
    uint64_t timeout_ns;
    int *status;
};

struct MoePairSmem {
    uint64_t full[kMoePStages];     // in the leader: both CTAs' loads landed
    uint64_t empty[kMoePStages];    // per CTA
    uint64_t tmem_full;             // per CTA
    uint64_t tmem_empty;            // in the leader: 8 epilogue warps of the pair
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    TileQueue tq;
    int pprefix[kMoeMaxLocalExperts + 1];    // exclusive prefix of pair tiles (256 rows) over the local experts
    int uprefix[kMoeMaxLocalExperts + 1];    // exclusive prefix of received rows (no padding) over the local experts
};

struct MoePairTile {
    int le;          // local expert
    int ni;          // column tile
    int row0;        // first receive row of THIS CTA's 128 rows
    int rows;        // valid rows of this CTA's half (0..128)
    int mi;          // this CTA's 128-row tile inside the expert
};

template <int MODE, typename TOut, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMoePairThreads, 1)
    moe_pair_gemm_kernel(const __grid_constant__ MoePairParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem_a + kMoePStages * kMxPA;
    uint8_t *smem_side = smem_b + kMoePStages * kMxPB;
    MoePairSmem *sh = reinterpret_cast<MoePairSmem *>(smem_side + kMoePairSideBytes);
    static_assert(sizeof(MoePairSmem) <= 1024, "barrier block outgrew its budget");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int pair = cta >> 1, pairs = p.ctas_per_rank >> 1;
    const uint32_t cr = cluster_ctarank();
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const int EL = p.experts_per_rank;
    const MoePairRankArgs &ra = p.ranks[lrank];
    MoeMeta *meta = ra.meta;
    const int n_tiles = (MODE == 1) ? (p.Nw / 2) / 128 : (p.Nw + BN - 1) / BN;
    const int nb128 = (p.Nw + 127) / 128;          // weight scale atoms (128 weight rows each) per expert
    const int kblocks = (p.Kin + MX_BK - 1) / MX_BK;          // pipeline stages per tile (128 bytes of K each)
    const int katoms = p.fp4 ? 2 * kblocks : kblocks;          // scale atoms per 128-row tile (one per 128 elements of K)
    constexpr uint32_t kSfCols = 24;                           // TMEM scale columns per stage: MXFP8 uses 12, MXFP4 24
    const bool skip_all = meta->overflow != 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMoePStages; ++s) {
            mbar_init(&sh->full[s], 2 + 8);      // two producers (with their bytes) + the pair's eight scale-factor warps
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 16);         // eight epilogue warps in each CTA of the pair
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        tq_init(&sh->tq);
        int run = 0, rows = 0;
        for (int le = 0; le < EL; ++le) {
            sh->pprefix[le] = run;
            sh->uprefix[le] = rows;
            run += (meta->tile_prefix[le + 1] - meta->tile_prefix[le] + 1) / 2;
            rows += meta->seg_rows[le];
        }
        sh->pprefix[EL] = skip_all ? 0 : run;
        sh->uprefix[EL] = rows;
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
    const uint32_t tmem_sf0 = tmem_base + BN;      // 4 (A) + 8 (B) scale columns per pipeline stage, written by warps 8-11
    const int num_tiles = sh->pprefix[EL] * n_tiles;

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;

    // linear pair-tile id -> this CTA's part of the tile; ids grow inside a pair, so `le_hint` only moves forward
    auto decode = [&](int t, int &le_hint) {
        MoePairTile tl;
        const int g = t / n_tiles;
        tl.ni = t - g * n_tiles;
        while (le_hint + 1 < EL && g >= sh->pprefix[le_hint + 1]) ++le_hint;
        tl.le = le_hint;
        tl.mi = (g - sh->pprefix[le_hint]) * 2 + static_cast<int>(cr);
        tl.row0 = meta->seg_base[le_hint] + tl.mi * BM;
        tl.rows = max(0, min(BM, meta->seg_rows[le_hint] - tl.mi * BM));
        return tl;
    };

    if (warp == 0) {
        // --------------------------------------- tile queue (leader, lane 1) ----
        if (lane == 1 && cr == 0) {
            int *const counters = meta->tile_queue[p.counter_slot & 1];
            bool ok = true;
            for (uint32_t seq = 0; ok; ++seq) {
                uint32_t tq;
                if (!(ok = tq_claim(&sh->tq, seq, pair, pairs, num_tiles, counters, ctl, tq)) || tq == kTileEnd) break;
            }
            if (!ok) tq_publish_end(&sh->tq);
        }
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int le_hint = 0;
            for (uint32_t seq = 0; ok; ++seq) {
                uint32_t tq;
                if (!(ok = tq_get(&sh->tq, seq, tq, ctl)) || tq == kTileEnd) break;
                const MoePairTile tl = decode(static_cast<int>(tq), le_hint);
                // the two 128-wide halves of the pair's weight tile (columns inside the expert); this CTA loads one
                // of them, and the scale atoms of both
                int n0, n1;
                if (MODE == 1) {
                    n0 = tl.ni * 128;                 // act rows
                    n1 = n0 + p.Nw / 2;               // gate rows
                } else {
                    n0 = tl.ni * BN;
                    n1 = n0 + 128;
                }
                const int n_mine = cr == 0 ? n0 : n1;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMoePStages;
                    const uint32_t ph = (it / kMoePStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    mbar_expect_tx_cluster(full_leader, kMxPA + kMxPB);
                    tma_load_2d_pair(smem_a + st * kMxPA, &ra.tmA, full_leader, kb * MX_BK, tl.row0);
                    if (B_MN)
                        tma_load_3d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, n_mine, kb * MX_BK, tl.le);
                    else
                        tma_load_2d_pair(smem_b + st * kMxPB, &ra.tmB, full_leader, kb * MX_BK, tl.le * p.Nw + n_mine);
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
            for (;;) {
                uint32_t tq;
                if (!(ok = tq_get(&sh->tq, tcount, tq, ctl)) || tq == kTileEnd) break;
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMoePStages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kMoePStages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + st * kMxPA);
                    const uint32_t b_addr = smem_u32(smem_b + st * kMxPB);
                    const uint32_t tmem_sfa = tmem_sf0 + static_cast<uint32_t>(st) * kSfCols;
                    if (!B_MN && p.fp4) {
                        // MXFP4: four MMAs of K = 64; atom a = k / 2 of the stage: A at +4a, B at +8 + 8a (two 128-column halves)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
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
            if (!ok) {
                umma_commit_pair(mapa_cluster(smem_u32(&sh->drain), 0));
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(&sh->drain, 0)) {
                    if (globaltimer_ns() - t0 > 2000000ull) break;
                }
            }
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------------- epilogue ----
        // Eight warps: warp w drains TMEM lane quarter w % 4 (32 rows) and column half (w - 2) / 4 of the
        // accumulator, so a row's epilogue arithmetic is shared by two warps on different schedulers.
        const int q = warp & 3;
        const int ch = (warp - 2) >> 2;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        bool ok = true;
        int le_hint = 0;
        for (;;) {
            uint32_t tq;
            if (!(ok = tq_get(&sh->tq, tcount, tq, ctl)) || tq == kTileEnd) break;
            const MoePairTile tl = decode(static_cast<int>(tq), le_hint);
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const bool row_ok = row_in_tile < tl.rows;
            const int row = tl.row0 + row_in_tile;
            const uint32_t lane_field = static_cast<uint32_t>(q * 32) << 16;
            if (MODE == 1) {
                // This warp's 64 act columns and the 64 gate columns that go with them leave TMEM at once, rounded
                // to bf16 as the golden rounds the up projection, and the accumulator is handed back before any of
                // the SwiGLU / quantisation arithmetic, which then overlaps the next tile's main loop.
                uint32_t act[32], gate[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    const int col = (c < 2) ? ch * 64 + c * 32 : 128 + ch * 64 + (c - 2) * 32;
                    tmem_ld_32x32(tmem_base + col + lane_field, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t pk2 = Pack2<__nv_bfloat16>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                        if (c < 2) act[c * 16 + i] = pk2; else gate[(c - 2) * 16 + i] = pk2;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty), 0));
                uint32_t scale_half = 0;
                const int half_n = p.Nw / 2;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t ypk[16];            // y rounded to bf16, two per word
                    uint32_t am = 0;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 a2 = Pack2<__nv_bfloat16>::unpack(act[c * 16 + i]);
                        const float2 g2 = Pack2<__nv_bfloat16>::unpack(gate[c * 16 + i]);
                        // act * sigmoid(act) * gate; exp and reciprocal through the special-function unit
                        const float y0 = a2.x * __frcp_rn(1.0f + __expf(-a2.x)) * g2.x;
                        const float y1 = a2.y * __frcp_rn(1.0f + __expf(-a2.y)) * g2.y;
                        ypk[i] = Pack2<__nv_bfloat16>::pack(y0, y1);
                        am = max(am, max(ypk[i] & 0x7FFFu, (ypk[i] >> 16) & 0x7FFFu));
                    }
                    const float amax = __uint_as_float(am << 16);
                    uint32_t sb = 127u;
                    float inv = 1.0f;
                    if (!(amax < 1e-12f)) {
                        const uint32_t e8 = (am >> 7) & 0xFFu;
                        sb = e8 - 8u;
                        inv = __uint_as_float((262u - e8) << 23);
                    }
                    scale_half |= sb << (8 * c);
                    uint32_t code[8];
                    if (am <= 0x7F80u) {
                        // no NaN in the chunk: two values per conversion
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 ya = Pack2<__nv_bfloat16>::unpack(ypk[2 * i]), yb = Pack2<__nv_bfloat16>::unpack(ypk[2 * i + 1]);
                            const uint32_t lo = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(
                                make_float2(ya.x * inv, ya.y * inv), __NV_SATFINITE, __NV_E4M3));
                            const uint32_t hi = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(
                                make_float2(yb.x * inv, yb.y * inv), __NV_SATFINITE, __NV_E4M3));
                            code[i] = lo | (hi << 16);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            uint32_t w = 0;
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const float2 yv = Pack2<__nv_bfloat16>::unpack(ypk[2 * i + (b >> 1)]);
                                const float x = ((b & 1) ? yv.y : yv.x) * inv;
                                const uint32_t cb8 = (x != x) ? (0x7Fu | ((__float_as_uint(x) >> 24) & 0x80u))
                                                              : static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
                                w |= cb8 << (8 * b);
                            }
                            code[i] = w;
                        }
                    }
                    if (row_ok) {
                        uint8_t *dst = ra.act_codes + static_cast<size_t>(row) * half_n + tl.ni * 128 + ch * 64 + c * 32;
                        *reinterpret_cast<uint4 *>(dst) = make_uint4(code[0], code[1], code[2], code[3]);
                        *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(code[4], code[5], code[6], code[7]);
                    }
                }
                // the tile's 128 output columns are 4 k-blocks of the down projection = one 4-byte atom entry per row,
                // of which this warp owns two bytes; rows past the expert's count get the neutral scale so that stale
                // bytes never reach the MMA.  An empty half beyond the expert's last 128-row tile is left alone.
                if (tl.rows > 0) {
                    const int kb4_2 = (half_n + 127) / 128;
                    uint8_t *sfdst = ra.act_sf + (static_cast<size_t>(row >> 7) * kb4_2 + tl.ni) * 512 + (row & 31) * 16 +
                                     ((row >> 5) & 3) * 4 + ch * 2;
                    *reinterpret_cast<uint16_t *>(sfdst) = static_cast<uint16_t>(row_ok ? scale_half : 0x7F7Fu);
                }
            } else {
                // this warp's 128 columns, packed to the output type; then the accumulator goes back
                uint32_t pk[64];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + ch * 128 + c * 32 + lane_field, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[c * 16 + i] = Pack2<TOut>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty), 0));
                const int col0 = tl.ni * BN + ch * 128;
                const int w = tl.mi * BM + row_in_tile;              // row inside the expert
                if (MODE == 3) {
                    // receive order without padding: rows of the experts before this one, then w
                    if (row_ok) {
                        TOut *dst = static_cast<TOut *>(ra.out) + static_cast<size_t>(sh->uprefix[tl.le] + w) * p.Nw + col0;
#pragma unroll
                        for (int g = 0; g < 16; ++g)
                            if (col0 + g * 8 < p.Nw)
                                *reinterpret_cast<uint4 *>(dst + g * 8) =
                                    make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
                    }
                } else {
                    // which rank does this row go back to, and where in its expert-sorted order
                    TOut *dst = nullptr;
                    if (row_ok) {
                        int src = 0;
                        while (src + 1 < R && w >= meta->cum_src[src + 1][tl.le]) ++src;
                        const int e = rank * EL + tl.le;
                        const int drow = meta->prefix_all[src][e] + (w - meta->cum_src[src][tl.le]);
                        dst = reinterpret_cast<TOut *>(p.heap_base[src] + p.combine_off) + static_cast<size_t>(drow) * p.Nw + col0;
                    }
                    // 128-byte pieces of the row through this thread's own staging slot (one per column half)
                    uint8_t *my_row = smem_side + (ch * BM + row_in_tile) * 128;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        bulk_wait_read<0>();
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            *reinterpret_cast<uint4 *>(my_row + g * 16) = make_uint4(
                                pk[h * 32 + g * 4], pk[h * 32 + g * 4 + 1], pk[h * 32 + g * 4 + 2], pk[h * 32 + g * 4 + 3]);
                        fence_proxy_async_smem();
                        const int cols_left = p.Nw - (col0 + h * 64);        // Nw is a multiple of 8: whole 16-byte pieces
                        if (row_ok && cols_left > 0) {
                            bulk_store(dst + h * 64, my_row, static_cast<uint32_t>(min(64, cols_left)) * 2u);
                            bulk_commit();
                        }
                    }
                }
            }
            ++tcount;
            if (warp == 2 && lane == 0) tq_done(&sh->tq, cr, tcount);
        }
        if (MODE == 2) {
            bulk_wait<0>();
            fence_proxy_async_global();
        }
    } else {
        // ---------------------------------------------------------- scale factors ----
        // Warps 10-13 own TMEM lane quarters 2, 3, 0, 1 (a warp reaches the quarter warp % 4).  Per pipeline stage every lane reads its 16-byte row of the
        // activation atom and of the two weight atoms from global memory (512 contiguous bytes per atom: one
        // coalesced request per warp) and stores them into the stage's scale columns with tcgen05.st; the
        // stage's "full" barrier in the leader counts these eight warps of the pair next to the operand loads.
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint8_t *sfa_all = reinterpret_cast<const uint8_t *>(ra.sfa), *sfb_all = reinterpret_cast<const uint8_t *>(ra.sfb);
        uint32_t it = 0;
        bool ok = true;
        int le_hint = 0;
        for (uint32_t seq = 0; ok; ++seq) {
            uint32_t tq = 0;
            if (lane == 0) ok = tq_get(&sh->tq, seq, tq, ctl);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            tq = __shfl_sync(0xffffffffu, tq, 0);
            if (!ok || tq == kTileEnd) break;
            const MoePairTile tl = decode(static_cast<int>(tq), le_hint);
            int n0, n1;
            if (MODE == 1) {
                n0 = tl.ni * 128;
                n1 = n0 + p.Nw / 2;
            } else {
                n0 = tl.ni * BN;
                n1 = n0 + 128;
            }
            const uint8_t *sfa = sfa_all + static_cast<size_t>(tl.row0 >> 7) * katoms * 512 + lane * 16;
            const uint8_t *sfb0 = sfb_all + static_cast<size_t>(tl.le * nb128 + (n0 >> 7)) * katoms * 512 + lane * 16;
            const uint8_t *sfb1 = (n1 < p.Nw) ? sfb_all + static_cast<size_t>(tl.le * nb128 + (n1 >> 7)) * katoms * 512 + lane * 16 : sfb0;
            // an empty half past the receive buffer has no atoms of its own: any valid ones do (rows are masked)
            if (tl.row0 >= p.rows_cap) sfa = sfa_all + lane * 16;
            if (!B_MN && p.fp4) {
                // MXFP4: two atoms per operand tile and stage; the next stage's six rows are in flight
                uint4 cur[6], nxt[6];
                auto load6 = [&](uint4 (&v)[6], int kb) {
                    const size_t o = static_cast<size_t>(kb) * 1024;
                    v[0] = *reinterpret_cast<const uint4 *>(sfa + o);
                    v[1] = *reinterpret_cast<const uint4 *>(sfa + o + 512);
                    v[2] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + o));
                    v[3] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + o));
                    v[4] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + o + 512));
                    v[5] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + o + 512));
                };
                load6(nxt, 0);
                for (int kb = 0; kb < kblocks && ok; ++kb) {
#pragma unroll
                    for (int j = 0; j < 6; ++j) cur[j] = nxt[j];
                    load6(nxt, kb + 1 < kblocks ? kb + 1 : kb);
                    const int st = it % kMoePStages;
                    const uint32_t ph = (it / kMoePStages) & 1;
                    ++it;
                    if (lane == 0) ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t col = tmem_sf0 + static_cast<uint32_t>(st) * kSfCols + lane_field;
                    tmem_st_32x4(col, cur[0]);            // A, atom 0 and 1
                    tmem_st_32x4(col + 4, cur[1]);
                    tmem_st_32x4(col + 8, cur[2]);        // B atom 0: columns 0-127, 128-255
                    tmem_st_32x4(col + 12, cur[3]);
                    tmem_st_32x4(col + 16, cur[4]);       // B atom 1
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
                va[d] = *reinterpret_cast<const uint4 *>(sfa + static_cast<size_t>(kk) * 512);
                vb0[d] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + static_cast<size_t>(kk) * 512));
                vb1[d] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + static_cast<size_t>(kk) * 512));
            }
            for (int kb0 = 0; kb0 < kblocks && ok; kb0 += kSfAhead) {
#pragma unroll
                for (int d = 0; d < kSfAhead; ++d) {
                    const int kb = kb0 + d;
                    if (kb >= kblocks) break;
                    const int st = it % kMoePStages;
                    const uint32_t ph = (it / kMoePStages) & 1;
                    ++it;
                    const uint4 a = va[d], b0 = vb0[d], b1 = vb1[d];
                    {
                        const int kk = kb + kSfAhead < kblocks ? kb + kSfAhead : kblocks - 1;
                        va[d] = *reinterpret_cast<const uint4 *>(sfa + static_cast<size_t>(kk) * 512);
                        vb0[d] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + static_cast<size_t>(kk) * 512));
                        vb1[d] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + static_cast<size_t>(kk) * 512));
                    }
                    // the MMAs that read this stage's scale columns one round ago have finished
                    if (lane == 0) ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t col = tmem_sf0 + static_cast<uint32_t>(st) * kSfCols + lane_field;
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
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
    // MODE 2: the last CTA of this rank tells every rank that its combine rows are in place
    if (MODE == 2 && threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(&ra.meta->done_counter[p.counter_slot], 1u);
        if (prev == static_cast<unsigned>(p.ctas_per_rank) - 1u) {
            fence_sys();
            for (int r = 0; r < R; ++r)
                st_release_sys(reinterpret_cast<uint32_t *>(p.heap_base[r]) + kMoeFlagCombine + rank, p.epoch);
        }
    }
}

}  // namespace cb
