// Grouped (ragged-M) block-scaled MXFP8 GEMM for the MoE expert FFN (sm_100a).
//
// One persistent CTA per SM walks the tiles of all local experts; an expert's rows start on a
// multiple of 128 in the receive buffer, so every 128-row tile belongs to one expert and maps to
// whole scale-factor atoms.  Both operands are K-major e4m3 with UE8M0 scales per 32 along K.
//   MODE 1 (up projection): B tile = 128 "act" rows + 128 "gate" rows of the expert's [N, K] weight
//     (rows j and N/2 + j), so one accumulator holds both halves of 128 output columns; the
//     epilogue rounds both to bf16, applies y = bf16(act * sigmoid(act) * gate) in fp32 and
//     MX-quantises y (one 32-block per accumulator chunk) into the activation buffer of the
//     down projection, scales written straight in atom layout.
//   MODE 2 (down projection): plain 128 x 256 tile; every output row is written as bf16 into the
//     combine buffer of the rank the token came from, at the row's position in that rank's
//     expert-sorted order (bulk copies of 128-byte row pieces staged in shared memory).
// Reference: include/catccos/dgemm/kernel/ascend950_alltoall_gmm.hpp:57-506,
// examples/aux_ops/ascend950_swiglu_from_ub.h:214-394, include/catccos/dgemm/kernel/ascend950_gmm_alltoall.hpp:104-486;
// golden examples/utils/gen_data_moe.py:546-588.
#pragma once
#include <cuda_fp8.h>

#include "moe_common.h"
#include "mx_gemm.cuh"

namespace cb {

constexpr int kMoeStageBytes = kMxAStage + kMxBStage + kMxSfStage;     // 50 KiB
constexpr int kMoeStages = 4;
constexpr int kMoeSideBytes = 16 * 1024;                               // MODE 2: 128 rows x 128 B staging
constexpr int kMoeSmemBytes = kMoeStages * kMoeStageBytes + kMoeSideBytes + 1024 + 512;

struct alignas(64) MoeGemmRankArgs {
    CUtensorMap tmA;          // activations [rows_cap, Kin] bytes, box {128, 128}
    CUtensorMap tmB;          // weights [E_local * Nw, Kin] bytes, box {128, 128}
    const uint8_t *sfa;       // activation scale atoms [rows_cap/128][Kin/128][512]
    const uint8_t *sfb;       // weight scale atoms [E_local*Nw/128][Kin/128][512]
    uint8_t *act_codes;       // MODE 1 out: [rows_cap, Nw/2]
    uint8_t *act_sf;          // MODE 1 out: atoms [rows_cap/128][(Nw/2)/128][512]
    MoeMeta *meta;
};

struct MoeGemmParams {
    MoeGemmRankArgs ranks[kMaxRanks];
    uint8_t *heap_base[kMaxRanks];
    uint64_t combine_off;      // MODE 2: bf16 [m*topK, Nw] combine buffer inside every heap
    int world, rank_base, n_local, ctas_per_rank;
    int Kin;                   // contraction length
    int Nw;                    // weight rows per expert (MODE 1: N = 2 * intermediate; MODE 2: hidden size)
    int experts, experts_per_rank;
    int counter_slot;          // which MoeMeta::done_counter this launch uses
    uint32_t epoch;
    uint64_t timeout_ns;
    int *status;
};

struct MoeGemmSmem {
    uint64_t full[kMoeStages];
    uint64_t empty[kMoeStages];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct MoeTile {
    int le;          // local expert
    int mi, ni;
    int row0;        // first receive row of the tile
    int rows;        // valid rows (1..128)
};

// linear tile id -> tile; `le_hint` only moves forward (tile ids grow inside a CTA)
__device__ __forceinline__ MoeTile moe_decode(const MoeMeta *meta, int EL, int n_tiles, int t, int &le_hint) {
    MoeTile tl;
    const int g = t / n_tiles;
    tl.ni = t - g * n_tiles;
    while (le_hint + 1 < EL && g >= meta->tile_prefix[le_hint + 1]) ++le_hint;
    tl.le = le_hint;
    tl.mi = g - meta->tile_prefix[le_hint];
    tl.row0 = meta->seg_base[le_hint] + tl.mi * BM;
    tl.rows = min(BM, meta->seg_rows[le_hint] - tl.mi * BM);
    return tl;
}

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1) moe_grouped_gemm_kernel(const __grid_constant__ MoeGemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_side = smem + kMoeStages * kMoeStageBytes;
    MoeGemmSmem *sh = reinterpret_cast<MoeGemmSmem *>(smem_side + kMoeSideBytes);
    static_assert(sizeof(MoeGemmSmem) <= 512, "barrier block outgrew its budget");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const int EL = p.experts_per_rank;
    const MoeGemmRankArgs &ra = p.ranks[lrank];
    const MoeMeta *meta = ra.meta;
    const int n_tiles = (MODE == 1) ? (p.Nw / 2) / 128 : p.Nw / BN;
    const int kblocks = (p.Kin + MX_BK - 1) / MX_BK;
    const bool skip_all = meta->overflow != 0;
    const int num_tiles = skip_all ? 0 : meta->tile_prefix[EL] * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMoeStages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 4);
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        mbar_init_fence();
        prefetch_tensormap(&ra.tmA);
        prefetch_tensormap(&ra.tmB);
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            int le_hint = 0;
            for (int t = cta; t < num_tiles && ok; t += p.ctas_per_rank) {
                const MoeTile tl = moe_decode(meta, EL, n_tiles, t, le_hint);
                int b_row0, b_row1;
                if (MODE == 1) {
                    b_row0 = tl.le * p.Nw + tl.ni * 128;
                    b_row1 = b_row0 + p.Nw / 2;
                } else {
                    b_row0 = tl.le * p.Nw + tl.ni * BN;
                    b_row1 = b_row0 + 128;
                }
                const uint8_t *sfa = ra.sfa + static_cast<size_t>(tl.row0 >> 7) * kblocks * 512;
                const uint8_t *sfb0 = ra.sfb + static_cast<size_t>(b_row0 >> 7) * kblocks * 512;
                const uint8_t *sfb1 = ra.sfb + static_cast<size_t>(b_row1 >> 7) * kblocks * 512;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kMoeStages;
                    const uint32_t ph = (it / kMoeStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    uint8_t *sa = smem + st * kMoeStageBytes;
                    uint8_t *sb = sa + kMxAStage;
                    uint8_t *ssf = sb + kMxBStage;
                    mbar_expect_tx(&sh->full[st], kMxAStage + kMxBStage + 1536);
                    tma_load_2d(sa, &ra.tmA, &sh->full[st], kb * MX_BK, tl.row0);
                    tma_load_2d(sb, &ra.tmB, &sh->full[st], kb * MX_BK, b_row0);
                    tma_load_2d(sb + 128 * MX_BK, &ra.tmB, &sh->full[st], kb * MX_BK, b_row1);
                    bulk_load(ssf, sfa + static_cast<size_t>(kb) * 512, 512, &sh->full[st]);
                    bulk_load(ssf + 512, sfb0 + static_cast<size_t>(kb) * 512, 512, &sh->full[st]);
                    bulk_load(ssf + 1024, sfb1 + static_cast<size_t>(kb) * 512, 512, &sh->full[st]);
                }
            }
            if (!ok) {
                for (uint32_t back = 1; back <= kMoeStages && back <= it; ++back) {
                    const uint32_t i2 = it - back;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(&sh->full[i2 % kMoeStages], (i2 / kMoeStages) & 1)) {
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
                    const int st = it % kMoeStages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kMoeStages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + st * kMoeStageBytes);
                    const uint32_t b_addr = a_addr + kMxAStage;
                    const uint32_t sf_addr = b_addr + kMxBStage;
                    const uint32_t tmem_sfa = tmem_sf0 + (it & 3u) * 16u;
                    const uint32_t tmem_sfb = tmem_sfa + 4;
                    tmem_cp_32x128b_warpx4(tmem_sfa, make_smem_desc_noswizzle(sf_addr, 16, 128));
                    tmem_cp_32x128b_warpx4(tmem_sfb, make_smem_desc_noswizzle(sf_addr + 512, 16, 128));
                    tmem_cp_32x128b_warpx4(tmem_sfb + 4, make_smem_desc_noswizzle(sf_addr + 1024, 16, 128));
#pragma unroll
                    for (int k = 0; k < MX_BK / 32; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
                        const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                        umma_mxf8(tmem_base, ad, bd, make_idesc_mxf8(BM, BN, k, k), tmem_sfa, tmem_sfb, (kb | k) != 0);
                    }
                    umma_commit(&sh->empty[st]);
                }
                if (!ok) break;
                umma_commit(&sh->tmem_full);
                ++tcount;
            }
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
        int le_hint = 0;
        for (int t = cta; t < num_tiles && ok; t += p.ctas_per_rank) {
            const MoeTile tl = moe_decode(meta, EL, n_tiles, t, le_hint);
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            const bool row_ok = row_in_tile < tl.rows;
            const int row = tl.row0 + row_in_tile;
            if (MODE == 1) {
                // Both halves leave TMEM at once, rounded to bf16 as the golden rounds the up projection, and the
                // accumulator is handed back before any of the SwiGLU / quantisation arithmetic: that arithmetic
                // (about as long as a tile's main loop on one warp per scheduler) then overlaps the next tile.
                uint32_t act[64], gate[64];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t pk2 = Pack2<__nv_bfloat16>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                        if (c < 4) act[c * 16 + i] = pk2; else gate[(c - 4) * 16 + i] = pk2;
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->tmem_empty);
                uint32_t scale_word = 0;
                const int half_n = p.Nw / 2;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
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
                    scale_word |= sb << (8 * c);
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
                        uint8_t *dst = ra.act_codes + static_cast<size_t>(row) * half_n + tl.ni * 128 + c * 32;
                        *reinterpret_cast<uint4 *>(dst) = make_uint4(code[0], code[1], code[2], code[3]);
                        *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(code[4], code[5], code[6], code[7]);
                    }
                }
                // the tile's 128 output columns are 4 k-blocks of the down projection = one atom column group;
                // rows past the expert's count get the neutral scale so that stale bytes never reach the MMA
                const int kb4_2 = (half_n + 127) / 128;
                uint8_t *sfdst = ra.act_sf + (static_cast<size_t>(row >> 7) * kb4_2 + tl.ni) * 512 + (row & 31) * 16 +
                                 ((row >> 5) & 3) * 4;
                *reinterpret_cast<uint32_t *>(sfdst) = row_ok ? scale_word : 0x7F7F7F7Fu;
            } else {
                uint32_t pk[BN / 2];
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[c * 16 + i] =
                            Pack2<__nv_bfloat16>::pack(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->tmem_empty);
                // which rank does this row go back to, and where in its expert-sorted order
                __nv_bfloat16 *dst = nullptr;
                if (row_ok) {
                    const int w = tl.mi * BM + row_in_tile;
                    int src = 0;
                    while (src + 1 < R && w >= meta->cum_src[src + 1][tl.le]) ++src;
                    const int e = rank * EL + tl.le;
                    const int drow = meta->prefix_all[src][e] + (w - meta->cum_src[src][tl.le]);
                    dst = reinterpret_cast<__nv_bfloat16 *>(p.heap_base[src] + p.combine_off) +
                          static_cast<size_t>(drow) * p.Nw + tl.ni * BN;
                }
                uint8_t *my_row = smem_side + row_in_tile * 128;
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    bulk_wait_read<0>();
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        *reinterpret_cast<uint4 *>(my_row + g * 16) = make_uint4(
                            pk[h * 32 + g * 4], pk[h * 32 + g * 4 + 1], pk[h * 32 + g * 4 + 2], pk[h * 32 + g * 4 + 3]);
                    fence_proxy_async_smem();
                    if (row_ok) {
                        bulk_store(dst + h * 64, my_row, 128);
                        bulk_commit();
                    }
                }
            }
            ++tcount;
        }
        if (MODE == 2) {
            bulk_wait<0>();
            fence_proxy_async_global();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
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
