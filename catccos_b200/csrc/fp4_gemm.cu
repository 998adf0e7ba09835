// Block-scaled FP4 GEMM (sm_100a): C[m, n] = alpha * dequant(A)[m, k] x dequant(B)[n, k]^T.
//   NVFP4: e2m1 codes (two per byte), one UE4M3 scale per 16 along k, fp32 tensor scales folded into alpha;
//   MXFP4: e2m1 codes, one UE8M0 scale per 32 along k (the reference's FP4: examples/ascend950_fp4_mx_*,
//          golden examples/utils/gen_data_fp4_mx_allgather_matmul.py).
// Both operands K-major (B as [n, k], i.e. transB = 1; 4-bit operands have no MN-major form on tcgen05).
// A K-step of 128 bytes = 256 elements = four `tcgen05.mma.kind::mxf4nvf4.block_scale` of K = 64.  Scale factors
// travel as the same 512-byte atoms as MXFP8 (128 rows x 4 scale bytes); NVFP4 consumes one atom of A and two of B
// per MMA, MXFP4 half as many.  Two kernels: CTA pairs (default: 256 x 256 tiles, cta_group::2, scale factors
// written to TMEM by helper warps) and one persistent CTA per SM with 128 x 256 tiles (CATCCOS_TWO_CTA=0: scale
// atoms through shared memory and tcgen05.cp).  Single rank.
#include "fp4_gemm.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "common.h"
#include "mx_quant.h"
#include "ptx.cuh"

namespace cb {

namespace {

constexpr int kF4BK = 128;                      // bytes of K per stage (256 e2m1 elements)
constexpr int kF4A = BM * kF4BK;                // 16 KiB
constexpr int kF4B = BN * kF4BK;                // 32 KiB
constexpr int kF4Sf = 6 * 1024;                 // NVFP4: 4 atoms of A + 2 x 4 atoms of B; MXFP4 uses half
constexpr int kF4Stage = kF4A + kF4B + kF4Sf;   // 54 KiB
constexpr int kF4Stages = 4;
constexpr int kF4SmemBytes = kF4Stages * kF4Stage + 1024 + 512;
static_assert(kF4SmemBytes <= 232448, "shared memory budget");

struct Fp4Params {
    CUtensorMap tmA;          // [m, k/2] bytes, box {128, 128}
    CUtensorMap tmB;          // [n, k/2] bytes, box {128, 256 rows as 2 x 128}
    const uint8_t *sfa;       // scale atoms of A: [ceil(m/128)][atoms_per_row_tile][512]
    const uint8_t *sfb;       // scale atoms of B: [ceil(n/128)][atoms_per_row_tile][512]
    void *C;
    int M, N, K;              // K in elements
    int atoms_per_tile;       // scale atoms per 128-row tile = ceil(scales per row / 4)
    float alpha;
    uint64_t timeout_ns;
    int *status;
};

struct Fp4Smem {
    uint64_t full[kF4Stages];
    uint64_t empty[kF4Stages];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

template <typename TOut, bool NV>
__global__ void __launch_bounds__(kGemmThreads, 1) fp4_gemm_kernel(const __grid_constant__ Fp4Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Fp4Smem *sh = reinterpret_cast<Fp4Smem *>(smem + kF4Stages * kF4Stage);
    static_assert(sizeof(Fp4Smem) <= 512, "barrier block outgrew its budget");
    constexpr int kAtomsA = NV ? 4 : 2;           // atoms of A per K-step
    constexpr int kSfBytesA = kAtomsA * 512;
    constexpr int kSetCols = NV ? 48 : 24;        // TMEM columns of one set of scales: A atoms + 2 x B atoms, 4 columns each

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int mt = (p.M + BM - 1) / BM, nt = (p.N + BN - 1) / BN;
    const int num_tiles = mt * nt;
    const int kbytes = p.K / 2;
    const int kblocks = (kbytes + kF4BK - 1) / kF4BK;
    const int mmas_total = p.K / 64;              // K is a multiple of 64

    if (threadIdx.x == 0) {
        for (int s = 0; s < kF4Stages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 4);
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        mbar_init_fence();
        prefetch_tensormap(&p.tmA);
        prefetch_tensormap(&p.tmB);
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    const uint32_t tmem_sf0 = tmem_base + BN;     // two sets of scale columns, used in turn

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = 0;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int mi = t / nt, ni = t - mi * nt;
                const uint8_t *sfa = p.sfa + static_cast<size_t>(mi) * p.atoms_per_tile * 512;
                const uint8_t *sfb0 = p.sfb + static_cast<size_t>(ni * 2) * p.atoms_per_tile * 512;
                const uint8_t *sfb1 = sfb0 + static_cast<size_t>(p.atoms_per_tile) * 512;
                const bool second_b = (ni * BN + 128) < p.N;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kF4Stages;
                    const uint32_t ph = (it / kF4Stages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    uint8_t *sa = smem + st * kF4Stage;
                    uint8_t *sb = sa + kF4A;
                    uint8_t *ssf = sb + kF4B;
                    // the last K-step may hold fewer than four MMAs' worth of scales
                    const int atoms = min(kAtomsA, p.atoms_per_tile - kb * kAtomsA);
                    const uint32_t sf_bytes = static_cast<uint32_t>(atoms) * 512;
                    mbar_expect_tx(&sh->full[st], kF4A + kF4B + sf_bytes * (second_b ? 3 : 2));
                    tma_load_2d(sa, &p.tmA, &sh->full[st], kb * kF4BK, mi * BM);
                    tma_load_2d(sb, &p.tmB, &sh->full[st], kb * kF4BK, ni * BN);
                    tma_load_2d(sb + 128 * kF4BK, &p.tmB, &sh->full[st], kb * kF4BK, ni * BN + 128);
                    bulk_load(ssf, sfa + static_cast<size_t>(kb) * kSfBytesA, sf_bytes, &sh->full[st]);
                    bulk_load(ssf + kSfBytesA, sfb0 + static_cast<size_t>(kb) * kSfBytesA, sf_bytes, &sh->full[st]);
                    if (second_b)
                        bulk_load(ssf + 2 * kSfBytesA, sfb1 + static_cast<size_t>(kb) * kSfBytesA, sf_bytes, &sh->full[st]);
                }
            }
            if (!ok) {
                for (uint32_t back = 1; back <= kF4Stages && back <= it; ++back) {
                    const uint32_t i2 = it - back;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(&sh->full[i2 % kF4Stages], (i2 / kF4Stages) & 1)) {
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
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kF4Stages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kF4Stages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + st * kF4Stage);
                    const uint32_t b_addr = a_addr + kF4A;
                    const uint32_t sf_addr = b_addr + kF4B;
                    const uint32_t sfa_t = tmem_sf0 + (it & 1u) * kSetCols;          // kAtomsA atoms x 4 columns
                    const uint32_t sfb_t = sfa_t + kAtomsA * 4;                      // per atom index: 4 (n 0-127) + 4 (n 128-255)
                    const int mmas = min(4, mmas_total - kb * 4);
                    const int atoms = NV ? mmas : (mmas + 1) / 2;
                    for (int a = 0; a < atoms; ++a) {
                        tmem_cp_32x128b_warpx4(sfa_t + a * 4, make_smem_desc_noswizzle(sf_addr + a * 512, 16, 128));
                        tmem_cp_32x128b_warpx4(sfb_t + a * 8, make_smem_desc_noswizzle(sf_addr + kSfBytesA + a * 512, 16, 128));
                        tmem_cp_32x128b_warpx4(sfb_t + a * 8 + 4,
                                               make_smem_desc_noswizzle(sf_addr + 2 * kSfBytesA + a * 512, 16, 128));
                    }
                    for (int k = 0; k < mmas; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);   // 64 e2m1 = 32 bytes of a 128-byte row
                        const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                        const int atom = NV ? k : (k >> 1);
                        const uint32_t sf_id = NV ? 0u : static_cast<uint32_t>(k & 1) * 2u;
                        const uint32_t idesc = make_idesc_fp4(BM, BN, sf_id, sf_id, NV ? 0u : 1u);
                        umma_fp4<NV>(tmem_base, ad, bd, idesc, sfa_t + atom * 4, sfb_t + atom * 8, (kb | k) != 0);
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
        TOut *const C = reinterpret_cast<TOut *>(p.C);
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const int mi = t / nt, ni = t - mi * nt;
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            uint32_t pk[BN / 2];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[c * 16 + i] = Pack2<TOut>::pack(__uint_as_float(v[2 * i]) * p.alpha, __uint_as_float(v[2 * i + 1]) * p.alpha);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty);
            const int row = mi * BM + row_in_tile;
            if (row < p.M) {
                TOut *dst = C + static_cast<size_t>(row) * p.N + ni * BN;
#pragma unroll
                for (int g = 0; g < BN / 8; ++g)
                    if (ni * BN + g * 8 < p.N)
                        *reinterpret_cast<uint4 *>(dst + g * 8) =
                            make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
            }
            ++tcount;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ CTA pairs ----
// The same GEMM on CTA pairs (cluster of 2, tcgen05 cta_group::2): a pair computes a 256 x 256 tile, every CTA
// loads its own 128 rows of A, its own 128 columns of B, the scale atoms of its rows and of all 256 columns, and
// keeps the accumulator of its 128 rows in its own TMEM; the leader issues the M = 256 MMAs.  Per K-step an SM
// pulls 32 KiB of operands from L2 instead of 48 KiB.  The scale factors never enter shared memory or the MMA
// queue: four helper warps (one per TMEM lane quarter) read the 512-byte atoms from global memory and write them
// into a ring of TMEM columns with tcgen05.st (NVFP4 needs twelve atoms per K-step -- as tcgen05.cp in front of
// four MMAs they cost more than the MMAs).
constexpr int kF4PStages = 5;                   // also the depth of the scale ring: 256 + 5 x 48 TMEM columns
constexpr int kF4PA = 128 * kF4BK;              // 16 KiB: this CTA's rows of A
constexpr int kF4PB = 128 * kF4BK;              // 16 KiB: this CTA's columns of B
constexpr int kF4PStage = kF4PA + kF4PB;
constexpr int kF4PairThreads = 320;             // warp 0 TMA, 1 MMA, 2-5 epilogue, 6-9 scale factors
constexpr int kF4PSmemBytes = kF4PStages * kF4PStage + 1024 + 512;
static_assert(kF4PSmemBytes <= 232448, "shared memory budget");

struct Fp4PairParams {
    CUtensorMap tmA;          // [m, k/2] bytes, box {128, 128}
    CUtensorMap tmB;          // [n, k/2] bytes, box {128, 128}
    const uint8_t *sfa;       // scale atoms of A: [ceil(m/128)][atoms_per_tile][512]
    const uint8_t *sfb;       // scale atoms of B: [ceil(n/128)][atoms_per_tile][512]
    void *C;
    int M, N, K;
    int atoms_per_tile;
    float alpha;
    uint64_t timeout_ns;
    int *status;
};

struct Fp4PairSmem {
    uint64_t full[kF4PStages];     // used in the leader: both CTAs' loads of a stage have landed
    uint64_t empty[kF4PStages];    // per CTA: the pair's MMAs have finished reading this stage
    uint64_t tmem_full;
    uint64_t tmem_empty;           // leader: 8 epilogue warps of the pair have drained the accumulator
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};

template <typename TOut, bool NV>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kF4PairThreads, 1)
    fp4_pair_gemm_kernel(const __grid_constant__ Fp4PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Fp4PairSmem *sh = reinterpret_cast<Fp4PairSmem *>(smem + kF4PStages * kF4PStage);
    static_assert(sizeof(Fp4PairSmem) <= 512, "barrier block outgrew its budget");
    constexpr int kAtoms = NV ? 4 : 2;            // scale atoms per operand tile and K-step
    constexpr uint32_t kSetCols = NV ? 48 : 24;   // TMEM columns of one K-step's scales: A atoms + 2 x B atoms, 4 columns each

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t cr = cluster_ctarank();
    const int mt2 = (p.M + 2 * BM - 1) / (2 * BM), nt = (p.N + BN - 1) / BN;
    const int num_tiles = mt2 * nt;
    const int kblocks = (p.K / 2 + kF4BK - 1) / kF4BK;
    const int mmas_total = p.K / 64;
    const int a_atom_rows = (p.M + BM - 1) / BM;
    const int apt = p.atoms_per_tile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kF4PStages; ++s) {
            mbar_init(&sh->full[s], 2 + 8);      // both CTAs' operand loads + their four scale warps each
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->tmem_full, 1);
        mbar_init(&sh->tmem_empty, 8);
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        mbar_init_fence();
        prefetch_tensormap(&p.tmA);
        prefetch_tensormap(&p.tmB);
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
    const uint32_t tmem_sf0 = tmem_base + BN;     // one set of scale columns per pipeline stage

    WaitCtl ctl;
    ctl.abort_smem = &sh->abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = 0;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += pairs) {
                const int mi2 = t / nt, ni = t - mi2 * nt;
                const int a_row = mi2 * 2 * BM + static_cast<int>(cr) * BM;            // rows past M read as zero
                const int n_half = ni * BN + static_cast<int>(cr) * 128;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kF4PStages;
                    const uint32_t ph = (it / kF4PStages) & 1;
                    if (!(ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY))) break;
                    const uint32_t full_leader = mapa_cluster(smem_u32(&sh->full[st]), 0);
                    uint8_t *sa = smem + st * kF4PStage;
                    uint8_t *sb = sa + kF4PA;
                    mbar_expect_tx_cluster(full_leader, kF4PA + kF4PB);
                    tma_load_2d_pair(sa, &p.tmA, full_leader, kb * kF4BK, a_row);
                    tma_load_2d_pair(sb, &p.tmB, full_leader, kb * kF4BK, n_half);
                }
            }
            if (!ok) {      // give loads in flight time to land before the CTA's shared memory goes away
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
                if (!(ok = mbar_wait(&sh->tmem_empty, (tcount & 1) ^ 1, ctl, W_TMEM_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int st = it % kF4PStages;
                    if (!(ok = mbar_wait(&sh->full[st], (it / kF4PStages) & 1, ctl, W_MBAR_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + st * kF4PStage);
                    const uint32_t b_addr = a_addr + kF4PA;
                    const uint32_t sfa_t = tmem_sf0 + static_cast<uint32_t>(st) * kSetCols;   // atom a of A at +4a
                    const uint32_t sfb_t = sfa_t + kAtoms * 4;                     // atom a of B at +8a (n 0-127) and +8a+4 (n 128-255)
                    const int mmas = min(4, mmas_total - kb * 4);
                    for (int k = 0; k < mmas; ++k) {
                        const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);   // 64 e2m1 = 32 bytes of a 128-byte row
                        const uint64_t bd = make_smem_desc(b_addr + k * 32, 16, 1024);
                        if (NV) {
                            umma_nvfp4_pair(tmem_base, ad, bd, make_idesc_fp4(2 * BM, BN, 0u, 0u, 0u), sfa_t + k * 4, sfb_t + k * 8,
                                            (kb | k) != 0);
                        } else {
                            const uint32_t sf_id = static_cast<uint32_t>(k & 1) * 2u;
                            umma_mxfp4_pair(tmem_base, ad, bd, make_idesc_fp4(2 * BM, BN, sf_id, sf_id, 1u), sfa_t + (k >> 1) * 4,
                                            sfb_t + (k >> 1) * 8, (kb | k) != 0);
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
    } else if (warp < 6) {
        // ---------------------------------------------------------------- epilogue ----
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        uint32_t tcount = 0;
        bool ok = true;
        TOut *const C = reinterpret_cast<TOut *>(p.C);
        for (int t = pair; t < num_tiles && ok; t += pairs) {
            const int mi2 = t / nt, ni = t - mi2 * nt;
            if (!(ok = mbar_wait(&sh->tmem_full, tcount & 1, ctl, W_TMEM_FULL))) break;
            tc_fence_after();
            uint32_t pk[BN / 2];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_base + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[c * 16 + i] = Pack2<TOut>::pack(__uint_as_float(v[2 * i]) * p.alpha, __uint_as_float(v[2 * i + 1]) * p.alpha);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->tmem_empty), 0));
            const int row = mi2 * 2 * BM + static_cast<int>(cr) * BM + row_in_tile;
            if (row < p.M) {
                TOut *dst = C + static_cast<size_t>(row) * p.N + ni * BN;
#pragma unroll
                for (int g = 0; g < BN / 8; ++g)
                    if (ni * BN + g * 8 < p.N)
                        *reinterpret_cast<uint4 *>(dst + g * 8) =
                            make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
            }
            ++tcount;
        }
    } else {
        // ---------------------------------------------------------- scale factors ----
        // warps 6-9 own TMEM lane quarters 2, 3, 0, 1.  Per K-step a lane reads its 16-byte row of every atom of the
        // step (A, and B for both column halves) and stores it into the stage's scale columns; one K-step ahead is
        // kept in flight.
        const uint32_t lane_field = static_cast<uint32_t>((warp & 3) * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += pairs) {
            const int mi2 = t / nt, ni = t - mi2 * nt;
            const int a_row = mi2 * 2 * BM + static_cast<int>(cr) * BM;
            // a half-tile past the matrix has no atoms of its own: any valid ones do (its rows are never stored)
            const uint8_t *sfa = p.sfa + static_cast<size_t>(min(a_row >> 7, a_atom_rows - 1)) * apt * 512 + lane * 16;
            const uint8_t *sfb0 = p.sfb + static_cast<size_t>(ni * 2) * apt * 512 + lane * 16;
            const uint8_t *sfb1 = (ni * BN + 128) < p.N ? sfb0 + static_cast<size_t>(apt) * 512 : sfb0;
            uint4 cur[3 * kAtoms], nxt[3 * kAtoms];
            auto load_step = [&](uint4 (&v)[3 * kAtoms], int kb) {
#pragma unroll
                for (int a = 0; a < kAtoms; ++a) {
                    const size_t o = static_cast<size_t>(min(kb * kAtoms + a, apt - 1)) * 512;
                    v[a] = __ldg(reinterpret_cast<const uint4 *>(sfa + o));
                    v[kAtoms + 2 * a] = __ldg(reinterpret_cast<const uint4 *>(sfb0 + o));
                    v[kAtoms + 2 * a + 1] = __ldg(reinterpret_cast<const uint4 *>(sfb1 + o));
                }
            };
            load_step(nxt, 0);
            for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
#pragma unroll
                for (int j = 0; j < 3 * kAtoms; ++j) cur[j] = nxt[j];
                load_step(nxt, kb + 1 < kblocks ? kb + 1 : kb);
                const int st = it % kF4PStages;
                const uint32_t ph = (it / kF4PStages) & 1;
                // the MMAs that read this stage's scale columns one round ago have finished
                if (lane == 0) ok = mbar_wait(&sh->empty[st], ph ^ 1, ctl, W_MBAR_EMPTY);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                tc_fence_after();
                const uint32_t col = tmem_sf0 + static_cast<uint32_t>(st) * kSetCols + lane_field;
#pragma unroll
                for (int a = 0; a < kAtoms; ++a) {
                    tmem_st_32x4(col + a * 4, cur[a]);
                    tmem_st_32x4(col + kAtoms * 4 + a * 8, cur[kAtoms + 2 * a]);
                    tmem_st_32x4(col + kAtoms * 4 + a * 8 + 4, cur[kAtoms + 2 * a + 1]);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&sh->full[st]), 0));
            }
        }
    }

    // neither CTA may leave while the other can still signal its barriers or read its shared memory
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

int encode_bytes(const DriverApi *api, CUtensorMap *tm, const void *base, uint64_t inner, uint64_t outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner};
    cuuint32_t box[2] = {128, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = api->TensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
                                           box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (fp4) failed: %d", static_cast<int>(r));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename TOut, bool NV>
int launch(const Fp4Params &p, int grid, cudaStream_t stream) {
    auto kern = fp4_gemm_kernel<TOut, NV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kF4SmemBytes);
    if (e == cudaSuccess) {
        kern<<<grid, kGemmThreads, kF4SmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("FP4 GEMM launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename TOut, bool NV>
int launch_pair(const Fp4PairParams &p, int grid, cudaStream_t stream) {
    auto kern = fp4_pair_gemm_kernel<TOut, NV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kF4PSmemBytes);
    if (e == cudaSuccess) {
        kern<<<grid, kF4PairThreads, kF4PSmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("FP4 pair GEMM launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

size_t align1k(size_t v) { return (v + 1023) / 1024 * 1024; }

}  // namespace

size_t fp4_gemm_workspace_bytes(int format, int m, int n, int k) {
    const int blk = format == 1 ? 16 : 32;
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    // sf_atoms_bytes(rows, 32 * scales) is the atom layout's size for `scales` scale bytes per row
    return align1k(sf_atoms_bytes(m, 32 * (k / blk))) + align1k(sf_atoms_bytes(n, 32 * (k / blk))) + 64;
}

int launch_fp4_gemm(cudaStream_t stream, int format, int out_dtype, const uint8_t *A, const uint8_t *B, void *C,
                    const uint8_t *a_scale, const uint8_t *b_scale, float alpha, int m, int n, int k, uint8_t *workspace,
                    uint32_t block_num) {
    std::string why;
    const DriverApi *api = driver_api(&why);
    if (!api) {
        set_error("CUDA driver unavailable: %s", why.c_str());
        return CATCCOS_ERR_CUDA;
    }
    if (format != 0 && format != 1) {
        set_error("FP4 format must be 0 (MXFP4: E8M0 per 32) or 1 (NVFP4: E4M3 per 16), got %d", format);
        return CATCCOS_ERR_INVALID;
    }
    if (out_dtype != CATCCOS_FP16 && out_dtype != CATCCOS_BF16) {
        set_error("FP4 GEMM writes FP16 (1) or BF16 (27), got %d", out_dtype);
        return CATCCOS_ERR_INVALID;
    }
    if (m <= 0 || n <= 0 || k <= 0 || (k % 64) != 0 || (n % 8) != 0) {
        set_error("unsupported shape m=%d n=%d k=%d (k multiple of 64, n multiple of 8)", m, n, k);
        return CATCCOS_ERR_INVALID;
    }
    if (!A || !B || !C || !a_scale || !b_scale || !workspace || (reinterpret_cast<uintptr_t>(A) & 15) ||
        (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
        (reinterpret_cast<uintptr_t>(workspace) & 15)) {
        set_error("A, B, C, both scale tensors and the workspace must be non-null (16-byte aligned data)");
        return CATCCOS_ERR_INVALID;
    }
    const int blk = format == 1 ? 16 : 32;
    const int scales = k / blk;                                  // per row
    const int ld = format == 1 ? scales : (scales + 1) / 2 * 2;  // MXFP4 rows are padded to an even count, as for MXFP8
    static thread_local Fp4Params p;
    memset(&p, 0, sizeof(p));
    uint8_t *sfa = workspace;
    uint8_t *sfb = workspace + align1k(sf_atoms_bytes(m, 32 * scales));
    int *status = reinterpret_cast<int *>(workspace + fp4_gemm_workspace_bytes(format, m, n, k) - 64);
    cudaError_t e = cudaMemsetAsync(status, 0, 64, stream);
    if (e != cudaSuccess) {
        set_error("cudaMemsetAsync failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    int rc = sf_to_atoms_launch(stream, a_scale, 0, m, scales, ld, sfa);
    if (rc) return rc;
    if ((rc = sf_to_atoms_launch(stream, b_scale, 0, n, scales, ld, sfb))) return rc;
    if ((rc = encode_bytes(api, &p.tmA, A, k / 2, m))) return rc;
    if ((rc = encode_bytes(api, &p.tmB, B, k / 2, n))) return rc;
    p.sfa = sfa;
    p.sfb = sfb;
    p.C = C;
    p.M = m;
    p.N = n;
    p.K = k;
    p.atoms_per_tile = (scales + 3) / 4;
    p.alpha = alpha;
    p.timeout_ns = 10ull * 1000 * 1000 * 1000;
    p.status = status;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = sms;
    if (block_num > 0 && static_cast<int>(block_num) < grid) grid = static_cast<int>(block_num);
    // CTA pairs (cta_group::2) unless CATCCOS_TWO_CTA=0 or fewer than two CTAs are allowed
    bool use_pair = grid >= 2;
    if (const char *e2 = getenv("CATCCOS_TWO_CTA")) use_pair = use_pair && atoi(e2) != 0;
    if (use_pair) {
        static thread_local Fp4PairParams q;
        memset(&q, 0, sizeof(q));
        q.tmA = p.tmA;
        q.tmB = p.tmB;
        const int apt = p.atoms_per_tile;
        q.sfa = sfa;
        q.sfb = sfb;
        q.C = C;
        q.M = m;
        q.N = n;
        q.K = k;
        q.atoms_per_tile = apt;
        q.alpha = alpha;
        q.timeout_ns = p.timeout_ns;
        q.status = status;
        const int g2 = grid & ~1;
        if (format == 1)
            return out_dtype == CATCCOS_BF16 ? launch_pair<__nv_bfloat16, true>(q, g2, stream) : launch_pair<__half, true>(q, g2, stream);
        return out_dtype == CATCCOS_BF16 ? launch_pair<__nv_bfloat16, false>(q, g2, stream) : launch_pair<__half, false>(q, g2, stream);
    }
    if (format == 1)
        return out_dtype == CATCCOS_BF16 ? launch<__nv_bfloat16, true>(p, grid, stream) : launch<__half, true>(p, grid, stream);
    return out_dtype == CATCCOS_BF16 ? launch<__nv_bfloat16, false>(p, grid, stream) : launch<__half, false>(p, grid, stream);
}

}  // namespace cb
